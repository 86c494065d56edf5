"""Dafolorn without a GPU: the plain implementation's mechanisms against values worked out by hand,
its configuration and plan, and the engine's host logic (plan, cache and state manager, batching,
scheduler) run on the plain kernel table against the plain implementation."""
import math

import numpy as np
import pytest
import torch

import dafolorn_models as dm
import helpers
from plain import plain_dafolorn as P
from plain.plain_kernels import PlainKernels


@pytest.fixture(scope="module")
def dafolorn_dirs(tmp_path_factory):
    out = {}
    for i, (name, (raw, page)) in enumerate(dm.configs().items()):
        out[name] = (dm.write_model(raw, tmp_path_factory.mktemp(f"dafolorn_{name}"), seed=31 + i), page, raw)
    return out


# ------------------------------------------------------------------ mechanisms, by hand

def test_norms_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    rms = math.sqrt(12.5)
    assert torch.allclose(P.unit_norm(x, 0.0), x / rms)
    assert torch.allclose(P.offset_norm(x, torch.tensor([0.0, -0.5], dtype=torch.float64), 0.0),
                          torch.tensor([[3.0 / rms, 2.0 / rms]], dtype=torch.float64))
    assert torch.allclose(P.plain_weight_norm(x, torch.tensor([2.0, 0.0], dtype=torch.float64), 0.0),
                          torch.tensor([[6.0 / rms, 0.0]], dtype=torch.float64))
    assert float(P.unit_norm(torch.zeros(1, 4, dtype=torch.float64), 1e-6).abs().max()) == 0.0      # eps inside the root


def test_short_conv_by_hand():
    h = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 0.25, 2.0]], dtype=torch.float64)                # oldest tap first, the present input last
    out = P.short_conv(h, w)
    assert out[:, 0].tolist() == [1 + 2.0, 10 + 20 + 0.25, 100 + 200 + 2.5 + 0.5, 1000 + 2000 + 25 + 5]
    one = P.short_conv(h, torch.tensor([[3.0]], dtype=torch.float64))
    assert one[:, 0].tolist() == [4.0, 40.0, 400.0, 4000.0]


def test_xielu_by_hand():
    sp = lambda v: math.log1p(math.exp(v))
    z = torch.tensor([0.0, 1.0, -1.0, 2.0, -30.0], dtype=torch.float64)
    y = P.xielu(z, 0.3, -0.2)
    want = [0.0, sp(0.3) + 0.5, (0.5 + sp(-0.2)) * (math.exp(-1) - 1 + 1) - 0.5,
            4 * sp(0.3) + 1.0, (0.5 + sp(-0.2)) * (math.exp(-30) - 1 + 30) - 15.0]
    assert torch.allclose(y, torch.tensor(want, dtype=torch.float64), atol=1e-12)
    eps = 1e-7                                                               # slope 1/2 on both sides of zero
    assert abs(float(P.xielu(torch.tensor([eps]), 0.3, -0.2)) / eps - 0.5) < 1e-5
    assert abs(float(P.xielu(torch.tensor([-eps]), 0.3, -0.2)) / -eps - 0.5) < 1e-5


def test_sink_softmax_by_hand():
    s = torch.tensor([0.0, math.log(2.0)], dtype=torch.float64)
    p = P.windowed_sink_softmax(s, math.log(5.0))
    assert torch.allclose(p, torch.tensor([1 / 8, 2 / 8], dtype=torch.float64))       # the sink takes 5 of 8
    p = P.windowed_sink_softmax(s, -1e9)
    assert torch.allclose(p, torch.tensor([1 / 3, 2 / 3], dtype=torch.float64))
    p = P.windowed_sink_softmax(torch.tensor([800.0], dtype=torch.float64), 900.0)     # no overflow
    assert abs(float(p[0]) - math.exp(-100.0)) < 1e-50


def _attention_tensors(H, dk, dv, r, width, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    return {"q": mk(H * dk, width), "dkv": mk(r, width), "dkv.norm": 1 + 0.1 * mk(r), "uk": mk(H * dk, r),
            "uv": mk(H * dv, r), "sink": mk(H), "o": mk(width, H * dv)}


def test_latent_attention_window_sink_and_latent_form():
    H, dk, dv, r, width, n, size = 2, 4, 6, 5, 8, 12, 4
    t = _attention_tensors(H, dk, dv, r, width, 3)
    g = torch.Generator().manual_seed(4)
    h = torch.randn(n, width, generator=g, dtype=torch.float64)
    mixer = {"heads": H, "dim": dk, "vdim": dv, "kv_rank": r, "scale": 0.5, "mask": {"size": size}}
    out = P.latent_attention(h, t, "", mixer, 1e-6)
    # a key just outside the window changes nothing, the one just inside does
    for j, changes in ((n - 1 - size, False), (n - size, True)):
        h2 = h.clone()
        h2[j] += 1.0
        diff = float((P.latent_attention(h2, t, "", mixer, 1e-6)[n - 1] - out[n - 1]).abs().max())
        assert (diff > 1e-6) == changes, (j, diff)
    # the same through the latent: scores from Wuk^T q against c, values from Wuv applied to the weighted latent
    i = n - 1
    c = P.plain_weight_norm(h @ t["dkv"].T, t["dkv.norm"], 1e-6)
    heads = []
    for a in range(H):
        q = t["q"][a * dk:(a + 1) * dk] @ h[i]
        ql = t["uk"][a * dk:(a + 1) * dk].T @ q
        s = (c[i - size + 1:i + 1] @ ql) * 0.5
        p = P.windowed_sink_softmax(s, t["sink"][a])
        heads.append(t["uv"][a * dv:(a + 1) * dv] @ (p @ c[i - size + 1:i + 1]))
    assert torch.allclose(out[i], t["o"] @ torch.cat(heads), atol=1e-10)
    # a large sink takes the weight away: the output shrinks towards zero
    t2 = dict(t, sink=t["sink"] + 60.0)
    assert float(P.latent_attention(h, t2, "", mixer, 1e-6).abs().max()) < 1e-3 * float(out.abs().max())
    # without a mask every earlier key counts
    nomask = {k: v for k, v in mixer.items() if k != "mask"}
    h2 = h.clone()
    h2[0] += 1.0
    assert float((P.latent_attention(h2, t, "", nomask, 1e-6)[n - 1] - P.latent_attention(h, t, "", nomask, 1e-6)[n - 1]).abs().max()) > 1e-9


def test_run_order_of_looped_layers():
    cfg = {"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}
    assert [(i, rep) for i, rep, _f in P.run_order(cfg)] == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2),
                                                             (3, None), (4, None)]
    assert [i for i, _r, first in P.run_order(cfg) if first] == [1, 1, 1]
    assert [i for i, _r, _f in P.run_order({"layers": [0] * 3})] == [0, 1, 2]


@pytest.mark.parametrize("name", ["P", "R", "U"])
def test_whole_model_is_causal_and_its_options_matter(name, dafolorn_dirs):
    d, _page, raw = dafolorn_dirs[name]
    _raw, W = dm.load(d)
    toks = dm.requests_for(raw, [45], 5)["r0"]
    full = P.forward(raw, W, toks)
    assert torch.allclose(full[:19], P.forward(raw, W, toks[:19]), atol=1e-10), "a position depends on later tokens"
    assert float(full.abs().max()) > 0.5, "the test model's logits are too flat to show anything"
    assert float(full.abs().max()) <= raw["logit_softcap"]
    f32 = P.forward(raw, W, toks, dtype=torch.float32)
    assert float((f32.double() - full).abs().max()) < 1e-3

    def differs(other_raw=None, other_W=None):
        return float((P.forward(other_raw or raw, other_W or W, toks) - full).abs().max())
    assert differs(other_W={k: (v + 1.0 if k.endswith(".mix.sink") else v) for k, v in W.items()}) > 1e-4     # sinks
    assert differs(other_W={k: (v * 0 if ".canon" in k else v) for k, v in W.items()}) > 1e-4                  # convolutions
    assert differs(other_W={k: (v * 0 if k == "loop.step" else v) for k, v in W.items()}) > 1e-4               # the run's vector
    no_loop = {k: v for k, v in raw.items() if k != "loop"}
    assert differs(other_raw=no_loop) > 1e-4
    wide = {**raw, "layers": [{**l, "mixer": {**l["mixer"], "mask": {"size": l["mixer"]["mask"]["size"] + 1}}}
                              if l["mixer"].get("mask") else l for l in raw["layers"]]}
    assert differs(other_raw=wide) > 1e-5, "a window one token wider gives the same logits"


# ------------------------------------------------------------------ configuration and plan

def test_config_round_trip_and_plan(dafolorn_dirs):
    from inferflux_b200.config import ConfigError, DafolornConfig, config_from_dict, load_config
    from inferflux_b200.models.model import Model
    d, _page, raw = dafolorn_dirs["P"]
    cfg = load_config(d)
    assert isinstance(cfg, DafolornConfig) and cfg.to_dict() == raw
    plan = cfg.to_plan()
    # 2 looped layers x 3 runs + a merge in front of every run + the third layer
    kinds = [plan.layers[e.layer].block.kind for e in plan.schedule]
    assert kinds == ["reinject", "sandwich", "sandwich"] * 3 + ["sandwich"]
    assert [e.repeat for e in plan.schedule] == [0, 0, 0, 1, 1, 1, 2, 2, 2, 0]
    assert len({e.cache for e in plan.schedule}) == len(plan.schedule)          # a cache of its own per run
    model = Model(plan)
    names = set(model.expected_tensors())
    assert {"embed", "final.norm", "loop.in", "loop.step", "l0.norm1", "l0.norm1b", "l0.canon1", "l0.canon2",
            "l0.mix.q", "l0.mix.dkv", "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.sink", "l0.mix.o",
            "l0.mlp.up", "l0.mlp.down", "l0.mlp.act", "l1.norm1b"} <= names
    assert not {"l1.norm2", "l1.canon2", "l1.mlp.up"} & names                   # the layer without feed-forward
    specs = model.cache_specs()
    kv, st = specs[1]
    assert (kv.planes, kv.num_kv_heads, kv.head_dim, kv.window) == (1, 1, 40, 21) and st.shape == (2, 2, 64)
    assert specs[0] == (None, None) and specs[2][1].shape == (1, 2, 64) and specs[9][0].window is None
    for bad in ({**raw, "layers": []}, {**raw, "loop": {"start": 2, "stop": 5, "times": 2}},
                {**raw, "layers": [{**raw["layers"][0], "type": "other"}]}, {k: v for k, v in raw.items() if k != "width"},
                {**raw, "canon": {"taps": 40}}):
        with pytest.raises(ConfigError):
            config_from_dict(bad)
    # no loop, no convolution, no cap: none of their parts or tensors
    _d, _p, raw_s = dafolorn_dirs["S"]
    bare = {k: v for k, v in raw_s.items() if k != "loop"}
    plan = config_from_dict(bare).to_plan()
    assert not plan.keeps_embedding_output and not any("canon" in n or n.startswith("loop.") for n in Model(plan).expected_tensors())


def test_wrong_weights_are_refused(dafolorn_dirs, tmp_path):
    from inferflux_b200.models import load_model
    from inferflux_b200.weights import WeightError, write_safetensors
    d, _page, raw = dafolorn_dirs["Q"]
    _raw, W = dm.load(d)
    (tmp_path / "config.json").write_text((d / "config.json").read_text())
    W2 = {k: v for k, v in W.items() if k != "l1.mix.sink"}
    W2["l0.mix.uv"] = W["l0.mix.uv"][:, :-1].contiguous()
    write_safetensors(tmp_path / "model.safetensors", W2)
    with pytest.raises(WeightError) as e:
        load_model(tmp_path, dtype="float32", device="cpu")
    assert e.value.missing == ["l1.mix.sink"] and [w[0] for w in e.value.wrong_shape] == ["l0.mix.uv"]


# ------------------------------------------------------------------ the engine's host logic on plain kernels

LENS = [40, 33, 50, 61, 97, 70, 25, 64, 1, 2]


@pytest.mark.parametrize("name", ["P", "Q", "R", "S", "U", "V"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_engine_host_logic_on_plain_kernels(name, cutting, dafolorn_dirs):
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    d, page, raw = dafolorn_dirs[name]
    reqs = dm.requests_for(raw, LENS, 100)
    want = dm.plain_logits(d, reqs)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, 256)}[cutting](reqs)
    _c, model = load_model(d, dtype="float32", device="cpu")
    runner = ModelRunner(model, PlainKernels(wide=True), page_size=page, num_pages=256 // page, max_seqs=4, max_seq_len=512)
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"])
    bad = helpers.first_bad(got, want, 2e-4)
    assert bad is None, f"first wrong row (request, position, diff): {bad}"
    assert not runner.cache.live_requests() and runner.cache.free_pages() == [256 // page] * len(runner.cache.groups)


def test_a_slot_that_is_used_again_starts_from_zero_state(dafolorn_dirs):
    """Four slots, ten requests one after the other and side by side: a request that gets a slot someone
    else has used must not see that request's convolution inputs or latents."""
    from inferflux_b200.engine import ModelRunner, StepEntry
    from inferflux_b200.models import load_model
    d, page, raw = dafolorn_dirs["U"]
    reqs = dm.requests_for(raw, [9, 1, 3, 2, 30, 5], 7)
    want = dm.plain_logits(d, reqs)
    _c, model = load_model(d, dtype="float32", device="cpu")
    runner = ModelRunner(model, PlainKernels(wide=True), page_size=page, num_pages=4, max_seqs=1, max_seq_len=64)
    for rid, toks in reqs.items():                         # one slot: everybody inherits it
        got = runner.step([StepEntry(rid, toks, list(range(len(toks))))]).double().numpy()
        assert float(np.abs(got - want[rid]).max()) < 2e-4, rid
        assert any(float(s[0].abs().max()) > 0 for s in runner.cache.state if s is not None)
        runner.end_request(rid)


def test_greedy_generation_through_engine_and_scheduler(dafolorn_dirs):
    from inferflux_b200 import Engine, SamplingParams
    d, page, raw = dafolorn_dirs["P"]
    _raw, W = dm.load(d)
    prompts = list(dm.requests_for(raw, [7, 19, 33, 4, 1], 40).values())

    def greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(P.forward(raw, W, seq)[-1].argmax()))
        return seq[len(prompt):]
    want = [greedy(p, 12) for p in prompts]
    for pages in (64, 12):                                 # 12 pages of 8: the requests do not all fit at once
        eng = Engine(d, dtype="float32", device="cpu", kernels=PlainKernels(wide=True), kv_page_size=page,
                     kv_num_pages=pages, kv_max_batch=4, kv_max_seq=128, chunked_prefill_tokens=16, max_batch_tokens=48)
        res = eng.generate(prompts, SamplingParams(temperature=0.0), max_tokens=12)
        assert [r.token_ids for r in res] == want
        assert not eng.runner.cache.live_requests()
