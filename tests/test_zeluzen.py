"""Zeluzen without a GPU: the plain implementation's mechanisms against values worked out by hand, the
configuration and plan, and the engine's host logic (plan, cache and state manager, batching, scheduler)
run on the plain kernel table against the plain implementation."""
import math

import numpy as np
import pytest
import torch

import helpers
import zeluzen_models as zm
from plain import plain_zeluzen as P
from plain.plain_kernels import PlainKernels

F64 = torch.float64


@pytest.fixture(scope="module")
def zeluzen_dirs(tmp_path_factory):
    out = {}
    for i, (name, (raw, page)) in enumerate(zm.configs().items()):
        out[name] = (zm.write_model(raw, tmp_path_factory.mktemp(f"zeluzen_{name}"), seed=51 + i), page, raw)
    return out


# ------------------------------------------------------------------ mechanisms, by hand

def test_norm_has_eps_under_the_root():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    assert torch.allclose(P.unit_rms(x, 0.0), x / math.sqrt(12.5))
    assert torch.allclose(P.rmsnorm(x, torch.tensor([2.0, 0.0], dtype=F64), 0.0), torch.tensor([[6 / math.sqrt(12.5), 0.0]], dtype=F64))
    assert float(P.unit_rms(torch.zeros(1, 4, dtype=F64), 1e-6).abs().max()) == 0.0
    assert abs(float(P.unit_rms(torch.tensor([[1e-3]], dtype=F64), 1e-6)) - 1e-3 / math.sqrt(2e-6)) < 1e-12


def test_recurrence_by_hand():
    # one head, one key channel, one value channel: S is a number
    r = torch.tensor([[[2.0]], [[3.0]], [[5.0]]], dtype=F64)
    k = torch.tensor([[[1.0]], [[2.0]], [[1.0]]], dtype=F64)
    v = torch.tensor([[[10.0]], [[1.0]], [[4.0]]], dtype=F64)
    w = torch.tensor([[[0.5]], [[0.25]], [[0.1]]], dtype=F64)
    u = torch.tensor([[7.0]], dtype=F64)
    out, S = P.wkv_scan(r, k, v, w, u)
    # S: 0 -> 10 -> 0.25 * 10 + 2 = 4.5 -> 0.1 * 4.5 + 4 = 4.45; the bonus u counts for the present token only
    assert out[:, 0, 0].tolist() == [2 * (0 + 7 * 10), 3 * (10 + 7 * 2), 5 * (4.5 + 7 * 4)]
    assert abs(float(S) - 4.45) < 1e-12
    # the decay scales S's rows (key channels), not its columns
    r2 = torch.ones(2, 1, 2, dtype=F64)
    k2 = torch.tensor([[[1.0, 1.0]], [[0.0, 0.0]]], dtype=F64)
    v2 = torch.tensor([[[1.0, 2.0]], [[0.0, 0.0]]], dtype=F64)
    w2 = torch.tensor([[[1.0, 1.0]], [[0.5, 0.25]]], dtype=F64)
    _o, S2 = P.wkv_scan(r2, k2, v2, w2, torch.zeros(1, 2, dtype=F64))
    assert S2[0].tolist() == [[0.5, 1.0], [0.25, 0.5]]
    # carried state: two halves give what the whole gives
    g = torch.Generator().manual_seed(1)
    mk = lambda *s: torch.rand(*s, generator=g, dtype=F64)
    r, k, v, w, u = mk(9, 2, 3), mk(9, 2, 3), mk(9, 2, 3), mk(9, 2, 3), mk(2, 3)
    whole, S_whole = P.wkv_scan(r, k, v, w, u)
    first, S_mid = P.wkv_scan(r[:4], k[:4], v[:4], w[:4], u)
    second, S_end = P.wkv_scan(r[4:], k[4:], v[4:], w[4:], u, state=S_mid)
    assert torch.allclose(torch.cat([first, second]), whole) and torch.allclose(S_end, S_whole)


def test_shift_and_decay_by_hand():
    h = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=F64)
    assert P.shifted(h).tolist() == [[0.0, 0.0], [1.0, 2.0], [3.0, 4.0]]
    assert abs(float(P.decay(torch.tensor(0.0, dtype=F64))) - math.exp(-1.0)) < 1e-15
    assert 0.0 < float(P.decay(torch.tensor(3.0, dtype=F64))) < 1e-8 and float(P.decay(torch.tensor(-9.0, dtype=F64))) > 0.9998


def test_rotation_and_frequency_scaling_by_hand():
    x = torch.tensor([[[1.0, 0.0, 5.0, 6.0, 7.0, 8.0]]], dtype=F64)             # one token, one head of six
    out = P.rotate_pairs(x, [1], [math.pi / 2, math.pi])
    assert torch.allclose(out[0, 0], torch.tensor([0.0, 1.0, -5.0, -6.0, 7.0, 8.0], dtype=F64), atol=1e-12)
    assert torch.equal(P.rotate_pairs(x, [0], [0.3, 0.7]), x)
    plain = P.scaled_frequencies(100.0, 8, None)
    assert plain == [100.0 ** (-2.0 * i / 8) for i in range(4)]
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    f = P.scaled_frequencies(100.0, 8, sc)
    # wavelengths 6.3, 19.9, 62.8, 198.7 against 64 / 4 = 16 and 64 / 1 = 64
    assert f[0] == plain[0] and abs(f[3] - plain[3] / 4.0) < 1e-18
    for i in (1, 2):
        s = (64 * plain[i] / (2 * math.pi) - 1.0) / 3.0
        assert 0.0 < s < 1.0 and abs(f[i] - ((1 - s) * plain[i] / 4.0 + s * plain[i])) < 1e-15


def test_chunks_and_sink_by_hand():
    assert [j for j in range(10) if P.visible(6, j, 4)] == [4, 5, 6]
    assert [j for j in range(10) if P.visible(8, j, 4)] == [8]
    assert [j for j in range(10) if P.visible(7, j, 4)] == [4, 5, 6, 7]
    assert [j for j in range(5) if P.visible(3, j, None)] == [0, 1, 2, 3]
    s = torch.tensor([0.0, math.log(3.0)], dtype=F64)
    assert torch.allclose(P.sink_softmax(s), torch.tensor([1 / 5, 3 / 5], dtype=F64))      # the sink takes 1 of 5
    assert abs(float(P.sink_softmax(torch.tensor([-800.0], dtype=F64))[0])) < 1e-300        # far below the sink
    assert abs(float(P.sink_softmax(torch.tensor([800.0], dtype=F64))[0]) - 1.0) < 1e-12    # no overflow


def test_router_by_hand():
    W = {"m.router": torch.eye(4, dtype=F64), "m.correction": torch.tensor([0.0, 0.0, 0.0, 0.5], dtype=F64)}
    h = torch.log(torch.tensor([[4.0, 3.0, 2.0, 1.0]], dtype=F64))                        # scores 0.4, 0.3, 0.2, 0.1
    chosen, weight = P.route(h, W, "m.", {"top": 2})
    assert sorted(chosen[0].tolist()) == [0, 3]                                              # 0.1 + 0.5 beats 0.3
    got = dict(zip(chosen[0].tolist(), weight[0].tolist()))
    assert abs(got[0] - 0.4) < 1e-12 and abs(got[3] - 0.1) < 1e-12                           # the weights are the scores
    # two experts with weights, two that pass the input on
    W.update({"m.e0.up": torch.tensor([[1.0, 0, 0, 0], [-1.0, 0, 0, 0]], dtype=F64), "m.e0.down": torch.ones(4, 2, dtype=F64),
              "m.e1.up": torch.zeros(2, 4, dtype=F64), "m.e1.down": torch.zeros(4, 2, dtype=F64)})
    out = P.moe_ff(h, W, "m.", {"experts": 2, "identity": 2, "top": 2})
    a = math.log(4.0) ** 2                                                                    # relu(x)^2, relu(-x)^2 = 0
    assert torch.allclose(out[0], 0.4 * torch.full((4,), a, dtype=F64) + 0.1 * h[0])


# ------------------------------------------------------------------ the whole model, stated plainly

@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_model_is_causal_and_its_options_matter(name, zeluzen_dirs):
    d, _page, raw = zeluzen_dirs[name]
    _raw, W = zm.load(d)
    toks = zm.requests_for(raw, [45], 5)["r0"]
    full = P.forward(raw, W, toks)
    assert torch.allclose(full[:19], P.forward(raw, W, toks[:19]), atol=1e-10), "a position depends on later tokens"
    assert float(full.abs().max()) > 0.5, "the test model's logits are too flat to show anything"
    assert float((P.forward(raw, W, toks, dtype=torch.float32).double() - full).abs().max()) < 1e-3

    def differs(other_raw=None, other_W=None):
        return float((P.forward(other_raw or raw, other_W or W, toks) - full).abs().max())
    assert differs(other_W={k: (v + 0.3 if k.endswith(".mix.u") else v) for k, v in W.items()}) > 1e-5          # the bonus
    assert differs(other_W={k: (v * 0 if ".mix.mu." in k else v) for k, v in W.items()}) > 1e-5                  # the mixes
    assert differs(other_W={k: (v + 1.0 if k.endswith(".mix.w0") else v) for k, v in W.items()}) > 1e-5          # the decay
    if name == "A":           # the other models' routers choose all, or choose among experts that all pass the input on
        assert differs(other_W={k: (v * 0 if k.endswith(".mlp.correction") else v) for k, v in W.items()}) > 1e-6
    assert differs(other_W={k: (v * 1.5 if k.endswith(".k.norm") else v) for k, v in W.items()}) > 1e-5
    assert differs(other_W={k: (v + 0.5 if k == "embed.norm" else v) for k, v in W.items()}) > 1e-5

    def edit(change):
        layers = []
        for l in raw["layers"]:
            m = dict(l["mixer"])
            if l["type"] == "attention":
                change(m)
            layers.append({**l, "mixer": m})
        return {**raw, "layers": layers}

    def wider(m):
        if m.get("mask"):
            m["mask"] = {"size": m["mask"]["size"] + 1}

    def unturned(m):
        m.pop("rot", None)
    assert differs(other_raw=edit(wider)) > 1e-5, "chunks one token longer give the same logits"
    if any(l["mixer"].get("rot") for l in raw["layers"]):
        assert differs(other_raw=edit(unturned)) > 1e-5


def test_a_layer_without_keys_reads_the_other_layers(zeluzen_dirs):
    d, _page, raw = zeluzen_dirs["A"]
    _raw, W = zm.load(d)
    toks = zm.requests_for(raw, [30], 6)["r0"]
    streams, other = [], []
    P.forward(raw, W, toks, streams=streams)
    W2 = dict(W)
    W2["l0.mix.k.norm"] = W["l0.mix.k.norm"] * 1.3          # layer 2 has no keys: it must see layer 0's change
    W2["l0.mix.q"] = W["l0.mix.q"]
    P.forward(raw, W2, toks, streams=other)
    assert float((streams[2] - other[2]).abs().max()) > 1e-6
    assert not any(k.startswith("l2.mix.k") or k.startswith("l2.mix.v") for k in W)


# ------------------------------------------------------------------ configuration and plan

def test_config_round_trip_and_plan(zeluzen_dirs):
    from inferflux_b200.config import ConfigError, ZeluzenConfig, config_from_dict, load_config
    from inferflux_b200.models.model import Model
    d, _page, raw = zeluzen_dirs["A"]
    cfg = load_config(d)
    assert isinstance(cfg, ZeluzenConfig) and cfg.to_dict() == raw
    plan = cfg.to_plan()
    assert [plan.layers[e.layer].block.kind for e in plan.schedule] == ["postnorm"] * 4
    assert [(e.cache, e.writes_cache) for e in plan.schedule] == [(0, True), (1, True), (0, False), (2, True)]
    model = Model(plan)
    names = set(model.expected_tensors())
    assert {"embed", "embed.norm", "final.norm", "head", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.v",
            "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.o", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l1.mix.mu.r",
            "l1.mix.mu.w", "l1.mix.r", "l1.mix.g", "l1.mix.w1", "l1.mix.w2", "l1.mix.w0", "l1.mix.u", "l1.mix.norm",
            "l1.mix.o", "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e0.up", "l1.mlp.e4.down", "l2.mix.q",
            "l2.mix.q.norm", "l2.mix.o", "l2.mlp.e2.up", "l3.norm1"} <= names
    assert not {"l2.mix.k", "l2.mix.v", "l2.mix.k.norm", "l3.norm2", "l3.mlp.gate", "l1.mlp.e5.up", "l2.mlp.e3.up"} & names
    specs = model.cache_specs()
    kv, st = specs[0]
    assert (kv.planes, kv.num_kv_heads, kv.head_dim, kv.chunk, kv.window) == (2, 2, 24, 16, None) and st is None
    assert specs[1][0] is None and specs[1][1].shape == (2 * 32 * 32 + 64,)
    assert specs[2][1].shape == (3 * 24 * 24 + 64,)
    # a reader that cuts its positions differently keeps every page of the cache it reads
    _d, _p, raw_b = zeluzen_dirs["B"]
    specs_b = Model(config_from_dict(raw_b).to_plan()).cache_specs()
    assert specs_b[1][0].chunk is None and specs_b[1][0].head_dim == 8 and specs_b[2][0].chunk is None
    # the decay's inner size: given, or left to the file
    exp = model.expected_tensors()
    assert exp["l3.mix.w1"].shape == (5, 64) and exp["l1.mix.w1"].shape == (-1, 64) and exp["l1.mix.w1"].fits((11, 64))
    bad_kv = {**raw, "layers": [raw["layers"][1], raw["layers"][0], {**raw["layers"][2], "mixer": {**raw["layers"][2]["mixer"], "kv_from": 0}}]}
    odd = {**raw, "layers": [{**raw["layers"][0], "mixer": {**raw["layers"][0]["mixer"], "dim": 15}}]}
    for bad in ({**raw, "layers": []}, {**raw, "layers": [{**raw["layers"][0], "type": "other"}]}, bad_kv, odd,
                {k: v for k, v in raw.items() if k != "width"},
                {**raw, "layers": [{**raw["layers"][1], "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 2, "identity": 0, "top": 3}}}]}):
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_wrong_weights_are_refused_and_the_decay_rank_comes_from_the_file(zeluzen_dirs, tmp_path):
    from inferflux_b200.models import load_model
    from inferflux_b200.weights import WeightError, write_safetensors
    d, _page, raw = zeluzen_dirs["D"]
    _raw, W = zm.load(d)
    (tmp_path / "config.json").write_text((d / "config.json").read_text())
    W2 = {k: v for k, v in W.items() if k != "l1.mlp.correction"}
    W2["l0.mix.u"] = W["l0.mix.u"][:, :-1].contiguous()
    write_safetensors(tmp_path / "model.safetensors", W2)
    with pytest.raises(WeightError) as e:
        load_model(tmp_path, dtype="float32", device="cpu")
    assert e.value.missing == ["l1.mlp.correction"] and [w[0] for w in e.value.wrong_shape] == ["l0.mix.u"]
    W3 = dict(W)                                            # another inner size of the decay: taken from the tensors
    W3["l0.mix.w1"] = torch.cat([W["l0.mix.w1"], W["l0.mix.w1"][:3] * 0.5])
    W3["l0.mix.w2"] = torch.cat([W["l0.mix.w2"], W["l0.mix.w2"][:, :3] * 0.5], dim=1)
    write_safetensors(tmp_path / "model.safetensors", W3)
    _c, model = load_model(tmp_path, dtype="float32", device="cpu")
    assert model.layers[0].mixer.rank == W["l0.mix.w1"].shape[0] + 3


# ------------------------------------------------------------------ the engine's host logic on plain kernels

LENS = [40, 33, 50, 61, 97, 70, 25, 64, 1, 2]


def _plain_runner(d, page, pages=None, max_seqs=4, max_seq_len=512):
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    _c, model = load_model(d, dtype="float32", device="cpu")
    return ModelRunner(model, PlainKernels(wide=True), page_size=page, num_pages=pages or 256 // page, max_seqs=max_seqs,
                       max_seq_len=max_seq_len)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_engine_host_logic_on_plain_kernels(name, cutting, zeluzen_dirs):
    d, page, raw = zeluzen_dirs[name]
    reqs = zm.requests_for(raw, LENS, 100)
    want = zm.plain_logits(d, reqs)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, 256)}[cutting](reqs)
    runner = _plain_runner(d, page)
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"])
    bad = helpers.first_bad(got, want, 2e-4)
    assert bad is None, f"first wrong row (request, position, diff): {bad}"
    assert not runner.cache.live_requests() and runner.cache.free_pages() == [256 // page] * len(runner.cache.groups)


def test_pages_leave_with_their_chunk_and_come_back(zeluzen_dirs):
    """Chunks of 16 in pages of 8: once a request is past a chunk, that chunk's two pages are free again, in
    prompts and in decoding; a pool of 7 pages serves a request of 150 tokens (19 pages without that)."""
    from inferflux_b200.engine import StepEntry
    d, page, raw = zeluzen_dirs["A"]
    toks = zm.requests_for(raw, [150], 8)["r0"]
    want = zm.plain_logits(d, {"r0": toks})["r0"]
    runner = _plain_runner(d, page, pages=7)
    got, pos, sizes = [], 0, [21, 1, 1, 40, 3, 1, 1, 1, 16, 17, 2]
    i = 0
    while pos < len(toks):
        n = min(sizes[i % len(sizes)], len(toks) - pos)
        i += 1
        got += list(runner.step([StepEntry("r0", toks[pos:pos + n], list(range(n)))]).double().numpy())
        pos += n
        held = runner.cache.pages_of("r0")
        assert min(held) == (pos // 16 * 16) // page, (pos, sorted(held))
        runner.cache.check()
    assert float(np.abs(np.stack(got) - want).max()) < 2e-4
    assert runner.cache.groups[0].alloc.allocations > 7                      # pages were used again
    runner.end_request("r0")
    assert runner.cache.free_pages() == [7]


def test_a_slot_that_is_used_again_starts_from_zero_state(zeluzen_dirs):
    from inferflux_b200.engine import StepEntry
    d, page, raw = zeluzen_dirs["D"]
    reqs = zm.requests_for(raw, [9, 1, 3, 2, 30, 5], 7)
    want = zm.plain_logits(d, reqs)
    runner = _plain_runner(d, page, pages=4, max_seqs=1, max_seq_len=64)
    for rid, toks in reqs.items():                         # one slot: everybody inherits it
        got = runner.step([StepEntry(rid, toks, list(range(len(toks))))]).double().numpy()
        assert float(np.abs(got - want[rid]).max()) < 2e-4, rid
        assert all(float(s[0].abs().max()) > 0 for s in runner.cache.state if s is not None)
        runner.end_request(rid)


def test_greedy_generation_through_engine_and_scheduler(zeluzen_dirs):
    from inferflux_b200 import Engine, SamplingParams
    d, page, raw = zeluzen_dirs["A"]
    _raw, W = zm.load(d)
    prompts = list(zm.requests_for(raw, [7, 19, 33, 4, 1], 40).values())

    def greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(P.forward(raw, W, seq)[-1].argmax()))
        return seq[len(prompt):]
    want = [greedy(p, 12) for p in prompts]
    for pages in (64, 8):                                  # 8 pages of 8: the requests do not all fit at once
        eng = Engine(d, dtype="float32", device="cpu", kernels=PlainKernels(wide=True), kv_page_size=page,
                     kv_num_pages=pages, kv_max_batch=4, kv_max_seq=128, chunked_prefill_tokens=16, max_batch_tokens=48)
        res = eng.generate(prompts, SamplingParams(temperature=0.0), max_tokens=12)
        assert [r.token_ids for r in res] == want
        assert not eng.runner.cache.live_requests()
