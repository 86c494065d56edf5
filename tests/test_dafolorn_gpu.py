"""Dafolorn on the GPU: every new kernel and part alone against the plain implementation's
functions, then whole models through the step function, the replay program and the engine."""
import math

import numpy as np
import pytest
import torch

import dafolorn_models as dm
import helpers
from plain import plain_dafolorn as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def _rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.fixture(scope="module")
def dafolorn_dirs(tmp_path_factory):
    out = {}
    for i, (name, (raw, page)) in enumerate(dm.configs().items()):
        out[name] = (dm.write_model(raw, tmp_path_factory.mktemp(f"dafolorn_{name}"), seed=31 + i), page, raw)
    return out


def _step_ctx(kernels, dtype, cache, spans, providers=()):
    """A step context for `spans` = [(request, number of tokens)], pages reserved and the table updated."""
    from inferflux_b200.engine.batch import StepContext, StepEntry
    entries, starts, slots = [], [], []
    for rid, n in spans:
        if rid not in cache:
            cache.add_request(rid)
        start = cache.length(rid)
        cache.reserve(rid, start + n)
        entries.append(StepEntry(rid, [0] * n, []))
        starts.append(start)
        slots.append(cache.slot(rid))
    ctx = StepContext.build(kernels, dtype, DEV, entries, starts, slots, cache.drain_table_updates(), providers=providers)
    for g, (idx, page) in zip(cache.groups, ctx.table_updates):
        kernels.scatter_i32(g.table, idx, page)
    return ctx, starts


def _commit(cache, spans, starts):
    for (rid, n), start in zip(spans, starts):
        cache.commit(rid, start + n)


# ------------------------------------------------------------------ element and row kernels

@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H", [64, 100, 4104])
def test_postnorm_add_and_next_norm(cuda_kernels, dtype, tol, H):
    T = 7
    x, y = _rnd(T, H, seed=1, scale=3.0), _rnd(T, H, seed=2, scale=0.7).to(dtype)
    wb, wn = _rnd(H, seed=3, scale=0.3), _rnd(H, seed=4, scale=0.3)              # stored around zero
    want_x = x.double() + P.offset_norm(y.double(), wb.double(), 1e-5)
    want_h = P.offset_norm(want_x, wn.double(), 1e-3)
    xs = x.to(DEV).clone()
    h = cuda_kernels.postnorm_add(xs, y.to(DEV), (1 + wb).to(DEV), 1e-5, (1 + wn).to(DEV), 1e-3, dtype)
    assert float((xs.cpu().double() - want_x).abs().max()) < 1e-5 * float(want_x.abs().max())      # the sum is float32
    assert float((h.cpu().double() - want_h).abs().max()) < tol * float(want_h.abs().max())
    xs = x.to(DEV).clone()
    assert cuda_kernels.postnorm_add(xs, y.to(DEV), (1 + wb).to(DEV), 1e-5) is None
    assert float((xs.cpu().double() - want_x).abs().max()) < 1e-5 * float(want_x.abs().max())
    # y as the partial sums of a K-split product: added in the same pass
    from inferflux_b200.csrc.ops import PartialSum
    parts = _rnd(3, T, H, seed=5, scale=0.5)
    parts[2] = y.float() - parts[0] - parts[1]
    xp = x.to(DEV).clone()
    hp = cuda_kernels.postnorm_add(xp, PartialSum(parts.to(DEV), dtype), (1 + wb).to(DEV), 1e-5, (1 + wn).to(DEV), 1e-3)
    assert hp.dtype == dtype and float((xp.cpu().double() - want_x).abs().max()) < 1e-5 * float(want_x.abs().max())
    assert float((hp.cpu().double() - want_h).abs().max()) < tol * float(want_h.abs().max())
    one = x[:1].to(DEV).clone()                                                   # a row's result does not depend on the others
    cuda_kernels.postnorm_add(one, y[:1].to(DEV), (1 + wb).to(DEV), 1e-5)
    assert torch.equal(one, xs[:1])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 8e-3)])
def test_xielu_softcap_concat(cuda_kernels, dtype, tol):
    z = torch.cat([_rnd(3, 333, seed=5, scale=4.0), torch.tensor([[0.0, -0.0, 1e-4, -1e-4, 30.0, -60.0] + [0.0] * 327])]).to(dtype)
    p, q = 0.37, -0.81
    sp = lambda v: math.log1p(math.exp(v))
    got = cuda_kernels.xielu(z.to(DEV), sp(p), 0.5 + sp(q)).cpu().double()
    want = P.xielu(z.double(), p, q)
    assert float(((got - want).abs() / (1 + want.abs())).max()) < tol
    from inferflux_b200.csrc.ops import PartialSum
    parts = _rnd(4, 4, 333, seed=15, scale=2.0)
    got = cuda_kernels.xielu(PartialSum(parts.to(DEV), dtype), sp(p), 0.5 + sp(q)).cpu()
    want = P.xielu(parts.double().sum(0), p, q)
    assert got.dtype == dtype and float(((got.double() - want).abs() / (1 + want.abs())).max()) < tol
    logits = _rnd(5, 1001, seed=6, scale=40.0)
    dev = logits.to(DEV).clone()
    cuda_kernels.softcap(dev, 12.5)
    assert float((dev.cpu().double() - 12.5 * torch.tanh(logits.double() / 12.5)).abs().max()) < 2e-5
    a, b = _rnd(4, 50, seed=7), _rnd(4, 50, seed=8)
    both = cuda_kernels.concat_cast(a.to(DEV), b.to(DEV), dtype).cpu()
    assert torch.equal(both, torch.cat([a, b], dim=1).to(dtype))


@pytest.mark.parametrize("T,N,K", [(8, 9600, 256), (37, 9472, 136), (8, 640, 256), (200, 9600, 64)])
def test_product_with_the_activation_in_its_epilogue(cuda_kernels, T, N, K):
    """Wide products of few rows apply xIELU before they store (one kernel); the others take the product and
    the activation kernel.  Both against the plain functions."""
    a, w = _rnd(T, K, seed=1).to(torch.bfloat16), _rnd(N, K, seed=2, scale=0.2).to(torch.bfloat16)
    p, q = 0.2, -0.4
    sp = lambda v: math.log1p(math.exp(v))
    before = cuda_kernels.launches + cuda_kernels.library_calls
    got = cuda_kernels.linear_xielu(a.to(DEV), w.to(DEV), sp(p), 0.5 + sp(q)).cpu().double()
    cuda_kernels.check_errors()
    assert (cuda_kernels.launches + cuda_kernels.library_calls - before == 1) == (T <= 160 and N >= 74 * 128 - 127)
    want = P.xielu(a.double() @ w.double().T, p, q)
    # the unfused path rounds the product to bfloat16 before the activation squares it: two roundings and a doubling
    assert float(((got - want).abs() / (1 + want.abs())).max()) < 2e-2


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_conv_over_steps_and_requests(cuda_kernels, dtype, tol, taps):
    """Two requests cut differently (single tokens, two tokens, fewer than taps - 1, many), a third joining
    later on a slot that the first gave back: every row equals the convolution over the whole sequence."""
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.parts import StateSpec
    C = 200
    w = _rnd(C, taps, seed=9, scale=0.5)
    seqs = {"a": _rnd(40, C, seed=10).to(dtype), "b": _rnd(23, C, seed=11).to(dtype), "c": _rnd(9, C, seed=12).to(dtype)}
    want = {r: P.short_conv(h.double(), w.double()) for r, h in seqs.items()}
    state = None if taps == 1 else StateSpec((2, taps - 1, C), torch.float32)
    cache = CacheManager([(None, state)], page_size=16, num_pages=1, max_seqs=2, max_seq_len=64, dtype=dtype, device=DEV)
    plan = [[("a", 1)], [("a", 2), ("b", 5)], [("a", 1), ("b", 1)], [("a", 30), ("b", 2)], [("b", 1), ("a", 6)],
            [("b", 14)], [("c", 2)], [("c", 1)], [("c", 6)]]
    at = {r: 0 for r in seqs}
    for spans in plan:
        if spans[0][0] == "c" and "a" in cache:
            cache.free("a")
            cache.free("b")
        ctx, starts = _step_ctx(cuda_kernels, dtype, cache, spans)
        h = torch.cat([seqs[r][at[r]:at[r] + n] for r, n in spans]).to(DEV)
        out = cuda_kernels.short_conv(h, w.to(DEV), taps, cache.state[0], 1, ctx).cpu().double()
        row = 0
        for r, n in spans:
            ref = want[r][at[r]:at[r] + n]
            assert float((out[row:row + n] - ref).abs().max()) < tol * float(ref.abs().max()), (spans, r)
            row += n
            at[r] += n
        _commit(cache, spans, starts)
        if taps > 1:
            assert float(cache.state[0][:, 0].abs().max()) == 0.0          # the layer's other convolution is not touched


# ------------------------------------------------------------------ latent attention

def _attention_case(kernels, dtype, window, sink, H=3, dk=40, dv=24, r=40, n=420, page=16, seed=0, decode_only=False):
    """Latents through the norm-and-append kernel into pages, queries planted so that single keys stand
    out at a window's two sides, at page borders, among the first tokens and far back; the requests
    are a decoded token, a two-token portion and a longer portion, all in one step (or, `decode_only`,
    three decoded tokens of requests of different lengths)."""
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import ScheduleEntry
    from inferflux_b200.parts import KVCacheSpec
    rows = _rnd(n, dk * H + r, seed=seed + 1).to(dtype)                   # [queries | latent before its norm]
    g = (1 + _rnd(r, seed=seed + 2, scale=0.2)).float()
    w_uk, w_uv = _rnd(H * dk, r, seed=seed + 3, scale=0.4).to(dtype), _rnd(H * dv, r, seed=seed + 4, scale=0.3).to(dtype)
    sinks = _rnd(H, seed=seed + 5, scale=2.0) if sink else None
    W = window or n
    if decode_only:                                                       # request -> (tokens before the step, tokens after)
        spans_of = {"dec": (n - 1, n), "two": (n - 31, n - 30), "long": (n // 2, n // 2 + 1)}
    else:
        spans_of = {"dec": (n - 1, n), "two": (n - 2, n), "long": (n - 50, n)}
    planted = sorted({e - 1 for _h, e in spans_of.values()} | {n - 17, n - 33, n - 50})
    for i in planted:                                                     # plant: the key's latent points along the query's
        for head, j in ((0, i - W + 1), (1, i - W), (2, 3), (0, (i // page) * page), (1, (i // page) * page - 1)):
            head %= H
            if 0 <= j < i:
                ql = w_uk.double()[head * dk:(head + 1) * dk].T @ rows[i, head * dk:(head + 1) * dk].double()
                rows[j, H * dk:] = (ql / ql.norm() * 3.0).to(dtype)
    c = P.plain_weight_norm(rows[:, H * dk:].double(), g.double(), 1e-6)
    c = c.to(dtype).double()                                              # what the cache holds
    scale = 1.7 / math.sqrt(dk)
    cache = CacheManager([(KVCacheSpec(1, r, window, planes=1), None)], page_size=page, num_pages=3 * (n // page + 1),
                         max_seqs=4, max_seq_len=max(512, n + 16), dtype=dtype, device=DEV)
    view = lambda: cache.view(ScheduleEntry(0, 0))
    spans = [(rid, head) for rid, (head, _e) in spans_of.items()]         # first the prefixes, in one step
    ctx, starts = _step_ctx(kernels, dtype, cache, spans)
    kernels.latent_norm_append(torch.cat([rows[:m] for _r, m in spans]).to(DEV), H * dk, r, g.to(DEV), 1e-6, ctx, view())
    _commit(cache, spans, starts)
    spans = [(rid, e - head) for rid, (head, e) in spans_of.items()]
    ctx, starts = _step_ctx(kernels, dtype, cache, spans)
    step_rows = torch.cat([rows[head:e] for head, e in spans_of.values()]).to(DEV).contiguous()
    kernels.latent_norm_append(step_rows, H * dk, r, g.to(DEV), 1e-6, ctx, view())
    got = kernels.latent_attention(step_rows, w_uk.to(DEV), w_uv.to(DEV), None if sinks is None else sinks.to(DEV),
                                   H, dk, dv, r, window, scale, ctx, view()).cpu().double()
    _commit(cache, spans, starts)
    kernels.check_errors()
    worst, yard, row = 0.0, 0.0, 0
    for rid, (head, end) in spans_of.items():
        for i in range(head, end):
            lo = max(0, i - W + 1)
            for a in range(H):
                q = rows[i, a * dk:(a + 1) * dk].double()
                s = (c[lo:i + 1] @ (w_uk.double()[a * dk:(a + 1) * dk].T @ q)) * scale
                p = P.windowed_sink_softmax(s, sinks[a].double() if sink else -1e30)
                want = w_uv.double()[a * dv:(a + 1) * dv] @ (p @ c[lo:i + 1])
                worst = max(worst, float((got[row, a * dv:(a + 1) * dv] - want).abs().max()) / (1e-3 + float(want.abs().max())))
                if dtype == torch.bfloat16:      # the yardstick: the same sums with the three roundings any bfloat16 path through latent space has
                    rb = lambda t: t.to(torch.bfloat16).double()
                    s2 = (c[lo:i + 1] @ rb(w_uk.double()[a * dk:(a + 1) * dk].T @ q)) * scale
                    p2 = P.windowed_sink_softmax(s2, sinks[a].double() if sink else -1e30)
                    rough = w_uv.double()[a * dv:(a + 1) * dv] @ rb(rb(p2) @ c[lo:i + 1])
                    yard = max(yard, float((rough - want).abs().max()) / (1e-3 + float(want.abs().max())))
            row += 1
    # bfloat16: up to three times what those roundings alone do to this case (its planted scores are 20 and more)
    return worst if dtype == torch.float32 else worst / max(1.0, 3.0 * yard / 2e-2)


# bfloat16 takes the tensor-core tiles for latents that are multiples of 16 (up to 256), else the per-token kernel
# (bfloat16: the planted keys have scores of 20 and more, so that rounding a query or a latent moves a weight by percents;
# _attention_case scales its result by what the unavoidable roundings do to the case, so the bound stays 2e-2)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("window,sink", [(37, True), (16, True), (17, False), (1, True), (None, True), (300, False)])
@pytest.mark.parametrize("r", [40, 64])
def test_latent_attention_kernels_planted_keys(cuda_kernels, dtype, tol, window, sink, r):
    assert _attention_case(cuda_kernels, dtype, window, sink, r=r) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("sizes", [(1, 8, 8, 24), (5, 16, 40, 72), (2, 64, 64, 128), (4, 24, 16, 200), (2, 128, 128, 512),
                                   (6, 24, 40, 48), (16, 32, 32, 256), (70, 8, 8, 32), (3, 16, 16, 16), (64, 8, 16, 80)])
def test_latent_attention_kernels_other_sizes(cuda_kernels, dtype, tol, sizes):
    H, dk, dv, r = sizes
    assert _attention_case(cuda_kernels, dtype, 45, True, H=H, dk=dk, dv=dv, r=r, n=140, seed=20) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("window", [None, 290, 130])
@pytest.mark.parametrize("sizes", [(3, 40, 24, 40), (4, 16, 24, 64), (16, 16, 16, 128), (2, 32, 32, 256)])
def test_latent_attention_decoded_tokens_alone(cuda_kernels, dtype, tol, window, sizes):
    """A step of single tokens only: the tiled kernel cuts the keys over several blocks and merges."""
    H, dk, dv, r = sizes
    assert _attention_case(cuda_kernels, dtype, window, True, H=H, dk=dk, dv=dv, r=r, n=420, seed=30, decode_only=True) < tol


@pytest.mark.parametrize("window", [None, 600, 300])
@pytest.mark.parametrize("sizes", [(4, 16, 24, 64), (12, 8, 8, 128), (3, 40, 24, 40)])
def test_latent_attention_prompt_portions_over_many_keys(cuda_kernels, window, sizes):
    """Portions behind 1,000 cached tokens: with few blocks and many keys the tiled kernel cuts the keys of
    prompt portions too, and merges."""
    H, dk, dv, r = sizes
    assert _attention_case(cuda_kernels, torch.bfloat16, window, True, H=H, dk=dk, dv=dv, r=r, n=1100, seed=70) < 2e-2
    assert _attention_case(cuda_kernels, torch.float32, window, True, H=H, dk=dk, dv=dv, r=r, n=1100, seed=70) < 2e-5


def test_latent_attention_tiles_against_the_per_token_kernel(cuda_kernels):
    """The two bfloat16 paths on the same case."""
    try:
        tiles = _attention_case(cuda_kernels, torch.bfloat16, 70, True, H=5, dk=24, dv=40, r=96, n=300, seed=50)
        cuda_kernels.latent_tiles = False
        plain = _attention_case(cuda_kernels, torch.bfloat16, 70, True, H=5, dk=24, dv=40, r=96, n=300, seed=50)
    finally:
        cuda_kernels.latent_tiles = True
    assert tiles < 2e-2 and plain < 2e-2


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
def test_latent_attention_part_alone(cuda_kernels, dtype, tol):
    """The mixer over its own cache, whole and in portions, against the plain function that makes keys and
    values of every head explicitly."""
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import PartSpec, ScheduleEntry
    from inferflux_b200.parts import build_part
    width, H, dk, dv, r, T, size = 88, 3, 16, 24, 40, 61, 19
    mixer = build_part("mixer", PartSpec("latent_attention", {
        "hidden_size": width, "num_heads": H, "qk_dim": dk, "v_dim": dv, "kv_rank": r, "window": size, "scale": 0.3,
        "latent_norm_eps": 1e-5, "sink": True}))
    tensors = {n: _rnd(*s.shape, seed=40 + i, scale=0.3).to(dtype) for i, (n, s) in enumerate(mixer.param_specs().items())}
    tensors["q"] = tensors["q"] * 4
    mixer.load(tensors, dtype, DEV)
    h = _rnd(T, width, seed=60).to(dtype)
    want = P.latent_attention(h.double(), {k: v.double() for k, v in tensors.items()}, "",
                              {"heads": H, "dim": dk, "vdim": dv, "kv_rank": r, "scale": 0.3, "mask": {"size": size}}, 1e-5)
    for cuts in ([T], [40, 21], [5, 1, 1, 2, 52]):
        cache = CacheManager([(mixer.cache_spec(), None)], page_size=4, num_pages=20, max_seqs=2, max_seq_len=64,
                             dtype=dtype, device=DEV)
        outs, pos = [], 0
        for n in cuts:
            ctx, starts = _step_ctx(cuda_kernels, dtype, cache, [("r", n)], providers=[mixer])
            outs.append(cuda_kernels.materialize(mixer.forward(h[pos:pos + n].to(DEV).contiguous(), ctx,
                                                               cache.view(ScheduleEntry(0, 0)))))
            _commit(cache, [("r", n)], starts)
            pos += n
        got = torch.cat(outs).float().cpu().double()
        assert float((got - want).abs().max()) < tol * float(want.abs().max()), f"cuts {cuts}"


# ------------------------------------------------------------------ whole models

LENS = [40, 33, 50, 61, 97, 70, 25, 64, 1, 2]


@pytest.fixture(scope="module")
def oracle(dafolorn_dirs):
    memo = {}

    def get(name):
        if name not in memo:
            d, _page, raw = dafolorn_dirs[name]
            reqs = dm.requests_for(raw, LENS, 100)
            memo[name] = {"reqs": reqs, "float32": dm.plain_logits(d, reqs),
                          "bfloat16": dm.plain_logits(d, reqs, weights_as=torch.bfloat16),
                          "yard": dm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16)}
        return memo[name]
    return get


def _runner(d, dtype, page, kernels, pages=None, **kw):
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    _c, model = load_model(d, dtype=dtype, device=DEV)
    return ModelRunner(model, kernels, page_size=page, num_pages=pages or 256 // page, max_seqs=4, max_seq_len=512, **kw)


def _bf16_close(name, got, want, yard):
    """bfloat16 logits against the exact ones.  The yardstick is the plain implementation run in bfloat16 arithmetic
    on the same rounded weights: what rounding alone does to this model.  These models are made sharp (scores of 20
    and more), so two correct bfloat16 computations that round at different places differ by about as much as either
    differs from the exact result; the engine may be up to three times as far off as the yardstick in the worst row,
    twice on average, and has to agree with the exact best token about as often."""
    err, bound = np.abs(got - want).max(axis=1), np.abs(yard - want).max(axis=1)
    assert float(err.max()) <= 3.0 * float(bound.max()), \
        f"{name}: row {int(err.argmax())} is off by {float(err.max()):.4f}; rounding alone gives {float(bound.max()):.4f}"
    assert float(err.mean()) <= 2.0 * float(bound.mean()), f"{name}: mean error {float(err.mean()):.4f} against {float(bound.mean()):.4f}"
    agree = float(np.mean(got.argmax(-1) == want.argmax(-1)))
    assert agree >= float(np.mean(yard.argmax(-1) == want.argmax(-1))) - 0.1, f"{name}: best token agrees at {agree:.2f}"


def _check(name, dtype, got, o):
    if dtype == "float32":
        top = max(float(np.abs(v).max()) for v in o["float32"].values())
        bad = helpers.first_bad(got, o["float32"], 2e-4 + 1e-5 * top)          # float32 rounding grows with the logits
        assert bad is None, f"{name}: first wrong row (request, position, diff): {bad}"
    else:
        for rid in o["reqs"]:
            _bf16_close(f"{name} {rid}", got[rid], o["bfloat16"][rid], o["yard"][rid])


@pytest.mark.parametrize("name", ["P", "Q", "R", "S", "U", "V"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_step_function_cuttings(name, dtype, cutting, dafolorn_dirs, oracle, cuda_kernels):
    d, page, raw = dafolorn_dirs[name]
    o = oracle(name)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, 256)}[cutting](o["reqs"])
    runner = _runner(d, dtype, page, cuda_kernels, cuda_graphs=(cutting == "tail"))
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"])
    cuda_kernels.check_errors()
    _check(f"{name} {cutting}", dtype, got, o)
    assert not runner.cache.live_requests()


@pytest.mark.parametrize("name", ["P", "U"])
def test_float32_is_the_same_under_every_cutting(name, dafolorn_dirs, oracle, cuda_kernels):
    d, page, raw = dafolorn_dirs[name]
    reqs = oracle(name)["reqs"]
    results = []
    for make in (helpers.trace_whole, helpers.trace_tail, helpers.trace_portions, lambda r: helpers.trace_mixed(r, 256)):
        steps = make(reqs)
        runner = _runner(d, "float32", page, cuda_kernels)
        results.append(helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"]))
    for other in results[1:]:
        for rid in reqs:
            assert np.array_equal(results[0][rid], other[rid]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_pages_given_back_and_graphs(dtype, dafolorn_dirs, cuda_kernels):
    """12 prompt tokens, then 300 decoded one by one beside a second request that joins and leaves: the windows
    pass over decoded tokens, pages are given back and used again, decode steps replay a CUDA graph."""
    from inferflux_b200.engine import StepEntry
    d, page, raw = dafolorn_dirs["U"]
    reqs = dm.requests_for(raw, [312, 90], 9)
    want = dm.plain_logits(d, reqs, weights_as=torch.bfloat16 if dtype == "bfloat16" else None)
    yard = dm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16) if dtype == "bfloat16" else None
    runner = _runner(d, dtype, page, cuda_kernels, pages=9, cuda_graphs=True)
    a, b = reqs["r0"], reqs["r1"]
    got = {"r0": [], "r1": []}
    got["r0"] += list(runner.step([StepEntry("r0", a[:12], list(range(12)))]).cpu().numpy())
    pb = 0
    for i in range(12, len(a)):
        entries = [StepEntry("r0", [a[i]], [0])]
        if 100 <= i and pb < len(b):
            n = 7 if pb < 49 else 1
            entries.append(StepEntry("r1", b[pb:pb + n], list(range(n))))
            pb += n
        out = runner.step(entries).cpu().numpy()
        got["r0"].append(out[0])
        got["r1"] += list(out[1:])
        if pb == len(b) and "r1" in runner.cache:
            runner.end_request("r1")
        runner.cache.check()
    cuda_kernels.check_errors()
    assert runner.graph_replays > 50
    got = {k: np.stack(v) for k, v in got.items()}
    for rid in reqs:
        if dtype == "float32":
            assert float(np.abs(got[rid] - want[rid]).max()) < 3e-4, rid
        else:
            _bf16_close(rid, got[rid], want[rid], yard[rid])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, dafolorn_dirs, oracle, tmp_path):
    d, page, raw = dafolorn_dirs["R"]
    o = oracle("R")
    steps = helpers.trace_mixed(o["reqs"], 256)
    got = helpers.collect(steps, helpers.run_trace_cli(d, dtype, steps, tmp_path / "out", 256, raw["vocab"], page_size=page),
                          raw["vocab"])
    _check("R through the program", dtype, got, o)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_engine_and_scheduler(dtype, dafolorn_dirs):
    from inferflux_b200 import Engine, SamplingParams
    d, page, raw = dafolorn_dirs["P"]
    _raw, W = dm.load(d)
    if dtype == "bfloat16":
        W = {k: v.to(torch.bfloat16) for k, v in W.items()}
    prompts = list(dm.requests_for(raw, [7, 19, 33, 4, 1, 70], 40).values())
    for pages in (64, 14):                                 # 14 pages of 8: the requests do not all fit at once
        eng = Engine(d, dtype=dtype, device=DEV, kv_page_size=page, kv_num_pages=pages, kv_max_batch=4, kv_max_seq=128,
                     chunked_prefill_tokens=16, max_batch_tokens=48)
        res = eng.generate(prompts, SamplingParams(temperature=0.0), max_tokens=24)
        for prompt, r in zip(prompts, res):
            seq = list(prompt) + list(r.token_ids)
            exact = P.forward(raw, W, seq)
            rough = P.forward(raw, W, seq, dtype=torch.bfloat16).double() if dtype == "bfloat16" else None
            for i, tok in enumerate(r.token_ids):
                row = len(prompt) - 1 + i
                gap = float(exact[row].max() - exact[row, tok])
                slack = 1e-3 if rough is None else 2.0 * float((rough[row] - exact[row]).abs().max())
                assert gap <= slack, f"token {i}: {gap:.4f} below the best logit, rounding allows {slack:.4f}"
        assert not eng.runner.cache.live_requests()
