"""Zeluzen on the GPU: every new kernel alone against the plain kernel statements (themselves held to the plain
implementation by the CPU tests), then whole models through the step function, the replay program and the engine."""
import math

import numpy as np
import pytest
import torch

import helpers
import zeluzen_models as zm
from plain import plain_zeluzen as P
from plain.plain_kernels import PlainKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def _rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.fixture(scope="module")
def zeluzen_dirs(tmp_path_factory):
    out = {}
    for i, (name, (raw, page)) in enumerate(zm.configs().items()):
        out[name] = (zm.write_model(raw, tmp_path_factory.mktemp(f"zeluzen_{name}"), seed=51 + i), page, raw)
    return out


class _Ctx:
    """The few fields of a step context that the kernels of this file read, on a device."""

    def __init__(self, spans, slots, device):
        cu, pos, req = [0], [], []
        for r, (start, n) in enumerate(spans):
            cu.append(cu[-1] + n)
            pos += list(range(start, start + n))
            req += [r] * n
        mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        self.cu_seqlens, self.positions, self.token_req, self.req_slot = mk(cu), mk(pos), mk(req), mk(slots)
        self.num_requests, self.num_tokens = len(spans), cu[-1]
        self.spans, self.slots_host = list(spans), list(slots)
        self.max_span = max(n for _s, n in spans)
        self.max_kv_len = max(s + n for s, n in spans)
        self.extra, self.extra_len = {}, {}


class _Cache:
    def __init__(self, kv, table, page_size, writes=True, state=None):
        self.kv, self.block_table, self.page_size, self.writes, self.state = kv, table, page_size, writes, state


# ------------------------------------------------------------------ the recurrence

@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 8e-3)])
def test_token_shift_mix_cast_tanh(cuda_kernels, dtype, tol):
    C, spans, slots = 72, [(0, 5), (9, 1), (3, 2)], [2, 0, 3]
    T = sum(n for _s, n in spans)
    x, mu = _rnd(T, C, seed=1), torch.rand(5, C, generator=torch.Generator().manual_seed(2))
    state = _rnd(4, 30 + C, seed=3)
    want = PlainKernels(wide=True).token_shift_mix(x, mu, state, 30, _Ctx(spans, slots, "cpu"), torch.float32)
    got = cuda_kernels.token_shift_mix(x.to(DEV), mu.to(DEV), state.to(DEV), 30, _Ctx(spans, slots, DEV), dtype)
    assert got.dtype == dtype and float((got.float().cpu() - want).abs().max()) <= tol * 4
    assert torch.allclose(want[:, 0], x[0] + (state[2, 30:] - x[0]) * mu, atol=1e-6)        # a span's first row reads the state
    assert torch.equal(cuda_kernels.cast_rows(x.to(DEV), dtype).cpu(), x.to(dtype))
    z = _rnd(7, 33, seed=4, scale=2.0).to(dtype)
    assert float((cuda_kernels.tanh(z.to(DEV)).float().cpu() - torch.tanh(z.float())).abs().max()) <= tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H,D", [(3, 8), (2, 24), (4, 32), (2, 64), (1, 128), (2, 160), (5, 40)])
def test_recurrence_over_steps_and_requests(cuda_kernels, dtype, tol, H, D):
    """Three requests over four steps: portions of 1 to 37 tokens (more and fewer than the 16 the kernel stages), a
    request that sits a step out, states carried in slots; against the plain statement in float64."""
    C, HD = 48, H * D
    plain = PlainKernels(wide=True)
    state_g = torch.zeros(4, H * D * D + C, dtype=torch.float32, device=DEV)
    state_p = torch.zeros(4, H * D * D + C, dtype=F64)
    g = torch.Generator().manual_seed(H * 100 + D)
    w0, u, nw = torch.randn(HD, generator=g) - 1.0, 0.5 * torch.randn(HD, generator=g), 1 + 0.2 * torch.randn(HD, generator=g)
    starts = [0, 0, 0]
    for step, lens in enumerate([(37, 1, 5), (1, 16, 0), (2, 17, 1), (1, 1, 1)]):
        spans, slots = [], []
        for q, n in enumerate(lens):
            if n:
                spans.append((starts[q], n))
                slots.append([3, 0, 2][q])
                starts[q] += n
        T = sum(n for _s, n in spans)
        r, k, v, g_in = (torch.randn(T, HD, generator=g) for _ in range(4))
        w_raw = torch.randn(T, HD, generator=g)
        x = torch.randn(T, C, generator=g)
        want = plain.wkv_scan(r, k, v, w_raw, g_in, w0, u, nw, 1e-5, H, D, state_p, H * D * D, x.double(), _Ctx(spans, slots, "cpu"), F64)
        got = cuda_kernels.wkv_scan(*(t.to(DEV) for t in (r, k, v, w_raw, g_in, w0, u, nw)), 1e-5, H, D, state_g, H * D * D,
                                    x.to(DEV), _Ctx(spans, slots, DEV), dtype)
        scale = float(want.abs().max())
        assert float((got.double().cpu() - want).abs().max()) <= tol * max(1.0, scale), (step, H, D)
        assert float((state_g.double().cpu() - state_p).abs().max()) <= 2e-5 * max(1.0, float(state_p.abs().max()))
    assert float(state_g[1].abs().max()) == 0.0                                # a slot nobody had stays untouched


def test_recurrence_is_the_same_however_it_is_cut(cuda_kernels):
    H, D, C, T = 2, 32, 40, 53
    g = torch.Generator().manual_seed(9)
    r, k, v, gi, wr = (torch.randn(T, H * D, generator=g).to(DEV) for _ in range(5))
    w0, u, nw = (torch.randn(H * D, generator=g).to(DEV) for _ in range(3))
    x = torch.randn(T, C, generator=g).to(DEV)

    def run(cuts):
        state = torch.zeros(1, H * D * D + C, dtype=torch.float32, device=DEV)
        out, pos = [], 0
        for n in cuts:
            sl = slice(pos, pos + n)
            out.append(cuda_kernels.wkv_scan(r[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), wr[sl].contiguous(),
                                             gi[sl].contiguous(), w0, u, nw, 1e-6, H, D, state, H * D * D, x[sl].contiguous(),
                                             _Ctx([(pos, n)], [0], DEV), torch.float32))
            pos += n
        return torch.cat(out), state
    whole, s0 = run([T])
    for cuts in ([1] * T, [16, 16, 16, 5], [2, 31, 1, 17, 2]):
        got, s1 = run(cuts)
        assert torch.equal(got, whole) and torch.equal(s0, s1), cuts


# ------------------------------------------------------------------ the mixture of experts

@pytest.mark.parametrize("n,top", [(5, 1), (20, 3), (7, 7), (300, 8), (1, 1)])
def test_router_choice_and_weights(cuda_kernels, n, top):
    T = 19
    z, corr = _rnd(T, n, seed=n, scale=2.0), _rnd(n, seed=n + 1, scale=0.2)
    ids, w = cuda_kernels.moe_route(z.to(DEV), corr.to(DEV), top)
    want_ids, want_w = PlainKernels(wide=True).moe_route(z, corr, top)
    assert torch.equal(ids.cpu().sort(dim=1).values, want_ids.sort(dim=1).values)
    s = torch.softmax(z.double(), dim=-1)
    assert float((w.cpu().double() - torch.gather(s, 1, ids.cpu().long())).abs().max()) < 1e-6   # the scores, uncorrected
    ids0, _w0 = cuda_kernels.moe_route(z.to(DEV), None, top)
    assert torch.equal(ids0.cpu().sort(dim=1).values, torch.topk(z, top, dim=1).indices.sort(dim=1).values.to(torch.int32))
    if top < n and n > 3:
        assert not torch.equal(ids0.cpu().sort(dim=1).values, ids.cpu().sort(dim=1).values)      # the correction steers


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("sizes", [(64, 24, 3, 2, 2), (100, 50, 1, 0, 1), (48, 16, 0, 3, 2), (256, 96, 6, 1, 4), (72, 33, 4, 0, 4)])
def test_experts_against_the_plain_statement(cuda_kernels, dtype, tol, sizes):
    width, ff, experts, identity, top = sizes
    T = 11
    h = _rnd(T, width, seed=1).to(dtype)
    up = _rnd(max(experts, 1), ff, width, seed=2, scale=width ** -0.5).to(dtype)
    down = _rnd(max(experts, 1), width, ff, seed=3, scale=ff ** -0.5).to(dtype)
    g = torch.Generator().manual_seed(4)
    ids = torch.stack([torch.randperm(experts + identity, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top, generator=g)
    want = PlainKernels(wide=True).moe_experts(h, up, down, ids, wts, experts, F64)
    got = cuda_kernels.moe_experts(h.to(DEV), up.to(DEV) if experts else None, down.to(DEV) if experts else None, ids.to(DEV),
                                   wts.to(DEV), experts, dtype)
    assert float((got.double().cpu() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    if identity:                                            # a token that chose only input-passing experts gets its input back
        ids2 = torch.full((T, 1), experts, dtype=torch.int32)
        got2 = cuda_kernels.moe_experts(h.to(DEV), up.to(DEV) if experts else None, down.to(DEV) if experts else None,
                                        ids2.to(DEV), torch.full((T, 1), 0.5).to(DEV), experts, torch.float32)
        assert float((got2.cpu() - 0.5 * h.float()).abs().max()) < 1e-6


@pytest.mark.parametrize("sizes", [(64, 24, 3, 2, 2, 300), (256, 96, 6, 1, 4, 700), (136, 200, 16, 0, 8, 130), (72, 40, 9, 3, 1, 1100)])
def test_experts_as_sorted_tiles_against_the_per_token_kernels(cuda_kernels, sizes, monkeypatch):
    """Many tokens in bfloat16: the sorted tensor-core tiles against the per-token kernels and the plain statement,
    with experts that nobody chose, experts with more than one tile of rows, and input-passing experts."""
    width, ff, experts, identity, top, T = sizes
    bf = torch.bfloat16
    h = _rnd(T, width, seed=1).to(bf)
    up = _rnd(experts, ff, width, seed=2, scale=width ** -0.5).to(bf)
    down = _rnd(experts, width, ff, seed=3, scale=ff ** -0.5).to(bf)
    g = torch.Generator().manual_seed(4)
    pool = torch.tensor([e for e in range(experts + identity) if e != 1])            # expert 1 is never chosen
    ids = torch.stack([pool[torch.randperm(len(pool), generator=g)[:top]] for _ in range(T)]).to(torch.int32)
    ids[: T // 2, 0] = 0                                                              # expert 0 gets rows for several tiles
    wts = torch.rand(T, top, generator=g)
    args = (h.to(DEV), up.to(DEV), down.to(DEV), ids.to(DEV), wts.to(DEV), experts, bf)
    assert T * top >= cuda_kernels.MOE_TILES_MIN_PAIRS
    launches = cuda_kernels.launches
    tiles = cuda_kernels.moe_experts(*args).float().cpu()
    assert cuda_kernels.launches - launches == 5
    cuda_kernels.check_errors()
    monkeypatch.setenv("INFERFLUX_B200_MOE_TILES", "0")
    rows = cuda_kernels.moe_experts(*args).float().cpu()
    want = PlainKernels(wide=True).moe_experts(h, up, down, ids, wts, experts, F64)
    scale = max(1.0, float(want.abs().max()))
    assert float((tiles.double() - want).abs().max()) <= 2e-2 * scale and float((rows.double() - want).abs().max()) <= 2e-2 * scale
    assert float((tiles - rows).abs().max()) <= 2e-2 * scale


# ------------------------------------------------------------------ attention: head norms, chunks, sink, value size

def _attention_setup(cuda_kernels, dtype, nq, nkv, d, dv, page, n, seed):
    """Keys and values of one request of n tokens written through the rotate-and-append kernel in two steps."""
    from inferflux_b200.parts.base import RotaryTable
    row = -(-max(d, dv) // 8) * 8
    pages = -(-n // page) + 1
    kv = torch.zeros(pages, 2, nkv, page, row, dtype=dtype, device=DEV)
    table = torch.zeros(2, pages, dtype=torch.int32, device=DEV)
    table[1] = torch.arange(pages - 1, -1, -1, dtype=torch.int32)          # slot 1, pages in reverse order
    qkv = _rnd(n, (nq + nkv) * d + nkv * dv, seed=seed)
    qn, kn = 1 + 0.3 * _rnd(d, seed=seed + 1), 1 + 0.3 * _rnd(d, seed=seed + 2)
    rot = RotaryTable(torch.tensor([0.7 ** i for i in range(d // 4)], dtype=torch.float32, device=DEV), d // 2, True)
    return kv, table, qkv, qn, kn, rot


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("sizes", [(4, 2, 16, 24, 8), (3, 3, 32, 8, 16), (6, 1, 8, 8, 4), (2, 2, 64, 64, 16), (5, 5, 12, 20, 16)])
def test_normed_heads_rotation_and_cache_write(cuda_kernels, dtype, tol, sizes):
    nq, nkv, d, dv, page = sizes
    n = 37
    kv, table, qkv, qn, kn, rot = _attention_setup(cuda_kernels, dtype, nq, nkv, d, dv, page, n, 5)
    plain = PlainKernels(wide=True)
    kv_p, rot_p = torch.zeros(kv.shape, dtype=F64), type(rot)(rot.inv_freq.cpu(), rot.rotary_dim, True)
    for lo, hi in ((0, 30), (30, 37)):
        rows = qkv[lo:hi].to(dtype)
        q = cuda_kernels.rope_append(rows.to(DEV), None, rot, nq, nkv, d, _Ctx([(lo, hi - lo)], [1], DEV),
                                     _Cache(kv, table, page), q_norm=qn.to(DEV), k_norm=kn.to(DEV), norm_eps=1e-5, dv=dv)
        q_p = plain.rope_append(rows.double(), None, rot_p, nq, nkv, d, _Ctx([(lo, hi - lo)], [1], "cpu"),
                                _Cache(kv_p, table.cpu(), page), q_norm=qn, k_norm=kn, norm_eps=1e-5, dv=dv)
        assert float((q.double().cpu() - q_p).abs().max()) <= tol * 4
    assert float((kv.double().cpu() - kv_p).abs().max()) <= tol * 4
    assert float(kv[..., max(d, dv):].abs().max()) == 0.0 if kv.shape[-1] > max(d, dv) else True
    # queries only, nothing stored: the cache stays as it is
    before = kv.clone()
    q_only = qkv[:5, :nq * d].contiguous().to(dtype)
    q2 = cuda_kernels.rope_append(q_only.to(DEV), None, rot, nq, nkv, d, _Ctx([(0, 5)], [1], DEV), _Cache(kv, table, page, writes=False),
                                  q_norm=qn.to(DEV), norm_eps=1e-5, dv=dv, own_kv=False)
    want2 = plain.rope_append(qkv[:5].to(dtype).double(), None, rot_p, nq, nkv, d, _Ctx([(0, 5)], [1], "cpu"),
                              _Cache(torch.zeros(kv.shape, dtype=F64), table.cpu(), page), q_norm=qn, k_norm=kn, norm_eps=1e-5, dv=dv)
    assert torch.equal(kv, before) and float((q2.double().cpu() - want2).abs().max()) <= tol * 4


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("chunk", [None, 1, 7, 16, 24, 300])
@pytest.mark.parametrize("sizes", [(4, 2, 16, 24, 8), (2, 2, 64, 64, 16), (6, 1, 8, 40, 16), (4, 2, 32, 32, 8), (8, 2, 128, 128, 16)])
def test_attention_with_chunks_and_sink_planted_keys(cuda_kernels, dtype, tol, chunk, sizes):
    """One key is made to stand out for one query at a time: far back, at a page border, just inside and just outside
    the query's chunk, in a prompt portion and in a token decoded alone.  The output must be that key's value when
    it is seen and must not change at all when it is not."""
    nq, nkv, d, dv, page = sizes
    n, row = 150, -(-max(d, dv) // 8) * 8
    pages = -(-n // page)
    g = torch.Generator().manual_seed(11)
    K = (0.1 * torch.randn(n, nkv, d, generator=g)).to(dtype)
    V = torch.randn(n, nkv, dv, generator=g).to(dtype)
    order = torch.randperm(pages, generator=g).to(torch.int32)
    table = torch.zeros(3, pages, dtype=torch.int32)
    table[2] = order

    def pool(Kx):
        kv = torch.zeros(pages, 2, nkv, page, row, dtype=dtype)
        for j in range(n):
            kv[order[j // page], 0, :, j % page, :d] = Kx[j]
            kv[order[j // page], 1, :, j % page, :dv] = V[j]
        return kv
    plain = PlainKernels(wide=True)
    for qpos in (n - 1, 96, 17):
        first = 0 if not chunk else qpos // chunk * chunk
        for key in {0, first - 1, first, (qpos // page) * page, (qpos // page) * page - 1, qpos}:
            if key < 0 or key > qpos:
                continue
            Kx = K.clone()
            qvec = torch.randn(nq, d, generator=g)
            qvec = qvec / qvec.norm(dim=-1, keepdim=True)
            for h in range(nq):                               # the planted key answers this head's query with a score of 30
                Kx[key, h // (nq // nkv)] = (30.0 * qvec[h]).to(dtype)
            qrows = torch.zeros(3, nq * d)
            qrows[1] = qvec.reshape(-1)
            for spans in ([(qpos - 1, 3)] if qpos + 2 <= n else [(qpos - 1, 2)], [(qpos, 1)]):
                at = 1 if spans[0][1] > 1 else 0
                T = spans[0][1]
                q = torch.zeros(T, nq * d)
                q[at] = qvec.reshape(-1)
                q = q.to(dtype)
                outs = []
                for Kuse in (Kx, K):
                    kv = pool(Kuse)
                    got = cuda_kernels.attention(q.to(DEV), nq, nkv, d, None, 1.0, _Ctx(spans, [2], DEV), _Cache(kv.to(DEV), table.to(DEV), page),
                                                 chunk=chunk, sink=True, dv=dv)
                    want = plain.attention(q.double(), nq, nkv, d, None, 1.0, _Ctx(spans, [2], "cpu"), _Cache(kv.double(), table, page),
                                           chunk=chunk, sink=True, dv=dv)
                    assert float((got.double().cpu() - want).abs().max()) <= tol * 4, (qpos, key, spans)
                    outs.append(got[at].float().cpu().view(nq, dv))
                seen = key >= first
                if seen and nq // nkv == 1:
                    assert float((outs[0] - V[key].float()).abs().max()) < 0.05, (qpos, key, "a key inside the chunk is not used")
                if not seen:
                    assert torch.equal(outs[0], outs[1]), (qpos, key, "a key outside the chunk changes the result")
    # the sink: with scores far below zero almost nothing is left of the values; without it the softmax is a plain one
    kv = pool(K)
    q = torch.cat([-40.0 * K[5, h // (nq // nkv)].float() for h in range(nq)]).view(1, nq * d).to(dtype)
    ctx, cache = _Ctx([(5, 1)], [2], DEV), _Cache(kv.to(DEV), table.to(DEV), page)
    with_sink = cuda_kernels.attention(q.to(DEV), nq, nkv, d, None, 25.0, ctx, cache, chunk=1, sink=True, dv=dv)
    assert float(with_sink.float().abs().max()) < 1e-2 * float(V[5].float().abs().max())


@pytest.mark.parametrize("chunk", [None, 1024, 300, 64])
@pytest.mark.parametrize("sizes", [(8, 2, 128, 16), (4, 4, 64, 16), (6, 2, 32, 8), (16, 1, 96, 32)])
def test_masked_attention_tiles_against_the_per_token_kernel(cuda_kernels, chunk, sizes, monkeypatch):
    """bfloat16: three requests with 1,500, 700 and 40 cached keys; a step that decodes one token of the first two and
    brings a portion of 300 of a fourth, a step with that request's next 333 tokens (tiles that begin in the middle of
    a chunk), and a step of single tokens only (the key range cut over a cluster)."""
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import ScheduleEntry
    from inferflux_b200.engine.batch import StepContext, StepEntry
    from inferflux_b200.parts import KVCacheSpec
    nq, nkv, d, page = sizes
    bf = torch.bfloat16
    cache = CacheManager([(KVCacheSpec(nkv, d, None), None)], page_size=page, num_pages=3000 // page + 8, max_seqs=4,
                         max_seq_len=2048, dtype=bf, device=DEV)
    cache.groups[0].pool.normal_()
    cache.groups[0].pool[:, :, 0] *= 0.3                                     # keys: scores that are no flat softmax

    def step(spans):
        entries, starts, slots = [], [], []
        for rid, n in spans:
            if rid not in cache:
                cache.add_request(rid)
            start = cache.length(rid)
            cache.reserve(rid, start + n)
            entries.append(StepEntry(rid, [0] * n, []))
            starts.append(start)
            slots.append(cache.slot(rid))
        ctx = StepContext.build(cuda_kernels, bf, DEV, entries, starts, slots, cache.drain_table_updates())
        for g, (idx, pg) in zip(cache.groups, ctx.table_updates):
            cuda_kernels.scatter_i32(g.table, idx, pg)
        for (rid, n), start in zip(spans, starts):
            cache.commit(rid, start + n)
        return ctx
    step([("a", 1499), ("b", 699), ("c", 39)])
    view = cache.view(ScheduleEntry(0, 0))
    for spans in ([("a", 1), ("b", 1), ("d", 300)], [("d", 333), ("c", 1)], [("a", 1), ("b", 1), ("c", 1)]):
        ctx = step(spans)
        T = ctx.num_tokens
        q = _rnd(T, nq * d, seed=T).to(bf).to(DEV)
        outs = []
        for tiles in ("1", "0"):
            monkeypatch.setenv("INFERFLUX_B200_MASKED_TILES", tiles)
            launches = cuda_kernels.launches
            outs.append(cuda_kernels.attention(q, nq, nkv, d, None, d ** -0.5, ctx, view, chunk=chunk, sink=True).float())
            assert cuda_kernels.launches - launches == (1 if tiles == "0" else len({n == 1 for _r, n in spans}))
        cuda_kernels.check_errors()
        assert float((outs[0] - outs[1]).abs().max()) < 2e-2, (spans, float((outs[0] - outs[1]).abs().max()))
        # without the sink the weights sum to one: the outputs are larger
        plain = cuda_kernels.attention(q, nq, nkv, d, None, d ** -0.5, ctx, view, chunk=chunk or 4096, sink=False).float()
        assert float(plain.abs().mean()) > float(outs[0].abs().mean())


def test_postnorm_add_hands_on_the_rows_themselves(cuda_kernels):
    for T, H in ((5, 72), (600, 256)):
        x, y, w = _rnd(T, H, seed=1, scale=2.0), _rnd(T, H, seed=2).to(torch.bfloat16), 1 + 0.2 * _rnd(H, seed=3)
        xp = x.clone().double()
        want = PlainKernels(wide=True).postnorm_add(xp, y, w, 1e-5, out_dtype=torch.bfloat16, cast_out=True)
        xg = x.to(DEV)
        got = cuda_kernels.postnorm_add(xg, y.to(DEV), w.to(DEV), 1e-5, out_dtype=torch.bfloat16, cast_out=True)
        assert float((xg.cpu().double() - xp).abs().max()) < 1e-5 and torch.equal(got.cpu(), xg.cpu().to(torch.bfloat16))


# ------------------------------------------------------------------ whole models

LENS = [40, 33, 50, 61, 97, 70, 25, 64, 1, 2]


@pytest.fixture(scope="module")
def oracle(zeluzen_dirs):
    memo = {}

    def get(name):
        if name not in memo:
            d, _page, raw = zeluzen_dirs[name]
            reqs = zm.requests_for(raw, LENS, 100)
            memo[name] = {"reqs": reqs, "float32": zm.plain_logits(d, reqs),
                          "bfloat16": zm.plain_logits(d, reqs, weights_as=torch.bfloat16),
                          "yard": zm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16)}
        return memo[name]
    return get


def _runner(d, dtype, page, kernels, pages=None, **kw):
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    _c, model = load_model(d, dtype=dtype, device=DEV)
    return ModelRunner(model, kernels, page_size=page, num_pages=pages or 256 // page, max_seqs=4, max_seq_len=512, **kw)


def _bf16_close(name, got, want, yard):
    """bfloat16 logits against the exact ones, with the plain implementation in bfloat16 arithmetic on the same rounded
    weights as the yardstick.  The test models are sharp and their routers decide by small margins, so two correct
    bfloat16 computations differ by about as much as either differs from the exact result: up to three times the
    yardstick's worst row, twice on average.  A router whose margin is below what rounding moves sends a token to
    another expert in one computation and not in the other; both are right, so one row in fifty may lie further out."""
    err, bound = np.abs(got - want).max(axis=1), np.abs(yard - want).max(axis=1)
    far = int((err > 3.0 * float(bound.max())).sum())
    assert far <= max(1, len(err) // 50) and float(err.max()) <= 12.0 * float(bound.max()), \
        f"{name}: row {int(err.argmax())} is off by {float(err.max()):.4f} ({far} rows far out); rounding alone gives {float(bound.max()):.4f}"
    assert float(err.mean()) <= 2.0 * float(bound.mean()), f"{name}: mean error {float(err.mean()):.4f} against {float(bound.mean()):.4f}"


def _check(name, dtype, got, o):
    if dtype == "float32":
        top = max(float(np.abs(v).max()) for v in o["float32"].values())
        bad = helpers.first_bad(got, o["float32"], 2e-4 + 1e-5 * top)
        assert bad is None, f"{name}: first wrong row (request, position, diff): {bad}"
    else:
        for rid in o["reqs"]:
            _bf16_close(f"{name} {rid}", got[rid], o["bfloat16"][rid], o["yard"][rid])


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_step_function_cuttings(name, dtype, cutting, zeluzen_dirs, oracle, cuda_kernels):
    d, page, raw = zeluzen_dirs[name]
    o = oracle(name)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, 256)}[cutting](o["reqs"])
    runner = _runner(d, dtype, page, cuda_kernels, cuda_graphs=(cutting == "tail"))
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"])
    cuda_kernels.check_errors()
    _check(f"{name} {cutting}", dtype, got, o)
    assert not runner.cache.live_requests()


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_is_the_same_under_every_cutting(name, zeluzen_dirs, oracle, cuda_kernels):
    d, page, raw = zeluzen_dirs[name]
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
def test_medium_model_with_long_prompts(dtype, tmp_path, cuda_kernels):
    """Prompts of 700 and 300 tokens through a model of seven layers: whole, then in portions of 128 and 200 beside
    each other's decoded tokens.  These steps reach the kernels of many rows (library and tcgen05 products, sorted
    expert tiles, the tensor-core attention with chunks and a sink, the scan's long spans) inside a whole model."""
    from inferflux_b200.engine import StepEntry
    raw, page = zm.medium_config()
    d = zm.write_model(raw, tmp_path / "medium", seed=77)
    reqs = zm.requests_for(raw, [700, 300], 12)
    rows = {"r0": [0, 1, 127, 128, 129, 255, 256, 257, 383, 384, 511, 512, 640, 698, 699], "r1": [0, 63, 64, 127, 128, 200, 298, 299]}
    rounded = torch.bfloat16 if dtype == "bfloat16" else None
    want = {k: v[rows[k]] for k, v in zm.plain_logits(d, reqs, weights_as=rounded).items()}
    yard = {k: v[rows[k]] for k, v in zm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16).items()} \
        if dtype == "bfloat16" else None

    def compare(name, got):
        for rid in reqs:
            if dtype == "float32":
                assert float(np.abs(got[rid] - want[rid]).max()) < 5e-4, (name, rid, float(np.abs(got[rid] - want[rid]).max()))
            else:
                _bf16_close(f"{name} {rid}", got[rid], want[rid], yard[rid])
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    _c, model = load_model(d, dtype=dtype, device=DEV)
    runner = ModelRunner(model, cuda_kernels, page_size=page, num_pages=80, max_seqs=4, max_seq_len=1024)
    got = {}
    for rid, toks in reqs.items():
        got[rid] = runner.step([StepEntry(rid, toks, rows[rid])]).cpu().numpy()
        runner.end_request(rid)
    cuda_kernels.check_errors()
    compare("whole", got)
    # portions of both side by side, then the last tokens one by one beside the other's portions
    got = {rid: {} for rid in reqs}
    at = {"r0": 0, "r1": 0}
    size = {"r0": 200, "r1": 128}
    while any(at[r] < len(reqs[r]) for r in reqs):
        entries, asked = [], []
        for rid, toks in reqs.items():
            if at[rid] >= len(toks):
                continue
            n = 1 if len(toks) - at[rid] <= 20 else min(size[rid], len(toks) - 20 - at[rid])
            w = [p - at[rid] for p in rows[rid] if at[rid] <= p < at[rid] + n]
            entries.append(StepEntry(rid, toks[at[rid]:at[rid] + n], w))
            asked += [(rid, p) for p in rows[rid] if at[rid] <= p < at[rid] + n]
            at[rid] += n
        out = runner.step(entries).cpu().numpy()
        for (rid, p), row in zip(asked, out):
            got[rid][p] = row
        for rid in reqs:
            if at[rid] == len(reqs[rid]) and rid in runner.cache:
                runner.end_request(rid)
        runner.cache.check()
    cuda_kernels.check_errors()
    compare("portions", {rid: np.stack([got[rid][p] for p in rows[rid]]) for rid in reqs})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_pages_given_back_and_graphs(dtype, zeluzen_dirs, cuda_kernels):
    """12 prompt tokens, then 300 decoded one by one beside a second request that joins and leaves: chunk borders are
    crossed by decoded tokens, pages are given back and used again, states live in slots, decode steps replay a CUDA graph."""
    from inferflux_b200.engine import StepEntry
    d, page, raw = zeluzen_dirs["A"]
    reqs = zm.requests_for(raw, [312, 90], 9)
    want = zm.plain_logits(d, reqs, weights_as=torch.bfloat16 if dtype == "bfloat16" else None)
    yard = zm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16) if dtype == "bfloat16" else None
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
def test_trace_run_program(dtype, zeluzen_dirs, oracle, tmp_path):
    d, page, raw = zeluzen_dirs["B"]
    o = oracle("B")
    steps = helpers.trace_mixed(o["reqs"], 256)
    got = helpers.collect(steps, helpers.run_trace_cli(d, dtype, steps, tmp_path / "out", 256, raw["vocab"], page_size=page),
                          raw["vocab"])
    _check("B through the program", dtype, got, o)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_engine_and_scheduler(dtype, zeluzen_dirs):
    from inferflux_b200 import Engine, SamplingParams
    d, page, raw = zeluzen_dirs["A"]
    _raw, W = zm.load(d)
    if dtype == "bfloat16":
        W = {k: v.to(torch.bfloat16) for k, v in W.items()}
    prompts = list(zm.requests_for(raw, [7, 19, 33, 4, 1, 70], 40).values())
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
