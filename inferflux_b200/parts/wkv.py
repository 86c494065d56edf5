"""A mixer that keeps, per head, a matrix of state (key channels x value channels) instead of a cache of keys.

With h' the input of the token before (zeros in front of a sequence), five mixes of the two,
m_s = h + (h' - h) * mu_s for s in r, k, v, g, w, feed five projections:

    r, k, v = W_r m_r, W_k m_k, W_v m_v      (heads x dim each)        gate = silu(W_g m_g)
    decay   = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))                      per head and key channel, in (0, 1)
    out_t   = (S + diag(u) k_t v_t^T)^T r_t                            u: a bonus the present token alone gets
    S       = diag(decay_t) S + k_t v_t^T
    y       = W_o ((out / rms(out) per head) * norm * gate)

S (float32) and the last input row are the request's state: a slot of fixed size, whatever the length,
zeroed when a request is admitted.  The mixes are made from the float32 residual stream itself; the
projections take them in the run's dtype and hand r, k, v, the decay's exponent and the gate to the
recurrence in float32, where everything else happens in float32 too.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Mixer, StateSpec, WeightBuffers, register_part

_MIXES = ("r", "k", "v", "g", "w")


@register_part("mixer", "wkv")
class WKV(Mixer):
    """params: hidden_size, num_heads, head_dim, decay_rank (None: the file's `w1` says; random weights then
    use 16 or a quarter of the width, whichever is smaller), norm_eps (of the per-head norm of the output),
    names (tensor names of mu_r .. mu_w, r, k, v, g, w1, w2, w0, u, norm, o)."""

    takes_stream = True               # the mixes are made from the float32 rows
    STACK_MAX_TOKENS = 32             # up to this many tokens a step the four projections run as one product

    _NAMES = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w", "r": "r", "k": "k",
              "v": "v", "g": "g", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u", "norm": "norm", "o": "o"}

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dim = int(p["head_dim"])
        if self.hidden <= 0 or self.heads <= 0 or self.dim <= 0:
            raise ValueError("wkv: sizes must be positive")
        if self.dim > 256:
            raise ValueError(f"wkv: a head size of {self.dim} is beyond the kernel's 256")
        self.rank = None if p.get("decay_rank") is None else int(p["decay_rank"])
        self.eps = float(p.get("norm_eps", 1e-6))
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})
        self.mu = self.w = self.w0 = self.u = self.norm_w = None

    # ---------------------------------------------------------------- declarations
    def state_spec(self):
        """[heads * dim * dim floats of S, then the last input row]."""
        return StateSpec((self.heads * self.dim * self.dim + self.hidden,), torch.float32)

    def param_specs(self):
        n, HD, C = self.names, self.heads * self.dim, self.hidden
        rank = -1 if self.rank is None else self.rank
        made = self.rank if self.rank is not None else max(1, min(16, C // 4))
        specs = {n["mu_" + s]: TensorSpec((C,), init="zeros") for s in _MIXES}
        for s in ("r", "k", "v", "g"):
            specs[n[s]] = TensorSpec((HD, C))
        specs[n["w1"]] = TensorSpec((rank, C), made_shape=(made, C))
        specs[n["w2"]] = TensorSpec((HD, rank), made_shape=(HD, made))
        specs[n["w0"]] = TensorSpec((HD,), init="zeros")
        specs[n["u"]] = TensorSpec((self.heads, self.dim), init="zeros")
        specs[n["norm"]] = TensorSpec((HD,), init="ones")
        specs[n["o"]] = TensorSpec((C, HD))
        return specs

    def load(self, tensors, dtype, device):
        n, HD, C = self.names, self.heads * self.dim, self.hidden
        rank = int(tensors[n["w1"]].shape[0])
        if tensors[n["w2"]].shape[1] != rank:
            raise ValueError(f"wkv: the decay's two matrices meet at {rank} and {tensors[n['w2']].shape[1]}")
        layout = {"rkvg": ((4 * HD, C), dtype)}             # the four projections one below the other
        layout.update({"w1": ((rank, C), dtype), "w2": ((HD, rank), dtype), "o": ((C, HD), dtype),
                       "mu": ((len(_MIXES), C), torch.float32), "w0": ((HD,), torch.float32),
                       "u": ((HD,), torch.float32), "norm": ((HD,), torch.float32)})
        self.buffers = buf = WeightBuffers(device, layout)
        for i, s in enumerate(("r", "k", "v", "g")):
            buf["rkvg"][i * HD:(i + 1) * HD].copy_(tensors[n[s]])
        for s in ("w1", "w2", "o"):
            buf[s].copy_(tensors[n[s]])
        for i, s in enumerate(_MIXES):
            buf["mu"][i].copy_(tensors[n["mu_" + s]])
        buf["w0"].copy_(tensors[n["w0"]])
        buf["u"].copy_(tensors[n["u"]].reshape(HD))
        buf["norm"].copy_(tensors[n["norm"]])
        self.w = {s: buf[s] for s in ("w1", "w2", "o")}
        self.w.update({s: buf["rkvg"][i * HD:(i + 1) * HD] for i, s in enumerate(("r", "k", "v", "g"))})
        self.w_rkvg = buf["rkvg"]
        self.mu, self.w0, self.u, self.norm_w = buf["mu"], buf["w0"], buf["u"], buf["norm"]
        self.rank = rank

    # --------------------------------------------------------------------- forward
    def forward(self, x, ctx, cache):
        """`x`: the float32 residual stream [T, hidden], read only."""
        k = ctx.kernels
        f32 = torch.float32
        matrices = self.heads * self.dim * self.dim
        mixes = k.token_shift_mix(x, self.mu, cache.state, matrices, ctx, ctx.dtype)          # [5, T, hidden]
        T, HD = x.shape[0], self.heads * self.dim
        if ctx.dtype == torch.bfloat16 and T <= self.STACK_MAX_TOKENS:
            # few tokens: a step reads every weight once whatever it computes, so the four mixes go through the four
            # stacked matrices in one product (of its sixteen blocks the four on the diagonal are used)
            both = k.materialize(k.linear(mixes[:4].view(4 * T, self.hidden), self.w_rkvg, out_dtype=f32, allow_partial=True))
            r, kk, v, g = (both[i * T:(i + 1) * T, i * HD:(i + 1) * HD] for i in range(4))
        else:
            r, kk, v, g = (k.linear(mixes[i], self.w[s], out_dtype=f32) for i, s in enumerate(("r", "k", "v", "g")))
        low = k.tanh(k.linear(mixes[4], self.w["w1"]))                                         # [T, rank]
        w_raw = k.linear(low, self.w["w2"], out_dtype=f32)
        y = k.wkv_scan(r, kk, v, w_raw, g, self.w0, self.u, self.norm_w, self.eps, self.heads, self.dim,
                       cache.state, matrices, x, ctx, ctx.dtype)                               # [T, heads * dim]
        return k.linear(y, self.w["o"], allow_partial=True)
