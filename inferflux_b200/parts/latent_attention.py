"""Attention whose keys and values are made, for all heads, from one low-rank latent per token.

    q_h = Wq_h x                      c = rmsnorm(Wdkv x) * g          (the latent, `kv_rank` numbers)
    k_h = Wuk_h c,  v_h = Wuv_h c     score = scale * q_h . k_h        no position encoding
    weights = softmax over the window, with exp(sink_h) added to the denominator (optional)
    y = Wo [o_1; ...; o_H]

Only c is cached: one plane of one head of size kv_rank per token, in pages through the same
block tables as every other cache.  The kernels never make k or v: the query head is carried
into latent space (Wuk_h^T q_h), the weighted sum runs over cached latents, and Wuv_h is applied
to that sum.  Query and latent projections are stacked at load so that one product makes both.
"""
from __future__ import annotations

import math

import torch

from ..weights.loader import TensorSpec
from .base import KVCacheSpec, Mixer, WeightBuffers, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """params: hidden_size, num_heads, qk_dim, v_dim, kv_rank, window (None or int), scale (None for
    1/sqrt(qk_dim)), latent_norm_eps, sink (whether heads have a learned sink), names (tensor names of
    q, dkv, dkv_norm, uk, uv, sink, o; default: those words with `_` as `.`)."""

    _NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "sink": "sink", "o": "o"}

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dk = int(p["qk_dim"])
        self.dv = int(p["v_dim"])
        self.rank = int(p["kv_rank"])
        for name in ("hidden", "heads", "dk", "dv", "rank"):
            if getattr(self, name) <= 0:
                raise ValueError(f"latent_attention: {name} must be positive, got {getattr(self, name)}")
        if self.rank > 1024:
            raise ValueError(f"latent_attention: a latent of {self.rank} is beyond the kernels' 1024")
        self.window = None if p.get("window") is None else int(p["window"])
        if self.window is not None and self.window <= 0:
            raise ValueError(f"latent_attention: window must be positive, got {self.window}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dk)
        self.eps = float(p.get("latent_norm_eps", 1e-6))
        self.has_sink = bool(p.get("sink", False))
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})
        self.w_q_dkv = self.w_uk = self.w_uv = self.w_o = self.latent_norm = self.sinks = None

    # ---------------------------------------------------------------- declarations
    def cache_spec(self):
        return KVCacheSpec(1, self.rank, self.window, planes=1)

    def param_specs(self):
        n, H = self.names, self.heads
        specs = {
            n["q"]: TensorSpec((H * self.dk, self.hidden)),
            n["dkv"]: TensorSpec((self.rank, self.hidden)),
            n["dkv_norm"]: TensorSpec((self.rank,), init="ones"),
            n["uk"]: TensorSpec((H * self.dk, self.rank)),
            n["uv"]: TensorSpec((H * self.dv, self.rank)),
            n["o"]: TensorSpec((self.hidden, H * self.dv)),
        }
        if self.has_sink:
            specs[n["sink"]] = TensorSpec((H,), init="zeros")
        return specs

    def load(self, tensors, dtype, device):
        n, H = self.names, self.heads
        q = H * self.dk
        self.buffers = buf = WeightBuffers(device, {
            "w_q_dkv": ((q + self.rank, self.hidden), dtype), "w_uk": ((q, self.rank), dtype),
            "w_uv": ((H * self.dv, self.rank), dtype), "w_o": ((self.hidden, H * self.dv), dtype),
            "latent_norm": ((self.rank,), torch.float32), "sinks": ((H,), torch.float32)})
        buf["w_q_dkv"][:q].copy_(tensors[n["q"]])
        buf["w_q_dkv"][q:].copy_(tensors[n["dkv"]])
        buf["w_uk"].copy_(tensors[n["uk"]])
        buf["w_uv"].copy_(tensors[n["uv"]])
        buf["w_o"].copy_(tensors[n["o"]])
        buf["latent_norm"].copy_(tensors[n["dkv_norm"]])
        if self.has_sink:
            buf["sinks"].copy_(tensors[n["sink"]])
        self.w_q_dkv, self.w_uk, self.w_uv, self.w_o = buf["w_q_dkv"], buf["w_uk"], buf["w_uv"], buf["w_o"]
        self.latent_norm = buf["latent_norm"]
        self.sinks = buf["sinks"] if self.has_sink else None

    def step_sections(self, ctx):
        """The work lists of the kernel table's latent attention kernels, if it has any."""
        make = getattr(ctx.kernels, "latent_attention_sections", None)
        return make(ctx) if make is not None else {}

    # --------------------------------------------------------------------- forward
    def forward(self, h, ctx, cache):
        k = ctx.kernels
        q_dkv = k.materialize(k.linear(h, self.w_q_dkv, allow_partial=True))   # [T, H dk + rank]
        k.latent_norm_append(q_dkv, self.heads * self.dk, self.rank, self.latent_norm, self.eps, ctx, cache)
        a = k.latent_attention(q_dkv, self.w_uk, self.w_uv, self.sinks, self.heads, self.dk, self.dv, self.rank,
                               self.window, self.scale, ctx, cache)         # [T, H dv]
        return k.linear(a, self.w_o, allow_partial=True)
