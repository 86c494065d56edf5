"""Pre-norm residual block: x += mixer(norm(x)); x += ffn(norm(x))
(runtime/backends/cuda/native/llama_forward.h:88-90).  The block hands its last
delta on unadded, so that whatever normalises next adds it in the same kernel
(runtime/backends/cuda/native/transformer_forward.cu:2203-2211, 2564-2586)."""
from __future__ import annotations

from typing import Optional

import torch

from ..weights.loader import TensorSpec
from .base import Block, NormedDelta, StateSpec, StreamMerge, register_part, settle_pending
from .norm import RMSNorm


@register_part("block", "prenorm")
class PreNormBlock(Block):
    sub_parts = {"norm_mixer": "norm", "mixer": "mixer", "norm_ffn": "norm", "ffn": "ffn"}

    def forward(self, x, pending, ctx, cache):
        if isinstance(pending, NormedDelta):                         # the layer before norms its output itself
            pending.add_to(x, ctx)
            pending = None
        fused = getattr(ctx.kernels, "fused_prenorm_layer", None)    # a kernel table may run the whole layer itself
        if fused is not None:
            done = fused(self, x, pending, ctx, cache)
            if done is not None:
                return done
        h = self.norm_mixer.forward(x, pending, ctx, lazy=self.mixer.takes_scaled_rows)   # x += pending; h = norm(x)
        a = self.mixer.forward(h, ctx, cache)
        h = self.norm_ffn.forward(x, a, ctx, lazy=self.ffn.takes_scaled_rows)             # x += a; h = norm(x)
        f = self.ffn.forward(h, ctx)
        return x, f


class _StoresForBlock:
    """What a layer stores when its block keeps state of its own beside the mixer's cache."""

    def __init__(self, mixer, state: Optional[StateSpec]):
        self.mixer, self.state = mixer, state

    def cache_spec(self):
        return self.mixer.cache_spec()

    def state_spec(self):
        return self.state


@register_part("block", "sandwich")
class SandwichBlock(Block):
    """Norms on both sides of every sublayer, and optionally a short convolution over time in front of it:

        x += norm_b(mixer(conv(norm_a(x))));   x += norm_d(ffn(conv(norm_c(x))))

    params: ffn (False: the layer ends after the mixer), conv (False: no convolutions).  Parts, as far as
    present: norm_mixer, conv_mixer, mixer, postnorm_mixer, norm_ffn, conv_ffn, ffn, postnorm_ffn.  The
    convolutions' inputs of the last few tokens are the layer's state, [convolutions, rows, width] per request.
    A sublayer's output is handed on unadded with its norm (`NormedDelta`), so that sum, that norm and the
    next one run as one kernel."""

    def __init__(self, spec, parts):
        self.has_ffn = bool(spec.params.get("ffn", True))
        self.has_conv = bool(spec.params.get("conv", True))
        names = {"norm_mixer": "norm", "mixer": "mixer", "postnorm_mixer": "norm"}
        if self.has_ffn:
            names.update({"norm_ffn": "norm", "ffn": "ffn", "postnorm_ffn": "norm"})
        if self.has_conv:
            names["conv_mixer"] = "conv"
            if self.has_ffn:
                names["conv_ffn"] = "conv"
        self.sub_parts = names
        super().__init__(spec, parts)
        for name, role in names.items():
            if role == "norm" and not isinstance(parts[name], RMSNorm):
                raise ValueError(f"sandwich block: {name} must be an RMS norm (its weight and eps go into fused kernels)")
        self.convs = [parts[n] for n in ("conv_mixer", "conv_ffn") if n in parts]
        rows = {c.state_rows for c in self.convs}
        if len(rows) > 1:
            raise ValueError("sandwich block: the layer's convolutions must keep the same number of inputs")
        self.state_rows = rows.pop() if rows else None

    def cache_part(self):
        if self.mixer.state_spec() is not None and self.state_rows:
            raise ValueError("sandwich block: a mixer with state of its own beside convolutions is not built")
        if not self.state_rows:
            return self.mixer
        width = self.convs[0].channels
        return _StoresForBlock(self.mixer, StateSpec((len(self.convs), self.state_rows, width), torch.float32))

    def _sublayer_input(self, x, pending, norm, conv, index, ctx, cache):
        k = ctx.kernels
        if isinstance(pending, NormedDelta):
            if conv is not None and ctx.max_span == 1 and getattr(k, "fuses_single_token_conv", False):
                # decoded tokens only: sum, both norms and the convolution (its history is all state) in one kernel
                return k.postnorm_add(x, pending.y, pending.weight, pending.eps, norm.weight, norm.eps, ctx.dtype,
                                      conv=(conv.weight, conv.taps, cache.state, index, ctx))
            h = k.postnorm_add(x, pending.y, pending.weight, pending.eps, norm.weight, norm.eps, ctx.dtype)
        else:
            h = norm.forward(x, pending, ctx)
        return conv.forward(h, ctx, cache.state, index) if conv is not None else h

    def forward(self, x, pending, ctx, cache):
        conv = self.parts.get("conv_mixer")
        h = self._sublayer_input(x, pending, self.norm_mixer, conv, 0, ctx, cache)
        y = self.mixer.forward(h, ctx, cache)
        pending = NormedDelta(y, self.postnorm_mixer.weight, self.postnorm_mixer.eps)
        if not self.has_ffn:
            return x, pending
        h = self._sublayer_input(x, pending, self.norm_ffn, self.parts.get("conv_ffn"), 1, ctx, cache)
        y = self.ffn.forward(h, ctx)
        return x, NormedDelta(y, self.postnorm_ffn.weight, self.postnorm_ffn.eps)


@register_part("block", "postnorm")
class PostNormBlock(Block):
    """A norm on each sublayer's output only; the sublayers read the residual stream itself:

        x += norm_a(mixer(x));   x += norm_b(ffn(x))

    params: ffn (False: the layer ends after the mixer).  Parts: mixer, postnorm_mixer and, with a feed-forward,
    ffn, postnorm_ffn.  A sublayer's output travels unadded with its norm (`NormedDelta`); the sum, that norm
    and the rounding of x to the run's dtype for the next sublayer are one kernel.  A sublayer that sets
    `takes_stream` gets the float32 rows themselves."""

    def __init__(self, spec, parts):
        self.has_ffn = bool(spec.params.get("ffn", True))
        names = {"mixer": "mixer", "postnorm_mixer": "norm"}
        if self.has_ffn:
            names.update({"ffn": "ffn", "postnorm_ffn": "norm"})
        self.sub_parts = names
        super().__init__(spec, parts)
        for name, role in names.items():
            if role == "norm" and not isinstance(parts[name], RMSNorm):
                raise ValueError(f"postnorm block: {name} must be an RMS norm (its weight and eps go into a fused kernel)")

    @staticmethod
    def _sublayer_input(x, pending, reader, ctx):
        """Settle what is pending and give the reader its rows."""
        k = ctx.kernels
        as_stream = reader.takes_stream or ctx.dtype == torch.float32
        if isinstance(pending, NormedDelta):
            if as_stream:
                pending.add_to(x, ctx)
                return x
            return k.postnorm_add(x, pending.y, pending.weight, pending.eps, out_dtype=ctx.dtype, cast_out=True)
        settle_pending(x, pending, ctx)
        return x if as_stream else k.cast_rows(x, ctx.dtype)

    def forward(self, x, pending, ctx, cache):
        h = self._sublayer_input(x, pending, self.mixer, ctx)
        y = self.mixer.forward(h, ctx, cache)
        pending = NormedDelta(y, self.postnorm_mixer.weight, self.postnorm_mixer.eps)
        if not self.has_ffn:
            return x, pending
        h = self._sublayer_input(x, pending, self.ffn, ctx)
        y = self.ffn.forward(h, ctx)
        return x, NormedDelta(y, self.postnorm_ffn.weight, self.postnorm_ffn.eps)


@register_part("merge", "linear_reinject")
class LinearReinject(StreamMerge):
    """x' = W [x; x0] + step[repeat]: the stream and the embedding output side by side through one matrix
    [width, 2 width] (x first), plus a learned vector per run.  The product takes its inputs in the run's
    dtype; its result and the sum stay float32, as the residual stream is.
    params: width, times, names (tensor names of `in`, `step`)."""

    _NAMES = {"in": "in", "step": "step"}

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["width"])
        self.times = int(spec.params["times"])
        self.names = dict(self._NAMES)
        self.names.update(spec.params.get("names") or {})
        self.w_in = self.steps = None

    def param_specs(self):
        return {self.names["in"]: TensorSpec((self.width, 2 * self.width)),
                self.names["step"]: TensorSpec((self.times, self.width))}

    def load(self, tensors, dtype, device):
        self.w_in = tensors[self.names["in"]].to(device=device, dtype=dtype).contiguous()
        self.steps = tensors[self.names["step"]].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, x0, repeat, ctx):
        if not 0 <= repeat < self.times:
            raise ValueError(f"linear_reinject: run {repeat} of {self.times}")
        k = ctx.kernels
        both = k.concat_cast(x, x0, ctx.dtype)                                  # [T, 2 width]
        return k.linear(both, self.w_in, bias=self.steps[repeat], out_dtype=torch.float32)


@register_part("block", "reinject")
class ReinjectBlock(Block):
    """Not a layer of sublayers: replaces the residual stream by a merge of it with the embedding output
    (`ctx.embedding_output`); which run of a looped stretch this is comes from the schedule entry
    (`ctx.entry.repeat`).  Stores nothing."""

    sub_parts = {"merge": "merge"}

    def cache_part(self):
        return None

    def forward(self, x, pending, ctx, cache):
        settle_pending(x, pending, ctx)
        return self.merge.forward(x, ctx.embedding_output, ctx.entry.repeat, ctx), None
