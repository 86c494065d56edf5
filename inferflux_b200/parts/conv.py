"""A short causal convolution over time on each channel, added to its input:
out_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j), zeros before a request's first
token.  The taps - 1 inputs before a step's first token are the request's state."""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import TimeConv, register_part


@register_part("conv", "causal_depthwise")
class CausalDepthwiseConv(TimeConv):
    """params: channels, taps, tensor_name (the weight [channels, taps]; default `weight`)."""

    def __init__(self, spec):
        super().__init__(spec)
        self.channels = int(spec.params["channels"])
        self.taps = int(spec.params["taps"])
        if self.taps < 1:
            raise ValueError(f"causal_depthwise: taps must be at least 1, got {self.taps}")
        self.tensor_name = str(spec.params.get("tensor_name", "weight"))
        self.state_rows = self.taps - 1 if self.taps > 1 else None
        self.weight = None

    def param_specs(self):
        return {self.tensor_name: TensorSpec((self.channels, self.taps))}

    def load(self, tensors, dtype, device):
        self.weight = tensors[self.tensor_name].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, h, ctx, state, index):
        return ctx.kernels.short_conv(h, self.weight, self.taps, state, index, ctx)
