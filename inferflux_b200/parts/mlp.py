"""SwiGLU feed-forward: (silu(h Wg^T) * (h Wu^T)) Wd^T, no biases
(runtime/backends/cuda/native/transformer_forward.cu:2384-2535).  Gate and up
weights are stacked at load so that one product makes both."""
from __future__ import annotations

import math

import torch

from ..weights.loader import TensorSpec
from .base import FeedForward, WeightBuffers, register_part


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size, names (tensor names of gate, up, down)."""

    takes_scaled_rows = True          # h goes only into the stacked projection

    _NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.names = dict(self._NAMES)
        self.names.update(spec.params.get("names") or {})
        self.w_gate_up = None
        self.w_down = None

    def param_specs(self):
        n = self.names
        return {
            n["gate"]: TensorSpec((self.inter, self.hidden)),
            n["up"]: TensorSpec((self.inter, self.hidden)),
            n["down"]: TensorSpec((self.hidden, self.inter)),
        }

    def load(self, tensors, dtype, device):
        self.buffers = buf = WeightBuffers(device, {"w_gate_up": ((2 * self.inter, self.hidden), dtype),
                                                    "w_down": ((self.hidden, self.inter), dtype)})
        buf["w_gate_up"][:self.inter].copy_(tensors[self.names["gate"]])
        buf["w_gate_up"][self.inter:].copy_(tensors[self.names["up"]])
        buf["w_down"].copy_(tensors[self.names["down"]])
        self.w_gate_up, self.w_down = buf["w_gate_up"], buf["w_down"]

    def forward(self, h, ctx):
        k = ctx.kernels
        act = k.linear_swiglu(h, self.w_gate_up)         # [T, I] = silu(h Wg^T) * (h Wu^T)
        return k.linear(act, self.w_down, allow_partial=True)


def _softplus(v: float) -> float:
    return max(v, 0.0) + math.log1p(math.exp(-abs(v)))


@register_part("ffn", "up_act_down")
class ActivationMLP(FeedForward):
    """W_down act(W_up h), no gate and no biases.
    params: hidden_size, intermediate_size, activation, names (tensor names of up, down, act).

    activation `xielu`: two learned numbers (p, q) in the tensor `act`;
    act(z) = softplus(p) z^2 + z/2 for z > 0, (1/2 + softplus(q)) (e^z - 1 - z) + z/2 for z <= 0."""

    _NAMES = {"up": "up", "down": "down", "act": "act"}

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = str(spec.params.get("activation", "xielu"))
        if self.activation != "xielu":
            raise ValueError(f"up_act_down: unknown activation {self.activation!r} (known: xielu)")
        self.names = dict(self._NAMES)
        self.names.update(spec.params.get("names") or {})
        self.w_up = self.w_down = None
        self.a_pos = self.a_neg = 0.0

    def param_specs(self):
        n = self.names
        return {n["up"]: TensorSpec((self.inter, self.hidden)), n["down"]: TensorSpec((self.hidden, self.inter)),
                n["act"]: TensorSpec((2,), init="zeros")}

    def load(self, tensors, dtype, device):
        n = self.names
        self.buffers = buf = WeightBuffers(device, {"w_up": ((self.inter, self.hidden), dtype),
                                                    "w_down": ((self.hidden, self.inter), dtype)})
        buf["w_up"].copy_(tensors[n["up"]])
        buf["w_down"].copy_(tensors[n["down"]])
        self.w_up, self.w_down = buf["w_up"], buf["w_down"]
        p, q = (float(v) for v in tensors[n["act"]].to(torch.float32).cpu().tolist())
        self.a_pos, self.a_neg = _softplus(p), 0.5 + _softplus(q)

    def forward(self, h, ctx):
        k = ctx.kernels
        act = k.linear_xielu(h, self.w_up, self.a_pos, self.a_neg)     # the activation in the product's epilogue where it can be
        return k.linear(act, self.w_down, allow_partial=True)
