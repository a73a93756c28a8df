"""Dense feed-forwards: gated, ``down(act(gate x) * (up x))`` with ``act = silu``, and ungated,
``down(act(up x))`` with ``act`` the square of relu.

The gate and up matrices are held as one, so a step is two library products and one activation kernel.
The result is float32 (the accumulator of the down product), for blocks that norm it before the sum.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import FeedForward, TensorSpec, register


@register("feed_forward", "gated_dense")
class GatedDense(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, inner_size: int, names: dict, activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"gated_dense: activation {activation!r} is not built (silu is)")
        self.hidden, self.inner, self.names = int(hidden_size), int(inner_size), dict(names)   # gate, up, down
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        n = self.names
        return [TensorSpec(n["gate"], (self.inner, self.hidden)), TensorSpec(n["up"], (self.inner, self.hidden)),
                TensorSpec(n["down"], (self.hidden, self.inner))]

    def load(self, fetch):
        gate = fetch(self.names["gate"])
        self.w_gate_up = torch.empty((2 * self.inner, self.hidden), dtype=gate.dtype, device=gate.device)
        self.w_gate_up[: self.inner].copy_(gate)
        del gate
        self.w_gate_up[self.inner:].copy_(fetch(self.names["up"]))
        self.w_down = fetch(self.names["down"])

    def forward(self, x, ctx):
        T = x.shape[0]
        gate_up = linear(x, self.w_gate_up)
        act = empty_rows(T, self.inner, dtype=x.dtype, device=x.device)
        kernels.silu_mul(gate_up, act)
        return linear(act, self.w_down, out_dtype=torch.float32)


@register("feed_forward", "ungated_dense")
class UngatedDense(FeedForward):
    """``down(act(up x))``; ``activation``: ``"relu_squared"`` (``relu(z)^2``)."""

    graph_safe = True

    def __init__(self, hidden_size: int, inner_size: int, names: dict, activation: str = "relu_squared"):
        if activation != "relu_squared":
            raise ValueError(f"ungated_dense: activation {activation!r} is not built (relu_squared is)")
        self.hidden, self.inner, self.names = int(hidden_size), int(inner_size), dict(names)   # up, down
        self.w_up = self.w_down = None

    def tensor_specs(self):
        n = self.names
        return [TensorSpec(n["up"], (self.inner, self.hidden)), TensorSpec(n["down"], (self.hidden, self.inner))]

    def load(self, fetch):
        self.w_up, self.w_down = fetch(self.names["up"]), fetch(self.names["down"])

    def forward(self, x, ctx):
        T = x.shape[0]
        up = linear(x, self.w_up)
        act = empty_rows(T, self.inner, dtype=x.dtype, device=x.device)
        kernels.relu_squared(up, act)
        return linear(act, self.w_down, out_dtype=torch.float32)
