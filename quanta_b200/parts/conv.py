"""Short causal convolution over time with the input added back: ``y_t = x_t + sum_j w[:, j] x_(t-taps+1+j)``.

One weight row per channel (``[channels, taps]``, no bias); positions before a sequence's start count as
zeros.  The last ``taps - 1`` inputs of every request live in its state slot (float32, zero at admission),
so a portion that starts anywhere sees the same numbers as the whole prompt.
"""

from __future__ import annotations

import torch

from .. import kernels
from .base import TensorSpec, TimeConv, register


@register("time_conv", "residual_short_conv")
class ResidualShortConv(TimeConv):
    graph_safe = True

    def __init__(self, channels: int, taps: int, weight_name: str, state_name: str = "conv_inputs"):
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        self.C, self.taps, self.weight_name, self.state_name = int(channels), int(taps), weight_name, state_name
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.C, self.taps), kind="f32", init="normal")]

    def load(self, fetch):
        self.weight = fetch(self.weight_name).contiguous()

    def state_spec(self):
        return {self.state_name: ((self.taps - 1, self.C), torch.float32)}

    def forward(self, x, ctx, state, out):
        kernels.short_conv(x, self.weight, state[self.state_name], out, ctx.tok_req, ctx.req_start, ctx.req_slot)
