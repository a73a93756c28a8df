"""Generalized delta rule: a linear recurrence per head whose state is a matrix S [key channel, value channel].

With r, k, v = W_r x, W_k x, W_v x (heads x dim each), the unit key u = k / sqrt(|k|^2 + unit_eps), the
decay per key channel w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 x) + w0)) and the removal rate
a = sigmoid(W_a x + a_b):

    S_t = diag(w) S_(t-1) - (a * u)(u^T S_(t-1)) + k v^T          o_t = S_t^T r

Each head's o is divided by its root mean square, multiplied by a gain over all heads and by
sigmoid(W_g x), and projected by W_o.  S is float32, zero at admission, one matrix per (request, head)
in the request's state slot; everything from the projections' outputs to the gated result is float32.
All projections that read x are one library product (r, k, v, g, a and the inner part of the decay).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import Mixer, TensorSpec, register


@register("mixer", "delta_rule")
class DeltaRule(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_heads: int, dim: int, decay_rank: int, decay_scale: float,
                 unit_eps: float, norm_eps: float, names: dict, state_name: str = "delta_state"):
        if dim > kernels.DELTA_RULE_MAX_DIM:
            raise ValueError(f"delta_rule: head size {dim} above the kernel's {kernels.DELTA_RULE_MAX_DIM}")
        self.hidden, self.H, self.D, self.L = int(hidden_size), int(n_heads), int(dim), int(decay_rank)
        self.decay_scale, self.unit_eps, self.norm_eps = float(decay_scale), float(unit_eps), float(norm_eps)
        self.names, self.state_name = dict(names), state_name
        self.w_in = self.w_decay = self.w_o = self.a_bias = self.w_bias = self.gain = None

    # r, k, v, g, a are heads*dim rows each of the fused input matrix, then the decay's inner rows
    _FUSED = ("r", "k", "v", "g", "a")

    def tensor_specs(self):
        n, HD, W = self.names, self.H * self.D, self.hidden
        specs = [TensorSpec(n[k], (HD, W)) for k in self._FUSED]
        specs += [TensorSpec(n["w1"], (self.L, W)), TensorSpec(n["w2"], (HD, self.L)),
                  TensorSpec(n["o"], (W, HD)),
                  TensorSpec(n["a_bias"], (HD,), "f32", "bias"), TensorSpec(n["w_bias"], (HD,), "f32", "bias"),
                  TensorSpec(n["gain"], (HD,), "f32", "gain")]
        return specs

    def load(self, fetch):
        n, HD = self.names, self.H * self.D
        first = fetch(n["r"])
        self.w_in = torch.empty((5 * HD + self.L, self.hidden), dtype=first.dtype, device=first.device)
        self.w_in[:HD].copy_(first)
        del first
        for i, key in enumerate(self._FUSED[1:], start=1):
            self.w_in[i * HD:(i + 1) * HD].copy_(fetch(n[key]))
        self.w_in[5 * HD:].copy_(fetch(n["w1"]))
        self.w_decay, self.w_o = fetch(n["w2"]), fetch(n["o"])
        self.a_bias, self.w_bias, self.gain = fetch(n["a_bias"]), fetch(n["w_bias"]), fetch(n["gain"])

    def state_spec(self):
        return {self.state_name: ((self.H, self.D, self.D), torch.float32)}

    def forward(self, x, ctx, cache, state):
        T, HD = x.shape[0], self.H * self.D
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        inner = empty_rows(T, self.L, dtype=x.dtype, device=x.device)
        kernels.tanh_cols(proj, 5 * HD, self.L, inner)
        wpre = linear(inner, self.w_decay, out_dtype=torch.float32)
        o = torch.empty((T, self.H, self.D), dtype=torch.float32, device=x.device)
        kernels.delta_rule(proj, (0, HD, 2 * HD, 4 * HD), wpre, self.a_bias, self.w_bias, state[self.state_name], o,
                           ctx.req_start, ctx.req_slot, self.H, self.D, self.decay_scale, self.unit_eps)
        y = empty_rows(T, HD, dtype=x.dtype, device=x.device)
        kernels.head_norm_gate(o, proj, 3 * HD, self.gain, y, self.H, self.D, self.norm_eps)
        return linear(y, self.w_o, out_dtype=torch.float32)
