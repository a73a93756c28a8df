"""Gated linear attention: a linear recurrence per head whose state is a matrix S [key channel, value channel].

With q, k = W_q x * q_scale, W_k x (heads x dim each), v = W_v x (heads x value_dim) and a decay per key
channel alpha = sigmoid(W_a2 (W_a1 x) + b)^(1 / tau) (a low-rank pair of projections):

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          o_t = S_t^T q_t

Each head's o is divided by its root mean square over value_dim and multiplied by a gain of value_dim
elements that all heads share, the heads side by side are multiplied by silu(W_g x) and projected by W_o.
S is float32, zero at admission, one matrix per (request, head) in the request's state slot; the decay (its
second product, logarithm, root and exponential), the state, the per-head norm and the gate are float32.
All projections that read x are one library product (q, k, v, g and the inner part of the decay), whose
float32 accumulators feed the recurrence.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import Mixer, TensorSpec, register


@register("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_heads: int, dim: int, value_dim: int, decay_rank: int, tau: float,
                 q_scale: float, norm_eps: float, names: dict, state_name: str = "gla_state"):
        if not 0 < dim <= kernels.GLA_MAX_DIM or not 0 < value_dim <= kernels.GLA_MAX_DIM:
            raise ValueError(f"gated_linear_attention: head sizes {dim} / {value_dim} outside the kernel's 1 to "
                             f"{kernels.GLA_MAX_DIM}")
        if tau <= 0:
            raise ValueError(f"gated_linear_attention: tau {tau} must be positive")
        self.hidden, self.H, self.D, self.E, self.L = int(hidden_size), int(n_heads), int(dim), int(value_dim), int(decay_rank)
        self.tau, self.q_scale, self.norm_eps = float(tau), float(q_scale), float(norm_eps)
        self.names, self.state_name = dict(names), state_name
        self.w_in = self.w_decay = self.decay_bias = self.gain = self.w_o = None

    def tensor_specs(self):
        n, HD, HE, W = self.names, self.H * self.D, self.H * self.E, self.hidden
        return [TensorSpec(n["q"], (HD, W)), TensorSpec(n["k"], (HD, W)), TensorSpec(n["v"], (HE, W)),
                TensorSpec(n["g"], (HE, W)), TensorSpec(n["a1"], (self.L, W)), TensorSpec(n["a2"], (HD, self.L)),
                TensorSpec(n["a2_bias"], (HD,), "f32", "bias"), TensorSpec(n["gain"], (self.E,), "f32", "gain"),
                TensorSpec(n["o"], (W, HE))]

    def load(self, fetch):
        n, HD, HE = self.names, self.H * self.D, self.H * self.E
        first = fetch(n["q"])
        rows = 2 * HD + 2 * HE + self.L
        self.w_in = torch.empty((rows, self.hidden), dtype=first.dtype, device=first.device)
        self.w_in[:HD].copy_(first)
        del first
        self.w_in[HD: 2 * HD].copy_(fetch(n["k"]))
        self.w_in[2 * HD: 2 * HD + HE].copy_(fetch(n["v"]))
        self.w_in[2 * HD + HE: 2 * HD + 2 * HE].copy_(fetch(n["g"]))
        self.w_in[2 * HD + 2 * HE:].copy_(fetch(n["a1"]))
        self.w_decay = fetch(n["a2"]).contiguous()
        self.decay_bias, self.gain, self.w_o = fetch(n["a2_bias"]), fetch(n["gain"]), fetch(n["o"])

    def state_spec(self):
        return {self.state_name: ((self.H, self.D, self.E), torch.float32)}

    def forward(self, x, ctx, cache, state):
        T, HD, HE = x.shape[0], self.H * self.D, self.H * self.E
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        o = torch.empty((T, self.H, self.E), dtype=torch.float32, device=x.device)
        kernels.gla(proj, (0, HD, 2 * HD), 2 * HD + 2 * HE, self.L, self.w_decay, self.decay_bias,
                    state[self.state_name], o, ctx.req_start, ctx.req_slot, self.H, self.D, self.E, self.tau, self.q_scale)
        y = empty_rows(T, HE, dtype=x.dtype, device=x.device)
        kernels.head_norm_gate(o, proj, 2 * HD + HE, self.gain, y, self.H, self.E, self.norm_eps, gate="silu")
        return linear(y, self.w_o, out_dtype=torch.float32)
