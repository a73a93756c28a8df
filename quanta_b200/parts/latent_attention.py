"""Softmax attention through low-rank latents, with one rotated key part for all heads and a sink.

Queries: c_q = RMSNorm(W_dq x), q = W_uq c_q, per head ``dim`` plain and ``rot_dim`` rotated dimensions.
Keys and values: W_dkv x has ``kv_rank + rot_dim`` rows; the first ``kv_rank``, RMS-normed, are the latent
c, the rest are one rotated key part that every head shares.  A head's plain key is W_uk c, its value
W_uv c, its score ``(q_plain . k_plain + q_rot . k_rot) * scale``; the softmax's denominator also holds
``exp(sink_h)``.  Only c and the rotated key part are cached (one stream of ``kv_rank + rot_dim``).

The up-projections never touch the cache: ``q_plain . (W_uk c) = (W_uk^T q_plain) . c`` and
``sum_j p_j W_uv c_j = W_uv sum_j p_j c_j``, so the attention kernel works on the cached rows as they
are, with every head reading the same row, and W_uk / W_uv are two batched library products on the
step's own tokens.  Portions of prompts and single tokens are the same kernels, a token's keys cut into
ranges (more of them when the step has few tokens).  The float32 path (and shapes the tensor-core kernel
does not take) computes scores, softmax and the weighted sum in float32 on the CUDA cores; a bfloat16 cache
with a latent of 64, 128, 256 or 512 and a rotated part that is a multiple of 16 runs on the tensor cores
(bfloat16 operands, float32 sums and softmax), the rows of an MMA tile being the heads of a token.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import CacheSpec, CacheStream, KeepAll, Mixer, TensorSpec, make, register

STREAM = "latent"


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_heads: int, dim: int, rot_dim: int, value_dim: int, q_rank: int,
                 kv_rank: int, scale: float, norm_eps: float, position, names: dict, sink: bool = True):
        if kv_rank > kernels.LATENT_MAX_RANK:
            raise ValueError(f"latent_attention: latent of {kv_rank} above the kernel's {kernels.LATENT_MAX_RANK}")
        self.hidden, self.H, self.D, self.R, self.V = int(hidden_size), int(n_heads), int(dim), int(rot_dim), int(value_dim)
        self.q_rank, self.C = int(q_rank), int(kv_rank)
        self.scale, self.eps, self.has_sink = float(scale), float(norm_eps), bool(sink)
        self.position = make("position", position) if isinstance(position, tuple) else position
        self.names = dict(names)     # dq, dq_norm, uq, dkv, dkv_norm, uk, uv, o, sink
        self.w_dq = self.w_uq = self.w_dkv = self.w_uk = self.w_uv_t = self.w_o = None
        self.dq_gain = self.dkv_gain = self.sink = None

    def children(self):
        return [self.position]

    def tensor_specs(self):
        n, W = self.names, self.hidden
        specs = [TensorSpec(n["dq"], (self.q_rank, W)), TensorSpec(n["dq_norm"], (self.q_rank,), "f32", "gain"),
                 TensorSpec(n["uq"], (self.H * (self.D + self.R), self.q_rank)),
                 TensorSpec(n["dkv"], (self.C + self.R, W)), TensorSpec(n["dkv_norm"], (self.C,), "f32", "gain"),
                 TensorSpec(n["uk"], (self.H * self.D, self.C)), TensorSpec(n["uv"], (self.H * self.V, self.C)),
                 TensorSpec(n["o"], (W, self.H * self.V))]
        if self.has_sink:
            specs.append(TensorSpec(n["sink"], (self.H,), "f32", "bias"))
        return specs

    def load(self, fetch):
        n = self.names
        self.w_dq, self.w_uq, self.w_dkv, self.w_o = fetch(n["dq"]), fetch(n["uq"]), fetch(n["dkv"]), fetch(n["o"])
        self.w_uk = fetch(n["uk"]).view(self.H, self.D, self.C)                       # [h]: plain dims x latent
        self.w_uv_t = fetch(n["uv"]).view(self.H, self.V, self.C).transpose(1, 2)     # [h]: latent x value dims
        self.dq_gain, self.dkv_gain = fetch(n["dq_norm"]), fetch(n["dkv_norm"])
        self.sink = fetch(n["sink"]) if self.has_sink else None

    def cache_spec(self):
        return CacheSpec((CacheStream(STREAM, 1, self.C + self.R),), KeepAll())

    def _ranges(self, ctx, tensor_cores: bool) -> int:
        """Ranges a token's keys are cut into: one when the step has blocks enough to fill the GPU, else as
        many as give every SM two blocks, each at least 128 keys long."""
        if tensor_cores:
            blocks = -(-ctx.n_tokens * self.H // kernels.LATENT_MMA_ROWS)
        else:
            blocks = ctx.n_tokens * -(-self.H // 8)
        by_work = -(-296 // max(1, blocks))
        by_keys = -(-max(1, ctx.max_len_after) // 128)
        return max(1, min(64, by_work, by_keys))

    def forward(self, x, ctx, cache, state):
        T, H, dev = x.shape[0], self.H, x.device
        f32 = torch.float32
        tables = self.position.rotary_tables(dev)
        if tables is None:
            inv_freq, rd = torch.empty(0, dtype=f32, device=dev), 0
        else:
            inv_freq, pair_axis, rd, _ = tables
            if pair_axis is not None:
                raise ValueError("latent_attention: position encodings with several axes are not built")
        # queries through their latent
        cq_raw = linear(x, self.w_dq, out_dtype=f32)
        cq = empty_rows(T, self.q_rank, dtype=x.dtype, device=dev)
        kernels.add_rmsnorm(cq_raw, None, self.dq_gain, self.eps, cq)
        q = linear(cq, self.w_uq, out_dtype=f32)
        # this step's latent rows and rotated key parts go into the pages
        dkv = linear(x, self.w_dkv, out_dtype=f32)
        pages = cache.streams[STREAM]
        if cache.write:
            kernels.latent_write(dkv, self.dkv_gain, inv_freq, pages, ctx.tok_pos, ctx.tok_req, cache.block_table,
                                 self.C, self.R, rd, cache.page_size, self.eps, ctx.status)
        q_plain = torch.empty((H, T, self.D), dtype=x.dtype, device=dev)
        q_rot = torch.empty((T, H, self.R), dtype=f32, device=dev)
        kernels.latent_query(q, inv_freq, q_plain, q_rot, ctx.tok_pos, H, self.D, self.R, rd)
        q_lat = torch.bmm(q_plain, self.w_uk, out_dtype=f32) if x.dtype != f32 else torch.bmm(q_plain, self.w_uk)
        o_lat = torch.empty((H, T, self.C), dtype=x.dtype, device=dev)
        tc = kernels.latent_attend_uses_tensor_cores(pages.dtype, self.C, self.R)
        kernels.latent_attend(q_lat, q_rot, pages, self.sink, o_lat, ctx.tok_pos, ctx.tok_req, cache.block_table,
                              self.scale, self._ranges(ctx, tc), ctx.status, req_start=ctx.req_start)
        o = empty_rows(T, H * self.V, dtype=x.dtype, device=dev)
        torch.bmm(o_lat, self.w_uv_t, out=o.view(T, H, self.V).transpose(0, 1))
        return linear(o, self.w_o, out_dtype=f32)
