"""RMSNorm with the residual sum folded in (src/quanta/minimax/model_m3.py:60-65)."""

from __future__ import annotations

import torch

from .. import kernels
from .base import Norm, NormedPending, StreamsPending, TensorSpec, register


@register("norm", "rms_norm")
class RMSNorm(Norm):
    graph_safe = True

    """``weight * x * rsqrt(mean(x^2) + eps)`` with float32 statistics; plain weight (no ``1 + w``)."""

    def __init__(self, width: int, eps: float, weight_name: str):
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.width,), kind="f32", init="gain")]

    def load(self, fetch):
        self.weight = fetch(self.weight_name)

    def forward_streams(self, x, pending, read_w, out, rows=None, store=True):
        if x.dim() == 2:
            x = x.unsqueeze(1)          # one stream
        if pending is not None and not isinstance(pending, StreamsPending):
            raise TypeError(f"several residual streams take a StreamsPending, not {type(pending).__name__}")
        y, mix, out_w, mult = (pending.y, pending.mix, pending.out_w, pending.mult) if pending is not None else (None, None, None, 0.0)
        kernels.streams_mix_rmsnorm(x, y, mix, out_w, mult, read_w, self.weight, self.eps, out, rows=rows, store=store)

    def forward(self, h, delta, out, rows=None, store_h=True):
        if h.dim() == 3 or isinstance(delta, StreamsPending):
            # several residual streams: whoever asks for the plain norm (the output head) reads their sum
            self.forward_streams(h, delta, None, out, rows=rows, store=store_h)
            return
        if isinstance(delta, NormedPending):
            if isinstance(delta.norm, RMSNorm):
                # the norm of the sublayer's output, the sum and this norm in one launch
                kernels.normed_add_rmsnorm(h, delta.y, delta.norm.weight, delta.norm.eps, self.weight, self.eps, out,
                                           rows=rows, store_h=store_h)
                return
            delta = delta.materialize()
        kernels.add_rmsnorm(h, delta, self.weight, self.eps, out, rows=rows, store_h=store_h)
