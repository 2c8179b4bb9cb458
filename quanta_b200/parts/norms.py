"""RMSNorm with the residual sum folded in (src/quanta/minimax/model_m3.py:60-65)."""

from __future__ import annotations

import torch

from .. import kernels
from .base import Norm, TensorSpec, register


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

    def forward(self, h, delta, out, rows=None, store_h=True):
        kernels.add_rmsnorm(h, delta, self.weight, self.eps, out, rows=rows, store_h=store_h)
