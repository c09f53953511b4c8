"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, in float32 (engine/src/kernels.c:94-111).
LayerNorm: y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b, in float32."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Norm, StepContext


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, weight: torch.Tensor):
        if weight.shape != (width,):
            raise ValueError(f"RMSNorm weight is {tuple(weight.shape)}, expected ({width},)")
        self.width, self.eps = width, float(eps)
        self.weight = weight.to(torch.float32).contiguous()   # the norm's weights are float32 in both paths

    def tensors(self):
        return [self.weight]

    def as_rms(self):
        return self.weight, self.eps

    def forward(self, x: torch.Tensor, ctx: StepContext, name: str, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.workspace.rows(name, n, self.width, ctx.dtype)
        return ops.rmsnorm_rows(x, self.weight, self.eps, out, rows)


class LayerNorm(Norm):
    """The norm with a weight and a bias; it has no RMS form, so no product applies it in its own first kernel."""

    def __init__(self, width: int, eps: float, weight: torch.Tensor, bias: torch.Tensor):
        if weight.shape != (width,) or bias.shape != (width,):
            raise ValueError(f"LayerNorm weight and bias are {tuple(weight.shape)} and {tuple(bias.shape)}, expected ({width},)")
        self.width, self.eps = width, float(eps)
        self.weight = weight.to(torch.float32).contiguous()
        self.bias = bias.to(torch.float32).contiguous()

    def tensors(self):
        return [self.weight, self.bias]

    def forward(self, x: torch.Tensor, ctx: StepContext, name: str, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.workspace.rows(name, n, self.width, ctx.dtype)
        return ops.layernorm_rows(x, self.weight, self.bias, self.eps, out, rows)

    def in_place(self, x: torch.Tensor) -> torch.Tensor:
        """Norms the float32 rows where they lie (an embedding that is normed before the first layer)."""
        return ops.layernorm_rows(x, self.weight, self.bias, self.eps, x)
