"""Normalisation parts."""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm:
    """out = weight * (x / sqrt(mean(x^2) + eps)), computed in 32-bit from the 32-bit residual
    stream (src/kernels/kernels.cpp:72-83); the weight is used as is (no ``1 + w``) and is kept in
    32-bit whatever the checkpoint stores. Params: ``size``, ``eps`` and optionally ``weight_offset`` (0): a
    checkpoint that stores its norm weights around zero and applies ``offset + w`` is served by adding the
    offset once, in 32-bit, when the model is built. Weights: ``weight`` [size]."""

    def __init__(self, params, weights, build):
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        w = weights["weight"]
        if tuple(w.shape) != (self.size,):
            raise ValueError(f"rmsnorm: weight has shape {tuple(w.shape)}, expected ({self.size},)")
        self.weight_offset = float(params.get("weight_offset", 0.0))
        self.weight = w.to(device=build.device, dtype=torch.float32).contiguous()
        if self.weight_offset:
            self.weight += self.weight_offset

    def launch_key(self, ctx):
        """Its one launch depends on the number of rows only (which the caller's key holds)."""
        return ()

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        kernels.rmsnorm(x, self.weight, out, self.eps, rows)
        return out


@register_norm("rmsnorm_scalar")
class ScalarRMSNorm(RMSNorm):
    """out = g * (x / sqrt(mean(x^2) + eps)) with a single learned number g for all coordinates. Params: ``size``,
    ``eps``. Weights: ``weight``, one value (any shape). It runs the RMSNorm kernel over g repeated ``size`` times;
    ``scalar`` keeps the one number on the device for kernels that apply the norm themselves."""

    not_weights = ("weight",)       # g repeated: the model's weight is ``scalar``

    def __init__(self, params, weights, build):
        g = weights["weight"]
        if g.numel() != 1:
            raise ValueError(f"rmsnorm_scalar: the weight has {g.numel()} values, expected one")
        size = int(params["size"])
        super().__init__(params, {"weight": g.reshape(1).float().expand(size)}, build)
        self.scalar = g.reshape(1).to(device=build.device, dtype=torch.float32).contiguous()
