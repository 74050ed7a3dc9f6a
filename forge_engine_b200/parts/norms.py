"""RMS normalisation (src/forge_engine/qwen3.py:91-105), fused with the residual sum
(src/forge_engine/_triton_kernels.py:32-58).  Sum, variance, scaling and the weight
product are all taken in 32-bit; the result is rounded once, on store."""

from __future__ import annotations

import torch

from ..config.specs import local_name
from ..ops import native
from .base import BuildContext, Norm, WeightInfo, register_part


class RMSNorm(Norm):
    graph_safe = True
    stream_kind = native.NORM_RMS     # what the kernel over several residual streams is told

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        self.size = spec.size
        self.eps = float(spec.eps)
        self.weight = weights[local_name(spec, "weight")].to(device=ctx.device, dtype=torch.float32).contiguous()
        offset = float(getattr(spec, "weight_offset", 0.0) or 0.0)
        if offset:
            # the stored weight is the distance from ``offset``; the sum is taken once, in 32-bit
            self.weight = (self.weight + offset).contiguous()
        self.dtype = ctx.dtype

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        stored_near_zero = bool(getattr(spec, "weight_offset", 0.0))
        return {local_name(spec, "weight"): WeightInfo((spec.size,), "small" if stored_near_zero else "norm")}

    def add_forward(self, residual, update, row_map=None, shift=None):
        """residual (32-bit [N, size]) += update (+ ``shift``, a 32-bit vector added to every
        row); returns the normalised rows in the activation dtype.  With ``row_map`` only
        those rows are produced and the residual is left untouched."""
        rows = residual.shape[0] if row_map is None else row_map.numel()
        out = torch.empty((rows, self.size), dtype=self.dtype, device=residual.device)
        native.add_rmsnorm(residual, update, self.weight, out, self.eps, row_map,
                           write_residual=row_map is None, shift=shift)
        return out

    def forward(self, x):
        """Norm of a 32-bit tensor without a residual update."""
        return self.add_forward(x, None)


class LayerNorm(Norm):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight, no bias; mean, deviations and the
    weight product in 32-bit, one rounding on store."""

    graph_safe = True
    stream_kind = native.NORM_LAYER

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        self.size = spec.size
        self.eps = float(spec.eps)
        self.weight = weights[local_name(spec, "weight")].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.dtype = ctx.dtype

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        return {local_name(spec, "weight"): WeightInfo((spec.size,), "norm")}

    def add_forward(self, residual, update, row_map=None):
        """residual (32-bit [N, size]) += update; returns the normalised rows in the
        activation dtype.  With ``row_map`` only those rows are produced and the residual
        is left untouched."""
        rows = residual.shape[0] if row_map is None else row_map.numel()
        out = torch.empty((rows, self.size), dtype=self.dtype, device=residual.device)
        native.stream_mix_norm(residual, update, 1.0, None, None, None, native.NORM_LAYER, self.weight, self.eps,
                               out, row_map, write_streams=row_map is None)
        return out

    def forward(self, x):
        return self.add_forward(x, None)


register_part("rmsnorm", RMSNorm, replace=True)
register_part("layernorm", LayerNorm, replace=True)
