"""Position encodings for attention.

``RotaryEncoding`` restates src/forge_engine/qwen3.py:345-363: inv_freq_j =
1 / theta^(2j / rotary_dim) in 32-bit, angle = float(position) * inv_freq_j; the
rotation itself happens inside the fused q/k kernel.  Cosine and sine of a step's angles
are the same in every layer: ``table`` takes them once per step (in 32-bit, not rounded)."""

from __future__ import annotations

import torch

from ..ops import native
from .base import BuildContext, PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.rotary_dim = spec.rotary_dim
        self.theta = float(spec.theta)
        # which elements form a pair is the business of the kernel that rotates; the angles
        # are the same either way
        self.interleaved = bool(getattr(spec, "interleaved", False))
        if self.interleaved:
            # theta^(-2j / rotary_dim) worked out in 64-bit and rounded once
            exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float64) / spec.rotary_dim
            self.inv_freq = (self.theta ** -exponent).float().to(ctx.device).contiguous()
        else:
            exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32) / spec.rotary_dim
            self.inv_freq = (1.0 / (spec.theta**exponent)).to(ctx.device).contiguous()
        self.scaling = getattr(spec, "scaling", None)
        self.exact = bool(getattr(spec, "exact_frequencies", False))
        if self.scaling is not None or getattr(spec, "exact_frequencies", False):
            exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float64) / spec.rotary_dim
            freq = self.theta ** -exponent
            if self.scaling is not None:
                freq = self.stretch(freq, self.scaling)
            self.inv_freq = freq.float().to(ctx.device).contiguous()

    @staticmethod
    def stretch(freq: torch.Tensor, scaling: tuple) -> torch.Tensor:
        """Frequencies stretched by wavelength l = 2 pi / f (64-bit in, 64-bit out): kept below
        original / high, divided by ``factor`` above original / low, and blended in between with
        s = (original / l - low) / (high - low) as (1 - s) f / factor + s f."""
        import math

        factor, low, high, original = (float(v) for v in scaling)
        if factor <= 0 or high <= low or original <= 0:
            raise ValueError("frequency scaling needs factor > 0, original > 0 and high > low")
        wave = 2.0 * math.pi / freq
        s = (original / wave - low) / (high - low)
        blended = (1.0 - s) * freq / factor + s * freq
        return torch.where(wave < original / high, freq, torch.where(wave > original / low, freq / factor, blended))

    def rotary(self):
        return self.inv_freq, self.rotary_dim

    def table(self, batch) -> torch.Tensor:
        """[tokens, rotary_dim / 2, 2] (cos, sin) of this step's angles; worked out by the
        first layer that asks and shared through the batch."""
        key = ("rotary", self.theta, self.rotary_dim, self.interleaved, self.scaling, self.exact)
        table = batch.shared.get(key)
        if table is None:
            table = torch.empty((batch.n_tokens, self.rotary_dim // 2, 2), dtype=torch.float32, device=self.inv_freq.device)
            native.rope_table(batch.positions, self.inv_freq, table)
            batch.shared[key] = table
        return table


class NoPosition(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        pass


register_part("rope", RotaryEncoding, replace=True)
register_part("none", NoPosition, replace=True)
