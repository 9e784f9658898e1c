"""Rotary position encoding.

Reference formula (models/rope.py:14-35): ``inv_freq[j] = 1 / base**(2j/dim)`` for
``j < dim/2`` (32-bit), ``theta = pos * inv_freq[j]`` (32-bit), and the rotation of
**interleaved pairs**: ``out[2j] = x[2j]*cos - x[2j+1]*sin``,
``out[2j+1] = x[2j]*sin + x[2j+1]*cos``.  The reference's CUDA rope kernel rotates
half-split pairs ``(j, j+dim/2)`` instead (kernels/rope_kernel/rope_kernel.cu:133-157);
its serving path and its golden generation use the interleaved form, which is the
default here, and ``style="half"`` gives the other.  The base is fixed in the
reference (models/rope.py:6); here it is this part's parameter.

``inv_freq`` is built once with the reference's own expression so that the angle
``float(pos) * inv_freq[j]`` has the very same 32-bit rounding; the kernels take
sine and cosine of that product in 32-bit.

``scaling`` (optional; ``factor``, ``low``, ``high``, ``original``) rescales the frequencies by their wavelength
``l = 2 pi / f`` against a context length ``original``: a frequency with ``l < original / high`` stays, one with
``l > original / low`` becomes ``f / factor``, and between the two ``s = (original / l - low) / (high - low)`` blends
``(1 - s) f / factor + s f``.  ``dim`` is the number of rotated values; a mixer may rotate only the first ``dim``
values of a wider head.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from ..registry import register_part

ROTARY_STYLES = {"interleaved": 0, "half": 1}


@register_part("position", "rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, prefix: str, dim: int, base: float, style: str = "interleaved", scaling=None):
        super().__init__(prefix)
        if dim % 2:
            raise ValueError(f"rotary dimension {dim} must be even (models/rope.py:8)")
        if style not in ROTARY_STYLES:
            raise ValueError(f"unknown rotary style {style!r}; known: {sorted(ROTARY_STYLES)}")
        self.dim, self.base, self.style = int(dim), float(base), style
        self.scaling = None
        if scaling is not None:
            missing = [k for k in ("factor", "low", "high", "original") if k not in scaling]
            if missing:
                raise ValueError(f"rotary scaling lacks {missing}")
            self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")}
            if not self.scaling["high"] > self.scaling["low"] or self.scaling["factor"] <= 0 or self.scaling["low"] <= 0:
                raise ValueError(f"rotary scaling {scaling!r}: needs factor > 0 and high > low > 0")
        self._inv_freq = None

    def frequencies(self) -> torch.Tensor:
        """float32 [dim / 2]: the rotation frequency of every pair."""
        if self.scaling is None:
            return 1.0 / (self.base ** (torch.arange(0, self.dim, 2).float() / self.dim))
        sc, out = self.scaling, []
        for i in range(self.dim // 2):                               # few values, once: in 64-bit, rounded at the end
            f = self.base ** (-2.0 * i / self.dim)
            wavelength = 2.0 * math.pi / f
            if wavelength < sc["original"] / sc["high"]:
                out.append(f)
            elif wavelength > sc["original"] / sc["low"]:
                out.append(f / sc["factor"])
            else:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * f / sc["factor"] + s * f)
        return torch.tensor(out, dtype=torch.float64).to(torch.float32)

    def bind(self, ops, dtype, device):
        super().bind(ops, dtype, device)
        self._inv_freq = self.frequencies().to(device=device, dtype=torch.float32).contiguous()

    def rotary_table(self):
        return self._inv_freq, ROTARY_STYLES[self.style]

    def step_table(self, ctx):
        """cos/sin of every token of the step, computed once per step and shared by all layers whose
        encoding has the same dimension and base (kept in the step's context)."""
        if not hasattr(self.ops, "rope_table"):
            return None
        tables = ctx.step_cache
        key = ("rope_table", self.dim, self.base, None if self.scaling is None else tuple(sorted(self.scaling.items())))
        if key not in tables:
            tables[key] = self.ops.rope_table(ctx.positions, self._inv_freq)
        return tables[key]

    def apply(self, q, k, positions):
        raise NotImplementedError("rotary encoding runs inside the fused rotate-and-store kernel")


@register_part("position", "none")
class NoPosition(PositionEncoding):
    """No position encoding: keys and queries are stored and used as projected."""

    def __init__(self, prefix: str = ""):
        super().__init__(prefix)

    def rotary_table(self):
        return None, 0

    def step_table(self, ctx):
        return None

    def apply(self, q, k, positions):
        return None
