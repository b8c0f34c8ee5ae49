"""Position encodings that act on queries and keys inside the attention part.

``rope``: rotary encoding (half-split, or neighbouring dimensions paired); ``inv_freq[i] = theta^(-2i/rot_dim)``
(src/layers/rope.cpp:20-29); the rotation itself, with angles computed in
float32 from the absolute position, runs in the kernel that also adds the
projection bias and writes the cache (reference: cos/sin tables rounded to
FP16, src/kernels/rope_kernel.cu:65-77, and a separate rotation kernel, :27-54).

``none``: queries and keys are used as projected.

A further rotary variant (other frequencies, partial rotation) is a new class
that returns another table and ``rot_dim``; the kernel takes both as arguments.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from ..config.registry import register_part
from .base import PositionEncoding


class RotaryEncoding(PositionEncoding):
    """params: ``head_dim``, ``theta``, optional ``rot_dim`` (default ``head_dim``) and ``pairing``: which
    dimensions turn together, ``halves`` (default: ``i`` with ``i + rot_dim / 2``) or ``neighbours`` (``2i``
    with ``2i + 1``); pair ``i`` turns by ``position * theta^(-2i/rot_dim)`` either way."""

    graph_safe = True
    PAIRINGS = ("halves", "neighbours")

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.pairing = self.params.get("pairing", "halves")
        if self.pairing not in self.PAIRINGS:
            raise ValueError(f"rope: pairing '{self.pairing}' is not one of {self.PAIRINGS}")
        d = int(self.params["head_dim"])
        self.rot_dim = int(self.params.get("rot_dim", d))
        if self.rot_dim % 2 or not 0 < self.rot_dim <= d:
            raise ValueError(f"rope: rot_dim {self.rot_dim} must be even and within head_dim {d}")
        self.theta = float(self.params["theta"])
        self._table = {}

    def table(self, device) -> Optional[torch.Tensor]:
        key = str(device)
        if key not in self._table:
            i = torch.arange(self.rot_dim // 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rot_dim)
            self._table[key] = inv.to(torch.float32).to(device)
        return self._table[key]


class ScaledRotaryEncoding(RotaryEncoding):
    """Rotary frequencies rescaled by wavelength (the rule Llama 3.1 introduced for long contexts).

    params: as ``rope``, plus ``factor``, ``low``, ``high``, ``original``.  With wavelength
    ``l = 2 pi / f``: ``f`` stays where ``l < original / high``; becomes ``f / factor`` where
    ``l > original / low``; and in between, with ``s = (original / l - low) / (high - low)``, becomes
    ``(1 - s) f / factor + s f``."""

    def table(self, device) -> Optional[torch.Tensor]:
        key = str(device)
        if key not in self._table:
            p = self.params
            factor, low, high, original = (float(p[k]) for k in ("factor", "low", "high", "original"))
            i = torch.arange(self.rot_dim // 2, dtype=torch.float64)
            f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rot_dim)
            wavelength = 2.0 * math.pi / f
            s = (original / wavelength - low) / (high - low)
            blended = (1.0 - s) * f / factor + s * f
            f = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, blended))
            self._table[key] = f.to(torch.float32).to(device)
        return self._table[key]


class NoPositionEncoding(PositionEncoding):
    graph_safe = True
    rot_dim = 0
    pairing = "halves"

    def table(self, device) -> Optional[torch.Tensor]:
        return None


register_part("position", "rope", RotaryEncoding)
register_part("position", "rope_scaled", ScaledRotaryEncoding)
register_part("position", "none", NoPositionEncoding)
