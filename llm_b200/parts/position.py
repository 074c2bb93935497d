"""Rotary position encoding (rotate-half).

Tables as the reference builds them (kernel/embedding/RoPECache.h:15-20):
inv_i = theta^(-2i/HS), angle = pos * inv_i formed in float32, cos and sin of that
angle, for pos < max_position and i < HS/2.  The power and the cos/sin are evaluated
in float64 on the host and rounded once, so the table holds the correctly rounded
values of the 32-bit angle.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Part, register_part


class RotaryEmbedding(Part):
    role = "position"

    def __init__(self, head_dim: int, theta: float, max_position: int, prefix: str = "", dtype=None,
                 device=None):
        super().__init__(prefix, dtype, device)
        if head_dim % 2:
            raise ValueError(f"rope: head_dim {head_dim} must be even")
        self.head_dim, self.theta, self.max_position = head_dim, float(theta), int(max_position)
        self._tables = None

    def host_tables(self):
        half = self.head_dim // 2
        i = np.arange(half, dtype=np.float64)
        inv = np.power(np.float64(self.theta), -2.0 * i / self.head_dim).astype(np.float32)
        pos = np.arange(self.max_position, dtype=np.float32)
        ang = (pos[:, None] * inv[None, :]).astype(np.float32)        # one float32 product
        ang64 = ang.astype(np.float64)
        return np.cos(ang64).astype(np.float32), np.sin(ang64).astype(np.float32)

    def tables(self):
        """(cos, sin), float32 [max_position, head_dim/2] on the device."""
        if self._tables is None:
            key = (self.head_dim, self.theta, self.max_position, str(self.device))
            if key not in _TABLE_CACHE:      # layers with the same constants share one table
                c, s = self.host_tables()
                _TABLE_CACHE[key] = (torch.from_numpy(c).to(self.device).contiguous(),
                                     torch.from_numpy(s).to(self.device).contiguous())
            self._tables = _TABLE_CACHE[key]
        return self._tables


_TABLE_CACHE = {}


class PairRotary(Part):
    """RoPE on neighbouring pairs: channels 2i and 2i+1 of a head (i < dims/2) turn by position * f_i, the rest of
    the head passes.  f_i = base^(-2i/dims), rescaled by wavelength l = 2 pi / f if `scaling` is given
    ({factor, low, high, original}): kept where l < original/high, divided by factor where l > original/low,
    and in between blended, (1 - s) f / factor + s f with s = (original / l - low) / (high - low).  The part
    gives the frequencies (float32, evaluated in float64 and rounded once); the angle is one float32 product in
    the kernel that rotates and stores, so no table bounds the position.  layout "halves" pairs channel i with channel
    i + dims/2 (rotate-half on the first dims channels) with the same frequencies."""

    role = "position"

    def __init__(self, dims: int, base: float, scaling=None, layout: str = "pairs", prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if layout not in ("pairs", "halves"):
            raise ValueError(f"pair rotation: layout '{layout}' is neither 'pairs' nor 'halves'")
        self.layout = layout        # "halves": channel i turns against channel i + dims/2 instead of 2i against 2i + 1
        if dims < 0 or dims % 2:
            raise ValueError(f"pair rotation: dims {dims} must be even and not negative")
        self.dims, self.base = int(dims), float(base)
        self.scaling = dict(scaling) if scaling else None
        if self.scaling:
            for k in ("factor", "low", "high", "original"):
                if k not in self.scaling:
                    raise ValueError(f"pair rotation: scaling lacks '{k}'")
            if self.scaling["high"] == self.scaling["low"]:
                raise ValueError("pair rotation: scaling.high equals scaling.low")
        self._freqs = None

    def host_frequencies(self) -> np.ndarray:
        i = np.arange(self.dims // 2, dtype=np.float64)
        f = np.power(np.float64(self.base), -2.0 * i / max(self.dims, 1))
        sc = self.scaling
        if sc:
            factor, low, high, orig = (float(sc[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * np.pi / f
            s = (orig / wave - low) / (high - low)
            blended = (1.0 - s) * f / factor + s * f
            f = np.where(wave < orig / high, f, np.where(wave > orig / low, f / factor, blended))
        return f.astype(np.float32)

    def frequencies(self):
        """float32 [dims/2] on the device, or None when nothing turns."""
        if self.dims == 0:
            return None
        if self._freqs is None:
            self._freqs = torch.from_numpy(self.host_frequencies()).to(self.device).contiguous()
        return self._freqs


register_part("position", "rope_pairs", PairRotary)


register_part("position", "rope", RotaryEmbedding)
