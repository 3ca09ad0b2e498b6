"""Rotary position encoding, rotate-half ("NeoX") pairing.

As the reference builds it (src/models/qwen2.cpp:608-671): for pair index
``i < rotary/2`` the frequency is ``theta ** (-2i / rotary)`` evaluated in
float32, the angle of position ``p`` is ``float(p) * freq`` in float32, and
the tables hold ``cos`` and ``sin`` of that angle.  The rotation
(src/cpu/scalar/norm_rope_scalar.cpp:23-41) pairs element ``i`` with element
``i + rotary/2``:  ``lo' = lo*cos - hi*sin``, ``hi' = lo*sin + hi*cos``.
Values are not rotated, and keys are stored rotated.

The tables are computed on the host: the exponent and the angle in float32
exactly as above, ``pow``, ``cos`` and ``sin`` in float64 of those float32
arguments and rounded once, which is what a correctly rounded float32
routine returns.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .base import POSITIONS, PositionEncoding


def rescale_by_wavelength(freq: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Frequencies (float64) slowed down for long wavelengths: with l = 2 pi / f, f is kept where
    l < original / high, divided by ``factor`` where l > original / low, and between the two blended,
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    wavelength = 2.0 * math.pi / freq
    s = (original / wavelength - low) / (high - low)
    blended = (1.0 - s) * freq / factor + s * freq
    out = torch.where(wavelength > original / low, freq / factor, blended)
    return torch.where(wavelength < original / high, freq, out)


def rotary_tables(theta: float, rotary: int, positions: int,
                  scaling: Optional[Tuple[float, float, float, float]] = None,
                  precise: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of position * frequency, float32 [positions, rotary/2].  By default the exponent, the
    frequency and the angle are each rounded to float32 as described above; with ``precise`` all of it is
    float64 and only the cosine and the sine are rounded (an angle of a thousand radians in float32 is already
    off by 6e-5)."""
    half = rotary // 2
    if precise:
        index = torch.arange(half, dtype=torch.float64)
        freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * index / float(rotary))
        if scaling is not None:
            freq = rescale_by_wavelength(freq, *scaling)
        angle = torch.arange(positions, dtype=torch.float64)[:, None] * freq[None, :]
        return torch.cos(angle).float(), torch.sin(angle).float()
    index = torch.arange(half, dtype=torch.float32)
    exponent = (-2.0 * index) / torch.tensor(float(rotary), dtype=torch.float32)          # float32
    theta32 = torch.tensor(theta, dtype=torch.float32)
    freq = torch.pow(theta32.double(), exponent.double())
    if scaling is not None:
        freq = rescale_by_wavelength(freq, *scaling)
    freq = freq.float()                                                                     # rounded once
    angle = torch.arange(positions, dtype=torch.float32)[:, None] * freq[None, :]          # float32 product
    return torch.cos(angle.double()).float(), torch.sin(angle.double()).float()


_TABLES: dict = {}


@POSITIONS.register("rope_neox")
class RotaryNeoX(PositionEncoding):
    """params: ``head_dim``, ``theta``, optional ``rotary_dim`` (default head_dim), optional ``scaling``
    (``{"factor", "low", "high", "original"}``: frequencies rescaled by wavelength, see
    :func:`rescale_by_wavelength`), optional ``precise`` (tables from float64 angles)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        self.rotary = int(spec.params.get("rotary_dim", self.head_dim))
        if self.rotary <= 0 or self.rotary % 2 or self.rotary > self.head_dim:
            raise ValueError(f"rope: rotary width {self.rotary} must be even and within head_dim {self.head_dim}")
        if not self.theta > 0:
            raise ValueError("rope: theta must be positive")
        scaling = spec.params.get("scaling")
        self.scaling = None
        if scaling is not None:
            self.scaling = tuple(float(scaling[name]) for name in ("factor", "low", "high", "original"))
            factor, low, high, original = self.scaling
            if not (factor > 0 and original > 0 and high > low >= 0):
                raise ValueError(f"rope: scaling {scaling!r} needs factor > 0, original > 0 and high > low >= 0")
        # layers with the same base, width and length share one pair of tables
        self.precise = bool(spec.params.get("precise", False))
        key = (self.theta, self.rotary, env.max_positions, str(env.device), self.scaling, self.precise)
        if key not in _TABLES:
            if len(_TABLES) >= 8:
                _TABLES.pop(next(iter(_TABLES)))
            cos, sin = rotary_tables(self.theta, self.rotary, env.max_positions, self.scaling, self.precise)
            _TABLES[key] = (cos.to(env.device).contiguous(), sin.to(env.device).contiguous())
        self.cos, self.sin = _TABLES[key]

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor, int]]:
        return self.cos, self.sin, self.rotary


def pair_tables(theta: float, dims: int, positions: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of position * theta^(-2i / dims), i < dims / 2, float32 [positions, dims / 2]; frequencies and
    angles in float64, rounded once."""
    index = torch.arange(dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * index / float(dims))
    angle = torch.arange(positions, dtype=torch.float64)[:, None] * freq[None, :]
    return torch.cos(angle).float(), torch.sin(angle).float()


@POSITIONS.register("rope_interleaved")
class RotaryInterleaved(PositionEncoding):
    """Rotation of neighbouring pairs: element 2i is paired with element 2i+1 (i < dims / 2), and the pair (u, v) at
    position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * theta^(-2i / dims); elements from ``dims`` on
    pass unchanged.  The fused rotate-and-store kernel pairs halves, not neighbours, so this encoding is applied by a
    kernel of its own (``apply``), or by a mixer's own kernel from the tables (``pair_tables``).

    params: ``head_dim`` (width of the rotated run), ``theta``, optional ``rotary_dim`` (default head_dim)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        self.rotary = int(spec.params.get("rotary_dim", self.head_dim))
        if self.rotary < 0 or self.rotary % 2 or self.rotary > self.head_dim:
            raise ValueError(f"rope: rotary width {self.rotary} must be even and within {self.head_dim}")
        if not self.theta > 0:
            raise ValueError("rope: theta must be positive")
        key = ("pairs", self.theta, self.rotary, env.max_positions, str(env.device))
        if key not in _TABLES:
            if len(_TABLES) >= 8:
                _TABLES.pop(next(iter(_TABLES)))
            cos, sin = pair_tables(self.theta, max(self.rotary, 2), env.max_positions)
            _TABLES[key] = (cos.to(env.device).contiguous(), sin.to(env.device).contiguous())
        self.cos, self.sin = _TABLES[key]

    def pair_tables(self) -> Tuple[torch.Tensor, torch.Tensor, int]:
        return self.cos, self.sin, self.rotary

    def rotary_tables(self):
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        for t in (q, k):
            tokens, heads, dim = t.shape
            flat = t.reshape(tokens, heads * dim) if t.is_contiguous() else None
            if flat is None:
                # a view into a wider row (q or k inside a q/k/v row): rows stay dense, heads follow one another
                flat = t.as_strided((tokens, heads * dim), (t.stride(0), 1))
            before = flat.clone()
            self.ops.rotate_interleaved(before, dim, flat, dim, heads, dim, self.cos, self.sin, self.rotary, positions)


@POSITIONS.register("none")
class NoPosition(PositionEncoding):
    """Leaves queries and keys as they are."""
    graph_safe = True

    def rotary_tables(self):
        return None, None, 0
