"""Rotary position encoding: tables of cos/sin(pos * theta_j) and the pairing.

theta_j = base^(-2j/rot_dim), optionally divided by per-pair divisors, all in
float32 (zllm src/backend/candle/quantized_llama_fork.rs:579-590); tables for
positions 0..max_position as the float32 product pos * theta_j followed by
cos/sin (fork.rs:631-638).  The reference receives llama3 divisors precomputed in the
model file; from ``rope_scaling`` of a config.json they are computed here: with
wavelength lambda_j = 2 pi / theta_j, f_j = 1 below L/high, F above L/low, and a
linear blend of theta_j/F and theta_j in between.  ``linear`` scaling divides
every theta_j by the factor (fork.rs:592-597).

Pairing: ``interleaved`` rotates (x[2j], x[2j+1]) (the reference's ``rope_i``,
shaders.rs:576-586); otherwise (x[j], x[j + rot_dim/2]) (its ``rope_neox``,
fork.rs:447-451), which is the layout of unpermuted safetensors weights.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from ..errors import ConfigError
from .base import PositionEncoding, register_position_encoding


@dataclass
class RotaryTables:
    cos: torch.Tensor          # [max_position, rot_dim/2] float32, on device
    sin: torch.Tensor
    rot_dim: int
    interleaved: bool
    max_position: int


def frequency_divisors(rot_dim: int, theta: float, scaling: Optional[dict]) -> Optional[torch.Tensor]:
    """The per-pair divisors f_j of ``llama3`` scaling, float32, as a model file would store them
    (the reference reads them from ``rope_freqs.weight``, fork.rs:584-590, 722-734); None when the
    scaling has none.  This is the converter's share of the work, so it is done in double precision
    and rounded once: f_j = 1 where the wavelength is below L/high, F above L/low, and in between
    theta_j / ((1 - s) theta_j / F + s theta_j) with s = (L / wavelength - low) / (high - low)."""
    if not scaling or scaling.get("rope_type") != "llama3":
        return None
    F = float(scaling["factor"])
    lo = float(scaling["low_freq_factor"])
    hi = float(scaling["high_freq_factor"])
    L = float(scaling["original_max_position_embeddings"])
    if hi <= lo:
        raise ConfigError("rope_scaling (llama3): high_freq_factor must exceed low_freq_factor")
    j = torch.arange(0, rot_dim, 2, dtype=torch.float64)
    wavelen = 2.0 * math.pi * torch.pow(torch.tensor(float(theta), dtype=torch.float64), j / rot_dim)
    smooth = (L / wavelen - lo) / (hi - lo)
    blend = 1.0 / ((1.0 - smooth) / F + smooth)
    one = torch.ones_like(wavelen)
    return torch.where(wavelen < L / hi, one, torch.where(wavelen > L / lo, one * F, blend)).to(torch.float32)


def inverse_frequencies(rot_dim: int, theta: float, scaling: Optional[dict], freq_factors=None) -> torch.Tensor:
    """theta_j in float32, computed as the reference computes it: 1 / base^(i / rot_dim) with
    every operand float32 (fork.rs:579-583), then divided by the divisors that are not zero
    (fork.rs:584-590), then ``linear`` scaling as a multiplication by 1 / factor (fork.rs:592-597)."""
    f32 = torch.float32
    i = torch.arange(0, rot_dim, 2, dtype=f32)
    inv = 1.0 / torch.pow(torch.tensor(float(theta), dtype=f32), i / torch.tensor(float(rot_dim), dtype=f32))
    kind = scaling.get("rope_type") if scaling else None
    if kind not in (None, "default", "llama3", "linear"):
        raise ConfigError(f"rotary scaling {kind!r} is not supported (llama3, linear)")
    for div in (frequency_divisors(rot_dim, theta, scaling),
                torch.as_tensor(freq_factors, dtype=f32) if freq_factors is not None else None):
        if div is None:
            continue
        if div.numel() != inv.numel():
            raise ConfigError(f"rotary: {div.numel()} frequency divisors for {inv.numel()} pairs")
        inv = torch.where(div != 0, inv / torch.where(div != 0, div, torch.ones_like(div)), inv)
    if kind == "linear":
        inv = inv * (torch.tensor(1.0, dtype=f32) / max(float(scaling["factor"]), 1e-6))
    return inv


@register_position_encoding("rotary")
class Rotary(PositionEncoding):
    capturable = True

    def __init__(self, rot_dim: int, theta: float, max_position: int, scaling: Optional[dict] = None,
                 interleaved: bool = False, freq_factors=None):
        if rot_dim <= 0 or rot_dim % 2:
            raise ConfigError(f"rotary: rot_dim {rot_dim} must be positive and even")
        self.rot_dim = int(rot_dim)
        self.theta = float(theta)
        self.max_position = int(max_position)
        self.scaling = scaling
        self.interleaved = bool(interleaved)
        # explicit divisors are the reference's own mechanism (fork.rs:584-590); 0 means "leave"
        self.inv_freq = inverse_frequencies(self.rot_dim, self.theta, scaling, freq_factors)
        self._tables = None

    def bind(self, rt):
        super().bind(rt)
        pos = torch.arange(self.max_position, dtype=torch.float32)
        ang = pos[:, None] * self.inv_freq[None, :]          # float32 product, as the reference
        self._tables = RotaryTables(ang.cos().contiguous().to(rt.device), ang.sin().contiguous().to(rt.device),
                                    self.rot_dim, self.interleaved, self.max_position)

    def rotary(self):
        return self._tables


def yarn_frequencies(dims: int, base: float, factor: float, original: int, fast: float, slow: float):
    """(frequencies of the dims/2 pairs, magnitude) under YaRN scaling.

    g_i = base^(-2i/dims).  d(t) = dims ln(original / (2 pi t)) / (2 ln base) is the pair index whose
    wave makes t turns over ``original`` positions; lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)),
    dims - 1); ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); pair i gets
    g_i / factor * ramp_i + g_i * (1 - ramp_i): fast pairs keep their frequency, slow pairs are
    stretched by ``factor``, a linear blend in between.  cos and sin are multiplied by
    0.1 ln(factor) + 1.  Computed in double precision and rounded once to float32."""
    if dims <= 0 or dims % 2:
        raise ConfigError(f"rotary: dims {dims} must be positive and even")
    i = torch.arange(dims // 2, dtype=torch.float64)
    g = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)

    def d(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(d(fast)), 0)
    hi = min(math.ceil(d(slow)), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (g / factor * ramp + g * (1.0 - ramp)).to(torch.float32), 0.1 * math.log(factor) + 1.0


def stretched_frequencies(dims: int, base: float, factor: float, original: float, low: float, high: float):
    """The frequencies of the dims/2 pairs with long waves slowed down (the scheme of Llama 3.1).

    g_i = base^(-2i/dims) has the wavelength l_i = 2 pi / g_i.  A wave shorter than original/high keeps
    its frequency; one longer than original/low gets g_i / factor; in between, with
    s = (original / l_i - low) / (high - low), the pair gets (1 - s) g_i / factor + s g_i.
    Computed in double precision and rounded once to float32."""
    if dims <= 0 or dims % 2:
        raise ConfigError(f"rotary: dims {dims} must be positive and even")
    if not high > low:
        raise ConfigError("rotary scaling: 'high' must exceed 'low'")
    i = torch.arange(dims // 2, dtype=torch.float64)
    g = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    wavelength = 2.0 * math.pi / g
    s = (original / wavelength - low) / (high - low)
    blend = (1.0 - s) * g / factor + s * g
    return torch.where(wavelength < original / high, g, torch.where(wavelength > original / low, g / factor, blend)).to(torch.float32)


@dataclass
class RotaryFrequencies:
    freq: torch.Tensor        # [dims/2] float32, on device
    magnitude: float          # multiplies cos and sin
    dims: int
    interleaved: bool = False  # pairs (2i, 2i+1) instead of (i, i + dims/2)

    def as_tuple(self):
        return (self.freq, self.magnitude, self.dims)


@register_position_encoding("rotary_on_the_fly")
class RotaryOnTheFly(PositionEncoding):
    """Rotary encoding without tables: kernels get the pairs' frequencies and compute the angle
    position * frequency in float32 themselves, so there is no largest position.  Pairing:
    half-split (entry i with entry i + dims/2) or, with ``interleaved``, neighbours (2i, 2i+1).
    ``scaling`` None, the YaRN constants {factor, original, fast, slow}, or the constants of the
    stretching of long waves {factor, original, low, high} (``stretched_frequencies``)."""

    capturable = True

    def __init__(self, dims: int, base: float, scaling: Optional[dict] = None, interleaved: bool = False):
        self.dims = int(dims)
        self.base = float(base)
        self.scaling = dict(scaling) if scaling else None
        self.interleaved = bool(interleaved)
        if self.scaling and "low" in self.scaling:
            for k in ("factor", "original", "low", "high"):
                if k not in self.scaling:
                    raise ConfigError(f"rotary scaling is missing key {k!r}")
            self.freq = stretched_frequencies(self.dims, self.base, float(self.scaling["factor"]), float(self.scaling["original"]),
                                              float(self.scaling["low"]), float(self.scaling["high"]))
            self.magnitude = 1.0
        elif self.scaling:
            for k in ("factor", "original", "fast", "slow"):
                if k not in self.scaling:
                    raise ConfigError(f"rotary scaling is missing key {k!r}")
            self.freq, self.magnitude = yarn_frequencies(self.dims, self.base, float(self.scaling["factor"]),
                                                         self.scaling["original"], float(self.scaling["fast"]),
                                                         float(self.scaling["slow"]))
        else:
            if self.dims <= 0 or self.dims % 2:
                raise ConfigError(f"rotary: dims {self.dims} must be positive and even")
            i = torch.arange(self.dims // 2, dtype=torch.float64)
            self.freq = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / self.dims).to(torch.float32)
            self.magnitude = 1.0
        self._on_device = None

    def bind(self, rt):
        super().bind(rt)
        self._on_device = RotaryFrequencies(self.freq.to(rt.device).contiguous(), float(self.magnitude), self.dims,
                                            self.interleaved)

    def frequencies(self) -> RotaryFrequencies:
        return self._on_device
