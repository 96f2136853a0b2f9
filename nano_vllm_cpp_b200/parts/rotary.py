"""Rotary position encodings: split-halves (NeoX) pairing, and interleaved pairing with optional YaRN scaling."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from .registry import register_part


class RotaryNeoX(PositionEncoding):
    """Pairs ``(d, d + rotary_dim/2)`` of the first ``rotary_dim`` elements of a head are turned by
    ``float(pos) * inv_freq[d]`` with ``inv_freq[d] = float(1 / theta^(2d / rotary_dim))``, the
    power taken in double (src/model.cpp:416-419; kernel src/hip_ops.hip:431-450).  ``rotary_dim`` may be smaller
    than the head: the rest of the head passes unchanged.

    ``scaling`` = dict(factor, low, high, original) stretches the long waves (the rule of the Llama 3.1 models):
    with the wavelength ``l = 2 pi / f``, a frequency stays where ``l < original / high``, becomes ``f / factor``
    where ``l > original / low``, and in between is ``(1 - s) f / factor + s f`` with
    ``s = (original / l - low) / (high - low)``.  Computed in double, rounded once to float32."""

    def __init__(self, rotary_dim: int, theta: float, scaling: dict | None = None):
        if rotary_dim % 2 or rotary_dim < 0:
            raise ValueError("rotary_dim must be even")
        self.rotary_dim, self.theta = rotary_dim, float(theta)
        self.scaling = dict(scaling) if scaling else None
        if self.scaling:
            for key in ("factor", "low", "high", "original"):
                if key not in self.scaling:
                    raise ValueError(f"rotary scaling needs '{key}'")
            if float(self.scaling["high"]) == float(self.scaling["low"]):
                raise ValueError("rotary scaling: 'high' and 'low' must differ")
        self._inv = None

    def frequencies(self) -> list:
        half = self.rotary_dim // 2
        f = [1.0 / (self.theta ** ((2.0 * i) / self.rotary_dim)) for i in range(half)]
        if self.scaling:
            sc = self.scaling
            factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
            for i, fi in enumerate(f):
                wave = 2.0 * math.pi / fi
                if wave < orig / high:
                    continue
                if wave > orig / low:
                    f[i] = fi / factor
                else:
                    s = (orig / wave - low) / (high - low)
                    f[i] = (1.0 - s) * fi / factor + s * fi
        return f

    def load(self, fetch, ctx):
        self.ctx = ctx
        self._inv = torch.tensor(self.frequencies() or [0.0], dtype=torch.float64).to(torch.float32).to(ctx.device)

    def inv_freq(self):
        return self._inv


class RotaryInterleaved(PositionEncoding):
    """Pairs ``(2i, 2i + 1)`` of the first ``rotary_dim`` elements of a head are turned by ``float(pos) * f_i`` with
    ``f_i = theta^(-2i / rotary_dim)``; the rest of the head passes unchanged.

    ``scaling`` = dict(factor, original, fast, slow) stretches the slow pairs (YaRN): with
    ``dim(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)``, ``lo = max(floor(dim(fast)), 0)``,
    ``hi = min(ceil(dim(slow)), rotary_dim - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the
    frequency becomes ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``, and cosine and sine are multiplied by
    ``0.1 ln(factor) + 1``.  The frequencies are computed in double and rounded once to float32."""
    pairing = "interleaved"

    def __init__(self, rotary_dim: int, theta: float, scaling: dict | None = None):
        if rotary_dim % 2 or rotary_dim < 0:
            raise ValueError("rotary_dim must be even")
        self.rotary_dim, self.theta = int(rotary_dim), float(theta)
        self.scaling = dict(scaling) if scaling else None
        self.amplitude = 1.0
        if self.scaling:
            for key in ("factor", "original", "fast", "slow"):
                if key not in self.scaling:
                    raise ValueError(f"rotary scaling needs '{key}'")
            self.amplitude = 0.1 * math.log(float(self.scaling["factor"])) + 1.0
        self._inv = None

    def frequencies(self) -> list:
        dims, half = self.rotary_dim, self.rotary_dim // 2
        f = [self.theta ** (-2.0 * i / dims) for i in range(half)]
        if self.scaling:
            sc = self.scaling
            factor, orig = float(sc["factor"]), float(sc["original"])

            def at(turns):
                return dims * math.log(orig / (2.0 * math.pi * float(turns))) / (2.0 * math.log(self.theta))
            lo = max(math.floor(at(sc["fast"])), 0)
            hi = min(math.ceil(at(sc["slow"])), dims - 1)
            for i in range(half):
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        return f

    def load(self, fetch, ctx):
        self.ctx = ctx
        self._inv = torch.tensor(self.frequencies() or [0.0], dtype=torch.float64).to(torch.float32).to(ctx.device)

    def inv_freq(self):
        return self._inv


class NoPosition(PositionEncoding):
    rotary_dim = 0

    def load(self, fetch, ctx):
        self.ctx = ctx
        self._inv = torch.zeros(1, dtype=torch.float32, device=ctx.device)

    def inv_freq(self):
        return self._inv


register_part("position", "rotary_neox", RotaryNeoX)
register_part("position", "rotary_interleaved", RotaryInterleaved)
register_part("position", "none", NoPosition)
