"""Rotary position encoding.

Angles ``pos * f_i`` with ``f_i = theta^(-2i/n_rot)`` for i < n_rot/2; a pair (a, b) of each head is rotated:
``a' = a*cos - b*sin``, ``b' = a*sin + b*cos``; dimensions >= n_rot are untouched.  Pairing "half": the pair
(i, i + n_rot/2) (src/model.c:468-493; fixed by ``rope_neox`` for the reference's architecture, src/model.c:140);
pairing "interleaved": the pair (2i, 2i + 1).  The table of cos/sin is computed once in float64 and rounded to
float32, as the reference evaluates cos and sin in double (src/mathx.c:92-113).  The table is the same for both
pairings; the pairing is what the kernel that rotates does with it, so a mixer takes the pairings its kernels know.

``scaling`` stretches the table for contexts longer than the ``original`` one by ``factor``, frequency by frequency:
pairs that turn more than ``fast`` times over the original length keep their frequency, pairs that turn fewer than
``slow`` times have it divided by ``factor``, and between the two the pair index ramps linearly from one to the other;
cos and sin are both multiplied by ``0.1 ln(factor) + 1``.  A ``scaling`` with the keys ``low`` and ``high`` instead is the
form by wavelength: with l = 2 pi / f, a frequency stays where l < original / high, becomes f / factor where
l > original / low, and between the two is ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``; cos
and sin keep their size.
"""
from __future__ import annotations

import math

import torch

from ..config.base import UnsupportedError
from .base import PositionEncoding, register_part


class Rotary(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, n_rot: int, theta: float, pairing: str = "half", scaling=None, **_):
        if pairing not in ("half", "interleaved"):
            raise UnsupportedError(f"rotary pairing '{pairing}' is not supported (known: half, interleaved)")
        if n_rot % 2 or n_rot > head_dim or n_rot < 2:
            raise UnsupportedError(f"rotary width {n_rot} must be even and at most head_dim {head_dim}")
        self.head_dim, self.n_rot, self.theta, self.pairing = int(head_dim), int(n_rot), float(theta), pairing
        self.scaling = dict(scaling) if scaling else None
        self.by_wavelength = bool(self.scaling) and "low" in self.scaling and "high" in self.scaling
        if self.by_wavelength:
            for k in ("factor", "original", "low", "high"):
                if not float(self.scaling.get(k, 0)) > 0:
                    raise UnsupportedError(f"rotary scaling needs a positive '{k}'")
            if not float(self.scaling["high"]) > float(self.scaling["low"]):
                raise UnsupportedError("rotary scaling: 'high' must exceed 'low'")
        elif self.scaling:
            for k in ("factor", "original", "fast", "slow"):
                if not float(self.scaling.get(k, 0)) > 0:
                    raise UnsupportedError(f"rotary scaling needs a positive '{k}'")
        self.cos_sin = None     # float32 [positions, n_rot/2, 2]

    def frequencies(self):
        """(float64 frequency per pair, factor on cos and sin)."""
        half = self.n_rot // 2
        i = torch.arange(half, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.n_rot)
        if not self.scaling:
            return f, 1.0
        sc = self.scaling
        factor = float(sc["factor"])
        if self.by_wavelength:
            original, low, high = float(sc["original"]), float(sc["low"]), float(sc["high"])
            wave = 2.0 * math.pi / f
            s = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)        # 0 at the long end, 1 at the short end
            blended = (1.0 - s) * f / factor + s * f
            out = torch.where(wave < original / high, f, torch.where(wave > original / low, f / factor, blended))
            return out, 1.0

        def pair_turning(turns):          # the (fractional) pair index that makes ``turns`` turns over the original length
            return self.n_rot * math.log(float(sc["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
        lo = max(math.floor(pair_turning(float(sc["fast"]))), 0)
        hi = min(math.ceil(pair_turning(float(sc["slow"]))), self.n_rot - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    def prepare(self, max_positions, device):
        f, magnitude = self.frequencies()
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * f[None, :]
        table = torch.stack([ang.cos(), ang.sin()], dim=-1) * magnitude
        self.cos_sin = table.to(torch.float32).contiguous().to(device)


register_part("position", "rotary", Rotary)
