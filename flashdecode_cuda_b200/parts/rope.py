"""Rotary position encodings: tables of cos and sin per position and pair of dimensions.  Which dimensions form a
pair (j with j + d/2, or 2j with 2j + 1) is the business of the kernel that applies them."""

from __future__ import annotations

import math
from typing import Optional

import torch

from ..registry import register_part
from .base import Position, Runtime


@register_part("position", "rotary_half")
class RotaryHalf(Position):
    """cos/sin tables [positions, d/2] in float32.

    inv_freq_j = 1 / theta^(2j/d), angle[p, j] = p * inv_freq_j, both computed
    in float32 exactly as ``build_rope_cache`` of davidjoyme/flashdecode-cuda
    does (engine/ops.py:102-110); its tables repeat the d/2 angles twice, these
    keep one copy.  The table covers the configuration's
    ``max_position_embeddings`` (the reference caps at 8192,
    engine/model.py:82-91); a position beyond it sets a status bit instead of
    reading out of bounds.
    """

    # Tables longer than this many positions are built for what the first cache asks for instead of the
    # configuration's whole max_position_embeddings (8 bytes per position and pair of dims).
    FULL_TABLE_LIMIT = 1 << 18
    # ... but for at least this many, so that a configuration without a limit of its own serves later, longer caches
    MIN_TABLE = 1 << 16

    def __init__(self, head_dim: int, theta: float, max_positions: int):
        self.head_dim, self.theta, self.max_positions = head_dim, float(theta), max_positions
        self.cos = self.sin = None

    def prepare(self, n_positions: int, rt: Runtime) -> None:
        """Build the tables, once.  They are made for every position the configuration allows (or, beyond
        ``FULL_TABLE_LIMIT`` positions, for what this first cache needs) and never replaced: kernels
        captured into CUDA graphs hold their addresses and their length, so a later, longer cache must
        find the same tensors.  A cache that needs more positions than the tables have is refused."""
        n = min(n_positions, self.max_positions)
        if self.cos is not None:
            if self.cos.shape[0] < n:
                raise ValueError(f"the rotary tables were built for {self.cos.shape[0]} positions and cannot grow "
                                 f"(captured graphs hold their address); a cache of {n} positions needs a model "
                                 f"loaded anew, or a first cache at least as long")
            return
        if self.max_positions <= self.FULL_TABLE_LIMIT:
            n = self.max_positions
        else:
            n = max(n, self.MIN_TABLE)
        d = self.head_dim
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2).float() / d))
        freqs = torch.outer(torch.arange(n).float(), inv_freq)
        self.cos = freqs.cos().contiguous().to(rt.device)
        self.sin = freqs.sin().contiguous().to(rt.device)


@register_part("position", "rotary_scaled")
class RotaryScaled(Position):
    """cos/sin tables [positions, dims / 2] in float32 for the frequencies f_i = base^(-2i / dims), optionally
    stretched for contexts longer than the ``original`` one (``scaling`` = {factor, original, fast, slow}):

        pair(t) = dims ln(original / (2 pi t)) / (2 ln base)          the pair that makes t turns in `original` positions
        lo = max(floor(pair(fast)), 0);  hi = min(ceil(pair(slow)), dims - 1)
        ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        f_i <- f_i / factor * ramp_i + f_i * (1 - ramp_i);   cos, sin <- (0.1 ln(factor) + 1) * cos, sin

    so pairs that turn fast keep their frequency, slow ones are divided by ``factor``, with a linear ramp between.
    ``scaling`` = {factor, low, high, original} is the other form, by wavelength l_i = 2 pi / f_i: l_i < original / high
    keeps f_i; l_i > original / low gives f_i / factor; between them, with s = (original / l_i - low) / (high - low),
    f_i <- (1 - s) f_i / factor + s f_i; cos and sin are not rescaled.
    The tables are computed in float64 on the host and rounded once.  They grow with the first cache (there is no
    longest sequence in the configuration) and are never replaced afterwards, like those of ``rotary_half``."""

    MIN_TABLE = 1 << 16

    def __init__(self, dims: int, base: float, scaling: Optional[dict] = None, max_positions: int = 1 << 30):
        if dims <= 0 or dims % 2 or not base > 0:
            raise ValueError(f"a rotation needs an even, positive number of dimensions and a positive base, got {dims}, {base}")
        self.dims, self.base, self.max_positions = dims, float(base), max_positions
        self.scaling = dict(scaling) if scaling else None
        self.cos = self.sin = None

    def frequencies(self):
        """(frequencies [dims / 2] float64, the factor on cos and sin)."""
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        f = torch.tensor(self.base, dtype=torch.float64) ** (-2.0 * i / self.dims)
        if not self.scaling:
            return f, 1.0
        sc = self.scaling
        factor, orig = float(sc["factor"]), float(sc["original"])
        if "low" in sc:                                  # by wavelength
            low, high = float(sc["low"]), float(sc["high"])
            wavelength = 2.0 * math.pi / f
            s = ((orig / wavelength - low) / (high - low)).clamp(0.0, 1.0) if high != low else torch.ones_like(f)
            blended = (1.0 - s) * f / factor + s * f
            out = torch.where(wavelength < orig / high, f, torch.where(wavelength > orig / low, f / factor, blended))
            return out, 1.0

        def pair(turns: float) -> float:
            return self.dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
        lo = max(math.floor(pair(float(sc["fast"]))), 0)
        hi = min(math.ceil(pair(float(sc["slow"]))), self.dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    def prepare(self, n_positions: int, rt: Runtime) -> None:
        n = min(n_positions, self.max_positions)
        if self.cos is not None:
            if self.cos.shape[0] < n:
                raise ValueError(f"the rotary tables were built for {self.cos.shape[0]} positions and cannot grow "
                                 f"(captured graphs hold their address); a cache of {n} positions needs a model "
                                 f"loaded anew, or a first cache at least as long")
            return
        n = min(max(n, self.MIN_TABLE), self.max_positions)
        f, mag = self.frequencies()
        angles = torch.outer(torch.arange(n, dtype=torch.float64), f)
        self.cos = (angles.cos() * mag).float().contiguous().to(rt.device)
        self.sin = (angles.sin() * mag).float().contiguous().to(rt.device)
