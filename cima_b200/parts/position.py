"""Position encodings of a mixer's queries and keys.

``rope``: half-split rotary over the first ``rotary_dim`` dimensions of a head with
inv_freq[i] = theta^(-2i / rotary_dim) (src/kernels.cu:397-414; the reference computes the power in
float32 on the device, here the table is made once in float64 and rounded to float32; the angle,
sine and cosine are float32 on the device).  With ``params["scaling"]`` = {factor, low, high, original} the
frequencies are rescaled by their wavelength l = 2 pi / f: kept where l < original / high, divided by ``factor`` where
l > original / low, and between the two blended, (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
With ``params["linear"]`` = c every frequency is divided by c (positions compressed by c).
With ``params["yarn"]`` = {factor c, original L, fast, slow} the frequencies are blended by their index: with
d(z) = rotary_dim ln(L / (2 pi z)) / (2 ln theta), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary_dim - 1) and
g_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i <- g_i f_i / c + (1 - g_i) f_i; and sine and cosine are multiplied
by ``amplitude`` = 0.1 ln(c) + 1 (1 without "yarn"), which the rotating kernels take beside the table.
``params["interleaved"]``: the pairs are neighbours (2i, 2i + 1) instead of (i, i + rotary_dim / 2).  A score q . k does
not change when q and k are permuted alike, so a mixer whose kernels rotate half-split pairs permutes the rows of its
query and key projections at load (``to_half_split``); kernels that take the layout as a flag are given ``interleaved``.
``none``: nothing rotates.
A position part offers ``inv_freq`` (float32 [rotary_dim / 2]), ``rotary_dim``, ``amplitude`` and ``interleaved``; the
attention mixer hands them to the kernel that rotates and appends.
"""
from __future__ import annotations

import math

import torch

from .registry import register_position


class Rope:
    def __init__(self, spec, rt):
        if spec.rotary_dim % 2 or not (0 <= spec.rotary_dim <= spec.head_dim):
            raise ValueError(f"rope: rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        i = torch.arange(spec.rotary_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / max(spec.rotary_dim, 1))
        scaling = spec.params.get("scaling") if spec.params else None
        if scaling:
            inv = rescale_by_wavelength(inv, float(scaling["factor"]), float(scaling["low"]), float(scaling["high"]),
                                        float(scaling["original"]))
        linear = spec.params.get("linear") if spec.params else None
        if linear is not None:
            if float(linear) <= 0:
                raise ValueError(f"rope: the linear factor {linear} must be positive")
            inv = inv / float(linear)
        self.amplitude = 1.0
        yarn = spec.params.get("yarn") if spec.params else None
        if yarn:
            inv, self.amplitude = rescale_by_index(inv, float(spec.theta), float(yarn["factor"]), float(yarn["original"]),
                                                   float(yarn["fast"]), float(yarn["slow"]))
        self.interleaved = bool(spec.params.get("interleaved", False)) if spec.params else False
        self.inv_freq = inv.to(torch.float32).to(rt.device).contiguous()

    def to_half_split(self, heads: int, head_dim: int) -> torch.Tensor:
        """Row order that turns a projection whose heads rotate neighbouring pairs into one whose heads rotate the pairs
        (i, i + rotary_dim / 2): new row h * head_dim + j is old row h * head_dim + order[j].  The identity where the
        layout is half-split already."""
        r = self.rotary_dim
        one = list(range(head_dim))
        if self.interleaved:
            one = list(range(0, r, 2)) + list(range(1, r, 2)) + list(range(r, head_dim))
        return torch.tensor([h * head_dim + j for h in range(heads) for j in one], dtype=torch.long)


def rescale_by_wavelength(inv: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Frequencies (float64) rescaled as described at the top of this file."""
    if factor <= 0 or high <= low or original <= 0:
        raise ValueError(f"rope scaling: factor {factor} and original {original} must be positive and high {high} above low {low}")
    wave = 2.0 * math.pi / inv
    s = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
    blended = (1.0 - s) * inv / factor + s * inv
    return torch.where(wave < original / high, inv, torch.where(wave > original / low, inv / factor, blended))


def rescale_by_index(inv: torch.Tensor, theta: float, factor: float, original: float, fast: float, slow: float):
    """(frequencies (float64) blended by their index as described at the top of this file, the factor of sine and cosine)."""
    if factor <= 0 or original <= 0 or fast <= 0 or slow <= 0 or theta <= 1:
        raise ValueError(f"rope yarn: factor {factor}, original {original}, fast {fast} and slow {slow} must be positive, theta {theta} above 1")
    r = 2 * inv.numel()

    def index_of(turns: float) -> float:
        return r * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), r - 1)
    g = ((torch.arange(inv.numel(), dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return g * inv / factor + (1.0 - g) * inv, 0.1 * math.log(factor) + 1.0


class NoPosition:
    amplitude, interleaved = 1.0, False

    def to_half_split(self, heads: int, head_dim: int) -> torch.Tensor:
        return torch.arange(heads * head_dim, dtype=torch.long)

    def __init__(self, spec, rt):
        self.spec = spec
        self.rotary_dim = 0
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=rt.device)


register_position("rope", Rope)
register_position("none", NoPosition)
