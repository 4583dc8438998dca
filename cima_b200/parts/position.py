"""Position encodings of a mixer's queries and keys.

``rope``: half-split rotary over the first ``rotary_dim`` dimensions of a head with
inv_freq[i] = theta^(-2i / rotary_dim) (src/kernels.cu:397-414; the reference computes the power in
float32 on the device, here the table is made once in float64 and rounded to float32; the angle,
sine and cosine are float32 on the device).  With ``params["scaling"]`` = {factor, low, high, original} the
frequencies are rescaled by their wavelength l = 2 pi / f: kept where l < original / high, divided by ``factor`` where
l > original / low, and between the two blended, (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
With ``params["linear"]`` = c every frequency is divided by c (positions compressed by c).
``none``: nothing rotates.
A position part offers ``inv_freq`` (float32 [rotary_dim / 2]) and ``rotary_dim``; the attention
mixer hands both to the kernel that rotates and appends.
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
        self.inv_freq = inv.to(torch.float32).to(rt.device).contiguous()


def rescale_by_wavelength(inv: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Frequencies (float64) rescaled as described at the top of this file."""
    if factor <= 0 or high <= low or original <= 0:
        raise ValueError(f"rope scaling: factor {factor} and original {original} must be positive and high {high} above low {low}")
    wave = 2.0 * math.pi / inv
    s = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
    blended = (1.0 - s) * inv / factor + s * inv
    return torch.where(wave < original / high, inv, torch.where(wave > original / low, inv / factor, blended))


class NoPosition:
    def __init__(self, spec, rt):
        self.spec = spec
        self.rotary_dim = 0
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=rt.device)


register_position("rope", Rope)
register_position("none", NoPosition)
