"""Position encodings.  A position part turns a step's token positions into
whatever its mixers need, once per step for all layers that share it.

``rotary_half``: rotate-half rotary positions.  For ``i`` in ``[0, d/2)``:
``f_i = theta^(-2i/d)``, ``a = pos * f_i``, and the pair ``(x_i, x_{i+d/2})``
is rotated by ``a`` (reference: runtime/backends/cuda/native/cuda_kernels.cu:70-115,
rope_type 2, selected for ``qwen2`` at
runtime/backends/cuda/native/model_loader.h:45-58).  The reference evaluates
``powf/cosf/sinf`` per element, per layer; here the cos/sin tables are made
once per step in double precision and rounded to float32.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..config.registry import register_part
from ..kernels import ops
from .base import Part


def scaled_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]):
    """The ``rotary_dim / 2`` frequencies ``f_i = theta^(-2i / rotary_dim)`` in float64 and the factor on cos and
    sin; with ``scaling`` = {factor, original, fast, slow} the frequencies are stretched where they are slow
    (the YaRN rule): with ``where(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)``, ``lo =
    max(floor(where(fast)), 0)``, ``hi = min(ceil(where(slow)), rotary_dim - 1)`` and ``ramp_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1)``, ``f_i <- f_i / factor * ramp_i + f_i * (1 - ramp_i)``, and cos and sin are
    multiplied by ``0.1 ln(factor) + 1``."""
    half = rotary_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * i / max(rotary_dim, 1))
    if not scaling:
        return freq, 1.0
    if "low" in scaling:
        return banded_frequencies(freq, scaling), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    fast, slow = float(scaling["fast"]), float(scaling["slow"])
    where = lambda t: rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(theta))
    lo = max(math.floor(where(fast)), 0)
    hi = min(math.ceil(where(slow)), rotary_dim - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def banded_frequencies(freq: torch.Tensor, scaling: dict) -> torch.Tensor:
    """Frequency scaling by wavelength bands, ``scaling`` = {factor, low, high, original}: with the wavelength
    ``l = 2 pi / f``, a frequency stays where ``l < original / high``, becomes ``f / factor`` where ``l > original /
    low``, and in between, with ``s = (original / l - low) / (high - low)``, becomes ``(1 - s) f / factor + s f``.
    cos and sin keep their size."""
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    wavelength = 2.0 * math.pi / freq
    s = (original / wavelength - low) / (high - low)
    mid = (1.0 - s) * freq / factor + s * freq
    out = torch.where(wavelength > original / low, freq / factor, mid)
    return torch.where(wavelength < original / high, freq, out)


class RotaryHalf(Part):
    """params: ``rotary_dim`` (how many leading dims of a head rotate), ``theta``, ``scaling`` (None,
    {factor, original, fast, slow}: see :func:`scaled_frequencies`, or {factor, low, high, original}: see
    :func:`banded_frequencies`).  The table it makes is one cosine and one
    sine per token and pair; how a mixer pairs the dimensions (halves or neighbours) is the mixer's business."""

    family = "position"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.rotary_dim = int(params["rotary_dim"])
        self.theta = float(params["theta"])
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ValueError(f"rotary_dim must be even and >= 0, got {self.rotary_dim}")
        half = self.rotary_dim // 2
        freq, self.magnitude = scaled_frequencies(self.rotary_dim, self.theta, params.get("scaling"))
        self.inv_freq = freq.to(device)

    def prepare(self, ctx) -> None:
        """Make ``(cos, sin)`` float32 ``[N, rotary_dim/2]`` for the step's positions."""
        half = self.rotary_dim // 2
        cos = torch.empty((ctx.n_tokens, half), dtype=torch.float32, device=ctx.device)
        sin = torch.empty((ctx.n_tokens, half), dtype=torch.float32, device=ctx.device)
        if half:
            ops.rope_table(ctx.positions, self.inv_freq, cos, sin, self.magnitude)
        return cos, sin


register_part("position", "rotary_half", RotaryHalf)
register_part("position", "rotary", RotaryHalf)
