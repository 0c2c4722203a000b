"""Position encodings.

``RotaryEncoding`` rotates pairs of a head's elements by ``position * inv_freq[j]``.  Llama 4
pairs neighbours, ``(2j, 2j+1)`` (src/SharpInference.Cpu/SimdKernels.cs:4591-4629; the
architecture is absent from the reference's list of half-split models,
src/SharpInference.Core/ModelGraph.cs:308-328).  The frequencies are
``theta^(-2j/d)`` (src/SharpInference.Cpu/SimdKernels.cs:4789-4811), optionally rescaled by the
"llama3" rule, which the reference only knows as a stored table of divisors
(src/SharpInference.Engine/ForwardPass.cs:259-276):

    wavelength = 2 pi / f
    wavelength < L / high_freq_factor  ->  f                      (short waves stay)
    wavelength > L / low_freq_factor   ->  f / factor             (long waves are stretched)
    otherwise                           ->  (1 - s) f / factor + s f,
                                            s = (L / wavelength - low) / (high - low)

with ``L = original_max_position_embeddings``.  The table is float32 and built once; the angle
``position * inv_freq`` and its sine and cosine are float32 in the kernel.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .base import PositionEncoding, register_part


def rotary_inv_freq(head_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """float32 ``[head_dim / 2]`` rotation frequencies (CPU tensor).

    The unscaled frequency is the reference's ``1 / pow(theta, 2 j / d)`` in float32
    (src/SharpInference.Cpu/SimdKernels.cs:4795); the rescaling follows the three cases of the
    module docstring, one frequency at a time.
    """
    pairs = head_dim // 2
    two_j_over_d = torch.arange(pairs, dtype=torch.float32) * 2.0 / float(head_dim)
    freqs = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), two_j_over_d)
    if scaling is None:
        return freqs
    span = float(scaling.original_max_position_embeddings)
    low, high, factor = float(scaling.low_freq_factor), float(scaling.high_freq_factor), float(scaling.factor)
    out = torch.empty_like(freqs)
    for j in range(pairs):
        f = freqs[j]                                   # float32 scalar tensor: the arithmetic stays float32
        turns = span * f / (2.0 * math.pi)             # L / wavelength
        if turns > high:                               # wavelength < L / high: short waves stay
            out[j] = f
        elif turns < low:                              # wavelength > L / low: long waves are stretched
            out[j] = f / factor
        elif high == low:                              # the band between them is empty
            out[j] = f
        else:
            s = (turns - low) / (high - low)
            out[j] = (1.0 - s) * f / factor + s * f
    return out


def partial_rotary_inv_freq(head_dim: int, rot_dims: int, base: float) -> torch.Tensor:
    """float32 ``[head_dim / 2]`` frequencies of a rotation that turns only the first ``rot_dims`` elements of a
    head: pair ``j < rot_dims / 2`` gets ``base^(-2j / rot_dims)`` (formed in float64, rounded once), the pairs
    beyond get 0, which is the rotation by no angle: those elements pass unchanged, bit for bit."""
    if rot_dims % 2 or not (0 <= rot_dims <= head_dim) or head_dim % 2:
        raise ValueError(f"rotated size {rot_dims} must be even and at most the (even) head size {head_dim}")
    out = torch.zeros(head_dim // 2, dtype=torch.float64)
    if rot_dims:
        j = torch.arange(rot_dims // 2, dtype=torch.float64)
        out[: rot_dims // 2] = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * j / float(rot_dims))
    return out.to(torch.float32)


def leading_rotary_inv_freq(rot_dims: int, base: float) -> torch.Tensor:
    """float32 ``[rot_dims / 2]``: ``base^(-2i / rot_dims)``, formed in float64 and rounded once (the table of a
    :class:`RotaryEncoding` with ``rot_dims``)."""
    if rot_dims % 2 or rot_dims < 0:
        raise ValueError(f"rotated size {rot_dims} must be even and not negative")
    i = torch.arange(rot_dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / float(max(rot_dims, 1))).to(torch.float32)


def yarn_inv_freq(rot_dims: int, base: float, factor: float, original: float, fast: float, slow: float):
    """Frequencies and amplitude of a rotation whose long waves are stretched ("YaRN"): float32 ``[rot_dims / 2]`` and
    a float.  With ``f_i = base^(-2i / rot_dims)`` and ``at(t) = rot_dims * ln(original / (2 pi t)) / (2 ln base)`` (the
    pair whose wave makes ``t`` turns over ``original`` positions):

        lo = max(floor(at(fast)), 0),  hi = min(ceil(at(slow)), rot_dims - 1)
        ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        frequency_i = f_i / factor * ramp_i + f_i * (1 - ramp_i)

    so pairs below ``lo`` keep their frequency, pairs above ``hi`` are slowed by ``factor``, and the ones between are
    blended.  Cosines and sines are multiplied by ``0.1 * ln(factor) + 1`` (the amplitude).  Formed in float64 and
    rounded once."""
    if rot_dims % 2 or rot_dims <= 0:
        raise ValueError(f"rotated size {rot_dims} must be even and positive")
    if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and base > 1):
        raise ValueError("factor, original, fast and slow must be positive and the base above 1")
    i = torch.arange(rot_dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / float(rot_dims))

    def at(turns: float) -> float:
        return rot_dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(at(fast)), 0)
    hi = min(math.ceil(at(slow)), rot_dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32), 0.1 * math.log(factor) + 1.0


@register_part("position", "rotary")
class RotaryEncoding(PositionEncoding):
    def __init__(self, inv_freq: torch.Tensor, pairing: str = "interleaved", rot_dims: Optional[int] = None,
                 amplitude: float = 1.0):
        """``rot_dims``: only the first ``rot_dims`` elements of a head are turned, paired among themselves
        (``halves``: ``(i, i + rot_dims / 2)``; ``interleaved``: ``(2i, 2i + 1)``), and ``inv_freq`` has
        ``rot_dims / 2`` entries; None: the whole head, ``inv_freq`` of half the head size.  ``amplitude``
        multiplies every cosine and sine (:func:`yarn_inv_freq`); the mixers that take it say so."""
        if pairing not in ("interleaved", "halves"):
            raise ValueError(f"rotary pairing '{pairing}' is not one of interleaved, halves")
        if rot_dims is not None and (rot_dims % 2 or inv_freq.numel() != rot_dims // 2):
            raise ValueError(f"{rot_dims} rotated elements need {rot_dims // 2} frequencies, found {inv_freq.numel()}")
        self.inv_freq = inv_freq
        self.pairing = pairing
        self.rot_dims = rot_dims
        self.amplitude = float(amplitude)

    def rotary(self) -> Optional[Tuple[torch.Tensor, str]]:
        return self.inv_freq, self.pairing


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Layers that see positions only through the causal mask."""

    def rotary(self):
        return None

    def apply(self, ctx, q, k):
        return None
