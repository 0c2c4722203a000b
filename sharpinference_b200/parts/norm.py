"""Norm parts: RMSNorm with a weight, the weightless L2 norm used on q and k per head, the element-wise
squashing norm (``DynamicTanh``) and the layer norm with weight and bias (``LayerNorm``).

RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w`` (src/SharpInference.Cpu/SimdKernels.cs:4209-4246);
the weightless form drops ``w`` (src/SharpInference.Cpu/SimdKernels.cs:4252-4283).  The sum of
squares, the rsqrt and the scaling are float32.  Models that store the weight around zero and scale by
``1 + w`` pass ``unit_offset=True``: the sum is formed once, in float32, when the part is built.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Norm, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, weight: torch.Tensor, eps: float, unit_offset: bool = False):
        self.weight = (weight.to(torch.float32) + 1.0) if unit_offset else weight
        self.eps = float(eps)
        self.unit_offset = bool(unit_offset)

    def apply(self, x, delta, *, rows=None, out_dtype=torch.bfloat16, want_fp32=False):
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, out_dtype, rows=rows, want_fp32=want_fp32)


@register_part("norm", "l2")
class L2Norm(Norm):
    """``x * rsqrt(mean(x^2) + eps)`` over the last axis, no weight.  As the q/k norm after a rotary encoding
    the attention mixer runs it fused with the rotation and the cache write (``fuses_into_rotation``); anywhere
    else it is a launch of its own like every norm."""

    fuses_into_rotation = True

    def __init__(self, eps: float):
        self.eps = float(eps)

    def apply(self, x, delta, *, rows=None, out_dtype=torch.bfloat16, want_fp32=False):
        return ops.add_rmsnorm(x, delta, None, self.eps, out_dtype, rows=rows, want_fp32=want_fp32)


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Norm):
    """``tanh(alpha x) w + b`` element by element, with one learned scalar ``alpha``: a norm that forms no mean and no
    variance, so a row's element depends on that element alone.  Float32; the residual add is fused as in the others."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor):
        self.weight, self.bias = weight, bias
        self.alpha = alpha.reshape(1).to(torch.float32).contiguous()      # read on the device: nothing to bake into a graph

    def apply(self, x, delta, *, rows=None, out_dtype=torch.bfloat16, want_fp32=False):
        return ops.add_dyt(x, delta, self.weight, self.bias, self.alpha, out_dtype, rows=rows, want_fp32=want_fp32)


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w + b`` over the last axis, ``var`` the mean of the squared deviations from the
    mean (formed in a second pass, so nothing cancels).  Float32; the residual add is fused as in the others."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float):
        self.weight, self.bias, self.eps = weight, bias, float(eps)

    def apply(self, x, delta, *, rows=None, out_dtype=torch.bfloat16, want_fp32=False):
        return ops.add_layernorm(x, delta, self.weight, self.bias, self.eps, out_dtype, rows=rows, want_fp32=want_fp32)
