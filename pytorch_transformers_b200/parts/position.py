"""Position-encoding parts. A position part never touches activations itself: it hands the
mixer the constants that the kernels need, a rotation table and/or per-head score slopes.

Rotary: ``inv_freq_i = theta^(-2i/dim)`` in float32, divided by ``factor`` for linear scaling
(src/transformers/modeling_rope_utils.py:67, 100-108); pairs ``(i, i + dim/2)`` are rotated by
``position * inv_freq_i`` (src/transformers/models/falcon/modeling_falcon.py:76-108, 155-164).
ALiBi: per-head slopes of build_alibi_tensor (modeling_falcon.py:175-188), rounded to bfloat16
because the reference forms ``slope * position`` in bfloat16 (:196-197); the kernels round the
position and the product the same way.
"""
from __future__ import annotations

import math

import torch

from .base import BuildContext, Part, PartSpec, register_part


@register_part("position", "none")
class NoPosition(Part):
    graph_safe = True
    def __init__(self, build: BuildContext, spec: PartSpec):
        super().__init__(build, spec)

    def rotation(self):
        return None

    def score_bias(self):
        return None


@register_part("position", "rotary")
class RotaryPosition(NoPosition):
    def __init__(self, build: BuildContext, spec: PartSpec, head_dim: int, theta: float, factor: float = 1.0,
                 rotary_dim: int = 0, interleaved: bool = False):
        super().__init__(build, spec)
        # which dims make a rotated pair: (i, i + dim / 2), the reference's rotate_half, or (2 i, 2 i + 1)
        self.interleaved = bool(interleaved)
        dim = int(rotary_dim) if rotary_dim else int(head_dim)
        if dim % 2 or dim > head_dim or dim <= 0:
            raise ValueError(f"rotary_dim must be even and in 2..head_dim, got {dim} for head_dim {head_dim}")
        exponent = torch.arange(0, dim, 2, dtype=torch.int64).float() / dim
        inv_freq = 1.0 / (float(theta) ** exponent)
        if factor != 1.0:
            inv_freq = inv_freq / float(factor)
        self.inv_freq = inv_freq.to(torch.float32).to(build.device)
        # layers whose rotation has the same constants share one table of angles per step
        self.rotation_key = ("rotary", dim, float(theta), float(factor))

    def rotation(self):
        return self.inv_freq


def alibi_slopes(heads: int) -> torch.Tensor:
    """float32 slopes: a geometric series for the largest power of two below ``heads``, and the
    odd powers of the next finer series for the remaining heads."""
    n = 2 ** math.floor(math.log2(heads))
    first = torch.tensor(2.0 ** (-(2.0 ** -(math.log2(n) - 3))), dtype=torch.float32)
    slopes = torch.pow(first, torch.arange(1, n + 1, dtype=torch.int32))
    if n != heads:
        finer = torch.tensor(2.0 ** (-(2.0 ** -(math.log2(2 * n) - 3))), dtype=torch.float32)
        extra = torch.arange(1, 1 + 2 * min(n, heads - n), 2, dtype=torch.int32)
        slopes = torch.cat([slopes, torch.pow(finer, extra)])
    return slopes


@register_part("position", "alibi")
class AlibiPosition(NoPosition):
    def __init__(self, build: BuildContext, spec: PartSpec, heads: int):
        super().__init__(build, spec)
        self.slopes = alibi_slopes(int(heads)).bfloat16().float().to(build.device)

    def score_bias(self):
        return self.slopes
