"""The linear layer that mixers and feed-forwards share: y = act(x @ W.T + b) [+ add].

float32 models run the library's own true-float32 kernel (CUDA-core FMAs, bias and activation
in its epilogue). bfloat16 models with a few rows (decode steps) run the hand-written
weight-streaming kernel, which also takes the bias, the activation and a tensor to add (a
residual) in its float32 epilogue. bfloat16 models with many rows (prompts) use the library
matrix product that the reference's engine uses too (cuBLAS; ``FalconLinear``,
src/transformers/models/falcon/modeling_falcon.py:67-72, multiplies and then adds the bias as a
separate step), followed by hand-written kernels for bias, activation and sum, in float32.
"""
from __future__ import annotations

from typing import Optional

import torch


# Output width from which decode steps use stream_linear (the TMA ring) instead of skinny_linear. Off:
# alone the ring is as fast as register loads (both meet the same per-launch ramp), but its 190 KB of
# shared memory keep the other graph branch's kernels off the SM, and the whole step gets slower.
STREAM_MIN_WIDTH = None


def linear(kernels, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: str = "none", add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x @ weight.T + bias) + add, in the model dtype; ``add`` has the result's shape."""
    if weight.dtype == torch.float32:
        y = kernels.linear_f32(x, weight, bias, act)
        return y if add is None else kernels.residual(add, y)
    rows, k = x.shape
    if (STREAM_MIN_WIDTH is not None and rows <= 8 and weight.shape[0] >= STREAM_MIN_WIDTH
            and kernels.stream_linear_takes(rows, k)):
        # wide outputs: the TMA ring keeps more bytes in flight than register loads can
        return kernels.stream_linear(x, weight, bias, act, add)
    if kernels.skinny_linear_preferred(rows, k):
        return kernels.skinny_linear(x, weight, bias, act, add)
    y = kernels.matmul_nt(x, weight)
    if bias is not None or act != "none":
        kernels.bias_act_(y, bias, act)
    return y if add is None else kernels.residual(add, y)
