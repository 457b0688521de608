"""The linear layer that mixers and feed-forwards share: y = act(x @ W.T + b).

float32 models run the library's own true-float32 kernel (CUDA-core FMAs, bias and activation
in its epilogue). bfloat16 models use the library matrix product that the reference's engine
uses too (cuBLAS; ``FalconLinear``, src/transformers/models/falcon/modeling_falcon.py:67-72,
multiplies and then adds the bias as a separate step) followed by one hand-written kernel for
bias and activation, computed in float32.
"""
from __future__ import annotations

from typing import Optional

import torch


def linear(kernels, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: str = "none") -> torch.Tensor:
    if weight.dtype == torch.float32:
        return kernels.linear_f32(x, weight, bias, act)
    y = kernels.matmul_nt(x, weight)
    if bias is not None or act != "none":
        kernels.bias_act_(y, bias, act)
    return y
