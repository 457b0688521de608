"""The linear layer that mixers and feed-forwards share: y = act(x @ W.T + b) [+ add].

float32 models run the library's own true-float32 kernel (CUDA-core FMAs, bias and activation
in its epilogue). bfloat16 models with a few rows (decode steps) run the hand-written
weight-streaming kernel, which also takes the bias, the activation and a tensor to add (a
residual) in its float32 epilogue. bfloat16 models with many rows (prompts) use the library
matrix product that the reference's engine uses too (cuBLAS; ``FalconLinear``,
src/transformers/models/falcon/modeling_falcon.py:67-72, multiplies and then adds the bias as a
separate step); a tensor to add goes into that product's own float32 epilogue, and bias and
activation, where a layer has them, are a hand-written kernel after it, in float32.
"""
from __future__ import annotations

from typing import Optional

import torch


# Rows up to which steps of more than a few tokens use tc_linear (TMA ring, tcgen05, accumulators
# in tensor memory, bias / activation / residual in its epilogue) instead of the library product.
# Off: on matrices of 40 to 170 MB it is 10 to 30 % behind the library product (`bench.py --only linear`
# times both), and the fused epilogue does not make up for it.
TC_LINEAR_ROWS = None


def linear(kernels, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: str = "none", add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x @ weight.T + bias) + add, in the model dtype; ``add`` has the result's shape."""
    if weight.dtype == torch.float32:
        y = kernels.linear_f32(x, weight, bias, act)
        return y if add is None else kernels.residual(add, y)
    rows, k = x.shape
    if kernels.skinny_linear_preferred(rows, k, weight.shape[0]):
        return kernels.skinny_linear(x, weight, bias, act, add)
    if TC_LINEAR_ROWS is not None and rows <= TC_LINEAR_ROWS and kernels.tc_linear_takes(rows, k):
        return kernels.tc_linear(x, weight, bias, act, add)
    if bias is None and act == "none":
        return kernels.matmul_nt(x, weight, add=add)   # the sum with `add` in the product's own epilogue
    y = kernels.matmul_nt(x, weight)
    kernels.bias_act_(y, bias, act)
    return y if add is None else kernels.residual(add, y)
