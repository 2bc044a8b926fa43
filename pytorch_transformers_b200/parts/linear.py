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


def linear_pending(kernels, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """A product whose result is to be added to a float32 stream by a later kernel: (the float32 sums unrounded, the
    bias that is still to be added or None when it is in already)."""
    if weight.dtype == torch.float32:
        return kernels.linear_f32(x, weight, bias, "none"), None
    return linear(kernels, x, weight, wide_out=True), bias


def linear(kernels, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: str = "none", add: Optional[torch.Tensor] = None, wide_out: bool = False) -> torch.Tensor:
    """act(x @ weight.T + bias) + add, in the model dtype; ``add`` has the result's shape. ``wide_out``: a plain
    product (no bias, activation or addend) whose float32 sums are returned unrounded (for a float32 norm or
    sum that follows)."""
    if wide_out and weight.dtype != torch.float32:
        if bias is not None or act != "none" or add is not None:
            raise ValueError("linear: wide_out is for a plain product")
        if kernels.skinny_linear_preferred(x.shape[0], x.shape[1], weight.shape[0]):
            return kernels.skinny_linear(x, weight, out_dtype=torch.float32)
        return kernels.matmul_nt(x, weight, out_dtype=torch.float32)
    if weight.dtype == torch.float32:
        y = kernels.linear_f32(x, weight, bias, act)
        return y if add is None else kernels.residual(add, y)
    if x.dtype != weight.dtype:
        raise ValueError(f"linear: input of {x.dtype} meets a matrix of {weight.dtype}")
    rows, k = x.shape
    if add is not None and add.dtype == torch.float32:
        # a float32 residual stream beside bfloat16 matrices: the product leaves its float32 accumulator
        # unrounded and the sum is formed in float32
        if bias is None and act == "none":
            if kernels.skinny_linear_preferred(rows, k, weight.shape[0]):
                y = kernels.skinny_linear(x, weight, out_dtype=torch.float32)
            else:
                y = kernels.matmul_nt(x, weight, out_dtype=torch.float32)
        elif act == "none":
            # with a bias: the float32 sums take the bias before they meet the stream, still unrounded
            y = linear(kernels, x, weight, wide_out=True)
            kernels.bias_act_(y, bias, "none")
        else:
            y = linear(kernels, x, weight, bias, act)
        return kernels.add_stream(add, y)
    if kernels.skinny_linear_preferred(rows, k, weight.shape[0]):
        return kernels.skinny_linear(x, weight, bias, act, add)
    if TC_LINEAR_ROWS is not None and rows <= TC_LINEAR_ROWS and kernels.tc_linear_takes(rows, k):
        return kernels.tc_linear(x, weight, bias, act, add)
    if bias is None and act == "none":
        return kernels.matmul_nt(x, weight, add=add)   # the sum with `add` in the product's own epilogue
    y = kernels.matmul_nt(x, weight)
    kernels.bias_act_(y, bias, act)
    return y if add is None else kernels.residual(add, y)
