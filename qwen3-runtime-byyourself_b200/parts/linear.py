"""y = x . W^T for weights stored [out, in], the one matrix product of the model.

32-bit operands go to the library's own fmaf kernel (true 32-bit, fixed summation
order).  bfloat16 operands go to the library's own tensor-core kernels: to its
weight-streaming kernel for the few rows of a decode step and to its TMA + tcgen05
kernels beyond (weights first with K split over a cluster up to 128 rows, tokens first
and persistent for prompts); widths that are no multiple of 8 go to a CUDA-core kernel
with 32-bit accumulation.  No product goes to a library, where the reference's engine
calls cublasGemmEx for every projection (src/ops/linear.cpp:165-193: bfloat16 in, 32-bit
accumulate).  Another kernel can be registered for a shape (`set_bf16_kernel`).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..csrc import ops

_bf16_kernel: Optional[Callable] = None
skinny_rows = 8      # up to this many rows the weight-streaming kernel runs
prompt_rows = 129    # from this many rows on the persistent tokens-first kernel runs; in between, weights first


def set_bf16_kernel(fn: Optional[Callable]) -> None:
    """`fn(x, w, out) -> bool` may take a bfloat16 product; False hands it to the library."""
    global _bf16_kernel
    _bf16_kernel = fn


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T; out is float32 or x's type."""
    if x.dtype == torch.float32:
        if out.dtype != torch.float32:
            raise ops.KernelError("a 32-bit product writes 32-bit output")
        return ops.gemm_f32(x, w, out)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ops.KernelError(f"linear: unsupported operand types {x.dtype}, {w.dtype}")
    if not x.is_cuda:
        raise ops.KernelError("linear: CUDA tensors only")
    if _bf16_kernel is not None and _bf16_kernel(x, w, out):
        return out
    if x.shape[0] <= skinny_rows and ops.gemm_skinny_fits(x.shape[0], x.shape[1]):
        return ops.gemm_skinny(x, w, out)
    if x.shape[1] % 8 == 0:
        if x.shape[0] >= prompt_rows:
            return ops.gemm_tcgen05_prompt(x, w, out)
        return ops.gemm_tcgen05_mid(x, w, out)
    return ops.gemm_bf16_any_width(x, w, out)
