"""y = x . W^T for weights stored [out, in], the one matrix product of the model.

32-bit operands go to the library's own fmaf kernel (true 32-bit, fixed summation
order).  bfloat16 operands go to the library's own tensor-core kernels: to its
weight-streaming kernel for the few rows of a decode step and to its TMA + tcgen05
kernels beyond (weights first with K split over a cluster for up to a few hundred rows,
tokens first and persistent on pairs of SMs for prompts); widths that are no multiple of 8 go to a CUDA-core kernel
with 32-bit accumulation.  No product goes to a library, where the reference's engine
calls cublasGemmEx for every projection (src/ops/linear.cpp:165-193: bfloat16 in, 32-bit
accumulate).  Another kernel can be registered for a shape (`set_bf16_kernel`).
"""
from __future__ import annotations

import functools
from typing import Callable, Optional

import torch

from ..csrc import ops

_bf16_kernel: Optional[Callable] = None
skinny_rows = 8      # up to this many rows the weight-streaming kernel runs


def set_bf16_kernel(fn: Optional[Callable]) -> None:
    """`fn(x, w, out) -> bool` may take a bfloat16 product; False hands it to the kernels below."""
    global _bf16_kernel
    _bf16_kernel = fn


def set_bf16_kernel_active() -> bool:
    """Whether another kernel has been registered for bfloat16 products (fused projections then stand back)."""
    return _bf16_kernel is not None


# Microseconds per 64-wide K step of a tile and per block for its start and end, measured on B200.
_STEP_US = {"pair": 0.33, "prompt128": 0.29, "weights_first": 0.40}
_BLOCK_US = {"pair": 8.0, "prompt128": 5.0}
# A tile with K split over the pairs of a cluster is not persistent: every wave pays the start of the stream and the
# meeting of the partial tiles over distributed shared memory, and the launch a little more.
_PAIR_SPLIT_WAVE_US, _PAIR_SPLIT_LAUNCH_US = 8.5, 2.5


@functools.lru_cache(maxsize=4096)
def pair_plan(M: int, N: int, K: int) -> tuple:
    """(estimated microseconds, K ranges) of the pairs-of-SMs form: the number of K ranges per tile (1 = persistent
    pairs, no split) whose waves of tiles x K steps cost least."""
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    nkb, tiles = -(-K // 64), -(-M // 256) * -(-N // 256)
    best = (-(-tiles // (sms // 2)) * nkb * _STEP_US["pair"] + _BLOCK_US["pair"], 1)
    for splits in range(2, ops.PAIR_MAX_SPLITS + 1):
        capacity = ops.gemm_tcgen05_pair_capacity(splits)
        if capacity <= 0 or splits > nkb or tiles > 65535:
            continue
        cost = (-(-tiles * splits // capacity) * (-(-nkb // splits) * _STEP_US["pair"] + _PAIR_SPLIT_WAVE_US)
                + _PAIR_SPLIT_LAUNCH_US)
        if cost < best[0]:
            best = (cost, splits)
    return best


@functools.lru_cache(maxsize=4096)
def tcgen05_form(M: int, N: int, K: int, gated: bool = False) -> str:
    """Which form of the tcgen05 product takes M rows (M > skinny_rows, K a multiple of 8): weights first
    (K split over a cluster; the only form that fills the GPU when M and N give few tiles), or tokens first
    and persistent, on single SMs with 128 x 128 tiles or on pairs of SMs with 256 x 256 tiles.  A small
    cost model: waves of blocks times K steps."""
    if M <= 128:
        return "weights_first"
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    nkb = -(-K // 64)

    def waves(blocks, slots):
        return -(-blocks // slots)

    cost = {"pair": pair_plan(M, N, K)[0]}
    if not gated:                                        # the gated epilogue exists for the 256-row tiles
        cost["prompt128"] = waves(-(-M // 128) * -(-N // 128), sms) * nkb * _STEP_US["prompt128"] + _BLOCK_US["prompt128"]
    if M <= 1024:
        splits = ops.gemm_tcgen05_mid_splits(M, N, K)
        blocks = -(-N // 128) * -(-M // 256) * splits
        cost["weights_first"] = waves(blocks, sms) * (-(-nkb // splits) * _STEP_US["weights_first"] + (10.0 if splits > 1 else 5.0))
    return min(cost, key=cost.get)


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
    M, K = x.shape
    if K % 8 != 0:
        return ops.gemm_bf16_any_width(x, w, out)
    if M <= skinny_rows:
        return ops.gemm_skinny(x, w, out)
    form = tcgen05_form(M, w.shape[0], K)
    if form == "weights_first":
        return ops.gemm_tcgen05_mid(x, w, out)
    if form == "pair":
        return ops.gemm_tcgen05_pair(x, w, out, splits=pair_plan(M, w.shape[0], K)[1])
    return ops.gemm_tcgen05_prompt(x, w, out, tile_n=128)
