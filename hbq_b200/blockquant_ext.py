"""Drop-in for the reference's ``blockquant_ext`` extension module
(blockquant_ext_src/blockquant_ext.cpp:51-72): the same five functions, fp16 CUDA tensors
A [M, K] and B [K, N] in, a new fp16 [M, N] tensor out, ``RuntimeError`` on bad inputs.
Unlike the reference the kernels run on the current torch stream, not the legacy default one.
Every function also takes ``b_is_nk=True`` to pass B as W [N, K] (how ``nn.Linear`` stores it),
which skips the transpose the reference's caller has to make (src/ops.py:41), ``out=`` to write
into an existing fp16 [M, N] tensor, and ``bias=`` (fp16 [N]) to add the layer's bias in the kernel's
store (one fp16 add per output, the same rounding as the reference's separate ``out + bias``,
src/ops.py:59-60).

    import hbq_b200.blockquant_ext as blockquant_ext
"""
from __future__ import annotations

import torch

from . import _lib
from .gemm import gemm as _gemm


def gemm_fp32_accum(A: torch.Tensor, B: torch.Tensor, *, b_is_nk: bool = False, out=None, bias=None) -> torch.Tensor:
    """GEMM with fp32 accumulator (inputs fp16)."""
    return _gemm(A, B, _lib.ACC_FP32, b_is_nk=b_is_nk, out=out, bias=bias)


def gemm_fp16_accum(A: torch.Tensor, B: torch.Tensor, *, b_is_nk: bool = False, out=None, bias=None) -> torch.Tensor:
    """GEMM with fp16 accumulator (inputs fp16)."""
    return _gemm(A, B, _lib.ACC_FP16, b_is_nk=b_is_nk, out=out, bias=bias)


def gemm_fp16_grouped_accum(A: torch.Tensor, B: torch.Tensor, group_k: int, *, b_is_nk: bool = False, out=None,
                            bias=None) -> torch.Tensor:
    """GEMM with grouped FP32-within, FP16-across accumulate (inputs fp16)."""
    if group_k not in (16, 32, 64, 128):
        raise RuntimeError("group_k must be one of {16,32,64,128}")
    return _gemm(A, B, _lib.ACC_GROUPED, group_k, b_is_nk=b_is_nk, out=out, bias=bias)


def _check_blockquant(A, B, group_k, group_n, b_is_nk):
    if group_k not in (64, 128, 256):
        raise RuntimeError("group_k must be one of {64,128,256}")
    if group_n not in (4, 8, 16, 32):
        raise RuntimeError("group_n must be one of {4,8,16,32}")
    if A.dim() == 2 and B.dim() == 2:
        if A.shape[1] % group_k != 0:
            raise RuntimeError("K must be divisible by group_k")
        if B.shape[0 if b_is_nk else 1] % group_n != 0:
            raise RuntimeError("N must be divisible by group_n")


def gemm_blockquant_mxfp8(A: torch.Tensor, B: torch.Tensor, group_k: int, group_n: int, *,
                          b_is_nk: bool = False, out=None, bias=None) -> torch.Tensor:
    """GEMM with block-quantized FP8 (E3M4) MX style within K-groups (inputs fp16, output fp16)."""
    _check_blockquant(A, B, group_k, group_n, b_is_nk)
    return _gemm(A, B, _lib.ACC_PSUM_E3M4, group_k, group_n, b_is_nk=b_is_nk, out=out, bias=bias)


def gemm_blockquant_mxint8(A: torch.Tensor, B: torch.Tensor, group_k: int, group_n: int, *,
                           b_is_nk: bool = False, out=None, bias=None) -> torch.Tensor:
    """GEMM with block-quantized INT8 (power-of-two scaled) within K-groups (inputs fp16, output fp16)."""
    _check_blockquant(A, B, group_k, group_n, b_is_nk)
    return _gemm(A, B, _lib.ACC_PSUM_INT8, group_k, group_n, b_is_nk=b_is_nk, out=out, bias=bias)
