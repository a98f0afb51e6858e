"""GEMM with modelled low-precision accumulation: ``FP16AccumMatMul`` (src/ops.py:16-62).

Same constructor, ``forward(x, w, bias=None)`` and validation errors as the reference.  The
reference transposes ``w`` ([N, K]) into a fresh [K, N] tensor on every call before handing it
to the extension; here ``w`` is consumed as it is stored (K-major) by the tensor-core kernel.
``forward`` additionally takes ``out=`` (a contiguous fp16 ``[rows, N]`` tensor to write into).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import blockquant_ext as ext


class FP16AccumMatMul(nn.Module):
    """FP16 accumulation matrix multiplication (src/ops.py:16-62).

    group_size: K-chunk accumulated in fp32 before the fp16 add (None: pure fp16 chain);
    quant_block_size: columns per MXINT8 partial-sum quantisation block (None: no quantisation)."""

    def __init__(self, group_size: int = None, quant_block_size: int = None):
        super().__init__()
        self.group_size = group_size
        self.quant_block_size = quant_block_size

    def forward(self, x, w, bias=None, out=None) -> torch.Tensor:
        orig_shape = x.shape
        x2d = x.reshape(-1, x.shape[-1])
        if x2d.dtype != torch.float16:
            x2d = x2d.half()
        x2d = x2d.to(w.device, non_blocking=True)
        wh = w if w.dtype == torch.float16 else w.half()

        if self.quant_block_size is not None:
            if self.group_size not in [4, 8, 16, 32, 64, 128]:
                raise ValueError(f"Invalid group size: {self.group_size}")
            if self.quant_block_size not in [4, 8, 16, 32]:
                raise ValueError(f"Invalid quant block size: {self.quant_block_size}")
            out2d = ext.gemm_blockquant_mxint8(x2d, wh, self.group_size, self.quant_block_size, b_is_nk=True, out=out,
                                               bias=bias)
        elif self.group_size is not None:
            if self.group_size not in [4, 8, 16, 32, 64, 128]:
                raise ValueError(f"Invalid group size: {self.group_size}")
            out2d = ext.gemm_fp16_grouped_accum(x2d, wh, self.group_size, b_is_nk=True, out=out, bias=bias)
        else:
            out2d = ext.gemm_fp16_accum(x2d, wh, b_is_nk=True, out=out, bias=bias)
        # the bias was added by the kernel's store (one fp16 add per output, as the reference's `out2d + bias`,
        # src/ops.py:59-60), so with `out=` the result, bias included, is in `out`
        return out2d.view(*orig_shape[:-1], -1)


class FP32AccumMatMul(nn.Module):
    """``F.linear`` with fp32 accumulation (what ``_QBaseLinear.forward`` runs when no accumulation operator is set,
    src/module.py:47-48) on the library's tensor-core kernel instead of cuBLAS, as an ``ops`` object."""

    def forward(self, x, w, bias=None, out=None) -> torch.Tensor:
        x2d = x.reshape(-1, x.shape[-1])
        if x2d.dtype != torch.float16:
            x2d = x2d.half()
        y = ext.gemm_fp32_accum(x2d, w if w.dtype == torch.float16 else w.half(), b_is_nk=True, out=out, bias=bias)
        return y.view(*x.shape[:-1], -1)
