"""``hbq_gemm`` for torch tensors: C = A @ B with one of the reference's accumulation models
(blockquant_ext_src/gemm.cu)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from .quantizer import _ptr, _stream_ptr


def gemm(a: torch.Tensor, b: torch.Tensor, mode: int, group_k: int = 0, group_n: int = 0,
         bias: Optional[torch.Tensor] = None, b_is_nk: bool = False, force_simt: bool = False,
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hbq_gemm``: a [M, K] fp16, b [K, N] (or [N, K] when ``b_is_nk``) fp16 -> [M, N] fp16.
    ``out``: write into this contiguous fp16 [M, N] tensor instead of a new one."""
    if a.dtype != torch.float16 or b.dtype != torch.float16:
        raise RuntimeError("A must be fp16" if a.dtype != torch.float16 else "B must be fp16")
    if a.dim() != 2 or b.dim() != 2:
        raise RuntimeError("A and B must be 2D")
    if not (a.is_cuda and b.is_cuda):
        raise RuntimeError("A and B must be CUDA tensors")
    if a.device != b.device:
        raise RuntimeError("A and B must be on the same CUDA device")
    M, K = a.shape
    N = b.shape[0] if b_is_nk else b.shape[1]
    if (b.shape[1] if b_is_nk else b.shape[0]) != K:
        raise RuntimeError("A's K dimension must match B's K dimension")
    a = a.contiguous()
    b = b.contiguous()
    if bias is not None:
        bias = bias.to(device=a.device, dtype=torch.float16).contiguous()
    if out is None:
        c = torch.empty((M, N), dtype=torch.float16, device=a.device)
    else:
        if (out.dtype != torch.float16 or tuple(out.shape) != (M, N) or out.device != a.device
                or not out.is_contiguous()):
            raise RuntimeError("out must be a contiguous fp16 [M, N] tensor on A's device")
        c = out
    L = _lib.lib()
    with _lib.device_guard(a.device):
        stream = _stream_ptr(a.device)
        if force_simt:
            rc = L.hbq_gemm_simt(_ptr(a), _ptr(b), _ptr(c), M, N, K, int(b_is_nk), mode, group_k, group_n,
                                 _ptr(bias), stream)
        else:
            # scratch: the transposed operand of the [K,N] layout, and the partial sums of decode-sized fp32 products
            # that run as equal runs of K blocks per SM
            ws_bytes = int(L.hbq_gemm_workspace_bytes(M, N, K, int(b_is_nk), mode, group_k, group_n))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device) if ws_bytes else None
            rc = L.hbq_gemm(_ptr(a), _ptr(b), _ptr(c), M, N, K, int(b_is_nk), mode, group_k, group_n,
                            _ptr(bias), _ptr(ws), ws_bytes, stream)
    _lib.check(rc, "hbq_gemm")
    return c


def gemm_status() -> int:
    """Device status word of the tensor-core kernel (0 = ok); synchronises the device."""
    v = ctypes.c_int(0)
    _lib.check(_lib.lib().hbq_gemm_status(ctypes.byref(v)), "hbq_gemm_status")
    return v.value


def gemm_status_reset() -> None:
    """Clear the status word (``hbq_gemm_status_reset``)."""
    _lib.check(_lib.lib().hbq_gemm_status_reset(), "hbq_gemm_status_reset")


def gemm_wait_selftest(a: torch.Tensor, w: torch.Tensor, mode: int, group_k: int = 0, group_n: int = 0,
                       poll_limit: int = 4096) -> torch.Tensor:
    """``hbq_gemm_wait_selftest``: run the tensor-core kernel on ``a`` [M, K] and ``w`` [N, K] with its loader
    switched off and every wait bounded by ``poll_limit`` polls.  The kernel returns with nothing computed
    and ``gemm_status()`` becomes non-zero until ``gemm_status_reset()``.  Returns the (undefined) output."""
    M, K = a.shape
    N = w.shape[0]
    c = torch.empty((M, N), dtype=torch.float16, device=a.device)
    with _lib.device_guard(a.device):
        rc = _lib.lib().hbq_gemm_wait_selftest(_ptr(a), _ptr(w), _ptr(c), M, N, K, mode, group_k, group_n,
                                               int(poll_limit), _stream_ptr(a.device))
    _lib.check(rc, "hbq_gemm_wait_selftest")
    return c


def gemm_reserve_sms(n: int) -> int:
    """``hbq_gemm_reserve_sms``: later tensor-core GEMM launches leave ``n`` SMs free for a kernel of
    another stream (a collective running under the GEMM); returns the previous value."""
    return int(_lib.lib().hbq_gemm_reserve_sms(int(n)))
