"""Row-wise producers fused into the activation quantizer (``hbq_rmsnorm_quantize``, ``hbq_softmax_quantize``).

The patched decoder layers of the reference quantise two tensors that exist only to be quantised and whose
producer needs a whole-row reduction: the RMS-normalised hidden state that feeds q/k/v_proj and gate/up_proj
(``_QBaseLinear.forward``: ``self.aq(x)``, src/module.py:45, with ``x`` the output of the layer norm) and the
attention probabilities (``attn_wgt_quantizer.q(softmax(...))``, src/module.py:108-115).  Each function here
gives that quantised tensor in one kernel; for quantizer formats outside the fused kernel the producer runs
alone in the same kernel and the plain quantizer follows.  ``fused_last`` tells which path ran.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from .quantizer import _CudaBlockQuantizer, _ptr, _stream_ptr

fused_last = False


def _fusable(quantizer) -> bool:
    return (isinstance(quantizer, _CudaBlockQuantizer) and quantizer.out_dtype in (None, torch.float16)
            and not getattr(quantizer, "keep_l2_scale", False))


def rmsnorm_quantize(x: torch.Tensor, weight: torch.Tensor, eps: float, quantizer=None,
                     residual: Optional[torch.Tensor] = None, inplace: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(quantizer(weight * rmsnorm(x + residual)), x + residual)`` for fp16 ``x`` ``[..., K]``.

    ``quantizer=None`` (or the identity ``_QBase``) returns the normalised tensor itself.  With ``residual`` the
    sum is written into ``x`` when ``inplace`` (the decoder layer's ``hidden_states = residual + branch``), else
    into a new tensor.  Rounding points are those of transformers' ``LlamaRMSNorm`` on an fp16 tensor."""
    global fused_last
    if not x.is_cuda:
        raise _lib.HbqError("rmsnorm_quantize needs CUDA tensors (there is no CPU fallback)")
    if x.dtype != torch.float16 or weight.dtype != torch.float16:
        raise NotImplementedError("rmsnorm_quantize is an fp16 path (the reference's models are fp16)")
    K = x.shape[-1]
    xc = x if x.is_contiguous() else x.contiguous()
    rows = xc.numel() // K if K else 0
    res = None
    x_out = xc
    if residual is not None:
        res = residual if residual.is_contiguous() else residual.contiguous()
        if res.shape != xc.shape or res.dtype != torch.float16:
            raise ValueError("residual must have x's shape and dtype")
        x_out = xc if inplace else torch.empty_like(xc)
    out = torch.empty_like(xc)
    L = _lib.lib()
    want_q = quantizer is not None and isinstance(quantizer, _CudaBlockQuantizer)
    fmt = quantizer._format() if (want_q and _fusable(quantizer)) else None

    def run(f):
        with _lib.device_guard(xc.device):
            return L.hbq_rmsnorm_quantize(_ptr(xc), _ptr(res), _ptr(weight), ctypes.c_float(eps), rows, K,
                                          ctypes.byref(f) if f is not None else None, _ptr(x_out), _ptr(out),
                                          _stream_ptr(xc.device))
    rc = run(fmt)
    fused_last = fmt is not None and rc == 0
    if fmt is not None and rc == _lib.ERR_UNSUPPORTED:
        # the sum (if any) has not been written yet: the refusal comes before any launch
        rc = run(None)
        fmt = None
    if rc in (_lib.ERR_UNSUPPORTED, _lib.ERR_ALIGN):
        # a row length the kernel does not take (not a multiple of 8) or unaligned views: the reference's ops
        xs = xc if res is None else xc + res
        if res is not None and inplace:
            xc.copy_(xs)
            xs = xc
        xf = xs.float()
        out = weight * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(torch.float16)
        x_out, rc = xs, 0
    _lib.check(rc, "hbq_rmsnorm_quantize")
    if fmt is None and quantizer is not None:
        out = quantizer(out)
    return out, x_out


def softmax_quantize(scores: torch.Tensor, scale: float, quantizer=None, causal: bool = False, q_len: Optional[int] = None,
                     heads: Optional[int] = None, mask: Optional[torch.Tensor] = None, inplace: bool = True) -> torch.Tensor:
    """``quantizer(softmax(scores * scale + bias, dim=-1))`` for raw fp16 scores ``[..., L, S]``.

    ``bias`` is the causal mask of ``manual_sdpa`` (key j masked for query i when ``j > i + S - L``) and / or an
    additive fp16 ``mask`` ``[B or 1, 1, L, S]``.  ``q_len`` (= L) and ``heads`` (query rows per batch entry / L)
    default to the tensor's own ``[B, H, L, S]`` shape; pass them when the head axis has been folded into the
    rows.  The probabilities overwrite ``scores`` when ``inplace``."""
    global fused_last
    if not scores.is_cuda:
        raise _lib.HbqError("softmax_quantize needs a CUDA tensor (there is no CPU fallback)")
    if scores.dtype != torch.float16:
        raise NotImplementedError("softmax_quantize is an fp16 path (the reference's models are fp16)")
    S = scores.shape[-1]
    sc = scores if scores.is_contiguous() else scores.contiguous()
    Lq = q_len if q_len is not None else sc.shape[-2]
    rows = sc.numel() // S if S else 0
    if heads is None:
        heads = sc.shape[-3] if sc.dim() >= 3 else 1
    mb = 0
    mk = None
    if mask is not None:
        if mask.dtype != torch.float16 or mask.shape[-1] != S or mask.shape[-2] != Lq:
            raise ValueError("mask must be fp16 [B or 1, 1, L, S]")
        mk = mask.contiguous()
        mb = mk.numel() // (Lq * S)
    out = sc if inplace else torch.empty_like(sc)
    L = _lib.lib()
    want_q = quantizer is not None and isinstance(quantizer, _CudaBlockQuantizer)
    fmt = quantizer._format() if (want_q and _fusable(quantizer)) else None

    def run(f):
        with _lib.device_guard(sc.device):
            return L.hbq_softmax_quantize(_ptr(sc), rows, S, Lq, heads, ctypes.c_float(scale), int(causal), _ptr(mk), mb,
                                          ctypes.byref(f) if f is not None else None, _ptr(out), _stream_ptr(sc.device))
    rc = run(fmt)
    fused_last = fmt is not None and rc == 0
    if fmt is not None and rc == _lib.ERR_UNSUPPORTED:
        rc = run(None)
        fmt = None
    if rc in (_lib.ERR_UNSUPPORTED, _lib.ERR_ALIGN):
        # a key count the kernel does not take (not a multiple of 8) or unaligned views: the reference's ops
        w = sc * scale
        if causal:
            i = torch.arange(Lq, device=sc.device)[:, None] + (S - Lq)
            w = w + torch.zeros((Lq, S), dtype=sc.dtype, device=sc.device).masked_fill_(
                torch.arange(S, device=sc.device)[None, :] > i, float("-inf"))
        if mk is not None:
            w = w + mk.view(mb, 1, Lq, S) if sc.dim() == 4 else w + mk.view(-1, Lq, S)
        out, rc = torch.softmax(w, dim=-1), 0
    _lib.check(rc, "hbq_softmax_quantize")
    if fmt is None and quantizer is not None:
        out = quantizer(out)
    return out
