"""Fused KV-cache writes of the quantised attention block.

``QLlamaAttention.forward`` (src/module.py:147-168) produces the cached K and V in several
passes over HBM: view + transpose, ``apply_rotary_pos_emb``, ``kv_quantizer.q`` for K, and
transpose + ``kv_quantizer.q`` + transpose for V.  ``write_k_cache`` / ``write_v_cache`` give
the same tensors in one kernel each, reading the projection output ``[B, T, H*D]`` once and
writing the cache layout ``[B, H, T, D]`` once.

When the quantizer's format is outside the fused kernels the functions run the reference's
steps one by one (torch for the rotation and the transposes, the CUDA quantizer for ``q``);
``fused_last`` tells which path ran.
"""
import ctypes
from typing import Optional

import torch

from . import _lib
from .quantizer import _CudaBlockQuantizer, _dtype_code, _ptr, _stream_ptr

fused_last = False


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """``rotate_half`` of transformers' Llama: cat(-x[..., D/2:], x[..., :D/2])."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``apply_rotary_pos_emb`` for one tensor ``[B, H, T, D]`` with cos/sin ``[B or 1, T, D]``."""
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return (x * cos) + (rotate_half(x) * sin)


def _head_dim(x: torch.Tensor, num_heads: int) -> int:
    if x.dim() == 4 and x.shape[2] == num_heads:
        return x.shape[3]
    if x.dim() == 3 and x.shape[2] % num_heads == 0:
        return x.shape[2] // num_heads
    raise ValueError(f"expected [B, T, H*D] or [B, T, H, D] with H={num_heads}; got {tuple(x.shape)}")


def _tables(cos: torch.Tensor, sin: torch.Tensor, B: int, T: int, D: int):
    if cos.shape != sin.shape or cos.shape[-1] != D or cos.shape[-2] != T:
        raise ValueError(f"cos/sin must be [B or 1, T, D]; got {tuple(cos.shape)} and {tuple(sin.shape)}")
    lead = cos.numel() // (T * D)
    if lead not in (1, B):
        raise ValueError("cos/sin batch dimension must be 1 or B")
    return cos.contiguous(), sin.contiguous(), lead * T


def write_k_cache(k: torch.Tensor, num_heads: int, quantizer: _CudaBlockQuantizer,
                  cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                  center: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RoPE + quantise along head_dim + ``[B,T,H,D] -> [B,H,T,D]`` for the k_proj (or q_proj) output.

    ``k`` is ``[B, T, H*D]`` (or ``[B, T, H, D]``); returns what the reference computes as
    ``quantizer.q(apply_rotary_pos_emb(k.view(B,T,H,D).transpose(1,2)))`` (src/module.py:147-162).
    ``center`` (``[B, H, 1, D]`` or ``[B, H, D]``, fp16) is subtracted after the rotation: the
    K-cache centring of the Qwen2 block (``kv_quantizer.q(key_states - center)``,
    src/module.py:221-244), with the centre computed by the caller at prefill."""
    global fused_last
    if not k.is_cuda:
        raise _lib.HbqError("write_k_cache needs a CUDA tensor (there is no CPU fallback)")
    B, T = k.shape[0], k.shape[1]
    D = _head_dim(k, num_heads)
    kc = k.contiguous()
    fmt = quantizer._format()
    odt = quantizer.out_dtype or kc.dtype
    out = torch.empty((B, num_heads, T, D), dtype=odt, device=kc.device)
    rope_rows = 0
    if cos is not None:
        cos, sin, rope_rows = _tables(cos, sin, B, T, D)
    if center is not None:
        if center.numel() != B * num_heads * D:
            raise ValueError(f"center must hold B*H*D = {B * num_heads * D} values; got {tuple(center.shape)}")
        center = center.reshape(B, num_heads, D).contiguous()
    fusable = (cos is None or (kc.dtype == torch.float16 and cos.dtype == torch.float16 and sin.dtype == torch.float16))
    fusable = fusable and (center is None or (kc.dtype == torch.float16 and center.dtype == torch.float16))
    rc = _lib.ERR_UNSUPPORTED
    if fusable:
        with _lib.device_guard(kc.device):
            rc = _lib.lib().hbq_kv_write_k(_ptr(kc), _dtype_code(kc), B, T, num_heads, D, _ptr(cos), _ptr(sin),
                                           rope_rows, _ptr(center), ctypes.byref(fmt), _ptr(out), _dtype_code(out),
                                           _stream_ptr(kc.device))
    if rc == _lib.ERR_UNSUPPORTED:
        fused_last = False
        x = kc.view(B, T, num_heads, D).transpose(1, 2)
        if cos is not None:
            x = apply_rope(x, cos.view(-1, T, D), sin.view(-1, T, D))
        if center is not None:
            x = x - center.view(B, num_heads, 1, D).to(x.dtype)
        return quantizer.q(x.contiguous())
    _lib.check(rc, "hbq_kv_write_k")
    fused_last = True
    return out


def write_v_cache(v: torch.Tensor, num_heads: int, quantizer: _CudaBlockQuantizer,
                  token_major: bool = False) -> torch.Tensor:
    """Quantise the v_proj output along the TOKEN axis and store it as ``[B,H,T,D]``.

    Equals the reference's transpose / ``kv_quantizer.q`` / transpose (src/module.py:163-168).
    ``token_major=True`` returns ``[B,T,H,D]`` instead (the input's layout), which is what a serving
    engine with a flattened-token cache wants (vllm/src/hbq_vllm_quant.py:322-345: one call per
    sequence span with B = 1)."""
    global fused_last
    if not v.is_cuda:
        raise _lib.HbqError("write_v_cache needs a CUDA tensor (there is no CPU fallback)")
    B, T = v.shape[0], v.shape[1]
    D = _head_dim(v, num_heads)
    vc = v.contiguous()
    fmt = quantizer._format()
    odt = quantizer.out_dtype or vc.dtype
    out = torch.empty((B, T, num_heads, D) if token_major else (B, num_heads, T, D), dtype=odt, device=vc.device)
    with _lib.device_guard(vc.device):
        rc = _lib.lib().hbq_kv_write_v(_ptr(vc), _dtype_code(vc), B, T, num_heads, D, ctypes.byref(fmt), _ptr(out),
                                       _dtype_code(out), int(token_major), _stream_ptr(vc.device))
    if rc == _lib.ERR_UNSUPPORTED:
        fused_last = False
        x = vc.view(B, T, num_heads, D).permute(0, 2, 3, 1).contiguous()          # [B,H,D,T]
        y = quantizer.q(x)
        return y.permute(0, 3, 1, 2).contiguous() if token_major else y.transpose(-1, -2).contiguous()
    _lib.check(rc, "hbq_kv_write_v")
    fused_last = True
    return out


FUSE_SWIGLU = True      # False: always run the separate ops (for A/B timing)


def swiglu_quantize(gate: torch.Tensor, up: torch.Tensor, quantizer) -> torch.Tensor:
    """``quantizer.q(silu(gate) * up)`` in one pass over the two projection outputs: the input of the
    down projection of a gated MLP (``down_proj(act_fn(gate_proj(x)) * up_proj(x))`` in the patched
    transformers blocks, with ``down_proj.aq`` as the quantizer, src/module.py:45).  Same bits as the
    three separate ops; formats outside the fused kernel (and non-fp16 inputs) run those ops."""
    global fused_last
    if not (gate.is_cuda and up.is_cuda):
        raise _lib.HbqError("swiglu_quantize needs CUDA tensors (there is no CPU fallback)")
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up must have the same shape and dtype")
    fusable = (FUSE_SWIGLU and isinstance(quantizer, _CudaBlockQuantizer) and gate.dtype == torch.float16
               and quantizer.out_dtype in (None, torch.float16) and not getattr(quantizer, "keep_l2_scale", False))
    if fusable:
        g, u = gate.contiguous(), up.contiguous()
        K = g.shape[-1]
        rows = g.numel() // K if K else 0
        out = torch.empty_like(u)
        fmt = quantizer._format()
        with _lib.device_guard(g.device):
            rc = _lib.lib().hbq_swiglu_quantize(_ptr(g), _ptr(u), rows, K, ctypes.byref(fmt), _ptr(out), _stream_ptr(g.device))
        if rc != _lib.ERR_UNSUPPORTED:
            _lib.check(rc, "hbq_swiglu_quantize")
            fused_last = True
            return out
    fused_last = False
    return quantizer(torch.nn.functional.silu(gate) * up)
