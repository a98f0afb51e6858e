"""The hot path as a serving engine calls it: flattened token batches, decode-sized shapes.

The reference's second caller is its vLLM plugin (vllm/src/hbq_vllm_quant.py): a linear method that fake-quantises
the loaded weights once and the activations on every call (``HBQNVFP4LinearMethod``, :493-554), and an attention
forward patched to quantise post-RoPE Q, K and V of a flattened ``[tokens, heads * head_dim]`` batch
(:288-345, :398-454), V per sequence span along the token axis.  The functions below are those hooks on this
library's kernels, with the reference functions' names and argument meaning; they do not import the engine, so the
plugin's registration code (``register_quantization_config``, the attention-class patching) stays where it is and
only its calls into ``src.quantizer`` change.  Quantizers are passed in (the plugin builds them from its YAML with
``PTQConfig.map_act_quantizer`` / ``map_kv_quantizer``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from . import blockquant_ext as ext
from .kvcache import write_v_cache
from .quantizer import _CudaBlockQuantizer


def quantize_post_rope_q(q: torch.Tensor, num_heads: int, head_dim: int, quantizer) -> torch.Tensor:
    """``_quantize_post_rope_q`` (:288-294): the activation quantizer along head_dim of ``[tokens, H * D]``."""
    return quantizer.q(q.reshape(-1, num_heads, head_dim)).reshape(q.shape).to(q.dtype)


def quantize_k_cache(k: torch.Tensor, num_kv_heads: int, head_dim: int, quantizer) -> torch.Tensor:
    """``_quantize_k_cache`` (:297-304): the KV quantizer along head_dim of ``[tokens, Hkv * D]``, after RoPE."""
    return quantizer.q(k.reshape(-1, num_kv_heads, head_dim)).reshape(k.shape).to(k.dtype)


def sequence_spans_from_positions(positions: Optional[torch.Tensor], n_tokens: int) -> List[Tuple[int, int]]:
    """``_sequence_spans_from_positions`` (:307-318): ``[left, right)`` runs of consecutive positions -- a new run
    starts wherever a position is not its predecessor + 1.  One device-to-host read instead of one per token."""
    if positions is None or positions.numel() != n_tokens or n_tokens == 0:
        return [(0, n_tokens)]
    pos = positions.detach().flatten().to(torch.long)
    breaks = (torch.nonzero(pos[1:] != pos[:-1] + 1).flatten() + 1).tolist()
    starts = [0] + breaks + [n_tokens]
    return list(zip(starts, starts[1:]))


def quantize_v_cache(v: torch.Tensor, num_kv_heads: int, head_dim: int, quantizer,
                     positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``_quantize_v_cache`` (:321-345): V quantised along the TOKEN axis, each sequence span on its own (blocks and
    scales never straddle two requests).  Per span the reference permutes to ``[Hkv, D, tokens]``, quantises and
    permutes back; here each span is one launch of the token-axis kernel that keeps the flattened layout."""
    vv = v.reshape(-1, num_kv_heads, head_dim)
    out = torch.empty_like(vv)
    for left, right in sequence_spans_from_positions(positions, vv.shape[0]):
        if right <= left:
            continue
        seq = vv[left:right]
        if isinstance(quantizer, _CudaBlockQuantizer):
            out[left:right] = write_v_cache(seq.unsqueeze(0), num_kv_heads, quantizer, token_major=True)[0]
        else:
            out[left:right] = quantizer.q(seq.permute(1, 2, 0).contiguous()).permute(2, 0, 1)
    return out.reshape(v.shape).to(v.dtype)


class KCenterTracker:
    """``_center_qwen_k_cache`` (:348-395): K of a Qwen2 block is centred over the prefill tokens of a sequence and
    the same centre serves that sequence's later decode tokens.  The engine hands over flattened batches without
    sequence ids, so centres are queued by the next position that will consume them, as in the reference."""

    def __init__(self):
        self.center_by_pos: Dict[int, List[torch.Tensor]] = {}

    def __call__(self, k: torch.Tensor, positions: torch.Tensor, num_kv_heads: int, head_dim: int) -> torch.Tensor:
        if positions.numel() != k.shape[0]:
            return k
        kv = k.reshape(-1, num_kv_heads, head_dim)
        pos = positions.detach().flatten().to(torch.long).tolist()
        centered = None
        for left, right in sequence_spans_from_positions(positions, kv.shape[0]):
            if right - left > 1:                                  # a prefill span: its own mean, queued for the next position
                center = kv[left:right].mean(dim=0, keepdim=True).detach()
                nxt = pos[right - 1] + 1
            else:                                                 # a decode token: the centre queued for its position
                queue = self.center_by_pos.get(pos[left])
                if not queue:
                    continue
                center = queue.pop(0).to(device=kv.device, dtype=kv.dtype)
                if not queue:
                    self.center_by_pos.pop(pos[left], None)
                nxt = pos[left] + 1
            if centered is None:
                centered = kv.clone()
            centered[left:right] = kv[left:right] - center
            self.center_by_pos.setdefault(nxt, []).append(center)
        return k if centered is None else centered.reshape_as(k).to(k.dtype)


class HBQLinearMethod:
    """``HBQNVFP4LinearMethod`` (:493-554) without the engine's base class: ``process_weights_after_loading``
    fake-quantises ``layer.weight`` once (idempotent through the ``hbq_weight_quantized`` mark, as the reference;
    no row chunking -- the reference chunks only to bound its eager quantizer's temporaries), ``apply`` quantises the
    activations and multiplies.  The product is the reference's ``F.linear`` (fp32 accumulation) on the tensor-core
    kernel, whose 128-column tile serves decode-sized batches."""

    def __init__(self, act_quantizer, wgt_quantizer, packed_weights: bool = False, packed_max_rows: int = 0):
        """``packed_weights``: keep each weight ONLY as 4-bit codes and scales in the tile order of ``hbq_gemm_w4``
        (0.56 B per weight; formats and shapes outside that kernel keep the fp16 tensor) -- the engine then holds a
        3.6x smaller model and every batch multiplies against codes expanded on chip.
        ``packed_max_rows`` (1..128, with ``packed_weights`` off): keep the packed weight BESIDE the fp16 tensor and
        send batches of up to that many tokens -- decode steps -- through the packed kernel, which streams 3.6x fewer
        bytes per step; larger batches multiply against the fp16 tensor."""
        self.act_quantizer = act_quantizer
        self.wgt_quantizer = wgt_quantizer
        self.packed_weights = packed_weights
        self.packed_max_rows = 0 if packed_weights else max(0, min(int(packed_max_rows), 128))

    @torch.inference_mode()
    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        if getattr(layer, "hbq_weight_quantized", False) or getattr(layer, "weight", None) is None:
            return
        w4 = None
        if (self.packed_weights or self.packed_max_rows) and layer.weight.is_cuda and layer.weight.dtype == torch.float16 and \
                hasattr(self.wgt_quantizer, "quantize_packed"):
            from ._lib import HbqError
            from .packed_gemm import W4Weight
            try:
                packed = self.wgt_quantizer.quantize_packed(layer.weight.data)
                if W4Weight.supported(packed):
                    w4 = W4Weight.from_packed(packed)
            except (NotImplementedError, HbqError):
                w4 = None
        if w4 is not None:
            layer.hbq_w4_weight = w4
        if w4 is not None and self.packed_weights:
            layer.weight.data = torch.empty(0, dtype=layer.weight.dtype, device=layer.weight.device)
        else:
            layer.weight.data = self.wgt_quantizer.q(layer.weight.data).to(layer.weight.dtype)
        setattr(layer, "hbq_weight_quantized", True)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        xq = self.act_quantizer.q(x)
        w4 = getattr(layer, "hbq_w4_weight", None)
        if w4 is not None and (layer.weight.numel() == 0 or xq.numel() // xq.shape[-1] <= self.packed_max_rows):
            x2d = xq.reshape(-1, xq.shape[-1])
            y = torch.empty((x2d.shape[0], w4.shape[0]), dtype=torch.float16, device=x2d.device)
            for r0 in range(0, x2d.shape[0], 128):
                w4.matmul(x2d[r0:r0 + 128], bias, out=y[r0:r0 + 128])
            return y.view(*x.shape[:-1], w4.shape[0])
        w = layer.weight
        if xq.is_cuda and xq.dtype == torch.float16 and w.dtype == torch.float16:
            y = ext.gemm_fp32_accum(xq.reshape(-1, xq.shape[-1]), w, b_is_nk=True, bias=bias)
            return y.view(*x.shape[:-1], w.shape[0])
        return torch.nn.functional.linear(xq, w, bias)
