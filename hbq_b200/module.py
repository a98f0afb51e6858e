"""Quantizer-carrying linear layer with the reference's fields (``_QBaseLinear``,
src/module.py:21-67): ``wq`` / ``aq`` / ``yq`` quantizers and an optional ``ops`` GEMM operator.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .ops import FP16AccumMatMul
from .quantizer import PackedTensor, _QBase, dequantize_packed


_HOST_PIPES = {}      # device -> streams and staging buffers of forward_host


class QLinear(nn.Linear):
    """y = yq(ops(aq(x), W, b)); W is expected to be fake-quantised already (static weight
    quantisation, src/ptq.py:337-382).  ``ops=None`` uses ``F.linear`` like the reference
    (fp16 GEMM with fp32 accumulation).  ``check_finite`` keeps the reference's non-finite
    guard (src/module.py:52-65), which synchronises the host on every call."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, ops=None,
                 check_finite: bool = True, device=None, dtype=None):
        super().__init__(in_features, out_features, bias, device=device, dtype=dtype)
        self.wq = _QBase()
        self.aq = _QBase()
        self.yq = _QBase()
        self.ops = ops
        self.check_finite = check_finite
        self.packed_weight = None
        self.w4_weight = None          # the packed weight in the decode GEMM's tile order (prepare_decode)
        self.w4_max_rows = 0           # batches up to this many rows take it while the fp16 tensor is kept.
                                       # prepare_decode sets 8: up to there the packed kernels beat the library
                                       # fp16 GEMM on every Llama-3-8B shape on B200 (1.2-2.2x); at 16 rows they are
                                       # faster on the MLP shapes and slower on the 4096 x 4096 projections

    def forward(self, x: torch.Tensor, input_quantized: bool = False):
        """``input_quantized``: ``x`` has been through ``self.aq`` already (a producer that fuses the
        quantizer, e.g. ``swiglu_quantize``)."""
        wq = self.weight
        xq = x if input_quantized else self.aq(x)
        w4 = self.w4_weight
        rows = xq.numel() // xq.shape[-1] if xq.shape[-1] else 0
        if w4 is not None and self.ops is None and xq.is_cuda and xq.dtype == torch.float16 and \
                (0 < rows <= self.w4_max_rows or wq.numel() == 0):
            # the packed weight streams at 0.56 B per element instead of 2; 128 rows per launch
            x2d = xq.reshape(-1, xq.shape[-1])
            if rows <= 128:
                y = w4.matmul(x2d, self.bias)
            else:
                y = torch.empty((rows, self.out_features), dtype=torch.float16, device=xq.device)
                for r0 in range(0, rows, 128):
                    w4.matmul(x2d[r0:r0 + 128], self.bias, out=y[r0:r0 + 128])
            y = y.view(*xq.shape[:-1], self.out_features)
        elif self.ops is None:
            y = F.linear(xq, wq, self.bias)
        else:
            y = self.ops(xq, wq, self.bias)
        if self.check_finite and isinstance(self.ops, FP16AccumMatMul) and y.is_cuda:
            # the host synchronises for the non-finite guard below anyway: also ask whether a bounded wait
            # of the tensor-core kernel ran out (its output would be undefined)
            from .gemm import gemm_status
            st = gemm_status()
            if st != 0:
                raise RuntimeError(f"tensor-core GEMM gave up on a wait (status {st}); the output is undefined. "
                                   "Clear with hbq_gemm_status_reset after finding the cause.")
        if self.check_finite and not torch.isfinite(y).all():
            ops_name = type(self.ops).__name__ if self.ops is not None else "F.linear"
            raise RuntimeError(
                f"Non-finite output from {type(self).__name__}"
                f"({self.in_features} -> {self.out_features}): "
                f"{int(y.isnan().sum())} NaN and {int(y.isinf().sum())} Inf "
                f"out of {y.numel()} elements.\n"
                f"  activation quantizer: {type(self.aq).__name__}\n"
                f"  weight quantizer:     {type(self.wq).__name__}\n"
                f"  matmul:               {ops_name}")
        return self.yq(y)

    # ---- packed weight storage -----------------------------------------------------------------
    def pack_weight(self, wq=None):
        """Quantise the weight with ``wq`` (default ``self.wq``) into packed codes and scales
        (``PackedTensor``, 0.52-0.54 B per element for the HBQ weight formats), keep that as
        ``self.packed_weight`` and install its dequantised form as the fp16 weight the GEMM reads.
        The reference keeps only the fp16 fake-quantised weight (src/ptq.py:349) and re-runs the
        quantizer (12 s per 4096x4096 matrix on CPU) whenever a model is loaded."""
        wq = self.wq if wq is None else wq
        self.packed_weight = wq.quantize_packed(self.weight.data)
        self.weight.data = dequantize_packed(self.packed_weight).to(self.weight.dtype)
        return self.packed_weight

    def prepare_decode(self, wq=None, drop_fp16: bool = False) -> bool:
        """Keep the packed weight also in the tile order of ``hbq_gemm_w4`` so that batches of up to
        ``w4_max_rows`` rows (8 unless set before) multiply against 4-bit codes and scales expanded on chip (same products as
        with the fp16 tensor: the expanded values are its values bit for bit).  ``drop_fp16`` frees the fp16 tensor:
        the layer then holds 0.56 B per weight and EVERY batch goes through the packed kernel, 128 rows per launch
        (a capacity mode: large batches are slower than on the fp16 tensor).  Returns False, and changes nothing, for
        formats and shapes outside that kernel or when the layer has an accumulation operator (the kernel
        accumulates in fp32 like ``F.linear``)."""
        from .packed_gemm import W4Weight
        if self.ops is not None or not self.weight.is_cuda or self.weight.dtype != torch.float16:
            return False
        if self.packed_weight is None:
            wq = self.wq if wq is None else wq
            if not hasattr(wq, "quantize_packed"):
                return False
            try:
                self.pack_weight(wq)
            except NotImplementedError:
                return False
        if not W4Weight.supported(self.packed_weight):
            return False
        from ._lib import HbqError
        try:
            self.w4_weight = W4Weight.from_packed(self.packed_weight)
        except HbqError:               # a micro-scale table the kernel does not expand
            self.w4_weight = None
            return False
        if drop_fp16:
            self.weight.data = torch.empty(0, dtype=self.weight.dtype, device=self.weight.device)
            self.packed_weight = None
        elif self.w4_max_rows == 0:
            self.w4_max_rows = 8
        return True

    def load_packed_weight(self, packed):
        """Install a weight from its packed form (``PackedTensor`` or its ``state_dict()``)."""
        if isinstance(packed, dict):
            packed = PackedTensor.from_state_dict(packed, device=self.weight.device)
        if tuple(packed.shape) != tuple(self.weight.shape):
            raise ValueError(f"packed weight has shape {tuple(packed.shape)}, layer expects {tuple(self.weight.shape)}")
        self.packed_weight = packed
        self.weight.data = dequantize_packed(packed).to(self.weight.dtype)

    # ---- host-buffer entry -------------------------------------------------------------------
    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor = None, row_chunks: int = 2,
                     wait: bool = True):
        """The same layer for callers whose activations live in (pinned) host memory.

        Rows are cut into ``row_chunks`` pieces that travel through three streams: host-to-device
        copy, quantize + GEMM, device-to-host copy of the result, with two staging buffers, so the
        two PCIe directions and the kernels overlap within a call and across consecutive calls.
        Returns ``out_host`` (pinned fp16 ``[rows, out_features]``) after the host has waited for
        the last download, so the caller may read it at once.  With ``wait=False`` nothing waits;
        ``(out_host, event)`` is returned and the caller synchronises on the event before reading,
        which lets the next call's uploads start under this call's downloads."""
        dev = self.weight.device
        if x_host.is_cuda or x_host.dim() != 2 or x_host.shape[1] != self.in_features:
            raise ValueError("forward_host expects a host tensor of shape [rows, in_features]")
        rows = x_host.shape[0]
        if out_host is None:
            out_host = torch.empty((rows, self.out_features), dtype=self.weight.dtype, pin_memory=True)
        P = _HOST_PIPES.get(dev)
        if P is None:
            # one set of streams and staging buffers per device, shared by every layer
            P = _HOST_PIPES[dev] = {"h2d": torch.cuda.Stream(dev), "comp": torch.cuda.Stream(dev),
                                    "d2h": torch.cuda.Stream(dev), "xbuf": [None, None], "x_free": [None, None], "n": 0}
        h2d, comp, d2h = P["h2d"], P["comp"], P["d2h"]
        cur = torch.cuda.current_stream(dev)
        start = torch.cuda.Event()
        start.record(cur)
        h2d.wait_event(start)                      # inputs prepared on the calling stream are visible
        step = -(-rows // max(1, row_chunks))
        step = max(128, -(-step // 128) * 128)     # whole GEMM row tiles per piece
        done = None
        for r0 in range(0, rows, step):
            r1 = min(rows, r0 + step)
            slot = P["n"] & 1
            P["n"] += 1
            with torch.cuda.stream(h2d):
                if P["x_free"][slot] is not None:
                    h2d.wait_event(P["x_free"][slot])          # the kernels that read this buffer are done
                xb = P["xbuf"][slot]
                need = (r1 - r0) * self.in_features
                if xb is None or xb.numel() < need or xb.dtype != x_host.dtype:
                    xb = P["xbuf"][slot] = torch.empty(step * self.in_features, dtype=x_host.dtype, device=dev)
                xv = xb[:need].view(r1 - r0, self.in_features)
                xv.copy_(x_host[r0:r1], non_blocking=True)
                up = torch.cuda.Event()
                up.record(h2d)
            with torch.cuda.stream(comp):
                comp.wait_event(up)
                y = self.forward(xv)
                ev = torch.cuda.Event()
                ev.record(comp)
                P["x_free"][slot] = ev
            with torch.cuda.stream(d2h):
                d2h.wait_event(ev)
                out_host[r0:r1].copy_(y, non_blocking=True)
                y.record_stream(d2h)
                done = torch.cuda.Event()
                done.record(d2h)
        if done is None:
            return out_host if wait else (out_host, start)
        if wait:
            done.synchronize()
            return out_host
        return out_host, done
