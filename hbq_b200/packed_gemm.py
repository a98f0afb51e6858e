"""GEMM on the packed 4-bit weight for decode-sized batches (``hbq_gemm_w4``).

The reference keeps a statically quantised weight as the fp16 fake-quantised tensor (src/ptq.py:349) and multiplies
with ``F.linear`` (src/module.py:64).  ``W4Weight`` holds the same weight as codes, block scales and micro-scale
indices in the tile order of the kernel (0.5625 B per weight); ``matmul`` gives ``x @ w.T`` with fp32 accumulation for
up to 128 rows of ``x``, every product taken on the fp16 value the fake-quantised tensor would hold.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from .quantizer import PackedTensor, _ptr, _stream_ptr

MAX_ROWS = 128                      # tokens per call the kernel takes


class W4Weight:
    """A quantised weight ``[N, K]`` prepacked for ``hbq_gemm_w4``."""

    def __init__(self, data: torch.Tensor, fmt: "_lib.Format", shape: Tuple[int, int], container_bits: int = 4):
        self.data, self.fmt, self.shape = data, fmt, (int(shape[0]), int(shape[1]))
        self.container_bits = container_bits
        self._workspaces: Dict[Tuple[int, int], torch.Tensor] = {}

    @staticmethod
    def supported(packed: PackedTensor) -> bool:
        """True when the kernel expands this format and shape (otherwise multiply with the fp16 tensor)."""
        if packed.codes is None or not packed.codes.is_cuda or len(packed.shape) != 2:
            return False
        N, K = packed.shape
        return int(_lib.lib().hbq_gemm_w4_prepacked_bytes(N, K, 4)) > 0 and packed.l2_packed is not None and \
            packed.sign is None

    @classmethod
    def from_packed(cls, packed: PackedTensor, container_bits: int = 4) -> "W4Weight":
        """Rearrange the planes of ``quantize_packed`` (``hbq_gemm_w4_prepack``); raises for formats outside the kernel.
        ``container_bits``: 4 keeps the codes as nibbles (0.5625 B per weight), expanded by the hardware's E2M1
        conversion -- the smaller and on B200 the faster form; 8 stores each code as the top byte of its value's fp16
        pattern (1.0625 B per weight), expanded by a byte permute."""
        N, K = packed.shape
        L = _lib.lib()
        nbytes = int(L.hbq_gemm_w4_prepacked_bytes(N, K, container_bits))
        if nbytes <= 0:
            raise _lib.HbqError(f"hbq_gemm_w4: weight shape {tuple(packed.shape)} is not a multiple of 128 x 128 "
                                f"(or container_bits {container_bits} is not 4 or 8)")
        dev = packed.codes.device
        out = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        po = _lib.PackedOut(packed.codes.data_ptr(), None, packed.scale_u8.data_ptr(), None,
                            packed.l2_packed.data_ptr() if packed.l2_packed is not None else None, None,
                            packed.scheme.data_ptr() if packed.scheme is not None else None)
        with _lib.device_guard(dev):
            rc = L.hbq_gemm_w4_prepack(ctypes.byref(po), N, K, ctypes.byref(packed.fmt), container_bits, _ptr(out),
                                       _stream_ptr(dev))
        _lib.check(rc, "hbq_gemm_w4_prepack")
        return cls(out, packed.fmt, (N, K), container_bits)

    def nbytes(self) -> int:
        return self.data.numel()

    def _workspace(self, rows: int) -> torch.Tensor:
        """Zeroed once per (row count, stream); the kernel hands it back zeroed where it matters."""
        N, K = self.shape
        key = (rows, _stream_ptr(self.data.device))
        ws = self._workspaces.get(key)
        if ws is None:
            n = int(_lib.lib().hbq_gemm_w4_workspace_bytes(rows, N, K))
            if n < 0:
                raise _lib.HbqError(f"hbq_gemm_w4: {rows} rows are outside the kernel (1..{MAX_ROWS})")
            ws = torch.zeros(max(n, 16), dtype=torch.uint8, device=self.data.device)
            self._workspaces[key] = ws
        return ws

    def matmul(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x [M, K] fp16 -> x @ w.T (+ bias) [M, N] fp16``, M <= 128."""
        N, K = self.shape
        if x.dtype != torch.float16 or x.dim() != 2 or x.shape[1] != K or x.device != self.data.device:
            raise RuntimeError("x must be an fp16 [M, K] tensor on the weight's device")
        M = x.shape[0]
        x = x.contiguous()
        if bias is not None:
            bias = bias.to(device=x.device, dtype=torch.float16).contiguous()
        c = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=x.device)
        if M == 0:
            return c
        ws = self._workspace(M)
        with _lib.device_guard(x.device):
            rc = _lib.lib().hbq_gemm_w4(_ptr(x), _ptr(self.data), _ptr(c), M, N, K, ctypes.byref(self.fmt), self.container_bits, _ptr(bias),
                                        _ptr(ws), ws.numel(), _stream_ptr(x.device))
        _lib.check(rc, "hbq_gemm_w4")
        return c
