"""Block quantizers with the reference's Python surface, computed by the CUDA library.

Mirrors ``src/quantizer.py`` of HBQ: ``_QBase``, ``MXFPQuantizer`` (:430-539),
``MXINTQuantizer`` (:347-428) and ``HBQQuantizer`` (:704-859) keep their constructor
signatures, are ``nn.Module``s, and ``q(x)`` / ``forward(x)`` return the fake-quantised tensor
with ``x``'s shape and dtype, bit-identical to the reference's eager fp16 result.  Differences:

* inputs must be CUDA tensors (there is no CPU path);
* bf16 inputs are accepted by every class: they are converted to fp16, quantised with the fp16
  semantics of the reference, and the result is rounded to bf16 (the reference's MXFP / MXINT
  raise ``NotImplementedError`` for bf16);
* fp32 inputs raise ``NotImplementedError`` (the reference would quantise them with fp32
  roundings, which these kernels do not model);
* ``quantize_packed(x)`` additionally returns the element codes and scales in the packed device
  layout described in ``include/hbq_b200.h``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from . import _lib


def get_max_norm(ebit: int, mbit: int, unsigned: bool = False):
    """Largest normal value of E<ebit>M<mbit>, or of INT<mbit> when ``ebit == 0``
    (src/quantizer.py:148-164)."""
    if ebit == 0:
        return 2 ** mbit - 1 if unsigned else 2 ** (mbit - 1) - 1
    if (ebit, mbit) == (4, 3):
        return 448
    emax = 15 if ebit == 5 else 2 ** (ebit - 1)
    return 2 ** emax * float(2 ** (mbit + 1) - 1) / 2 ** mbit


def get_min_norm(ebit: int, mbit: int):
    """src/quantizer.py:166-178"""
    if ebit == 0:
        return 0
    if ebit == 1:
        return 1
    return 2 ** (2 - 2 ** (ebit - 1))


def get_min_subnorm(ebit: int, mbit: int):
    """src/quantizer.py:180-185"""
    return 2 ** (2 - 2 ** (ebit - 1)) * 2 ** (-mbit)


@dataclass
class PackedTensor:
    """Packed result of ``quantize_packed``: device tensors in the layout of ``hbq_packed_out``."""
    shape: torch.Size
    dtype: torch.dtype
    fmt: "_lib.Format"
    codes: torch.Tensor
    sign: Optional[torch.Tensor]
    scale_u8: torch.Tensor
    l2_packed: Optional[torch.Tensor]
    scheme: Optional[torch.Tensor]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in
                   (self.codes, self.sign, self.scale_u8, self.l2_packed, self.scheme) if t is not None)

    _PLANES = ("codes", "sign", "scale_u8", "l2_packed", "scheme")

    def state_dict(self) -> dict:
        """Plain dict (tensors, ints, strings) for ``torch.save``: the packed planes plus the format
        fields, so a quantised weight is stored at its real size and restored without re-quantising."""
        d = {"shape": tuple(self.shape), "dtype": str(self.dtype).replace("torch.", ""),
             "format": {n: int(getattr(self.fmt, n)) for n, _ in _lib.Format._fields_}}
        for n in self._PLANES:
            t = getattr(self, n)
            if t is not None:
                d[n] = t
        return d

    @classmethod
    def from_state_dict(cls, d: dict, device=None) -> "PackedTensor":
        fmt = _lib.Format(*[int(d["format"][n]) for n, _ in _lib.Format._fields_])
        planes = {n: (d[n].to(device) if device is not None else d[n]) if n in d else None for n in cls._PLANES}
        return cls(torch.Size(d["shape"]), getattr(torch, d["dtype"]), fmt, planes["codes"], planes["sign"],
                   planes["scale_u8"], planes["l2_packed"], planes["scheme"])


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return _lib.DTYPE_F16
    if t.dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    raise NotImplementedError(f"Non-supported data type: {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def dequantize_packed(p: PackedTensor) -> torch.Tensor:
    """Rebuild the fake-quantised tensor from packed codes and scales (``hbq_dequantize``)."""
    K = p.shape[-1]
    rows = p.codes.shape[0]
    out = torch.empty(p.shape, dtype=p.dtype, device=p.codes.device)
    po = _lib.PackedOut(p.codes.data_ptr(), p.sign.data_ptr() if p.sign is not None else None,
                        p.scale_u8.data_ptr(), None,
                        p.l2_packed.data_ptr() if p.l2_packed is not None else None, None,
                        p.scheme.data_ptr() if p.scheme is not None else None)
    with _lib.device_guard(out.device):
        rc = _lib.lib().hbq_dequantize(ctypes.byref(po), rows, K, ctypes.byref(p.fmt), _ptr(out),
                                       _dtype_code(out), _stream_ptr(out.device))
    _lib.check(rc, "hbq_dequantize")
    return out


class _QBase(nn.Module):
    """Base quantizer: identity (src/quantizer.py:330-345)."""

    def __init__(self):
        super().__init__()

    def q(self, x: torch.Tensor):
        return x

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.q(x)


class _CudaBlockQuantizer(_QBase):
    """Shared launch logic of the three block quantizers.

    ``out_dtype`` (attribute, default ``None`` = the input's dtype as in the reference) lets a
    caller ask for the fake-quantised tensor in fp16 whatever the input type, which is what the
    accumulation-modelling GEMM consumes."""

    out_dtype: Optional[torch.dtype] = None

    def _format(self) -> "_lib.Format":
        raise NotImplementedError

    def _code_bits(self) -> int:
        f = self._format()
        if f.kind == _lib.KIND_MXINT:
            return 4 if f.mbit <= 4 else 8
        b = 1 + f.ebit + f.mbit
        return 4 if b < 4 else (b if b <= 5 else 8)

    def _launch(self, x: torch.Tensor, want_deq: bool, out_struct, keep=None) -> Optional[torch.Tensor]:
        if not x.is_cuda:
            raise _lib.HbqError("hbq_b200 quantizers need a CUDA tensor (there is no CPU fallback)")
        fmt = self._format()
        xc = x.contiguous()
        K = xc.shape[-1] if xc.dim() > 0 else 1
        rows = xc.numel() // K if K else 0
        odt = self.out_dtype or xc.dtype
        deq = torch.empty(xc.shape, dtype=odt, device=xc.device) if want_deq else None
        amax = None
        with _lib.device_guard(xc.device):
            stream = _stream_ptr(xc.device)
            L = _lib.lib()
            if fmt.kind == _lib.KIND_MXFP and fmt.per_tensor_scale and xc.numel():
                amax = torch.empty(1, dtype=torch.float32, device=xc.device)
                scratch = torch.empty(int(L.hbq_absmax_scratch_bytes()), dtype=torch.uint8, device=xc.device)
                _lib.check(L.hbq_absmax(_ptr(xc), _dtype_code(xc), xc.numel(), _ptr(amax), _ptr(scratch), stream),
                           "hbq_absmax")
            rc = L.hbq_quantize(_ptr(xc), _dtype_code(xc), rows, K, ctypes.byref(fmt), _ptr(deq),
                                _dtype_code(deq) if deq is not None else 0,
                                ctypes.byref(out_struct) if out_struct is not None else None,
                                _ptr(amax), stream)
        _lib.check(rc, f"hbq_quantize[{type(self).__name__}]")
        return deq

    def q(self, x: torch.Tensor) -> torch.Tensor:
        return self._launch(x, True, None)          # allocated with x's shape

    def quantize_packed(self, x: torch.Tensor, with_deq: bool = False):
        """Quantise ``x`` along its last axis into packed codes and scales.

        Returns ``PackedTensor`` (and the fake-quantised tensor too when ``with_deq``)."""
        fmt = self._format()
        K = x.shape[-1]
        rows = x.numel() // K
        B = fmt.block_size
        nblk = -(-K // B)
        Kp = nblk * B
        dev = x.device
        bits = self._code_bits()
        u8 = dict(dtype=torch.uint8, device=dev)
        codes = torch.empty((rows, Kp // 2 if bits <= 5 else Kp), **u8)
        sign = torch.empty((rows, Kp // 8), **u8) if bits == 5 else None
        scale_u8 = torch.empty((rows, nblk), **u8)
        l2p = scheme = None
        if fmt.kind == _lib.KIND_HBQ:
            tb = (B // fmt.l2_block_size) * fmt.l2_sc_bit
            l2p = torch.empty((rows, nblk, max(tb // 8, 1)), **u8)
            if fmt.l2_scheme == _lib.L2_SCHEMES.index("Mix"):
                scheme = torch.empty((rows, nblk), **u8)
        po = _lib.PackedOut(codes.data_ptr(), sign.data_ptr() if sign is not None else None,
                            scale_u8.data_ptr(), None, l2p.data_ptr() if l2p is not None else None, None,
                            scheme.data_ptr() if scheme is not None else None)
        deq = self._launch(x, with_deq, po)
        packed = PackedTensor(x.shape, self.out_dtype or x.dtype, fmt, codes, sign, scale_u8, l2p, scheme)
        return (packed, deq.view(x.shape)) if with_deq else packed


class MXINTQuantizer(_CudaBlockQuantizer):
    """MXINT quantization (src/quantizer.py:347-428).

    nbit: element bit width; sc_ebit / sc_mbit: shared-scale format (sc_mbit = 0: power of two,
    exponent clipped to [-14, 15]); block_size: elements per shared scale."""

    def __init__(self, nbit: int, sc_ebit: int = 8, sc_mbit: int = 0, block_size: int = 32,
                 per_tensor_scale: bool = False, scale_allow_subnormal: bool = False, use_ceil: bool = False):
        super().__init__()
        self.nbit = nbit
        self.sc_ebit = sc_ebit
        self.sc_mbit = sc_mbit
        self.block_size = block_size
        self.per_tensor_scale = per_tensor_scale
        self.scale_allow_subnormal = scale_allow_subnormal
        self.shared_exp = None
        self.use_ceil = use_ceil

    def _format(self):
        return _lib.Format(_lib.KIND_MXINT, 0, self.nbit, self.sc_ebit, self.sc_mbit, self.block_size,
                           int(self.scale_allow_subnormal), 0, int(self.use_ceil), 0, 0, 0, 0, 0)


class MXFPQuantizer(_CudaBlockQuantizer):
    """MXFP / NVFP quantization (src/quantizer.py:430-539).

    ebit / mbit: element format; sc_ebit / sc_mbit: shared-scale format (sc_mbit = 0: power of two);
    per_tensor_scale: scale the tensor into (element range x scale range) first, as official NVFP4;
    use_round: round instead of floor the power-of-two exponent; use_ceil: ceil the FP scale;
    activate_dynamo: accepted for signature compatibility (the CUDA kernel is always used)."""

    def __init__(self, block_size: int = 32, ebit: int = 2, mbit: int = 3, sc_ebit: int = 0, sc_mbit: int = 8,
                 per_tensor_scale: bool = False, scale_allow_subnormal: bool = False, use_round: bool = False,
                 use_ceil: bool = False, activate_dynamo: bool = False):
        super().__init__()
        self.ebit = ebit
        self.mbit = mbit
        self.sc_ebit = sc_ebit
        self.sc_mbit = sc_mbit
        self.block_size = block_size
        self.per_tensor_scale = per_tensor_scale
        self.scale_allow_subnormal = scale_allow_subnormal
        self.use_round = use_round
        self.use_ceil = use_ceil

    def _format(self):
        return _lib.Format(_lib.KIND_MXFP, self.ebit, self.mbit, self.sc_ebit, self.sc_mbit, self.block_size,
                           int(self.scale_allow_subnormal), int(self.use_round), int(self.use_ceil),
                           0, 0, 0, int(self.per_tensor_scale), 0)


class HBQQuantizer(MXFPQuantizer):
    """HBQ two-level quantization (src/quantizer.py:704-859): an FP (E5M3) shared scale per block
    and, per micro-block of ``l2_block_size`` elements, the micro-scale among ``2**l2_sc_bit``
    candidates of ``l2_scheme`` that minimises the squared error ("Mix": also the better of two
    candidate tables per block).  With ``keep_l2_scale`` the chosen scales are kept as
    ``shared_scale`` / ``l2_scale`` / ``blk_l2_scheme`` / ``real_l2_scale`` like the reference.
    ``per_tensor_scale`` and ``use_round`` are accepted and ignored, as in the reference."""

    L2_SCHEME = ["PoT", "INT", "SIG-1", "FP-1", "FP1", "FP-10", "FP-100", "Mix"]

    def __init__(self, block_size: int = 128, ebit: int = 2, mbit: int = 3, sc_ebit: int = 5, sc_mbit: int = 3,
                 l2_block_size: int = 4, l2_sc_bit: int = 1, l2_scheme: str = "PoT", keep_l2_scale: bool = False,
                 per_tensor_scale: bool = False, scale_allow_subnormal: bool = False, use_round: bool = False,
                 use_ceil: bool = False, use_quant_kernel: bool = True):
        super().__init__(block_size, ebit, mbit, sc_ebit, sc_mbit, per_tensor_scale, scale_allow_subnormal,
                         use_round, use_ceil, use_quant_kernel)
        assert block_size % l2_block_size == 0, "block_size must be divisible by l2_block_size"
        assert l2_scheme in self.L2_SCHEME, f"Invalid L2 scheme: {l2_scheme}"
        self.keep_l2_scale = keep_l2_scale
        self.l2_block_size = l2_block_size
        self.l2_sc_bit = l2_sc_bit
        self.l2_scheme = l2_scheme
        self.win_rate = []

    def _format(self):
        return _lib.Format(_lib.KIND_HBQ, self.ebit, self.mbit, self.sc_ebit, self.sc_mbit, self.block_size,
                           int(self.scale_allow_subnormal), 0, int(self.use_ceil), self.l2_block_size,
                           self.l2_sc_bit, self.L2_SCHEME.index(self.l2_scheme), 0, 0)

    def l2_table(self, device=None) -> torch.Tensor:
        """Candidate micro-scales [n_scheme, 2**l2_sc_bit] (src/quantizer.py:745-770)."""
        r = torch.arange(2 ** self.l2_sc_bit, dtype=torch.float32)
        n = 2 ** self.l2_sc_bit
        tabs = {"PoT": 2 ** r, "INT": r + 1, "SIG-1": 1 + r / 2, "FP-1": 1 + r / n, "FP1": 1 + (r + 1) / n,
                "FP-10": 1 + r / (2 * n), "FP-100": 1 + r / (4 * n)}
        t = torch.stack([tabs["FP-1"], tabs["FP-10"]]) if self.l2_scheme == "Mix" else tabs[self.l2_scheme][None]
        return t.to(torch.float16).to(device) if device is not None else t.to(torch.float16)

    def q(self, x: torch.Tensor) -> torch.Tensor:
        if not self.keep_l2_scale:
            return super().q(x)
        K = x.shape[-1]
        lead = tuple(x.shape[:-1])
        rows = x.numel() // K
        B = self.block_size
        nblk = -(-K // B)
        nl2 = B // self.l2_block_size
        dev = x.device
        scale_h = torch.empty((rows, nblk), dtype=torch.float16, device=dev)
        l2_idx = torch.empty((rows, nblk, nl2), dtype=torch.uint8, device=dev)
        scheme = torch.zeros((rows, nblk), dtype=torch.uint8, device=dev)
        po = _lib.PackedOut(None, None, None, scale_h.data_ptr(), None, l2_idx.data_ptr(), scheme.data_ptr())
        deq = self._launch(x, True, po)
        self.shared_scale = scale_h.view(*lead, nblk)
        self.l2_scale = l2_idx.view(*lead, nblk, nl2).long()
        self.blk_l2_scheme = scheme.view(*lead, nblk).long()
        tab = self.l2_table(dev)
        self.real_l2_scale = tab[self.blk_l2_scheme[..., None].expand_as(self.l2_scale), self.l2_scale]
        return deq.view(x.shape)


class MXExQuantizer(_CudaBlockQuantizer):
    """MicroExponent quantization (src/quantizer.py:541-628): a power-of-two shared scale per block
    and, per micro-block of ``l2_block_size`` elements, the better of an integer grid with step 1
    and one with step 2.  ``l2_block_size`` up to 8."""

    def __init__(self, block_size: int = 16, l2_block_size: int = 2, sc_bit: int = 8, l2_sc_bit: int = 1,
                 mbit: int = 3):
        super().__init__()
        self.sc_bit = sc_bit
        self.l2_sc_bit = l2_sc_bit
        self.mbit = mbit
        self.block_size = block_size
        self.l2_block_size = l2_block_size

    def _format(self):
        return _lib.Format(_lib.KIND_MXEX, 0, self.mbit, self.sc_bit, 0, self.block_size, 0, 0, 0,
                           self.l2_block_size, self.l2_sc_bit, 0, 0, 0)

    def quantize_packed(self, x, with_deq: bool = False):
        raise NotImplementedError("MXExQuantizer has no packed storage form")


class VSQQuantizer(_CudaBlockQuantizer):
    """VSQ two-level integer quantization (src/quantizer.py:630-702): a per-vector scale quantised to
    ``sc_mbit`` unsigned bits against a per-row first-level scale."""

    def __init__(self, nbit: int, block_size: int = 16, sc_mbit: int = 4):
        super().__init__()
        self.nbit = nbit
        self.block_size = block_size
        self.sc_mbit = sc_mbit

    def _format(self):
        return _lib.Format(_lib.KIND_VSQ, 0, self.nbit, 0, self.sc_mbit, self.block_size, 0, 0, 0, 0, 0, 0, 0, 0)

    def quantize_packed(self, x, with_deq: bool = False):
        raise NotImplementedError("VSQQuantizer has no packed storage form")
