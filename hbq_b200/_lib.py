"""ctypes binding of ``libhbq_b200.so`` (the C ABI declared in ``include/hbq_b200.h``).

There is no fallback: if the shared object is missing, or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libhbq_b200.so")

KIND_MXFP, KIND_MXINT, KIND_HBQ, KIND_MXEX, KIND_VSQ = 0, 1, 2, 3, 4
ERR_UNSUPPORTED = -2          # HBQ_ERR_UNSUPPORTED
ERR_ALIGN = -4                # HBQ_ERR_ALIGN
DTYPE_F16, DTYPE_BF16 = 0, 1
L2_SCHEMES = ["PoT", "INT", "SIG-1", "FP-1", "FP1", "FP-10", "FP-100", "Mix"]
ACC_FP32, ACC_FP16, ACC_GROUPED, ACC_PSUM_INT8, ACC_PSUM_E3M4 = range(5)
GEMM_NOALLOC_MAX_ELEMS = 4 * 1024 * 1024      # HBQ_GEMM_NOALLOC_MAX_ELEMS

# every symbol include/hbq_b200.h declares
EXPORTS = [
    "hbq_quantize", "hbq_absmax", "hbq_absmax_scratch_bytes", "hbq_dequantize", "hbq_fp_quant",
    "hbq_gemm", "hbq_gemm_workspace_bytes", "hbq_gemm_uses_tensor_cores", "hbq_gemm_simt",
    "hbq_gemm_kn_noalloc", "hbq_gemm_w4", "hbq_gemm_w4_prepack", "hbq_gemm_w4_prepacked_bytes",
    "hbq_gemm_w4_workspace_bytes", "hbq_kv_write_k", "hbq_kv_write_v", "hbq_swiglu_quantize", "hbq_rmsnorm_quantize", "hbq_softmax_quantize",
    "hbq_gemm_status", "hbq_gemm_status_reset", "hbq_gemm_wait_selftest", "hbq_gemm_reserve_sms", "hbq_error_string", "hbq_last_cuda_error",
    "hbq_version", "hbq_launch_count",
]


class Format(ctypes.Structure):
    """``hbq_format``"""
    _fields_ = [(n, ctypes.c_int32) for n in (
        "kind", "ebit", "mbit", "sc_ebit", "sc_mbit", "block_size", "scale_allow_subnormal",
        "use_round", "use_ceil", "l2_block_size", "l2_sc_bit", "l2_scheme", "per_tensor_scale",
        "reserved")]


class PackedOut(ctypes.Structure):
    """``hbq_packed_out``"""
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "codes", "sign", "scale_u8", "scale_h", "l2_packed", "l2_idx", "scheme")]


class HbqError(RuntimeError):
    pass


_lib = None


def lib() -> ctypes.CDLL:
    """Load the library once.  Raises if it has not been built (``python -m hbq_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise HbqError(f"{LIB_PATH} is missing: build it with `python -m hbq_b200.build` "
                       "(there is no CPU or PyTorch fallback)")
    L = ctypes.CDLL(LIB_PATH)
    i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
    L.hbq_quantize.argtypes = [vp, ci, i64, i64, ctypes.POINTER(Format), vp, ci,
                               ctypes.POINTER(PackedOut), vp, vp]
    L.hbq_absmax.argtypes = [vp, ci, i64, vp, vp, vp]
    L.hbq_absmax_scratch_bytes.restype = i64
    L.hbq_dequantize.argtypes = [ctypes.POINTER(PackedOut), i64, i64, ctypes.POINTER(Format), vp, ci, vp]
    L.hbq_fp_quant.argtypes = [vp, i64, ci, ci, ci, ci, ci, vp, vp]
    L.hbq_gemm.argtypes = [vp, vp, vp, i64, i64, i64, ci, ci, ci, ci, vp, vp, i64, vp]
    L.hbq_gemm_simt.argtypes = [vp, vp, vp, i64, i64, i64, ci, ci, ci, ci, vp, vp]
    L.hbq_gemm_kn_noalloc.argtypes = [vp, vp, vp, i64, i64, i64, ci, ci, ci, vp, vp]
    L.hbq_kv_write_k.argtypes = [vp, ci, i64, i64, i64, i64, vp, vp, i64, vp, ctypes.POINTER(Format), vp, ci, vp]
    L.hbq_kv_write_v.argtypes = [vp, ci, i64, i64, i64, i64, ctypes.POINTER(Format), vp, ci, ci, vp]
    L.hbq_swiglu_quantize.argtypes = [vp, vp, i64, i64, ctypes.POINTER(Format), vp, vp]
    L.hbq_rmsnorm_quantize.argtypes = [vp, vp, vp, ctypes.c_float, i64, i64, ctypes.POINTER(Format), vp, vp, vp]
    L.hbq_softmax_quantize.argtypes = [vp, i64, i64, i64, i64, ctypes.c_float, ci, vp, i64, ctypes.POINTER(Format), vp, vp]
    L.hbq_gemm_workspace_bytes.argtypes = [i64, i64, i64, ci, ci, ci, ci]
    L.hbq_gemm_workspace_bytes.restype = i64
    L.hbq_gemm_uses_tensor_cores.argtypes = [i64, i64, i64, ci, ci, ci, ci]
    L.hbq_gemm_w4_prepacked_bytes.argtypes = [i64, i64, ci]
    L.hbq_gemm_w4_prepacked_bytes.restype = i64
    L.hbq_gemm_w4_prepack.argtypes = [ctypes.POINTER(PackedOut), i64, i64, ctypes.POINTER(Format), ci, vp, vp]
    L.hbq_gemm_w4_workspace_bytes.argtypes = [i64, i64, i64]
    L.hbq_gemm_w4_workspace_bytes.restype = i64
    L.hbq_gemm_w4.argtypes = [vp, vp, vp, i64, i64, i64, ctypes.POINTER(Format), ci, vp, vp, i64, vp]
    L.hbq_gemm_status.argtypes = [ctypes.POINTER(ci)]
    L.hbq_gemm_wait_selftest.argtypes = [vp, vp, vp, i64, i64, i64, ci, ci, ci, ctypes.c_uint32, vp]
    L.hbq_gemm_reserve_sms.argtypes = [ci]
    L.hbq_error_string.argtypes = [ci]
    L.hbq_error_string.restype = ctypes.c_char_p
    L.hbq_last_cuda_error.restype = ctypes.c_char_p
    L.hbq_launch_count.restype = i64
    _lib = L
    return L


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def device_guard(device):
    """``torch.cuda.device(device)`` when ``device`` is not the current one, else nothing: the context
    manager costs several microseconds, which is most of a decode-sized kernel."""
    import torch
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def check(rc: int, what: str) -> None:
    if rc != 0:
        L = lib()
        msg = L.hbq_error_string(rc).decode()
        extra = L.hbq_last_cuda_error().decode()
        raise HbqError(f"{what}: {msg}" + (f" [{extra}]" if rc == -3 and extra else ""))


def launch_count() -> int:
    return int(lib().hbq_launch_count())
