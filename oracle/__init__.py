"""CPU oracle for the HBQ hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

ctypes front-end of ``libhbq_oracle.so`` (built from ``hbq_oracle.c`` by the
Makefile beside it).  Only tests, the smoke check and the CPU-baseline leg of the
benchmark may import this package; the CUDA library never does.

Parity status: pinned.  ``tests/test_oracle_golden.py`` checks every function
here against vectors made by importing the reference's own Python quantizers
(``tests/golden/make_golden.py``), including exhaustive sweeps over all 65 536
fp16 inputs of the element and scale quantizers.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libhbq_oracle.so")

KIND_MXFP, KIND_MXINT, KIND_HBQ, KIND_MXEX, KIND_VSQ = 0, 1, 2, 3, 4
L2_SCHEMES = ["PoT", "INT", "SIG-1", "FP-1", "FP1", "FP-10", "FP-100", "Mix"]
ACC_FP32, ACC_FP16, ACC_GROUPED, ACC_PSUM_INT8, ACC_PSUM_E3M4 = range(5)


class _Fmt(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "kind", "ebit", "mbit", "sc_ebit", "sc_mbit", "block_size", "scale_allow_subnormal",
        "use_round", "use_ceil", "l2_block_size", "l2_sc_bit", "l2_scheme", "per_tensor_scale",
        "reserved")]


@dataclass
class Format:
    """Mirror of ``orc_format``; field meaning as the reference constructors
    (src/quantizer.py:348-357, 431-443, 709-725)."""
    kind: int
    ebit: int = 2
    mbit: int = 1
    sc_ebit: int = 5
    sc_mbit: int = 0
    block_size: int = 32
    scale_allow_subnormal: bool = False
    use_round: bool = False
    use_ceil: bool = False
    l2_block_size: int = 8
    l2_sc_bit: int = 2
    l2_scheme: str = "SIG-1"
    per_tensor_scale: bool = False

    def c(self) -> _Fmt:
        return _Fmt(self.kind, self.ebit, self.mbit, self.sc_ebit, self.sc_mbit, self.block_size,
                    int(self.scale_allow_subnormal), int(self.use_round), int(self.use_ceil),
                    self.l2_block_size, self.l2_sc_bit, L2_SCHEMES.index(self.l2_scheme),
                    int(self.per_tensor_scale), 0)


def build(force: bool = False) -> str:
    """Compile the oracle if the shared object is missing or older than its sources."""
    srcs = [os.path.join(_HERE, f) for f in ("hbq_oracle.c", "hbq_oracle.h")]
    stale = (not os.path.exists(_LIB_PATH)
             or any(os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs))
    if force or stale:
        subprocess.check_call(["make", "-B", "-C", _HERE, "libhbq_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with open("/proc/cpuinfo") as fh:
            if "f16c" not in fh.read():
                raise RuntimeError("the CPU oracle needs a host CPU with F16C")
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_quantize.restype = ctypes.c_int
        _lib.orc_gemm_rows.restype = ctypes.c_int
        _lib.orc_num_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _u16(x) -> np.ndarray:
    """fp16 values (numpy float16 array or torch fp16 tensor) -> contiguous uint16 bit patterns."""
    if hasattr(x, "detach"):
        x = x.detach().cpu().contiguous().numpy()
    x = np.ascontiguousarray(x)
    if x.dtype == np.float16:
        return x.view(np.uint16)
    if x.dtype == np.uint16:
        return x
    raise TypeError(f"fp16 input expected, got {x.dtype}")


def quantize(x, fmt: Format, want_codes: bool = True) -> dict:
    """Block quantize-dequantize ``x`` [rows, K] (fp16) along K.

    Returns numpy arrays: ``deq`` float16 [rows, K]; ``scale`` float16 [rows, nblk];
    ``l2`` uint8 [rows, nblk, block/l2_block] and ``scheme`` uint8 [rows, nblk] (HBQ; MXEx: ``l2`` is 1
    where the step-2 grid won; VSQ: ``l2`` [rows, nblk, 1] second-level scales, ``scale`` the row's first);
    ``codes`` uint8 [rows, nblk, block] (one element code per byte)."""
    xu = _u16(x)
    rows, K = xu.shape
    B = fmt.block_size
    nblk = -(-K // B)
    deq = np.empty((rows, K), np.uint16)
    scale = np.empty((rows, nblk), np.uint16)
    hbq = fmt.kind == KIND_HBQ
    l2 = None
    if hbq or fmt.kind == KIND_MXEX:
        l2 = np.zeros((rows, nblk, B // fmt.l2_block_size), np.uint8)
    elif fmt.kind == KIND_VSQ:
        l2 = np.zeros((rows, nblk, 1), np.uint8)
    scheme = np.zeros((rows, nblk), np.uint8) if hbq else None
    codes = np.zeros((rows, nblk, B), np.uint8) if want_codes and fmt.kind <= KIND_HBQ else None
    c = fmt.c()
    rc = lib().orc_quantize(_p(xu), ctypes.c_int64(rows), ctypes.c_int64(K), ctypes.byref(c),
                            _p(deq), _p(scale), _p(l2), _p(scheme), _p(codes))
    if rc != 0:
        raise ValueError(f"orc_quantize: unsupported format (rc={rc})")
    return {"deq": deq.view(np.float16), "scale": scale.view(np.float16), "l2": l2,
            "scheme": scheme, "codes": codes}


def fp_quant(x, ebit, mbit, allow_subnormal=True, use_ceil=False, elem_variant=True) -> np.ndarray:
    xu = _u16(x).reshape(-1)
    out = np.empty_like(xu)
    lib().orc_fp_quant(_p(xu), ctypes.c_int64(xu.size), ebit, mbit, int(allow_subnormal),
                       int(use_ceil), int(elem_variant), _p(out))
    return out.view(np.float16)


def floor_log2_h(x) -> np.ndarray:
    xu = _u16(x).reshape(-1)
    out = np.empty(xu.size, np.float32)
    lib().orc_floor_log2_h(_p(xu), ctypes.c_int64(xu.size), _p(out))
    return out


def gemm(A, B, mode: int, group_k: int = 0, group_n: int = 0, rows=None) -> np.ndarray:
    """Accumulation-model GEMM, A [M,K] @ B [K,N] -> float16 [M,N].  ``rows=(m0, m1)``
    computes only those rows of C (the others are left zero)."""
    Au, Bu = _u16(A), _u16(B)
    M, K = Au.shape
    K2, N = Bu.shape
    assert K == K2
    C = np.zeros((M, N), np.uint16)
    m0, m1 = rows if rows is not None else (0, M)
    rc = lib().orc_gemm_rows(_p(Au), _p(Bu), _p(C), ctypes.c_int64(M), ctypes.c_int64(N),
                             ctypes.c_int64(K), mode, group_k, group_n,
                             ctypes.c_int64(m0), ctypes.c_int64(m1))
    if rc != 0:
        raise ValueError(f"orc_gemm: bad arguments (rc={rc})")
    return C.view(np.float16)


def num_threads() -> int:
    return lib().orc_num_threads()


def use_all_cores() -> int:
    """Use every host core the process may run on (torchrun exports OMP_NUM_THREADS=1)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(int(n))
    return num_threads()
