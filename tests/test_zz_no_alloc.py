"""GPU: hbq_gemm_kn_noalloc, the GEMM entry point for callers that may not allocate device memory
(plugins inside a host framework's memory pool, servers with frozen allocations).  It keeps the
transposed operand in a fixed array inside the library, so this test checks, through the C ABI,
that it returns what hbq_gemm returns with caller-provided scratch -- on two calls in a row of
different shapes, because the array is shared and keeps the previous call's contents -- and that
it refuses operands beyond the array's size.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _call_both(M, N, K, mode, gk, gn, seed):
    from hbq_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = torch.randn(M, K, device="cuda", generator=g).half()
    B = (0.05 * torch.randn(K, N, device="cuda", generator=g)).half()
    c_ref = torch.empty(M, N, device="cuda", dtype=torch.float16)
    c_new = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16)
    ws_bytes = int(L.hbq_gemm_workspace_bytes(M, N, K, 0, mode, gk, gn))
    assert ws_bytes == N * K * 2, "shape should take the tensor-core path, which needs the scratch"
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    vp = ctypes.c_void_p
    _lib.check(L.hbq_gemm(vp(A.data_ptr()), vp(B.data_ptr()), vp(c_ref.data_ptr()), M, N, K, 0, mode, gk, gn,
                          None, vp(ws.data_ptr()), ws_bytes, stream), "hbq_gemm")
    _lib.check(L.hbq_gemm_kn_noalloc(vp(A.data_ptr()), vp(B.data_ptr()), vp(c_new.data_ptr()), M, N, K, mode, gk, gn,
                                     None, stream), "hbq_gemm_kn_noalloc")
    torch.cuda.synchronize()
    return c_ref, c_new


def test_noalloc_matches_gemm_two_calls_in_a_row():
    import hbq_b200 as H
    # same tolerance as the GEMM tests (relative Frobenius error <= 2^-9); equality is expected
    for (M, N, K, mode, gk, gn, seed) in [(192, 512, 1024, 3, 128, 32, 1), (96, 264, 2048, 2, 64, 0, 2)]:
        c_ref, c_new = _call_both(M, N, K, mode, gk, gn, seed)
        assert H.gemm_status() == 0
        r, n = c_ref.double(), c_new.double()
        assert torch.isfinite(n).all()
        rel = float((n - r).norm() / r.norm())
        assert rel <= 2.0 ** -9, rel
        assert torch.equal(c_ref.view(torch.int16), c_new.view(torch.int16))


def test_noalloc_rejects_operands_beyond_its_scratch():
    from hbq_b200 import _lib
    L = _lib.lib()
    N, K = 4096, 2048                      # N*K = 2 * HBQ_GEMM_NOALLOC_MAX_ELEMS
    assert N * K > _lib.GEMM_NOALLOC_MAX_ELEMS
    A = torch.zeros(8, K, device="cuda", dtype=torch.float16)
    B = torch.zeros(K, N, device="cuda", dtype=torch.float16)
    C = torch.zeros(8, N, device="cuda", dtype=torch.float16)
    vp = ctypes.c_void_p
    rc = L.hbq_gemm_kn_noalloc(vp(A.data_ptr()), vp(B.data_ptr()), vp(C.data_ptr()), 8, N, K, 0, 0, 0, None, None)
    assert rc == -7
    assert b"HBQ_GEMM_NOALLOC_MAX_ELEMS" in L.hbq_error_string(rc)
