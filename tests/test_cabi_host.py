"""CPU: the C-ABI library loads and exports every symbol include/hbq_b200.h declares; host-side
logic (YAML mapping, argument checks, closed forms used by the kernels) without touching a GPU."""
import os
import re

import numpy as np
import pytest

from util import bits, load_npz

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from hbq_b200 import _lib
    from hbq_b200.build import build_library
    build_library()
    hdr = open(os.path.join(ROOT, "include", "hbq_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(hbq_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    L = _lib.lib()
    missing = [n for n in sorted(declared) if not hasattr(L, n)]
    assert not missing, missing
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    assert L.hbq_version() >= 100
    assert L.hbq_error_string(-2).decode().startswith("format or shape")
    # shape rules of the GEMM dispatcher, no launch involved
    assert L.hbq_gemm_uses_tensor_cores(4096, 14336, 4096, 1, 3, 128, 32) == 1
    assert L.hbq_gemm_uses_tensor_cores(4096, 14336, 4096, 1, 1, 0, 0) == 0       # pure fp16 chain
    assert L.hbq_gemm_uses_tensor_cores(100, 50, 333, 1, 2, 128, 0) == 0          # unaligned K, N
    assert L.hbq_gemm_workspace_bytes(8, 64, 128, 0, 2, 64, 0) == 64 * 128 * 2
    assert L.hbq_gemm_workspace_bytes(8, 64, 128, 1, 2, 64, 0) == 0
    assert L.hbq_absmax_scratch_bytes() > 0
    # packed-weight GEMM: one 9216-byte record per (128 rows, 128 k); other shapes are not served
    assert L.hbq_gemm_w4_prepacked_bytes(14336, 4096, 4) == 14336 * 4096 * 9216 // (128 * 128) == 33030144
    assert L.hbq_gemm_w4_prepacked_bytes(14336, 4096, 8) == 14336 * 4096 * 17408 // (128 * 128)
    assert L.hbq_gemm_w4_prepacked_bytes(14336, 4000, 4) == -1 and L.hbq_gemm_w4_prepacked_bytes(100, 4096, 4) == -1
    assert L.hbq_gemm_w4_prepacked_bytes(14336, 4096, 5) == -1
    assert L.hbq_gemm_w4_workspace_bytes(129, 4096, 4096) == -1 and L.hbq_gemm_w4_workspace_bytes(0, 4096, 4096) == -1


def test_no_cpu_fallback():
    torch = pytest.importorskip("torch")
    import hbq_b200 as H
    with pytest.raises(H.HbqError):
        H.HBQQuantizer().q(torch.zeros(2, 128, dtype=torch.float16))
    with pytest.raises(RuntimeError):
        H.blockquant_ext.gemm_fp32_accum(torch.zeros(2, 8, dtype=torch.float16), torch.zeros(8, 4, dtype=torch.float16))
    for q in (H.MXExQuantizer(), H.VSQQuantizer(4), H.MXFPQuantizer(), H.MXINTQuantizer(8)):
        with pytest.raises(H.HbqError):
            q.q(torch.zeros(2, 64, dtype=torch.float16))
    with pytest.raises(H.HbqError):
        H.write_k_cache(torch.zeros(1, 4, 256, dtype=torch.float16), 2, H.HBQQuantizer())
    with pytest.raises(H.HbqError):
        H.write_v_cache(torch.zeros(1, 4, 256, dtype=torch.float16), 2, H.HBQQuantizer())


def test_kvcache_argument_checks():
    torch = pytest.importorskip("torch")
    from hbq_b200 import kvcache
    x = torch.arange(8, dtype=torch.float16).view(1, 1, 1, 8)
    assert kvcache.rotate_half(x).flatten().tolist() == [-4, -5, -6, -7, 0, 1, 2, 3]
    with pytest.raises(ValueError):
        kvcache._head_dim(torch.zeros(1, 4, 250), 4)                 # H does not divide the last axis
    assert kvcache._head_dim(torch.zeros(2, 4, 8, 16), 8) == 16 and kvcache._head_dim(torch.zeros(2, 4, 128), 8) == 16
    cos = torch.zeros(1, 4, 16)
    with pytest.raises(ValueError):
        kvcache._tables(cos, torch.zeros(1, 4, 8), 2, 4, 16)         # cos / sin shapes differ
    with pytest.raises(ValueError):
        kvcache._tables(torch.zeros(3, 4, 16), torch.zeros(3, 4, 16), 2, 4, 16)   # batch neither 1 nor B
    assert kvcache._tables(cos, cos, 2, 4, 16)[2] == 4 and kvcache._tables(cos.expand(2, 4, 16), cos.expand(2, 4, 16), 2, 4, 16)[2] == 8


HBQ_E_PSUM_YAML = """
quantization: {xqtype: hbq, wqtype: hbq, quant_4b_kv: True, quant_k_cache: True}
block_quant:
  act_ebit: 2
  act_mbit: 2
  act_block_size: 128
  act_sc_ebit: 5
  act_sc_mbit: 3
  wgt_ebit: 2
  wgt_mbit: 1
  wgt_block_size: 128
  wgt_sc_ebit: 5
  wgt_sc_mbit: 3
  wgt_l2_sc_bit: 2
  wgt_l2_block_size: 32
  wgt_l2_scheme: "Mix"
  act_l2_sc_bit: 2
  act_l2_block_size: 32
  act_l2_scheme: "SIG-1"
  scale_allow_subnormal: False
accumulation: {type: fp16_quant, group_size: 128, quant_block_size: 32}
"""


def test_ptq_config_mapping():
    """YAML keys and defaults of the reference's PTQ (src/ptq.py:40-105, 107-257, 384-404)."""
    yaml = pytest.importorskip("yaml")
    import hbq_b200 as H
    cfg = H.PTQConfig(yaml.full_load(HBQ_E_PSUM_YAML))
    a, w, kv = cfg.map_act_quantizer(), cfg.map_wgt_quantizer(), cfg.map_kv_quantizer()
    assert isinstance(a, H.HBQQuantizer) and (a.ebit, a.mbit, a.l2_block_size, a.l2_scheme) == (2, 2, 32, "SIG-1")
    assert (w.ebit, w.mbit, w.l2_scheme, w.block_size) == (2, 1, "Mix", 128)
    assert (kv.ebit, kv.mbit, kv.l2_scheme, kv.block_size) == (2, 1, "SIG-1", 128)   # KV4 with the act settings
    op = cfg.make_accum_op()
    assert isinstance(op, H.FP16AccumMatMul) and (op.group_size, op.quant_block_size) == (128, 32)
    d = H.PTQConfig({"quantization": {"xqtype": "mxfp", "wqtype": "mxint"}})
    assert d.scale_allow_subnormal is True and d.accumulation_group_size == 128 and d.make_accum_op() is None
    assert isinstance(d.map_act_quantizer(use_round=True), H.MXFPQuantizer) and d.map_act_quantizer(True).use_round
    assert isinstance(d.map_wgt_quantizer(), H.MXINTQuantizer)
    with pytest.raises(ValueError):
        H.PTQConfig({"quantization": {"xqtype": "none", "wqtype": "none"}, "accumulation": {"type": "int4"}}).make_accum_op()
    assert H.get_max_norm(2, 2) == 7 and H.get_max_norm(4, 3) == 448 and H.get_max_norm(0, 8) == 127
    assert H.get_min_norm(5, 3) == 2 ** -14 and H.get_min_subnorm(2, 1) == 0.5


def _rn16(x):
    return np.asarray(x, np.float64).astype(np.float16)


def test_kernel_closed_forms_against_reference_tables():
    """numpy restatement of the bit tricks the kernels use, over all fp16 inputs, against the tables
    produced by the reference: E2Mx = integer round-half-up above 1, one fp16 FMA + floor below;
    E5M3 scale = round-half-up on the pattern."""
    ex = load_npz("exhaustive.npz")
    allb = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    fin = ex["finite"]
    u = allb[fin]
    a = u & 0x7FFF
    av = a.view(np.float16).astype(np.float64)
    for mb in (1, 2, 3, 5):
        half, mask = 0x0200 >> mb, 0xFFFF ^ ((0x0400 >> mb) - 1)
        mx = 0x4400 | (((1 << mb) - 1) << (10 - mb))
        n = np.minimum((a.astype(np.uint32) + half) & mask, mx).astype(np.uint16)
        w = _rn16(av * (1 << mb) + 0.50048828125)
        s = _rn16(np.floor(w.astype(np.float64)) / (1 << mb)).view(np.uint16)
        if mb == 1:
            s = np.where(a == 0x39FF, 0, s).astype(np.uint16)
        r = np.where(a >= 0x3C00, n, s).astype(np.uint16)
        r = r | np.where(a != 0, u & 0x8000, 0).astype(np.uint16)
        assert np.array_equal(r, ex[f"elem_e2m{mb}"]), f"E2M{mb}"
    # E5M3 scale after the clip to [2^-14, 61440]
    pos = (u & 0x8000) == 0
    sb = np.clip(u[pos].astype(np.uint32), 0x0400, 0x7B80)
    got = ((sb + 0x40) & 0xFF80).astype(np.uint16)
    clipped = np.clip(u[pos].view(np.float16).astype(np.float64), 2.0 ** -14, 61440.0).astype(np.float16).view(np.uint16)
    idx = {int(k): i for i, k in enumerate(u)}
    ref = ex["scale_e5m3_ceil0_sub0"][[idx[int(c)] for c in clipped]]
    assert np.array_equal(got, ref)


def test_reciprocal_division_is_exact():
    """x / s rounded to fp16 equals fp16(fp32(x) * fp32(1/s)) for every fp16 x and E5M3 scale s in range,
    and for the micro-scale tables (the identity the kernels rely on instead of dividing)."""
    x = np.arange(0x0400, 0x7C00, dtype=np.uint16).view(np.float16).astype(np.float32)
    scales = [np.float32((1 + m / 8) * 2.0 ** e) for e in (-14, -3, 0, 5, 11) for m in range(8)]
    scales += [np.float32(t) for t in (1.5, 2.5, 1.25, 1.75, 1.125, 1.375, 3, 5, 7, 17.5, 10.5, 8.25)]
    for s in scales:
        exact = (x.astype(np.float64) / np.float64(s)).astype(np.float16)
        fast = (x * (np.float32(1) / s)).astype(np.float16)
        keep = exact.astype(np.float64) >= 2.0 ** -14          # subnormal quotients always quantise to 0
        assert np.array_equal(bits(exact[keep]), bits(fast[keep])), s


def test_packed_weight_wrapper_without_a_gpu():
    """Host side of the packed-weight GEMM: CPU tensors and shapes outside the kernel are reported as not served, and
    nothing falls back to a CPU product."""
    torch = pytest.importorskip("torch")
    import hbq_b200 as H
    from hbq_b200 import _lib
    fmt = _lib.Format(_lib.KIND_HBQ, 2, 1, 5, 3, 128, 0, 0, 0, 8, 2, _lib.L2_SCHEMES.index("Mix"), 0, 0)
    u8 = lambda *shape: torch.zeros(shape, dtype=torch.uint8)
    packed = H.PackedTensor(torch.Size((256, 256)), torch.float16, fmt, u8(256, 128), None, u8(256, 2), u8(256, 2, 4), u8(256, 2))
    assert not H.W4Weight.supported(packed)                       # planes on the host
    lin = H.QLinear(256, 256, bias=False)
    assert not lin.prepare_decode() and lin.w4_weight is None     # CPU layer: unchanged

