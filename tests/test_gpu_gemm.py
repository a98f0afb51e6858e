"""GPU: GEMM with modelled accumulation.  The CUDA-core kernel follows the reference's own
summation order and must equal the CPU oracle bit for bit; the tcgen05 kernel sums each K-chunk
in tensor memory and is held to a stated tolerance against both."""
import numpy as np
import pytest

from util import bits, load_formats, make_quantizer, seeded_inputs

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

# Tolerance of the tensor-core path against the sequential-fp32 model of the reference
# (gemm.cu): the chunk sums may differ in the last fp32 bits, which can move an fp16 / INT8
# rounding of a chunk by one step.  Stated bound: relative Frobenius error <= 2^-9 and at most
# 1% of the outputs differing by more than 2 fp16 ulps.
REL_FRO_TOL = 2.0 ** -9
FAR_ULP_FRACTION = 0.01


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def compare(got, ref, what):
    g = got.astype(np.float64)
    r = ref.astype(np.float64)
    rel = np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30)
    mism = int((bits(got) != bits(ref)).sum())
    # fp16 patterns on a monotone integer line (negative values mirrored), so that differences count ulps
    gl, rl = bits(got).astype(np.int32), bits(ref).astype(np.int32)
    gl, rl = np.where(gl & 0x8000, -(gl & 0x7FFF), gl), np.where(rl & 0x8000, -(rl & 0x7FFF), rl)
    ulp = np.abs(gl - rl)
    far = float((ulp > 2).mean())
    print(f"{what}: mismatches {mism}/{ref.size}, rel_fro {rel:.3e}, >2ulp {far:.2e}")
    assert rel <= REL_FRO_TOL, f"{what}: relative Frobenius error {rel}"
    assert far <= FAR_ULP_FRACTION, f"{what}: {far:.3%} of the outputs are more than 2 fp16 ulps away"
    return mism


MODES = [("fp32", 0, 0, 0), ("fp16", 1, 0, 0), ("grouped", 2, 32, 0), ("grouped", 2, 128, 0),
         ("int8", 3, 64, 8), ("int8", 3, 128, 32), ("e3m4", 4, 64, 16)]


@pytest.mark.parametrize("shape", [(70, 72, 200), (128, 256, 256), (33, 40, 128)])
@pytest.mark.parametrize("mode", MODES, ids=lambda m: f"{m[0]}-{m[2]}-{m[3]}")
def test_simt_equals_oracle(oracle, shape, mode):
    """Sequential-fp32 CUDA-core kernel == CPU oracle, bit for bit, including edge tiles."""
    import hbq_b200 as H
    M, N, K = shape
    _, m, gk, gn = mode
    if m >= 3 and N % gn:
        pytest.skip("N must divide into group_n")
    rng = np.random.default_rng(M * 7 + K)
    A = rng.standard_normal((M, K)).astype(np.float16)
    B = (0.05 * rng.standard_normal((K, N))).astype(np.float16)
    ref = oracle.gemm(A, B, m, gk, gn)
    got = H.gemm(dev(A), dev(B), m, gk, gn, force_simt=True).cpu().numpy()
    assert np.array_equal(bits(got), bits(ref)), f"{(bits(got) != bits(ref)).sum()} mismatches"
    got2 = H.gemm(dev(A), dev(np.ascontiguousarray(B.T)), m, gk, gn, b_is_nk=True, force_simt=True).cpu().numpy()
    assert np.array_equal(bits(got2), bits(ref))


@pytest.mark.parametrize("shape", [(128, 256, 256), (200, 520, 384), (64, 264, 1024), (300, 256, 72)])
@pytest.mark.parametrize("mode", [m for m in MODES if m[1] != 1], ids=lambda m: f"{m[0]}-{m[2]}-{m[3]}")
def test_tensor_core_vs_oracle_small(oracle, shape, mode):
    """tcgen05 kernel on small and ragged shapes (M, N edge tiles; K not a multiple of 64)."""
    import hbq_b200 as H
    from hbq_b200 import _lib
    M, N, K = shape
    _, m, gk, gn = mode
    assert _lib.lib().hbq_gemm_uses_tensor_cores(M, N, K, 1, m, gk, gn) == 1
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float16)
    W = (0.05 * rng.standard_normal((N, K))).astype(np.float16)
    ref = oracle.gemm(A, np.ascontiguousarray(W.T), m, gk, gn)
    got = H.gemm(dev(A), dev(W), m, gk, gn, b_is_nk=True)
    torch.cuda.synchronize()
    assert H.gemm_status() == 0, "a bounded wait expired inside the tensor-core kernel"
    compare(got.cpu().numpy(), ref, f"tc {mode[0]} {shape}")
    # B given as [K, N] (the reference extension's layout): transposed into the workspace first
    got_kn = H.gemm(dev(A), dev(np.ascontiguousarray(W.T)), m, gk, gn)
    assert torch.equal(got_kn.view(torch.int16), got.view(torch.int16))


@pytest.mark.parametrize("mode", [m for m in MODES if m[1] != 1], ids=lambda m: f"{m[0]}-{m[2]}-{m[3]}")
def test_tensor_core_exact_on_integer_operands(oracle, mode):
    """Small-integer operands make every chunk sum exact in fp32 whatever the summation order, so the
    tensor-core kernel must equal the oracle bit for bit: this pins the epilogue arithmetic itself
    (scales, ties-to-even rounding, the +-127 clamp of the INT8 partial sums, the E3M4 grid)."""
    import hbq_b200 as H
    _, m, gk, gn = mode
    M, N, K = 256, 512, 512
    rng = np.random.default_rng(99)
    Ai = rng.integers(-8, 9, size=(M, K))
    Wi = rng.integers(-8, 9, size=(N, K))
    if m == 3:
        # the case the clamp exists for: a partial sum that rounds to 128 steps of its group's scale
        g = gk
        hits = 0
        for c in range(K // g):
            ps = Ai[:, c * g:(c + 1) * g] @ Wi[:, c * g:(c + 1) * g].T
            mx = np.abs(ps).reshape(M, N // gn, gn).max(axis=2)
            scale = 2.0 ** (np.floor(np.log2(np.maximum(mx, 1))) - 6)
            hits += int((np.rint(mx / scale) == 128).sum())
        assert hits > 0, "inputs do not exercise the clamp"
    A = Ai.astype(np.float16)
    W = Wi.astype(np.float16)
    ref = oracle.gemm(A, np.ascontiguousarray(W.T), m, gk, gn)
    got = H.gemm(dev(A), dev(W), m, gk, gn, b_is_nk=True)
    torch.cuda.synchronize()
    assert H.gemm_status() == 0
    assert np.array_equal(bits(got.cpu().numpy()), bits(ref)), mode


def _hbq_operands(M, N, K, seed):
    """HBQ-E fake-quantised activation and weight (the operands of the benchmark GEMM)."""
    f = load_formats()
    xa = dev(seeded_inputs("act", M, K, seed))
    w = dev(seeded_inputs("wgt", N, K, seed + 1))
    return make_quantizer(f["hbq_e_act"]).q(xa), make_quantizer(f["hbq_e_wgt"]).q(w)


@pytest.mark.parametrize("mode", [("grouped", 2, 128, 0), ("int8", 3, 128, 32), ("fp32", 0, 0, 0)],
                         ids=lambda m: m[0])
def test_tensor_core_hbq_operands(oracle, mode):
    """HBQ-E operands, K = 4096: tensor-core kernel vs the exact-order kernel and the oracle."""
    import hbq_b200 as H
    _, m, gk, gn = mode
    M, N, K = 256, 512, 4096
    xq, wq = _hbq_operands(M, N, K, 11)
    tc = H.gemm(xq, wq, m, gk, gn, b_is_nk=True)
    simt = H.gemm(xq, wq, m, gk, gn, b_is_nk=True, force_simt=True)
    torch.cuda.synchronize()
    assert H.gemm_status() == 0
    ref = oracle.gemm(xq.cpu().numpy()[:64], np.ascontiguousarray(wq.cpu().numpy().T), m, gk, gn)
    assert np.array_equal(bits(simt.cpu().numpy()[:64]), bits(ref))
    compare(tc.cpu().numpy(), simt.cpu().numpy(), f"tc vs exact-order, HBQ-E operands, {mode[0]}")


def test_full_size_linearity_and_bias():
    """M=4096, K=4096, N=14336 (the benchmark shape): properties that need no CPU reference.
    fp32 mode is linear in A up to fp16 output rounding; rows are independent; bias is added."""
    import hbq_b200 as H
    M, N, K = 4096, 14336, 4096
    xq, wq = _hbq_operands(M, N, K, 3)
    y = H.gemm(xq, wq, 3, 128, 32, b_is_nk=True)
    torch.cuda.synchronize()
    assert H.gemm_status() == 0
    assert torch.isfinite(y).all()
    # rows are independent: a row subset gives the same rows
    ysub = H.gemm(xq[1000:1128].contiguous(), wq, 3, 128, 32, b_is_nk=True)
    assert torch.equal(ysub.view(torch.int16), y[1000:1128].view(torch.int16))
    # column subset on a group_n boundary gives the same columns (column-parallel sharding)
    ycol = H.gemm(xq, wq[7168:7168 + 1792].contiguous(), 3, 128, 32, b_is_nk=True)
    assert torch.equal(ycol.view(torch.int16), y[:, 7168:7168 + 1792].contiguous().view(torch.int16))
    # against the exact-order kernel on a sample of rows
    ys = H.gemm(xq[:128].contiguous(), wq, 3, 128, 32, b_is_nk=True, force_simt=True)
    compare(y[:128].cpu().numpy(), ys.cpu().numpy(), "full-size int8 psum, rows 0..127")
    # power-of-two scaling of A scales the result exactly (all models are scale-equivariant)
    y2 = H.gemm((xq * 2).contiguous(), wq, 3, 128, 32, b_is_nk=True)
    assert torch.equal((y * 2).view(torch.int16), y2.view(torch.int16))
    bias = torch.randn(N, device="cuda").half()
    yb = H.gemm(xq[:256].contiguous(), wq, 2, 128, 0, bias=bias, b_is_nk=True)
    y0 = H.gemm(xq[:256].contiguous(), wq, 2, 128, 0, b_is_nk=True)
    assert torch.equal(yb.view(torch.int16), (y0 + bias).view(torch.int16))


def test_ops_and_extension_api():
    """FP16AccumMatMul and the blockquant_ext functions keep the reference's argument checks."""
    import hbq_b200 as H
    ext = H.blockquant_ext
    A = torch.randn(64, 256, device="cuda").half()
    B = torch.randn(256, 96, device="cuda").half()
    for fn, args in [(ext.gemm_fp32_accum, ()), (ext.gemm_fp16_accum, ()), (ext.gemm_fp16_grouped_accum, (64,)),
                     (ext.gemm_blockquant_mxfp8, (64, 16)), (ext.gemm_blockquant_mxint8, (128, 32))]:
        c = fn(A, B, *args)
        assert c.shape == (64, 96) and c.dtype == torch.float16 and c.is_cuda
    with pytest.raises(RuntimeError):
        ext.gemm_fp16_grouped_accum(A, B, 8)
    with pytest.raises(RuntimeError):
        ext.gemm_blockquant_mxint8(A, B, 32, 32)
    with pytest.raises(RuntimeError):
        ext.gemm_fp32_accum(A.float(), B)
    with pytest.raises(RuntimeError):
        ext.gemm_fp32_accum(A, B[:100])
    op = H.FP16AccumMatMul(group_size=128, quant_block_size=32)
    x = torch.randn(2, 8, 256, device="cuda").half()
    w = torch.randn(96, 256, device="cuda").half() * 0.05
    b = torch.randn(96, device="cuda").half()
    y = op(x, w, b)
    assert y.shape == (2, 8, 96)
    ref = ext.gemm_blockquant_mxint8(x.view(-1, 256), w.t().contiguous(), 128, 32) + b
    assert torch.equal(y.view(-1, 96).view(torch.int16), ref.view(torch.int16))
    with pytest.raises(ValueError):
        H.FP16AccumMatMul(group_size=48)(x, w)
    with pytest.raises(ValueError):
        H.FP16AccumMatMul(group_size=128, quant_block_size=64)(x, w)


def test_qlinear_layer(oracle):
    """One HBQ-A linear layer (X [2048,4096]-style input with outlier channels, W ~ N(0, 0.02)):
    quantizers + fp32-accumulate GEMM against the oracle's quantizers and an fp32 matmul."""
    import hbq_b200 as H
    f = load_formats()
    M, K, N = 512, 1024, 768
    x = seeded_inputs("act", M, K, 21)
    w = seeded_inputs("wgt", N, K, 22)
    cfg = H.PTQConfig({"quantization": {"xqtype": "hbq", "wqtype": "hbq"},
                       "block_quant": {"act_ebit": 2, "act_mbit": 2, "act_block_size": 128, "act_sc_ebit": 5,
                                       "act_sc_mbit": 3, "wgt_ebit": 2, "wgt_mbit": 1, "wgt_block_size": 128,
                                       "wgt_sc_ebit": 5, "wgt_sc_mbit": 3, "wgt_l2_sc_bit": 2, "wgt_l2_block_size": 8,
                                       "wgt_l2_scheme": "Mix", "act_l2_sc_bit": 2, "act_l2_block_size": 8,
                                       "act_l2_scheme": "SIG-1", "scale_allow_subnormal": False},
                       "accumulation": {"type": "fp32"}})
    lin = H.QLinear(K, N, bias=False, device="cuda", dtype=torch.float16)
    lin.weight.data = dev(w)
    cfg.apply_to_linear(lin)
    from util import oracle_format
    wq = oracle.quantize(w, oracle_format(oracle, f["hbq_a_wgt"]), False)["deq"]
    xq = oracle.quantize(x, oracle_format(oracle, f["hbq_a_act"]), False)["deq"]
    assert np.array_equal(bits(lin.weight.data.cpu().numpy()), bits(wq))
    with torch.no_grad():
        y = lin(dev(x)).float().cpu().numpy()
    ref = xq.astype(np.float32) @ wq.astype(np.float32).T
    rel = np.linalg.norm(y - ref) / np.linalg.norm(ref)
    assert rel < 1e-3, rel


@pytest.mark.parametrize("K", [384, 320, 256])
@pytest.mark.parametrize("mode", [("grouped", 2, 128, 0), ("int8", 3, 128, 32), ("grouped64", 2, 64, 0), ("fp32", 0, 0, 0)],
                         ids=lambda m: m[0])
def test_tensor_core_several_tiles_per_cta(oracle, K, mode):
    """156 output tiles on 148 SMs: some CTAs run two tiles back to back, with an odd number of
    chunks per tile (K = 384: the two MMA-issuing warps swap accumulators from tile to tile), a
    ragged last chunk (K = 320: one issuing warp) and an even count (K = 256)."""
    import hbq_b200 as H
    M, N = 128 * 13, 256 * 12
    _, m, gk, gn = mode
    rng = np.random.default_rng(K)
    A = rng.standard_normal((M, K)).astype(np.float16)
    W = (0.05 * rng.standard_normal((N, K))).astype(np.float16)
    ref = oracle.gemm(A, np.ascontiguousarray(W.T), m, gk, gn)
    got = H.gemm(dev(A), dev(W), m, gk, gn, b_is_nk=True)
    torch.cuda.synchronize()
    assert H.gemm_status() == 0, "a bounded wait expired inside the tensor-core kernel"
    compare(got.cpu().numpy(), ref, f"tc {mode[0]} K={K}")


def test_output_quantizer_roles():
    """quant_before_* switches give the named projections an output quantizer (src/ptq.py:287-324)."""
    import hbq_b200 as H
    cfg = H.PTQConfig({"quantization": {"xqtype": "mxfp", "wqtype": "mxfp", "quant_before_rms_norm": True},
                       "block_quant": {"act_ebit": 2, "act_mbit": 1, "act_sc_ebit": 5, "act_sc_mbit": 0, "act_block_size": 32,
                                       "wgt_ebit": 2, "wgt_mbit": 1, "wgt_sc_ebit": 5, "wgt_sc_mbit": 0, "wgt_block_size": 32,
                                       "scale_allow_subnormal": False},
                       "accumulation": {"type": "fp32"}})
    K, N = 256, 128
    x = dev(seeded_inputs("act", 64, K, 41))

    def layer(role):
        lin = H.QLinear(K, N, bias=False, device="cuda", dtype=torch.float16)
        lin.weight.data = dev(seeded_inputs("wgt", N, K, 42))
        return cfg.apply_to_linear(lin, role=role)

    down, gate = layer("down_proj"), layer("gate_proj")
    assert isinstance(down.yq, H.MXFPQuantizer) and not isinstance(gate.yq, H.MXFPQuantizer)
    with torch.no_grad():
        assert torch.equal(down(x), down.yq.q(gate(x)))
    with pytest.raises(ValueError):
        layer("nonsense")


def test_cuda_graph_capture_of_the_layer():
    """Quantize + GEMM make no allocation or synchronisation of their own, so a layer step can be
    captured in a CUDA graph and replayed on new input."""
    import hbq_b200 as H
    M, K, N = 256, 512, 512
    aq = H.HBQQuantizer(128, 2, 2, 5, 3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")
    lin = H.QLinear(K, N, bias=False, device="cuda", dtype=torch.float16, check_finite=False)
    lin.weight.data = dev(seeded_inputs("wgt", N, K, 61))
    lin.aq = aq
    lin.ops = H.FP16AccumMatMul(group_size=128, quant_block_size=32)
    x_static = dev(seeded_inputs("act", M, K, 62))
    with torch.no_grad():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                lin(x_static)                         # warm-up: table plans, kernel attributes, allocator pools
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y_static = lin(x_static)
        for seed in (63, 64):
            x_new = dev(seeded_inputs("act", M, K, seed))
            x_static.copy_(x_new)
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(y_static, lin(x_new))
    assert H.gemm_status() == 0


def test_packed_weight_storage(tmp_path):
    """A layer's weight survives pack -> torch.save -> load -> unpack bit for bit, at its packed size."""
    import hbq_b200 as H
    K, N = 512, 256
    w = dev(seeded_inputs("wgt", N, K, 51))
    wq = H.HBQQuantizer(128, 2, 1, 5, 3, l2_block_size=8, l2_sc_bit=2, l2_scheme="Mix")
    lin = H.QLinear(K, N, bias=False, device="cuda", dtype=torch.float16)
    lin.weight.data = w.clone()
    lin.wq = wq
    p = lin.pack_weight()
    assert torch.equal(lin.weight.data, wq.q(w))
    assert p.nbytes() < 0.56 * w.numel()
    path = tmp_path / "w.pt"
    torch.save(p.state_dict(), path)
    lin2 = H.QLinear(K, N, bias=False, device="cuda", dtype=torch.float16)
    lin2.load_packed_weight(torch.load(path))
    assert torch.equal(lin2.weight.data, lin.weight.data)
    with pytest.raises(ValueError):
        H.QLinear(K, N + 8, bias=False, device="cuda", dtype=torch.float16).load_packed_weight(p)


def test_qlinear_forward_host_matches_forward():
    """The pipelined host-buffer entry (chunked copies and kernels on three streams) returns exactly
    what forward() returns for the same rows, for ragged row counts, repeated calls and wait=False."""
    import hbq_b200 as H
    M, K, N = 1000, 512, 384
    x = torch.from_numpy(seeded_inputs("act", M, K, 31)).to(torch.bfloat16)
    w = seeded_inputs("wgt", N, K, 32)
    aq = H.HBQQuantizer(128, 2, 2, 5, 3, l2_block_size=32, l2_sc_bit=2, l2_scheme="FP-1")
    aq.out_dtype = torch.float16
    lin = H.QLinear(K, N, bias=True, device="cuda", dtype=torch.float16, check_finite=False)
    lin.weight.data = dev(w)
    lin.bias.data = torch.linspace(-1, 1, N, device="cuda", dtype=torch.float16)
    lin.aq = aq
    lin.ops = H.FP16AccumMatMul(group_size=128, quant_block_size=32)
    with torch.no_grad():
        want = lin(x.cuda()).cpu()
        xp = x.pin_memory()
        for chunks in (1, 2, 3, 8):
            got = lin.forward_host(xp, row_chunks=chunks)      # wait=True: readable on return
            assert torch.equal(got, want), chunks
        out = torch.empty((M, N), dtype=torch.float16).pin_memory()
        ev = None
        for _ in range(3):
            _, ev = lin.forward_host(xp, out, row_chunks=2, wait=False)
        ev.synchronize()
        assert torch.equal(out, want)
        assert lin.forward_host(xp[:0]).shape == (0, N)


def _load_reference_ext():
    """The reference's own extension compiled by oracle/build_ref.py, if it has been built."""
    import importlib.util
    import os
    so = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "blockquant_ext.so")
    if not os.path.exists(so):
        return None
    spec = importlib.util.spec_from_file_location("blockquant_ext", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_against_reference_extension():
    """Both kernels against the reference's gemm.cu itself (rebuilt for sm_100a, run on this GPU)
    on HBQ-E operands: the exact-order kernel must match bit for bit, the tensor-core kernel
    within the stated tolerance."""
    import hbq_b200 as H
    ref_ext = _load_reference_ext()
    if ref_ext is None:
        pytest.skip("oracle/_ref/blockquant_ext.so not built")
    M, N, K = 512, 1024, 4096
    xq, wq = _hbq_operands(M, N, K, 31)
    wt = wq.t().contiguous()
    cases = [("grouped", lambda: ref_ext.gemm_fp16_grouped_accum(xq, wt, 128), (2, 128, 0)),
             ("int8", lambda: ref_ext.gemm_blockquant_mxint8(xq, wt, 128, 32), (3, 128, 32)),
             ("fp32", lambda: ref_ext.gemm_fp32_accum(xq, wt), (0, 0, 0)),
             ("fp16", lambda: ref_ext.gemm_fp16_accum(xq, wt), (1, 0, 0)),
             ("e3m4", lambda: ref_ext.gemm_blockquant_mxfp8(xq, wt, 128, 32), (4, 128, 32))]
    for name, fn, (m, gk, gn) in cases:
        torch.cuda.synchronize()
        ref = fn()
        torch.cuda.synchronize()           # the reference launches on the legacy default stream
        simt = H.gemm(xq, wq, m, gk, gn, b_is_nk=True, force_simt=True)
        mism = int((simt.view(torch.int16) != ref.view(torch.int16)).sum())
        if name == "e3m4":
            # the reference build uses fast-math division / log2 in this path: tolerance, not bits
            compare(simt.cpu().numpy(), ref.cpu().numpy(), "exact-order vs reference gemm.cu, e3m4")
        else:
            assert mism == 0, f"{name}: exact-order kernel differs from the reference in {mism} outputs"
        if m != 1:
            tc = H.gemm(xq, wq, m, gk, gn, b_is_nk=True)
            torch.cuda.synchronize()
            assert H.gemm_status() == 0
            compare(tc.cpu().numpy(), ref.cpu().numpy(), f"tensor-core vs reference gemm.cu, {name}")


def test_out_argument_and_reserved_sms():
    """`out=` writes into the caller's tensor; leaving SMs free for a neighbouring kernel changes the
    persistent grid, not the result."""
    import hbq_b200 as H
    from hbq_b200.gemm import gemm_reserve_sms
    M, N, K = 1500, 2048, 512
    a = torch.randn((M, K), device="cuda").half()
    w = (0.05 * torch.randn((N, K), device="cuda")).half()
    y0 = H.gemm(a, w, 3, 128, 32, b_is_nk=True)
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    y1 = H.gemm(a, w, 3, 128, 32, b_is_nk=True, out=out)
    assert y1.data_ptr() == out.data_ptr() and torch.equal(out.view(torch.int16), y0.view(torch.int16))
    prev = gemm_reserve_sms(40)
    try:
        y2 = H.gemm(a, w, 3, 128, 32, b_is_nk=True)
        assert gemm_reserve_sms(10 ** 6) == 40                 # more than the device has: one CTA does everything
        y3 = H.gemm(a[:256].contiguous(), w, 0, b_is_nk=True)
    finally:
        gemm_reserve_sms(prev)
    torch.cuda.synchronize()
    assert H.gemm_status() == 0
    assert torch.equal(y2.view(torch.int16), y0.view(torch.int16))
    assert torch.equal(y3.view(torch.int16), H.gemm(a[:256].contiguous(), w, 0, b_is_nk=True).view(torch.int16))
    with pytest.raises(RuntimeError):
        H.gemm(a, w, 3, 128, 32, b_is_nk=True, out=out[:, :100])
    op = H.FP16AccumMatMul(group_size=128, quant_block_size=32)
    buf = torch.empty((M, N), dtype=torch.float16, device="cuda")
    assert torch.equal(op(a, w, None, out=buf).view(torch.int16), y0.view(torch.int16))


def test_bounded_wait_runs_out_and_the_kernel_returns():
    """The give-up path of the tensor-core kernel, without faulting anything: its loader is switched off
    (nothing is ever in flight) and the wait bound lowered, so every wait runs out, every role leaves, tensor
    memory is freed and the kernel returns; the status word names the wait, QLinear's guard reports it,
    the reset clears it, and the next normal GEMM is bit-equal to the one before."""
    import hbq_b200 as H
    from hbq_b200.gemm import gemm_wait_selftest
    M, N, K = 512, 1024, 512
    a = torch.randn((M, K), device="cuda").half()
    w = (0.05 * torch.randn((N, K), device="cuda")).half()
    H.gemm_status_reset()
    before = {m: H.gemm(a, w, m, gk, gn, b_is_nk=True) for (m, gk, gn) in [(3, 128, 32), (0, 0, 0)]}
    assert H.gemm_status() == 0
    for (m, gk, gn) in [(3, 128, 32), (0, 0, 0), (2, 32, 0)]:
        gemm_wait_selftest(a, w, m, gk, gn, poll_limit=2048)
        torch.cuda.synchronize()                      # the kernel came back
        st = H.gemm_status()
        assert st in (2, 4), f"mode {m}: status {st} (2 = operand wait, 4 = accumulator wait)"
        lin = H.QLinear(K, N, bias=False, device="cuda", dtype=torch.float16)
        lin.weight.data = w
        lin.ops = H.FP16AccumMatMul(group_size=128, quant_block_size=32)
        with pytest.raises(RuntimeError, match="gave up on a wait"):
            lin(a)                                    # sticky until reset: the layer's guard refuses to go on
        H.gemm_status_reset()
        assert H.gemm_status() == 0
    for (m, gk, gn) in [(3, 128, 32), (0, 0, 0)]:
        again = H.gemm(a, w, m, gk, gn, b_is_nk=True)
        assert torch.equal(again.view(torch.int16), before[m].view(torch.int16))
    assert H.gemm_status() == 0
    from hbq_b200 import _lib
    vp = __import__("ctypes").c_void_p
    L = _lib.lib()
    assert L.hbq_gemm_wait_selftest(vp(a.data_ptr()), vp(w.data_ptr()), vp(before[0].data_ptr()), M, N, K, 0, 0, 0, 0, None) == -1
    assert L.hbq_gemm_wait_selftest(vp(a.data_ptr()), vp(w.data_ptr()), vp(before[0].data_ptr()), M, N, 12, 0, 0, 0, 64, None) == -2


def test_int8_partial_sums_non_finite_like_the_reference(oracle):
    """NaN and Inf partial sums in the INT8 partial-sum mode (gemm.cu:1145-1152, 1236-1249): a NaN stays NaN
    and does not count towards its run's maximum; an infinite value makes the whole run of group_n columns
    NaN.  Tensor-core kernel == exact-order kernel == the reference's kernel (where built), position by
    position, and the finite outputs keep the usual tolerance."""
    import hbq_b200 as H
    M, N, K = 128, 256, 256
    rng = np.random.default_rng(5)
    A = rng.standard_normal((M, K)).astype(np.float16)
    W = (0.05 * rng.standard_normal((N, K))).astype(np.float16)
    A[3, 10] = np.nan            # row 3: every output NaN (a NaN partial sum in each run of chunk 0)
    W[70, 200] = np.inf          # column 70: infinite partial sums in chunk 1 -> its whole run of 32 columns NaN
    W[9, 5] = -np.inf
    a, w = dev(A), dev(W)
    tc = H.gemm(a, w, 3, 128, 32, b_is_nk=True)
    simt = H.gemm(a, w, 3, 128, 32, b_is_nk=True, force_simt=True)
    torch.cuda.synchronize()
    assert H.gemm_status() == 0
    for name, other in [("exact-order kernel", simt)]:
        assert torch.equal(torch.isnan(tc), torch.isnan(other)), f"NaN positions differ from the {name}"
        assert torch.equal(torch.isinf(tc), torch.isinf(other)), f"Inf positions differ from the {name}"
    nan = torch.isnan(tc)
    assert bool(nan[3].all()) and bool(nan[:, 64:96].all()) and bool(nan[:, 0:32].all())
    assert not bool(nan[5, 96:128].any())
    fin = ~nan & ~torch.isinf(tc)
    g, r = tc[fin].double(), simt[fin].double()
    assert float((g - r).norm() / r.norm()) <= REL_FRO_TOL
    ref_ext = _load_reference_ext()
    if ref_ext is not None:
        ref = ref_ext.gemm_blockquant_mxint8(a, w.t().contiguous(), 128, 32)
        torch.cuda.synchronize()
        assert torch.equal(torch.isnan(tc), torch.isnan(ref)), "NaN positions differ from the reference's gemm.cu"


def test_bias_is_fused_and_lands_in_out():
    """FP16AccumMatMul passes the bias to the kernel; with `out=` the biased result is in `out`."""
    import hbq_b200 as H
    M, N, K = 300, 512, 256
    a = torch.randn((M, K), device="cuda").half()
    w = (0.05 * torch.randn((N, K), device="cuda")).half()
    b = torch.randn(N, device="cuda").half()
    for op in (H.FP16AccumMatMul(group_size=128, quant_block_size=32), H.FP16AccumMatMul(group_size=64), H.FP16AccumMatMul()):
        want = op(a, w) + b
        buf = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        l0 = H.launch_count()
        got = op(a, w, b, out=buf)
        assert H.launch_count() - l0 == 1             # one kernel: no separate bias add
        assert got.data_ptr() == buf.data_ptr()
        assert torch.equal(buf.view(torch.int16), want.view(torch.int16))
