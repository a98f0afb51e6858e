"""GPU: the benchmark configurations themselves, at their stated sizes and seeds, as parity tests.

configs[0]  one HBQ-A linear layer: X bf16 [2048,4096] ~ N(0,1) with 1 % of the input channels x20,
            W bf16 [4096,4096] ~ N(0, 0.02); codes, block scales, micro-scale indices and scheme bits
            against the CPU oracle (mismatch COUNTS), Y against an fp32 matmul of the oracle's tensors.
configs[1]  HBQ-E quant-GEMM M=4096, K=4096, N=14336 in both accumulation modes of the shipped YAMLs
            (fp16 grouped 128; INT8 partial sums 128/32) against the reference's own gemm.cu compiled for
            this GPU, over ALL rows.
configs[2]  [8192,8192] bf16 Student-t tensor through the activation quantizer of six formats, bf16 in,
            packed codes + scales + bf16 fake-quantised tensor out, against the oracle on 256 rows spread
            over the tensor.
Integer / byte / fp16-pattern outputs of the quantizers must be equal bit for bit.  The tensor-core GEMM
is held to: relative Frobenius error <= 2^-9 and at most 1 % of the outputs further than 2 fp16 ulps away.
"""
import numpy as np
import pytest

from util import bits, load_formats, make_quantizer, oracle_format

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_FRO_TOL = 2.0 ** -9
FAR_ULP_FRACTION = 0.01


def _randn(shape, seed):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed))


def _outlier_input(rows, K, frac, gain, seed, perm_seed):
    x = _randn((rows, K), seed)
    cols = torch.randperm(K, generator=torch.Generator().manual_seed(perm_seed))[: max(1, int(K * frac))]
    x[:, cols] *= gain
    return x.to(torch.bfloat16)


def _fp16_np(t_bf16):
    """bf16 tensor -> the fp16 array the reference would quantise (exact inside fp16's normal range)."""
    return t_bf16.to(torch.float16).cpu().numpy()


def _unpack_nibbles(pc):
    return np.stack([pc & 0xF, pc >> 4], axis=-1).reshape(pc.shape[0], -1)


def packed_mismatches(packed, o, spec):
    """Mismatch counts of every packed plane against the oracle's outputs."""
    rows = o["deq"].shape[0]
    oc = o["codes"].reshape(rows, -1).astype(np.uint8)
    pc = packed.codes.cpu().numpy()
    nbits = 1 + spec.get("ebit", 0) + spec.get("mbit", 0) if spec["kind"] != "mxint" else spec["nbit"]
    out = {}
    if nbits <= 4:
        out["codes"] = int((_unpack_nibbles(pc) != (oc & 0xF)).sum())
    elif nbits == 5:
        out["codes"] = int((_unpack_nibbles(pc) != (oc & 0xF)).sum())
        sg = np.unpackbits(packed.sign.cpu().numpy(), axis=-1, bitorder="little")
        out["sign"] = int((sg != (oc >> 4)).sum())
    else:
        out["codes"] = int((pc != oc).sum())
    out["scale"] = int((packed.scale_u8.cpu().numpy() != (bits(o["scale"]) >> 7).astype(np.uint8)).sum())
    if spec["kind"] == "hbq":
        l2 = o["l2"].astype(np.uint64)
        nb = spec["l2_sc_bit"]
        word = np.zeros(l2.shape[:2], np.uint64)
        for u in range(l2.shape[2]):
            word |= l2[:, :, u] << np.uint64(u * nb)
        got = packed.l2_packed.cpu().numpy().astype(np.uint64)
        gw = np.zeros_like(word)
        for b in range(got.shape[-1]):
            gw |= got[:, :, b] << np.uint64(8 * b)
        out["l2"] = int((gw != word).sum())
        if packed.scheme is not None:
            out["scheme"] = int((packed.scheme.cpu().numpy() != o["scheme"]).sum())
    return out


def gemm_report(got, ref, what):
    """Mismatch count, largest distance in fp16 ulps, fraction further than 2 ulps, relative Frobenius error."""
    gb = got.view(torch.int16).to(torch.int32)
    rb = ref.view(torch.int16).to(torch.int32)
    # fp16 patterns as a monotone integer line (negative values mirrored), so differences count ulps
    gl = torch.where(gb < 0, -(gb & 0x7FFF), gb)
    rl = torch.where(rb < 0, -(rb & 0x7FFF), rb)
    ulp = (gl - rl).abs()
    mism = int((ulp != 0).sum())
    far = float((ulp > 2).float().mean())
    d = got.double() - ref.double()
    rel = float(d.norm() / ref.double().norm().clamp_min(1e-30))
    print(f"{what}: mismatches {mism}/{ref.numel()}, max ulp {int(ulp.max())}, >2ulp {far:.2e}, rel_fro {rel:.3e}")
    assert rel <= REL_FRO_TOL, f"{what}: relative Frobenius error {rel}"
    assert far <= FAR_ULP_FRACTION, f"{what}: {far:.3%} of the outputs are more than 2 fp16 ulps away"
    return mism


def test_config0_hbq_a_linear_layer(oracle):
    import hbq_b200 as H
    f = load_formats()
    M, K, N = 2048, 4096, 4096
    x = _outlier_input(M, K, 0.01, 20.0, seed=0, perm_seed=0)
    w = (0.02 * _randn((N, K), 1)).to(torch.bfloat16)
    aq = make_quantizer(f["hbq_a_act"])
    wq = make_quantizer(f["hbq_a_wgt"])
    aq.out_dtype = wq.out_dtype = torch.float16        # bf16 in, fp16 fake-quantised out: the GEMM's operand type
    pa, xq = aq.quantize_packed(x.cuda(), with_deq=True)
    pw, wqt = wq.quantize_packed(w.cuda(), with_deq=True)
    torch.cuda.synchronize()
    oa = oracle.quantize(_fp16_np(x), oracle_format(oracle, f["hbq_a_act"]))
    ow = oracle.quantize(_fp16_np(w), oracle_format(oracle, f["hbq_a_wgt"]))
    ma = packed_mismatches(pa, oa, f["hbq_a_act"])
    mw = packed_mismatches(pw, ow, f["hbq_a_wgt"])
    ma["deq"] = int((bits(xq.cpu().numpy()) != bits(oa["deq"])).sum())
    mw["deq"] = int((bits(wqt.cpu().numpy()) != bits(ow["deq"])).sum())
    print("activation mismatches", ma, "weight mismatches", mw)
    assert set(mw) >= {"codes", "scale", "l2", "scheme", "deq"} and set(ma) >= {"codes", "sign", "scale", "l2", "deq"}
    assert not any(ma.values()), ma
    assert not any(mw.values()), mw
    # the plain fake-quantise call (the per-step kernel, no side outputs) gives the same tensor
    assert torch.equal(aq.q(x.cuda()).view(torch.int16), xq.view(torch.int16))
    assert torch.equal(wq.q(w.cuda()).view(torch.int16), wqt.view(torch.int16))
    # Y with fp32 accumulation against an fp32 matmul of the oracle's fake-quantised tensors
    lin = H.QLinear(K, N, bias=False, device="cuda", dtype=torch.float16)
    lin.weight.data = wqt
    lin.aq = aq
    with torch.no_grad():
        y_default = lin(x.cuda())                                   # ops=None: F.linear, as the reference
        y_tc = H.blockquant_ext.gemm_fp32_accum(xq, wqt, b_is_nk=True)
    ref = torch.from_numpy(oa["deq"].astype(np.float32)) @ torch.from_numpy(ow["deq"].astype(np.float32)).T
    for name, y in (("F.linear", y_default), ("tcgen05 fp32 accumulation", y_tc)):
        rel = float((y.float().cpu() - ref).norm() / ref.norm())
        print(f"configs[0] Y via {name}: rel_fro {rel:.3e}")
        assert rel <= REL_FRO_TOL, (name, rel)
    assert H.gemm_status() == 0


def _reference_ext():
    import importlib.util
    import os
    so = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "blockquant_ext.so")
    if not os.path.exists(so):
        return None
    spec = importlib.util.spec_from_file_location("blockquant_ext", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_config1_hbq_e_quant_gemm_all_rows(oracle):
    import hbq_b200 as H
    ref_ext = _reference_ext()
    if ref_ext is None:
        pytest.skip("oracle/_ref/blockquant_ext.so not built")
    f = load_formats()
    M, K, N = 4096, 4096, 14336
    x = _outlier_input(M, K, 0.005, 30.0, seed=0, perm_seed=0)
    w = (0.02 * _randn((N, K), 1)).to(torch.bfloat16)
    aq = make_quantizer(f["hbq_e_act"])
    wq = make_quantizer(f["hbq_e_wgt"])
    aq.out_dtype = wq.out_dtype = torch.float16
    xq = aq.q(x.cuda())
    wqt = wq.q(w.cuda())
    # operands against the oracle on rows spread over both tensors
    ra = np.arange(0, M, 32)
    rw = np.arange(0, N, 64)
    oa = oracle.quantize(_fp16_np(x)[ra], oracle_format(oracle, f["hbq_e_act"]), False)["deq"]
    ow = oracle.quantize(_fp16_np(w)[rw], oracle_format(oracle, f["hbq_e_wgt"]), False)["deq"]
    assert int((bits(xq.cpu().numpy()[ra]) != bits(oa)).sum()) == 0
    assert int((bits(wqt.cpu().numpy()[rw]) != bits(ow)).sum()) == 0
    w_kn = wqt.t().contiguous()                      # the layout the reference extension receives (src/ops.py:41)
    cases = [("config/hbq_e_fp16.yaml: fp16 grouped 128", lambda: ref_ext.gemm_fp16_grouped_accum(xq, w_kn, 128), (2, 128, 0)),
             ("config/hbq_e_psum_quant.yaml: INT8 partial sums 128/32", lambda: ref_ext.gemm_blockquant_mxint8(xq, w_kn, 128, 32),
              (3, 128, 32))]
    for name, run_ref, (mode, gk, gn) in cases:
        torch.cuda.synchronize()
        ref = run_ref()
        torch.cuda.synchronize()                     # the reference launches on the legacy default stream
        got = H.gemm(xq, wqt, mode, gk, gn, b_is_nk=True)
        torch.cuda.synchronize()
        assert H.gemm_status() == 0
        gemm_report(got, ref, f"configs[1] {name}, all {M} rows")
        del ref, got


C3_FORMATS = ["mxfp4", "nvfp4", "mxint8", "mxfp_a8", "hbq_a_act", "hbq_e_act"]


@pytest.fixture(scope="module")
def student_t_tensor():
    torch.manual_seed(2)
    t = 0.5 * torch.distributions.StudentT(3.0).sample((8192, 8192))
    return t.to(torch.bfloat16)


@pytest.mark.parametrize("name", C3_FORMATS)
def test_config2_quantize_sweep(oracle, student_t_tensor, name):
    spec = load_formats()[name]
    q = make_quantizer(spec)
    x = student_t_tensor.cuda()
    packed, y = q.quantize_packed(x, with_deq=True)
    assert y.dtype == torch.bfloat16 and y.shape == x.shape
    y_plain = q.q(x)                                   # fake-quantised tensor only: the lean kernels
    torch.cuda.synchronize()
    assert torch.equal(y_plain.view(torch.int16), y.view(torch.int16))
    rows = np.arange(5, 8192, 32)                      # 256 rows spread over the tensor
    o = oracle.quantize(_fp16_np(student_t_tensor)[rows], oracle_format(oracle, spec))
    ref_bf16 = torch.from_numpy(o["deq"].copy()).to(torch.bfloat16).view(torch.int16)
    sel = torch.from_numpy(rows).cuda()

    class _Rows:                                       # the sampled rows of every packed plane
        pass
    pr = _Rows()
    for plane in ("codes", "sign", "scale_u8", "l2_packed", "scheme"):
        t = getattr(packed, plane)
        setattr(pr, plane, None if t is None else t.view(8192, *t.shape[1:])[sel])
    mism = packed_mismatches(pr, o, spec)
    mism["deq_bf16"] = int((y[sel].cpu().view(torch.int16) != ref_bf16).sum())
    print(f"configs[2] {name}: mismatches on {rows.size} rows", mism)
    assert not any(mism.values()), mism
