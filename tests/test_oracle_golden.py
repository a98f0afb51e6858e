"""CPU: the oracle (oracle/hbq_oracle.c) against the golden vectors produced by the reference's
own Python quantizers (tests/golden/make_golden.py).  This is what pins the oracle."""
import numpy as np
import pytest

from util import bits, load_formats, load_npz, oracle_format


def test_element_quantizer_exhaustive(oracle):
    ex = load_npz("exhaustive.npz")
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    xs = allh[ex["finite"]]
    for e, m in [(2, 1), (2, 2), (2, 3), (2, 5), (3, 2), (4, 3), (5, 2)]:
        got = oracle.fp_quant(xs, e, m, True, False, True)
        assert np.array_equal(bits(got), ex[f"elem_e{e}m{m}"]), f"E{e}M{m}"


def test_scale_quantizer_exhaustive(oracle):
    ex = load_npz("exhaustive.npz")
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    xs = allh[ex["finite"]]
    for se, sm in [(5, 3), (4, 3)]:
        for ceil in (0, 1):
            for sub in (0, 1):
                got = oracle.fp_quant(xs, se, sm, bool(sub), bool(ceil), False)
                assert np.array_equal(bits(got), ex[f"scale_e{se}m{sm}_ceil{ceil}_sub{sub}"])


def test_floor_log2_fp16_quirk(oracle):
    """floor(log2(x)) on fp16 tensors is one too high for 94 values just below a power of two."""
    ex = load_npz("exhaustive.npz")
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    pos = allh[ex["finite"] & (allh > 0)]
    got = oracle.floor_log2_h(pos)
    assert np.array_equal(got.astype(np.int8), ex["floor_log2_pos"])
    true = np.floor(np.log2(pos.astype(np.float64)))
    assert int((got != true).sum()) == 94


@pytest.mark.parametrize("name", sorted(load_formats().keys()))
def test_quantizers_match_reference(oracle, name):
    spec = load_formats()[name]
    g = load_npz("quantizers.npz")
    fmt = oracle_format(oracle, spec)
    ins = sorted(k[3:] for k in g.files if k.startswith("in/"))
    assert ins
    for k in ins:
        x = g[f"in/{k}"]
        o = oracle.quantize(x, fmt)
        assert np.array_equal(bits(o["deq"]), g[f"out/{name}/{k}/deq"]), f"{name}/{k} deq"
        if spec["kind"] == "hbq":
            assert np.array_equal(bits(o["scale"]), g[f"out/{name}/{k}/scale"]), f"{name}/{k} scale"
            assert np.array_equal(o["l2"], g[f"out/{name}/{k}/l2"]), f"{name}/{k} l2"
            assert np.array_equal(o["scheme"], g[f"out/{name}/{k}/scheme"]), f"{name}/{k} scheme"


def test_codes_reconstruct_dequantised_value(oracle):
    """codes + scales carry the whole result: decode(code) * l2 * l1 == deq exactly."""
    spec = load_formats()["hbq_a_act"]
    g = load_npz("quantizers.npz")
    x = g["in/act"]
    o = oracle.quantize(x, oracle_format(oracle, spec))
    code = o["codes"].astype(np.int32)
    sgn = np.where(code >> 4, -1.0, 1.0)
    ef, mf = (code >> 2) & 3, code & 3
    mag = np.where(ef == 0, mf / 4.0, (1 + mf / 4.0) * 2.0 ** (ef - 1))
    tab = np.array([1, 1.5, 2, 2.5])
    l2 = np.repeat(tab[o["l2"]], spec["l2_block_size"], axis=-1)
    rec = sgn * mag * l2 * o["scale"].astype(np.float64)[..., None]
    rows, K = x.shape
    assert np.array_equal(rec.reshape(rows, -1)[:, :K].astype(np.float16).view(np.uint16), bits(o["deq"]))


def test_gemm_models_small(oracle):
    """Accumulation models against a straightforward numpy restatement on a tiny case."""
    rng = np.random.default_rng(0)
    M, N, K = 5, 8, 48
    A = rng.standard_normal((M, K)).astype(np.float16)
    B = (0.1 * rng.standard_normal((K, N))).astype(np.float16)
    # grouped: fp32 sequential inside 16-chunks, fp16 add across
    ref = np.zeros((M, N), np.float16)
    for m in range(M):
        for n in range(N):
            acc = np.float16(0)
            for k0 in range(0, K, 16):
                g = np.float32(0)
                for k in range(k0, k0 + 16):
                    g = np.float32(np.float64(A[m, k]) * np.float64(B[k, n]) + np.float64(g))
                acc = np.float16(np.float32(acc) + np.float32(np.float16(g)))
            ref[m, n] = acc
    got = oracle.gemm(A, B, oracle.ACC_GROUPED, 16)
    assert np.array_equal(bits(got), bits(ref))
    # fp32 accumulate equals the grouped model with one group spanning K, rounded once
    got32 = oracle.gemm(A, B, oracle.ACC_FP32)
    assert np.allclose(got32.astype(np.float32), A.astype(np.float32) @ B.astype(np.float32), rtol=2e-3, atol=1e-3)
    # INT8 partial sums: every dequantised chunk is an integer multiple of its power-of-two scale
    gi = oracle.gemm(A, B, oracle.ACC_PSUM_INT8, 16, 4)
    assert np.isfinite(gi.astype(np.float32)).all()
    rel = np.abs(gi.astype(np.float32) - got32.astype(np.float32)).max() / np.abs(got32.astype(np.float32)).max()
    assert rel < 0.05
