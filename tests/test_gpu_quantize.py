"""GPU: the CUDA quantize kernels against the golden vectors of the reference and against the
CPU oracle on seeded inputs.  Bit-exact: every comparison is on fp16 / integer bit patterns."""
import numpy as np
import pytest

from util import bits, load_formats, load_npz, make_quantizer, oracle_format, seeded_inputs

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if t.dtype == torch.uint16:
        t = t.view(torch.float16)
    t = t.cuda()
    return t if dtype is None else t.to(dtype)


def hbits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def test_library_loaded_and_no_fallback():
    import hbq_b200
    from hbq_b200 import _lib
    assert _lib.lib().hbq_version() >= 100
    with pytest.raises(hbq_b200.HbqError):
        hbq_b200.MXFPQuantizer(32, 2, 1, 5, 0).q(torch.zeros(4, 32, dtype=torch.float16))   # CPU tensor


def test_element_quantizer_exhaustive_gpu(oracle):
    """All 65 536 fp16 inputs through the kernel's packed E2Mx quantizer and the generic chain."""
    import ctypes
    from hbq_b200 import _lib
    ex = load_npz("exhaustive.npz")
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    fin = ex["finite"]
    x = dev(allh[fin])
    out = torch.empty_like(x)
    L = _lib.lib()
    for (e, m) in [(2, 1), (2, 2), (2, 3), (2, 5), (3, 2), (4, 3), (5, 2)]:
        _lib.check(L.hbq_fp_quant(x.data_ptr(), x.numel(), e, m, 1, 0, 1, out.data_ptr(), None), "fp_quant")
        torch.cuda.synchronize()
        got = hbits(out)
        bad = got != ex[f"elem_e{e}m{m}"]
        assert not bad.any(), f"E{e}M{m}: {bad.sum()} mismatches, first input 0x{allh[fin][bad][0]:04x}"
    for se, sm in [(5, 3), (4, 3)]:
        for ceil in (0, 1):
            for sub in (0, 1):
                _lib.check(L.hbq_fp_quant(x.data_ptr(), x.numel(), se, sm, sub, ceil, 0, out.data_ptr(), None), "fp_quant")
                torch.cuda.synchronize()
                bad = hbits(out) != ex[f"scale_e{se}m{sm}_ceil{ceil}_sub{sub}"]
                assert not bad.any(), f"scale E{se}M{sm} ceil={ceil} sub={sub}: {bad.sum()} mismatches"


def test_block_scale_exhaustive_gpu(oracle):
    """Every positive finite fp16 value as the absmax of a block: power-of-two scales (floor and
    round of the fp16 log2, including its 94 quirk values) and the E5M3 scale."""
    import hbq_b200 as H
    pos = np.arange(1, 0x7C00, dtype=np.uint16)
    cases = [
        (H.MXFPQuantizer(16, 2, 1, 5, 0), oracle.Format(oracle.KIND_MXFP, 2, 1, 5, 0, 16)),
        (H.MXFPQuantizer(16, 2, 1, 5, 0, use_round=True), oracle.Format(oracle.KIND_MXFP, 2, 1, 5, 0, 16, use_round=True)),
        (H.MXFPQuantizer(16, 2, 1, 5, 3), oracle.Format(oracle.KIND_MXFP, 2, 1, 5, 3, 16)),
        (H.MXFPQuantizer(16, 2, 1, 5, 3, use_ceil=True), oracle.Format(oracle.KIND_MXFP, 2, 1, 5, 3, 16, use_ceil=True)),
        (H.MXFPQuantizer(16, 2, 1, 4, 3), oracle.Format(oracle.KIND_MXFP, 2, 1, 4, 3, 16)),
        (H.MXINTQuantizer(8, 8, 0, 16), oracle.Format(oracle.KIND_MXINT, 0, 8, 8, 0, 16)),
        (H.HBQQuantizer(16, 2, 2, 5, 3, 8, 2, "SIG-1"), oracle.Format(oracle.KIND_HBQ, 2, 2, 5, 3, 16, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")),
    ]
    x = np.zeros((pos.size, 16), np.uint16)
    x[:, 3] = pos                                    # the block maximum
    x[:, 7] = (pos >> 1)                             # a second, smaller value
    x[:, 11] = pos | 0x8000
    for q, fmt in cases:
        got = hbits(q.q(dev(x)))
        ref = bits(oracle.quantize(x, fmt, want_codes=False)["deq"])
        bad = (got != ref).any(axis=1)
        assert not bad.any(), f"{type(q).__name__} {fmt}: {bad.sum()} blocks differ, first absmax 0x{pos[bad][0]:04x}"


@pytest.mark.parametrize("name", sorted(load_formats().keys()))
def test_quantizers_match_reference_golden(name):
    """deq / shared scale / L2 index / scheme against what the reference produced."""
    spec = load_formats()[name]
    g = load_npz("quantizers.npz")
    extra = {"keep_l2_scale": True} if spec["kind"] == "hbq" else {}
    q = make_quantizer(spec, **extra)
    q_plain = make_quantizer(spec)            # no side outputs: the kernels specialised for that case
    for k in sorted(f[3:] for f in g.files if f.startswith("in/")):
        x = dev(g[f"in/{k}"])
        n = int((hbits(q_plain.q(x)) != g[f"out/{name}/{k}/deq"]).sum())
        assert n == 0, f"{name}/{k}: {n} deq mismatches without side outputs"
        y = q.q(x)
        assert y.shape == x.shape and y.dtype == x.dtype
        n = int((hbits(y) != g[f"out/{name}/{k}/deq"]).sum())
        assert n == 0, f"{name}/{k}: {n} deq mismatches"
        if spec["kind"] == "hbq":
            assert np.array_equal(hbits(q.shared_scale), g[f"out/{name}/{k}/scale"]), f"{name}/{k} scale"
            assert np.array_equal(q.l2_scale.cpu().numpy().astype(np.uint8), g[f"out/{name}/{k}/l2"]), f"{name}/{k} l2"
            assert np.array_equal(q.blk_l2_scheme.cpu().numpy().astype(np.uint8), g[f"out/{name}/{k}/scheme"]), f"{name}/{k} scheme"


@pytest.mark.parametrize("name", ["hbq_a_act", "hbq_a_wgt", "hbq_e_act", "hbq_e_wgt", "hbq_a_kv4", "mxfp4",
                                  "nvfp4", "mxint8", "mxint4", "mxfp_a8", "mxfp6_e2m3"])
@pytest.mark.parametrize("kind", ["act", "wgt", "studt"])
def test_quantizers_match_oracle_seeded(oracle, name, kind):
    """Larger seeded tensors (benchmark value distributions): deq, codes, scales vs the oracle."""
    spec = load_formats()[name]
    x = seeded_inputs(kind, 256, 2048, seed=hash((name, kind)) % 1000)
    o = oracle.quantize(x, oracle_format(oracle, spec))
    q = make_quantizer(spec)
    packed, y = q.quantize_packed(dev(x), with_deq=True)
    torch.cuda.synchronize()
    n = int((hbits(y) != bits(o["deq"])).sum())
    assert n == 0, f"{n} deq mismatches of {x.size}"
    # shared scale byte: bits 14..7 of the fp16 scale
    assert np.array_equal(packed.scale_u8.cpu().numpy(), (bits(o["scale"]) >> 7).astype(np.uint8))
    # element codes
    oc = o["codes"].reshape(x.shape[0], -1).astype(np.uint8)
    pc = packed.codes.cpu().numpy()
    fmtbits = 1 + spec.get("ebit", 0) + spec.get("mbit", 0) if spec["kind"] != "mxint" else spec["nbit"]
    if fmtbits <= 4:
        un = np.stack([pc & 0xF, pc >> 4], axis=-1).reshape(x.shape[0], -1)
        assert np.array_equal(un, oc & 0xF), "4-bit codes"
    elif fmtbits == 5:
        un = np.stack([pc & 0xF, pc >> 4], axis=-1).reshape(x.shape[0], -1)
        assert np.array_equal(un, oc & 0xF), "5-bit codes: nibble plane"
        sg = np.unpackbits(packed.sign.cpu().numpy(), axis=-1, bitorder="little")
        assert np.array_equal(sg, oc >> 4), "5-bit codes: sign plane"
    else:
        assert np.array_equal(pc, oc), "byte codes"
    if spec["kind"] == "hbq":
        l2 = o["l2"].astype(np.uint32)
        nb = spec["l2_sc_bit"]
        word = np.zeros(l2.shape[:2], np.uint64)
        for u in range(l2.shape[2]):
            word |= l2[:, :, u].astype(np.uint64) << np.uint64(u * nb)
        nbytes = packed.l2_packed.shape[-1]
        got = packed.l2_packed.cpu().numpy().astype(np.uint64)
        gw = np.zeros_like(word)
        for b in range(nbytes):
            gw |= got[:, :, b] << np.uint64(8 * b)
        assert np.array_equal(gw, word), "packed L2 indices"
        if packed.scheme is not None:
            assert np.array_equal(packed.scheme.cpu().numpy(), o["scheme"])
    # codes + scales rebuild the fake-quantised tensor exactly
    import hbq_b200 as H
    rec = H.dequantize_packed(packed)
    a, b = hbits(rec), hbits(y).copy()
    if spec["kind"] == "mxint":
        b[b == 0x8000] = 0          # two's-complement codes cannot carry the reference's -0.0
    assert np.array_equal(a, b), "dequantize(packed) != deq"


def test_per_tensor_scale(oracle):
    import hbq_b200 as H
    for scale in (1.0, 0.02, 300.0):
        x = (scale * seeded_inputs("act", 64, 512, seed=5).astype(np.float32)).astype(np.float16)
        for (sce, scm, B, m) in [(4, 3, 16, 1), (5, 3, 16, 1), (5, 0, 32, 3)]:
            q = H.MXFPQuantizer(B, 2, m, sce, scm, per_tensor_scale=True)
            ref = oracle.quantize(x, oracle.Format(oracle.KIND_MXFP, 2, m, sce, scm, B, per_tensor_scale=True), False)
            assert np.array_equal(hbits(q.q(dev(x))), bits(ref["deq"]))


def test_bf16_and_shapes(oracle):
    """bf16 input = convert to fp16, quantise, round the result to bf16; leading dims and a ragged K."""
    import hbq_b200 as H
    spec = load_formats()["hbq_a_act"]
    q = make_quantizer(spec)
    x32 = torch.randn(3, 5, 200, generator=torch.Generator().manual_seed(1))
    xb = x32.to(torch.bfloat16).cuda()
    y = q.q(xb)
    assert y.dtype == torch.bfloat16 and y.shape == xb.shape
    xh = xb.to(torch.float16)
    ref = oracle.quantize(xh.reshape(-1, 200), oracle_format(oracle, spec), False)["deq"]
    refb = torch.from_numpy(ref.copy()).to(torch.bfloat16).reshape(3, 5, 200)
    assert torch.equal(y.cpu().view(torch.int16), refb.view(torch.int16))
    # ragged K with a K that is not a multiple of 8 either (scalar load path)
    x = seeded_inputs("studt", 33, 333, seed=9)
    for name in ("hbq_a_act", "mxfp4", "mxint8", "nvfp4"):
        sp = load_formats()[name]
        got = hbits(make_quantizer(sp).q(dev(x)))
        assert np.array_equal(got, bits(oracle.quantize(x, oracle_format(oracle, sp), False)["deq"])), name
    # empty tensors
    assert q.q(torch.empty(0, 128, dtype=torch.float16, device="cuda")).shape == (0, 128)
    with pytest.raises(NotImplementedError):
        q.q(torch.zeros(2, 128, device="cuda"))       # fp32 is not modelled


def test_full_size_properties():
    """[8192, 8192] Student-t tensor: determinism, row-shard invariance and packed round trip."""
    import hbq_b200 as H
    spec = load_formats()["hbq_a_act"]
    q = make_quantizer(spec)
    g = torch.Generator(device="cuda").manual_seed(2)
    x = (0.5 * torch.distributions.StudentT(3.0).sample((8192, 1024)).cuda()).repeat(1, 8)
    x = (x * (1 + 0.001 * torch.rand(8192, 8192, device="cuda", generator=g))).to(torch.float16)
    packed, y = q.quantize_packed(x, with_deq=True)
    y2 = q.q(x)
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    # any row split gives the same rows (the path shards by rows without exchange)
    ya = q.q(x[:3000].contiguous())
    yb = q.q(x[3000:].contiguous())
    assert torch.equal(torch.cat([ya, yb]).view(torch.int16), y.view(torch.int16))
    assert torch.equal(H.dequantize_packed(packed).view(torch.int16), y.view(torch.int16))
    # quantisation error is bounded by the coarsest step of the format: |x - y| <= amax(block) / 7 * 0.5 * 2.5
    err = (x.float() - y.float()).abs().view(8192, -1, 128)
    bound = x.float().abs().view(8192, -1, 128).amax(-1, keepdim=True) * (0.5 / 7) * 2.5 * 1.07 + 1e-7
    assert bool((err <= bound).all())
    assert packed.nbytes() == x.numel() * 5 // 8 + x.numel() // 128 + x.numel() // 8 * 2 // 8


@pytest.mark.parametrize("name", ["hbq_e_act", "hbq_a_wgt", "mxfp4", "nvfp4"])
def test_more_than_2_31_elements(name):
    """A tensor of 2^31 + 2^20 elements (4.3 GB of fp16): element offsets pass 2^31.  Blocks are
    independent, so slices quantised on their own must give the same bits as the same slices of the
    whole; the packed path (codes, scales, side outputs) is checked by its round trip on the tail."""
    import hbq_b200 as H
    q = make_quantizer(load_formats()[name])
    K = 8192
    rows = (2 ** 31 + 2 ** 20) // K
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.empty((rows, K), dtype=torch.float16, device="cuda")
    for r0 in range(0, rows, 32768):                     # filled in pieces: no fp32 copy of the whole
        n = min(32768, rows - r0)
        x[r0:r0 + n] = torch.randn((n, K), device="cuda", generator=g).to(torch.float16)
    y = q.q(x)
    assert y.shape == x.shape
    for r0 in (0, rows // 2 - 64, 2 ** 31 // K - 64, rows - 128):       # head, middle, across 2^31, tail
        part = q.q(x[r0:r0 + 128].contiguous())
        assert torch.equal(part.view(torch.int16), y[r0:r0 + 128].view(torch.int16)), (name, r0)
    del y
    packed, yd = q.quantize_packed(x, with_deq=True)
    tail = q.q(x[rows - 128:].contiguous())
    assert torch.equal(yd[rows - 128:].view(torch.int16), tail.view(torch.int16))
    back = H.dequantize_packed(packed)
    assert torch.equal(back[rows - 128:].view(torch.int16), tail.view(torch.int16))
    assert torch.equal(back[2 ** 31 // K - 64:2 ** 31 // K + 64].view(torch.int16),
                       yd[2 ** 31 // K - 64:2 ** 31 // K + 64].view(torch.int16))


def test_packed_form_round_trips_or_is_refused():
    """Every format with a packed form: dequantize(pack(x)) == q(x) bit for bit.  Formats whose scale does not
    fit the packed layout (a per-tensor scale, a scale mantissa wider than 3 bits, a power-of-two scale beyond
    fp16's exponent range) are refused by both directions instead of dequantising to other values."""
    import hbq_b200 as H
    x = dev(seeded_inputs("act", 64, 1024, seed=77))
    f = load_formats()
    for name, spec in sorted(f.items()):
        if spec["kind"] in ("mxex", "vsq"):
            continue
        q = make_quantizer(spec)
        fmt = q._format()
        refused = (spec.get("per_tensor_scale", False) or fmt.sc_mbit > 3 or
                   (spec["kind"] == "mxfp" and fmt.sc_mbit == 0 and fmt.sc_ebit > 5))
        if spec["kind"] == "hbq":           # packed micro-scale indices: whole bytes per block, up to one 32-bit word
            refused = refused or (spec["block_size"] // spec["l2_block_size"]) * spec["l2_sc_bit"] not in (8, 16, 32)
        if refused:
            with pytest.raises(H.HbqError):
                q.quantize_packed(x)
            continue
        packed, y = q.quantize_packed(x, with_deq=True)
        back = H.dequantize_packed(packed)
        a, b = hbits(back), hbits(y).copy()
        if spec["kind"] == "mxint":
            b[b == 0x8000] = 0            # two's-complement codes cannot carry the reference's -0.0
        assert np.array_equal(a, b), name
    for q in (H.MXFPQuantizer(16, 2, 1, 4, 3, per_tensor_scale=True), H.MXFPQuantizer(32, 2, 1, 8, 0),
              H.MXINTQuantizer(8, 5, 6, 32)):
        q.q(x)                                          # the fake-quantised tensor itself is served
        with pytest.raises(H.HbqError):
            q.quantize_packed(x)
        lin = H.QLinear(1024, 64, bias=False, device="cuda", dtype=torch.float16)
        lin.weight.data = x.clone()
        with pytest.raises(H.HbqError):
            lin.pack_weight(q)
