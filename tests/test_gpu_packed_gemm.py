"""GPU: the GEMM on the packed 4-bit weight (hbq_gemm_w4, both code containers) against the same product on the fp16 fake-quantised tensor
the reference keeps (src/ptq.py:349, F.linear in src/module.py:64).

Two bars.  (1) The values the kernel expands on chip are the fake-quantised weights BIT FOR BIT: one-hot rows
of X make every output a single product 1 * w, so C spells out the expanded tile.  (2) With real activations the
result is the fp32-accumulated product rounded to fp16: relative Frobenius error <= 2^-9 against an fp64 product of
the same fp16 operands and at most 1 % of the outputs further than 2 fp16 ulps from it (the bound of the fp16-operand
tensor-core kernel); K slices are added in a fixed order, so two runs give the same bits."""
import pytest

from util import load_formats, make_quantizer

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 2.0 ** -9
FAR_ULP_FRACTION = 0.01


def _weight(name, N, K, seed, bits=4):
    import hbq_b200 as H
    from hbq_b200.packed_gemm import W4Weight
    q = make_quantizer(load_formats()[name])
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (0.02 * torch.randn((N, K), device="cuda", generator=g)).half()
    w[:, ::97] *= 8                                       # a few large columns: more than one scale binade per row
    packed, deq = q.quantize_packed(w, with_deq=True)
    assert W4Weight.supported(packed)
    assert torch.equal(H.dequantize_packed(packed).view(torch.int16), deq.view(torch.int16))
    return W4Weight.from_packed(packed, container_bits=bits), deq


def _ulps(a, b):
    ia, ib = a.view(torch.int16).to(torch.int32), b.view(torch.int16).to(torch.int32)
    ia = torch.where(ia < 0, -(ia & 0x7FFF), ia)
    ib = torch.where(ib < 0, -(ib & 0x7FFF), ib)
    return (ia - ib).abs()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("name", ["hbq_a_wgt", "hbq_e_wgt", "hbq_fp1", "hbq_fpm100"])
@pytest.mark.parametrize("shape", [(256, 512), (1024, 4096), (19200, 2048)])
def test_expanded_values_are_the_fake_quantised_weights(name, shape, bits):
    spec = load_formats()[name]
    if spec["mbit"] != 1 or spec["block_size"] != 128 or spec["l2_block_size"] not in (8, 32) or spec["l2_sc_bit"] != 2:
        pytest.skip("not a 4-bit block-128 weight format")
    N, K = shape
    w4, deq = _weight(name, N, K, seed=N + K, bits=bits)
    assert w4.nbytes() == N * K * (9216 if bits == 4 else 17408) // (128 * 128)
    for rows in (128, 16, 5, 2, 1):                      # 2 and 1: the kernel without the tensor core (nibble container)
        for off in range(0, K, 128 if K <= 512 else 1024):
            x = torch.zeros((rows, K), device="cuda", dtype=torch.float16)
            cols = (off + torch.arange(rows, device="cuda") * 7) % K
            x[torch.arange(rows, device="cuda"), cols] = 1.0
            c = w4.matmul(x)
            want = deq[:, cols].t().contiguous()
            # -0 * 1 accumulated into +0 reads +0: compare values, then the bits of everything non-zero
            nz = want != 0
            assert torch.equal(c[nz].view(torch.int16), want[nz].view(torch.int16)), (name, rows, off)
            assert bool((c[~nz] == 0).all())


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("name", ["hbq_a_wgt", "hbq_e_wgt"])
# the three ways the work is cut: whole tiles per SM (14336 x 4096, 128 x 128), a tile's K split over a cluster
# (4096 x 14336, 1024 x 4096), equal runs of records per SM with tiles shared between CTAs (19200 x 2048); 19200 x 256 is
# more whole tiles than SMs
@pytest.mark.parametrize("N,K", [(14336, 4096), (4096, 14336), (1024, 4096), (128, 128), (19200, 2048), (19200, 256)])
def test_against_the_fp16_operand_product(name, N, K, bits):
    import hbq_b200 as H
    from hbq_b200 import blockquant_ext as ext
    w4, deq = _weight(name, N, K, seed=1, bits=bits)
    aq = make_quantizer(load_formats()["hbq_a_act" if name == "hbq_a_wgt" else "hbq_e_act"])
    g = torch.Generator(device="cuda").manual_seed(N)
    bias = torch.randn(N, device="cuda", generator=g).half()
    for M in (1, 2, 7, 16, 33, 64, 128):
        x = aq.q(torch.randn((M, K), device="cuda", generator=g).half())
        for b in (None, bias):
            c = w4.matmul(x, bias=b)
            assert H.gemm_status() == 0
            ref = x.double() @ deq.double().t()
            ref16 = ref.float().half()
            if b is not None:
                ref16 = ref16 + b
                ref = ref16.double()
            rel = float((c.double() - ref).norm() / ref.norm())
            far = float((_ulps(c, ref16 if b is not None else ref.float().half()) > 2).float().mean())
            assert rel <= REL_TOL and far <= FAR_ULP_FRACTION, (M, rel, far)
            # the same call again: slices are added in a fixed order
            assert torch.equal(w4.matmul(x, bias=b), c)
        # and the tensor-core kernel on the fp16 tensor agrees to the same bound
        c16 = ext.gemm_fp32_accum(x, deq, b_is_nk=True)
        assert float((w4.matmul(x).double() - c16.double()).norm() / c16.double().norm()) <= REL_TOL


def test_shapes_and_formats_outside_the_kernel_are_refused():
    import hbq_b200 as H
    from hbq_b200 import _lib
    from hbq_b200.packed_gemm import W4Weight
    w4, _ = _weight("hbq_a_wgt", 256, 256, seed=2)
    with pytest.raises(_lib.HbqError):
        w4.matmul(torch.zeros((129, 256), device="cuda", dtype=torch.float16))
    with pytest.raises(RuntimeError):
        w4.matmul(torch.zeros((4, 128), device="cuda", dtype=torch.float16))
    fm = load_formats()
    for name, shape in (("hbq_a_act", (256, 256)), ("hbq_a_wgt", (200, 256)), ("mxfp4", (256, 256))):
        q = make_quantizer(fm[name])
        packed = q.quantize_packed(torch.randn(shape, device="cuda").half())
        assert not W4Weight.supported(packed), name
    # a 4-bit HBQ weight whose micro-scale table is not base + idx * step (SIG-1): the library refuses it
    spec = dict(fm["hbq_a_wgt"], l2_scheme="SIG-1")
    packed = make_quantizer(spec).quantize_packed(torch.randn((256, 256), device="cuda").half())
    with pytest.raises(_lib.HbqError):
        W4Weight.from_packed(packed)
    assert H.gemm_status() == 0


def test_linear_layer_on_the_packed_weight():
    """QLinear.prepare_decode: decode-sized batches take the packed kernel, larger ones the fp16 tensor; with the fp16
    tensor dropped every batch goes through the packed kernel and the layer holds 0.5625 B per weight."""
    import hbq_b200 as H
    fm = load_formats()
    N, K = 1024, 2048
    lin = H.QLinear(K, N, bias=True, device="cuda", dtype=torch.float16, check_finite=False)
    g = torch.Generator(device="cuda").manual_seed(9)
    lin.weight.data = (0.02 * torch.randn((N, K), device="cuda", generator=g)).half()
    lin.bias.data = torch.randn(N, device="cuda", generator=g).half()
    lin.wq = make_quantizer(fm["hbq_a_wgt"])
    lin.aq = make_quantizer(fm["hbq_a_act"])
    assert lin.prepare_decode() and lin.w4_max_rows == 8     # the batch sizes where the packed kernels always win
    lin.w4_max_rows = 32
    wq = lin.weight.data.clone()
    for rows in (1, 20, 32, 33, 300):
        x = torch.randn((rows, K), device="cuda", generator=g).half()
        l0 = H.launch_count()
        y = lin(x)
        ours = H.launch_count() - l0                          # quantize + packed GEMM; F.linear is not counted
        ref = (lin.aq.q(x).double() @ wq.double().t()).float().half() + lin.bias.data
        rel = float((y.double() - ref.double()).norm() / ref.double().norm())
        assert y.shape == (rows, N) and rel <= REL_TOL, (rows, rel)
        assert ours == (2 if rows <= lin.w4_max_rows else 1)
    before = lin.weight.numel()
    assert lin.prepare_decode(drop_fp16=True) and lin.weight.numel() == 0 and before == N * K
    assert lin.w4_weight.nbytes() * 128 * 128 == N * K * 9216
    x = torch.randn((300, K), device="cuda", generator=g).half()
    y = lin(x)
    ref = (lin.aq.q(x).double() @ wq.double().t()).float().half() + lin.bias.data
    assert float((y.double() - ref.double()).norm() / ref.double().norm()) <= REL_TOL
    assert H.gemm_status() == 0
    # a layer with an accumulation operator keeps its own kernel
    lin2 = H.QLinear(K, N, bias=False, device="cuda", dtype=torch.float16, ops=H.FP16AccumMatMul(group_size=128))
    lin2.wq = make_quantizer(fm["hbq_a_wgt"])
    assert not lin2.prepare_decode()


def test_cuda_graph_capture_of_a_decode_step():
    """A decode step on the packed weight (activation quantize + hbq_gemm_w4) allocates and synchronises nothing of its
    own once warmed up, so a serving engine can capture it in a CUDA graph and replay it on new tokens."""
    import hbq_b200 as H
    fm = load_formats()
    K, N, rows = 2048, 1024, 8
    lin = H.QLinear(K, N, bias=True, device="cuda", dtype=torch.float16, check_finite=False)
    g0 = torch.Generator(device="cuda").manual_seed(21)
    lin.weight.data = (0.02 * torch.randn((N, K), device="cuda", generator=g0)).half()
    lin.bias.data = torch.randn(N, device="cuda", generator=g0).half()
    lin.wq, lin.aq = make_quantizer(fm["hbq_e_wgt"]), make_quantizer(fm["hbq_e_act"])
    assert lin.prepare_decode(drop_fp16=True)
    x_static = torch.randn((rows, K), device="cuda", generator=g0).half()
    with torch.no_grad():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                lin(x_static)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y_static = lin(x_static)
        for seed in (22, 23, 24):
            x_new = torch.randn((rows, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed)).half()
            x_static.copy_(x_new)
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(y_static, lin(x_new))
    assert H.gemm_status() == 0
