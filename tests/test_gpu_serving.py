"""GPU: the serving-side hooks (hbq_b200/serving.py) on flattened token batches and decode-sized shapes, against the
steps the reference's vLLM plugin runs (vllm/src/hbq_vllm_quant.py:288-345, 348-395, 493-554) done one by one with
the same quantizers: bit for bit for the quantisation hooks, the GEMM tolerance for the linear method."""
import numpy as np
import pytest

from util import load_formats, make_quantizer

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _spans_ref(positions, n):
    pos = positions.cpu().tolist()
    starts = [0] + [i for i in range(1, n) if pos[i] != pos[i - 1] + 1] + [n]
    return list(zip(starts, starts[1:]))


@pytest.mark.parametrize("name", ["hbq_a_kv4", "nvfp4", "hbq_a_act"])
def test_flattened_token_hooks(name):
    from hbq_b200 import serving
    q = make_quantizer(load_formats()[name])
    Hq, Hkv, D = 8, 2, 128
    # a scheduled batch: a 300-token prefill, three decode tokens of other requests, a 130-token prefill
    positions = torch.cat([torch.arange(300), torch.tensor([57, 9, 1200]), torch.arange(130)]).cuda()
    n = positions.numel()
    g = torch.Generator(device="cuda").manual_seed(3)
    qf = torch.randn((n, Hq * D), device="cuda", generator=g).half()
    kf = torch.randn((n, Hkv * D), device="cuda", generator=g).half()
    vf = torch.randn((n, Hkv * D), device="cuda", generator=g).half()
    assert serving.sequence_spans_from_positions(positions, n) == _spans_ref(positions, n)
    assert serving.sequence_spans_from_positions(positions[:5], n) == [(0, n)]
    assert torch.equal(serving.quantize_post_rope_q(qf, Hq, D, q), q.q(qf.view(n, Hq, D)).view(n, Hq * D))
    assert torch.equal(serving.quantize_k_cache(kf, Hkv, D, q), q.q(kf.view(n, Hkv, D)).view(n, Hkv * D))
    got = serving.quantize_v_cache(vf, Hkv, D, q, positions)
    want = torch.empty_like(vf.view(n, Hkv, D))
    for left, right in _spans_ref(positions, n):          # the reference's permute / quantise / permute per span
        seq = vf.view(n, Hkv, D)[left:right].permute(1, 2, 0).contiguous()
        want[left:right] = q.q(seq).permute(2, 0, 1)
    assert torch.equal(got.view(torch.int16), want.view(n, Hkv * D).view(torch.int16))
    # without positions the whole batch is one span
    one = serving.quantize_v_cache(vf, Hkv, D, q)
    assert torch.equal(one.view(n, Hkv, D), q.q(vf.view(n, Hkv, D).permute(1, 2, 0).contiguous()).permute(2, 0, 1))


def test_k_centre_follows_a_sequence_from_prefill_to_decode():
    from hbq_b200 import serving
    Hkv, D = 2, 64
    tr = serving.KCenterTracker()
    g = torch.Generator(device="cuda").manual_seed(4)
    k0 = torch.randn((40, Hkv * D), device="cuda", generator=g).half()
    c0 = tr(k0, torch.arange(40).cuda(), Hkv, D)
    centre = k0.view(40, Hkv, D).mean(dim=0, keepdim=True)
    assert torch.equal(c0.view(40, Hkv, D), k0.view(40, Hkv, D) - centre)
    k1 = torch.randn((2, Hkv * D), device="cuda", generator=g).half()          # its next token + a stranger's
    c1 = tr(k1, torch.tensor([40, 7]).cuda(), Hkv, D)
    assert torch.equal(c1.view(2, Hkv, D)[0], (k1.view(2, Hkv, D)[0:1] - centre)[0])
    assert torch.equal(c1[1], k1[1])                                             # no centre queued for position 7
    c2 = tr(k1[:1], torch.tensor([41]).cuda(), Hkv, D)                           # the centre moved on to position 41
    assert torch.equal(c2.view(1, Hkv, D), k1.view(2, Hkv, D)[0:1] - centre)
    assert list(tr.center_by_pos) == [42]


@pytest.mark.parametrize("tokens", [1, 8, 96])
def test_linear_method_at_decode_shapes(tokens):
    import hbq_b200 as H
    from hbq_b200 import serving
    f = load_formats()
    method = serving.HBQLinearMethod(make_quantizer(f["hbq_a_act"]), make_quantizer(f["hbq_a_wgt"]))
    K, N = 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(tokens)
    layer = torch.nn.Linear(K, N, bias=True, device="cuda", dtype=torch.float16)
    layer.weight.data = (0.02 * torch.randn((N, K), device="cuda", generator=g)).half()
    w0 = layer.weight.data.clone()
    method.process_weights_after_loading(layer)
    assert torch.equal(layer.weight.data, method.wgt_quantizer.q(w0))
    method.process_weights_after_loading(layer)                    # marked: not quantised twice
    assert torch.equal(layer.weight.data, method.wgt_quantizer.q(w0))
    x = torch.randn((tokens, K), device="cuda", generator=g).half()
    l0 = H.launch_count()
    y = method.apply(layer, x, layer.bias)
    assert H.launch_count() - l0 == 2 and H.gemm_status() == 0     # one quantize, one GEMM (bias in its store)
    ref = torch.nn.functional.linear(method.act_quantizer.q(x).float(), layer.weight.detach().float(), layer.bias.detach().float())
    rel = float((y.float() - ref).norm() / ref.norm())
    assert y.shape == (tokens, N) and rel <= 2.0 ** -9, rel
    y3 = method.apply(layer, x.view(1, tokens, K), layer.bias)
    assert y3.shape == (1, tokens, N) and torch.equal(y3[0], y)


def test_linear_method_on_packed_weights():
    """``packed_weights``: the layer keeps 0.5625 B per weight and no fp16 tensor; outputs agree with the fp16 path."""
    from hbq_b200 import serving
    fm = load_formats()
    K, N = 2048, 1024
    g = torch.Generator(device="cuda").manual_seed(11)
    w0 = (0.02 * torch.randn((N, K), device="cuda", generator=g)).half()
    outs = []
    for packed in (False, True):
        method = serving.HBQLinearMethod(make_quantizer(fm["hbq_e_act"]), make_quantizer(fm["hbq_e_wgt"]), packed_weights=packed)
        layer = torch.nn.Linear(K, N, bias=True, device="cuda", dtype=torch.float16)
        layer.weight.data = w0.clone()
        layer.bias.data = torch.linspace(-1, 1, N, device="cuda").half()
        method.process_weights_after_loading(layer)
        assert (layer.weight.numel() == 0) == packed
        if packed:
            assert layer.hbq_w4_weight.nbytes() * 128 * 128 == N * K * 9216
        x = torch.randn((3, 50, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(12)).half()
        outs.append(method.apply(layer, x, layer.bias.data))
        assert outs[-1].shape == (3, 50, N)
    rel = float((outs[0].double() - outs[1].double()).norm() / outs[0].double().norm())
    assert rel <= 2.0 ** -9, rel


def test_linear_method_decode_batches_on_the_packed_weight():
    """``packed_max_rows``: the fp16 tensor stays, decode-sized batches take the packed kernel (one GEMM launch of this
    library per call either way), larger ones the fp16 tensor; both agree with the plain method."""
    import hbq_b200 as H
    from hbq_b200 import serving
    fm = load_formats()
    K, N = 2048, 1024
    g = torch.Generator(device="cuda").manual_seed(13)
    w0 = (0.02 * torch.randn((N, K), device="cuda", generator=g)).half()
    layers = []
    for rows_max in (0, 16):
        method = serving.HBQLinearMethod(make_quantizer(fm["hbq_a_act"]), make_quantizer(fm["hbq_a_wgt"]), packed_max_rows=rows_max)
        layer = torch.nn.Linear(K, N, bias=False, device="cuda", dtype=torch.float16)
        layer.weight.data = w0.clone()
        method.process_weights_after_loading(layer)
        assert layer.weight.numel() == N * K and (getattr(layer, "hbq_w4_weight", None) is not None) == (rows_max > 0)
        layers.append((method, layer))
    assert torch.equal(layers[0][1].weight.data, layers[1][1].weight.data)
    for rows in (1, 16, 17, 200):
        x = torch.randn((rows, K), device="cuda", generator=g).half()
        y0 = layers[0][0].apply(layers[0][1], x)
        y1 = layers[1][0].apply(layers[1][1], x)
        rel = float((y0.double() - y1.double()).norm() / y0.double().norm())
        assert y1.shape == (rows, N) and rel <= 2.0 ** -9, (rows, rel)
        if rows > 16:
            assert torch.equal(y0, y1)                 # the same kernel on the same fp16 tensor
    assert H.gemm_status() == 0
