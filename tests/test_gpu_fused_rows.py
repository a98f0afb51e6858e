"""GPU: the row-wise producers fused into the activation quantizer (hbq_rmsnorm_quantize, hbq_softmax_quantize).

Two statements per kernel.  (1) The producer alone (no quantizer) against the reference's chain of fp16 tensor ops
run by torch on the same GPU: the reductions are summed in another order, so the comparison allows one fp16 ulp (two after
the norm's second rounding) on a small fraction of the outputs (stated below).  (2) The fused quantised output against the CPU oracle's quantizer
applied to the producer's own output: bit for bit -- the fusion must not change a single code."""
import math

import numpy as np
import pytest

from util import bits, load_formats, make_quantizer, oracle_format

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ULP_FRACTION = 2e-3        # share of outputs that may sit one fp16 ulp from torch's (different summation order)


def _ulp(a, b):
    ai, bi = a.view(torch.int16).to(torch.int32), b.view(torch.int16).to(torch.int32)
    al = torch.where(ai < 0, -(ai & 0x7FFF), ai)
    blv = torch.where(bi < 0, -(bi & 0x7FFF), bi)
    return (al - blv).abs()


def _close(got, ref, what, max_ulp=1):
    d = _ulp(got, ref)
    assert int(d.max()) <= max_ulp, f"{what}: {int(d.max())} ulps"
    frac = float((d != 0).float().mean())
    assert frac <= ULP_FRACTION, f"{what}: {frac:.2e} of the outputs differ"


def _rmsnorm_ref(x, w, eps):
    xf = x.float()
    return w * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(torch.float16)


@pytest.mark.parametrize("name", ["hbq_a_act", "hbq_e_act", "hbq_a_kv4", "mxfp4", None])
@pytest.mark.parametrize("K", [4096, 1152])
def test_rmsnorm_quantize(oracle, name, K):
    import hbq_b200 as H
    from hbq_b200 import fused
    g = torch.Generator(device="cuda").manual_seed(K + (hash(name) % 97))
    rows = 300
    x = torch.randn((rows, K), device="cuda", generator=g).half()
    x[:, 7] *= 20                                          # an outlier channel, as real hidden states have
    x[5, :64] = 0
    x[6, 3] = -0.0
    r = (0.3 * torch.randn((rows, K), device="cuda", generator=g)).half()
    w = (1 + 0.1 * torch.randn(K, device="cuda", generator=g)).half()
    eps = 1e-5
    spec = load_formats()[name] if name else None
    q = make_quantizer(spec) if spec else None
    # (1) the producer alone
    h, xs = H.rmsnorm_quantize(x.clone(), w, eps, None, residual=r)
    assert torch.equal(xs, x + r)
    # two roundings follow the reduction (x * rstd, then * weight): one ulp in the first can become two after the second
    _close(h, _rmsnorm_ref(x + r, w, eps), "rmsnorm", max_ulp=2)
    h0, x0 = H.rmsnorm_quantize(x, w, eps, None)
    assert x0.data_ptr() == x.data_ptr()
    _close(h0, _rmsnorm_ref(x, w, eps), "rmsnorm without residual", max_ulp=2)
    if q is None:
        return
    # (2) fused == quantizer on the producer's output, bit for bit (oracle on every row)
    xin = x.clone()
    hq, xs2 = H.rmsnorm_quantize(xin, w, eps, q, residual=r)
    assert xs2.data_ptr() == xin.data_ptr() and torch.equal(xs2, x + r)
    assert fused.fused_last == (spec["kind"] == "hbq")
    ref = oracle.quantize(h.cpu().numpy(), oracle_format(oracle, spec), False)["deq"]
    n = int((bits(hq.cpu().numpy()) != bits(ref)).sum())
    assert n == 0, f"{n} mismatches against the oracle"
    assert torch.equal(hq.view(torch.int16), q.q(h).view(torch.int16))
    hq_np, _ = H.rmsnorm_quantize(x.clone(), w, eps, q, residual=r, inplace=False)
    assert torch.equal(hq_np.view(torch.int16), hq.view(torch.int16))


def _softmax_ref(s, scale, causal, mask):
    """manual_sdpa's chain on fp16 tensors (src/module.py:93-113)."""
    L, S = s.shape[-2], s.shape[-1]
    bias = torch.zeros(L, S, dtype=s.dtype, device=s.device)
    if causal:
        keep = torch.ones(L, S, dtype=torch.bool, device=s.device).tril(diagonal=S - L)
        bias.masked_fill_(keep.logical_not(), float("-inf"))
    w = s * scale
    w = w + bias
    if mask is not None:
        w = w + mask
    return torch.softmax(w, dim=-1)


@pytest.mark.parametrize("name", ["hbq_a_act", "hbq_e_act", "mxfp4_round", None])
@pytest.mark.parametrize("shape", [(2, 4, 384, 384), (1, 3, 130, 2560), (2, 2, 1, 1280)], ids=["prefill", "chunked", "decode"])
def test_softmax_quantize(oracle, name, shape):
    import hbq_b200 as H
    from hbq_b200 import fused
    B, Hh, L, S = shape
    g = torch.Generator(device="cuda").manual_seed(L + S)
    s = (8 * torch.randn(shape, device="cuda", generator=g)).half()
    scale = 1 / math.sqrt(128)
    spec = load_formats()[name] if name else None
    q = make_quantizer(spec) if spec else None
    for causal, with_mask in ((True, False), (False, False), (False, True)):
        mask = None
        if with_mask:
            mask = torch.zeros((B, 1, L, S), device="cuda", dtype=torch.float16)
            mask[..., S // 3: S // 2] = float("-inf")
            mask[0, ..., :5] = -2.0
        p = H.softmax_quantize(s, scale, None, causal=causal, mask=mask, inplace=False)
        _close(p, _softmax_ref(s, scale, causal, mask), f"softmax causal={causal} mask={with_mask}")
        assert torch.isfinite(p).all() and float(p.sum(-1).sub(1).abs().max()) < 2e-2
        if q is None:
            continue
        pq = H.softmax_quantize(s, scale, q, causal=causal, mask=mask, inplace=False)
        assert fused.fused_last == (spec["kind"] == "hbq")
        sel = np.arange(0, B * Hh * L, 3)                        # a third of the rows through the oracle
        ref = oracle.quantize(p.reshape(-1, S)[sel].cpu().numpy(), oracle_format(oracle, spec), False)["deq"]
        n = int((bits(pq.reshape(-1, S)[sel].cpu().numpy()) != bits(ref)).sum())
        assert n == 0, f"{n} mismatches against the oracle (causal={causal}, mask={with_mask})"
        assert torch.equal(pq.view(torch.int16), q.q(p).view(torch.int16))
    # the head axis folded into the rows (how a grouped-query block batches its matmuls), in place
    if q is not None:
        want = H.softmax_quantize(s, scale, q, causal=True, inplace=False)
        folded = s.reshape(B, Hh * L, S).clone()
        got = H.softmax_quantize(folded, scale, q, causal=True, q_len=L, heads=Hh)
        assert torch.equal(got.view(B, Hh, L, S), want)
        assert got.data_ptr() == folded.data_ptr() or not fused.fused_last       # in place when fused


def test_ragged_rows_take_the_reference_ops():
    """Row lengths outside the kernels (not a multiple of 8) run the reference's own tensor ops."""
    import hbq_b200 as H
    x = torch.randn((9, 100), device="cuda").half()
    w = torch.ones(100, device="cuda").half()
    h, _ = H.rmsnorm_quantize(x, w, 1e-6)
    _close(h, _rmsnorm_ref(x, w, 1e-6), "ragged rmsnorm", max_ulp=2)
    s = torch.randn((2, 2, 5, 77), device="cuda").half()
    p = H.softmax_quantize(s, 0.5, None, causal=True, inplace=False)
    _close(p, _softmax_ref(s, 0.5, True, None), "ragged softmax")
    h2, _ = H.rmsnorm_quantize(torch.randn((4, 200), device="cuda").half(), torch.ones(200, device="cuda").half(), 1e-6)
    assert h2.shape == (4, 200)                      # K = 200: a multiple of 8 but not of 128, unquantised form
