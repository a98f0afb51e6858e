"""GPU: the fused KV-cache write kernels against the steps the reference runs one by one
(view/transpose, apply_rotary_pos_emb in fp16, kv_quantizer.q; src/module.py:147-168), and
against the CPU oracle applied to the rotated tensor.  Bit-exact on fp16 patterns."""
import numpy as np
import pytest

from util import seeded_inputs

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def hbits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def rope_tables(B, T, D, per_batch, seed=0):
    """cos/sin as LlamaRotaryEmbedding builds them (fp32 angles, cast to fp16), [B or 1, T, D]."""
    g = torch.Generator().manual_seed(seed)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    lead = B if per_batch else 1
    pos = torch.stack([torch.randperm(4096, generator=g)[:T].float() for _ in range(lead)])      # [lead, T]
    ang = pos[:, :, None] * inv_freq[None, None, :]
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().half().cuda(), emb.sin().half().cuda()


def unfused_k(k, H, q, cos, sin):
    from hbq_b200.kvcache import apply_rope
    B, T = k.shape[:2]
    x = k.view(B, T, H, -1).transpose(1, 2)
    if cos is not None:
        x = apply_rope(x, cos, sin)
    return x.contiguous(), q.q(x.contiguous())


def quantizers():
    import hbq_b200 as Hq
    return {
        "hbq_a_sig1_l8": lambda: Hq.HBQQuantizer(128, 2, 2, 5, 3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1"),
        "hbq_e_fp1_l32": lambda: Hq.HBQQuantizer(128, 2, 1, 5, 3, l2_block_size=32, l2_sc_bit=2, l2_scheme="FP-1"),
        "hbq_b64": lambda: Hq.HBQQuantizer(64, 2, 3, 5, 3, l2_block_size=8, l2_sc_bit=2, l2_scheme="INT"),
        "hbq_sig1_b32": lambda: Hq.HBQQuantizer(32, 2, 2, 5, 3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1"),
        "mxfp4_b32": lambda: Hq.MXFPQuantizer(32, 2, 1, 8, 0),
        "mxfp4_e5_b32": lambda: Hq.MXFPQuantizer(32, 2, 1, 5, 0),        # config/mxfp4.yaml
        "nvfp4_b16": lambda: Hq.MXFPQuantizer(16, 2, 1, 5, 3),
        "mxfp8ish_b32": lambda: Hq.MXFPQuantizer(32, 2, 5, 5, 0),
        "mxint8_b32": lambda: Hq.MXINTQuantizer(8, 5, 0, 32),
        "mxfp_e4m3_b32": lambda: Hq.MXFPQuantizer(32, 4, 3, 8, 0),
        "hbq_mix_l4": lambda: Hq.HBQQuantizer(128, 2, 1, 5, 3, l2_block_size=4, l2_sc_bit=1, l2_scheme="Mix"),
        "mxfp_pts": lambda: Hq.MXFPQuantizer(32, 2, 1, 5, 3, per_tensor_scale=True),       # needs the tensor maximum first
    }


@pytest.mark.parametrize("name", list(quantizers()))
@pytest.mark.parametrize("per_batch", [False, True])
def test_k_write_matches_unfused(name, per_batch, oracle):
    from hbq_b200 import kvcache
    from util import oracle_format  # noqa: F401
    B, T, H, D = 2, 77, 8, 128
    q = quantizers()[name]()
    k = torch.from_numpy(seeded_inputs("act", B * T, H * D, seed=5).astype(np.float16)).cuda().view(B, T, H * D)
    cos, sin = rope_tables(B, T, D, per_batch)
    got = kvcache.write_k_cache(k, H, q, cos, sin)
    assert kvcache.fused_last == (name != "mxfp_pts")
    rot, want = unfused_k(k, H, q, cos, sin)
    torch.cuda.synchronize()
    assert got.shape == (B, H, T, D)
    bad = hbits(got) != hbits(want)
    assert not bad.any(), f"{name}: {bad.sum()} of {bad.size} differ"
    if name.startswith("hbq_a"):
        # the oracle on the rotated tensor: pins the chain to the CPU restatement as well
        f = q._format()
        of = oracle.Format(oracle.KIND_HBQ, f.ebit, f.mbit, f.sc_ebit, f.sc_mbit, f.block_size,
                           l2_block_size=f.l2_block_size, l2_sc_bit=f.l2_sc_bit, l2_scheme="SIG-1")
        ref = oracle.quantize(hbits(rot).reshape(-1, D), of)["deq"]
        assert np.array_equal(hbits(got).reshape(-1, D), np.ascontiguousarray(ref).view(np.uint16).reshape(-1, D))


@pytest.mark.parametrize("D", [64, 128, 256])
def test_k_write_head_dims(D):
    from hbq_b200 import kvcache
    import hbq_b200 as Hq
    B, T, H = 1, 130, 3
    for q in (Hq.HBQQuantizer(64, 2, 2, 5, 3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1"), Hq.MXFPQuantizer(32, 2, 1, 8, 0)):
        k = torch.from_numpy(seeded_inputs("studt", B * T, H * D, seed=D).astype(np.float16)).cuda().view(B, T, H, D)
        cos, sin = rope_tables(B, T, D, False, seed=D)
        got = kvcache.write_k_cache(k, H, q, cos, sin)
        assert kvcache.fused_last
        _, want = unfused_k(k.view(B, T, H * D), H, q, cos, sin)
        assert np.array_equal(hbits(got), hbits(want))


def test_k_write_no_rope_bf16_and_empty():
    from hbq_b200 import kvcache
    import hbq_b200 as Hq
    q = Hq.HBQQuantizer(128, 2, 2, 5, 3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")
    B, T, H, D = 2, 33, 4, 128
    k = torch.from_numpy(seeded_inputs("act", B * T, H * D, seed=9)).cuda().to(torch.bfloat16).view(B, T, H * D)
    got = kvcache.write_k_cache(k, H, q)
    assert kvcache.fused_last and got.dtype == torch.bfloat16
    want = q.q(k.view(B, T, H, D).transpose(1, 2).contiguous())
    assert torch.equal(got, want)
    # bf16 with RoPE: the rotation is bf16 arithmetic in the reference, which the fp16 kernel does not model
    cos, sin = rope_tables(B, T, D, False)
    got = kvcache.write_k_cache(k, H, q, cos.bfloat16(), sin.bfloat16())
    assert not kvcache.fused_last
    e = kvcache.write_k_cache(k[:, :0], H, q)
    assert e.shape == (B, H, 0, D)


@pytest.mark.parametrize("name", ["hbq_a_sig1_l8", "hbq_e_fp1_l32", "hbq_sig1_b32", "hbq_b64", "mxfp4_b32",
                                  "mxfp4_e5_b32", "nvfp4_b16", "mxfp8ish_b32", "mxint8_b32"])
@pytest.mark.parametrize("T", [1, 128, 300])
def test_v_write_matches_unfused(name, T):
    from hbq_b200 import kvcache
    B, H, D = 2, 4, 128
    q = quantizers()[name]()
    v = torch.from_numpy(seeded_inputs("act", B * T, H * D, seed=T).astype(np.float16)).cuda().view(B, T, H * D)
    got = kvcache.write_v_cache(v, H, q)
    # the token-axis kernels serve the table-driven HBQ formats and the MX / NV fast-path formats;
    # the others (8-bit scale exponent, E2M3 with an INT table) run the three steps
    assert kvcache.fused_last == (name not in ("hbq_b64", "mxfp4_b32"))
    x = v.view(B, T, H, D).transpose(1, 2)                                  # [B,H,T,D]
    want = q.q(x.transpose(-1, -2).contiguous()).transpose(-1, -2).contiguous()      # src/module.py:163-168
    assert got.shape == (B, H, T, D)
    bad = hbits(got) != hbits(want)
    assert not bad.any(), f"{name} T={T}: {bad.sum()} of {bad.size} differ"


def test_v_write_bf16_d64():
    from hbq_b200 import kvcache
    import hbq_b200 as Hq
    q = Hq.HBQQuantizer(128, 2, 2, 5, 3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")
    B, T, H, D = 1, 200, 5, 64
    v = torch.from_numpy(seeded_inputs("wgt", B * T, H * D, seed=2)).cuda().to(torch.bfloat16).view(B, T, H * D)
    got = kvcache.write_v_cache(v, H, q)
    assert kvcache.fused_last
    want = q.q(v.view(B, T, H, D).permute(0, 2, 3, 1).contiguous()).transpose(-1, -2).contiguous()
    assert torch.equal(got, want)
    assert kvcache.write_v_cache(v[:, :0], H, q).shape == (B, H, 0, D)


@pytest.mark.parametrize("name", ["hbq_a_sig1_l8", "nvfp4_b16", "hbq_mix_l4", "mxfp_e4m3_b32"])
def test_k_write_with_centre(name):
    """K-cache centring of the Qwen2 block (src/module.py:221-244): quantise key_states - center."""
    from hbq_b200 import kvcache
    B, T, H, D = 2, 50, 4, 128
    q = quantizers()[name]()
    k = torch.from_numpy(seeded_inputs("act", B * T, H * D, seed=11).astype(np.float16)).cuda().view(B, T, H * D) + 3.0
    cos, sin = rope_tables(B, T, D, False)
    rot = kvcache.apply_rope(k.view(B, T, H, D).transpose(1, 2), cos, sin)
    center = rot.mean(dim=-2, keepdim=True)                       # [B,H,1,D], as the reference computes it at prefill
    got = kvcache.write_k_cache(k, H, q, cos, sin, center=center)
    assert kvcache.fused_last
    want = q.q((rot - center).contiguous())
    bad = hbits(got) != hbits(want)
    assert not bad.any(), f"{name}: {bad.sum()} of {bad.size} differ"
    # without rotation
    got = kvcache.write_k_cache(k, H, q, center=center)
    want = q.q((k.view(B, T, H, D).transpose(1, 2) - center).contiguous())
    assert np.array_equal(hbits(got), hbits(want))


@pytest.mark.parametrize("name", ["hbq_a_sig1_l8", "nvfp4_b16", "mxfp4_b32"])
def test_v_write_token_major(name):
    """Flattened-token layout of a serving engine: the result stays [B,T,H,D]."""
    from hbq_b200 import kvcache
    B, T, H, D = 1, 173, 8, 128
    q = quantizers()[name]()
    v = torch.from_numpy(seeded_inputs("act", B * T, H * D, seed=13).astype(np.float16)).cuda().view(B, T, H * D)
    got = kvcache.write_v_cache(v, H, q, token_major=True)
    assert got.shape == (B, T, H, D)
    want = kvcache.write_v_cache(v, H, q)                      # [B,H,T,D], checked against the unfused chain above
    assert torch.equal(got, want.permute(0, 2, 1, 3).contiguous())


@pytest.mark.parametrize("name", ["hbq_a_sig1_l8", "hbq_e_fp1_l32", "hbq_sig1_b32", "mxfp4_b32", "hbq_mix_l4"])
def test_swiglu_quantize_matches_the_three_ops(name):
    """silu(gate) * up followed by the quantizer, fused (HBQ table formats) or not (the rest): the
    same bits as torch's silu, multiplication and the quantizer run one after the other."""
    import torch.nn.functional as F
    import hbq_b200 as Hq
    from hbq_b200 import kvcache
    q = quantizers()[name]()
    g = torch.Generator(device="cuda").manual_seed(17)
    gate = (3.0 * torch.randn((2, 777, 1024), device="cuda", generator=g)).half()
    up = torch.randn((2, 777, 1024), device="cuda", generator=g).half()
    gate[0, 0, :8] = torch.tensor([0.0, -0.0, 65504.0, -65504.0, 1e-7, -1e-7, 20.0, -20.0], device="cuda").half()
    want = q.q(F.silu(gate) * up)
    got = Hq.swiglu_quantize(gate, up, q)
    assert kvcache.fused_last == (name.startswith("hbq_") and name != "hbq_mix_l4")
    assert got.shape == want.shape and got.dtype == want.dtype
    assert np.array_equal(hbits(got), hbits(want)), name
    # every fp16 value as the gate (silu itself, against torch's)
    allg = torch.arange(65536, dtype=torch.int32, device="cuda").to(torch.int16).view(torch.float16)
    allg = allg[torch.isfinite(allg)]
    n = (allg.numel() // 128) * 128
    allg = allg[:n].view(-1, 128).contiguous()
    ones = torch.full_like(allg, 1.0)
    want = q.q(F.silu(allg) * ones)
    got = Hq.swiglu_quantize(allg, ones, q)
    assert np.array_equal(hbits(got), hbits(want)), name + " (all gate values)"
