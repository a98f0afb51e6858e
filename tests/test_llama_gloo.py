"""CPU, world_size 2 over gloo: the host logic of the tensor/sequence-parallel Llama decoder -- which heads, MLP
features, vocabulary columns and tokens a rank owns, the all-gather / reduce-scatter of token shards, the batch cut
into pieces.  The CUDA kernels are replaced by their torch definitions (identity quantizers), so the two-rank model
must reproduce the one-rank model up to fp16 summation order."""
import os
import socket

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torch_stand_ins():
    """torch definitions of the kernels the model calls, for CPU ranks."""
    import hbq_b200.llama as L

    def rmsnorm_quantize(x, weight, eps, quantizer=None, residual=None, inplace=True):
        xs = x if residual is None else x + residual
        xf = xs.float()
        h = weight * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
        return (h if quantizer is None else quantizer(h)), xs

    def softmax_quantize(scores, scale, quantizer=None, causal=False, q_len=None, heads=None, mask=None, inplace=True):
        S = scores.shape[-1]
        w = scores.float() * scale
        if causal:
            rows = torch.arange(scores.shape[-2]) % q_len
            keep = torch.arange(S)[None, :] <= (rows[:, None] + S - q_len)
            w = w.masked_fill(~keep, float("-inf"))
        p = torch.softmax(w, dim=-1).to(scores.dtype)
        return p if quantizer is None else quantizer(p)

    L.rmsnorm_quantize, L.softmax_quantize = rmsnorm_quantize, softmax_quantize
    L.ext.gemm_fp32_accum = lambda a, w, b_is_nk=True, bias=None, out=None: torch.nn.functional.linear(a.float(), w.float(), bias).to(a.dtype)
    L.kvcache.swiglu_quantize = lambda g, u, q: q(torch.nn.functional.silu(g) * u)


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import hbq_b200 as H
    _torch_stand_ins()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    arch = H.LlamaArch(hidden=128, layers=2, heads=4, kv_heads=2, head_dim=32, ffn=256, vocab=64)
    ids = torch.randint(0, arch.vocab, (4, 16), generator=torch.Generator().manual_seed(0))
    whole = H.QLlamaModel(arch, parallel=False)
    whole.init_weights(5)
    want = whole(ids).float()
    ok = True
    for pieces in (1, 2):
        tp = H.QLlamaModel(arch, pieces=pieces)
        tp.init_weights(5)
        at, ml = tp.layers[0].self_attn, tp.layers[0].mlp
        ok = ok and (tp.world, at.num_heads, at.num_key_value_heads, ml.f, tp.lm_head.out_features) == (2, 2, 1, 128, 32)
        ok = ok and (at.h0, at.kv0, ml.f0) == (2 * rank, rank, 128 * rank)
        ok = ok and torch.equal(at.q_proj.weight, whole.layers[0].self_attn.q_proj.weight[at.h0 * 32:(at.h0 + 2) * 32])
        ok = ok and torch.equal(ml.down_proj.weight, whole.layers[0].mlp.down_proj.weight[:, ml.f0:ml.f0 + 128])
        cols = tp(ids).float()                                   # this rank's vocabulary columns
        ok = ok and cols.shape == (64, 32)
        ok = ok and torch.allclose(cols, want[:, 32 * rank:32 * rank + 32], rtol=2e-2, atol=2e-3)
        full = tp(ids, gather_logits=True).float()
        ok = ok and full.shape == want.shape and torch.allclose(full, want, rtol=2e-2, atol=2e-3)
    # the Mixtral layer: attention as above, experts spread over the ranks, tokens routed by all-to-all
    moe_arch = H.LlamaArch(hidden=128, layers=2, heads=4, kv_heads=2, head_dim=32, ffn=256, vocab=64, num_experts=4, top_k=2)
    whole = H.QLlamaModel(moe_arch, parallel=False)
    whole.init_weights(6)
    want = whole(ids).float()
    ep = H.QLlamaModel(moe_arch, pieces=2)
    ep.init_weights(6)
    moe = ep.layers[0].block_sparse_moe
    ok = ok and (moe.world, moe.per_rank, moe.e0, len(whole.layers[0].block_sparse_moe.experts)) == (2, 2, 2 * rank, 4)
    ok = ok and torch.equal(moe.experts[1].w2.weight, whole.layers[0].block_sparse_moe.experts[2 * rank + 1].w2.weight)
    full = ep(ids, gather_logits=True).float()
    # a token whose two best router scores nearly tie may take another expert when the hidden state differs in its
    # last fp16 bit: rows are compared one by one and a few may differ
    good = ((full - want).abs() <= 2e-3 + 2e-2 * want.abs()).all(dim=1)
    ok = ok and full.shape == want.shape and float(good.float().mean()) >= 0.95
    try:
        H.QLlamaModel(H.LlamaArch(hidden=128, layers=1, heads=3, kv_heads=3, head_dim=32, ffn=256, vocab=64))
        ok = False                                               # 3 heads do not divide over 2 ranks
    except ValueError:
        pass
    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    if rank == 0:
        with open(os.path.join(out_dir, "ok"), "w") as fh:
            fh.write("1" if all(flags) else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_decoder_equals_one_rank(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").read_text() == "1"
