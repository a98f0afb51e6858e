"""CPU, world_size 2 over gloo: routing, dispatch and combine of the expert-parallel MoE block with
identity quantizers and ``F.linear`` experts in fp32, against a dense single-process evaluation of the
same block (every expert applied to its tokens, weighted and summed)."""
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


def _make_weights(E, hidden, inter):
    g = torch.Generator().manual_seed(5)
    gate = torch.randn(E, hidden, generator=g)
    ws = [(torch.randn(inter, hidden, generator=g) * 0.1, torch.randn(inter, hidden, generator=g) * 0.1,
           torch.randn(hidden, inter, generator=g) * 0.1) for _ in range(E)]
    x = torch.randn(3, 11, hidden, generator=g)
    return gate, ws, x


def _dense(gate, ws, x, top_k):
    import torch.nn.functional as F
    x2 = x.reshape(-1, x.shape[-1])
    p = F.softmax(x2 @ gate.t(), dim=-1, dtype=torch.float32)
    w, idx = torch.topk(p, top_k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    y = torch.zeros_like(x2)
    for t in range(x2.shape[0]):
        for j in range(top_k):
            w1, w3, w2 = ws[int(idx[t, j])]
            h = F.silu(x2[t] @ w1.t()) * (x2[t] @ w3.t())
            y[t] += w[t, j] * (h @ w2.t())
    return y.reshape(x.shape)


def _load(moe, gate, ws):
    with torch.no_grad():
        moe.gate.weight.copy_(gate)
        for i, ex in enumerate(moe.experts):
            w1, w3, w2 = ws[moe.e0 + i]
            ex.w1.weight.copy_(w1); ex.w3.weight.copy_(w3); ex.w2.weight.copy_(w2)


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import hbq_b200 as H
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    E, hidden, inter, k = 4, 32, 48, 2
    gate, ws, x = _make_weights(E, hidden, inter)
    moe = H.ExpertParallelMoE(hidden, inter, E, top_k=k)
    _load(moe, gate, ws)
    with torch.no_grad():
        y = moe(x)
    ok = moe.per_rank == E // world and torch.allclose(y, _dense(gate, ws, x, k), rtol=1e-4, atol=1e-5)
    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    if rank == 0:
        with open(os.path.join(out_dir, "ok"), "w") as fh:
            fh.write("1" if all(flags) else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_world2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").read_text() == "1"


def test_single_process_all_experts_local():
    import hbq_b200 as H
    E, hidden, inter, k = 4, 32, 48, 2
    gate, ws, x = _make_weights(E, hidden, inter)
    moe = H.ExpertParallelMoE(hidden, inter, E, top_k=k)
    _load(moe, gate, ws)
    with torch.no_grad():
        y = moe(x)
    assert torch.allclose(y, _dense(gate, ws, x, k), rtol=1e-4, atol=1e-5)
