"""GPU: the expert-parallel MoE block with the CUDA quantizers and GEMM kernels.  Rows are independent
in every kernel of the path, so however the token copies are grouped and wherever they are computed
the block's output must be the same bits: packed dispatch == fp16 dispatch == a direct per-expert
evaluation, on one GPU and (two ranks over NCCL, skipped with fewer than two GPUs) across ranks."""
import os
import socket

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ACT = dict(block_size=128, ebit=2, mbit=2, sc_ebit=5, sc_mbit=3, l2_block_size=32, l2_sc_bit=2, l2_scheme="SIG-1")
E, HID, INT, TOPK = 4, 256, 512, 2


def _build(H, dev, group, packed, seed=9):
    g = torch.Generator(device=dev).manual_seed(seed)
    gate = torch.randn((E, HID), device=dev, generator=g).half()
    ws = [tuple((0.05 * torch.randn(shape, device=dev, generator=g)).half() for shape in ((INT, HID), (INT, HID), (HID, INT)))
          for _ in range(E)]
    moe = H.ExpertParallelMoE(HID, INT, E, top_k=TOPK, group=group, packed_dispatch=packed, device=dev, dtype=torch.float16,
                              ops_factory=lambda: H.FP16AccumMatMul(group_size=128, quant_block_size=32))
    moe.aq = H.HBQQuantizer(**ACT)
    with torch.no_grad():
        moe.gate.weight.copy_(gate)
        for i, ex in enumerate(moe.experts):
            w1, w3, w2 = ws[moe.e0 + i]
            ex.w1.weight.copy_(w1); ex.w3.weight.copy_(w3); ex.w2.weight.copy_(w2)
            ex.w2.aq = H.HBQQuantizer(**ACT)
    return moe, ws


def _direct(H, moe, ws, x):
    """Every expert on the tokens routed to it, with the same kernels, no sorting or exchange."""
    import torch.nn.functional as F
    x2 = x.reshape(-1, HID)
    w, idx = moe.route(x2)
    aq, aq2 = H.HBQQuantizer(**ACT), H.HBQQuantizer(**ACT)
    op = H.FP16AccumMatMul(group_size=128, quant_block_size=32)
    y = torch.zeros_like(x2)
    for e in range(E):
        tok, choice = torch.where(idx == e)
        if tok.numel() == 0:
            continue
        xq = aq(x2[tok])
        h = F.silu(op(xq, ws[e][0])) * op(xq, ws[e][1])
        y.index_add_(0, tok, op(aq2(h), ws[e][2]) * w[tok, choice].unsqueeze(1))
    return y.reshape(x.shape)


def test_one_gpu_packed_equals_plain_equals_direct():
    import hbq_b200 as H
    dev = torch.device("cuda", 0)
    x = torch.randn((3, 100, HID), device=dev).half()
    plain, ws = _build(H, dev, None, False)
    packed, _ = _build(H, dev, None, True)
    with torch.no_grad():
        y0, y1, y2 = plain(x), packed(x), _direct(H, plain, ws, x)
    assert torch.isfinite(y0).all()
    assert torch.equal(y0.view(torch.int16), y1.view(torch.int16))
    assert torch.equal(y0.view(torch.int16), y2.view(torch.int16))
    assert H.gemm_status() == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import hbq_b200 as H
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    solo = [dist.new_group([r]) for r in range(world)][rank]          # a one-rank group: all experts local
    x = torch.randn((2, 150 + 40 * rank, HID), device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank)).half()
    msgs = []
    local, ws = _build(H, dev, solo, False)
    with torch.no_grad():
        want = local(x)
        for packed in (False, True):
            ep, _ = _build(H, dev, None, packed)
            got = ep(x)
            if ep.per_rank != E // world:
                msgs.append("experts not split")
            if not torch.equal(got.view(torch.int16), want.view(torch.int16)):
                msgs.append(f"expert-parallel result differs (packed={packed})")
    torch.cuda.synchronize()
    if H.gemm_status() != 0:
        msgs.append("a bounded wait expired inside the tensor-core kernel")
    allm = [None] * world
    dist.all_gather_object(allm, msgs)
    if rank == 0:
        with open(os.path.join(out_dir, "result"), "w") as fh:
            fh.write("ok" if not any(allm) else repr(allm))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpus_equal_all_experts_local(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "result").read_text() == "ok"
