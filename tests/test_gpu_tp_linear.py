"""GPU, two ranks over NCCL (skipped with fewer than two GPUs): the tensor-parallel linear layers with
the CUDA quantizers and GEMM kernels.  Column-parallel outputs are the unsharded layer's columns bit
for bit; the row-parallel sum differs from the single chain by the ranks' extra fp16 roundings and is
held to the tensor-core tolerance (relative Frobenius error <= 2^-9)."""
import os
import socket

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


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
    g = torch.Generator(device=dev).manual_seed(3)
    T, Hd, I = 1000, 512, 1024
    x = torch.randn((T, Hd), device=dev, generator=g).half()
    w_up = (0.05 * torch.randn((I, Hd), device=dev, generator=g)).half()
    w_down = (0.05 * torch.randn((Hd, I), device=dev, generator=g)).half()
    bias = torch.randn(Hd, device=dev, generator=g).half()
    act = dict(block_size=128, ebit=2, mbit=2, sc_ebit=5, sc_mbit=3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")
    msgs = []
    for ops_kw in (None, dict(group_size=128, quant_block_size=32)):
        mk_ops = (lambda: None) if ops_kw is None else (lambda: H.FP16AccumMatMul(**ops_kw))
        up = H.ColumnParallelQLinear(Hd, I, bias=False, ops=mk_ops(), multiple=128, device=dev, dtype=torch.float16)
        down = H.RowParallelQLinear(I, Hd, bias=True, ops=mk_ops(), row_chunks=3, device=dev, dtype=torch.float16)
        up.load_full(w_up)
        down.load_full(w_down, bias)
        up.aq = H.HBQQuantizer(**act)
        down.aq = H.HBQQuantizer(**act)
        # the unsharded pair on this rank's own GPU
        up1 = H.QLinear(Hd, I, bias=False, ops=mk_ops(), check_finite=False, device=dev, dtype=torch.float16)
        down1 = H.QLinear(I, Hd, bias=True, ops=mk_ops(), check_finite=False, device=dev, dtype=torch.float16)
        up1.weight.data.copy_(w_up); down1.weight.data.copy_(w_down); down1.bias.data.copy_(bias)
        up1.aq = H.HBQQuantizer(**act); down1.aq = H.HBQQuantizer(**act)
        with torch.no_grad():
            h = up(x)
            y = down(h)
            h1 = up1(x)
            y1 = down1(h1)
        torch.cuda.synchronize()
        if ops_kw is not None and not torch.equal(h.view(torch.int16), h1[:, up.n0:up.n1].contiguous().view(torch.int16)):
            msgs.append(f"column-parallel columns differ ({ops_kw})")
        if ops_kw is None:      # F.linear (cuBLAS) against the tensor-core kernel of the sharded layer: tolerance
            rel_h = float((h.float() - h1[:, up.n0:up.n1].float()).norm() / h1[:, up.n0:up.n1].float().norm())
            if rel_h > 2.0 ** -9:
                msgs.append(f"column-parallel fp32 rel {rel_h}")
        rel = float((y.float() - y1.float()).norm() / y1.float().norm())
        if not (rel <= 2.0 ** -9):
            msgs.append(f"row-parallel rel {rel} ({ops_kw})")
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        if not all(torch.equal(ys[0], t) for t in ys):
            msgs.append("ranks hold different reduced results")
    if H.gemm_status() != 0:
        msgs.append("a bounded wait expired inside the tensor-core kernel")
    allm = [None] * world
    dist.all_gather_object(allm, msgs)
    if rank == 0:
        with open(os.path.join(out_dir, "result"), "w") as fh:
            fh.write("ok" if not any(allm) else repr(allm))
    dist.barrier()
    dist.destroy_process_group()


def test_tensor_parallel_pair_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "result").read_text() == "ok"
