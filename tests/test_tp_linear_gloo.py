"""CPU, world_size 2 over gloo: the host logic of the tensor-parallel linear layers (slicing,
the all-reduce of the row-parallel partial products, the all-gather of a column-parallel output).
The kernels themselves need a GPU; here the layers run with the identity quantizer and
``F.linear`` in fp32, so the sharded block must equal the unsharded one up to summation order."""
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


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import hbq_b200 as H
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(7)
    T, Hd, I = 24, 256, 512
    x = torch.randn(2, T // 2, Hd, generator=g)
    w_up = torch.randn(I, Hd, generator=g) * 0.05
    b_up = torch.randn(I, generator=g)
    w_down = torch.randn(Hd, I, generator=g) * 0.05
    b_down = torch.randn(Hd, generator=g)
    up = H.ColumnParallelQLinear(Hd, I, bias=True, multiple=128)     # cut where the K split of `down` cuts
    down = H.RowParallelQLinear(I, Hd, bias=True, row_chunks=2)
    up.load_full(w_up, b_up)
    down.load_full(w_down, b_down)
    ok = (up.n1 - up.n0 == I // world) and (down.k0, down.k1) == (up.n0, up.n1)
    with torch.no_grad():
        h = torch.nn.functional.silu(up(x))                      # stays sharded: [2, T/2, I / world]
        y = down(h)
        ref = torch.nn.functional.linear(torch.nn.functional.silu(torch.nn.functional.linear(x, w_up, b_up)), w_down, b_down)
        gathered = H.ColumnParallelQLinear(Hd, I, bias=True, gather_output=True)
        gathered.load_full(w_up, b_up)
        full_up = gathered(x)
    ok = ok and y.shape == ref.shape and torch.allclose(y, ref, rtol=1e-5, atol=1e-5)
    ok = ok and torch.equal(full_up, torch.nn.functional.linear(x, w_up, b_up))
    # shards of unequal width cannot be all-gathered into equal buffers: refused at construction
    try:
        H.ColumnParallelQLinear(Hd, 96, bias=False, gather_output=True, multiple=32)      # 3 blocks over 2 ranks
        ok = False
    except ValueError:
        pass
    uneven = H.ColumnParallelQLinear(Hd, 96, bias=False, multiple=32)                    # fine while it stays sharded
    ok = ok and (uneven.n1 - uneven.n0) == (64 if rank == 0 else 32)
    # a per-tensor-scaled activation quantizer would make the result depend on the sharding: refused
    down.aq = H.MXFPQuantizer(16, 2, 1, 4, 3, per_tensor_scale=True)
    try:
        down(h)
        ok = False
    except ValueError:
        pass
    # every rank holds the same reduced result
    ys = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(ys, y)
    ok = ok and all(torch.equal(ys[0], t) for t in ys)
    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    if rank == 0:
        with open(os.path.join(out_dir, "ok"), "w") as fh:
            fh.write("1" if all(flags) else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_column_then_row_parallel_world2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").read_text() == "1"


def test_k_split_must_keep_whole_blocks():
    import hbq_b200 as H
    with pytest.raises(ValueError):
        H.RowParallelQLinear(200, 64)            # K not a multiple of the 128-element block
    lin = H.RowParallelQLinear(256, 64, bias=False)      # no process group: the whole layer
    assert (lin.k0, lin.k1) == (0, 256)
