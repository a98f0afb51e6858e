"""CPU, world_size 2 over gloo: the sharding rules of the multi-GPU path.  Each rank quantises /
multiplies only its slice with the CPU oracle; gathered, the slices must equal the unsharded
result bit for bit (no collective sits on the data path itself)."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

from util import seeded_inputs


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import oracle as O
    from hbq_b200.shard import column_range, row_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = seeded_inputs("act", 37, 512, 3)
    w = seeded_inputs("wgt", 96, 512, 4)
    fmt = O.Format(O.KIND_HBQ, 2, 2, 5, 3, 128, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")
    # quantize: row shards
    b, e = row_range(x.shape[0], rank, world)
    mine = O.quantize(x[b:e], fmt, False)["deq"].view(np.int16)
    parts = [None] * world
    dist.all_gather_object(parts, mine)      # test-side gather only: the path itself exchanges nothing
    full = np.concatenate(parts)
    # GEMM: column shards on multiples of group_n
    xq = O.quantize(x, fmt, False)["deq"]
    cb, ce = column_range(w.shape[0], rank, world, 32)
    y_mine = O.gemm(xq, np.ascontiguousarray(w[cb:ce].T), O.ACC_PSUM_INT8, 128, 32).view(np.int16)
    ys = [None] * world
    dist.all_gather_object(ys, y_mine)
    if rank == 0:
        ref = O.quantize(x, fmt, False)["deq"].view(np.int16)
        yref = O.gemm(xq, np.ascontiguousarray(w.T), O.ACC_PSUM_INT8, 128, 32).view(np.int16)
        ok = np.array_equal(full, ref) and np.array_equal(np.concatenate(ys, axis=1), yref)
        with open(os.path.join(out_dir, "ok"), "w") as fh:
            fh.write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_row_and_column_shards_world2(tmp_path, oracle):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").read_text() == "1"


def test_shard_ranges():
    from hbq_b200.shard import column_range, k_range, row_range
    for rows in (0, 1, 7, 4096):
        for world in (1, 2, 3, 8):
            spans = [row_range(rows, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1
    assert column_range(14336, 3, 8, 32) == (5376, 7168)
    assert all((b % 32, e % 32) == (0, 0) for b, e in (column_range(14336, r, 8, 32) for r in range(8)))
    assert k_range(4096, 1, 2, 128) == (2048, 4096)
    with pytest.raises(ValueError):
        column_range(100, 0, 2, 32)
    with pytest.raises(ValueError):
        row_range(4, 2, 2)
