"""GPU, two ranks over NCCL (skipped with fewer than two GPUs): the tensor/sequence-parallel decoder and the
expert-parallel Mixtral layer against the whole model held by each rank on its own GPU.  Without quantizers the
two-rank logits differ only by summation order (relative Frobenius error <= 2e-3); with config/hbq_a_kv.yaml /
hbq_e.yaml the partial sums of o_proj / down_proj are rounded per rank, which moves values across quantisation
boundaries further down, so the bound is the model test's 5e-2."""
import json
import os
import socket

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(HERE))
    import hbq_b200 as H
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    with open(os.path.join(HERE, "golden", "ptq_configs.json")) as fh:
        cfgs = json.load(fh)
    msgs = []

    def rel(a, b):
        return float((a.double() - b.double()).norm() / b.double().norm())

    cases = [("llama", None, 2e-3), ("llama", "hbq_a_kv.yaml", 5e-2), ("mixtral", None, 2e-3), ("mixtral", "hbq_e.yaml", 5e-2)]
    for kind, yaml_name, tol in cases:
        arch = H.LlamaArch(hidden=256, layers=2, heads=4, kv_heads=2, head_dim=128, ffn=512, vocab=512,
                           num_experts=4 if kind == "mixtral" else 0)
        ids = torch.randint(0, arch.vocab, (4, 256), generator=torch.Generator().manual_seed(1)).to(dev)
        whole = H.QLlamaModel(arch, device=dev, parallel=False)
        whole.init_weights(9)
        both = []
        for pieces in (1, 2):
            tp = H.QLlamaModel(arch, device=dev, pieces=pieces)
            tp.init_weights(9)
            both.append(tp)
        if yaml_name is not None:
            for m in [whole] + both:
                m.apply_ptq(H.PTQConfig(cfgs[yaml_name]["config"]))
        want = whole(ids).float()
        for tp in both:
            got = tp(ids, gather_logits=True).float()
            torch.cuda.synchronize()
            r = rel(got, want)
            if not r <= tol:
                msgs.append(f"{kind} {yaml_name} pieces={tp.pieces}: rel {r:.3e} > {tol}")
            cols = tp(ids).float()
            v = arch.vocab // world
            if not torch.equal(cols, got[:, rank * v:(rank + 1) * v]):
                msgs.append(f"{kind} {yaml_name}: sharded logits are not the gathered ones' columns")
        if not torch.equal(both[0](ids, gather_logits=True), both[1](ids, gather_logits=True)):
            msgs.append(f"{kind} {yaml_name}: the batch in pieces changed the result")
    if H.gemm_status() != 0:
        msgs.append("a bounded wait expired inside the tensor-core kernel")
    allm = [None] * world
    dist.all_gather_object(allm, msgs)
    if rank == 0:
        with open(os.path.join(out_dir, "result"), "w") as fh:
            fh.write("ok" if not any(allm) else repr(allm))
    dist.barrier()
    dist.destroy_process_group()


def test_decoder_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "result").read_text() == "ok"
