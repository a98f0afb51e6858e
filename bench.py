#!/usr/bin/env python
"""Benchmark of the HBQ hot path on B200: one quantised linear layer, with the whole-model prefills beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-model] [--no-cpu-baseline]
    python bench.py --sweep [CASE]      # configs[2] quantize sweep and KV-cache writes, one line per case
    python bench.py --llama | --mixtral # configs[3] / configs[4] prefill alone over the launched ranks
    python bench.py --tp-mlp | --ep-moe # the tensor-parallel MLP / expert-parallel MoE block alone

Workload of the line's `value` (the reference's HBQ-E quant-GEMM configuration with partial-sum-quantised
accumulation, config/hbq_e_psum_quant.yaml): X bf16 [4096, 4096] ~ N(0,1) with 0.5 % outlier channels x30,
W bf16 [14336, 4096] ~ N(0, 0.02) (the Llama-3-8B MLP up-projection shape), synthetic and seeded.  The weight is
fake-quantised once (static weight quantisation, not timed).  One step = HBQ-E activation quantize of X followed by
the GEMM whose fp32 partial sums are INT8-quantised per (128 k, 32 n) block and accumulated in fp16.  The metric
counts 2*M*N*K flops per step and nothing else.  After 0.8 s of the same load, blocks of exactly K steps run back to
back for at least 1.5 s; the reported step time is the median block (device time, max over ranks) / K.

With N > 1 (torchrun, one rank per GPU) every rank runs its own batch X against the same W: the layer shards over
rows without any exchange, so `value` scales weakly with no collective on its data path.  The collectives of the
path are in the sub-records of the same line: `llama_prefill` (configs[3], tensor/sequence-parallel: reduce-scatter +
all-gather), `mixtral_prefill` (configs[4], expert-parallel all-to-all), `tp_mlp`, `ep_moe`, each with the one-GPU
time measured in the same call.

`--impl reference` times the CPU restatement of the reference's path (oracle/, all host threads) on a bounded sample
of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, K, N = 4096, 4096, 14336
GROUP_K, GROUP_N = 128, 32
WARM_SECONDS = 0.8         # continuous load before the timed interval
TIMED_SECONDS = 1.5        # least duration of the timed interval (blocks of --steps steps, back to back)
WORKLOAD = ("configs[1]: HBQ-E linear, X[4096,4096] (0.5% outlier channels x30) * W[14336,4096]^T, "
            "act E2M2 / wgt E2M1, block 128, micro-block 32, accumulation fp16_quant(group 128, block 32)")
ACT = dict(block_size=128, ebit=2, mbit=2, sc_ebit=5, sc_mbit=3, l2_block_size=32, l2_sc_bit=2, l2_scheme="SIG-1")
WGT = dict(block_size=128, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3, l2_block_size=32, l2_sc_bit=2, l2_scheme="Mix")
# algorithmic HBM bytes per element of the activation quantize: 2 in + 2 fake-quantised out
QUANT_BYTES_PER_ELEM = 4.0


def make_inputs(rank: int):
    import torch
    g = torch.Generator().manual_seed(1000 + rank)
    x = torch.randn(M, K, generator=g)
    cols = torch.randperm(K, generator=torch.Generator().manual_seed(7))[: max(1, int(K * 0.005))]
    x[:, cols] *= 30
    w = 0.02 * torch.randn(N, K, generator=torch.Generator().manual_seed(1))
    return x.to(torch.bfloat16), w.to(torch.bfloat16)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d.get("hbm_gbs"), "tf_burst": d.get("bf16_tflops"),
                "tf_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tf_burst": 1590.0, "tf_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms (read only)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    @staticmethod
    def _stats(rows):
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for _, r in rows:
            try:
                sm.append(float(r[0])); smax.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            try:
                power.append(float(r[2]))
            except (ValueError, IndexError):
                pass
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "power_w_max": max(power) if power else None, "reasons": sorted(reasons)}

    def window(self, t0: float, t1: float):
        """Statistics of the samples taken inside [t0, t1] (host wall clock)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        return self._stats([r for r in list(self.rows) if t0 <= r[0] <= t1])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        return self._stats(list(self.rows))


def cpu_baseline_sample(x_bf16, wq_f16, seconds_target: float = 15.0):
    """The CPU oracle (a port of the reference's eager fp16 quantizer and of gemm.cu's INT8
    partial-sum model) on a bounded row sample of the workload, all host threads."""
    import numpy as np
    import oracle as O
    O.use_all_cores()
    fa = O.Format(O.KIND_HBQ, ACT["ebit"], ACT["mbit"], 5, 3, 128, l2_block_size=32, l2_sc_bit=2, l2_scheme="SIG-1")
    xh = x_bf16.to(dtype=__import__("torch").float16).numpy()
    wt = np.ascontiguousarray(wq_f16.numpy().T)
    rows, dt = 64, 0.0
    while True:                      # grow the sample until it costs about seconds_target of CPU time
        t0 = time.perf_counter()
        xq = O.quantize(xh[:rows], fa, want_codes=False)["deq"]
        O.gemm(xq, wt, O.ACC_PSUM_INT8, GROUP_K, GROUP_N)
        dt = time.perf_counter() - t0
        if dt >= 0.6 * seconds_target or rows >= M:
            break
        rows = int(min(M, max(rows * 2, rows * seconds_target / max(dt, 1e-3)) // 8 * 8))
    return {"value": 2.0 * rows * N * K / dt / 1e12, "unit": "TFLOP/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"{rows} of {M} rows of X through oracle HBQ-E quantize + INT8-psum GEMM vs full W, {dt:.1f} s"}


def run_reference(args, rank: int, world: int):
    """Reference arm: the CPU implementation of the path (oracle port; the reference's Python
    quantizer cannot travel to the GPU box and its GEMM has no CPU implementation)."""
    if rank != 0:
        return
    import numpy as np
    import torch
    import oracle as O
    O.build()
    O.use_all_cores()
    x, w = make_inputs(0)
    fw = O.Format(O.KIND_HBQ, 2, 1, 5, 3, 128, l2_block_size=32, l2_sc_bit=2, l2_scheme="Mix")
    fa = O.Format(O.KIND_HBQ, 2, 2, 5, 3, 128, l2_block_size=32, l2_sc_bit=2, l2_scheme="SIG-1")
    wq = O.quantize(w.to(torch.float16).numpy(), fw, want_codes=False)["deq"]
    wt = np.ascontiguousarray(wq.T)
    xh = x.to(torch.float16).numpy()
    rows = 256           # per step: bounded sample (~2 s of CPU work) so that K+W steps end within minutes

    def step(i):
        r0 = (i * rows) % M
        xq = O.quantize(xh[r0:r0 + rows], fa, want_codes=False)["deq"]
        return O.gemm(xq, wt, O.ACC_PSUM_INT8, GROUP_K, GROUP_N)

    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(args.warmup + i)
    dt = (time.perf_counter() - t0) / args.steps
    val = 2.0 * rows * N * K / dt / 1e12
    sample = f"{rows} rows of X per step (of {M}), full W; oracle HBQ-E quantize + INT8-psum GEMM"
    print(json.dumps({
        "impl": "reference", "metric": "quant_gemm_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist
    import hbq_b200 as H

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # threads and pinned buffers of this rank on the GPU's own NUMA node (HBQ_BENCH_NO_BIND=1: leave as found)
    from hbq_b200.shard import bind_host_to_device
    binding = None if os.environ.get("HBQ_BENCH_NO_BIND") == "1" else bind_host_to_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    x_host, w_host = make_inputs(rank)
    aq = H.HBQQuantizer(**ACT)
    aq.out_dtype = torch.float16          # bf16 in, fp16 fake-quantised out: the GEMM's operand type
    wq = H.HBQQuantizer(**WGT)
    wq.out_dtype = torch.float16
    lin = H.QLinear(K, N, bias=False, device=dev, dtype=torch.float16, check_finite=False)
    lin.weight.data = wq.q(w_host.to(dev))                              # static weight quantisation (not timed)
    lin.aq = aq
    lin.ops = H.FP16AccumMatMul(group_size=GROUP_K, quant_block_size=GROUP_N)
    x = x_host.to(dev)
    wq_host = lin.weight.data.cpu() if (rank == 0 and world == 1 and not args.no_cpu_baseline) else None
    torch.cuda.synchronize()

    def step():
        return lin(x)

    # clocks are sampled from the warm-up on: the timed interval below lasts >= TIMED_SECONDS
    sampler = ClockSampler(local_rank)
    sampler.start()
    t_warm = time.perf_counter()
    for _ in range(max(args.warmup, 3)):
        y = step()
    torch.cuda.synchronize()
    while time.perf_counter() - t_warm < WARM_SECONDS:       # bring clocks and power to their sustained state
        for _ in range(args.steps):
            y = step()
        torch.cuda.synchronize()
    barrier()
    if H.gemm_status() != 0:
        raise RuntimeError("tensor-core GEMM reported an expired wait")

    # ---- timed region: blocks of exactly K steps, back to back for >= TIMED_SECONDS; the reported step time is
    #      the MEDIAN block (device time between events, max over ranks per block) ----
    one = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    one[0].record()
    for _ in range(args.steps):
        y = step()
    one[1].record()
    torch.cuda.synchronize()
    est_ms = max(one[0].elapsed_time(one[1]), 1e-3)
    nblocks = int(min(2000, max(5, TIMED_SECONDS * 1e3 / est_ms)))
    if world > 1:
        nb = torch.tensor([nblocks], device=dev)
        dist.all_reduce(nb, op=dist.ReduceOp.MAX)
        nblocks = int(nb.item())
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(nblocks + 1)]
    l0 = H.launch_count()
    barrier()
    t_timed0 = time.time()
    evs[0].record()
    for b in range(nblocks):
        for _ in range(args.steps):
            y = step()
        evs[b + 1].record()
    barrier()
    t_timed1 = time.time()
    launches = (H.launch_count() - l0) // nblocks
    block_ms = torch.tensor([evs[b].elapsed_time(evs[b + 1]) for b in range(nblocks)], device=dev)
    if world > 1:
        dist.all_reduce(block_ms, op=dist.ReduceOp.MAX)
    total_ms = float(block_ms.median().item())
    ms_step = total_ms / args.steps
    flops_step = 2.0 * M * N * K
    value = flops_step * world / (ms_step * 1e-3) / 1e12
    clocks_timed = sampler.window(t_timed0, t_timed1)

    # ---- per-kernel device times (events on the launching stream, same sustained state) ----
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(max(args.steps, 50))]
    barrier()
    for a, b, c in kev:
        a.record()
        xq_i = aq.q(x)
        b.record()
        lin.ops(xq_i, lin.weight)
        c.record()
    torch.cuda.synchronize()
    q_ms = statistics.median(a.elapsed_time(b) for a, b, c in kev)
    g_ms = statistics.median(b.elapsed_time(c) for a, b, c in kev)
    peaks = measured_peaks()
    g_tf = flops_step / (g_ms * 1e-3) / 1e12
    q_gbs = M * K * QUANT_BYTES_PER_ELEM / (q_ms * 1e-3) / 1e9

    # ---- end to end through the plugin API: pinned host X -> device -> layer -> host Y ----
    x_pin = x_host.pin_memory()
    y_pin = torch.empty((M, N), dtype=torch.float16).pin_memory()
    x_dev = torch.empty_like(x)

    last = [None]

    def e2e_step():
        # the host-buffer entry of the layer: pinned X in, pinned Y out, copies and kernels pipelined
        _, last[0] = lin.forward_host(x_pin, y_pin, row_chunks=2, wait=False)

    for _ in range(max(8, args.warmup)):      # freshly pinned pages: the first copies into them are slow
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    torch.cuda.current_stream().wait_event(last[0])      # the last step's result has reached the host
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_val = flops_step * world / (e2e_ms / args.steps * 1e-3) / 1e12
    clocks = sampler.stop()
    if H.gemm_status() != 0:
        raise RuntimeError("tensor-core GEMM reported an expired wait")

    # ---- the metric's second leg: HBQ-A activation quantize of configs[2]'s tensor (rank 0) ----
    act_quant = act_quant_record(dev, peaks) if rank == 0 else None
    # ---- the reference's own CUDA-core kernel on the same GPU and shape (rank 0, outside every timed region) ----
    ref_gpu = reference_gemm_record(lin.aq.q(x), lin.weight.data) if (rank == 0 and world == 1) else None
    # ---- decode-sized GEMMs: the packed-weight kernel beside the fp16-operand ones (rank 0) ----
    decode = decode_gemm_record(dev) if (rank == 0 and world == 1) else None
    torch.cuda.empty_cache()

    # ---- whole-model and collective sub-records ----
    sub = {}
    if not args.no_model:
        one = llama_prefill_record(rank, world, dev, 2, 1, 1, layers=args.llama_layers, parallel=False)
        sub["llama_prefill"] = {"one_gpu": one}
        if world > 1:
            tp = llama_prefill_record(rank, world, dev, 3, 2, args.llama_pieces, layers=args.llama_layers)
            sub["llama_prefill"]["tensor_parallel"] = tp
            sub["llama_prefill"]["speedup_over_one_gpu"] = one["ms_per_forward"] / tp["ms_per_forward"]
            m1 = llama_prefill_record(rank, world, dev, 2, 1, 1, layers=args.llama_layers, batch=4, seq=4096, parallel=False,
                                      mixtral=True)
            mp_ = llama_prefill_record(rank, world, dev, 3, 2, 1, layers=args.llama_layers, batch=4, seq=4096, mixtral=True)
            sub["mixtral_prefill"] = {"one_gpu": m1, "expert_parallel": mp_,
                                      "speedup_over_one_gpu": m1["ms_per_forward"] / mp_["ms_per_forward"]}
            sa = argparse.Namespace(**vars(args))
            sa.steps, sa.warmup = 5, 3
            sub["tp_mlp"] = run_tp_mlp(sa, rank, world, local_rank, standalone=False)
            sub["ep_moe"] = run_ep_moe(sa, rank, world, local_rank, standalone=False)

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline_sample(x_host, wq_host)
        traffic, traffic_src = profile_traffic("gemm_tc_kernel_int8psum_M4096_K4096_N14336.md")
        line = {
            "metric": "quant_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_rows": M * world, "parallelism": f"row-sharded x{world}, no collective",
                       "l2": "no flush: per-step working set 266 MB (X 32 + Xq 32 + W 117 + Y 117) exceeds the 126 MB L2",
                       "timed_interval": f"{nblocks} blocks of {args.steps} steps back to back after {WARM_SECONDS} s of the same "
                                         f"load; ms_per_step = median block / {args.steps}",
                       "host_binding": binding},
            "clocks": clocks_timed, "clocks_whole_run": clocks,
            "mhz_ms_per_step": (clocks_timed["sm_mhz"] or 0) * ms_step,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2},
            "gpu_launches": int(launches) * nblocks, "gpu_launches_per_block": int(launches), "blocks": nblocks,
            # the kernel is timed inside a seconds-long load: its denominator is the SUSTAINED measured peak
            "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel<PSUM_INT8,32>", "achieved": g_tf,
                         "peak": peaks["tf_sustained"], "unit": "TFLOP/s", "frac": g_tf / peaks["tf_sustained"],
                         "peak_kind": "sustained (kernel timed inside a >= 2 s load)",
                         "peak_burst": peaks["tf_burst"], "frac_of_burst": g_tf / peaks["tf_burst"],
                         "peak_source": peaks["source"], "ms_per_launch": g_ms, "traffic": traffic, "traffic_source": traffic_src},
            "quantize": {"kernel": "hbq_tab_kernel (HBQ-E act, bf16 in, fp16 fake-quant out)", "bound": "hbm",
                         "achieved": q_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": q_gbs / peaks["hbm_gbs"],
                         "ms_per_launch": q_ms, "bytes_per_elem": QUANT_BYTES_PER_ELEM},
            "act_quant": act_quant,
        }
        if ref_gpu is not None:
            line["ref_gpu"] = ref_gpu
        if decode is not None:
            line["decode_gemm"] = decode
        line.update(sub)
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def profile_traffic(name: str):
    """DRAM bytes per launch from the committed ncu summary `profiles/<name>` (its line
    `traffic_bytes_per_launch = N`), so the number always belongs to the capture that is on file."""
    import re
    path = os.path.join(ROOT, "profiles", name)
    try:
        with open(path) as fh:
            m = re.search(r"traffic_bytes_per_launch\s*=\s*(\d+)", fh.read())
        if m:
            return int(m.group(1)), f"ncu dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch, profiles/{name}"
    except OSError:
        pass
    return None, "no capture on file"


def act_quant_record(dev, peaks, steps: int = 30):
    """HBQ-A activation quantize of configs[2]'s tensor, [8192, 8192] bf16 ~ 0.5 * Student-t(3) (268 MB in + out: larger
    than L2).  `as_stated`: bf16 in, packed codes + scales AND the bf16 dequantised tensor out (the configuration's
    own wording); `fake_quant_only`: fp16 in, fp16 fake-quantised tensor out (what a linear layer's step runs).
    Algorithmic bytes per element: 2 in + 2 dequantised out (+ 0.6641 codes and scales)."""
    import torch
    import hbq_b200 as H
    torch.manual_seed(2)
    t = (0.5 * torch.distributions.StudentT(3.0).sample((8192, 8192))).to(dev)
    q = H.HBQQuantizer(block_size=128, ebit=2, mbit=2, sc_ebit=5, sc_mbit=3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")
    rec = {"workload": "configs[2] hbq_a: activation quantizer of config/hbq_a.yaml on [8192, 8192]", "peak": peaks["hbm_gbs"],
           "unit": "GB/s", "peak_source": peaks["source"]}
    for name, x, fn, bpe in (("as_stated", t.to(torch.bfloat16), lambda v: q.quantize_packed(v, with_deq=True), 4.6641),
                             ("fake_quant_only", t.to(torch.float16), lambda v: q.q(v), 4.0)):
        for _ in range(5):
            fn(x)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record()
        for i in range(steps):
            fn(x)
            ev[i + 1].record()
        torch.cuda.synchronize()
        ms = statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(steps))
        gbs = x.numel() * bpe / ms / 1e6
        rec[name] = {"ms": ms, "achieved": gbs, "frac": gbs / peaks["hbm_gbs"], "bytes_per_elem": bpe}
    # the headline fraction is the configuration as stated
    rec["achieved"], rec["frac"] = rec["as_stated"]["achieved"], rec["as_stated"]["frac"]
    return rec


def decode_gemm_record(dev, rows: int = 16, copies: int = 8, reps: int = 6):
    """Decode-sized linear layers of configs[3] (the seven linears of a Llama-3-8B decoder layer, `rows` tokens, HBQ-A
    weights; `llama3_8b_layer_linears` is their sum per layer): the GEMM on the packed 4-bit weight (hbq_gemm_w4, 0.5625 B per weight) beside the same product on the
    fp16 fake-quantised tensor by this library's tensor-core kernel and by F.linear (the reference's path,
    src/module.py:64).  Each variant walks `copies` separate weights back to back so that no call finds its weight in
    L2; the walk is replayed from a CUDA graph and timed with CUDA events: us per call on the device."""
    import torch
    import hbq_b200 as H
    from hbq_b200 import blockquant_ext as ext
    from hbq_b200.packed_gemm import W4Weight
    q = H.HBQQuantizer(**dict(WGT, l2_block_size=8))
    rec = {"rows": rows, "weight_format": "HBQ-A weight (E2M1, E5M3 per 128, Mix micro-scales per 8)", "unit": "us per call",
           "note": "w4 = packed-weight kernel, codes as nibbles (0.5625 B per weight); w4_in_8bit_containers = the same codes one per byte (1.0625 B); fp16_tc = gemm_tc_kernel on the fp16 tensor; fp16_library = F.linear", "shapes": {}}

    def walk(fns):
        # the walk over the copies is captured in a CUDA graph and replayed, so that the time per call is the device's
        # (kernel plus the gap to the next kernel of the graph), not the host's launch path
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                for f in fns:
                    f()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for f in fns:
                f()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = None
        for _ in range(3):
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1) * 1e3 / (reps * len(fns))
            best = t if best is None else min(best, t)
        del graph
        return best

    # the linear layers of one Llama-3-8B decoder layer: gate / up, down, q / o, k / v (times they occur)
    layer = {(14336, 4096): 2, (4096, 14336): 1, (4096, 4096): 2, (1024, 4096): 2}
    for (N, Kd) in layer:
        w = (0.02 * torch.randn(N, Kd, device=dev)).half()
        packed, deq = q.quantize_packed(w, with_deq=True)
        n_copies = max(copies, -(-300_000_000 // (N * Kd * 2)))       # the walk covers more than twice the L2
        w4s = [W4Weight.from_packed(packed) for _ in range(n_copies)]
        deqs = [deq.clone() for _ in range(n_copies)]
        x = torch.randn(rows, Kd, device=dev).half()
        outs = [torch.empty(rows, N, device=dev, dtype=torch.float16) for _ in range(n_copies)]
        t4 = walk([(lambda ww=ww, o=o: ww.matmul(x, out=o)) for ww, o in zip(w4s, outs)])
        tt = walk([(lambda d=d, o=o: ext.gemm_fp32_accum(x, d, b_is_nk=True, out=o)) for d, o in zip(deqs, outs)])
        tl = walk([(lambda d=d, o=o: torch.mm(x, d.t(), out=o)) for d, o in zip(deqs, outs)])
        one = {"w4": t4, "fp16_tc": tt, "fp16_library": tl, "w4_bytes": w4s[0].nbytes(), "fp16_bytes": N * Kd * 2,
               "w4_GBs": w4s[0].nbytes() / t4 / 1e3, "fp16_library_GBs": N * Kd * 2 / tl / 1e3}
        if Kd * N >= 4096 * 14336:
            w8s = [W4Weight.from_packed(packed, container_bits=8) for _ in range(n_copies)]
            one["w4_in_8bit_containers"] = walk([(lambda ww=ww, o=o: ww.matmul(x, out=o)) for ww, o in zip(w8s, outs)])
            one["w8_bytes"] = w8s[0].nbytes()
            del w8s
        rec["shapes"][f"N{N}_K{Kd}"] = one
        del w4s, deqs, outs
    rec["llama3_8b_layer_linears"] = {k: sum(layer[(N, Kd)] * rec["shapes"][f"N{N}_K{Kd}"][k] for (N, Kd) in layer)
                                      for k in ("w4", "fp16_tc", "fp16_library")}
    # fewer tokens: the packed weight has a kernel without the tensor core for one token and a warp-level-MMA kernel
    # (weights expanded into register fragments) for two to eight
    rec["fewer_tokens"] = {}
    for (N, Kd) in ((14336, 4096), (4096, 4096)):
        w = (0.02 * torch.randn(N, Kd, device=dev)).half()
        packed, deq = q.quantize_packed(w, with_deq=True)
        n_copies = max(copies, -(-300_000_000 // (N * Kd * 2)))
        w4s = [W4Weight.from_packed(packed) for _ in range(n_copies)]
        deqs = [deq.clone() for _ in range(n_copies)]
        for r in (1, 8):
            x = torch.randn(r, Kd, device=dev).half()
            outs = [torch.empty(r, N, device=dev, dtype=torch.float16) for _ in range(n_copies)]
            rec["fewer_tokens"][f"N{N}_K{Kd}_rows{r}"] = {
                "w4": walk([(lambda ww=ww, o=o: ww.matmul(x, out=o)) for ww, o in zip(w4s, outs)]),
                "fp16_library": walk([(lambda d=d, o=o: torch.mm(x, d.t(), out=o)) for d, o in zip(deqs, outs)])}
        del w4s, deqs, outs
    torch.cuda.empty_cache()
    return rec


def reference_gemm_record(xq, wq, launches: int = 3):
    """The reference's own `gemm_blockquant_mxint8` (blockquant_ext_src/gemm.cu compiled for sm_100a into oracle/_ref/,
    CUDA cores only) on the benchmark's operands, on this GPU: the kernel the tensor-core kernel replaces.  The
    reference's caller also transposes the weight on every call (src/ops.py:41); that copy is timed separately."""
    import importlib.util
    import torch
    so = os.path.join(ROOT, "oracle", "_ref", "blockquant_ext.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref/blockquant_ext.so has not been built (python oracle/build_ref.py REFERENCE_DIR)"}
    spec = importlib.util.spec_from_file_location("blockquant_ext", so)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    torch.cuda.synchronize()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    legacy = torch.cuda.default_stream()
    with torch.cuda.stream(legacy):                  # the reference launches on the legacy default stream
        wt = wq.t().contiguous()
        ref.gemm_blockquant_mxint8(xq, wt, GROUP_K, GROUP_N)          # warm-up
        torch.cuda.synchronize()
        e[0].record(legacy)
        for _ in range(launches):
            wt = wq.t().contiguous()
        e[1].record(legacy)
        for _ in range(launches):
            ref.gemm_blockquant_mxint8(xq, wt, GROUP_K, GROUP_N)
        e[2].record(legacy)
    torch.cuda.synchronize()
    g_ms, t_ms = e[1].elapsed_time(e[2]) / launches, e[0].elapsed_time(e[1]) / launches
    return {"kernel": "gemm_blockquant_mxint8_core_kernel<128,32> (reference gemm.cu, sm_100a build)", "ms_per_launch": g_ms,
            "achieved": 2.0 * M * N * K / (g_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "weight_transpose_ms_per_call": t_ms,
            "launches": launches}


# ---- quantize sweep (configs[2]: [8192, 8192] over the six shipped activation formats) and the fused
#      KV-cache writes; not part of the default run --------------------------------------------------
SWEEP_FORMATS = {
    "mxfp4": ("mxfp", dict(block_size=32, ebit=2, mbit=1, sc_ebit=5, sc_mbit=0)),
    "nvfp4": ("mxfp", dict(block_size=16, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3)),
    "mxint8": ("mxint", dict(nbit=8, sc_ebit=8, sc_mbit=0, block_size=32)),
    "mxfp_a8": ("mxfp", dict(block_size=32, ebit=2, mbit=5, sc_ebit=5, sc_mbit=0)),
    "hbq_a": ("hbq", dict(block_size=128, ebit=2, mbit=2, sc_ebit=5, sc_mbit=3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")),
    "hbq_e": ("hbq", ACT),
}


def run_sweep(args):
    """One JSON line per case: `--sweep` runs all, `--sweep NAME` one (a format name, `k_write` or `v_write`)."""
    import torch
    import hbq_b200 as H
    from hbq_b200 import kvcache
    torch.cuda.set_device(0)
    peaks = measured_peaks()
    torch.manual_seed(2)
    cls = {"mxfp": H.MXFPQuantizer, "mxint": H.MXINTQuantizer, "hbq": H.HBQQuantizer}

    def timed(fn, numel, label, extra):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        gbs = numel * QUANT_BYTES_PER_ELEM / ms / 1e6
        print(json.dumps({"case": label, "ms": ms, "GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                          "bytes_per_elem": QUANT_BYTES_PER_ELEM, **extra}))

    want = None if args.sweep == "all" else args.sweep
    x = None
    for name, (kind, kw) in SWEEP_FORMATS.items():
        if want not in (None, name):
            continue
        if x is None:      # configs[2]: 0.5 * Student-t(3), [8192, 8192], inputs larger than L2
            x = (0.5 * torch.distributions.StudentT(3.0).sample((8192, 8192))).to(torch.float16).cuda()
        q = cls[kind](**kw)
        timed(lambda: q.q(x), x.numel(), f"quantize {name}", {"shape": [8192, 8192], "dtype": "f16"})
    if want in (None, "hbq_a_packed"):       # configs[2] as stated: bf16 in, packed codes + scales + bf16 dequantised out
        xb = (0.5 * torch.distributions.StudentT(3.0).sample((8192, 8192))).to(torch.bfloat16).cuda()
        q = cls["hbq"](**SWEEP_FORMATS["hbq_a"][1])
        timed(lambda: q.quantize_packed(xb, with_deq=True), xb.numel() * 4.6641 / QUANT_BYTES_PER_ELEM,
              "quantize hbq_a (packed + dequantised)", {"shape": [8192, 8192], "dtype": "bf16", "bytes_per_elem_counted": 4.6641})
        del xb
    if want in (None, "gemm"):               # the benchmark step's GEMM alone (INT8 partial sums, group 128, block 32)
        xq = cls["hbq"](**ACT).q(torch.randn(M, K, device="cuda", dtype=torch.float16))
        wt = cls["hbq"](**WGT).q((0.02 * torch.randn(N, K, device="cuda")).half())
        ops = H.FP16AccumMatMul(group_size=GROUP_K, quant_block_size=GROUP_N)
        for _ in range(max(args.warmup, 3)):
            ops(xq, wt)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            ops(xq, wt)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        print(json.dumps({"case": "gemm int8-psum", "ms": ms, "TFLOP/s": 2.0 * M * N * K / ms / 1e9, "shape": [M, K, N],
                          "status": H.gemm_status()}))
        del xq, wt
    if want in (None, "gemm_w4"):            # the decode GEMM on the packed weight: 16 tokens, Llama-3-8B up projection
        from hbq_b200.packed_gemm import W4Weight
        packed = cls["hbq"](**dict(WGT, l2_block_size=8)).quantize_packed((0.02 * torch.randn(N, K, device="cuda")).half())
        w4 = W4Weight.from_packed(packed)
        # 16 tokens: the tcgen05 kernel; 8: the warp-level-MMA kernel; 1: the kernel without the tensor core
        for rows in (16, 8, 1):
            xr = torch.randn(rows, K, device="cuda", dtype=torch.float16)
            for _ in range(max(args.warmup, 3)):
                w4.matmul(xr)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                w4.matmul(xr)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            print(json.dumps({"case": "gemm on the packed weight (weight L2-resident after the first call)", "ms": ms, "shape": [rows, K, N],
                              "packed_bytes": w4.nbytes(), "status": H.gemm_status()}))
        del w4, packed
    if want in (None, "softmax", "rmsnorm"):  # the fused row kernels at configs[3]'s shapes (one batch row of the prefill)
        from hbq_b200 import fused
        q = cls["hbq"](**SWEEP_FORMATS["hbq_a"][1])
        if want in (None, "softmax"):
            Hh, T = 32, 2048
            sc = torch.randn(4, Hh, T, T, device="cuda", dtype=torch.float16)
            timed(lambda: fused.softmax_quantize(sc, 128 ** -0.5, q, causal=True, q_len=T, heads=Hh, inplace=False),
                  sc.numel(), "softmax + quantize (causal)",
                  {"shape": [4, Hh, T, T], "dtype": "f16", "format": "hbq_a"})
            del sc
        if want in (None, "rmsnorm"):
            xr = torch.randn(16384, 4096, device="cuda", dtype=torch.float16)
            wr = torch.ones(4096, device="cuda", dtype=torch.float16)
            timed(lambda: fused.rmsnorm_quantize(xr, wr, 1e-5, q, inplace=False), xr.numel(), "rmsnorm + quantize",
                  {"shape": [16384, 4096], "dtype": "f16", "format": "hbq_a"})
            del xr
    if want in (None, "k_write", "v_write"):
        B, T, Hh, D = 8, 4096, 32, 128
        k = torch.randn(B, T, Hh * D, device="cuda", dtype=torch.float16)
        inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))
        ang = torch.arange(T).float()[:, None] * inv[None]
        emb = torch.cat((ang, ang), -1)[None]
        cos, sin = emb.cos().half().cuda(), emb.sin().half().cuda()
        q = cls["hbq"](**SWEEP_FORMATS["hbq_a"][1])
        shape = {"shape": [B, T, Hh, D], "dtype": "f16", "format": "hbq_a"}
        if want in (None, "k_write"):
            timed(lambda: kvcache.write_k_cache(k, Hh, q, cos, sin), k.numel(), "k_write (RoPE + quantize + layout)", shape)
        if want in (None, "v_write"):
            timed(lambda: kvcache.write_v_cache(k, Hh, q), k.numel(), "v_write (token-axis quantize + layout)", shape)


# config/hbq_a_kv.yaml of the reference as PTQ reads it: HBQ-A W4A5 on every linear, 4-bit K/V, post-RoPE Q and
# attention-probability quantisation, fp32 accumulation
HBQ_A_KV = {
    "quantization": {"xqtype": "hbq", "wqtype": "hbq", "quant_attn_wgt": True, "quant_post_rope_q": True, "quant_4b_kv": True,
                     "quant_k_cache": True, "quant_v_cache": True, "quant_attn_wgt_use_quant_kernel": False},
    "block_quant": {"act_ebit": 2, "act_mbit": 2, "act_block_size": 128, "act_sc_ebit": 5, "act_sc_mbit": 3,
                    "act_l2_sc_bit": 2, "act_l2_block_size": 8, "act_l2_scheme": "SIG-1",
                    "wgt_ebit": 2, "wgt_mbit": 1, "wgt_block_size": 128, "wgt_sc_ebit": 5, "wgt_sc_mbit": 3,
                    "wgt_l2_sc_bit": 2, "wgt_l2_block_size": 8, "wgt_l2_scheme": "Mix",
                    "scale_allow_subnormal": False, "qk_mx_round": False},
    "accumulation": {"type": "fp32"},
}


# config/hbq_e.yaml of the reference as PTQ reads it: HBQ-E W4A5 (micro-block 32) on every linear, fp32 accumulation
HBQ_E = {
    "quantization": {"xqtype": "hbq", "wqtype": "hbq"},
    "block_quant": {"act_ebit": 2, "act_mbit": 2, "act_block_size": 128, "act_sc_ebit": 5, "act_sc_mbit": 3,
                    "act_l2_sc_bit": 2, "act_l2_block_size": 32, "act_l2_scheme": "SIG-1",
                    "wgt_ebit": 2, "wgt_mbit": 1, "wgt_block_size": 128, "wgt_sc_ebit": 5, "wgt_sc_mbit": 3,
                    "wgt_l2_sc_bit": 2, "wgt_l2_block_size": 32, "wgt_l2_scheme": "Mix",
                    "scale_allow_subnormal": False, "qk_mx_round": False},
    "accumulation": {"type": "fp32"},
}


def llama_prefill_record(rank: int, world: int, dev, steps: int, warmup: int, pieces: int, layers: int = 32,
                         batch: int = 8, seq: int = 2048, parallel: bool = True, mixtral: bool = False):
    """configs[3]: Llama-3-8B-architecture random-init model, HBQ-A W4A5 + KV quantisation (hbq_a_kv.yaml), prefill of
    `batch` x `seq` tokens, tensor/sequence-parallel over `world` ranks (strong scaling: the batch is fixed).  Returns
    the record for the benchmark line (device time per forward, max over ranks)."""
    import torch
    import torch.distributed as dist
    import hbq_b200 as H
    arch = H.mixtral_8x7b() if mixtral else H.LlamaArch()
    arch.layers = layers
    model = H.QLlamaModel(arch, device=dev, pieces=pieces, parallel=parallel)
    tp = world if parallel else 1
    model.init_weights(seed=0)
    model.apply_ptq(H.PTQConfig(HBQ_E if mixtral else HBQ_A_KV))
    ids = torch.randint(0, arch.vocab, (batch, seq), generator=torch.Generator().manual_seed(3)).to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(1, warmup)):
        out = model(ids)
    barrier()
    l0 = H.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = model(ids)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms /= steps
    tokens = batch * seq
    flops = model.flops_per_token() * tokens + model.attention_flops(batch, seq)
    finite = bool(torch.isfinite(out[:256]).all().item())
    if H.gemm_status() != 0:
        raise RuntimeError("tensor-core GEMM reported an expired wait")
    what = (f"configs[4]: Mixtral-8x7B architecture, {layers} layers, 8 experts top-2, hbq_e.yaml" if mixtral
            else f"configs[3]: Llama-3-8B architecture, {layers} layers, hbq_a_kv.yaml")
    how = (f"tp{tp} attention heads over ranks (reduce-scatter + all-gather of token shards), ep{tp} experts over ranks "
           f"(all-to-all dispatch / combine of each rank's tokens), batch in {model.pieces} piece(s)" if mixtral else
           f"tp{tp} heads / MLP features over ranks, residual stream by tokens: reduce-scatter + all-gather per half-layer, "
           f"batch in {model.pieces} piece(s)")
    rec = {"workload": f"{what}, prefill {batch}x{seq}",
           "parallelism": how if tp > 1 else "1 GPU (whole model on every rank)",
           "ms_per_forward": ms, "tokens_per_s": tokens / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
           "flops_counted": "2*MAC of all linear layers + lm_head + uncausal attention matmuls",
           "kernel_launches_per_forward": (H.launch_count() - l0) // steps, "finite": finite,
           "logit_columns_per_rank": arch.vocab // tp}
    del model, out
    torch.cuda.empty_cache()
    return rec


def run_llama(args, rank: int, world: int, local_rank: int):
    """`--llama`: the whole-model prefill of configs[3] over the launched ranks, one JSON line from rank 0."""
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.tp_reserve_sms:
        from hbq_b200.gemm import gemm_reserve_sms
        gemm_reserve_sms(args.tp_reserve_sms)
    if args.mixtral:
        rec = llama_prefill_record(rank, world, dev, args.steps, args.warmup, args.llama_pieces, layers=args.llama_layers,
                                   batch=4, seq=4096, mixtral=True)
    else:
        rec = llama_prefill_record(rank, world, dev, args.steps, args.warmup, args.llama_pieces, layers=args.llama_layers)
    if rank == 0:
        print(json.dumps({"metric": "mixtral_prefill_tokens_per_s" if args.mixtral else "llama_prefill_tokens_per_s", "value": rec["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": rec["ms_per_forward"],
                          "higher_is_better": True, "scaling": "strong", "dtype": "f16", "data": "synthetic", "config": rec}))
    if world > 1:
        dist.destroy_process_group()


def run_tp_mlp(args, rank: int, world: int, local_rank: int, standalone: bool = True):
    """`--tp-mlp`: the MLP block of configs[3] (Llama-3-8B shapes: hidden 4096, intermediate 14336; 8 x 2048
    tokens) with HBQ-A activation quantizers and fp32 accumulation, tensor-parallel over the ranks: gate / up
    column-parallel, down row-parallel with its all-reduce.  Strong scaling: the token batch is fixed.  One
    JSON line from rank 0 (device time, max over ranks)."""
    import torch
    import torch.distributed as dist
    import hbq_b200 as H

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and standalone:
        dist.init_process_group("nccl", device_id=dev)
    hidden, inter, tokens = 4096, 14336, 8 * 2048
    act = dict(block_size=128, ebit=2, mbit=2, sc_ebit=5, sc_mbit=3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")
    wgt = dict(block_size=128, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3, l2_block_size=8, l2_sc_bit=2, l2_scheme="Mix")
    g = torch.Generator(device=dev).manual_seed(11)       # the same full tensors on every rank, sliced locally

    def mk(cls, i, o, **kw):
        lin = cls(i, o, bias=False, device=dev, dtype=torch.float16, **kw)
        w = (0.02 * torch.randn((o, i), device=dev, generator=g)).half()
        lin.load_full(H.HBQQuantizer(**wgt).q(w))
        lin.aq = H.HBQQuantizer(**act)
        return lin

    gate = mk(H.ColumnParallelQLinear, hidden, inter, multiple=128)
    up = mk(H.ColumnParallelQLinear, hidden, inter, multiple=128)
    down = mk(H.RowParallelQLinear, inter, hidden, row_chunks=args.tp_row_chunks, reserve_sms=args.tp_reserve_sms)
    x = torch.randn((tokens, hidden), device=dev, generator=g).half()

    def step():
        with torch.no_grad():
            xq = gate.aq(x)                                   # one quantize feeds both projections
            a = H.blockquant_ext.gemm_fp32_accum(xq, gate.weight, b_is_nk=True)
            b = H.blockquant_ext.gemm_fp32_accum(xq, up.weight, b_is_nk=True)
            return down(H.swiglu_quantize(a, b, down.aq), input_quantized=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        y = step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms /= args.steps
    flops = 3 * 2.0 * tokens * hidden * inter
    if H.gemm_status() != 0:
        raise RuntimeError("tensor-core GEMM reported an expired wait")
    line = None
    if rank == 0:
        line = ({"metric": "tp_mlp_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
                          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
                          "scaling": "strong", "dtype": "f16", "data": "synthetic",
                          "config": {"workload": "configs[3] MLP block: 16384 tokens, hidden 4096, intermediate 14336, HBQ-A "
                                                 "activations and weights, fp32 accumulation",
                                     "parallelism": f"tp{world}: gate/up column-parallel, down row-parallel, all-reduce of "
                                                    f"[16384,4096] fp16 in {down._pieces(tokens)} piece(s)"},
                          "finite": bool(torch.isfinite(y).all().item())})
    if not standalone:
        return line                  # a sub-record of the benchmark line (rank 0; None elsewhere)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_ep_moe(args, rank: int, world: int, local_rank: int, standalone: bool = True):
    """`--ep-moe`: the sparse MoE block of configs[4] (Mixtral-8x7B shapes: hidden 4096, intermediate 14336,
    8 experts, top-2; 4 x 4096 tokens) with HBQ-E quantizers and fp16 / partial-sum-quantised accumulation,
    experts spread over the ranks, each rank routing its share of the tokens.  Strong scaling: the token batch
    is fixed.  One JSON line from rank 0 (device time, max over ranks)."""
    import torch
    import torch.distributed as dist
    import hbq_b200 as H

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and standalone:
        dist.init_process_group("nccl", device_id=dev)
    hidden, inter, experts, top_k, tokens = 4096, 14336, 8, 2, 4 * 4096
    wq = H.HBQQuantizer(**WGT)
    moe = H.ExpertParallelMoE(hidden, inter, experts, top_k=top_k, packed_dispatch=args.ep_packed_dispatch, device=dev,
                              dtype=torch.float16, ops_factory=lambda: H.FP16AccumMatMul(group_size=128, quant_block_size=32))
    moe.aq = H.HBQQuantizer(**ACT)
    g = torch.Generator(device=dev).manual_seed(21)
    with torch.no_grad():
        moe.gate.weight.copy_(torch.randn((experts, hidden), device=dev, generator=g).half())
        for e in range(experts):                    # every rank draws all experts' weights, keeps its own
            ws = [(0.02 * torch.randn(shape, device=dev, generator=g)).half()
                  for shape in ((inter, hidden), (inter, hidden), (hidden, inter))]
            if moe.e0 <= e < moe.e0 + moe.per_rank:
                ex = moe.experts[e - moe.e0]
                for lin, w in zip((ex.w1, ex.w3, ex.w2), ws):
                    lin.weight.copy_(wq.q(w))
                ex.w2.aq = H.HBQQuantizer(**ACT)
    mine = tokens // world
    x = torch.randn((mine, hidden), device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank)).half()

    def step():
        with torch.no_grad():
            return moe(x)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        y = step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms /= args.steps
    flops = top_k * 3 * 2.0 * tokens * hidden * inter
    if H.gemm_status() != 0:
        raise RuntimeError("tensor-core GEMM reported an expired wait")
    line = None
    if rank == 0:
        line = ({"metric": "ep_moe_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
                          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
                          "scaling": "strong", "dtype": "f16", "data": "synthetic",
                          "config": {"workload": "configs[4] MoE block: 16384 tokens, 8 experts, top-2, hidden 4096, intermediate "
                                                 "14336, HBQ-E activations and weights, accumulation fp16_quant(group 128, block 32)",
                                     "parallelism": f"ep{world}: {moe.per_rank} expert(s) per rank, all-to-all dispatch "
                                                    f"({'packed codes and scales' if moe.packed_dispatch else 'fp16'}) and combine (fp16)"},
                          "finite": bool(torch.isfinite(y).all().item())})
    if not standalone:
        return line                  # a sub-record of the benchmark line (rank 0; None elsewhere)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-model", action="store_true",
                    help="leave out the whole-model and collective sub-records (configs[3] prefill; tensor-parallel MLP and "
                         "expert-parallel MoE blocks at N > 1)")
    ap.add_argument("--sweep", nargs="?", const="all", default=None,
                    help="instead of the benchmark line: quantize sweep of configs[2] and the KV-cache writes "
                         "(all cases, or one: " + ", ".join(SWEEP_FORMATS) + ", hbq_a_packed, gemm, gemm_w4, softmax, rmsnorm, k_write, v_write)")
    ap.add_argument("--tp-mlp", action="store_true",
                    help="instead of the benchmark line: the tensor-parallel MLP block of configs[3] over the launched ranks")
    ap.add_argument("--llama", action="store_true",
                    help="instead of the benchmark line: the Llama-3-8B-architecture prefill of configs[3] over the launched ranks")
    ap.add_argument("--mixtral", action="store_true",
                    help="instead of the benchmark line: the Mixtral-8x7B-architecture prefill of configs[4] over the launched ranks")
    ap.add_argument("--llama-layers", type=int, default=32)
    ap.add_argument("--llama-pieces", type=int, default=2,
                    help="--llama: pieces of whole sequences the batch is cut into (collectives of one run under the GEMMs of the next)")
    ap.add_argument("--ep-moe", action="store_true",
                    help="instead of the benchmark line: the expert-parallel MoE block of configs[4] over the launched ranks")
    ap.add_argument("--ep-packed-dispatch", action="store_true",
                    help="--ep-moe: dispatch packed codes and scales instead of fp16 rows")
    ap.add_argument("--no-fused-act", action="store_true",
                    help="--tp-mlp / --ep-moe: run silu, product and quantizer as separate ops (A/B of the fused kernel)")
    ap.add_argument("--tp-row-chunks", type=int, default=None,
                    help="--tp-mlp: pieces the row-parallel layer cuts its rows into (1 = all-reduce after the whole GEMM; "
                         "default: chosen from the per-rank GEMM size)")
    ap.add_argument("--tp-reserve-sms", type=int, default=0,
                    help="--tp-mlp / --llama / --mixtral: SMs the tensor-core GEMMs leave free for the collective running beside them")
    args = ap.parse_args()
    if args.sweep is not None:
        run_sweep(args)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.no_fused_act:
        from hbq_b200 import kvcache
        kvcache.FUSE_SWIGLU = False
    if args.llama or args.mixtral:
        run_llama(args, rank, world, local_rank)
        return
    if args.tp_mlp:
        run_tp_mlp(args, rank, world, local_rank)
        return
    if args.ep_moe:
        run_ep_moe(args, rank, world, local_rank)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
