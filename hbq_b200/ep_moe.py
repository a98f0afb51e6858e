"""Expert-parallel sparse MoE block with quantised expert layers (one process per GPU).

The reference patches ``MixtralSparseMoeBlock`` of transformers so that every expert's ``w1`` /
``w3`` / ``w2`` is a quantizer-carrying linear layer (src/patch.py, src/module.py:21-67) and runs all
experts on one device.  Here the experts are spread over the ranks of a process group; the
router is replicated.  Per call:

1. router: softmax over the expert logits in fp32, top-k, weights renormalised to sum to one;
2. the ranks learn each other's row counts from one small all-gather (the call's only host read);
   every (token, choice) copy is quantised with the experts' input quantizer *before* it travels --
   block quantisation is per row, so this gives the same values as quantising at the expert -- and
   sent to the rank that owns its expert (all-to-all with per-rank row counts).  With
   ``packed_dispatch`` the copies travel as packed codes and scales (0.52-0.66 B per element instead
   of 2) and are expanded on arrival;
3. each rank runs its experts on the rows it received: ``w2(aq2(silu(w1(x)) * w3(x)))``;
4. the results travel back (fp16), are weighted by the router and summed per token.

With one rank (or no process group) every expert is local and no collective runs.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .kvcache import swiglu_quantize
from .module import QLinear
from .quantizer import PackedTensor, _QBase, dequantize_packed


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


class QuantExpert(nn.Module):
    """One expert: ``w2(aq2(silu(w1(x)) * w3(x)))``; ``x`` arrives already quantised."""

    def __init__(self, hidden: int, inter: int, ops=None, device=None, dtype=None):
        super().__init__()
        kw = dict(bias=False, ops=ops, check_finite=False, device=device, dtype=dtype)
        self.w1 = QLinear(hidden, inter, **kw)
        self.w3 = QLinear(hidden, inter, **kw)
        self.w2 = QLinear(inter, hidden, **kw)

    def forward(self, xq: torch.Tensor) -> torch.Tensor:
        a, b = self.w1(xq), self.w3(xq)
        if a.is_cuda:
            # activation, product and w2's input quantizer in one pass where the format has the fused kernel
            return self.w2(swiglu_quantize(a, b, self.w2.aq), input_quantized=True)
        return self.w2(F.silu(a) * b)


class ExpertParallelMoE(nn.Module):
    """``num_experts`` experts over the ranks of ``group`` (contiguous slices), top-``top_k`` routing.

    ``aq``: the quantizer of the experts' input (applied once, before dispatch); the input
    quantizer of ``w2`` is each expert's ``w2.aq``.  ``packed_dispatch`` needs a CUDA block
    quantizer with a packed form (MXFP / MXINT / HBQ)."""

    def __init__(self, hidden: int, inter: int, num_experts: int, top_k: int = 2, group=None, ops_factory=None,
                 packed_dispatch: bool = False, device=None, dtype=None, local_only: bool = False):
        """``local_only``: every expert on this rank whatever process group exists."""
        super().__init__()
        world, rank = (1, 0) if local_only else (_world(group), _rank(group))
        if num_experts % world:
            raise ValueError(f"{num_experts} experts do not divide over {world} ranks")
        self.group, self.world, self.rank = group, world, rank
        self.hidden, self.inter, self.num_experts, self.top_k = hidden, inter, num_experts, top_k
        self.per_rank = num_experts // world
        self.e0 = rank * self.per_rank
        self.packed_dispatch = packed_dispatch
        self.gate = nn.Linear(hidden, num_experts, bias=False, device=device, dtype=dtype)     # replicated router
        self.aq = _QBase()
        self.experts = nn.ModuleList(
            QuantExpert(hidden, inter, ops=ops_factory() if ops_factory else None, device=device, dtype=dtype)
            for _ in range(self.per_rank))

    # ---- routing -------------------------------------------------------------------------------
    def route(self, x2d: torch.Tensor):
        """(weights [T, k] in x's dtype, expert ids [T, k])."""
        logits = self.gate(x2d)
        probs = F.softmax(logits, dim=-1, dtype=torch.float32)
        w, idx = torch.topk(probs, self.top_k, dim=-1)
        w = w / w.sum(dim=-1, keepdim=True)
        return w.to(x2d.dtype), idx

    # ---- exchange helpers ------------------------------------------------------------------------
    def _exchange_rows(self, rows: torch.Tensor, send_counts: List[int], recv_counts: List[int]) -> torch.Tensor:
        """All-to-all of a [n, width] tensor whose rows are grouped by destination rank."""
        out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=self.group)
        return out

    def _dispatch(self, x2d: torch.Tensor, src_rows: torch.Tensor, send_counts, recv_counts) -> torch.Tensor:
        """Quantise and bring every rank the rows of its experts (fake-quantised).  ``src_rows[c]`` is the
        token of copy c, copies sorted by expert."""
        if not self.packed_dispatch:
            # rows are quantised independently: quantise each token once, then copy it top_k times
            xq = self.aq(x2d).index_select(0, src_rows)
            return xq if self.world == 1 else self._exchange_rows(xq, send_counts, recv_counts)
        copies = x2d.index_select(0, src_rows)
        packed = self.aq.quantize_packed(copies)
        if self.world == 1:
            return dequantize_packed(packed)
        names = [n for n in PackedTensor._PLANES if getattr(packed, n) is not None]
        planes = [getattr(packed, n).reshape(copies.shape[0], -1) for n in names]
        widths = [p.shape[1] for p in planes]
        got = self._exchange_rows(torch.cat(planes, dim=1), send_counts, recv_counts)     # one buffer, one all-to-all
        n = got.shape[0]
        parts = dict(zip(names, torch.split(got, widths, dim=1)))
        shaped = {k: parts[k].contiguous().view((n,) + tuple(getattr(packed, k).shape[1:])) for k in names}
        arrived = PackedTensor(torch.Size((n, copies.shape[1])), packed.dtype, packed.fmt, shaped.get("codes"),
                               shaped.get("sign"), shaped.get("scale_u8"), shaped.get("l2_packed"), shaped.get("scheme"))
        return dequantize_packed(arrived)

    # ---- forward ---------------------------------------------------------------------------------
    # The block needs one host read (the per-rank row counts size the all-to-all).  It is split in two so that a caller
    # with several independent batches can put other launches between the exchange of the counts and the read:
    # ``begin`` routes, exchanges the counts and starts their copy to pinned host memory; ``finish`` waits for that
    # copy only, then dispatches, runs the local experts and combines.  ``forward`` is the two back to back.
    def begin(self, x: torch.Tensor) -> dict:
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.hidden)
        w, idx = self.route(x2d)
        flat_e = idx.reshape(-1)                                       # expert of copy c = (token c // k, choice c % k)
        order = torch.sort(flat_e, stable=True).indices               # copies grouped by expert, hence by rank
        src_rows = torch.div(order, self.top_k, rounding_mode="floor")
        per_expert = torch.bincount(flat_e, minlength=self.num_experts)
        if self.world == 1:
            counts = per_expert.unsqueeze(0)
        else:
            # every rank's copies per expert, in one small all-gather: row r is what rank r sends
            rows = [torch.empty_like(per_expert) for _ in range(self.world)]
            dist.all_gather(rows, per_expert.contiguous(), group=self.group)
            counts = torch.stack(rows)
        st = dict(lead=lead, x2d=x2d, w=w, order=order, src_rows=src_rows)
        if counts.is_cuda:
            host = torch.empty(counts.shape, dtype=counts.dtype, pin_memory=True)
            host.copy_(counts, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            st["counts"], st["event"] = host, ev
        else:
            st["counts"], st["event"] = counts, None
        return st

    def finish(self, st: dict) -> torch.Tensor:
        lead, x2d, w, order, src_rows = st["lead"], st["x2d"], st["w"], st["order"], st["src_rows"]
        T = x2d.shape[0]
        if st["event"] is not None:
            st["event"].synchronize()                                  # the call's one host read
        tl = st["counts"].tolist()
        if self.world == 1:
            recv_per_expert = tl[0]
            xq = self._dispatch(x2d, src_rows, None, None)
            send_counts = recv_counts = None
        else:
            # my row gives the split sizes of what I send and my experts' columns those of what I receive
            send_counts = [sum(tl[self.rank][d * self.per_rank:(d + 1) * self.per_rank]) for d in range(self.world)]
            got_l = [tl[s][self.e0:self.e0 + self.per_rank] for s in range(self.world)]
            recv_counts = [sum(g) for g in got_l]
            xq_by_src = self._dispatch(x2d, src_rows, send_counts, recv_counts)
            # arrived rows are grouped by source rank, then by expert: regroup by expert
            if self.per_rank == 1:
                xq = xq_by_src                                          # one expert here: already in order
            else:
                pieces = torch.split(xq_by_src, [c for src in got_l for c in src])
                by_expert = [[pieces[s * self.per_rank + e] for s in range(self.world)] for e in range(self.per_rank)]
                xq = torch.cat([p for e in by_expert for p in e]) if xq_by_src.shape[0] else xq_by_src
            recv_per_expert = [sum(got_l[s][e] for s in range(self.world)) for e in range(self.per_rank)]

        # local experts on their row segments
        outs = []
        r0 = 0
        for e, n in enumerate(recv_per_expert):
            if n:
                outs.append(self.experts[e](xq[r0:r0 + n]))
            r0 += n
        y_rows = torch.cat(outs) if outs else xq.new_empty((0, self.hidden))

        if self.world > 1:
            # back to (source rank, expert) order, then home
            if self.per_rank > 1:
                segs = torch.split(y_rows, [got_l[s][e] for e in range(self.per_rank) for s in range(self.world)])
                back = [segs[e * self.world + s] for s in range(self.world) for e in range(self.per_rank)]
                y_rows = torch.cat(back) if y_rows.shape[0] else y_rows
            y_rows = self._exchange_rows(y_rows, recv_counts, send_counts)

        # y_rows is in `order`: weight each copy and add it to its token
        wc = w.reshape(-1).index_select(0, order).unsqueeze(1)
        y = torch.zeros((T, self.hidden), dtype=x2d.dtype, device=x2d.device)
        y.index_add_(0, src_rows, y_rows * wc)
        return y.reshape(*lead, self.hidden)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.finish(self.begin(x))
