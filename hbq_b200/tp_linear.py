"""Tensor-parallel forms of the quantizer-carrying linear layer (one process per GPU).

The reference runs whole models on one device (or lets ``accelerate`` place layers); its linear
layer is ``_QBaseLinear`` (src/module.py:21-67).  These two classes are that layer cut the two
ways a transformer block needs:

* ``ColumnParallelQLinear``: this rank owns rows ``[n0, n1)`` of W (a slice of the output
  features, cut on multiples of the partial-sum block) and produces those output columns from the
  whole input.  No exchange; identical to the unsharded layer's columns bit for bit.
* ``RowParallelQLinear``: this rank owns columns ``[k0, k1)`` of W (whole quantisation blocks and
  accumulation groups) and receives the matching slice of the input, typically the output of a
  column-parallel layer.  Its partial products are summed over the ranks: the one real exchange
  step of the path.  The rows are cut into pieces; piece i is all-reduced on a side stream while
  the kernels of piece i+1 run, so that the transfer hides under the GEMM.

The cross-rank sum is not the reference's single sequential chain, so a K split changes the bits:
for the fp32 accumulation model the difference is one extra fp16 rounding per rank and partial
product.  At world size 1 the layer equals ``QLinear`` with the same operator bit for bit when an
``FP16AccumMatMul`` is set; with ``ops=None`` it runs the tensor-core fp32-accumulation kernel where
``QLinear`` calls ``F.linear`` (cuBLAS), two fp32-accumulating GEMMs whose outputs agree to the
fp16 output rounding, not bit for bit.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import blockquant_ext as ext
from .gemm import gemm_reserve_sms
from .module import QLinear
from .ops import FP16AccumMatMul
from .shard import column_range, k_range


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


class ColumnParallelQLinear(QLinear):
    """Output features ``[n0, n1)`` of a ``[N, K]`` linear layer.  ``gather_output=True`` returns the
    full ``[..., N]`` result (an all-gather along the last axis); the default leaves it sharded for
    a row-parallel layer to consume."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, ops=None, group=None,
                 gather_output: bool = False, multiple: int = 32, check_finite: bool = False,
                 device=None, dtype=None):
        self.group = group
        self.n0, self.n1 = column_range(out_features, _rank(group), _world(group), multiple)
        self.full_out_features = out_features
        self.gather_output = gather_output
        if gather_output and (out_features // multiple) % _world(group) != 0:
            raise ValueError(f"gather_output needs equal shards: {out_features // multiple} blocks of {multiple} output "
                             f"features do not divide over {_world(group)} ranks")
        super().__init__(in_features, self.n1 - self.n0, bias, ops=ops, check_finite=check_finite,
                         device=device, dtype=dtype)

    @torch.no_grad()
    def load_full(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        """Take this rank's slice of the unsharded parameters."""
        self.weight.data.copy_(weight[self.n0:self.n1])
        if bias is not None and self.bias is not None:
            self.bias.data.copy_(bias[self.n0:self.n1])

    def forward(self, x: torch.Tensor):
        y = super().forward(x)
        if not self.gather_output or _world(self.group) == 1:
            return y
        parts = [torch.empty_like(y) for _ in range(_world(self.group))]
        dist.all_gather(parts, y.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


_SIDE_STREAMS = {}      # device -> the stream the all-reduces of RowParallelQLinear run on


class RowParallelQLinear(QLinear):
    """Input features ``[k0, k1)`` of a ``[N, K]`` linear layer: ``y = sum over ranks of
    ops(aq(x[:, k0:k1]), W[:, k0:k1])`` + bias.  ``x`` is this rank's slice ``[..., k1 - k0]``.
    ``row_chunks`` pieces of rows are reduced while the next piece is computed; ``None`` chooses the
    count from the work: a piece must keep the GEMM busy for about the time its all-reduce takes
    (measured on 2 and 8 B200s: cutting pays with two ranks, where this rank's GEMM is long, and
    costs 12 % with eight, where the all-reduce outlasts the GEMM and every extra call adds latency)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, ops=None, group=None,
                 block: int = 128, row_chunks: Optional[int] = None, reserve_sms: int = 0, check_finite: bool = False,
                 device=None, dtype=None):
        self.group = group
        self.k0, self.k1 = k_range(in_features, _rank(group), _world(group), block)
        self.full_in_features = in_features
        self.row_chunks = None if row_chunks is None else max(1, int(row_chunks))
        self.reserve_sms = max(0, int(reserve_sms))     # SMs the GEMM leaves to the all-reduce running beside it
        super().__init__(self.k1 - self.k0, out_features, bias, ops=ops, check_finite=check_finite,
                         device=device, dtype=dtype)

    def _check_quantizer(self):
        # a per-tensor scale is the maximum over the WHOLE input; this layer sees one K slice of some rows
        # at a time, so the result would depend on the sharding and the row pieces
        if getattr(self.aq, "per_tensor_scale", False) and type(self.aq).__name__ == "MXFPQuantizer":
            raise ValueError("RowParallelQLinear does not take an activation quantizer with per_tensor_scale")

    @torch.no_grad()
    def load_full(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight.data.copy_(weight[:, self.k0:self.k1])
        if bias is not None and self.bias is not None:
            self.bias.data.copy_(bias)

    def _partial(self, x2d: torch.Tensor, out: Optional[torch.Tensor] = None, input_quantized: bool = False) -> torch.Tensor:
        """This rank's partial product, written into ``out`` when the operator can do that."""
        xq = x2d if input_quantized else self.aq(x2d)
        if self.ops is None:
            if xq.is_cuda and xq.dtype == torch.float16 and self.weight.dtype == torch.float16:
                # fp32 accumulation (what F.linear models in the reference) on the tensor-core kernel
                return ext.gemm_fp32_accum(xq.contiguous(), self.weight, b_is_nk=True, out=out)
            y = torch.nn.functional.linear(xq, self.weight)
        elif isinstance(self.ops, FP16AccumMatMul):
            return self.ops(xq, self.weight, None, out=out)
        else:
            y = self.ops(xq, self.weight, None)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def _pieces(self, rows: int) -> int:
        if self.row_chunks is not None:
            return self.row_chunks
        flops = 2.0 * rows * self.out_features * self.in_features          # this rank's GEMM
        return int(max(1, min(4, flops // 2.5e11)))                         # about 0.2 ms of GEMM per piece

    def forward(self, x: torch.Tensor, input_quantized: bool = False):
        world = _world(self.group)
        if not input_quantized:
            self._check_quantizer()
        lead = x.shape[:-1]
        x2d = x.reshape(-1, x.shape[-1])
        rows = x2d.shape[0]
        if world == 1:
            y = self._partial(x2d, input_quantized=input_quantized)
        elif not x2d.is_cuda:
            y = self._partial(x2d, input_quantized=input_quantized)
            dist.all_reduce(y, group=self.group)
        else:
            y = torch.empty((rows, self.out_features), dtype=self.weight.dtype, device=x2d.device)
            dev = x2d.device
            side = _SIDE_STREAMS.get(dev)
            if side is None:
                side = _SIDE_STREAMS[dev] = torch.cuda.Stream(dev)
            cur = torch.cuda.current_stream(dev)
            step = -(-rows // self._pieces(rows))
            step = max(128, -(-step // 128) * 128)          # whole GEMM row tiles per piece
            for r0 in range(0, rows, step):
                r1 = min(rows, r0 + step)
                piece = y[r0:r1]
                # from the second piece on an all-reduce is in flight beside the GEMM
                prev = gemm_reserve_sms(self.reserve_sms) if (self.reserve_sms and r0 > 0) else None
                try:
                    self._partial(x2d[r0:r1], out=piece, input_quantized=input_quantized)
                finally:
                    if prev is not None:
                        gemm_reserve_sms(prev)
                ev = torch.cuda.Event()
                ev.record(cur)
                side.wait_event(ev)
                with torch.cuda.stream(side):
                    dist.all_reduce(piece, group=self.group)
            done = torch.cuda.Event()
            done.record(side)
            cur.wait_event(done)
        if self.bias is not None:
            y = y + self.bias
        if self.check_finite and not torch.isfinite(y).all():
            raise RuntimeError(f"Non-finite output from {type(self).__name__}({self.full_in_features} -> {self.out_features})")
        return self.yq(y).reshape(*lead, self.out_features)
