"""Quantizer-carrying linear layer with the reference's fields (``_QBaseLinear``,
src/module.py:21-67): ``wq`` / ``aq`` / ``yq`` quantizers and an optional ``ops`` GEMM operator.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .quantizer import _QBase


class QLinear(nn.Linear):
    """y = yq(ops(aq(x), W, b)); W is expected to be fake-quantised already (static weight
    quantisation, src/ptq.py:337-382).  ``ops=None`` uses ``F.linear`` like the reference
    (fp16 GEMM with fp32 accumulation).  ``check_finite`` keeps the reference's non-finite
    guard (src/module.py:52-65), which synchronises the host on every call."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, ops=None,
                 check_finite: bool = True, device=None, dtype=None):
        super().__init__(in_features, out_features, bias, device=device, dtype=dtype)
        self.wq = _QBase()
        self.aq = _QBase()
        self.yq = _QBase()
        self.ops = ops
        self.check_finite = check_finite

    def forward(self, x: torch.Tensor):
        wq = self.weight
        xq = self.aq(x)
        if self.ops is None:
            y = F.linear(xq, wq, self.bias)
        else:
            y = self.ops(xq, wq, self.bias)
        if self.check_finite and not torch.isfinite(y).all():
            ops_name = type(self.ops).__name__ if self.ops is not None else "F.linear"
            raise RuntimeError(
                f"Non-finite output from {type(self).__name__}"
                f"({self.in_features} -> {self.out_features}): "
                f"{int(y.isnan().sum())} NaN and {int(y.isinf().sum())} Inf "
                f"out of {y.numel()} elements.\n"
                f"  activation quantizer: {type(self.aq).__name__}\n"
                f"  weight quantizer:     {type(self.wq).__name__}\n"
                f"  matmul:               {ops_name}")
        return self.yq(y)
