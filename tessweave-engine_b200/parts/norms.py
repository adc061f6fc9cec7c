"""Normalisation parts."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, Runtime, StepContext, WeightDecl, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * weight, statistics in fp32.

    Reference: flow_engine/model.py:15-23.  The pending delta of the previous
    sub-layer is added to the residual stream in the same kernel.  ``add_normed`` is the other
    arrangement: the norm of a sub-layer's output, added to the stream.  ``weight_name`` may be
    empty: the tensor then carries the part's own name.  ``unit_offset``: the checkpoint stores the weight
    around zero and the norm multiplies by ``1 + w`` (the one is added once, in fp32, when the weights are in).
    """
    accepts_split_sum = True

    def __init__(self, runtime: Runtime, size: int, eps: float, weight_name: str = "weight", unit_offset: bool = False):
        super().__init__(runtime)
        if size <= 0 or not eps > 0:
            raise ValueError("rmsnorm needs a positive size and eps")
        self.size, self.eps, self.weight_name = int(size), float(eps), weight_name
        self.unit_offset = bool(unit_offset)
        self._stored = runtime.empty(self.size, dtype=torch.float32) if self.unit_offset else None   # the checkpoint's w
        self.weight = runtime.empty(self.size, dtype=torch.float32)

    def weights(self) -> list[WeightDecl]:
        if self.unit_offset:
            return [WeightDecl(self.weight_name, (self.size,), role="vector", init="normal", dest=self._stored)]
        return [WeightDecl(self.weight_name, (self.size,), role="vector", init="one_plus_normal", dest=self.weight)]

    def finalize(self) -> None:
        if self.unit_offset:
            torch.add(self._stored, 1.0, out=self.weight)

    def forward(self, ctx: StepContext, out, resid, delta, n_rows, rows=None, delta_scale: float = 1.0) -> None:
        ops.add_rmsnorm(out, resid, delta, self.weight, self.eps, n_rows, rows, delta_scale=delta_scale)

    def add_normed(self, ctx: StepContext, resid, delta, n_rows, copy=None) -> None:
        ops.rmsnorm_to_residual(resid, delta, self.weight, self.eps, n_rows, copy)
