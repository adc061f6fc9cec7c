"""Position encodings."""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import PositionEncoding, RotaryPlan, Runtime, StepContext, register_part


def stretched_frequencies(theta: float, dims: int, yarn: dict) -> list[float]:
    """The turning rate of every pair under the YaRN rule (see ``RotaryEmbedding``), in double precision."""

    def pair_turning(t: float) -> float:        # the (fractional) pair that makes t turns over the original length
        return dims * math.log(yarn["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_turning(yarn["fast"])), 0)
    hi = min(math.ceil(pair_turning(yarn["slow"])), dims - 1)
    out = []
    for i in range(dims // 2):
        f = theta ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / yarn["factor"] * ramp + f * (1.0 - ramp))
    return out


def checked_yarn(yarn: dict | None, theta: float) -> tuple[dict | None, float]:
    """(the four numbers as floats, the factor on cos and sin) of a ``yarn`` parameter; (None, 1) without one."""
    if yarn is None:
        return None, 1.0
    y = {k: float(yarn[k]) for k in ("factor", "original", "fast", "slow")}
    if min(y.values()) <= 0 or not theta > 1:
        raise ValueError("rope: yarn needs positive factor, original, fast and slow, and theta above 1")
    return y, 0.1 * math.log(y["factor"]) + 1.0


@register_part("position", "rope")
class RotaryEmbedding(PositionEncoding):
    """Rotate-half rotary encoding over the whole head, or over its first ``dims`` values.

    inv_freq[i] = theta ** (-(2 i) / dims), angle = float(position) * inv_freq[i], pairs
    (i, i + dims/2); all in fp32 (reference: flow_engine/model.py:26-33, where dims is the head size).
    The table of inverse frequencies is made on the host with the reference's own expression and
    uploaded once per head size, so the device only multiplies by the position.  Values of a head from
    ``dims`` on pass unchanged; only the whole-head form has kernels that rotate on the way
    (``fused_rotary_table``).

    ``yarn`` (``factor``, ``original``, ``fast``, ``slow``) stretches the slow frequencies for contexts beyond the
    ``original`` length: with d(t) = dims * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at
    inv_freq[i] / factor * r_i + inv_freq[i] * (1 - r_i), and cos and sin are both multiplied by
    0.1 * ln(factor) + 1 (``magnitude``).  The table is made on the host in double precision and rounded once.
    """

    def __init__(self, runtime: Runtime, theta: float, dims: int | None = None, yarn: dict | None = None):
        super().__init__(runtime)
        self.yarn, self.magnitude = checked_yarn(yarn, theta)
        if not theta > 0:
            raise ValueError("rope theta must be positive")
        if dims is not None and (dims < 0 or dims % 2):
            raise ValueError(f"rope needs an even number of rotated dims, got {dims}")
        self.theta, self.dims = float(theta), dims
        self._tables: dict[int, torch.Tensor] = {}

    def _table(self, dims: int) -> torch.Tensor:
        table = self._tables.get(dims)
        if table is None:
            if dims % 2:
                raise ValueError(f"rope needs an even number of rotated dims, got {dims}")
            if self.yarn is None:
                inv = self.theta ** (-torch.arange(0, dims, 2, dtype=torch.float32) / max(dims, 1))
            else:
                inv = torch.tensor(self._yarn_frequencies(dims), dtype=torch.float64).to(torch.float32)
            table = inv.to(self.runtime.device)
            self._tables[dims] = table
        return table

    def _yarn_frequencies(self, dims: int) -> list[float]:
        return stretched_frequencies(self.theta, dims, self.yarn)

    def _dims(self, head_dim: int) -> int:
        dims = head_dim if self.dims is None else self.dims
        if dims > head_dim:
            raise ValueError(f"rope over {dims} dims does not fit a head of {head_dim}")
        return dims

    def fused_rotary_table(self, head_dim: int) -> torch.Tensor | None:
        # the kernels that rotate on the way know no magnitude
        return self._table(head_dim) if self._dims(head_dim) == head_dim and self.magnitude == 1.0 else None

    def rotary_plan(self, head_dim: int) -> RotaryPlan:
        dims = self._dims(head_dim)
        return RotaryPlan(self._table(dims), dims, interleaved=False, magnitude=self.magnitude)

    def apply(self, ctx: StepContext, qk: torch.Tensor, n_heads: int, head_dim: int) -> None:
        """Rotate ``n_heads`` heads at the start of each packed row in place (nothing else is touched).
        A mixer with a kernel that rotates on the way (``fused_rotary_table``) gets the same numbers."""
        dims = self._dims(head_dim)
        if dims == head_dim and self.magnitude == 1.0:
            ops.rotate_heads(qk, None, ctx.positions, ctx.seq_of_token, self._table(dims), ctx.n_tokens, n_heads, head_dim)
        elif dims:
            ops.rotate_pairs(qk, ctx.positions, ctx.seq_of_token, self._table(dims), ctx.n_tokens, n_heads, head_dim, dims, False,
                             magnitude=self.magnitude)


@register_part("position", "rope_interleaved")
class InterleavedRotaryEmbedding(PositionEncoding):
    """Rotary encoding on neighbouring pairs, over the first ``dims`` values of a head (all of it when
    ``dims`` is None); the rest of the head passes unchanged.

        f_i = theta ** (-(2 i) / dims),  a = float(position) * f_i,  i < dims / 2
        (x[2i], x[2i+1]) -> (x[2i] cos a - x[2i+1] sin a,  x[2i+1] cos a + x[2i] sin a)

    all in fp32.  The table of f_i is made once per head size on the host.  ``yarn`` as for ``rope``: stretched
    rates per pair, and cos and sin both multiplied by 0.1 ln(factor) + 1.
    """

    def __init__(self, runtime: Runtime, theta: float, dims: int | None = None, yarn: dict | None = None):
        super().__init__(runtime)
        self.yarn, self.magnitude = checked_yarn(yarn, theta)
        if not theta > 0:
            raise ValueError("rope theta must be positive")
        if dims is not None and (dims < 0 or dims % 2):
            raise ValueError(f"rope needs an even number of rotated dims, got {dims}")
        self.theta, self.dims = float(theta), dims
        self._plans: dict[int, RotaryPlan] = {}

    def rotary_plan(self, head_dim: int) -> RotaryPlan:
        plan = self._plans.get(head_dim)
        if plan is None:
            dims = head_dim if self.dims is None else self.dims
            if dims > head_dim or dims % 2:
                raise ValueError(f"rope over {dims} dims does not fit a head of {head_dim}")
            if self.yarn is None:
                inv = self.theta ** (-torch.arange(0, dims, 2, dtype=torch.float32) / max(dims, 1))
            else:
                inv = torch.tensor(stretched_frequencies(self.theta, dims, self.yarn), dtype=torch.float64).to(torch.float32)
            plan = RotaryPlan(inv.to(self.runtime.device), dims, interleaved=True, magnitude=self.magnitude)
            self._plans[head_dim] = plan
        return plan

    def apply(self, ctx: StepContext, qk: torch.Tensor, n_heads: int, head_dim: int) -> None:
        plan = self.rotary_plan(head_dim)
        ops.rotate_pairs(qk, ctx.positions, ctx.seq_of_token, plan.inv_freq, ctx.n_tokens, n_heads, head_dim,
                         plan.rot_dims, plan.interleaved, magnitude=plan.magnitude)


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Leaves queries and keys as they are."""

    def apply(self, ctx: StepContext, qk, n_heads, head_dim) -> None:
        return None
