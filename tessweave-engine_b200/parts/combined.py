"""Mixers made of other mixers."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import (Mixer, PartSpec, Runtime, SeveralNeeds, SeveralViews, StepContext, WeightDecl, build_part, dense_delta,
                   join_name, register_part)


@register_part("mixer", "weighted_sum")
class WeightedSumMixer(Mixer):
    """Several mixers side by side on the same input: delta = sum_m scale_m * mixer_m(h).

    ``members``: (checkpoint prefix, mixer spec, scale) per member, in order.  Each member keeps the cache or
    state it needs itself (``SeveralNeeds`` / ``SeveralViews``, in the members' order); the sum is formed in fp32
    and rounded once.

    With ``member_norm_eps`` every member's result is first divided by its root mean square over the width (eps
    inside the root) and multiplied by a learned weight of its own, ``<prefix>.<member_norm_name>``:
    delta = sum_m scale_m * rms(mixer_m(h)) * w_m, statistics and products in fp32.
    """

    def __init__(self, runtime: Runtime, hidden: int, members: tuple, member_norm_eps: float | None = None,
                 member_norm_name: str = "norm"):
        super().__init__(runtime)
        if member_norm_eps is not None and not member_norm_eps > 0:
            raise ValueError("weighted_sum: member_norm_eps must be positive")
        self.norm_eps, self.norm_name = member_norm_eps, member_norm_name
        self.norm_weights = (runtime.empty(len(members), hidden, dtype=torch.float32)
                             if member_norm_eps is not None else None)
        if not members:
            raise ValueError("weighted_sum: at least one member")
        self.hidden = hidden
        self.prefixes = [str(p) for p, _, _ in members]
        self.scales = [float(s) for _, _, s in members]
        self.members = [build_part("mixer", spec, runtime) for _, spec, _ in members]
        self.graph_safe = all(m.graph_safe for m in self.members)

    def weights(self) -> list[WeightDecl]:
        decls = [WeightDecl(join_name(prefix, w.name), w.shape, w.role, w.init, w.dest)
                 for prefix, member in zip(self.prefixes, self.members) for w in member.weights()]
        if self.norm_weights is not None:
            decls += [WeightDecl(join_name(prefix, self.norm_name), (self.hidden,), role="vector", init="one_plus_normal",
                                 dest=self.norm_weights[i]) for i, prefix in enumerate(self.prefixes)]
        return decls

    def redundant_names(self) -> list[str]:
        return [join_name(prefix, n) for prefix, member in zip(self.prefixes, self.members) for n in member.redundant_names()]

    def finalize(self) -> None:
        for member in self.members:
            member.finalize()

    def cache_need(self) -> SeveralNeeds:
        return SeveralNeeds(tuple(member.cache_need() for member in self.members))

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        if not isinstance(cache, SeveralViews) or len(cache.views) != len(self.members):
            raise TypeError("weighted_sum needs one cache view per member")
        n, dt, ws = ctx.n_tokens, self.runtime.dtype, ctx.workspace
        out = ws.get("weighted_sum.delta", (n, self.hidden), dt)
        if len(self.members) <= ops.WEIGHTED_SUM_MAX_MEMBERS:
            # every member works in workspace buffers of its own, so that all results exist side by side; one kernel
            # normalises (where asked), scales and adds them
            deltas, outer = [], ws.prefix
            for i, (member, view) in enumerate(zip(self.members, cache.views)):
                ws.prefix = f"{outer}member{i}."
                try:
                    deltas.append(dense_delta(ctx, member.forward(ctx, h, view, write_cache), dt)[:n])
                finally:
                    ws.prefix = outer
            ops.weighted_sum_rows(out, deltas, self.scales, self.norm_weights, self.norm_eps, n)
            return out
        acc = ws.get("weighted_sum.acc", (n, self.hidden), torch.float32)
        last = len(self.members) - 1
        for i, (member, scale, view) in enumerate(zip(self.members, self.scales, cache.views)):
            delta = dense_delta(ctx, member.forward(ctx, h, view, write_cache), dt)[:n]
            if self.norm_weights is not None:
                ops.normed_accumulate(acc, out if i == last else None, delta, self.norm_weights[i], self.norm_eps, scale,
                                      first=(i == 0), n_rows=n)
            else:
                ops.scaled_accumulate(acc, out if i == last else None, delta, scale, first=(i == 0))
        return out
