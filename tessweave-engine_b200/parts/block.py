"""Arrangements of parts around the residual stream."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import (Block, PartSpec, ResidualStream, Runtime, StepContext, WeightDecl, build_part, dense_delta, join_name,
                   register_part, unscaled_pending)


class ArrangedBlock(Block):
    """What every arrangement shares: sub-parts under their checkpoint prefixes (``names``), their
    weight declarations, and the mixer's cache need.  A sub-part may be absent (``None``)."""

    ROLES = ("norm1", "mixer", "norm2", "feed_forward")

    def __init__(self, runtime: Runtime, hidden: int, names: dict[str, str] | None = None):
        super().__init__(runtime)
        self.hidden = hidden
        self.names = {role: role for role in self.ROLES}
        self.names.update(names or {})

    def parts(self):
        return {role: getattr(self, role) for role in self.ROLES if getattr(self, role) is not None}

    def weights(self) -> list[WeightDecl]:
        return [WeightDecl(join_name(self.names[role], w.name), w.shape, w.role, w.init, w.dest)
                for role, part in self.parts().items() for w in part.weights()]

    def redundant_names(self) -> list[str]:
        return [join_name(self.names[role], name) for role, part in self.parts().items() for name in part.redundant_names()]

    def finalize(self) -> None:
        for part in self.parts().values():
            part.finalize()

    def cache_need(self):
        return self.mixer.cache_need()


@register_part("block", "pre_norm")
class PreNormBlock(ArrangedBlock):
    """x = x + mixer(norm1(x));  x = x + feed_forward(norm2(x)).

    Reference: flow_engine/model.py:179-202.  The residual stream is fp32; each
    sub-layer's output is handed to the next norm as a pending delta, so the add
    and the norm are one kernel.  ``names`` gives the checkpoint's prefix of each
    sub-part inside the layer.  ``residual_scale`` m: x = x + m * sublayer(norm(x)) for both sub-layers; the product
    is formed in fp32 by the kernel that adds the delta.
    """

    def __init__(self, runtime: Runtime, hidden: int, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec | None = None,
                 feed_forward: PartSpec | None = None, names: dict[str, str] | None = None, residual_scale: float = 1.0):
        super().__init__(runtime, hidden, names)
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("pre_norm block: norm2 and feed_forward come together or not at all")
        self.residual_scale = float(residual_scale)
        self.norm1 = build_part("norm", norm1, runtime)
        self.mixer = build_part("mixer", mixer, runtime)
        self.norm2 = build_part("norm", norm2, runtime) if norm2 is not None else None
        self.feed_forward = build_part("feed_forward", feed_forward, runtime) if feed_forward is not None else None
        self.graph_safe = all(p.graph_safe for p in self.parts().values())

    def forward(self, ctx: StepContext, stream: ResidualStream, cache, write_cache: bool) -> None:
        n = ctx.n_tokens
        stream.rounded = None
        h = ctx.workspace.get("block.h", (n, self.hidden), self.runtime.dtype)
        self.norm1.apply(ctx, h, stream.resid, stream.pending, n, delta_scale=stream.pending_scale)
        ctx.upcoming_weights = self.feed_forward.streamed_first() if self.feed_forward is not None else None
        delta = self.mixer.forward(ctx, h, cache, write_cache)
        ctx.upcoming_weights = None
        stream.pending_scale = self.residual_scale
        if self.feed_forward is None:
            stream.pending = delta                              # a layer of its first half only
            return
        self.norm2.apply(ctx, h, stream.resid, delta, n, delta_scale=self.residual_scale)
        stream.pending = self.feed_forward.forward(ctx, h)      # whoever normalises next adds it


@register_part("block", "output_norm")
class OutputNormBlock(ArrangedBlock):
    """x = x + norm1(mixer(x));  x = x + norm2(feed_forward(x)): the norm sits on what a sub-layer returns,
    and the sub-layers read the residual rows themselves.  ``feed_forward`` (with ``norm2``) may be None: the
    layer then has its first half only.

    The residual stream stays fp32; the matrix products read a copy of its rows in the run's type, which the
    norm kernel writes while it adds (in float32 runs the stream itself is read).  Nothing is left pending.
    """

    def __init__(self, runtime: Runtime, hidden: int, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec | None = None,
                 feed_forward: PartSpec | None = None, names: dict[str, str] | None = None):
        super().__init__(runtime, hidden, names)
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("output_norm block: norm2 and feed_forward come together or not at all")
        self.norm1 = build_part("norm", norm1, runtime)
        self.mixer = build_part("mixer", mixer, runtime)
        self.norm2 = build_part("norm", norm2, runtime) if norm2 is not None else None
        self.feed_forward = build_part("feed_forward", feed_forward, runtime) if feed_forward is not None else None
        self.graph_safe = all(p.graph_safe for p in self.parts().values())

    def _rows(self, ctx: StepContext, stream: ResidualStream) -> tuple[torch.Tensor, torch.Tensor | None]:
        """(the rows a sub-layer reads, the buffer the next norm writes their successor into)."""
        n = ctx.n_tokens
        if self.runtime.dtype == torch.float32:
            return stream.resid[:n], None
        copy = ctx.workspace.get("block.rows", (n, self.hidden), self.runtime.dtype)
        if stream.rounded is None or stream.rounded.data_ptr() != copy.data_ptr():
            ops.round_rows(copy, stream.resid, n)
        return copy, copy

    def forward(self, ctx: StepContext, stream: ResidualStream, cache, write_cache: bool) -> None:
        n = ctx.n_tokens
        if stream.pending is not None:
            raise RuntimeError("output_norm block: the block before left a delta that only a norm of its own kind can add")
        stream.pending_scale = 1.0
        h, copy = self._rows(ctx, stream)
        ctx.upcoming_weights = self.feed_forward.streamed_first() if self.feed_forward is not None else None
        delta = self.mixer.forward(ctx, h, cache, write_cache)
        ctx.upcoming_weights = None
        self.norm1.add_normed(ctx, stream.resid, delta, n, copy)
        stream.rounded = copy
        if self.feed_forward is not None:
            delta = self.feed_forward.forward(ctx, h)
            self.norm2.add_normed(ctx, stream.resid, delta, n, copy)


@register_part("block", "hyper_pre_norm")
class HyperPreNormBlock(ArrangedBlock):
    """A pre-norm block over ``copies`` parallel copies of the residual stream (hyper-connections).

    For sub-layer q (1: the mixer, 2: the feed-forward) with the block's own tensors ``hc<q>.in`` [copies],
    ``hc<q>.out`` [copies] and ``hc<q>.mix`` [copies, copies] (indexed [from, to]):

        u   = sum_s in[s] x_s;   y = sublayer(norm_q(u))
        x_t <- sum_s mix[s, t] x_s + out[t] y             every copy at once, from the old ones

    All copies start as the embedding's rows; behind the last block the residual is their sum.  ``feed_forward``
    (with ``norm2``) may be None.  One kernel (``ops.hyper_step``) writes a sub-layer's output into the copies and
    reads the next sub-layer's normalised input in the same pass, also across blocks: the last write of a block is
    left pending and done by whoever reads the copies next.  The norms must be RMS norms (their weight and eps go
    into that kernel).
    """

    def __init__(self, runtime: Runtime, hidden: int, copies: int, norm1: PartSpec, mixer: PartSpec,
                 norm2: PartSpec | None = None, feed_forward: PartSpec | None = None, names: dict[str, str] | None = None):
        super().__init__(runtime, hidden, names)
        if not 0 < copies <= ops.HYPER_MAX_COPIES:
            raise ValueError(f"hyper_pre_norm block: between 1 and {ops.HYPER_MAX_COPIES} copies of the stream, got {copies}")
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("hyper_pre_norm block: norm2 and feed_forward come together or not at all")
        self.copies = int(copies)
        self.norm1 = build_part("norm", norm1, runtime)
        self.mixer = build_part("mixer", mixer, runtime)
        self.norm2 = build_part("norm", norm2, runtime) if norm2 is not None else None
        self.feed_forward = build_part("feed_forward", feed_forward, runtime) if feed_forward is not None else None
        for norm in (self.norm1, self.norm2):
            if norm is not None and not (hasattr(norm, "weight") and hasattr(norm, "eps")):
                raise ValueError("hyper_pre_norm block: its norms must be RMS norms with a weight and an eps")
        self.graph_safe = all(p.graph_safe for p in self.parts().values())
        c = self.copies
        subs = 2 if self.feed_forward is not None else 1
        self.hc = runtime.empty(subs, c * c + 2 * c, dtype=torch.float32)      # per sub-layer: in | out | mix

    def _coef(self, q: int):
        c = self.copies
        row = self.hc[q]
        return row[:c], row[c:2 * c], row[2 * c:]

    def weights(self) -> list[WeightDecl]:
        decls, c = super().weights(), self.copies
        for q in range(self.hc.shape[0]):
            a, b, m = self._coef(q)
            decls += [WeightDecl(f"hc{q + 1}.in", (c,), role="vector", init="one_plus_normal", dest=a),
                      WeightDecl(f"hc{q + 1}.out", (c,), role="vector", init="one_plus_normal", dest=b),
                      WeightDecl(f"hc{q + 1}.mix", (c, c), role="vector", init="eye_plus_normal", dest=m.view(c, c))]
        return decls

    def _pass(self, ctx: StepContext, stream: ResidualStream, read: int | None, h=None, sum_out=None) -> None:
        """Do the pending write (or the start from the embedding's rows), then read for sub-layer ``read``."""
        n = ctx.n_tokens
        args = {}
        if stream.copies is None:
            if stream.pending is not None:
                raise RuntimeError("hyper_pre_norm block: the block before left a delta that only its own kind of norm can add")
            stream.copies = ctx.workspace.get("model.copies", (n, self.copies, self.hidden), torch.float32)
            stream.fold = self._fold
            args["init"] = stream.resid
        elif unscaled_pending(stream, "hyper_pre_norm block") is not None:
            y, mix, out = stream.pending
            args.update(y=y, mix=mix, out_coef=out)
        stream.pending = None
        if stream.copies.shape[1] != self.copies:
            raise RuntimeError("hyper_pre_norm block: the stream has another number of copies than this block")
        if read is not None:
            norm = self.norm1 if read == 0 else self.norm2
            args.update(in_coef=self._coef(read)[0], norm_weight=norm.weight, eps=norm.eps, h_out=h)
        if args or sum_out is not None:
            ops.hyper_step(stream.copies, n, sum_out=sum_out, **args)

    def _fold(self, ctx: StepContext, stream: ResidualStream) -> None:
        self._pass(ctx, stream, None, sum_out=stream.resid)
        stream.rounded = None

    def forward(self, ctx: StepContext, stream: ResidualStream, cache, write_cache: bool) -> None:
        n, dt = ctx.n_tokens, self.runtime.dtype
        stream.rounded = None
        h = ctx.workspace.get("block.h", (n, self.hidden), dt)
        self._pass(ctx, stream, 0, h)
        stream.fold = self._fold
        ctx.upcoming_weights = self.feed_forward.streamed_first() if self.feed_forward is not None else None
        delta = self.mixer.forward(ctx, h, cache, write_cache)
        ctx.upcoming_weights = None
        _, out1, mix1 = self._coef(0)
        stream.pending = (dense_delta(ctx, delta, dt, "hyper.y")[:n], mix1, out1)
        if self.feed_forward is None:
            return
        self._pass(ctx, stream, 1, h)
        delta = self.feed_forward.forward(ctx, h)
        _, out2, mix2 = self._coef(1)
        stream.pending = (dense_delta(ctx, delta, dt, "hyper.y")[:n], mix2, out2)


@register_part("block", "parallel_pre_norm")
class ParallelPreNormBlock(ArrangedBlock):
    """x = x + (mixer(norm1(x)) + feed_forward(norm1(x))): one norm, and both sub-layers read its output.
    ``feed_forward`` may be None: the layer then has its mixer only.

    The mixer's delta is added to the fp32 residual rows right away (nothing reads them before the next norm); the
    feed-forward's is left pending, so the next norm's kernel adds it while it normalises.
    """

    ROLES = ("norm1", "mixer", "feed_forward")

    def __init__(self, runtime: Runtime, hidden: int, norm1: PartSpec, mixer: PartSpec, feed_forward: PartSpec | None = None,
                 names: dict[str, str] | None = None):
        super().__init__(runtime, hidden, names)
        self.norm1 = build_part("norm", norm1, runtime)
        self.mixer = build_part("mixer", mixer, runtime)
        self.feed_forward = build_part("feed_forward", feed_forward, runtime) if feed_forward is not None else None
        self.graph_safe = all(p.graph_safe for p in self.parts().values())

    def forward(self, ctx: StepContext, stream: ResidualStream, cache, write_cache: bool) -> None:
        n, dt = ctx.n_tokens, self.runtime.dtype
        stream.rounded = None
        h = ctx.workspace.get("block.h", (n, self.hidden), dt)
        self.norm1.apply(ctx, h, stream.resid, stream.pending, n, delta_scale=stream.pending_scale)
        stream.pending_scale = 1.0
        ctx.upcoming_weights = self.feed_forward.streamed_first() if self.feed_forward is not None else None
        delta = self.mixer.forward(ctx, h, cache, write_cache)
        ctx.upcoming_weights = None
        if self.feed_forward is None:
            stream.pending = delta
            return
        ops.add_delta(stream.resid, delta, n)
        stream.pending = self.feed_forward.forward(ctx, h)
