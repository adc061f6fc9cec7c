"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, PartSpec, Runtime, StepContext, WeightDecl, build_part, dense_delta, join_name, register_part
from .linear import grouped_matmul_nt, grouped_product_on_device, linear


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """delta = (silu(h @ Wg.T) * (h @ Wu.T)) @ Wd.T, no biases.

    gate and up are one product.  The reference packs the rows [Wg; Wu]
    (flow_engine/model.py:82-85); here, when the intermediate size is a multiple of 8, the rows
    alternate between eight gate rows and their eight up rows -- an exact permutation -- so
    that a tensor-core tile of the small-batch kernel holds a gate and its up in one thread and
    writes silu(gate) * up directly.  The activation runs in fp32.
    Reference: flow_engine/model.py:68-85.
    """

    NAMES = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")

    def __init__(self, runtime: Runtime, hidden: int, intermediate: int, names: tuple[str, str, str] | None = None):
        """``names``: the checkpoint's names of the gate, up and down matrices (default: the reference's)."""
        super().__init__(runtime)
        self.names = tuple(names) if names else self.NAMES
        if min(hidden, intermediate) <= 0:
            raise ValueError("swiglu needs positive sizes")
        self.hidden, self.intermediate = hidden, intermediate
        self.w_gate_up = runtime.empty(2 * intermediate, hidden)
        self.w_down = runtime.empty(hidden, intermediate)
        self.interleaved = intermediate % 8 == 0

    def weights(self) -> list[WeightDecl]:
        i = self.intermediate
        if self.interleaved:
            groups = self.w_gate_up.view(i // 8, 2, 8, self.hidden)
            gate, up = groups[:, 0], groups[:, 1]          # [i / 8, 8, hidden] views; the loader reshapes the source
        else:
            gate, up = self.w_gate_up[:i], self.w_gate_up[i:]
        return [WeightDecl(self.names[0], (i, self.hidden), dest=gate),
                WeightDecl(self.names[1], (i, self.hidden), dest=up),
                WeightDecl(self.names[2], (self.hidden, i), dest=self.w_down)]

    def forward(self, ctx: StepContext, h: torch.Tensor):
        return self.down(ctx, self.gate_up(ctx, h))

    def streamed_first(self) -> torch.Tensor:
        return self.w_gate_up

    def down(self, ctx: StepContext, act: torch.Tensor):
        """delta = act @ Wd.T (a tensor, or the slices of the product for the next norm to add)."""
        return linear(ctx, "ffn.delta", act, self.w_down, allow_split=True, consumer_early=True)

    def gate_up(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        """act = silu(h @ Wg.T) * (h @ Wu.T), by whichever kernel takes the step's number of rows."""
        n, ws, dt = ctx.n_tokens, ctx.workspace, self.runtime.dtype
        act = ws.get("ffn.act", (n, self.intermediate), dt)
        if self.interleaved and ops.small_m_supported(h, self.w_gate_up, n):
            ops.gemm_small_m(act, h, self.w_gate_up, n, silu_mul_pairs=True,
                             prefetch=ops.weight_head(self.w_down, ops.product_prefetch_bytes()))
        elif (self.interleaved and ops.stream_product_preferred(h, self.w_gate_up, n)
              and (ops.stream_whole_k_balanced(2 * self.intermediate) or ops.stream_split_gate_up_enabled())):
            # decode steps of 9 to 64 requests: persistent tcgen05 kernel, weights as the 128-row operand
            if ops.stream_whole_k_balanced(2 * self.intermediate):
                ops.gemm_tcgen05_stream(act, h, self.w_gate_up, n, ctx.status, silu_mul_pairs=True,    # SiLU.mul in its epilogue
                                        prefetch=ops.weight_head(self.w_down, ops.product_prefetch_bytes()))
            else:
                # the row tiles alone would leave half of the blocks with half of the work: slices over k, added
                # by the SiLU.mul kernel
                split, kper = ops.stream_split(2 * self.intermediate, self.hidden)
                slices = ws.get("ffn.gate_up.slices", (split, n, 2 * self.intermediate), torch.float32)
                ops.gemm_tcgen05_stream(slices if split > 1 else slices[0], h, self.w_gate_up, n, ctx.status, kper=kper)
                ops.silu_mul(act, ops.SplitSum(slices), n, True)
        elif self.interleaved and ops.pair_product_preferred(h, self.w_gate_up, n):
            # prompt steps: 256 x 256 tiles on pairs of thread blocks (tcgen05.mma.cta_group::2), SiLU.mul in the
            # epilogue, so the [tokens, 2 * intermediate] product never reaches memory
            ops.gemm_tcgen05_pair(act, h, self.w_gate_up, n, ctx.status, silu_mul_pairs=True)
        else:
            gate_up = linear(ctx, "ffn.gate_up", h, self.w_gate_up)
            ops.silu_mul(act, gate_up, n, self.interleaved)
        return act


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of gated experts, of which every token uses the ``top`` with the largest router logits.

        z = Wr h + br                                  fp32
        chosen = the `top` largest z;  c = softmax(z[chosen])
        delta = sum_{e in chosen} c_e Wd_e (silu(Wg_e h) * (Wu_e h))   [+ sigmoid(ws . h) * shared(h)]

    ``shared``: the spec of a feed-forward every token runs (its weights under ``shared_prefix``); with
    ``shared_gate`` its output is scaled per token by sigmoid of one more dot product (tensor ``shared_gate_name``,
    [1, hidden]).  Expert e's matrices are ``<expert_prefix><e>.gate|up|down`` in the checkpoint and live stacked:
    gate and up as [experts, 2, ff, hidden], down as [experts, hidden, ff].  The weighted sum is fp32.

    bfloat16 steps with more than ``GROUPED_MIN_ROWS`` rows (and matrices whose rows start on 16-byte boundaries) sort
    the pairs by expert and run every expert's rows through one library product, whose group bounds stay on the device.
    Steps of one row, float32 steps and odd sizes run each (token, expert) pair as matrix-vector products that stream
    the chosen experts' matrices (csrc/moe.cu).

    Options of other designs.  ``score_all``: the scores are s = softmax(z) over *every* router output, the ``top``
    outputs with the largest s + ``correction`` (a stored fp32 vector named by ``correction``, or none) are chosen, and
    the weights are their s times ``weight_scale``, not renormalised.  ``identity`` n: the router has n outputs more
    than there are experts; such an output is an expert without tensors whose result is the token's row itself.
    ``activation``: ``{"kind": "clamped", "limit": l, "alpha": a}`` makes an expert's inner rows
    g sigmoid(a g) (u + 1) with g = min(Wg h, l), u = clamp(Wu h, -l, l) instead of silu(Wg h) (Wu h).
    """

    GROUPED_MIN_ROWS = 1       # measured at 7B and 1.5B layer sizes: the sorted way is the faster one from two or three rows on

    def __init__(self, runtime: Runtime, hidden: int, experts: int, top: int, intermediate: int,
                 shared: PartSpec | None = None, shared_gate: bool = False, router_bias: bool = True,
                 names: dict[str, str] | None = None, score_all: bool = False, correction: str | None = None,
                 weight_scale: float = 1.0, identity: int = 0, activation: dict | None = None):
        super().__init__(runtime)
        if min(hidden, experts, top, intermediate) <= 0 or identity < 0 or top > experts + identity:
            raise ValueError("routed_experts: sizes must be positive and top at most the number of router outputs")
        if shared_gate and shared is None:
            raise ValueError("routed_experts: a gate of the shared expert needs a shared expert")
        if (correction is not None or weight_scale != 1.0) and not score_all:
            raise ValueError("routed_experts: a correction of the choice and a scale of the weights go with score_all")
        self.hidden, self.experts, self.top, self.intermediate = hidden, experts, top, intermediate
        self.identity, self.outputs = int(identity), experts + int(identity)
        self.score_all, self.weight_scale = bool(score_all), float(weight_scale)
        self.glu, self.glu_limit, self.glu_alpha = ops.GLU_SILU, 0.0, 1.0
        if activation is not None:
            if activation.get("kind") != "clamped" or not float(activation["limit"]) > 0:
                raise ValueError(f"routed_experts: unknown activation {activation!r} (known: clamped with a positive limit)")
            self.glu, self.glu_limit, self.glu_alpha = ops.GLU_CLAMPED, float(activation["limit"]), float(activation.get("alpha", 1.0))
        self.names = {"router": "router", "router_bias": "router.b", "expert": "e", "gate": "gate", "up": "up", "down": "down",
                      "shared": "shared", "shared_gate": "shared.sg", **(names or {})}
        self.w_router = runtime.empty(self.outputs, hidden)
        self.b_router = runtime.empty(self.outputs, dtype=torch.float32) if router_bias else None
        self.correction_name = correction
        self.correction = runtime.empty(self.outputs, dtype=torch.float32) if correction is not None else None
        self.w_gate_up = runtime.empty(experts, 2, intermediate, hidden)
        self.w_down = runtime.empty(experts, hidden, intermediate)
        self.shared = build_part("feed_forward", shared, runtime) if shared is not None else None
        self.w_shared_gate = runtime.empty(1, hidden) if shared_gate else None
        self.graph_safe = self.shared is None or self.shared.graph_safe

    def weights(self) -> list[WeightDecl]:
        nm, f, hid = self.names, self.intermediate, self.hidden
        decls = [WeightDecl(nm["router"], (self.outputs, hid), dest=self.w_router)]
        if self.b_router is not None:
            decls.append(WeightDecl(nm["router_bias"], (self.outputs,), role="vector", dest=self.b_router))
        if self.correction is not None:
            decls.append(WeightDecl(self.correction_name, (self.outputs,), role="vector", init="wide_normal", dest=self.correction))
        for e in range(self.experts):
            p = f"{nm['expert']}{e}"
            decls += [WeightDecl(join_name(p, nm["gate"]), (f, hid), dest=self.w_gate_up[e, 0]),
                      WeightDecl(join_name(p, nm["up"]), (f, hid), dest=self.w_gate_up[e, 1]),
                      WeightDecl(join_name(p, nm["down"]), (hid, f), dest=self.w_down[e])]
        if self.shared is not None:
            decls += [WeightDecl(join_name(nm["shared"], w.name), w.shape, w.role, w.init, w.dest) for w in self.shared.weights()]
        if self.w_shared_gate is not None:
            decls.append(WeightDecl(nm["shared_gate"], (1, hid), dest=self.w_shared_gate))
        return decls

    def finalize(self) -> None:
        if self.shared is not None:
            self.shared.finalize()

    def streamed_first(self) -> torch.Tensor | None:
        return None

    def route(self, ctx: StepContext, h: torch.Tensor):
        """(chosen int32 [rows, top], weights fp32 [rows, top], gate of the shared expert fp32 [rows] or None)"""
        n, ws = ctx.n_tokens, ctx.workspace
        chosen = ws.get("moe.chosen", (n, self.top), torch.int32)
        weight = ws.get("moe.weight", (n, self.top), torch.float32)
        gate = ws.get("moe.shared_gate", (n,), torch.float32) if self.w_shared_gate is not None else None
        ops.moe_route(chosen, weight, gate, h, self.w_router, self.b_router,
                      self.w_shared_gate.view(-1) if self.w_shared_gate is not None else None, n, self.top,
                      score_all=self.score_all, correction=self.correction, weight_scale=self.weight_scale)
        return chosen, weight, gate

    def forward(self, ctx: StepContext, h: torch.Tensor):
        n, ws, dt = ctx.n_tokens, ctx.workspace, self.runtime.dtype
        chosen, weight, gate = self.route(ctx, h)
        shared = None
        if self.shared is not None:
            shared = dense_delta(ctx, self.shared.forward(ctx, h), dt, "moe.shared")
        out = ws.get("moe.delta", (n, self.hidden), dt)
        # both ways' buffers are asked for in every step, so that the workspace has its final size after the largest one
        act = ws.get("moe.act", (n, self.top, self.intermediate), dt)
        sorted_buffers = self._sorted_buffers(ctx)
        if self.grouped_for(n) and (grouped_product_on_device() or not ctx.fixed_shape):
            # (a library without a grouped product reads the group bounds on the host: not inside a captured step)
            self._grouped(ctx, h, chosen, weight, shared, gate, out, sorted_buffers)
            return out
        ops.moe_gate_up(act, h, self.w_gate_up, chosen, n, glu=self.glu, limit=self.glu_limit, alpha=self.glu_alpha)
        ops.moe_down(out, act, self.w_down, chosen, weight, shared, gate, n, h=h if self.identity else None, identity=self.identity)
        return out

    def grouped_for(self, n_rows: int) -> bool:
        """Whether a step of ``n_rows`` rows sorts its pairs by expert: bfloat16, more than ``GROUPED_MIN_ROWS`` rows, and
        rows of the matrices that start on 16-byte boundaries (the library's grouped product wants that)."""
        return (self.runtime.dtype == torch.bfloat16 and n_rows > self.GROUPED_MIN_ROWS and self.hidden % 8 == 0
                and self.intermediate % 8 == 0)

    def _sorted_buffers(self, ctx: StepContext):
        n, ws, dt = ctx.n_tokens, ctx.workspace, self.runtime.dtype
        pairs = n * self.top
        return (ws.get("moe.order", (pairs,), torch.int32), ws.get("moe.place", (pairs,), torch.int32),
                ws.get("moe.ends", (self.experts,), torch.int32), ws.get("moe.sorted_rows", (pairs, self.hidden), dt),
                ws.get("moe.sorted_act", (pairs, self.intermediate), dt))

    def _grouped(self, ctx: StepContext, h, chosen, weight, shared, gate, out, buffers) -> None:
        """The pairs sorted by expert; gate/up, SiLU.mul and down as products over each expert's rows; the weighted
        sum (and the shared expert) per token."""
        n = ctx.n_tokens
        pairs = n * self.top
        order, place, ends, xs, act = buffers
        ops.moe_sort(order, place, ends, chosen, n)
        ops.moe_gather(xs, h, order, pairs, self.top)
        gate_up = grouped_matmul_nt(xs, self.w_gate_up.view(self.experts, 2 * self.intermediate, self.hidden), ends)
        if self.glu == ops.GLU_SILU:
            ops.silu_mul(act, gate_up, pairs, False)
        else:
            ops.glu_rows(act, gate_up, pairs, self.glu, self.glu_limit, self.glu_alpha)
        ys = grouped_matmul_nt(act, self.w_down, ends)
        if self.identity:
            ops.moe_combine(out, ys, place, weight, shared, gate, n, chosen=chosen, h=h, experts=self.experts, identity=self.identity)
        else:
            ops.moe_combine(out, ys, place, weight, shared, gate, n)
