"""Grouped-query attention over a paged cache."""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import (Mixer, PagedKV, PagedView, PartSpec, Runtime, StepContext, WeightDecl, build_part,
                   register_part)
from .linear import SplitSum, linear


class PagedSoftmaxMixer(Mixer):
    """What mixers that attend with a softmax over a paged cache share: the choice of the attention kernel for a
    step.  A subclass sets ``n_heads, n_kv_heads, head_dim, v_dim, same_dims, q_size, window, scale, sink, bias_rows,
    bias_by_distance, score_terms`` (``score_terms``: the softmax has a sink or a distance table, or the values are
    the keys -- what only the exact and the mma.sync kernels know) and hands ``_attend`` rows whose first ``q_size``
    columns are the queries, after it has stored the step's keys and values."""

    b_qkv = None

    def _prefetch_plan(self, ctx: StepContext):
        return None, None

    def _decode_launch(self, ctx: StepContext, cache: PagedView) -> tuple[bool, int, int]:
        """(fed by TMA?, slices per request, blocks) of the decode attention this step will launch."""
        group = self.n_heads // self.n_kv_heads
        tma = not self.score_terms and ops.decode_tma_supported(self.runtime.dtype, self.head_dim, cache.page_size)
        splits = ops.decode_tma_splits if tma else ops.decode_splits
        # (the keys a request can see: a window bounds them, and the kernels cut those into the slices)
        nsplit = splits(ctx.n_seqs, self.n_kv_heads, group, min(ctx.max_kv_len, self.window) if self.window else ctx.max_kv_len)
        return tma, nsplit, ctx.n_seqs * self.n_kv_heads * -(-group // 8) * nsplit

    def _attend_tensor_cores(self, ctx: StepContext, out: torch.Tensor, q: torch.Tensor, cache: PagedView) -> None:
        """bfloat16: flash attention for requests with several tokens, split-KV attention for
        requests with one; both read the same flat batch and skip the other's requests."""
        window = self.window or 0
        singles = ctx.decode_only or ctx.fixed_shape or any(n == 1 for n in ctx.host_q_len)
        if not ctx.decode_only:
            # long portions: tcgen05 kernel (TMA, accumulators in tensor memory); short ones, and the shapes it
            # does not take, stay on the mma.sync kernel, which starts faster
            prefill = ops.attention_prefill
            # (not with a window: that kernel copies whole key tiles, and the pages of a tile's keys before the
            # earliest window may have been given back; the mma.sync kernel skips such keys one by one)
            if not window and not self.score_terms and ops.prefer_tcgen05_attention(self.runtime.dtype, self.head_dim, cache.k_pages.shape[2], ctx.max_q_len):
                prefill = ops.attention_prefill_tcgen05
            prefill(out, q, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len, ctx.seq_slot,
                                  cache.block_table, cache.k_pages, cache.v_pages, ctx.n_seqs, ctx.max_q_len,
                                  self.n_heads, self.n_kv_heads, self.head_dim, window, self.scale, singles, ctx.status,
                                  **self._terms())
        if singles:
            self._decode(ctx, out, q, cache)

    def _decode(self, ctx: StepContext, out: torch.Tensor, q: torch.Tensor | None, cache: PagedView, fused=None) -> None:
        """Split-KV attention for the requests that bring one token; with ``fused`` = (product, rotation table,
        write_cache) the kernel makes q, k and v of the new token from the product itself.  Head sizes that are
        multiples of 64 take the kernel that is fed by TMA, the others the one that loads keys through registers."""
        group = self.n_heads // self.n_kv_heads
        tma, nsplit, _ = self._decode_launch(ctx, cache)
        scratch = ctx.workspace.get("attn.decode_scratch", (ops.decode_scratch_floats(self.n_heads, self.head_dim),),
                                    torch.float32)
        counters = ctx.workspace.get(
            "attn.decode_counters", (ops.decode_counter_ints(ctx.n_seqs, self.n_kv_heads, group),), torch.int32, zero=True)
        window = self.window or 0
        product, table, write_cache = fused if fused is not None else (None, None, False)
        prefetch = self._prefetch_plan(ctx)[0] if fused is not None else None
        if tma:
            ops.attention_decode_tma(out, q, product, self.b_qkv if fused is not None else None, table, write_cache,
                                     ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len, ctx.seq_slot, cache.block_table,
                                     cache.k_pages, cache.v_pages, ctx.n_seqs, self.n_heads, self.n_kv_heads, self.head_dim,
                                     window, self.scale, nsplit, scratch, counters, ctx.status, prefetch=prefetch)
        elif fused is not None:
            ops.attention_decode_fused(out, product, self.b_qkv, table, write_cache, ctx.seq_q_start, ctx.seq_q_len,
                                       ctx.seq_kv_len, ctx.seq_slot, cache.block_table, cache.k_pages, cache.v_pages,
                                       ctx.n_seqs, self.n_heads, self.n_kv_heads, self.head_dim, window, self.scale,
                                       nsplit, scratch, counters, ctx.status, prefetch=prefetch)
        else:
            ops.attention_decode(out, q, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len, ctx.seq_slot,
                                 cache.block_table, cache.k_pages, cache.v_pages, ctx.n_seqs, self.n_heads,
                                 self.n_kv_heads, self.head_dim, window, self.scale, nsplit, scratch, counters,
                                 ctx.status, **self._terms())

    def _terms(self) -> dict:
        return {"sink": self.sink, "bias_rows": self.bias_rows} if self.score_terms else {}

    def _attend(self, ctx: StepContext, out: torch.Tensor, qkv: torch.Tensor, cache: PagedView) -> None:
        q = qkv[:, : self.q_size]
        if self.same_dims and ops.tensor_core_attention_supported(self.runtime.dtype, self.head_dim):
            self._attend_tensor_cores(ctx, out, q, cache)
            return
        ops.attention_generic(out, q, ctx.positions, ctx.seq_of_token, ctx.seq_slot, cache.block_table,
                              cache.k_pages, cache.v_pages, ctx.n_tokens, self.n_heads, self.n_kv_heads,
                              self.head_dim, self.window or 0, self.scale, ctx.status, sink=self.sink,
                              bias_by_distance=self.bias_by_distance)


@register_part("mixer", "gqa_attention")
class GQAAttention(PagedSoftmaxMixer):
    """q/k/v projections (optionally biased), position encoding on q and k, paged causal
    attention with ``n_heads / n_kv_heads`` query heads per key/value head, output projection.

        q, k, v = split(h @ Wqkv.T + b)                 rows packed [Wq; Wk; Wv]
        q, k    = position(q), position(k)
        cache[slot(position)] = k, v
        out_h   = softmax(q_h . k_{h // group} * scale  over keys p <= position [, p > position - window]) @ v
        delta   = out @ Wo.T

    Reference: flow_engine/model.py:36-55 (projections, packing), 183-201 (forward),
    flow_engine/cache.py:93-100 (slots).  Weight names are the checkpoint's (``names`` replaces them).

    ``v_head_dim``: the size of a value head where it differs from ``head_dim`` (the size of a query and a key
    head); the output then has ``n_heads`` heads of that size.  Heads above 256 (up to 1024) attend with the exact
    kernel in both run types.  Such a mixer, and one whose position encoding no
    kernel applies on the way, adds the bias, applies the encoding and stores keys and values as separate
    steps, and attends with the exact kernel; everything else takes the fused and tensor-core kernels.

    ``values_are_keys``: there is no value projection; a position's value is its key as projected (and encoded), and
    the cache keeps one set of pages for both.  ``sink`` (a tensor name): a learned number per query head whose
    exponential joins the softmax's denominator -- it has no key and no value, is not scaled and counts once.
    ``distance_bias`` (``name``, ``rows``, ``far``): a learned table [rows, n_heads] added to the scaled score by
    bucketed distance n = position - key position: bucket(n) = n below rows // 2, else
    min(rows - 1, rows // 2 + floor(ln(n / (rows // 2)) / ln(far / (rows // 2)) * (rows - rows // 2))); the table by
    plain distance is made once, when the weights are in.  A mixer with any of the three stores its keys with the
    separate step and attends with the mma.sync kernels (prefill and split-KV decode), which add the table's entry to
    each score and the sink to the denominator, and read a tile of keys once for both products; in 32-bit, and with
    head sizes those kernels do not take, it attends with the exact kernel.

    ``sink_value``: the same number for every head instead of a learned one (0: "one added to the denominator").
    ``qk_norm`` (``q``, ``k``: tensor names; ``eps``): every head of q and of k is divided by its root mean square and
    multiplied by a weight [head_dim] that all heads share, before the position encoding (fp32; one kernel for both).
    Such a mixer takes the separate steps too.
    """

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias"}

    def __init__(self, runtime: Runtime, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 qkv_bias: bool, position: PartSpec, scale: float | None = None, window: int | None = None,
                 out_bias: bool = False, v_head_dim: int | None = None, names: dict[str, str] | None = None,
                 values_are_keys: bool = False, sink: str | None = None, distance_bias: dict | None = None,
                 sink_value: float | None = None, qk_norm: dict | None = None):
        super().__init__(runtime)
        if min(hidden, n_heads, n_kv_heads, head_dim) <= 0 or n_heads % n_kv_heads:
            raise ValueError("attention: heads must be positive and n_heads a multiple of n_kv_heads")
        if (head_dim % 2 and position.kind != "none") or head_dim > 1024:
            raise ValueError(f"attention: head_dim {head_dim} must be at most 1024, and even where heads are rotated")
        if out_bias:
            raise ValueError("attention: a bias on the output projection is not implemented")
        if window is not None and window <= 0:
            raise ValueError("attention: window must be positive or None")
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.v_dim = head_dim if v_head_dim is None else int(v_head_dim)
        if not 0 < self.v_dim <= 1024:
            raise ValueError(f"attention: v_head_dim {self.v_dim} must lie in 1..1024")
        self.same_dims = self.v_dim == head_dim
        self.values_are_keys = bool(values_are_keys)
        if self.values_are_keys and (not self.same_dims or qkv_bias):
            raise ValueError("attention: values that are the keys have the keys' size and no bias of their own")
        self.names = {**self.NAMES, **(names or {})}
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.window = window
        self.q_size, self.kv_size = n_heads * head_dim, n_kv_heads * head_dim
        self.v_size, self.out_size = (0 if self.values_are_keys else n_kv_heads * self.v_dim), n_heads * self.v_dim
        self.qkv_width = self.q_size + self.kv_size + self.v_size
        self.position = build_part("position", position, runtime)
        self.w_qkv = runtime.empty(self.qkv_width, hidden)
        self.b_qkv = runtime.empty(self.qkv_width, dtype=torch.float32) if qkv_bias else None
        self.w_o = runtime.empty(hidden, self.out_size)
        if sink is not None and sink_value is not None:
            raise ValueError("attention: the sink is learned (sink) or a constant (sink_value), not both")
        self.sink_name = sink
        self.sink = runtime.empty(n_heads, dtype=torch.float32) if sink is not None else None
        if sink_value is not None:
            self.sink = torch.full((n_heads,), float(sink_value), dtype=torch.float32, device=runtime.device)
        self.qk_norm = None
        if qk_norm is not None:
            self.qk_norm = {"q": str(qk_norm["q"]), "k": str(qk_norm["k"]), "eps": float(qk_norm["eps"])}
            if not self.qk_norm["eps"] > 0:
                raise ValueError("attention: the eps of the q/k norm must be positive")
            self.q_norm_w = runtime.empty(head_dim, dtype=torch.float32)
            self.k_norm_w = runtime.empty(head_dim, dtype=torch.float32)
        self.distance_bias = None
        self.bias_by_distance = None
        if distance_bias is not None:
            rows, far = int(distance_bias["rows"]), float(distance_bias["far"])
            if rows < 2 or not far > rows // 2:
                raise ValueError(f"attention: a distance table needs at least 2 rows and a far distance beyond rows // 2, got {rows} and {far}")
            self.distance_bias = {"name": str(distance_bias["name"]), "rows": rows, "far": far}
            self.bias_table = runtime.empty(rows, n_heads, dtype=torch.float32)
        # terms of the softmax that the kernels fed by TMA and the kernels that rotate on the way do not know
        self.score_terms = self.values_are_keys or self.sink is not None or self.distance_bias is not None
        self.separate_steps = self.score_terms or self.qk_norm is not None     # no kernel that rotates on the way does these
        self.bias_rows = None

    @staticmethod
    def distance_bucket(n: int, rows: int, far: float) -> int:
        half = rows // 2
        if n < half:
            return n
        return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))

    def finalize(self) -> None:
        if self.distance_bias is not None:
            # every distance a query can see, row by row; distances from the last row on share its bucket (the last)
            rows, far = self.distance_bias["rows"], self.distance_bias["far"]
            reach = int(math.ceil(far)) + 1
            if self.window is not None:
                reach = min(reach, self.window)
            buckets = [self.distance_bucket(n, rows, far) for n in range(reach)]
            index = torch.tensor(buckets, dtype=torch.long, device=self.bias_table.device)
            self.bias_by_distance = self.bias_table.index_select(0, index).contiguous()
            self.bias_rows = self.bias_by_distance.t().contiguous()        # [heads, distances]: a head's row is contiguous

    def weights(self) -> list[WeightDecl]:
        q, kv, nm = self.q_size, self.kv_size, self.names
        spans = (("q", 0, q), ("k", q, q + kv)) + ((("v", q + kv, self.qkv_width),) if not self.values_are_keys else ())
        extra = []
        if self.qk_norm is not None:
            extra += [WeightDecl(self.qk_norm["q"], (self.head_dim,), role="vector", init="one_plus_normal", dest=self.q_norm_w),
                      WeightDecl(self.qk_norm["k"], (self.head_dim,), role="vector", init="one_plus_normal", dest=self.k_norm_w)]
        if self.sink_name is not None:
            extra.append(WeightDecl(self.sink_name, (self.n_heads,), role="vector", init="wide_normal", dest=self.sink))
        if self.distance_bias is not None:
            extra.append(WeightDecl(self.distance_bias["name"], (self.distance_bias["rows"], self.n_heads), role="vector",
                                    init="wide_normal", dest=self.bias_table))
        decls = [WeightDecl(nm[n], (e - b, self.hidden), dest=self.w_qkv[b:e]) for n, b, e in spans]
        if self.b_qkv is not None:
            decls += [WeightDecl(nm[f"{n}_bias"], (e - b,), role="vector", dest=self.b_qkv[b:e]) for n, b, e in spans]
        decls.append(WeightDecl(nm["o"], (self.hidden, self.out_size), dest=self.w_o))
        return decls + extra

    def cache_need(self) -> PagedKV:
        return PagedKV(self.n_kv_heads, self.head_dim, self.window, None if self.same_dims else self.v_dim,
                       values_are_keys=self.values_are_keys)

    def _fused_table(self):
        """The rotation table of the kernels that rotate on the way; None where the mixer takes the separate steps."""
        return self.position.fused_rotary_table(self.head_dim) if self.same_dims and not self.separate_steps else None

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        if not isinstance(cache, PagedView):
            raise TypeError("gqa_attention needs a paged key/value cache")
        return self.project_out(ctx, self.attend(ctx, self.project_qkv(ctx, h, cache), cache, write_cache))

    def _fused_decode(self, ctx: StepContext):
        """The rotation table, if this step's attention kernel adds the bias, rotates, writes the new key and value
        and attends all by itself (decode-only steps in bfloat16 with a rotary encoding); else None."""
        table = self._fused_table()
        if (table is not None and ctx.decode_only and ops.fused_decode_enabled()
                and ops.tensor_core_attention_supported(self.runtime.dtype, self.head_dim)):
            return table
        return None

    def project_qkv(self, ctx: StepContext, h: torch.Tensor, cache: PagedView | None = None):
        """h @ [Wq; Wk; Wv].T without the bias: a tensor, or the slices of a split product where the kernel
        that follows adds them itself (both rotary kernels do).  With the cache the attention will read, the
        product knows how large that launch will be and lets a small one settle on the SMs while it runs."""
        rotary = self._fused_table() is not None
        fused = self._fused_decode(ctx) is not None
        early = False
        if fused and cache is not None:
            tma, nsplit, blocks = self._decode_launch(ctx, cache)
            early = tma and ops.decode_attention_resident_early(blocks, nsplit)
        # the decode kernel reads the product once per block: up to four slices are one round trip to L2 for it
        return linear(ctx, "attn.qkv", h, self.w_qkv, allow_split=rotary, max_slices=4 if fused else 12,
                      consumer_early=early)

    def project_out(self, ctx: StepContext, out: torch.Tensor):
        return linear(ctx, "mixer.delta", out, self.w_o, allow_split=True, consumer_early=True,
                      prefetch=self._prefetch_plan(ctx)[1])

    def _prefetch_plan(self, ctx: StepContext):
        """What a decode-only step asks into L2 ahead of its kernel, of the weights the part after this one
        streams first (``ctx.upcoming_weights``): (the attention kernel's share, the output product's share).
        While the attention's slices merge and while the output product ends, the memory system has little to do.
        Not this part's own output matrix (the product that reads it starts fetching it before the attention has
        ended); and the attention only asks where its keys take longer to read than the output matrix, else the
        two fetches collide."""
        upcoming = ctx.upcoming_weights
        if upcoming is None or self._fused_decode(ctx) is None:
            return None, None
        window = self.window or 0
        keys = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        cache_bytes = ctx.n_seqs * keys * self.n_kv_heads * (self.head_dim + self.v_dim) * self.w_qkv.element_size()   # the cache has the weights' type
        first = ops.weight_prefetch_bytes() if cache_bytes >= ops.weight_prefetch_min_cache_bytes() else 0
        return (ops.weight_head(upcoming, first),
                ops.weight_head(upcoming, ops.output_product_prefetch_bytes(), skip_bytes=first))

    def attend(self, ctx: StepContext, qkv, cache: PagedView, write_cache: bool) -> torch.Tensor:
        """Bias, position encoding, cache write and attention for the step's rows; [rows, Hq * D]."""
        n, ws, dt = ctx.n_tokens, ctx.workspace, self.runtime.dtype
        table = self._fused_table()
        source = None
        if isinstance(qkv, SplitSum):       # the kernels below add the slices themselves
            source, qkv = qkv, ws.get("attn.qkv", (n, self.qkv_width), dt)
        out = ws.get("attn.out", (n, self.out_size), dt)
        if self._fused_decode(ctx) is not None:
            # decode-only step: the attention kernel adds the bias, rotates, writes the new key and value and attends
            self._decode(ctx, out, None, cache, fused=(source if source is not None else qkv, table, write_cache))
            return out
        if not self.same_dims or self.separate_steps:
            # keys and values of different sizes, or what only the exact kernel knows: bias, the norm of every head,
            # the position part's own transformation, then the store (values that are the keys share the keys' pages:
            # one store)
            if self.b_qkv is not None:
                ops.add_bias_rows(qkv, self.b_qkv, n)
            if self.qk_norm is not None:
                spans = [(0, self.n_heads, self.head_dim, self.q_norm_w), (self.q_size, self.n_kv_heads, self.head_dim, self.k_norm_w)]
                if self.position.kind == "none":
                    # the norms of the heads and the store in one pass over the token's row
                    ops.norm_rotate_store(qkv, n, spans, self.qk_norm["eps"], ctx.positions, ctx.seq_of_token, ctx.seq_slot,
                                          cache.block_table, cache.k_pages, None if self.values_are_keys else cache.v_pages,
                                          self.q_size, self.q_size + self.kv_size, write_cache, ctx.status)
                    self._attend(ctx, out, qkv, cache)
                    return out
                ops.span_rmsnorm(qkv, n, spans, self.qk_norm["eps"])
            self.position.apply(ctx, qkv, self.n_heads + self.n_kv_heads, self.head_dim)
            if write_cache:
                ops.kv_store(qkv, self.q_size, self.q_size + self.kv_size, ctx.positions, ctx.seq_of_token, ctx.seq_slot,
                             cache.block_table, cache.k_pages, None if self.values_are_keys else cache.v_pages, n, ctx.status)
            self._attend(ctx, out, qkv, cache)
            return out
        if table is None:
            # generic path: bias, then the position part's own transformation, then the cache write
            if self.b_qkv is not None:
                ops.rotate_heads(qkv, self.b_qkv, ctx.positions, ctx.seq_of_token, None, n,
                                 self.n_heads + 2 * self.n_kv_heads, self.head_dim)
            self.position.apply(ctx, qkv, self.n_heads + self.n_kv_heads, self.head_dim)
            bias = None
        else:
            bias = self.b_qkv
        ops.rope_kv_write(qkv, bias, ctx.positions, ctx.seq_of_token, ctx.seq_slot, cache.block_table, table,
                          cache.k_pages, cache.v_pages, n, self.n_heads, self.n_kv_heads, self.head_dim,
                          write_cache, ctx.status, source=source)
        self._attend(ctx, out, qkv, cache)
        return out
