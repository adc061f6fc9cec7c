"""Attention whose keys and values are expanded from one low-rank latent per token."""
from __future__ import annotations

import torch

from ..csrc import ops
from .attention import PagedSoftmaxMixer
from .base import PagedKV, PagedView, PartSpec, Runtime, StepContext, WeightDecl, build_part, register_part
from .linear import configure_matmul_precision, linear


@register_part("mixer", "latent_attention")
class LatentAttention(PagedSoftmaxMixer):
    """Softmax attention over a compressed cache: a token leaves one latent c [kv_rank] and one rotated key part
    r [rot_dim] behind, and every head's key and value are linear maps of c.

        cq = rms(Wdq h) * nq;   q_h = Wuq_h cq = [a_h (head_dim, not rotated) | b_h (rot_dim, rotated)]
        [c' | r] = Wdkv h;      c = rms(c') * nc;   r = rotate(r);  b_h = rotate(b_h)        (r is shared by all heads)
        k_h = Wuk_h c,  v_h = Wuv_h c
        s_h(i, j) = (a_h(i) . k_h(j) + b_h(i) . r(j)) * scale        over the keys the window lets i see
        o_h = sum_j softmax_j(s_h) v_h(j);   delta = Wo (o * sigmoid(Wg h))                   (the gate is optional)

    Neither k_h nor v_h is ever formed.  Because k_h is linear in c, a_h . k_h(j) = (Wuk_h^T a_h) . c(j): the query is
    carried into the latent space once per token, and then every head is an ordinary attention head of size
    kv_rank + rot_dim whose keys are the rows [c | r] of ONE key/value head and whose values are the same rows (the
    last rot_dim values of a result are not used); the head's value map is applied to the attention's result,
    o_h = Wuv_h (sum_j p_j c(j)).  The cache keeps [c | r] per token and nothing else (``values_are_keys``), and the
    paged kernels of the other attention mixers serve this one: exact, mma.sync prefill and split-KV decode (cached
    rows of more than 256 values: the exact kernel in both run types).

    The two per-head maps are batched library products.  The first one also moves b_h into place: head h multiplies by
    [[Wuk_h, 0], [0, I]], built once when the weights are in (the identity block copies bit for bit).

    ``position``: an encoding of neighbouring or half-apart pairs; it is applied to the last ``rot_dim`` values of a
    query head and to r.  ``names``: dq, dq_norm, uq, dkv, dkv_norm, uk, uv, gate, out.
    """

    NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
             "gate": "g", "out": "o"}

    def __init__(self, runtime: Runtime, hidden: int, n_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, q_rank: int,
                 kv_rank: int, scale: float, eps: float, position: PartSpec, window: int | None = None, output_gate: bool = True,
                 names: dict[str, str] | None = None):
        super().__init__(runtime)
        if min(hidden, n_heads, head_dim, v_head_dim, q_rank, kv_rank) <= 0 or rot_dim < 0 or rot_dim % 2:
            raise ValueError("latent_attention: sizes must be positive and the rotated part even")
        if kv_rank + rot_dim > 1024:
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {kv_rank + rot_dim} is more than the attention kernels' 1024")
        if window is not None and window <= 0:
            raise ValueError("latent_attention: window must be positive or None")
        if not eps > 0:
            raise ValueError("latent_attention: eps must be positive")
        self.hidden, self.n_heads, self.plain_dim, self.rot_dim, self.value_dim = hidden, n_heads, head_dim, rot_dim, v_head_dim
        self.q_rank, self.kv_rank, self.eps = q_rank, kv_rank, float(eps)
        self.q_head = head_dim + rot_dim                    # a query head as projected
        self.names = {**self.NAMES, **(names or {})}
        self.position = build_part("position", position, runtime)
        # what the shared kernel choice reads: H heads of size kv_rank + rot_dim on one key/value head
        self.n_kv_heads, self.head_dim = 1, kv_rank + rot_dim
        self.v_dim, self.same_dims = self.head_dim, True
        self.q_size = n_heads * self.head_dim
        self.window, self.scale = window, float(scale)
        self.sink = self.bias_rows = self.bias_by_distance = None
        self.score_terms = True                              # the values are the keys
        self.has_gate = bool(output_gate)
        self.out_size = n_heads * v_head_dim
        # rows [Wdq; Wdkv; Wg]: one product reads h
        self.in_width = q_rank + self.head_dim + (self.out_size if self.has_gate else 0)
        self.w_in = runtime.empty(self.in_width, hidden)
        self.w_uq = runtime.empty(n_heads * self.q_head, q_rank)
        self.q_norm_w = runtime.empty(q_rank, dtype=torch.float32)
        self.c_norm_w = runtime.empty(kv_rank, dtype=torch.float32)
        self.to_latent = torch.zeros(n_heads, self.q_head, self.head_dim, dtype=runtime.dtype, device=runtime.device)
        if rot_dim:
            self.to_latent[:, head_dim:, kv_rank:] = torch.eye(rot_dim, dtype=runtime.dtype, device=runtime.device)
        self.w_uv = runtime.empty(n_heads * v_head_dim, kv_rank)
        self.w_o = runtime.empty(hidden, self.out_size)

    def weights(self) -> list[WeightDecl]:
        nm, hid, H = self.names, self.hidden, self.n_heads
        a, b = self.q_rank, self.q_rank + self.head_dim
        decls = [WeightDecl(nm["dq"], (self.q_rank, hid), dest=self.w_in[:a]),
                 WeightDecl(nm["dq_norm"], (self.q_rank,), role="vector", init="one_plus_normal", dest=self.q_norm_w),
                 WeightDecl(nm["uq"], (H * self.q_head, self.q_rank), dest=self.w_uq),
                 WeightDecl(nm["dkv"], (self.head_dim, hid), dest=self.w_in[a:b]),
                 WeightDecl(nm["dkv_norm"], (self.kv_rank,), role="vector", init="one_plus_normal", dest=self.c_norm_w),
                 WeightDecl(nm["uk"], (H * self.plain_dim, self.kv_rank), dest=self.to_latent[:, :self.plain_dim, :self.kv_rank]),
                 WeightDecl(nm["uv"], (H * self.value_dim, self.kv_rank), dest=self.w_uv),
                 WeightDecl(nm["out"], (hid, self.out_size), dest=self.w_o)]
        if self.has_gate:
            decls.append(WeightDecl(nm["gate"], (self.out_size, hid), dest=self.w_in[b:]))
        return decls

    def cache_need(self) -> PagedKV:
        return PagedKV(1, self.head_dim, self.window, None, values_are_keys=True)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        if not isinstance(cache, PagedView):
            raise TypeError("latent_attention needs a paged cache")
        return self.project_out(ctx, self.attend(ctx, self.project_in(ctx, h), cache, write_cache))

    def project_in(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        """h @ [Wdq; Wdkv; Wg].T: rows [query latent | c' | r | gate] before norms and rotation."""
        return linear(ctx, "latent.in", h, self.w_in)

    def _plan(self):
        if not self.rot_dim:
            return None
        plan = self.position.rotary_plan(self.rot_dim)
        if plan is None or plan.rot_dims != self.rot_dim:
            raise ValueError("latent_attention: the position encoding must be a rotation of pairs over the whole rotated part")
        return plan

    def _rotate(self, ctx: StepContext, rows: torch.Tensor, n_heads: int, head_dim: int, first: int) -> None:
        plan = self._plan()
        if plan is None:
            return
        ops.rotate_pairs(rows, ctx.positions, ctx.seq_of_token, plan.inv_freq, ctx.n_tokens, n_heads, head_dim, plan.rot_dims,
                         plan.interleaved, magnitude=plan.magnitude, first=first)

    def prepare(self, ctx: StepContext, proj: torch.Tensor, cache: PagedView, write_cache: bool) -> torch.Tensor:
        """Norms, rotation, the store of [c | r], and the queries in the latent space: [rows, H * (kv_rank + rot_dim)]."""
        n, ws, dt, H = ctx.n_tokens, ctx.workspace, self.runtime.dtype, self.n_heads
        a = self.q_rank
        # one pass over a token's row: both latents' norms (the query latent into rows of its own, which the next
        # product reads), the rotation of the shared key part, the store of [c | r]
        plan = self._plan()
        cq = ws.get("latent.cq", (n, a), dt)
        ops.norm_rotate_store(proj, n, [(0, 1, self.q_rank, self.q_norm_w), (a, 1, self.kv_rank, self.c_norm_w)], self.eps,
                              ctx.positions, ctx.seq_of_token, ctx.seq_slot, cache.block_table, cache.k_pages, None, a, a,
                              write_cache, ctx.status, dst0=cq, rot_col=a + self.kv_rank, rot_dims=self.rot_dim,
                              inv_freq=plan.inv_freq if plan is not None else None,
                              interleaved=plan.interleaved if plan is not None else False,
                              magnitude=plan.magnitude if plan is not None else 1.0)
        q = linear(ctx, "latent.q", cq, self.w_uq)
        self._rotate(ctx, q, H, self.q_head, self.plain_dim)
        ql = ws.get("latent.q_latent", (n, self.q_size), dt)
        configure_matmul_precision()
        ops.note_call("library batched product")
        torch.bmm(q.view(n, H, self.q_head).transpose(0, 1), self.to_latent, out=ql.view(n, H, self.head_dim).transpose(0, 1))
        return ql

    def attend(self, ctx: StepContext, proj: torch.Tensor, cache: PagedView, write_cache: bool) -> torch.Tensor:
        """The heads' results after their value maps and the gate: [rows, H * v_head_dim]."""
        n, ws, dt, H = ctx.n_tokens, ctx.workspace, self.runtime.dtype, self.n_heads
        ql = self.prepare(ctx, proj, cache, write_cache)
        mixed = ws.get("latent.mixed", (n, self.q_size), dt)
        self._attend(ctx, mixed, ql, cache)
        out = ws.get("latent.out", (n, self.out_size), dt)
        ops.note_call("library batched product")
        torch.bmm(mixed.view(n, H, self.head_dim)[:, :, :self.kv_rank].transpose(0, 1),
                  self.w_uv.view(H, self.value_dim, self.kv_rank).transpose(1, 2),
                  out=out.view(n, H, self.value_dim).transpose(0, 1))
        if self.has_gate:
            ops.gate_mul(out, out, proj[:, self.q_rank + self.head_dim:], ops.GATE_SIGMOID, n)
        return out

    def project_out(self, ctx: StepContext, out: torch.Tensor):
        return linear(ctx, "mixer.delta", out, self.w_o, allow_split=True, consumer_early=True)
