"""Recurrent mixers: a state of fixed size per request instead of a cache that grows."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FixedState, Mixer, PartSpec, Runtime, StateView, StepContext, WeightDecl, build_part, register_part
from .linear import linear


@register_part("mixer", "mingru")
class MinGRU(Mixer):
    """A gated recurrence whose gates read only the current token.

        z = sigmoid(h Wz^T + bz),  u = h Wx^T + bx,  c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
        S_t = (1 - z_t) S_{t-1} + z_t c_t            element by element, fp32, zero before the first token
        delta = (S_t * silu(h Wg^T)) Wo^T

    The state (``width`` fp32 values per request) lives in a slot of the cache manager, which zeroes it
    when a request is admitted; a step reads it at a request's first row and writes it back after its
    last, so prompts may be cut anywhere.  z, u and the gate are one packed product [Wz; Wx; Wg].

    ``names`` gives the checkpoint's tensor names: z, z_bias, x, x_bias, gate, out.
    """

    NAMES = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "gate": "g", "out": "o"}

    def __init__(self, runtime: Runtime, hidden: int, width: int, names: dict[str, str] | None = None):
        super().__init__(runtime)
        if min(hidden, width) <= 0:
            raise ValueError("mingru needs positive sizes")
        self.hidden, self.width = hidden, width
        self.names = {**self.NAMES, **(names or {})}
        self.w_in = runtime.empty(3 * width, hidden)                  # rows [Wz; Wx; Wg]
        self.b_z = runtime.empty(width, dtype=torch.float32)
        self.b_x = runtime.empty(width, dtype=torch.float32)
        self.w_o = runtime.empty(hidden, width)

    def weights(self) -> list[WeightDecl]:
        w, nm = self.width, self.names
        return [WeightDecl(nm["z"], (w, self.hidden), dest=self.w_in[:w]),
                WeightDecl(nm["z_bias"], (w,), role="vector", dest=self.b_z),
                WeightDecl(nm["x"], (w, self.hidden), dest=self.w_in[w:2 * w]),
                WeightDecl(nm["x_bias"], (w,), role="vector", dest=self.b_x),
                WeightDecl(nm["gate"], (w, self.hidden), dest=self.w_in[2 * w:]),
                WeightDecl(nm["out"], (self.hidden, w), dest=self.w_o)]

    def cache_need(self) -> FixedState:
        return FixedState(self.width, torch.float32)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        if not isinstance(cache, StateView):
            raise TypeError("mingru needs a fixed-size state per request")
        return self.project_out(ctx, self.recur(ctx, self.project_in(ctx, h), cache, write_cache))

    def project_in(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        """h @ [Wz; Wx; Wg].T, rows [z | x | gate] before their biases and activations."""
        return linear(ctx, "mingru.in", h, self.w_in)

    def recur(self, ctx: StepContext, proj: torch.Tensor, cache: StateView, write_state: bool = True) -> torch.Tensor:
        """[rows, width]: S_t * silu(gate) for the step's rows; the requests' states move on."""
        out = ctx.workspace.get("mingru.out", (ctx.n_tokens, self.width), self.runtime.dtype)
        ops.mingru_scan(out, proj, self.b_z, self.b_x, cache.state, ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len,
                        ctx.n_seqs, ctx.max_q_len, self.width, write_state)
        return out

    def project_out(self, ctx: StepContext, out: torch.Tensor):
        return linear(ctx, "mixer.delta", out, self.w_o, allow_split=True)


class MatrixStateMixer(Mixer):
    """What the mixers below share: a matrix state S [key_dim, value_dim] per head in a fixed-size slot, walked by
    ``ops.linear_recurrence`` (one rule per mixer), then the norm over each head, an optional weight and a gate
    (``ops.head_norm_gate``), then the output matrix.  The raw outputs and the state are fp32."""

    rule: int = -1
    gate_act: int = ops.GATE_NONE

    def _sizes(self, hidden: int, n_heads: int, key_dim: int, value_dim: int, eps: float) -> None:
        if min(hidden, n_heads, key_dim, value_dim) <= 0 or not eps > 0:
            raise ValueError(f"{self.kind}: sizes and eps must be positive")
        if key_dim > ops.RECURRENCE_MAX_KEY_DIM or value_dim > 255:
            raise ValueError(f"{self.kind}: a head of {key_dim} x {value_dim} does not fit the recurrence kernel "
                             f"(keys up to {ops.RECURRENCE_MAX_KEY_DIM}, values up to 255)")
        self.hidden, self.n_heads, self.key_dim, self.value_dim, self.eps = hidden, n_heads, key_dim, value_dim, float(eps)
        self.qk_size, self.v_size = n_heads * key_dim, n_heads * value_dim
        self.state_numel = ops.recurrence_state_numel(self.rule, n_heads, key_dim, value_dim)

    def cache_need(self) -> FixedState:
        return FixedState(self.state_numel, torch.float32)

    def _check(self, cache) -> StateView:
        if not isinstance(cache, StateView):
            raise TypeError(f"{self.kind} needs a fixed-size state per request")
        return cache

    def _recur(self, ctx: StepContext, q, k, v, cache: StateView, write_state: bool, **rule_args):
        """(raw fp32 [rows, heads * value_dim], denominators or None)"""
        n, ws = ctx.n_tokens, ctx.workspace
        raw = ws.get("recurrence.raw", (n, self.v_size), torch.float32)
        den = ws.get("recurrence.den", (n, self.n_heads), torch.float32) if self.rule == ops.RECURRENCE_MLSTM else None
        ops.linear_recurrence(self.rule, raw, den, q, k, v, cache.state, ctx.positions, ctx.seq_slot, ctx.seq_q_start,
                              ctx.seq_q_len, ctx.n_seqs, self.n_heads, self.key_dim, self.value_dim, write_state,
                              max_q_len=ctx.max_q_len, **rule_args)
        return raw, den

    def _finish(self, ctx: StepContext, raw, den, weight, gate):
        out = ctx.workspace.get("recurrence.out", (ctx.n_tokens, self.v_size), self.runtime.dtype)
        ops.head_norm_gate(out, raw, den, weight, gate, self.gate_act, self.eps, ctx.n_tokens, self.n_heads, self.value_dim)
        return linear(ctx, "mixer.delta", out, self.w_o, allow_split=True)


@register_part("mixer", "retention")
class Retention(MatrixStateMixer):
    """Linear attention with a constant decay per head and no softmax or denominator.

        q, k, v, g = split(h W^T)                  heads of key_dim (q, k) and value_dim (v, g); rows [Wq; Wk; Wv; Wg]
        q, k = position(q), position(k);  k <- k * key_dim^-1/2
        S_t = decay_h S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t                     fp32, S zero before the first token
        delta = (rms_head(o) * silu(g)) Wo^T                                    the head norm has no weight

    A position encoding that is a rotation of (i, i + dims/2) pairs is applied inside the recurrence kernel (fp32,
    before the scale); any other encoding through its own ``apply``.  ``names``: q, k, v, gate, out.
    """

    rule = ops.RECURRENCE_RETENTION
    gate_act = ops.GATE_SILU
    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o"}

    def __init__(self, runtime: Runtime, hidden: int, n_heads: int, key_dim: int, value_dim: int, decay: tuple, eps: float,
                 position: PartSpec | None = None, names: dict[str, str] | None = None):
        super().__init__(runtime)
        self._sizes(hidden, n_heads, key_dim, value_dim, eps)
        if len(decay) != n_heads:
            raise ValueError(f"retention: {len(decay)} decays for {n_heads} heads")
        self.names = {**self.NAMES, **(names or {})}
        self.position = build_part("position", position, runtime) if position is not None else None
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32, device=runtime.device)
        self.w_in = runtime.empty(2 * self.qk_size + 2 * self.v_size, hidden)          # rows [Wq; Wk; Wv; Wg]
        self.w_o = runtime.empty(hidden, self.v_size)

    def weights(self) -> list[WeightDecl]:
        a, b, nm = self.qk_size, self.v_size, self.names
        return [WeightDecl(nm["q"], (a, self.hidden), dest=self.w_in[:a]),
                WeightDecl(nm["k"], (a, self.hidden), dest=self.w_in[a:2 * a]),
                WeightDecl(nm["v"], (b, self.hidden), dest=self.w_in[2 * a:2 * a + b]),
                WeightDecl(nm["gate"], (b, self.hidden), dest=self.w_in[2 * a + b:]),
                WeightDecl(nm["out"], (self.hidden, b), dest=self.w_o)]

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        cache = self._check(cache)
        a, b = self.qk_size, self.v_size
        proj = linear(ctx, "retention.in", h, self.w_in)
        plan = self.position.rotary_plan(self.key_dim) if self.position is not None else None
        rotate = {}
        if plan is not None and not plan.interleaved and plan.magnitude == 1.0:
            rotate = {"inv_freq": plan.inv_freq, "rot_dims": plan.rot_dims}
        elif self.position is not None:
            self.position.apply(ctx, proj, 2 * self.n_heads, self.key_dim)
        raw, _ = self._recur(ctx, proj[:, :a], proj[:, a:2 * a], proj[:, 2 * a:2 * a + b], cache, write_cache,
                             p0=self.decay, k_scale=self.key_dim ** -0.5, **rotate)
        return self._finish(ctx, raw, None, None, proj[:, 2 * a + b:])


@register_part("mixer", "wkv")
class WKV(MatrixStateMixer):
    """Time mixing with a decay per key channel that depends on the token, and a bonus for the token itself.

        x_s = h + (h' - h) * mu_s          s in r, k, v, g, w;  h' the row before in the request (zeros at its start)
        r, k, v = Wr x_r, Wk x_k, Wv x_v   heads of head_dim;   gate = silu(Wg x_g)
        w = exp(-exp(W2 tanh(W1 x_w) + w0))                                   fp32, per head and key channel
        o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t,   S_t = diag(w_t) S_{t-1} + k_t v_t^T      fp32
        delta = (rms_head(o) * norm * gate) Wo^T

    The state slot holds S of every head and, behind them, the last row h the mixer read (what the next step's
    first token is mixed with).  ``decay_rank`` is the inner size of W1 / W2.
    """

    rule = ops.RECURRENCE_WKV
    gate_act = ops.GATE_SILU
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, runtime: Runtime, hidden: int, n_heads: int, head_dim: int, decay_rank: int, eps: float):
        super().__init__(runtime)
        self._sizes(hidden, n_heads, head_dim, head_dim, eps)
        if decay_rank <= 0:
            raise ValueError("wkv: decay_rank must be positive")
        self.decay_rank = int(decay_rank)
        self.shift_offset = self.state_numel           # where the previous row sits in a request's slot
        self.state_numel += hidden
        size = self.qk_size
        self.mu = runtime.empty(len(self.MIXES), hidden, dtype=torch.float32)
        self.w_r, self.w_k, self.w_v, self.w_g = (runtime.empty(size, hidden) for _ in range(4))
        self.w_1 = runtime.empty(self.decay_rank, hidden)
        self.w_2 = runtime.empty(size, self.decay_rank)
        self.w_0 = runtime.empty(size, dtype=torch.float32)
        self.bonus = runtime.empty(size, dtype=torch.float32)
        self.norm = runtime.empty(size, dtype=torch.float32)
        self.w_o = runtime.empty(hidden, size)

    def weights(self) -> list[WeightDecl]:
        size, hid = self.qk_size, self.hidden
        decls = [WeightDecl(f"mu.{s}", (hid,), role="vector", dest=self.mu[i]) for i, s in enumerate(self.MIXES)]
        decls += [WeightDecl(n, (size, hid), dest=w) for n, w in (("r", self.w_r), ("k", self.w_k), ("v", self.w_v), ("g", self.w_g))]
        decls += [WeightDecl("w1", (self.decay_rank, hid), dest=self.w_1), WeightDecl("w2", (size, self.decay_rank), dest=self.w_2),
                  WeightDecl("w0", (size,), role="vector", dest=self.w_0),
                  WeightDecl("u", (self.n_heads, self.key_dim), role="vector", dest=self.bonus.view(self.n_heads, self.key_dim)),
                  WeightDecl("norm", (size,), role="vector", init="one_plus_normal", dest=self.norm),
                  WeightDecl("o", (hid, size), dest=self.w_o)]
        return decls

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        cache = self._check(cache)
        n, ws, dt = ctx.n_tokens, ctx.workspace, self.runtime.dtype
        mixes = ws.get("wkv.mixes", (len(self.MIXES), n, self.hidden), dt)
        ops.token_shift_mix(mixes, h, self.mu, cache.state, self.shift_offset, ctx.seq_of_token, ctx.seq_slot,
                            ctx.seq_q_start, n)
        r = linear(ctx, "wkv.r", mixes[0], self.w_r)
        k = linear(ctx, "wkv.k", mixes[1], self.w_k)
        v = linear(ctx, "wkv.v", mixes[2], self.w_v)
        g = linear(ctx, "wkv.g", mixes[3], self.w_g)
        inner = linear(ctx, "wkv.w1", mixes[4], self.w_1)
        ops.tanh_rows(inner)
        decay = linear(ctx, "wkv.w2", inner, self.w_2, out_dtype=torch.float32)
        raw, _ = self._recur(ctx, r, k, v, cache, write_cache, pre=decay, p0=self.w_0, p1=self.bonus,
                             tail=h, tail_offset=self.shift_offset)
        return self._finish(ctx, raw, None, self.norm, g)


@register_part("mixer", "mlstm")
class MLSTM(MatrixStateMixer):
    """A matrix memory with exponential input and forget gates, kept in range by a running maximum.

        q, k, v, g = split(h W^T);  q <- q * key_dim^-1/2                     rows [Wq; Wk; Wv; Wg]
        i = cap tanh((Wi h + bi) / cap),  f = logsigmoid(cap tanh((Wf h + bf) / cap))       per head, fp32
        m_t = max(f + m_{t-1}, i)                                             m is 0 before the first token
        S_t = e^(f + m_{t-1} - m_t) S_{t-1} + e^(i - m_t) k v^T,  n_t likewise with k alone
        o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6)
        delta = (rms_head(o) * norm * sigmoid(g)) Wo^T

    The gates' pre-activations come from a product of their own with an fp32 result.  ``names``: q, k, v, gate, out,
    norm, i, i_bias, f, f_bias.
    """

    rule = ops.RECURRENCE_MLSTM
    gate_act = ops.GATE_SIGMOID
    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "i": "i", "i_bias": "i.b",
             "f": "f", "f_bias": "f.b"}

    def __init__(self, runtime: Runtime, hidden: int, n_heads: int, key_dim: int, value_dim: int, gate_cap: float, eps: float,
                 names: dict[str, str] | None = None):
        super().__init__(runtime)
        self._sizes(hidden, n_heads, key_dim, value_dim, eps)
        if not gate_cap > 0:
            raise ValueError("mlstm: gate_cap must be positive")
        self.gate_cap = float(gate_cap)
        self.names = {**self.NAMES, **(names or {})}
        self.w_in = runtime.empty(2 * self.qk_size + 2 * self.v_size, hidden)          # rows [Wq; Wk; Wv; Wg]
        self.w_gates = runtime.empty(2 * n_heads, hidden)                              # rows [Wi; Wf]
        self.b_gates = runtime.empty(2 * n_heads, dtype=torch.float32)
        self.norm = runtime.empty(self.v_size, dtype=torch.float32)
        self.w_o = runtime.empty(hidden, self.v_size)

    def weights(self) -> list[WeightDecl]:
        a, b, H, nm = self.qk_size, self.v_size, self.n_heads, self.names
        return [WeightDecl(nm["q"], (a, self.hidden), dest=self.w_in[:a]),
                WeightDecl(nm["k"], (a, self.hidden), dest=self.w_in[a:2 * a]),
                WeightDecl(nm["v"], (b, self.hidden), dest=self.w_in[2 * a:2 * a + b]),
                WeightDecl(nm["gate"], (b, self.hidden), dest=self.w_in[2 * a + b:]),
                WeightDecl(nm["i"], (H, self.hidden), dest=self.w_gates[:H]),
                WeightDecl(nm["i_bias"], (H,), role="vector", dest=self.b_gates[:H]),
                WeightDecl(nm["f"], (H, self.hidden), dest=self.w_gates[H:]),
                WeightDecl(nm["f_bias"], (H,), role="vector", dest=self.b_gates[H:]),
                WeightDecl(nm["norm"], (b,), role="vector", init="one_plus_normal", dest=self.norm),
                WeightDecl(nm["out"], (self.hidden, b), dest=self.w_o)]

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        cache = self._check(cache)
        a, b = self.qk_size, self.v_size
        proj = linear(ctx, "mlstm.in", h, self.w_in)
        gates = linear(ctx, "mlstm.gates", h, self.w_gates, out_dtype=torch.float32)
        raw, den = self._recur(ctx, proj[:, :a], proj[:, a:2 * a], proj[:, 2 * a:2 * a + b], cache, write_cache,
                               pre=gates, p0=self.b_gates, q_scale=self.key_dim ** -0.5, cap=self.gate_cap)
        return self._finish(ctx, raw, den, self.norm, proj[:, 2 * a + b:])


@register_part("mixer", "gated_delta")
class GatedDelta(MatrixStateMixer):
    """The gated delta rule: a matrix memory that decays, then is corrected towards the token's value.

        q, k = Wq h, Wk h   (n_qk_heads heads of key_dim);   v = Wv h   (n_heads heads of value_dim)
        each of q, k, v: a causal convolution over time per channel (``conv_taps`` taps, zeros before the start), then silu
        q <- q / sqrt(sum q^2 + 1e-6) * key_dim^-1/2,  k <- k / sqrt(sum k^2 + 1e-6)          per head, fp32
        beta = sigmoid(Wb h)                                                                per head
        g = exp(-exp(A_h) softplus(d + dt_bias))       d = Wa h per head, or with ``channel_decay`` Wa2 (Wa1 h) per head
                                                       and key channel (inner size ``decay_rank``)
        S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                  fp32, S zero at the start
        delta = (rms_head(o) * norm * act(gate)) Wo^T        gate = Wg h, or with ``gate_rank`` Wg2 (Wg1 h); ``gate`` names
                                                       the activation (silu or sigmoid); norm [value_dim] serves every head

    Value head h reads q/k head h // (n_heads / n_qk_heads).  The state slot holds S of every head and, behind them, the
    last ``conv_taps - 1`` inputs of every convolved channel, so a request may be cut into steps anywhere.
    Tensor names: q, k, v (each with ``.conv`` [channels, taps]), b, A_log, dt_bias, norm, o, and a, g or a1, a2, g1, g2.
    """

    rule = ops.RECURRENCE_DELTA
    UNIT_EPS = 1e-6

    def __init__(self, runtime: Runtime, hidden: int, n_heads: int, n_qk_heads: int, key_dim: int, value_dim: int,
                 conv_taps: int, eps: float, channel_decay: bool = False, decay_rank: int | None = None, gate: str = "silu",
                 gate_rank: int | None = None):
        super().__init__(runtime)
        self._sizes(hidden, n_heads, key_dim, value_dim, eps)
        if n_qk_heads <= 0 or n_heads % n_qk_heads:
            raise ValueError("gated_delta: n_heads must be a multiple of n_qk_heads")
        if not 1 <= conv_taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"gated_delta: conv_taps must lie in 1..{ops.SHORT_CONV_MAX_TAPS}")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"gated_delta: unknown gate activation {gate!r}")
        if channel_decay and not decay_rank:
            raise ValueError("gated_delta: a decay per channel needs the inner size of its projection (decay_rank)")
        self.gate_act = ops.GATE_SILU if gate == "silu" else ops.GATE_SIGMOID
        self.n_qk_heads, self.taps = int(n_qk_heads), int(conv_taps)
        self.channel_decay = bool(channel_decay)
        self.decay_rank = int(decay_rank) if channel_decay else None
        self.gate_rank = int(gate_rank) if gate_rank else None
        self.qk_size = n_qk_heads * key_dim                      # (the base class counted a q/k head per value head)
        self.conv_channels = 2 * self.qk_size + self.v_size
        self.conv_offset = self.state_numel                      # where the convolutions' last inputs sit in a slot
        self.state_numel += self.conv_channels * (self.taps - 1)
        # rows [Wq; Wk; Wv] and, where the gate is projected directly, [Wg] behind them
        self.w_in = runtime.empty(self.conv_channels + (0 if self.gate_rank else self.v_size), hidden)
        self.conv = runtime.empty(self.conv_channels, self.taps, dtype=torch.float32)
        # the numbers that enter the recurrence in fp32: rows [Wb] and, where the decay is projected directly, [Wa]
        self.w_small = runtime.empty(n_heads * (1 if self.channel_decay else 2), hidden)
        self.w_a1 = runtime.empty(self.decay_rank, hidden) if self.channel_decay else None
        self.w_a2 = runtime.empty(n_heads * key_dim, self.decay_rank) if self.channel_decay else None
        self.w_g1 = runtime.empty(self.gate_rank, hidden) if self.gate_rank else None
        self.w_g2 = runtime.empty(self.v_size, self.gate_rank) if self.gate_rank else None
        self.rate_log = runtime.empty(n_heads, dtype=torch.float32)
        self.dt_bias = runtime.empty(n_heads * key_dim if self.channel_decay else n_heads, dtype=torch.float32)
        self.norm = runtime.empty(value_dim, dtype=torch.float32)
        self.norm_per_head = runtime.empty(self.v_size, dtype=torch.float32)
        self.w_o = runtime.empty(hidden, self.v_size)

    def weights(self) -> list[WeightDecl]:
        a, b, H, hid = self.qk_size, self.v_size, self.n_heads, self.hidden
        spans = (("q", 0, a), ("k", a, 2 * a), ("v", 2 * a, 2 * a + b))
        decls = [WeightDecl(n, (e - s, hid), dest=self.w_in[s:e]) for n, s, e in spans]
        decls += [WeightDecl(f"{n}.conv", (e - s, self.taps), role="vector", init="wide_normal", dest=self.conv[s:e]) for n, s, e in spans]
        decls += [WeightDecl("b", (H, hid), dest=self.w_small[:H]),
                  WeightDecl("A_log", (H,), role="vector", dest=self.rate_log),
                  WeightDecl("dt_bias", (self.dt_bias.numel(),), role="vector", dest=self.dt_bias),
                  WeightDecl("norm", (self.value_dim,), role="vector", init="one_plus_normal", dest=self.norm),
                  WeightDecl("o", (hid, b), dest=self.w_o)]
        if self.channel_decay:
            decls += [WeightDecl("a1", (self.decay_rank, hid), dest=self.w_a1),
                      WeightDecl("a2", (H * self.key_dim, self.decay_rank), dest=self.w_a2)]
        else:
            decls.append(WeightDecl("a", (H, hid), dest=self.w_small[H:]))
        if self.gate_rank:
            decls += [WeightDecl("g1", (self.gate_rank, hid), dest=self.w_g1), WeightDecl("g2", (b, self.gate_rank), dest=self.w_g2)]
        else:
            decls.append(WeightDecl("g", (b, hid), dest=self.w_in[2 * a + b:]))
        return decls

    def finalize(self) -> None:
        self.norm_per_head.view(self.n_heads, self.value_dim).copy_(self.norm.expand(self.n_heads, self.value_dim))

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        cache = self._check(cache)
        n, ws, H = ctx.n_tokens, ctx.workspace, self.n_heads
        a, b, C = self.qk_size, self.v_size, self.conv_channels
        proj = linear(ctx, "delta.in", h, self.w_in)
        small = linear(ctx, "delta.small", h, self.w_small, out_dtype=torch.float32)
        if self.channel_decay:
            decay = linear(ctx, "delta.a2", linear(ctx, "delta.a1", h, self.w_a1), self.w_a2, out_dtype=torch.float32)
        else:
            decay = small[:, H:]
        if self.gate_rank:
            gate = linear(ctx, "delta.g2", linear(ctx, "delta.g1", h, self.w_g1), self.w_g2)
        else:
            gate = proj[:, C:]
        # convolution, activation and unit length in one pass over the row; q's heads come first and carry the scale
        ready = ws.get("delta.ready", (n, C), torch.float32)
        ops.short_conv(ready, proj, self.conv, cache.state, self.conv_offset, ctx.seq_of_token, ctx.seq_slot, ctx.seq_q_start, n,
                       unit_heads=2 * self.n_qk_heads, unit_dim=self.key_dim, scaled_heads=self.n_qk_heads,
                       head_scale=self.key_dim ** -0.5, unit_eps=self.UNIT_EPS,
                       move_single=ctx.seq_q_len if write_cache else None)
        if write_cache and self.taps > 1 and not ctx.decode_only:
            # (a request that brings one row had its state moved on by the convolution itself)
            ops.short_conv_state(proj, self.taps, C, cache.state, self.conv_offset, ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len,
                                 ctx.n_seqs, skip_single=True)
        raw, _ = self._recur(ctx, ready[:, :a], ready[:, a:2 * a], ready[:, 2 * a:], cache, write_cache, pre=decay,
                             p0=self.rate_log, p1=self.dt_bias, write_pre=small, channel_decay=self.channel_decay,
                             qk_group=H // self.n_qk_heads)
        return self._finish(ctx, raw, None, self.norm_per_head, gate)


@register_part("mixer", "gla")
class GatedLinearAttention(MatrixStateMixer):
    """Linear attention whose state forgets through one gate per key channel that the token sets.

        q, k, v, g = split(h W^T);  q <- q * key_dim^-1/2              rows [Wq; Wk; Wv; Wg]
        z = Wa2 (Wa1 h) + b                                            per head and key channel, fp32 (inner size ``decay_rank``)
        a = sigmoid(z)^(1 / tau)                                       evaluated as exp(logsigmoid(z) / tau), fp32
        S_t = diag(a_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t         fp32, S zero before the first token
        delta = (rms_head(o) * norm * silu(g)) Wo^T                    norm [value_dim] serves every head

    ``names``: q, k, v, gate, out, norm, a1, a2, a2_bias.
    """

    rule = ops.RECURRENCE_GLA
    gate_act = ops.GATE_SILU
    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"}

    def __init__(self, runtime: Runtime, hidden: int, n_heads: int, key_dim: int, value_dim: int, decay_rank: int, tau: float,
                 eps: float, names: dict[str, str] | None = None):
        super().__init__(runtime)
        self._sizes(hidden, n_heads, key_dim, value_dim, eps)
        if decay_rank <= 0 or not tau > 0:
            raise ValueError("gla: decay_rank and tau must be positive")
        self.decay_rank, self.tau = int(decay_rank), float(tau)
        self.names = {**self.NAMES, **(names or {})}
        self.w_in = runtime.empty(2 * self.qk_size + 2 * self.v_size, hidden)          # rows [Wq; Wk; Wv; Wg]
        self.w_a1 = runtime.empty(self.decay_rank, hidden)
        self.w_a2 = runtime.empty(self.qk_size, self.decay_rank)
        self.b_a2 = runtime.empty(self.qk_size, dtype=torch.float32)
        self.norm = runtime.empty(value_dim, dtype=torch.float32)
        self.norm_per_head = runtime.empty(self.v_size, dtype=torch.float32)
        self.w_o = runtime.empty(hidden, self.v_size)

    def weights(self) -> list[WeightDecl]:
        a, b, nm, hid = self.qk_size, self.v_size, self.names, self.hidden
        return [WeightDecl(nm["q"], (a, hid), dest=self.w_in[:a]),
                WeightDecl(nm["k"], (a, hid), dest=self.w_in[a:2 * a]),
                WeightDecl(nm["v"], (b, hid), dest=self.w_in[2 * a:2 * a + b]),
                WeightDecl(nm["gate"], (b, hid), dest=self.w_in[2 * a + b:]),
                WeightDecl(nm["a1"], (self.decay_rank, hid), dest=self.w_a1),
                WeightDecl(nm["a2"], (a, self.decay_rank), dest=self.w_a2),
                WeightDecl(nm["a2_bias"], (a,), role="vector", init="wide_normal", dest=self.b_a2),
                WeightDecl(nm["norm"], (self.value_dim,), role="vector", init="one_plus_normal", dest=self.norm),
                WeightDecl(nm["out"], (hid, b), dest=self.w_o)]

    def finalize(self) -> None:
        self.norm_per_head.view(self.n_heads, self.value_dim).copy_(self.norm.expand(self.n_heads, self.value_dim))

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        cache = self._check(cache)
        a, b = self.qk_size, self.v_size
        proj = linear(ctx, "gla.in", h, self.w_in)
        decay = linear(ctx, "gla.a2", linear(ctx, "gla.a1", h, self.w_a1), self.w_a2, out_dtype=torch.float32)
        raw, _ = self._recur(ctx, proj[:, :a], proj[:, a:2 * a], proj[:, 2 * a:2 * a + b], cache, write_cache,
                             pre=decay, p0=self.b_a2, q_scale=self.key_dim ** -0.5, cap=1.0 / self.tau)
        return self._finish(ctx, raw, None, self.norm_per_head, proj[:, 2 * a + b:])
