"""The Nufatar decoder in the engine against the plain implementation (tests/plain_nufatar.py): every mechanism
alone, then whole models under every way of cutting and batching the work, in float32 and bfloat16.  The tiny
models and their weights are made here."""
import math

import numpy as np
import pytest
import torch

import plain_nufatar as plain
from helpers import (max_live_tokens, random_tokens, replay_in_process, schedule_mixed, schedule_portions, schedule_tail,
                     schedule_whole)
from test_gpu_linurax import close, ctx_of, fill
from test_gpu_sapatar import named, row_error, run_state_mixer, step_ctx
from tiny_nufatar import (NUFATAR_CONFIGS, NUFATAR_E, NUFATAR_PAGE, NUFATAR_SEEDS, NUFATAR_STD, delta, dense, parallel,
                          parallel_2, rotated, windowed, yarn)

import tessweave_engine_b200 as tw
from tessweave_engine_b200.config.nufatar_config import NufatarConfig
from tessweave_engine_b200.csrc import ops
from tessweave_engine_b200.models.nufatar import attention_spec, delta_rule_spec, mixer_spec
from tessweave_engine_b200.parts import PartSpec, Runtime, SeveralViews, build_part, dense_delta

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def typed_layer(width, layer, eps=1e-5):
    """The typed configuration of a model of one layer, and that layer."""
    typed = NufatarConfig.from_dict({"vocab": 8, "width": width, "norm": {"eps": eps}, "layers": [layer]})
    return typed, typed.layers[0]


def filled(mixer, seed, std):
    w = fill(mixer, seed, std)
    mixer.finalize()
    return w


def set_weight(mixer, w, name, value):
    """Replace one tensor of a filled part, in the part and in the dict of plain weights."""
    value = value.to(torch.bfloat16).float()
    decl = next(d for d in mixer.weights() if d.name == name)
    decl.dest.copy_(value.view(decl.dest.shape))
    w[name] = value
    mixer.finalize()


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,dims,base,scaling", [
    (16, 8, 1e3, yarn(4.0, 64, 8.0, 2.0)), (24, 24, 5e4, yarn(16.0, 32, 16.0, 1.0)), (64, 16, 1e6, yarn(8.0, 1024, 32.0, 1.0)),
    (32, 32, 1e4, None), (40, 4, 50.0, yarn(1.0, 8, 2.0, 1.0)), (64, 64, 3e5, yarn(2.5, 16, 4.0, 0.5)), (20, 0, 10.0, None)])
def test_rotation_with_stretched_frequencies(dtype, head_dim, dims, base, scaling):
    """Value i of a head turns with value i + dims / 2 at a rate that the stretching slows for the pairs that turn
    rarely, and the turned pairs grow by 0.1 ln(factor) + 1; the rest of a head and what lies behind the heads stay."""
    rt = Runtime(torch.device("cuda"), dtype)
    rope = build_part("position", PartSpec("rope", {"theta": base, "dims": dims, "yarn": scaling}), rt)
    positions = [0, 1, 2, 700, 3, 15, 16, 4095]
    ctx = ctx_of(rt, positions, [0, 0, 0, 1, 2, 2, 2, 3], [0, 1, 2, 3], [0, 3, 4, 7], [3, 1, 3, 1], [3, 701, 17, 4096])
    heads, extra = 5, 2
    x = torch.randn(len(positions), (heads + extra) * head_dim, generator=torch.Generator().manual_seed(4)).to(dtype)
    qk = x.cuda().clone()
    rope.apply(ctx, qk, heads, head_dim)
    ref = x.float().reshape(len(positions), heads + extra, head_dim)
    rates, magnitude = plain.stretched_frequencies(dims, base, scaling) if dims else ([], 1.0)
    want = plain.rotate_front(ref[:, :heads].double(), torch.tensor(positions), dims, rates, magnitude).float()
    got = qk.float().cpu().reshape(len(positions), heads + extra, head_dim)
    close(got[:, :heads], want, dtype, "rotation", f32=2e-4)      # fp32 angles of positions in the thousands
    assert torch.equal(got[:, heads:], ref[:, heads:])
    assert torch.equal(got[:, :heads, dims:], ref[:, :heads, dims:])
    if scaling is not None and scaling["factor"] > 1 and dims:
        assert magnitude > 1 and rates[-1] < base ** (-2.0 * (dims // 2 - 1) / dims)      # the slowest pair was slowed


def run_attention(rt, mixer, page, rows_of, plan, pages=None, poison=False):
    """Portions and single tokens of requests side by side through a cache manager; ``rows_of`` maps a request's name
    to its rows, ``plan`` is a list of {name: tokens of this step}.  Returns the outputs by request."""
    dtype = rt.dtype
    total = sum(len(r) for r in rows_of.values())
    cache = tw.CacheManager([(mixer.cache_need(), None)], page, pages or (total // page + 2 * len(rows_of) + 2), len(rows_of),
                            total + page * len(rows_of), dtype, rt.device, prefix_cache=False, poison_freed=poison)
    leases = {name: cache.admit(None) for name in rows_of}
    at = {lease.slot: 0 for lease in leases.values()}
    got = {name: [] for name in rows_of}
    for step in plan:
        live = [(name, n) for name, n in step.items() if n]
        for name, n in live:
            cache.ensure(leases[name], at[leases[name].slot] + n)
        cache.sync_tables()
        ctx = step_ctx(rt, [(leases[name].slot, n) for name, n in live], at)
        rows = torch.cat([rows_of[name][at[leases[name].slot]:at[leases[name].slot] + n] for name, n in live]).cuda()
        out = dense_delta(ctx, mixer.forward(ctx, rows, cache.view(0), True), dtype).float().cpu().clone()
        assert int(ctx.status) == 0
        start = 0
        for name, n in live:
            got[name].append(out[start:start + n])
            start += n
            at[leases[name].slot] += n
            cache.advance(leases[name], None, at[leases[name].slot])
    return {name: torch.cat(parts) for name, parts in got.items()}


SINK_SHAPES = [  # hidden, heads, kv heads, head size, window, rows of the table, far, page
    (48, 4, 2, 16, 9, 8, 30, 8), (40, 3, 1, 12, 5, 6, 11, 4), (36, 5, 5, 7, 3, 2, 3, 2), (64, 6, 3, 64, 40, 16, 120, 16),
    (64, 2, 2, 32, 150, 24, 60, 16), (32, 1, 1, 8, 2, 5, 1000, 4), (128, 8, 2, 64, 70, 32, 64, 16)]


def sink_mixer(rt, shape, scale=None):
    hidden, heads, kv, d, window, rows, far, _ = shape
    m = windowed(heads, kv, d, scale or 1.5 / d ** 0.5, window, rows, far)
    typed, layer = typed_layer(hidden, parallel(m, delta(1, 1, 8, 8, 2, 2, 2)))
    return build_part("mixer", attention_spec(typed, layer.mixer.left, "left"), rt), m


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SINK_SHAPES)
def test_window_attention_with_sink_and_distance_bias_alone(dtype, shape):
    """Values that are the keys, a table of biases by bucketed distance, a sink in the denominator, a sliding window;
    two requests side by side in portions and single tokens, windows shorter and longer than a page and than the
    table's reach, pages that the window gives back on the way."""
    hidden, page = shape[0], shape[7]
    rt = Runtime(torch.device("cuda"), dtype)
    mixer, m = sink_mixer(rt, shape)
    w = filled(mixer, 6, 1.2 / hidden ** 0.5)
    set_weight(mixer, w, "rel", torch.randn(w["rel"].shape, generator=torch.Generator().manual_seed(2)) * 1.5)
    set_weight(mixer, w, "sink", torch.linspace(-1.0, 2.5, shape[1]))
    assert "v" not in w and mixer.cache_need().values_are_keys
    wd = {k: v.double() for k, v in named(w).items()}
    g = torch.Generator().manual_seed(7)
    rows_of = {"a": torch.randn(190, hidden, generator=g).to(dtype), "b": torch.randn(60, hidden, generator=g).to(dtype)}
    plan = [{"a": na, "b": nb} for na, nb in [(0, 19), (13, 1), (150, 0), (1, 1), (1, 38), (2, 1), (1, 0), (22, 0)]]
    got = run_attention(rt, mixer, page, rows_of, plan, poison=True)
    for name, rows in rows_of.items():
        want = plain.mixer_attention(rows.double(), wd, "p", m, torch.arange(len(rows))).float()
        close(got[name], want, dtype, f"request {name}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_its_share_and_nothing_else(dtype):
    """A sink far above every score leaves almost nothing of the values; one far below changes nothing; in between
    the output is the sink-free output times sum / (sum + e^sink).  Neither the scale nor the bias touches it."""
    rt = Runtime(torch.device("cuda"), dtype)
    shape = (32, 2, 1, 16, 6, 4, 9, 4)
    mixer, m = sink_mixer(rt, shape, scale=0.01)          # scores near zero: the softmax without the sink is nearly uniform
    w = filled(mixer, 3, 0.1)
    set_weight(mixer, w, "rel", torch.zeros_like(w["rel"]))
    h = torch.randn(20, 32, generator=torch.Generator().manual_seed(5)).to(dtype)
    outs = {}
    for name, sink in (("low", -30.0), ("even", math.log(6.0)), ("high", 12.0)):
        set_weight(mixer, w, "sink", torch.tensor([sink, sink]))
        wd = {k: v.double() for k, v in named(w).items()}
        outs[name] = run_attention(rt, mixer, 4, {"a": h}, [{"a": 11}, {"a": 1}, {"a": 8}])["a"]
        close(outs[name], plain.mixer_attention(h.double(), wd, "p", m, torch.arange(20)).float(), dtype, name)
    full = outs["low"][8:]                                 # rows with a full window of six keys
    assert float((outs["even"][8:] - 0.5 * full).abs().max()) <= 0.03 * float(full.abs().max())
    assert float(outs["high"].abs().max()) <= 1e-3 * float(full.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(48, 2, 1, 16, 21, 8, 12, 8), (64, 2, 2, 32, 33, 16, 200, 16), (40, 1, 1, 24, 6, 4, 5, 4)])
def test_one_key_at_the_window_edge(dtype, shape):
    """One key answers the last token's query far above all others and carries a mark that no other key has (the
    values are the keys).  The key sits just inside the window, just outside, at page borders and at the first
    tokens; the asking token comes in a portion and alone.  An edge that is one token off changes the output by its
    whole size."""
    hidden, heads, kv, d, window, rows, far, page = shape
    rt = Runtime(torch.device("cuda"), dtype)
    mixer, m = sink_mixer(rt, shape, scale=6.4)
    w = filled(mixer, 8, 0.02)
    set_weight(mixer, w, "rel", torch.zeros_like(w["rel"]))
    set_weight(mixer, w, "sink", torch.full((heads,), -2.0))
    # queries read channel 0 alone, keys put it into their first value and channel 1 into their second: a marked row
    # (+1 in channel 0) meets a marked row with a score of +6.4 and an unmarked row (-1) with -6.4; only the marked
    # key carries something in its second value
    wq, wk = torch.zeros_like(w["q"]), torch.zeros_like(w["k"])
    wq.view(heads, d, hidden)[:, 0, 0] = 1.0
    wk.view(kv, d, hidden)[:, 0, 0] = 1.0
    wk.view(kv, d, hidden)[:, 1, 1] = 1.0
    set_weight(mixer, w, "q", wq)
    set_weight(mixer, w, "k", wk)
    wo = torch.zeros_like(w["o"])
    wo[0].view(heads, d)[:, 1] = 1.0                       # output channel 0 sums the heads' second values
    set_weight(mixer, w, "o", wo)
    wd = {k: v.double() for k, v in named(w).items()}
    g = torch.Generator().manual_seed(1)
    length = 4 * window + 7
    t = length - 1
    for j in [t - window + 1, t - window, t - window + 2, t - 1, 0, 1, page - 1, page, (t - window + 1) // page * page]:
        h = 0.1 * torch.randn(length, hidden, generator=g)
        h[:, 0] = -1.0
        h[:, 1] = 0.0
        h[j, 0], h[j, 1] = 1.0, 5.0
        h[t, 0] = 1.0
        h = h.to(dtype)
        want = plain.mixer_attention(h.double(), wd, "p", m, torch.arange(length)).float()
        for tail in (0, 1, 9):                           # the asking token inside a portion, alone, after single tokens
            plan = [{"a": length}] if tail == 0 else [{"a": length - tail}] + [{"a": 1}] * tail
            got = run_attention(rt, mixer, page, {"a": h}, plan, pages=-(-length // page) + 1, poison=True)["a"]
            close(got[-1:], want[-1:], dtype, f"key at {j} (edge at {t - window + 1}), last {tail} tokens alone", bf16=0.1)
        seen = 0 <= t - j < window
        assert (float(want[-1, 0].abs()) > 0.5 * heads) == seen, "the crafted key does not show in the plain output"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,far,window", [(8, 30, 64), (16, 120, 200), (6, 11, 9), (2, 3, 7), (10, 16, 40)])
def test_each_distance_reads_its_own_row_of_the_table(dtype, rows, far, window):
    """All keys alike, scores of zero, a table with one row far above the others: the softmax then sits on the
    distances of that row's bucket alone, and the keys carry their position, so the output names the distances that
    were read.  Every row of the table takes its turn; the rows that widen, the last row that everything from ``far``
    on shares, and distances beyond the table inside a longer window are all told apart."""
    hidden, heads, d, page = 16, 2, 8, 8
    rt = Runtime(torch.device("cuda"), dtype)
    mixer, m = sink_mixer(rt, (hidden, heads, 1, d, window, rows, far, page), scale=1.0)
    w = filled(mixer, 2, 0.02)
    set_weight(mixer, w, "q", torch.zeros_like(w["q"]))
    wk = torch.zeros_like(w["k"])
    wk[0, 0] = 1.0                                        # a key's first value is the row's channel 0
    set_weight(mixer, w, "k", wk)
    set_weight(mixer, w, "sink", torch.full((heads,), -20.0))
    length = min(window, int(far) * 2) + 12
    h = torch.zeros(length, hidden)
    h[:, 0] = torch.arange(length) / 8.0                  # exact in bfloat16 up to 256 tokens
    h = h.to(dtype)
    for loud in range(rows):
        table = torch.zeros(rows, heads)
        table[loud, 0] = 30.0
        table[(loud + 1) % rows, 1] = 30.0
        set_weight(mixer, w, "rel", table)
        wd = {k: v.double() for k, v in named(w).items()}
        want = plain.mixer_attention(h.double(), wd, "p", m, torch.arange(length)).float()
        got = run_attention(rt, mixer, page, {"a": h}, [{"a": length - 5}] + [{"a": 1}] * 5, poison=True)["a"]
        close(got, want, dtype, f"row {loud} of the table", f32=1e-4)


ROTATED_SHAPES = [  # hidden, heads, kv heads, key size, value size, rotated dims, base, stretching, page
    (48, 4, 2, 16, 32, 8, 1000.0, yarn(4.0, 64, 8.0, 2.0), 8), (40, 5, 5, 12, 20, 0, 10.0, None, 4),
    (64, 4, 1, 64, 128, 16, 1e6, yarn(8.0, 1024, 32.0, 1.0), 16), (128, 8, 2, 64, 64, 64, 3e5, None, 16),
    (64, 4, 4, 32, 32, 16, 2e4, yarn(16.0, 32, 16.0, 1.0), 16), (36, 3, 1, 24, 24, 12, 123.0, yarn(2.5, 16, 4.0, 0.5), 2),
    (40, 1, 1, 40, 8, 4, 50.0, yarn(1.0, 8, 2.0, 1.0), 8)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ROTATED_SHAPES)
def test_causal_attention_with_rotated_share_alone(dtype, shape):
    """Keys and values of their own sizes, part of a head rotated at stretched rates, a scale from the configuration,
    every earlier token visible; two requests in portions and single tokens."""
    hidden, heads, kv, dk, dv, dims, base, scaling, page = shape
    rt = Runtime(torch.device("cuda"), dtype)
    m = rotated(heads, kv, dk, dv, 1.5 / dk ** 0.5, dims, base, scaling)
    typed, layer = typed_layer(hidden, parallel_2(m, delta(1, 1, 8, 8, 2), 1.0, 1.0))
    mixer = build_part("mixer", attention_spec(typed, layer.mixer.left, "left"), rt)
    w = {k: v.double() for k, v in named(filled(mixer, 6, 1.2 / hidden ** 0.5)).items()}
    g = torch.Generator().manual_seed(7)
    rows_of = {"a": torch.randn(190, hidden, generator=g).to(dtype), "b": torch.randn(60, hidden, generator=g).to(dtype)}
    plan = [{"a": na, "b": nb} for na, nb in [(0, 19), (13, 1), (150, 0), (1, 1), (1, 38), (2, 1), (1, 0), (22, 0)]]
    got = run_attention(rt, mixer, page, rows_of, plan)
    for name, rows in rows_of.items():
        want = plain.mixer_attention(rows.double(), w, "p", m, torch.arange(len(rows))).float()
        close(got[name], want, dtype, f"request {name}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_hundreds_of_tokens_back_still_answers(dtype):
    """Causal attention without a window: one marked key at the start, in the middle or at a page border outweighs
    hundreds of others, from a portion and from a single token."""
    hidden, heads, kv, dk, dv, page = 32, 2, 1, 16, 8, 16
    rt = Runtime(torch.device("cuda"), dtype)
    m = rotated(heads, kv, dk, dv, 6.4, 0, 10.0)
    typed, layer = typed_layer(hidden, parallel_2(m, delta(1, 1, 8, 8, 2), 1.0, 1.0))
    mixer = build_part("mixer", attention_spec(typed, layer.mixer.left, "left"), rt)
    w = filled(mixer, 8, 0.02)
    wq, wk, wv = torch.zeros_like(w["q"]), torch.zeros_like(w["k"]), torch.zeros_like(w["v"])
    wq.view(heads, dk, hidden)[:, 0, 0] = 1.0
    wk.view(kv, dk, hidden)[:, 0, 0] = 1.0
    wv[:, 1] = 2.0
    for name, value in (("q", wq), ("k", wk), ("v", wv)):
        set_weight(mixer, w, name, value)
    wd = {k: v.double() for k, v in named(w).items()}
    length = 700
    g = torch.Generator().manual_seed(1)
    for j in (0, 1, 15, 16, 350, 698):
        h = 0.1 * torch.randn(length, hidden, generator=g)
        h[:, 0], h[:, 1] = -1.0, 0.0
        h[j, 0], h[j, 1] = 1.0, 5.0
        h[-1, 0] = 1.0
        h = h.to(dtype)
        want = plain.mixer_attention(h.double(), wd, "p", m, torch.arange(length)).float()
        assert float(want[-1].abs().max()) > 0.1
        for plan in ([{"a": length}], [{"a": length - 3}] + [{"a": 1}] * 3):
            got = run_attention(rt, mixer, page, {"a": h}, plan)["a"]
            close(got[-1:], want[-1:], dtype, f"key at {j}", bf16=0.1)


DELTA_SHAPES = [  # hidden, kind, heads, q/k heads, key size, value size, taps, decay rank, gate rank
    (48, "parallel_2", 4, 2, 16, 24, 4, None, None), (40, "parallel", 3, 3, 5, 7, 1, 4, 2), (36, "parallel", 2, 1, 16, 8, 3, 6, 5),
    (64, "parallel_2", 1, 1, 24, 40, 3, None, None), (64, "parallel_2", 5, 1, 8, 8, 7, None, None), (96, "parallel", 4, 1, 32, 16, 4, 16, 8),
    (64, "parallel_2", 6, 6, 64, 64, 4, None, None), (64, "parallel", 2, 2, 32, 32, 4, 24, 24), (32, "parallel_2", 2, 2, 10, 6, 5, None, None)]


def delta_mixer(rt, hidden, kind, heads, qk_heads, dk, dv, taps, decay_rank, gate_rank, eps=1e-5):
    m = delta(heads, qk_heads, dk, dv, taps, decay_rank, gate_rank)
    layer = (parallel(windowed(1, 1, 8, 0.3, 4, 4, 9), m) if kind == "parallel"
             else parallel_2(rotated(1, 1, 8, 8, 0.3, 0, 10.0), m, 1.0, 1.0))
    typed, layer = typed_layer(hidden, layer, eps)
    return build_part("mixer", delta_rule_spec(typed, layer.mixer.right, "right"), rt), m


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", DELTA_SHAPES)
def test_gated_delta_rule_alone(dtype, shape):
    """Both kinds (a decay per head and a silu gate; a decay per key channel and a sigmoid gate, both through two
    matrices), grouped heads, convolutions of one to seven taps whose last inputs cross the cuts, two requests in
    slots 2 and 0 cut into steps of 1 to 150 rows (steps shorter than the convolution among them)."""
    hidden = shape[0]
    rt = Runtime(torch.device("cuda"), dtype)
    mixer, m = delta_mixer(rt, *shape)
    w = filled(mixer, 11, 0.4)
    set_weight(mixer, w, "A_log", torch.linspace(-3.0, 0.5, shape[2]))
    set_weight(mixer, w, "dt_bias", torch.randn(w["dt_bias"].shape, generator=torch.Generator().manual_seed(3)))
    wd = {k: v.double() for k, v in named(w).items()}
    assert ("a1" in w) == (shape[1] == "parallel") and ("g" in w) == (shape[1] == "parallel_2")
    run_state_mixer(rt, mixer, hidden, lambda h, pos: plain.mixer_delta(h, wd, "p", m, 1e-5))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["parallel", "parallel_2"])
@pytest.mark.parametrize("loud_row", [0, 3, 149])
def test_one_token_far_back_outweighs_the_rest_in_the_state(dtype, kind, loud_row):
    """Decays close to 1 and one loud token: hundreds of tokens later the outputs still depend on what that token
    left in the state, through cuts into steps of 1 to 150 tokens.  A state that is lost, zeroed or taken from
    another slot on the way shows at once."""
    rt = Runtime(torch.device("cuda"), dtype)
    hidden = 48
    mixer, m = delta_mixer(rt, hidden, kind, 2, 1, 16, 16, 4, 8 if kind == "parallel" else None, 8 if kind == "parallel" else None, eps=1e-2)
    w = filled(mixer, 21, 0.3)
    set_weight(mixer, w, "A_log", torch.full((2,), -7.0))          # decays of exp(-e^-7 softplus(.)): about 0.999 per token
    set_weight(mixer, w, "b", w["b"] * 0.1 - 0.0)                  # beta near one half: a write is never wiped at once
    wd = {k: v.double() for k, v in named(w).items()}
    fn = lambda h, pos: plain.mixer_delta(h, wd, "p", m, 1e-2)     # noqa: E731
    g = torch.Generator().manual_seed(3)
    h = torch.randn(223, hidden, generator=g)
    with_loud = h.clone()
    with_loud[loud_row] *= 12.0
    moved = (fn(with_loud.double(), None) - fn(h.double(), None))[200:].abs().max() / fn(h.double(), None)[200:].abs().max()
    assert float(moved) > 0.02, f"the loud row no longer shows at the end ({float(moved):.3g})"
    run_state_mixer(rt, mixer, hidden, fn, loud_row=loud_row)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["parallel", "parallel_2"])
def test_the_two_mixers_side_by_side(dtype, kind):
    """Attention and delta rule on the same rows, each with its own cache or state.  One kind normalises each result
    over the width with a weight of its own and takes half the sum; the other adds them with two scales (one of them
    negative here)."""
    rt = Runtime(torch.device("cuda"), dtype)
    hidden = 48
    if kind == "parallel":
        layer = parallel(windowed(4, 2, 16, 0.3, 9, 8, 30), delta(2, 1, 16, 8, 3, 6, 5))
    else:
        layer = parallel_2(rotated(4, 2, 16, 32, 0.3, 8, 1000.0, yarn(4.0, 64, 8.0, 2.0)), delta(4, 2, 16, 24, 4), 0.7, -1.4)
    typed, typed_l = typed_layer(hidden, layer, eps=1e-3)
    mixer = build_part("mixer", mixer_spec(typed, typed_l, "layer"), rt)
    w = {k: v.double() for k, v in named(filled(mixer, 5, 0.3)).items()}
    assert ("p.left.out" in w and "p.right.out" in w) == (kind == "parallel")
    cache = tw.CacheManager([(mixer.cache_need(), None)], 8, 16, 2, 96, dtype, rt.device, prefix_cache=False)
    assert isinstance(cache.view(0), SeveralViews)
    lease = cache.admit(None)
    h = torch.randn(50, hidden, generator=torch.Generator().manual_seed(9)).to(dtype)
    want = plain.mixer(kind, h.double(), w, "p", layer["mixer"], 1e-3, torch.arange(50)).float()
    at, outs = {lease.slot: 0}, []
    for n in (20, 1, 1, 28):
        cache.ensure(lease, at[lease.slot] + n)
        cache.sync_tables()
        ctx = step_ctx(rt, [(lease.slot, n)], at)
        outs.append(dense_delta(ctx, mixer.forward(ctx, h[at[lease.slot]:at[lease.slot] + n].cuda(), cache.view(0), True), dtype).float().cpu().clone())
        at[lease.slot] += n
        cache.advance(lease, None, at[lease.slot])
    close(torch.cat(outs), want, dtype, "left and right")


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------
BF16_EPS = 0.05


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """(name, dtype) -> model folder.  The bfloat16 runs get a copy whose norms have a large eps: after a request's
    first token a head's state has rank one, its output is a multiple of one vector, and the norm over the head makes
    of that a sign times a unit vector unless eps is felt; with a tiny eps a rounding that turns the sign of a nearly
    orthogonal query and key moves the row, and the rows behind it, by tens of per cent.  (The float32 runs, which no
    rounding turns, keep the tiny eps.)"""
    tmp = tmp_path_factory.mktemp("nufatar")
    out = {}
    for name, cfg in NUFATAR_CONFIGS.items():
        out[name, "float32"] = tw.write_random_model(tmp / name, cfg, seed=NUFATAR_SEEDS[name], std=NUFATAR_STD[name])
        out[name, "bfloat16"] = tw.write_random_model(tmp / f"{name}_eps", {**cfg, "norm": {"eps": BF16_EPS}},
                                                      seed=NUFATAR_SEEDS[name], std=NUFATAR_STD[name])
    return out


LENGTHS = [70, 1, 45, 100, 2, 33, 64, 129]


def requests_for(name):
    return {f"r{i}": random_tokens(NUFATAR_CONFIGS[name]["vocab"], n, 20 + i) for i, n in enumerate(LENGTHS)}


@pytest.fixture(scope="module")
def plain_rows(folders):
    return {key: {rid: plain.logits_of(folder, t).numpy() for rid, t in requests_for(key[0]).items()}
            for key, folder in folders.items()}


def float32_noise_of(folder, reqs, want):
    """What 32-bit arithmetic alone does to each row: the plain implementation in float32 against itself in float64."""
    return {rid: [row_error(r, w) for r, w in zip(plain.logits_of(folder, t, torch.float32).numpy(), want[rid])]
            for rid, t in reqs.items()}


def bfloat16_noise_of(folder, reqs, want, seed=99):
    """What perturbations of bfloat16's size do to each row by themselves: the plain implementation (float64) with
    every matrix element moved by a relative 2^-8 times a normal draw, against itself."""
    config, weights = plain.read_folder(folder, torch.float64)
    g = torch.Generator().manual_seed(seed)
    moved = {k: v * (1 + 2.0 ** -8 * torch.randn(v.shape, generator=g, dtype=torch.float64)) if v.dim() == 2 else v
             for k, v in weights.items()}
    return {rid: [row_error(r, w) for r, w in zip(plain.forward(config, moved, t).float().numpy(), want[rid])]
            for rid, t in reqs.items()}


@pytest.fixture(scope="module")
def noise(folders, plain_rows):
    out = {}
    for (name, dtype), folder in folders.items():
        make = float32_noise_of if dtype == "float32" else bfloat16_noise_of
        out[name, dtype] = make(folder, requests_for(name), plain_rows[name, dtype])
    return out


def compare(rows, want, dtype, what, noise=None):
    """Every logits row against the plain one (float64).  float32: every row within 5e-5 of its spread plus four
    times what the plain implementation loses at that row when it runs in float32 itself.  bfloat16: the rows are
    judged together: the median within 6 %, at most five rows in a hundred beyond 8 % plus three times what a
    perturbation of bfloat16's size does to that row of the plain implementation (``noise``), none that is not
    finite.  A lost state, a key outside its window or a wrong page moves rows by their whole size."""
    errors, over = [], []
    for (rid, p), row in rows.items():
        err = row_error(row, want[rid][p])
        assert np.isfinite(row).all(), f"{what}: {rid}[{p}] is not finite"
        lost = noise[rid][p] if noise else 0.0
        if dtype == "float32":
            assert err <= 5e-5 + 4 * lost, f"{what}: {rid}[{p}] differs by {err:.3g} of the row's spread (float32 alone: {lost:.3g})"
        elif err > 8e-2 + 3 * lost:
            over.append((rid, p, round(err, 3)))
        errors.append(err)
    if dtype == "bfloat16":
        assert float(np.median(errors)) <= 6e-2, f"{what}: the median row differs by {float(np.median(errors)):.3g}"
        assert len(over) <= max(2, 5 * len(errors) // 100), f"{what}: {len(over)} of {len(errors)} rows are far off: {over[:8]}"


SCHEDULES = {
    "whole": schedule_whole,
    "tail": schedule_tail,
    "portions": schedule_portions,
    "one_by_one": lambda r: schedule_portions({k: v for k, v in r.items() if len(v) <= 70}, sizes=(1,)),
    "mixed": lambda r: schedule_mixed(r, live=4, seed=1),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_cutting_gives_the_plain_logits(name, dtype, folders, plain_rows, noise, tmp_path):
    """Whole prompts; most of a prompt and its last 32 tokens one by one; portions down to two tokens; token by
    token from the first; four live requests in mixed batches with so few pages and slots that both are used
    again (freed pages are filled with NaN first).  The models repeat a range of layers, each pass on a cache and
    state of its own."""
    reqs = requests_for(name)
    for kind, make in SCHEDULES.items():
        steps = make(reqs)
        rows = replay_in_process(folders[name, dtype], dtype, steps, tmp_path / kind, block_size=NUFATAR_PAGE[name],
                                 max_tokens=max_live_tokens(steps))
        assert rows, kind
        compare(rows, plain_rows[name, dtype], dtype, f"{name} {kind}", noise[name, dtype])


def test_batches_and_cuts_do_not_change_a_request(folders, tmp_path):
    """float32: a request's logits in a mixed batch, or cut into portions, equal those it gets alone, to rounding."""
    reqs = requests_for("A")
    folder = folders["A", "float32"]
    alone = replay_in_process(folder, "float32", schedule_whole(reqs), tmp_path / "alone", block_size=8)
    for kind, steps in (("mixed", schedule_mixed(reqs, live=4, seed=3)), ("portions", schedule_portions(reqs))):
        got = replay_in_process(folder, "float32", steps, tmp_path / kind, block_size=8)
        worst = max(float(np.abs(row - alone[key]).max() / np.abs(alone[key]).max()) for key, row in got.items())
        assert worst <= 1e-4, (kind, worst)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_windows_and_pages(dtype, folders, noise, tmp_path):
    """A short prompt and 300 tokens one by one: the window passes over decoded tokens only, its pages are given back
    and used again on the way, the states carry everything else."""
    name = "C"
    toks = random_tokens(NUFATAR_CONFIGS[name]["vocab"], 310, 77)
    steps = schedule_tail({"long": toks}, tail=300)
    rows = replay_in_process(folders[name, dtype], dtype, steps, tmp_path / "out", block_size=NUFATAR_PAGE[name], max_tokens=384)
    want = {"long": plain.logits_of(folders[name, dtype], toks).numpy()}
    make = float32_noise_of if dtype == "float32" else bfloat16_noise_of
    compare(rows, want, dtype, "long decoding", make(folders[name, dtype], {"long": toks}, want))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_hundreds_of_tokens_past_windows_and_tables(dtype, tmp_path):
    """Windows of 70 and 150 and distance tables that reach 60 and 400 tokens, prompts of 420 and 190 tokens: whole,
    with the last 40 tokens one by one, and in mixed batches, on pages of 16 that the windows give back on the way."""
    cfg = NUFATAR_E if dtype == "float32" else {**NUFATAR_E, "norm": {"eps": BF16_EPS}}
    folder = tw.write_random_model(tmp_path / "model", cfg, seed=31, std=0.1)
    reqs = {"long": random_tokens(cfg["vocab"], 420, 5), "mid": random_tokens(cfg["vocab"], 190, 6), "short": random_tokens(cfg["vocab"], 37, 7)}
    want = {rid: plain.logits_of(folder, t).numpy() for rid, t in reqs.items()}
    noise = (float32_noise_of if dtype == "float32" else bfloat16_noise_of)(folder, reqs, want)
    for kind, steps in (("whole", schedule_whole(reqs)), ("tail", schedule_tail(reqs, tail=40)),
                        ("mixed", schedule_mixed(reqs, live=3, seed=2, prefill=(33, 2, 70, 5, 128, 16)))):
        rows = replay_in_process(folder, dtype, steps, tmp_path / kind, block_size=16, max_tokens=max_live_tokens(steps))
        compare(rows, want, dtype, f"E {kind}", noise)


def test_the_pass_vectors_are_added_once_per_pass(tmp_path):
    """float32: a model whose repeated range is its middle; with the pass vectors made large, leaving one out, adding
    it at every layer of the pass or adding another pass's vector moves the logits by their whole size."""
    cfg = NUFATAR_CONFIGS["A"]
    folder = tw.write_random_model(tmp_path / "m", cfg, seed=4, std=0.12)
    from safetensors.torch import load_file, save_file
    t = load_file(str(folder / "model.safetensors"))
    g = torch.Generator().manual_seed(8)
    t["loop.step"] = (torch.randn(t["loop.step"].shape, generator=g) * 2.0).to(t["loop.step"].dtype)
    save_file(t, str(folder / "model.safetensors"), metadata={"format": "pt"})
    reqs = {"r": random_tokens(cfg["vocab"], 40, 3)}
    want = {"r": plain.logits_of(folder, reqs["r"]).numpy()}
    config, weights = plain.read_folder(folder, torch.float64)
    without = plain.forward(config, {**weights, "loop.step": torch.zeros_like(weights["loop.step"])}, reqs["r"]).float().numpy()
    assert row_error(without[-1], want["r"][-1]) > 0.3
    for kind, steps in (("whole", schedule_whole(reqs)), ("tail", schedule_tail(reqs, tail=8))):
        rows = replay_in_process(folder, "float32", steps, tmp_path / kind, block_size=8)
        compare(rows, want, "float32", f"pass vectors {kind}", float32_noise_of(folder, reqs, want))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_engine(name, dtype, folders):
    """``generate`` (scheduler, continuous batching, CUDA graphs, look-ahead) against the plain implementation;
    every chosen token must be the plain implementation's best on that path, or nearly."""
    prompts = [random_tokens(NUFATAR_CONFIGS[name]["vocab"], n, 60 + n) for n in (21, 5, 40)]
    model = tw.load_model(folders[name, dtype], dtype, "cuda")
    out = tw.generate(model, prompts, max_tokens=12, ignore_eos=True,
                      engine_config=tw.EngineConfig(block_size=NUFATAR_PAGE[name], kv_blocks=40, max_context=128, max_active=2,
                                                    prefill_chunk=16))
    config, weights = plain.read_folder(folders[name, dtype], torch.float64)
    for p, o in zip(prompts, out):
        assert len(o) == 12
        logits = plain.forward(config, weights, p + o).float()
        for i, t in enumerate(o):
            row = logits[len(p) + i - 1]
            gap = float(row.max() - row[t])
            spread = float(row.std())
            assert gap <= (1e-4 if dtype == "float32" else 0.15) * spread, f"token {i} lies {gap:.3g} below the best (spread {spread:.3g})"
