"""The Dugudra decoder in the engine against the plain implementation (tests/plain_dugudra.py): every mechanism
alone, then whole models under every way of cutting and batching the work, in float32 and bfloat16.  The tiny
models and their weights are made here."""
import numpy as np
import pytest
import torch

import plain_dugudra as plain
from helpers import (max_live_tokens, random_tokens, replay_in_process, schedule_mixed, schedule_portions, schedule_tail,
                     schedule_whole)
from test_gpu_linurax import close, ctx_of, fill
from test_gpu_nufatar import filled, run_attention, set_weight
from test_gpu_sapatar import named, row_error, run_state_mixer, step_ctx
from tiny_dugudra import (DUGUDRA_CONFIGS, DUGUDRA_E, DUGUDRA_PAGE, DUGUDRA_SEEDS, DUGUDRA_STD, attention, gla, latent, moe,
                          yarn)

import tessweave_engine_b200 as tw
from tessweave_engine_b200.config.dugudra_config import DugudraConfig
from tessweave_engine_b200.csrc import ops
from tessweave_engine_b200.csrc.ops import SplitSum
from tessweave_engine_b200.models.dugudra import experts_spec, mixer_spec
from tessweave_engine_b200.parts import PartSpec, Runtime, build_part, dense_delta

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def typed_layer(width, layer, eps=1e-5):
    """The typed configuration of a model of one layer, and that layer."""
    typed = DugudraConfig.from_dict({"vocab": 8, "width": width, "norm": {"eps": eps}, "layers": [layer]})
    return typed, typed.layers[0]


def mixer_of(rt, width, layer, eps=1e-5):
    typed, one = typed_layer(width, layer, eps)
    return build_part("mixer", mixer_spec(typed, one, "layers[0]"), rt)


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,first,dims,base,scaling", [
    (24, 16, 8, 1e3, yarn(4.0, 64, 8.0, 2.0)), (16, 0, 16, 5e4, yarn(16.0, 32, 16.0, 1.0)), (40, 6, 32, 7e4, yarn(8.0, 1024, 32.0, 1.0)),
    (12, 10, 2, 10.0, None), (64, 48, 16, 3e4, yarn(4.0, 256, 32.0, 1.0)), (20, 4, 4, 50.0, yarn(1.0, 8, 2.0, 1.0))])
def test_rotation_of_neighbours_inside_a_head(dtype, head_dim, first, dims, base, scaling):
    """Values first + 2i and first + 2i + 1 of a head turn together, at rates that the stretching slows for the pairs
    that turn rarely, and grow by 0.1 ln(factor) + 1; the rest of a head and what lies behind the heads stay."""
    rt = Runtime(torch.device("cuda"), dtype)
    rope = build_part("position", PartSpec("rope_interleaved", {"theta": base, "dims": dims, "yarn": scaling}), rt)
    plan = rope.rotary_plan(dims)
    positions = [0, 1, 2, 700, 3, 15, 16, 4095]
    ctx = ctx_of(rt, positions, [0, 0, 0, 1, 2, 2, 2, 3], [0, 1, 2, 3], [0, 3, 4, 7], [3, 1, 3, 1], [3, 701, 17, 4096])
    heads, extra = 5, 2
    x = torch.randn(len(positions), (heads + extra) * head_dim, generator=torch.Generator().manual_seed(4)).to(dtype)
    rows = x.cuda().clone()
    ops.rotate_pairs(rows, ctx.positions, ctx.seq_of_token, plan.inv_freq, len(positions), heads, head_dim, plan.rot_dims,
                     plan.interleaved, magnitude=plan.magnitude, first=first)
    ref = x.float().reshape(len(positions), heads + extra, head_dim)
    rates, magnitude = plain.stretched_rates(dims, base, scaling)
    want = ref.clone()
    want[:, :heads, first:first + dims] = plain.rotate_neighbours(ref[:, :heads, first:first + dims].double(), torch.tensor(positions),
                                                                  rates, magnitude).float()
    got = rows.float().cpu().reshape(len(positions), heads + extra, head_dim)
    close(got[:, :heads], want[:, :heads], dtype, "rotation", f32=2e-4)      # fp32 angles of positions in the thousands
    assert torch.equal(got[:, heads:], ref[:, heads:])
    assert torch.equal(got[:, :heads, :first], ref[:, :heads, :first]) and torch.equal(got[:, :heads, first + dims:], ref[:, :heads, first + dims:])
    assert plan.magnitude == magnitude
    if scaling is not None and scaling["factor"] > 1:
        assert magnitude > 1 and rates[-1] < base ** (-2.0 * (dims // 2 - 1) / dims)      # the slowest pair was slowed


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("spans", [[(0, 4, 16), (64, 2, 16)], [(5, 1, 37)], [(0, 1, 20), (20, 1, 40)], [(8, 3, 96), (300, 1, 96)]])
def test_norm_of_heads_side_by_side(dtype, spans):
    """Spans of heads inside wider rows, every head divided by its own root mean square and multiplied by the span's
    weight; the columns between and behind the spans stay."""
    g = torch.Generator().manual_seed(9)
    width = max(c + h * d for c, h, d in spans) + 3
    x = (torch.randn(11, width, generator=g) * 3).to(dtype)
    weights = [(1 + 0.3 * torch.randn(d, generator=g)) for _, _, d in spans]
    rows = x.cuda().clone()
    ops.span_rmsnorm(rows, 11, [(c, h, d, w.cuda()) for (c, h, d), w in zip(spans, weights)], 1e-3)
    want = x.float().clone()
    for (c, h, d), w in zip(spans, weights):
        heads = x.float()[:, c:c + h * d].reshape(11, h, d).double()
        want[:, c:c + h * d] = (plain.rms(heads, 1e-3) * w.double()).reshape(11, h * d).float()
    got = rows.float().cpu()
    close(got, want, dtype, "normalised heads")
    untouched = torch.ones(width, dtype=torch.bool)
    for c, h, d in spans:
        untouched[c:c + h * d] = False
    assert torch.equal(got[:, untouched], x.float()[:, untouched])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,rows", [(40, 5), (36, 70), (192, 300), (1024, 8), (2048, 3), (4100, 2)])
def test_residual_factor_in_the_norm_kernel(dtype, hidden, rows):
    """x <- x + m * delta with the product and the sum in 32 bits, then the norm: every form of the kernel (rows in
    registers, four values per thread, a cluster per row), with a dense delta and with slices of a split product."""
    g = torch.Generator().manual_seed(hidden + rows)
    resid = torch.randn(rows, hidden, generator=g)
    delta = torch.randn(rows, hidden, generator=g).to(dtype)
    weight = 1 + 0.1 * torch.randn(hidden, generator=g)
    m = -0.7
    want_x = resid + np.float32(m) * delta.float()
    want = (plain.rms(want_x.double(), 1e-5) * weight.double()).float()
    r = resid.cuda().clone()
    out = torch.empty(rows, hidden, dtype=dtype, device="cuda")
    ops.add_rmsnorm(out, r, delta.cuda(), weight.cuda(), 1e-5, rows, delta_scale=m)
    assert float((r.cpu() - want_x).abs().max()) <= 1e-6 * float(want_x.abs().max())
    close(out.float().cpu(), want, dtype, "norm behind the scaled sum", bf16=1e-2)
    slices = torch.randn(3, rows, hidden, generator=g)
    r = resid.cuda().clone()
    ops.add_rmsnorm(out, r, SplitSum(slices.cuda()), weight.cuda(), 1e-5, rows, delta_scale=m)
    want_x = resid + np.float32(m) * slices.sum(0)
    assert float((r.cpu() - want_x).abs().max()) <= 2e-6 * float(want_x.abs().max())
    picked = torch.tensor([rows - 1, 0], dtype=torch.int32)
    r = resid.cuda().clone()
    ops.add_rmsnorm(out, r, delta.cuda(), weight.cuda(), 1e-5, 2, rows=picked.cuda(), delta_scale=m)
    assert torch.equal(r.cpu(), resid)                  # with chosen rows the stream is left as it was
    close(out[:2].float().cpu(), want[picked.long()], dtype, "chosen rows", bf16=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_capped_logits(dtype):
    rt = Runtime(torch.device("cuda"), dtype)
    head = build_part("head", PartSpec("linear_head", {"vocab": 77, "hidden": 48, "weight_name": "", "softcap": 2.5}), rt)
    w = fill(head, 3, 0.6)
    g = torch.Generator().manual_seed(1)
    y = torch.randn(9, 48, generator=g).to(dtype)
    ctx = ctx_of(rt, list(range(9)), [0] * 9, [0], [0], [9], [9])
    logits = torch.empty(9, 77, dtype=torch.float32, device="cuda")
    head.forward(ctx, logits, y.cuda(), 9)
    raw = y.double() @ w[""].double().T
    want = (2.5 * torch.tanh(raw / 2.5)).float()
    assert float(raw.abs().max()) > 5.0                 # the cap is felt
    close(logits.cpu(), want, dtype, "capped logits")
    assert float(logits.abs().max()) <= 2.5


ATTENTION_SHAPES = [  # hidden, heads, kv heads, key size, value size, window, page
    (48, 4, 2, 16, 32, 9, 8), (40, 3, 1, 12, 20, 5, 4), (36, 5, 5, 7, 7, 3, 2), (64, 6, 3, 64, 64, 40, 16), (64, 2, 2, 32, 32, 150, 16),
    (32, 1, 1, 8, 24, 2, 4), (128, 8, 2, 64, 64, 70, 16), (96, 4, 1, 80, 80, 33, 16), (64, 2, 1, 48, 16, None, 8),
    (64, 2, 1, 320, 272, 50, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTENTION_SHAPES)
def test_attention_with_normed_heads_and_a_sink_alone(dtype, shape):
    """Every head of q and k normalised, no positions, one added to the denominator, a sliding window; two requests
    side by side in portions and single tokens, windows shorter and longer than a page, pages that the window gives
    back on the way (and are filled with NaN then)."""
    hidden, heads, kv, d, dv, window, page = shape
    rt = Runtime(torch.device("cuda"), dtype)
    layer = attention(heads, kv, d, dv, 1.5 / d ** 0.5, window)
    mixer = mixer_of(rt, hidden, layer)
    w = filled(mixer, 6, 1.2 / hidden ** 0.5)
    set_weight(mixer, w, "q.norm", 1 + 0.5 * torch.randn(d, generator=torch.Generator().manual_seed(2)))
    set_weight(mixer, w, "k.norm", 1 + 0.5 * torch.randn(d, generator=torch.Generator().manual_seed(3)))
    wd = {k: v.double() for k, v in named(w).items()}
    g = torch.Generator().manual_seed(7)
    rows_of = {"a": torch.randn(190, hidden, generator=g).to(dtype), "b": torch.randn(60, hidden, generator=g).to(dtype)}
    plan = [{"a": na, "b": nb} for na, nb in [(0, 19), (13, 1), (150, 0), (1, 1), (1, 38), (2, 1), (1, 0), (22, 0)]]
    got = run_attention(rt, mixer, page, rows_of, plan, poison=True)
    for name, rows in rows_of.items():
        want = plain.mixer_attention(rows.double(), wd, "p.", layer["mixer"], 1e-5).float()
        close(got[name], want, dtype, f"request {name}")


LATENT_SHAPES = [  # hidden, heads, plain size, rotated size, value size, q latent, kv latent, window, page, base, scaling
    (48, 3, 16, 8, 24, 20, 40, 9, 8, 1000.0, yarn(4.0, 64, 8.0, 2.0)), (40, 5, 6, 2, 7, 5, 11, 3, 4, 10.0, None),
    (64, 4, 32, 16, 32, 64, 48, 24, 16, 3e4, yarn(16.0, 32, 16.0, 1.0)), (64, 4, 32, 16, 16, 48, 64, 150, 16, 5e3, yarn(8.0, 128, 32.0, 1.0)),
    (32, 1, 8, 4, 8, 8, 12, 2, 4, 50.0, yarn(1.0, 8, 2.0, 1.0)), (96, 12, 16, 16, 8, 32, 112, 40, 16, 3e5, yarn(4.0, 256, 32.0, 1.0)),
    (64, 2, 8, 8, 8, 24, 24, None, 8, 5e4, None), (64, 2, 16, 8, 16, 24, 300, 40, 16, 1e4, yarn(4.0, 64, 8.0, 2.0))]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", LATENT_SHAPES)
def test_latent_attention_alone(dtype, shape):
    """Queries and keys/values through their latents, the shared rotated key part, stretched rates, the window and the
    output gate; the cache holds one row of kv_rank + rot_dim values per token."""
    hidden, heads, d, r, dv, qr, cr, window, page, base, scaling = shape
    rt = Runtime(torch.device("cuda"), dtype)
    layer = latent(heads, d, r, dv, qr, cr, 1.5 / (d + r) ** 0.5, base, window, scaling)
    mixer = mixer_of(rt, hidden, layer)
    need = mixer.cache_need()
    assert (need.kv_heads, need.head_dim, need.values_are_keys, need.window) == (1, cr + r, True, window)
    w = filled(mixer, 16, 1.2 / hidden ** 0.5)
    for name, fan_in in (("uq", qr), ("uk", cr), ("uv", cr)):          # the maps out of the latents keep what passes at size 1
        set_weight(mixer, w, name, torch.randn(w[name].shape, generator=torch.Generator().manual_seed(fan_in)) / fan_in ** 0.5)
    wd = {k: v.double() for k, v in named(w).items()}
    g = torch.Generator().manual_seed(8)
    rows_of = {"a": torch.randn(190, hidden, generator=g).to(dtype), "b": torch.randn(60, hidden, generator=g).to(dtype)}
    plan = [{"a": na, "b": nb} for na, nb in [(0, 19), (13, 1), (150, 0), (1, 1), (1, 38), (2, 1), (1, 0), (22, 0)]]
    got = run_attention(rt, mixer, page, rows_of, plan, poison=True)
    for name, rows in rows_of.items():
        want = plain.mixer_latent_attention(rows.double(), wd, "p.", layer["mixer"], 1e-5, torch.arange(len(rows))).float()
        close(got[name], want, dtype, f"request {name}")


def edge_case(rt, mixer, page, h, tail):
    """The last row's output when the sequence ``h`` runs as one portion (``tail`` 0) or with its last ``tail`` tokens
    one by one."""
    length = h.shape[0]
    cache = tw.CacheManager([(mixer.cache_need(), None)], page, -(-length // page) + 1, 1, length + page, rt.dtype, rt.device,
                            prefix_cache=False, poison_freed=True)
    lease = cache.admit(None)
    at = {lease.slot: 0}
    out = None
    for n in ([length] if tail == 0 else [length - tail] + [1] * tail):
        cache.ensure(lease, at[lease.slot] + n)
        cache.sync_tables()
        ctx = step_ctx(rt, [(lease.slot, n)], at)
        out = dense_delta(ctx, mixer.forward(ctx, h[at[lease.slot]:at[lease.slot] + n].cuda(), cache.view(0), True), rt.dtype).float().cpu().clone()
        assert int(ctx.status) == 0
        at[lease.slot] += n
        cache.advance(lease, None, at[lease.slot])
    return out[-1:]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind,page,window", [("attention", 8, 21), ("attention", 16, 33), ("attention", 4, 6),
                                              ("latent", 8, 21), ("latent", 16, 33), ("latent", 4, 6)])
def test_one_key_at_the_window_edge(dtype, kind, page, window):
    """One key answers the last token's query far above all others and carries a value of its own.  The key sits just
    inside the window, just outside, at page borders and at the first tokens; the asking token comes in a portion and
    alone.  An edge that is one token off, or a sink that is left out (the other keys then share the whole weight),
    changes the output by its whole size."""
    rt = Runtime(torch.device("cuda"), dtype)
    hidden = 48
    g = torch.Generator().manual_seed(1)
    if kind == "attention":
        heads, kv, d, dv = 2, 1, 16, 32
        layer = attention(heads, kv, d, dv, 6.4 / d, window)
        mixer = mixer_of(rt, hidden, layer)
        w = filled(mixer, 8, 0.02)
        # queries and keys read channel 0 alone: every normalised head is +-1 in every value, and a marked row (+1)
        # meets a marked row with a score of 6.4 and an unmarked one (-1) with -6.4; the values read channel 1
        for name in ("q", "k"):
            t = torch.zeros_like(w[name]); t[:, 0] = 1.0
            set_weight(mixer, w, name, t)
        t = torch.zeros_like(w["v"]); t[:, 1] = 2.0
        set_weight(mixer, w, "v", t)
        set_weight(mixer, w, "q.norm", torch.ones(d)); set_weight(mixer, w, "k.norm", torch.ones(d))
        run_plain = lambda h, wd: plain.mixer_attention(h, wd, "p.", layer["mixer"], 1e-5)     # noqa: E731
    else:
        heads, d, r, dv, qr, cr = 2, 16, 8, 24, 12, 24
        layer = latent(heads, d, r, dv, qr, cr, 6.4 / d, 1000.0, window, yarn(4.0, 64, 8.0, 2.0))
        mixer = mixer_of(rt, hidden, layer)
        w = filled(mixer, 8, 0.02)
        # the query latent and the first half of the key/value latent read channel 0 (+-1 in every value after their
        # norms), the second half of the key/value latent reads channel 1 (the payload, +-1 too, so that the norm leaves
        # both halves alone); the maps out of the latents average: every plain query and key value is +-1, the rotated
        # parts are silent, and a head's value is the payload times its map's row sums
        t = torch.zeros_like(w["dq"]); t[:, 0] = 1.0
        set_weight(mixer, w, "dq", t)
        t = torch.zeros_like(w["dkv"]); t[:cr // 2, 0] = 1.0; t[cr // 2:cr, 1] = 1.0
        set_weight(mixer, w, "dkv", t)
        t = torch.zeros(heads, d + r, qr); t[:, :d, :] = 1.0 / qr
        set_weight(mixer, w, "uq", t.reshape(heads * (d + r), qr))
        t = torch.zeros_like(w["uk"]); t[:, :cr // 2] = 2.0 / cr
        set_weight(mixer, w, "uk", t)
        t = torch.randn(w["uv"].shape, generator=g) * 0.5; t[:, :cr // 2] = 0.0
        set_weight(mixer, w, "uv", t)
        set_weight(mixer, w, "g", torch.zeros_like(w["g"]))
        set_weight(mixer, w, "dq.norm", torch.ones(qr)); set_weight(mixer, w, "dkv.norm", torch.ones(cr))
        run_plain = lambda h, wd: plain.mixer_latent_attention(h, wd, "p.", layer["mixer"], 1e-5, torch.arange(h.shape[0]))     # noqa: E731
    set_weight(mixer, w, "o", torch.randn(w["o"].shape, generator=g) * 0.3)
    wd = {k: v.double() for k, v in named(w).items()}
    length = 4 * window + 7
    t = length - 1
    seen_sizes, unseen_sizes, outputs = [], [], []
    for j in [t - window + 1, t - window, t - window + 2, t - 1, 0, 1, page - 1, page, (t - window + 1) // page * page]:
        h = 0.01 * torch.randn(length, hidden, generator=g)
        h[:, 0] = -1.0
        h[:, 1] = 1.0
        h[j, 0], h[j, 1] = 1.0, (-5.0 if kind == "attention" else -1.0)
        h[t, 0] = 1.0
        h = h.to(dtype)
        want = run_plain(h.double(), wd).float()
        for tail in (0, 1, 9):                           # the asking token inside a portion, alone, after single tokens
            got = edge_case(rt, mixer, page, h, tail)
            outputs.append((f"key at {j} (edge at {t - window + 1}), last {tail} tokens alone", got, want[-1:]))
        (seen_sizes if 0 <= t - j < window else unseen_sizes).append(want[-1])
    # the crafted key shows: the plain outputs with the key inside the window differ from those with it outside by their
    # whole size (which is what every output is measured against: some of them are sums that cancel)
    size = max(float(x.abs().max()) for x in seen_sizes + unseen_sizes)
    gap = float((seen_sizes[0] - unseen_sizes[0]).abs().max())
    assert gap > 0.4 * size and gap > 0.2
    for what, got, want_row in outputs:
        err = float((got - want_row).abs().max())
        assert err <= (2e-5 if dtype == torch.float32 else 0.1) * size, f"{what}: differs by {err:.3g} (size {size:.3g})"


GLA_SHAPES = [(48, 2, 16, 8, 4.0, 6), (40, 3, 10, 6, 1.0, 3), (64, 2, 32, 32, 16.0, 8), (36, 1, 16, 24, 2.0, 1), (96, 3, 32, 48, 16.0, 8),
              (64, 4, 64, 16, 8.0, 4), (64, 2, 48, 40, 3.0, 5), (40, 1, 24, 8, 16.0, 2), (128, 2, 128, 64, 16.0, 16), (96, 2, 96, 32, 6.0, 4)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,heads,dk,dv,tau,rank", GLA_SHAPES)
def test_gla_alone(dtype, hidden, heads, dk, dv, tau, rank):
    """The recurrence with a decay per key channel from a low-rank projection, the norm over each head with one shared
    weight, the silu gate; two requests in slots of their own, cut into steps of 1 to 150 rows."""
    rt = Runtime(torch.device("cuda"), dtype)
    layer = gla(heads, dk, dv, tau, rank)
    mixer = mixer_of(rt, hidden, layer)
    w = filled(mixer, 12, 0.3)
    set_weight(mixer, w, "a2", torch.randn(w["a2"].shape, generator=torch.Generator().manual_seed(5)) * 1.5)
    wd = {k: v.double() for k, v in named(w).items()}
    run_state_mixer(rt, mixer, hidden, lambda h, pos: plain.mixer_gla(h, wd, "p.", layer["mixer"], 1e-5))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("loud_row", [0, 3, 149])
def test_gla_keeps_one_token_from_far_back(dtype, loud_row):
    """Decays close to 1 and one loud token: hundreds of tokens later the outputs still consist mostly of what that
    token left in the state, through cuts into steps of 1 to 150 tokens.  A state that is lost, zeroed or taken from
    another slot on the way shows at once."""
    rt = Runtime(torch.device("cuda"), dtype)
    hidden, heads, dk, dv = 48, 2, 16, 16
    layer = gla(heads, dk, dv, 16.0, 4)
    mixer = mixer_of(rt, hidden, layer)
    w = filled(mixer, 22, 0.3)
    set_weight(mixer, w, "a2.b", torch.full_like(w["a2.b"], 4.0))       # sigmoid(4 + small)^(1/16): about 0.999 per token
    wd = {k: v.double() for k, v in named(w).items()}
    run_state_mixer(rt, mixer, hidden, lambda h, pos: plain.mixer_gla(h, wd, "p.", layer["mixer"], 1e-5), loud_row=loud_row)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,experts,identity,top,ff,limit,scale", [
    (64, 6, 2, 3, 40, 0.7, 2.0), (40, 3, 0, 1, 20, 1.0, 1.0), (36, 2, 3, 4, 9, 0.25, 0.5), (128, 10, 4, 4, 88, 1.5, 1.5), (48, 1, 1, 2, 16, 5.0, 1.0)])
def test_experts_with_scores_over_all_outputs_alone(dtype, hidden, experts, identity, top, ff, limit, scale):
    """Scores over every router output, the choice by score + correction, the weights the plain scores times a factor,
    identity experts that pass the token itself, the clamped activation; rows whose choice no rounding can turn."""
    rt = Runtime(torch.device("cuda"), dtype)
    typed, layer = typed_layer(hidden, attention(1, 1, 8, 8, 0.3, 4, moe(experts, identity, top, ff, limit, scale)))
    part = build_part("feed_forward", experts_spec(typed, layer.mlp), rt)
    w = fill(part, 14, 0.3)
    g = torch.Generator().manual_seed(2)
    rows = 37
    h = torch.randn(rows, hidden, generator=g).to(dtype)
    outputs = experts + identity
    w["router"] = (torch.randn(outputs, hidden, generator=g) * 0.4).to(torch.bfloat16).float()
    w["correction"] = (torch.randn(outputs, generator=g) * 0.3).to(torch.bfloat16).float()
    part.w_router.copy_(w["router"]); part.correction.copy_(w["correction"])
    wd = {k: v.double() for k, v in named(w).items()}
    mlp = moe(experts, identity, top, ff, limit, scale)
    want = plain.mixture(h.double(), wd, "p.", mlp).float()
    chosen_want, weight_want = plain.route(h.double(), wd, "p.", mlp["router"])
    ctx = ctx_of(rt, list(range(rows)), [0] * rows, [0], [0], [rows], [rows])
    chosen, weight, _ = part.route(ctx, h.cuda())
    choice = torch.softmax(h.double() @ wd["p.router"].T, -1) + wd["p.correction"]
    sure = torch.ones(rows, dtype=torch.bool)
    if top < outputs:
        ranked = choice.sort(dim=-1, descending=True).values
        sure = (ranked[:, top - 1] - ranked[:, top]) > 0.02
    assert int(sure.sum()) >= rows // 2
    assert torch.equal(chosen.cpu().long().sort(-1).values[sure], chosen_want.sort(-1).values[sure])
    lookup = torch.zeros(rows, outputs, dtype=torch.float64).scatter_(1, chosen_want, weight_want)
    close(weight.cpu()[sure], torch.gather(lookup, 1, chosen.cpu().long())[sure].float(), torch.float32, "weights of the chosen",
          f32=2e-2 if dtype == torch.bfloat16 else 1e-5)
    if identity:
        assert int((chosen_want >= experts).sum()) > 0              # identity experts are among the chosen
    gates = torch.einsum("th,efh->tef", h.double(), torch.stack([wd[f"p.e{e}.gate"] for e in range(experts)]))
    assert float(gates.max()) > limit                               # the limit is felt
    for n in (rows, 1):                                            # sorted by expert (bfloat16, several rows), and pair by pair
        one = ctx_of(rt, list(range(n)), [0] * n, [0], [0], [n], [n])
        got = dense_delta(one, part.forward(one, h[:n].cuda()), dtype).float().cpu()
        close(got[sure[:n]], want[:n][sure[:n]], dtype, f"routed feed-forward, {n} rows")


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------
def settle_router(folder):
    """For bfloat16 runs: a router whose choice no rounding can turn.  The corrections stand 3 apart in an order of the
    layer's own, far more than a score can differ, so every token of a layer chooses the same outputs, with weights
    that still depend on the token.  (The choice per token is what the float32 runs, whose routers are as random as
    every other matrix, and the test of the part alone check.)"""
    from safetensors.torch import load_file, save_file
    t = load_file(str(folder / "model.safetensors"))
    for name in sorted(t):
        if name.endswith(".mlp.correction"):
            g = torch.Generator().manual_seed(len(name) + t[name].shape[0])
            t[name] = (torch.randperm(t[name].shape[0], generator=g).float() * 3.0).to(t[name].dtype)
    save_file(t, str(folder / "model.safetensors"), metadata={"format": "pt"})
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """(name, dtype) -> model folder.  The bfloat16 runs get a copy whose routers are settled and whose norms have a
    large eps: a gla head's state after a request's first token has rank one, so its output is (q . k) v, and the norm
    over the head turns that into sign(q . k) times a unit vector unless eps is felt; with the tiny eps of the float32
    models a rounding of q or k that turns the sign of a nearly orthogonal pair moves the row, and the rows behind it,
    by tens of per cent.  (The float32 runs, which no rounding turns, keep the tiny eps.)"""
    tmp = tmp_path_factory.mktemp("dugudra")
    out = {}
    for name, cfg in DUGUDRA_CONFIGS.items():
        out[name, "float32"] = tw.write_random_model(tmp / name, cfg, seed=DUGUDRA_SEEDS[name], std=DUGUDRA_STD[name])
        out[name, "bfloat16"] = settle_router(tw.write_random_model(tmp / f"{name}_settled", {**cfg, "norm": {"eps": 0.05}},
                                                                    seed=DUGUDRA_SEEDS[name], std=DUGUDRA_STD[name]))
    return out


LENGTHS = [70, 1, 45, 100, 2, 33, 64, 129]


def requests_for(name):
    return {f"r{i}": random_tokens(DUGUDRA_CONFIGS[name]["vocab"], n, 20 + i) for i, n in enumerate(LENGTHS)}


@pytest.fixture(scope="module")
def plain_rows(folders):
    return {key: {rid: plain.logits_of(folder, t).numpy() for rid, t in requests_for(key[0]).items()}
            for key, folder in folders.items()}


def moved_weights(folder, seed):
    """The plain model with every matrix element moved by a relative 2^-8 times a normal draw."""
    config, weights = plain.read_folder(folder, torch.float64)
    g = torch.Generator().manual_seed(seed)
    return config, {k: v * (1 + 2.0 ** -8 * torch.randn(v.shape, generator=g, dtype=torch.float64)) if v.dim() == 2 else v
                    for k, v in weights.items()}


@pytest.fixture(scope="module")
def noise(folders, plain_rows):
    """Per (model, run type, request): what the arithmetic alone does to each row.  float32: the plain implementation in
    float32 against itself in float64.  bfloat16: the plain implementation (float64) with perturbed matrices against
    itself (rows behind a nearly orthogonal query and key at a request's first tokens move by tens of per cent)."""
    out = {}
    for name in DUGUDRA_CONFIGS:
        config, moved = moved_weights(folders[name, "bfloat16"], 99)
        for rid, t in requests_for(name).items():
            low = plain.logits_of(folders[name, "float32"], t, torch.float32).numpy()
            out[name, "float32", rid] = [row_error(low[p], plain_rows[name, "float32"][rid][p]) for p in range(len(t))]
            low = plain.forward(config, moved, t).float().numpy()
            out[name, "bfloat16", rid] = [row_error(low[p], plain_rows[name, "bfloat16"][rid][p]) for p in range(len(t))]
    return out


def compare(rows, want, dtype, what, lost=None):
    """Every logits row against the plain one (float64).  float32: every row within 5e-5 of its spread plus four
    times what the plain implementation loses at that row when it runs in float32 itself.  bfloat16: rounding alone
    moves some rows far (the sign of a nearly orthogonal query and key decides a gla head's output at a request's first
    tokens), so the rows are judged together: the median within 6 %, at most five rows in a hundred beyond 8 % plus
    three times what a perturbation of bfloat16's size does to that row of the plain implementation, none that is
    not finite.  A lost state, a key outside its window or a wrong page moves rows by their whole size."""
    errors, over = [], []
    for (rid, p), row in rows.items():
        err = row_error(row, want[rid][p])
        assert np.isfinite(row).all(), f"{what}: {rid}[{p}] is not finite"
        base = lost[rid][p] if lost else 0.0
        if dtype == "float32":
            assert err <= 5e-5 + 4 * base, f"{what}: {rid}[{p}] differs by {err:.3g} of the row's spread (float32 alone: {base:.3g})"
        elif err > 8e-2 + 3 * base:
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
    again (freed pages are filled with NaN first)."""
    reqs = requests_for(name)
    for kind, make in SCHEDULES.items():
        steps = make(reqs)
        rows = replay_in_process(folders[name, dtype], dtype, steps, tmp_path / kind, block_size=DUGUDRA_PAGE[name],
                                 max_tokens=max_live_tokens(steps))
        assert rows, kind
        compare(rows, plain_rows[name, dtype], dtype, f"{name} {kind}", {rid: noise[name, dtype, rid] for rid in reqs})


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
def test_slots_and_pages_used_again(dtype, folders, noise):
    """One request slot and barely enough pages: each request gets the slot and the pages its predecessor gave back,
    with the predecessor's states, latents and keys still in them (the manager zeroes the states at admission)."""
    from tessweave_engine_b200.engine.runner import ModelRunner, StepEntry
    name = "A"
    model = tw.load_model(folders[name, dtype], dtype, "cuda")
    cache = tw.CacheManager(model.cache_needs(), DUGUDRA_PAGE[name], 9, 1, 72, model.runtime.dtype, model.runtime.device,
                            prefix_cache=False)
    runner = ModelRunner(model, cache, 72, 1, cuda_graphs=False)
    config, weights = plain.read_folder(folders[name, dtype], torch.float64)
    _, moved = moved_weights(folders[name, dtype], 96)
    for i, n in enumerate([70, 64, 3, 71]):
        tokens = random_tokens(config["vocab"], n, 40 + i)
        lease = cache.admit(None)
        assert lease.slot == 0
        cut = max(1, n // 2)
        cache.ensure(lease, cut)
        runner.step([StepEntry(lease.slot, tokens[:cut], 0, [])])
        cache.ensure(lease, n)
        got = runner.step([StepEntry(lease.slot, tokens[cut:], cut, list(range(n - cut)))]).cpu().numpy()
        runner.check_status()
        cache.release(lease)
        cache.check_invariants()
        want = plain.forward(config, weights, tokens).numpy()
        if dtype == "float32":
            low = plain.logits_of(folders[name, dtype], tokens, torch.float32).numpy()
        else:
            low = plain.forward(config, moved, tokens).float().numpy()
        compare({("r", cut + k): got[k] for k in range(n - cut)}, {"r": want}, dtype, f"request {i} in a used slot",
                {"r": [row_error(low[p], want[p]) for p in range(n)]})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_windows_and_pages(dtype, folders, tmp_path):
    """A short prompt and 300 tokens one by one: the windows pass over decoded tokens only, pages of the windowed
    layers are given back and used again on the way, the states carry everything else."""
    name = "C"
    toks = random_tokens(DUGUDRA_CONFIGS[name]["vocab"], 310, 77)
    steps = schedule_tail({"long": toks}, tail=300)
    rows = replay_in_process(folders[name, dtype], dtype, steps, tmp_path / "out", block_size=DUGUDRA_PAGE[name], max_tokens=384)
    want = plain.logits_of(folders[name, dtype], toks).numpy()
    if dtype == "float32":
        low = plain.logits_of(folders[name, dtype], toks, torch.float32).numpy()
    else:
        low = plain.forward(*moved_weights(folders[name, dtype], 97), toks).float().numpy()
    compare(rows, {"long": want}, dtype, "long decoding", {"long": [row_error(low[p], want[p]) for p in range(len(toks))]})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_hundreds_of_tokens_past_windows_of_tensor_core_sizes(dtype, tmp_path):
    """Keys of 64 and cached latent rows of 80, windows of 70 and 150, prompts of 420 and 190 tokens: whole, with the
    last 40 tokens one by one, and in mixed batches, on pages of 16 that the windows give back on the way."""
    cfg = DUGUDRA_E if dtype == "float32" else {**DUGUDRA_E, "norm": {"eps": 0.05}}
    folder = tw.write_random_model(tmp_path / "model", cfg, seed=31, std=0.1)
    if dtype == "bfloat16":
        settle_router(folder)
    reqs = {"long": random_tokens(cfg["vocab"], 420, 5), "mid": random_tokens(cfg["vocab"], 190, 6), "short": random_tokens(cfg["vocab"], 37, 7)}
    want = {rid: plain.logits_of(folder, t).numpy() for rid, t in reqs.items()}
    if dtype == "float32":
        lost = {rid: [row_error(r, w) for r, w in zip(plain.logits_of(folder, t, torch.float32).numpy(), want[rid])] for rid, t in reqs.items()}
    else:
        config, moved = moved_weights(folder, 98)
        lost = {rid: [row_error(r, w) for r, w in zip(plain.forward(config, moved, t).float().numpy(), want[rid])] for rid, t in reqs.items()}
    for kind, steps in (("whole", schedule_whole(reqs)), ("tail", schedule_tail(reqs, tail=40)),
                        ("mixed", schedule_mixed(reqs, live=3, seed=2, prefill=(33, 2, 70, 5, 128, 16)))):
        rows = replay_in_process(folder, dtype, steps, tmp_path / kind, block_size=16, max_tokens=max_live_tokens(steps))
        compare(rows, want, dtype, f"E {kind}", lost)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_engine(name, dtype, folders):
    """``generate`` (scheduler, continuous batching, CUDA graphs, look-ahead) against the plain greedy loop;
    every chosen token must be the plain implementation's best on that path, or nearly."""
    prompts = [random_tokens(DUGUDRA_CONFIGS[name]["vocab"], n, 60 + n) for n in (21, 5, 40)]
    model = tw.load_model(folders[name, dtype], dtype, "cuda")
    out = tw.generate(model, prompts, max_tokens=12, ignore_eos=True,
                      engine_config=tw.EngineConfig(block_size=DUGUDRA_PAGE[name], kv_blocks=40, max_context=128, max_active=2,
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
