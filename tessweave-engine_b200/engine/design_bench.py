"""Two designs side by side at equal layer sizes: whole-step throughput (a prompt step, decode steps) of
each, and the kernels of the Linurax design alone with their rooflines.

The Linurax model of the comparison has the residual width, head counts, head size, feed-forward size and
vocabulary of the Qwen2 benchmark configuration; its layers alternate [attention + feed-forward, mingru,
mingru, attention + feed-forward], the recurrent width equals the residual width.  Weights are random.
``python bench.py --design linurax`` prints the record.
"""
from __future__ import annotations

import statistics

import torch

from ..cache.manager import CacheManager
from ..csrc import ops
from ..parts.base import Runtime, StateView, Workspace, build_part
from .kernel_bench import _context, _copies, _fill, _graph_us, _kernels_of


def linurax_config_like(qwen: dict, layers: int) -> dict:
    """A Linurax config.json with the sizes of the Qwen2 configuration ``qwen``."""
    heads, kv, dim = qwen["num_attention_heads"], qwen["num_key_value_heads"], qwen["head_dim"]
    attention = {"type": "attention",
                 "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                           "rot": {"dims": dim, "base": qwen["rope_theta"]}},
                 "mlp": {"kind": "dense", "ff": qwen["intermediate_size"]}}
    recurrent = {"type": "mingru", "mixer": {"width": qwen["hidden_size"]}, "mlp": None}
    pattern = [attention, recurrent, recurrent, attention]
    return {"architecture": "Linurax", "vocab": qwen["vocab_size"], "width": qwen["hidden_size"],
            "embedding": {"scale": 1.0}, "norm": {"eps": qwen["rms_norm_eps"]},
            "layers": [pattern[i % 4] for i in range(layers)]}


def build(config: dict):
    import tessweave_engine_b200 as tw
    cfg, spec = tw.resolve(config)
    model = tw.Model(spec, Runtime(torch.device("cuda:0"), torch.bfloat16), config=cfg)
    tw.fill_random(model, seed=0)
    return model


def step_times(model, batch: int, context: int, prefill_tokens: int, page_size: int, steps: int = 24, warmup: int = 4) -> dict:
    """Median time of a prompt step of ``prefill_tokens`` tokens, and time per decode step of ``batch``
    requests that hold ``context`` tokens each (CUDA graphs, random cache contents)."""
    from .runner import ModelRunner, StepEntry
    vocab = model.spec.vocab_size
    out = {}
    # ---- a prompt step
    cache = CacheManager(model.cache_needs(), page_size, -(-prefill_tokens // page_size), 1, prefill_tokens,
                         model.runtime.dtype, model.runtime.device, prefix_cache=False)
    runner = ModelRunner(model, cache, max_step_tokens=prefill_tokens, max_step_seqs=1, max_logit_rows=1, cuda_graphs=False)
    lease = cache.admit(None)
    cache.ensure(lease, prefill_tokens)
    ids = torch.randint(0, vocab, (prefill_tokens,), generator=torch.Generator().manual_seed(2)).tolist()
    entry = [StepEntry(lease.slot, ids, 0, [prefill_tokens - 1])]
    for _ in range(3):
        runner.step(entry)
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.step(entry)
        end.record()
        torch.cuda.synchronize()
        times.append(begin.elapsed_time(end))
    runner.check_status()
    out["prefill_ms"] = statistics.median(times)
    out["prefill_tok_s"] = prefill_tokens / (out["prefill_ms"] / 1e3)
    del runner, cache
    torch.cuda.empty_cache()
    # ---- decode steps
    for b in sorted({1, batch}):
        total = warmup + steps
        start = max(1, context - total)
        cache = CacheManager(model.cache_needs(), page_size, b * (-(-(start + total) // page_size)), b, start + total,
                             model.runtime.dtype, model.runtime.device, prefix_cache=False)
        for g in cache.groups:
            g.k.normal_(0, 0.5)
            g.v.normal_(0, 0.5)
        runner = ModelRunner(model, cache, max_step_tokens=b, max_step_seqs=b, cuda_graphs=True)
        leases = [cache.admit(None) for _ in range(b)]
        for lease in leases:
            cache.ensure(lease, start + total)
        tokens = torch.randint(0, vocab, (total, b), generator=torch.Generator().manual_seed(1)).tolist()

        def one(i):
            return runner.step([StepEntry(leases[r].slot, [tokens[i][r]], start + i, [0]) for r in range(b)])

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for i in range(warmup, total):
            one(i)
        end.record()
        torch.cuda.synchronize()
        runner.check_status()
        ms = begin.elapsed_time(end) / steps
        element = 2
        nbytes = model.step_weight_bytes(b) + b * (start + warmup + steps / 2) * model.cache_bytes_per_token(element)
        out[f"decode_b{b}_ms"] = ms
        out[f"decode_b{b}_tok_s"] = b / (ms / 1e3)
        out[f"decode_b{b}_step_bytes"] = nbytes
        bucket = next((k for k in sorted(runner.graph_kernels) if k >= b), None)
        out[f"decode_b{b}_kernels"] = runner.graph_kernels.get(bucket)
        del runner, cache
        torch.cuda.empty_cache()
    return out


def linurax_kernel_table(spec, batch: int, context: int, prefill_tokens: int, hbm_gbs: float, tflops: float,
                         page_size: int = 16) -> list[dict]:
    """The Linurax kernels alone, each inside a CUDA graph with operands rotated beyond L2: preparation of queries
    and keys, attention over the cache, the recurrence, the norm into the stream; decode (``batch`` rows) and a
    prompt step.  fraction = max(bytes / HBM peak, FLOPs / tensor peak) / time."""
    dev, bf = torch.device("cuda"), torch.bfloat16
    rt = Runtime(dev, bf)
    att_spec = next(l.block.params["mixer"] for l in spec.layers if l.block.params["mixer"].kind == "sigmoid_attention")
    rec_spec = next(l.block.params["mixer"] for l in spec.layers if l.block.params["mixer"].kind == "mingru")
    norm_spec = spec.layers[0].block.params["norm1"]
    H = spec.hidden_size
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rows: list[dict] = []

    def add(name, m, thunks, nbytes, flops, reps=4):
        kernel = _kernels_of(thunks[0])
        us = _graph_us(thunks, reps)
        floor = max(nbytes / (hbm_gbs * 1e9), flops / (tflops * 1e12)) * 1e6
        rows.append({"op": name, "rows": m, "kernel": kernel, "us": round(us, 2), "mbytes": round(nbytes / 1e6, 2),
                     "gflop": round(flops / 1e9, 2), "floor_us": round(floor, 2), "frac": round(floor / us, 3),
                     "bound": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / (tflops * 1e12) else "tensor"})

    for m, phase in ((batch, "decode"), (prefill_tokens, "prefill")):
        ws = Workspace(dev)
        if phase == "decode":
            ctx = _context(rt, ws, status, [context - 1] * m, list(range(m)), list(range(m)), list(range(m)), [1] * m, [context] * m)
        else:
            ctx = _context(rt, ws, status, list(range(m)), [0] * m, [0], [0], [m], [m])
        # ---- norm of a sub-layer's output into the stream
        norm = build_part("norm", norm_spec, rt)
        _fill(norm)
        sets = [(torch.randn(m, H, device=dev), torch.randn(m, H, device=dev, dtype=bf), torch.empty(m, H, device=dev, dtype=bf))
                for _ in range(_copies(m * H * 12))]
        add(f"{phase}: RMSNorm of the output + residual add", m,
            [(lambda r=r, d=d, c=c: norm.add_normed(ctx, r, d, m, c)) for r, d, c in sets], m * H * (2 + 4 + 4 + 2), 0.0, reps=8)
        del sets
        # ---- attention: preparation, then the keys
        att = build_part("mixer", att_spec, rt)
        _fill(att)
        att.mix.copy_(torch.eye(att.n_heads, device=dev) + 0.05 * torch.randn(att.n_heads, att.n_heads, device=dev))
        Hq, G, D = att.n_heads, att.n_kv_heads, att.head_dim
        requests = batch if phase == "decode" else 1
        kv_tokens = context if phase == "decode" else m
        blocks = -(-kv_tokens // page_size)
        page_bytes = 2 * requests * blocks * page_size * G * D * 2
        caches = []
        for _ in range(_copies(page_bytes)):
            cache = CacheManager([(att.cache_need(), None)], page_size, requests * blocks, requests, kv_tokens, bf, dev,
                                 prefix_cache=False)
            for g in cache.groups:
                g.k.normal_(0, 0.5)
                g.v.normal_(0, 0.5)
            for _r in range(requests):
                cache.ensure(cache.admit(None), kv_tokens)
            cache.sync_tables()
            caches.append(cache)
        views = [c.view(0) for c in caches]
        in_w = att.q_size + att.kv_size + att.gate_size
        projs = [torch.randn(m, in_w, device=dev, dtype=bf) for _ in range(_copies(m * in_w * 2) if phase == "prefill" else 1)]
        add(f"{phase}: q/k norms + rotation + cache write + fold of the heads' mixing", m,
            [(lambda v=v, i=i: att.prepare(ctx, projs[i % len(projs)], v, True)) for i, v in enumerate(views)],
            m * (att.q_size + att.kv_size) * 2 + m * 2 * att.kv_size * 2 + m * Hq * att.kv_size * 2, 2.0 * m * Hq * Hq * D)
        qf = att.prepare(ctx, projs[0], views[0], True).clone()
        if phase == "decode":
            nbytes = m * context * G * D * 2 * 2 + m * Hq * att.kv_size * 2
            flops = 2.0 * m * Hq * (att.kv_size + D) * context
            name = f"decode: sigmoid attention over {context} keys + output gate"
        else:
            nbytes = m * Hq * att.kv_size * 2 + 2 * m * att.kv_size * 2 + m * att.q_size * 2 * 2
            flops = 2.0 * Hq * (att.kv_size + D) * m * (m + 1) / 2
            name = f"prefill: causal sigmoid attention + output gate, {m} tokens"
        add(name, m, [(lambda v=v, i=i: att.attend_prepared(ctx, qf, projs[i % len(projs)], v)) for i, v in enumerate(views)],
            nbytes, flops)
        del caches, views, projs, att
        # ---- the recurrence
        rec = build_part("mixer", rec_spec, rt)
        _fill(rec)
        W = rec.width
        state = StateView(torch.zeros(max(requests, 1), W, device=dev))
        projs = [torch.randn(m, 3 * W, device=dev, dtype=bf) for _ in range(_copies(m * 3 * W * 2) if phase == "prefill" else 1)]
        add(f"{phase}: minGRU gates + recurrence + output gate", m, [(lambda p=p: rec.recur(ctx, p, state)) for p in projs],
            m * 3 * W * 2 + m * W * 2 + 2 * requests * W * 4, 0.0, reps=8)
        del projs, rec
        torch.cuda.empty_cache()
    if int(status) != 0:
        raise RuntimeError(f"a kernel reported status {int(status)} during the kernel table")
    return rows


# ---------------------------------------------------------------------------
# the Sapatar decoder
# ---------------------------------------------------------------------------
def sapatar_config_like(qwen: dict, layers: int) -> dict:
    """A Sapatar config.json with the sizes of the Qwen2 configuration ``qwen``: layers [attention beside mLSTM, wkv,
    retention, attention beside mLSTM] in turn, each with eight experts of a quarter of the dense feed-forward's size
    (two chosen) and a shared expert of that size, four copies of the residual stream.  The attention has Qwen2's
    head counts and head size (keys and values alike) and a window of 1,024; mLSTM and retention have half as many
    heads of the same size; wkv has heads of 64."""
    heads, kv, dim, width = qwen["num_attention_heads"], qwen["num_key_value_heads"], qwen["head_dim"], qwen["hidden_size"]
    ff = qwen["intermediate_size"] // 4
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": 8, "top": 2}, "shared": {"ff": ff}}
    rot = {"dims": dim, "base": qwen["rope_theta"]}
    half = max(1, heads // 2)
    parallel = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": 1024}, "rot": rot},
        "right": {"heads": half, "dim": dim, "vdim": dim, "gate_cap": 15.0}, "left_scale": 1.0, "right_scale": 1.0}}
    wkv = {"type": "wkv", "mlp": mlp, "mixer": {"heads": width // 64, "dim": 64, "decay_rank": 64}}
    retention = {"type": "retention", "mlp": mlp, "mixer": {"heads": half, "dim": dim, "vdim": dim, "rot": rot,
                                                            "decay": [1.0 - 2.0 ** -(5 + h % 8) for h in range(half)]}}
    pattern = [parallel, wkv, retention, parallel]
    return {"architecture": "Sapatar", "vocab": qwen["vocab_size"], "width": width, "norm": {"eps": qwen["rms_norm_eps"]},
            "streams": 4, "layers": [pattern[i % 4] for i in range(layers)]}


def sapatar_kernel_table(config: dict, batch: int, context: int, prefill_tokens: int, hbm_gbs: float, tflops: float) -> list[dict]:
    """The Sapatar kernels alone, each inside a CUDA graph with operands rotated beyond L2, for a decode step of
    ``batch`` rows and a prompt step: the pass over the stream's copies, the token shift, the three recurrences, the
    norm over heads with its gate, and the routed experts (router, and the experts' products).
    fraction = max(bytes / HBM peak, FLOPs / tensor peak) / time."""
    import tessweave_engine_b200 as tw
    dev, bf = torch.device("cuda"), torch.bfloat16
    rt = Runtime(dev, bf)
    cfg, _ = tw.resolve(config)
    W, S = cfg.width, cfg.streams or 1
    par = next(l.mixer for l in cfg.layers if l.type == "parallel")
    wk = next(l.mixer for l in cfg.layers if l.type == "wkv")
    ret = next(l.mixer for l in cfg.layers if l.type == "retention")
    mlp = next(l.mlp for l in cfg.layers if l.mlp is not None)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rows: list[dict] = []

    def add(name, m, thunks, nbytes, flops, reps=4, note=""):
        kernel = _kernels_of(thunks[0])
        us = _graph_us(thunks, reps)
        floor = max(nbytes / (hbm_gbs * 1e9), flops / (tflops * 1e12)) * 1e6
        rows.append({"op": name, "rows": m, "kernel": kernel, "us": round(us, 2), "mbytes": round(nbytes / 1e6, 2),
                     "gflop": round(flops / 1e9, 2), "floor_us": round(floor, 2), "frac": round(floor / us, 3),
                     "bound": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / (tflops * 1e12) else "tensor", "note": note})

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)     # noqa: E731
    for m, phase in ((batch, "decode"), (prefill_tokens, "prefill")):
        requests = batch if phase == "decode" else 1
        per = m // requests
        slots, starts, lens = i32(list(range(requests))), i32([r * per for r in range(requests)]), i32([per] * requests)
        seq_of = i32([r for r in range(requests) for _ in range(per)])
        positions = i32([context - 1] * m if phase == "decode" else list(range(m)))
        # ---- the copies of the stream: write a sub-layer's output, read the next one's input through its norm
        sets = [(torch.randn(m, S, W, device=dev), torch.randn(m, W, device=dev, dtype=bf), torch.empty(m, W, device=dev, dtype=bf))
                for _ in range(_copies(m * W * (8 * S + 4)))]
        mix, oc, ic, nw = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.ones(S, device=dev), torch.ones(W, device=dev)
        add(f"{phase}: write into {S} copies of the stream + read + RMSNorm", m,
            [(lambda x=x, y=y, h=h: ops.hyper_step(x, m, y=y, mix=mix, out_coef=oc, in_coef=ic, norm_weight=nw, eps=1e-6, h_out=h))
             for x, y, h in sets], m * W * (8 * S + 4), 0.0, reps=8)
        del sets
        # ---- token shift
        state = torch.zeros(requests, W, device=dev)
        mu = torch.rand(5, W, device=dev)
        sets = [(torch.randn(m, W, device=dev, dtype=bf), torch.empty(5, m, W, device=dev, dtype=bf)) for _ in range(_copies(m * W * 12))]
        add(f"{phase}: token shift, five blends", m,
            [(lambda h=h, o=o: ops.token_shift_mix(o, h, mu, state, 0, seq_of, slots, starts, m)) for h, o in sets], m * W * 12, 0.0, reps=8)
        del sets
        # ---- the three recurrences and what follows them
        for rule, name, H, Dk, Dv in ((ops.RECURRENCE_WKV, "wkv", wk.heads, wk.dim, wk.dim),
                                      (ops.RECURRENCE_RETENTION, "retention", ret.heads, ret.dim, ret.vdim),
                                      (ops.RECURRENCE_MLSTM, "mlstm", par.right.heads, par.right.dim, par.right.vdim)):
            numel = ops.recurrence_state_numel(rule, H, Dk, Dv)
            n_sets = _copies(max(requests * numel * 8, m * H * (2 * Dk + Dv) * 2))
            sets = []
            for _ in range(n_sets):
                q, k, v = (torch.randn(m, H * d, device=dev, dtype=bf) * 0.3 for d in (Dk, Dk, Dv))
                sets.append((q, k, v, torch.zeros(requests, numel, device=dev), torch.empty(m, H * Dv, device=dev),
                             torch.empty(m, H, device=dev)))
            extra = {}
            if rule == ops.RECURRENCE_WKV:
                extra = {"pre": torch.randn(m, H * Dk, device=dev), "p0": torch.zeros(H * Dk, device=dev), "p1": torch.zeros(H * Dk, device=dev)}
            elif rule == ops.RECURRENCE_RETENTION:
                extra = {"p0": torch.full((H,), 0.97, device=dev), "k_scale": Dk ** -0.5,
                         "inv_freq": torch.rand(Dk // 2, device=dev), "rot_dims": Dk}
            else:
                extra = {"pre": torch.randn(m, 2 * H, device=dev), "p0": torch.zeros(2 * H, device=dev), "q_scale": Dk ** -0.5, "cap": 15.0}
            nbytes = m * H * (2 * Dk + Dv) * 2 + m * H * Dv * 4 + 2 * requests * numel * 4 + (m * H * Dk * 4 if rule == ops.RECURRENCE_WKV else 0)
            add(f"{phase}: {name} recurrence, {H} heads of {Dk} x {Dv}", m,
                [(lambda s=s: ops.linear_recurrence(rule, s[4], s[5] if rule == ops.RECURRENCE_MLSTM else None, s[0], s[1], s[2], s[3],
                                                    positions, slots, starts, lens, requests, H, Dk, Dv, True, max_q_len=per, **extra)) for s in sets],
                nbytes, 0.0, reps=2 if phase == "prefill" else 8,
                note=f"{4.0 * m * H * Dk * Dv / 1e9:.2f} GFLOP of fp32 multiply-adds outside the tensor cores")
            del sets
        H, Dv = par.right.heads, par.right.vdim
        sets = [(torch.randn(m, H * Dv, device=dev), torch.rand(m, H, device=dev) + 0.5, torch.randn(m, H * Dv, device=dev, dtype=bf),
                 torch.empty(m, H * Dv, device=dev, dtype=bf)) for _ in range(_copies(m * H * Dv * 8))]
        nw2 = torch.ones(H * Dv, device=dev)
        add(f"{phase}: norm over each head + gate", m,
            [(lambda r=r, d=d, g=g, o=o: ops.head_norm_gate(o, r, d, nw2, g, ops.GATE_SIGMOID, 1e-6, m, H, Dv)) for r, d, g, o in sets],
            m * H * Dv * 8, 0.0, reps=8)
        del sets
        # ---- routed experts (without the shared expert, which is the dense feed-forward part)
        spec = tw.PartSpec("routed_experts", {"hidden": W, "experts": mlp.experts, "top": mlp.top, "intermediate": mlp.ff})
        part_bytes = mlp.experts * 3 * mlp.ff * W * 2
        parts = []
        for _ in range(_copies(part_bytes) if phase == "decode" else 2):
            part = build_part("feed_forward", spec, rt)
            _fill(part)
            part.w_router.normal_(0, 0.5)
            parts.append(part)
        ws = Workspace(dev)
        ctx = _context(rt, ws, status, positions.tolist(), seq_of.tolist(), list(range(requests)), starts.tolist(), lens.tolist(),
                       [context] * requests if phase == "decode" else [m])
        hs = [torch.randn(m, W, device=dev, dtype=bf) for _ in range(4)]
        touched = min(mlp.experts, m * mlp.top)
        add(f"{phase}: router, {mlp.experts} experts, {mlp.top} chosen", m,
            [(lambda p=p, i=i: p.route(ctx, hs[i % 4])) for i, p in enumerate(parts)], m * W * 2 + mlp.experts * W * 2, 0.0, reps=8)
        add(f"{phase}: the chosen experts' gate/up, SiLU.mul, down and the weighted sum", m,
            [(lambda p=p, i=i: p.forward(ctx, hs[i % 4])) for i, p in enumerate(parts)],
            touched * 3 * mlp.ff * W * 2 + m * W * 4, 2.0 * m * mlp.top * 3 * mlp.ff * W, reps=2,
            note="includes the router; bytes: the matrices of the experts a step of this size touches at most, once")
        del parts
        torch.cuda.empty_cache()
    if int(status) != 0:
        raise RuntimeError(f"a kernel reported status {int(status)} during the kernel table")
    return rows


# ---------------------------------------------------------------------------
# the Nufatar decoder
# ---------------------------------------------------------------------------
def nufatar_config_like(qwen: dict, layers: int) -> dict:
    """A Nufatar config.json with the sizes of the Qwen2 configuration ``qwen``: layers [causal, windowed, causal,
    causal] in turn, all of them with the dense feed-forward of ``qwen``.  Both attentions have Qwen2's head counts and
    head size (the causal one rotates half of a head at stretched rates; the windowed one sees 1,024 tokens through a
    distance table of 32 rows that reaches 512); the delta rules have half as many heads of the same size, a q/k head
    for every two of them and convolutions of four taps; the low-rank projections have an inner size of 64.  The first
    half of the layers is run twice."""
    heads, kv, dim, width = qwen["num_attention_heads"], qwen["num_key_value_heads"], qwen["head_dim"], qwen["hidden_size"]
    half = max(2, heads // 2)
    mlp = {"kind": "dense", "ff": qwen["intermediate_size"]}
    right = {"heads": half, "kv_heads": half // 2, "dim": dim, "vdim": dim, "conv": 4}
    causal = {"type": "parallel_2", "mlp": mlp, "mixer": {
        "left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                 "rot": {"dims": dim // 2, "base": qwen["rope_theta"],
                         "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
        "right": right, "left_scale": 0.6, "right_scale": 1.1}}
    windowed = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": 1024},
                 "bias_max": 512, "bias_rows": 32},
        "right": {**right, "decay_rank": 64, "gate_rank": 64}}}
    pattern = [causal, windowed, causal, causal]
    return {"architecture": "Nufatar", "vocab": qwen["vocab_size"], "width": width, "norm": {"eps": qwen["rms_norm_eps"]},
            "layers": [pattern[i % 4] for i in range(layers)], "loop": {"start": 0, "stop": max(1, layers // 2), "times": 2}}


def nufatar_kernel_table(config: dict, batch: int, context: int, prefill_tokens: int, hbm_gbs: float, tflops: float,
                         page_size: int = 16) -> list[dict]:
    """The Nufatar kernels alone, each inside a CUDA graph with operands rotated beyond L2, for a decode step of
    ``batch`` rows and a prompt step: both attentions over their caches (position encoding, store and attention), the
    short convolutions with their unit norms, the delta rule with either kind of decay, the norm over heads with its
    gate, and the normalised sum of the two sides.  fraction = max(bytes / HBM peak, FLOPs / tensor peak) / time."""
    import tessweave_engine_b200 as tw
    from ..models.nufatar import attention_spec
    dev, bf = torch.device("cuda"), torch.bfloat16
    rt = Runtime(dev, bf)
    cfg, _ = tw.resolve(config)
    W = cfg.width
    causal = next(l.mixer for l in cfg.layers if l.type == "parallel_2")
    windowed = next(l.mixer for l in cfg.layers if l.type == "parallel")
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rows: list[dict] = []

    def add(name, m, thunks, nbytes, flops, reps=4, note=""):
        kernel = _kernels_of(thunks[0])
        us = _graph_us(thunks, reps)
        floor = max(nbytes / (hbm_gbs * 1e9), flops / (tflops * 1e12)) * 1e6
        rows.append({"op": name, "rows": m, "kernel": kernel, "us": round(us, 2), "mbytes": round(nbytes / 1e6, 2),
                     "gflop": round(flops / 1e9, 2), "floor_us": round(floor, 2), "frac": round(floor / us, 3),
                     "bound": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / (tflops * 1e12) else "tensor", "note": note})

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)     # noqa: E731
    for m, phase in ((batch, "decode"), (prefill_tokens, "prefill")):
        requests = batch if phase == "decode" else 1
        per = m // requests
        slots, starts, lens = i32(list(range(requests))), i32([r * per for r in range(requests)]), i32([per] * requests)
        seq_of = i32([r for r in range(requests) for _ in range(per)])
        positions = i32([context - 1] * m if phase == "decode" else list(range(m)))
        ws = Workspace(dev)
        ctx = _context(rt, ws, status, positions.tolist(), seq_of.tolist(), list(range(requests)), starts.tolist(), lens.tolist(),
                       [context] * requests if phase == "decode" else [m])
        # ---- the two attentions: position encoding, store, attention
        for label, side in (("causal attention, half of a head rotated", causal.left),
                            (f"attention over a window of {windowed.left.window} with distance table and sink, values = keys", windowed.left)):
            att = build_part("mixer", attention_spec(cfg, side, "bench"), rt)
            _fill(att)
            att.finalize()
            Hq, G, D = att.n_heads, att.n_kv_heads, att.head_dim
            kv_tokens = context if phase == "decode" else m
            seen = min(kv_tokens, side.window) if side.window else kv_tokens
            blocks = -(-kv_tokens // page_size)
            per_key = G * D * 2 * (1 if att.values_are_keys else 2)
            caches = []
            for _ in range(_copies(requests * blocks * page_size * per_key)):
                cache = CacheManager([(att.cache_need(), None)], page_size, requests * blocks, requests, kv_tokens, bf, dev,
                                     prefix_cache=False)
                for g in cache.groups:
                    g.k.normal_(0, 0.5)
                    if g.v is not g.k:
                        g.v.normal_(0, 0.5)
                for _r in range(requests):
                    cache.ensure(cache.admit(None), kv_tokens)
                cache.sync_tables()
                caches.append(cache)
            views = [c.view(0) for c in caches]
            projs = [torch.randn(m, att.qkv_width, device=dev, dtype=bf) for _ in range(_copies(m * att.qkv_width * 2) if phase == "prefill" else 1)]
            if phase == "decode":
                nbytes = m * seen * per_key + m * (att.qkv_width + att.out_size) * 2
                flops = 2.0 * m * Hq * 2 * D * seen
            else:
                nbytes = m * (att.qkv_width * 2 + att.out_size) * 2 + m * per_key
                pairs = m * (m + 1) / 2 if not side.window else seen * (m - seen) + seen * (seen + 1) / 2
                flops = 2.0 * Hq * 2 * D * pairs
            add(f"{phase}: {label}", m,
                [(lambda v=v, i=i: att.attend(ctx, projs[i % len(projs)], v, True)) for i, v in enumerate(views)], nbytes, flops,
                reps=2 if phase == "prefill" else 4)
            del caches, views, projs, att
            torch.cuda.empty_cache()
        # ---- the delta rule: convolutions, recurrence, norm over heads
        for label, side in (("a decay per head", causal.right), ("a decay per key channel", windowed.right)):
            H, Gq, Dk, Dv, taps = side.heads, side.kv_heads, side.dim, side.vdim, side.conv
            C = 2 * Gq * Dk + H * Dv
            numel = ops.recurrence_state_numel(ops.RECURRENCE_DELTA, H, Dk, Dv)
            conv_w = torch.randn(C, taps, device=dev) * 0.3
            n_sets = _copies(max(requests * numel * 8, m * C * 6))
            sets = []
            for _ in range(n_sets):
                state = torch.zeros(requests, numel + C * (taps - 1), device=dev)
                sets.append((torch.randn(m, C, device=dev, dtype=bf) * 0.3, torch.empty(m, C, device=dev), state,
                             torch.empty(m, H * Dv, device=dev), torch.randn(m, 2 * H, device=dev),
                             torch.randn(m, H * Dk, device=dev) if side.channel_decay else None))
            if label == "a decay per head":
                def conv(s):      # as the delta rule calls them: single rows move their state on in the convolution itself
                    ops.short_conv(s[1], s[0], conv_w, s[2], numel, seq_of, slots, starts, m, unit_heads=2 * Gq, unit_dim=Dk,
                                   scaled_heads=Gq, head_scale=Dk ** -0.5, unit_eps=1e-6, move_single=lens)
                    if per > 1:
                        ops.short_conv_state(s[0], taps, C, s[2], numel, slots, starts, lens, requests, skip_single=True)
                add(f"{phase}: convolutions of {taps} taps + silu + unit norms, {C} channels", m, [(lambda s=s: conv(s)) for s in sets],
                    m * C * 6 + 2 * requests * C * (taps - 1) * 4, 0.0, reps=8)
            for s in sets:
                s[1].normal_(0, 0.1)
            rate = torch.full((H,), -1.0, device=dev)
            dt = torch.zeros(H * Dk if side.channel_decay else H, device=dev)
            a = Gq * Dk

            def recur(s):
                ops.linear_recurrence(ops.RECURRENCE_DELTA, s[3], None, s[1][:, :a], s[1][:, a:2 * a], s[1][:, 2 * a:], s[2], positions,
                                      slots, starts, lens, requests, H, Dk, Dv, True, pre=s[5] if side.channel_decay else s[4][:, H:],
                                      p0=rate, p1=dt, write_pre=s[4], channel_decay=side.channel_decay, qk_group=H // Gq, max_q_len=per)
            nbytes = m * C * 4 + m * H * Dv * 4 + 2 * requests * numel * 4 + (m * H * Dk * 4 if side.channel_decay else m * H * 8)
            add(f"{phase}: delta rule with {label}, {H} heads of {Dk} x {Dv}", m, [(lambda s=s: recur(s)) for s in sets], nbytes, 0.0,
                reps=2 if phase == "prefill" else 8,
                note=f"{6.0 * m * H * Dk * Dv / 1e9:.2f} GFLOP of fp32 multiply-adds outside the tensor cores")
            del sets
            torch.cuda.empty_cache()
        H, Dv = causal.right.heads, causal.right.vdim
        sets = [(torch.randn(m, H * Dv, device=dev), torch.randn(m, H * Dv, device=dev, dtype=bf), torch.empty(m, H * Dv, device=dev, dtype=bf))
                for _ in range(_copies(m * H * Dv * 8))]
        nw = torch.ones(H * Dv, device=dev)
        add(f"{phase}: norm over each head + gate", m,
            [(lambda r=r, g=g, o=o: ops.head_norm_gate(o, r, None, nw, g, ops.GATE_SILU, 1e-6, m, H, Dv)) for r, g, o in sets],
            m * H * Dv * 8, 0.0, reps=8)
        del sets
        # ---- the normalised sum of the two sides
        sets = [(torch.empty(m, W, device=dev, dtype=bf), torch.randn(m, W, device=dev, dtype=bf),
                 torch.randn(m, W, device=dev, dtype=bf)) for _ in range(_copies(m * W * 6))]
        nw = torch.ones(2, W, device=dev)

        def both(out, x, y):
            ops.weighted_sum_rows(out, [x, y], [0.5, 0.5], nw, 1e-6, m)
        add(f"{phase}: RMSNorm of each side + half their sum", m, [(lambda s=s: both(*s)) for s in sets], m * W * (2 + 2 + 2), 0.0, reps=8)
        del sets
        torch.cuda.empty_cache()
    if int(status) != 0:
        raise RuntimeError(f"a kernel reported status {int(status)} during the kernel table")
    return rows


# ---------------------------------------------------------------------------
# the Dugudra decoder
# ---------------------------------------------------------------------------
def dugudra_config_like(qwen: dict, layers: int) -> dict:
    """A Dugudra config.json with the sizes of the Qwen2 configuration ``qwen``: layers [attention, latent attention,
    gla, latent attention] in turn, each with eight experts of a quarter of the dense feed-forward's size and two
    identity experts (three chosen).  The attention has Qwen2's head counts and head size and a window of 1,024; the
    latent attention has as many heads of the same size with half as many rotated values more, a query latent of 1,536
    and cached rows of 192 + 64 values, the same window; gla has half as many heads of the same size."""
    heads, kv, dim, width = qwen["num_attention_heads"], qwen["num_key_value_heads"], qwen["head_dim"], qwen["hidden_size"]
    mlp = {"kind": "moe", "expert": {"ff": qwen["intermediate_size"] // 4, "limit": 7.0},
           "router": {"experts": 8, "identity": 2, "top": 3, "scale": 1.5}}
    half = max(1, heads // 2)
    attention = {"type": "attention", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim,
                                                            "scale": dim ** -0.5, "mask": {"size": 1024}}}
    latent = {"type": "latent_attention", "mlp": mlp, "mixer": {
        "heads": heads, "dim": dim, "rot_dim": dim // 2, "vdim": dim, "q_rank": 1536, "kv_rank": 256 - dim // 2,
        "scale": (dim + dim // 2) ** -0.5, "mask": {"size": 1024},
        "rot": {"dims": dim // 2, "base": qwen["rope_theta"], "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    gla = {"type": "gla", "mlp": mlp, "mixer": {"heads": half, "dim": dim, "vdim": dim, "tau": 16.0, "decay_rank": 64}}
    pattern = [attention, latent, gla, latent]
    return {"architecture": "Dugudra", "vocab": qwen["vocab_size"], "width": width, "norm": {"eps": qwen["rms_norm_eps"]},
            "embedding": {"scale": width ** 0.5}, "residual_mult": 0.7, "logit_softcap": 30.0,
            "layers": [pattern[i % 4] for i in range(layers)]}


def dugudra_kernel_table(config: dict, batch: int, context: int, prefill_tokens: int, hbm_gbs: float, tflops: float,
                         page_size: int = 16) -> list[dict]:
    """The Dugudra kernels alone, each inside a CUDA graph with operands rotated beyond L2, for a decode step of
    ``batch`` rows and a prompt step: both attentions over their caches (norms, rotation, store, the per-head maps of the
    latent kind, attention), the gla recurrence, the norm over heads with its gate, the routed experts with identity
    experts, and the norm that adds a scaled delta.  fraction = max(bytes / HBM peak, FLOPs / tensor peak) / time."""
    import tessweave_engine_b200 as tw
    from ..models.dugudra import experts_spec, mixer_spec
    dev, bf = torch.device("cuda"), torch.bfloat16
    rt = Runtime(dev, bf)
    cfg, _ = tw.resolve(config)
    W = cfg.width
    layer_of = {l.type: l for l in cfg.layers}
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rows: list[dict] = []

    def add(name, m, thunks, nbytes, flops, reps=4, note=""):
        kernel = _kernels_of(thunks[0])
        us = _graph_us(thunks, reps)
        floor = max(nbytes / (hbm_gbs * 1e9), flops / (tflops * 1e12)) * 1e6
        rows.append({"op": name, "rows": m, "kernel": kernel, "us": round(us, 2), "mbytes": round(nbytes / 1e6, 2),
                     "gflop": round(flops / 1e9, 2), "floor_us": round(floor, 2), "frac": round(floor / us, 3),
                     "bound": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / (tflops * 1e12) else "tensor", "note": note})

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)     # noqa: E731
    for m, phase in ((batch, "decode"), (prefill_tokens, "prefill")):
        requests = batch if phase == "decode" else 1
        per = m // requests
        slots, starts, lens = i32(list(range(requests))), i32([r * per for r in range(requests)]), i32([per] * requests)
        seq_of = i32([r for r in range(requests) for _ in range(per)])
        positions = i32([context - 1] * m if phase == "decode" else list(range(m)))
        ws = Workspace(dev)
        ctx = _context(rt, ws, status, positions.tolist(), seq_of.tolist(), list(range(requests)), starts.tolist(), lens.tolist(),
                       [context] * requests if phase == "decode" else [m])
        kv_tokens = context if phase == "decode" else m
        blocks = -(-kv_tokens // page_size)

        def caches_for(att, per_key):
            out = []
            for _ in range(_copies(requests * blocks * page_size * per_key)):
                cache = CacheManager([(att.cache_need(), None)], page_size, requests * blocks, requests, kv_tokens, bf, dev,
                                     prefix_cache=False)
                for g in cache.groups:
                    g.k.normal_(0, 0.5)
                    if g.v is not g.k:
                        g.v.normal_(0, 0.5)
                for _r in range(requests):
                    cache.ensure(cache.admit(None), kv_tokens)
                cache.sync_tables()
                out.append(cache)
            return out

        # ---- attention with normalised heads and a sink: norms + store, attention
        side = layer_of["attention"].mixer
        att = build_part("mixer", mixer_spec(cfg, layer_of["attention"], "bench"), rt)
        _fill(att)
        Hq, G, D = att.n_heads, att.n_kv_heads, att.head_dim
        seen = min(kv_tokens, side.window) if side.window else kv_tokens
        per_key = G * D * 2 * 2
        caches = caches_for(att, per_key)
        views = [c.view(0) for c in caches]
        projs = [torch.randn(m, att.qkv_width, device=dev, dtype=bf) for _ in range(_copies(m * att.qkv_width * 2) if phase == "prefill" else 1)]
        if phase == "decode":
            nbytes, flops = m * seen * per_key + m * (att.qkv_width + att.out_size) * 2, 2.0 * m * Hq * 2 * D * seen
        else:
            nbytes = m * (att.qkv_width * 2 + att.out_size) * 2 + m * per_key
            flops = 2.0 * Hq * 2 * D * (seen * (m - seen) + seen * (seen + 1) / 2)
        add(f"{phase}: attention over a window of {side.window}, normalised heads, sink", m,
            [(lambda v=v, i=i: att.attend(ctx, projs[i % len(projs)], v, True)) for i, v in enumerate(views)], nbytes, flops,
            reps=2 if phase == "prefill" else 4)
        del caches, views, projs, att
        torch.cuda.empty_cache()
        # ---- latent attention: norms + rotation + store + queries into the latent space; attention; value maps + gate
        side = layer_of["latent_attention"].mixer
        lat = build_part("mixer", mixer_spec(cfg, layer_of["latent_attention"], "bench"), rt)
        _fill(lat)
        Hq, Dl, C = lat.n_heads, lat.head_dim, lat.kv_rank
        seen = min(kv_tokens, side.window) if side.window else kv_tokens
        per_key = Dl * 2
        caches = caches_for(lat, per_key)
        views = [c.view(0) for c in caches]
        projs = [torch.randn(m, lat.in_width, device=dev, dtype=bf) for _ in range(_copies(m * lat.in_width * 2) if phase == "prefill" else 1)]
        maps = Hq * (lat.q_head * lat.q_rank + lat.q_head * Dl) * 2
        add(f"{phase}: latent norms + rotation + store, query product, rotation, queries into the latent space", m,
            [(lambda v=v, i=i: lat.prepare(ctx, projs[i % len(projs)], v, True)) for i, v in enumerate(views)],
            m * (lat.in_width + lat.q_rank + Dl + Hq * (2 * lat.q_head + Dl)) * 2 + maps,
            2.0 * m * Hq * lat.q_head * (lat.q_rank + Dl), note="the two products are the library's")
        ql = lat.prepare(ctx, projs[0], views[0], True).clone()
        outs = [torch.empty(m, lat.q_size, device=dev, dtype=bf) for _ in range(2)]
        if phase == "decode":
            nbytes, flops = m * seen * per_key + m * 2 * lat.q_size * 2, 2.0 * m * Hq * 2 * Dl * seen
        else:
            nbytes = m * (2 * lat.q_size + Dl) * 2
            flops = 2.0 * Hq * 2 * Dl * (seen * (m - seen) + seen * (seen + 1) / 2)
        add(f"{phase}: attention of {Hq} heads over cached rows of {Dl} values (keys and values at once), window {side.window}", m,
            [(lambda v=v, i=i: lat._attend(ctx, outs[i % 2], ql, v)) for i, v in enumerate(views)], nbytes, flops,
            reps=2 if phase == "prefill" else 4)
        del caches, views, projs, lat, ql, outs
        torch.cuda.empty_cache()
        # ---- gla: the recurrence, then the norm over heads with its gate
        side = layer_of["gla"].mixer
        H, Dk, Dv = side.heads, side.dim, side.vdim
        numel = ops.recurrence_state_numel(ops.RECURRENCE_GLA, H, Dk, Dv)
        sets = []
        for _ in range(_copies(max(requests * numel * 8, m * H * (2 * Dk + Dv) * 2))):
            q, k, v = (torch.randn(m, H * d, device=dev, dtype=bf) * 0.3 for d in (Dk, Dk, Dv))
            sets.append((q, k, v, torch.zeros(requests, numel, device=dev), torch.empty(m, H * Dv, device=dev),
                         torch.randn(m, H * Dk, device=dev)))
        bias = torch.full((H * Dk,), 3.0, device=dev)
        add(f"{phase}: gla recurrence, {H} heads of {Dk} x {Dv}", m,
            [(lambda s=s: ops.linear_recurrence(ops.RECURRENCE_GLA, s[4], None, s[0], s[1], s[2], s[3], positions, slots, starts, lens,
                                                requests, H, Dk, Dv, True, max_q_len=per, pre=s[5], p0=bias, q_scale=Dk ** -0.5,
                                                cap=1.0 / side.tau)) for s in sets],
            m * H * (2 * Dk + Dv) * 2 + m * H * Dv * 4 + 2 * requests * numel * 4 + m * H * Dk * 4, 0.0,
            reps=2 if phase == "prefill" else 8, note=f"{4.0 * m * H * Dk * Dv / 1e9:.2f} GFLOP of fp32 multiply-adds outside the tensor cores")
        del sets
        sets = [(torch.randn(m, H * Dv, device=dev), torch.randn(m, H * Dv, device=dev, dtype=bf), torch.empty(m, H * Dv, device=dev, dtype=bf))
                for _ in range(_copies(m * H * Dv * 8))]
        nw = torch.ones(H * Dv, device=dev)
        add(f"{phase}: norm over each head + gate", m,
            [(lambda r=r, g=g, o=o: ops.head_norm_gate(o, r, None, nw, g, ops.GATE_SILU, 1e-6, m, H, Dv)) for r, g, o in sets],
            m * H * Dv * 8, 0.0, reps=8)
        del sets
        # ---- routed experts with identity experts and the clamped activation
        mlp = layer_of["attention"].mlp
        parts = []
        for _ in range(_copies(mlp.experts * 3 * mlp.ff * W * 2) if phase == "decode" else 2):
            part = build_part("feed_forward", experts_spec(cfg, mlp), rt)
            _fill(part)
            part.w_router.normal_(0, 0.5)
            part.correction.normal_(0, 0.05)
            parts.append(part)
        hs = [torch.randn(m, W, device=dev, dtype=bf) for _ in range(4)]
        touched = min(mlp.experts, m * mlp.top)
        add(f"{phase}: router over {mlp.experts} + {mlp.identity} outputs, {mlp.top} chosen", m,
            [(lambda p=p, i=i: p.route(ctx, hs[i % 4])) for i, p in enumerate(parts)], m * W * 2 + (mlp.experts + mlp.identity) * W * 2, 0.0, reps=8)
        add(f"{phase}: the chosen experts' gate/up, clamped activation, down and the weighted sum", m,
            [(lambda p=p, i=i: p.forward(ctx, hs[i % 4])) for i, p in enumerate(parts)],
            touched * 3 * mlp.ff * W * 2 + m * W * 4, 2.0 * m * mlp.top * 3 * mlp.ff * W * mlp.experts / (mlp.experts + mlp.identity), reps=2,
            note="includes the router; bytes: the matrices of the experts a step of this size touches at most, once")
        del parts
        # ---- the norm that adds a scaled delta
        norm = build_part("norm", tw.PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps, "weight_name": ""}), rt)
        _fill(norm)
        sets = [(torch.randn(m, W, device=dev), torch.randn(m, W, device=dev, dtype=bf), torch.empty(m, W, device=dev, dtype=bf))
                for _ in range(_copies(m * W * 12))]
        add(f"{phase}: residual add of a scaled delta + RMSNorm", m,
            [(lambda r=r, d=d, o=o: norm.apply(ctx, o, r, d, m, delta_scale=cfg.residual_mult)) for r, d, o in sets],
            m * W * (4 + 2 + 4 + 2), 0.0, reps=8)
        del sets
        torch.cuda.empty_cache()
    if int(status) != 0:
        raise RuntimeError(f"a kernel reported status {int(status)} during the kernel table")
    return rows
