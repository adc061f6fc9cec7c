"""A plain, slow implementation of the Nufatar decoder: one function per mechanism, whole sequences, no cache, no
kernels, token-by-token loops where the design is a recurrence.  It shares no code with the engine and is what the
engine's parts and models are compared with.  ``w`` is a dict of tensors by checkpoint name, ``cfg`` the contents of
config.json.  Everything runs in the type of the tensors handed in (float64 for a sharp comparison).
"""
import math

import torch


# ---------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------
def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.clamp(x, min=0) + torch.log1p(torch.exp(-x.abs()))


def unit(x, eps=1e-6):
    """x / sqrt(sum(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def distance_bucket(n, rows, far):
    """The row of a distance table that distance n >= 0 reads: one row per distance below rows // 2, then rows that
    widen logarithmically until ``far``, and the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def stretched_frequencies(dims, base, scaling):
    """(turning rate of pair i for i < dims / 2, factor on cos and sin).  ``scaling`` None: base**(-2i/dims) and 1.
    Else the YaRN rule: pairs that turn often over the ``original`` length keep their rate, pairs that turn rarely
    are slowed by ``factor``, with a linear ramp between the pairs that make ``fast`` and ``slow`` turns."""
    rates = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling is None:
        return rates, 1.0
    factor = scaling["factor"]

    def pair_with_turns(t):
        return dims * math.log(scaling["original"] / (2 * math.pi * t)) / (2 * math.log(base))

    lo = max(math.floor(pair_with_turns(scaling["fast"])), 0)
    hi = min(math.ceil(pair_with_turns(scaling["slow"])), dims - 1)
    out = []
    for i, f in enumerate(rates):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_front(x, positions, dims, rates, magnitude):
    """x [T, H, D]: value i < dims / 2 of a head is paired with value i + dims / 2 and the pair is turned by
    position * rates[i], then stretched by ``magnitude``; values from ``dims`` on stay."""
    if dims == 0:
        return x
    half = dims // 2
    angle = positions.to(x.dtype)[:, None, None] * torch.tensor(rates, dtype=x.dtype)
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def short_convolution(x, taps):
    """x [T, C], taps [C, n]: y[t] = sum_j taps[:, j] * x[t - (n - 1) + j], rows before the first count as zero."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x])
    return sum(padded[j:j + T] * taps[:, j] for j in range(n))


# ---------------------------------------------------------------------------
# token mixing, each on tensors that are already projected
# ---------------------------------------------------------------------------
def softmax_attention(q, k, v, scale, window=None, bias_by_distance=None, sink=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; query head h reads key/value head h // (H / G); token t sees the
    tokens t - window + 1 .. t (all up to t without a window).  ``bias_by_distance`` [T, H]: added to the scaled
    score by t - j.  ``sink`` [H]: exp(sink[h]) joins the denominator and nothing else."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (k[lo:t + 1, g] @ q[t, h]) * scale
            if bias_by_distance is not None:
                s = s + bias_by_distance[t - torch.arange(lo, t + 1), h]
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() if sink is None else e.sum() + torch.exp(sink[h] - m)
            out[t, h] = (e / den) @ v[lo:t + 1, g]
    return out


def delta_rule(q, k, v, beta, decay):
    """q, k [T, H, Dk], v [T, H, Dv], beta [T, H], decay [T, H, Dk] (or [T, H, 1]): per head a matrix S [Dk, Dv], zero
    at the start, that first decays row by row, is then corrected towards v along k, and is read with q."""
    T, H, Dk = q.shape
    S = torch.zeros(H, Dk, v.shape[2], dtype=q.dtype)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S = S * decay[t][:, :, None]
        held = torch.einsum("hkv,hk->hv", S, k[t])
        S = S + k[t][:, :, None] * (beta[t][:, None] * (v[t] - held))[:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


# ---------------------------------------------------------------------------
# mixers: h [T, width] -> [T, width]
# ---------------------------------------------------------------------------
def mixer_attention(h, w, p, m, positions):
    """Softmax attention.  Without a tensor ``p.v`` the values are the keys as projected.  ``m["rot"]``: a rotation of
    the front of every query and key head.  ``m["mask"]["size"]``: a sliding window.  ``m["bias_max"]``: the table
    ``p.rel`` [rows, H] by bucketed distance on the scores, and the sink ``p.sink`` [H] in the denominator."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[f"{p}.q"].T).view(T, H, D)
    k = (h @ w[f"{p}.k"].T).view(T, G, D)
    v = (h @ w[f"{p}.v"].T).view(T, G, m["vdim"]) if f"{p}.v" in w else k
    rot = m.get("rot")
    if rot is not None:
        rates, magnitude = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot["dims"] else ([], 1.0)
        q, k = (rotate_front(x, positions, rot["dims"], rates, magnitude) for x in (q, k))
    window = m["mask"]["size"] if m.get("mask") else None
    bias = sink = None
    if m.get("bias_max") is not None:
        table = w[f"{p}.rel"]
        bias = torch.stack([table[distance_bucket(n, table.shape[0], m["bias_max"])] for n in range(T)])
        sink = w[f"{p}.sink"]
    o = softmax_attention(q, k, v, m["scale"], window, bias, sink)
    return o.reshape(T, -1) @ w[f"{p}.o"].T


def mixer_delta(h, w, p, m, eps):
    """The gated delta rule.  With ``p.a1`` / ``p.a2`` the decay has a value per key channel (through two matrices),
    else one per head (``p.a``); with ``p.g1`` / ``p.g2`` the output gate is a sigmoid of two matrices' product, else
    silu of ``p.g``."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (silu(short_convolution(h @ w[f"{p}.{n}"].T, w[f"{p}.{n}.conv"])) for n in "qkv")
    q = (unit(q.view(T, G, D)) * D ** -0.5).repeat_interleave(H // G, dim=1)
    k = unit(k.view(T, G, D)).repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ w[f"{p}.b"].T)
    rate = torch.exp(w[f"{p}.A_log"])
    if f"{p}.a1" in w:
        step = softplus(((h @ w[f"{p}.a1"].T) @ w[f"{p}.a2"].T + w[f"{p}.dt_bias"]).view(T, H, D))
        decay = torch.exp(-rate[None, :, None] * step)
    else:
        decay = torch.exp(-rate * softplus(h @ w[f"{p}.a"].T + w[f"{p}.dt_bias"]))[:, :, None]
    if f"{p}.g1" in w:
        gate = torch.sigmoid((h @ w[f"{p}.g1"].T) @ w[f"{p}.g2"].T)
    else:
        gate = silu(h @ w[f"{p}.g"].T)
    o = delta_rule(q, k, v.view(T, H, Dv), beta, decay)
    o = rms(o, eps) * w[f"{p}.norm"]
    return (o.reshape(T, -1) * gate) @ w[f"{p}.o"].T


def mixer(kind, h, w, p, m, eps, positions):
    """Attention (``left``) beside the delta rule (``right``) on the same rows.  ``parallel``: each result is
    normalised over the width and weighted, and the two are averaged.  ``parallel_2``: a sum with two scales."""
    a = mixer_attention(h, w, f"{p}.left", m["left"], positions)
    b = mixer_delta(h, w, f"{p}.right", m["right"], eps)
    if kind == "parallel":
        return 0.5 * (rms(a, eps) * w[f"{p}.left.out"] + rms(b, eps) * w[f"{p}.right.out"])
    if kind == "parallel_2":
        return m["left_scale"] * a + m["right_scale"] * b
    raise ValueError(kind)


def feed_forward(h, w, p):
    return (silu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------
def layer_runs(cfg):
    """[(layer, pass number or None)]: the order in which layers run; the pass number stands at a pass's first layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the stream behind every layer run)."""
    dtype = w["embed"].dtype
    eps = cfg["norm"]["eps"]
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.tensor(tokens)]
    after = []
    for i, new_pass in layer_runs(cfg):
        layer = cfg["layers"][i]
        if new_pass is not None:
            x = x + w["loop.step"][new_pass]
        h = rms(x, eps) * (1 + w[f"l{i}.norm1"])
        d = mixer(layer["type"], h, w, f"l{i}.mix", layer["mixer"], eps, positions)
        if layer.get("mlp") is not None:
            d = d + feed_forward(h, w, f"l{i}.mlp")
        x = x + d
        after.append(x)
    logits = (rms(x, eps) * (1 + w["final.norm"])) @ w["embed"].T
    assert logits.dtype == dtype
    return (logits, torch.stack(after)) if return_layers else logits


# ---------------------------------------------------------------------------
# model folders
# ---------------------------------------------------------------------------
def read_folder(folder, dtype=torch.float32):
    """config.json and every tensor of model.safetensors, read with nothing but slicing and torch."""
    import json
    from pathlib import Path
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    n = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32}
    weights = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=kinds[meta["dtype"]]).view(meta["shape"])
        weights[name] = t.to(dtype) if t.is_floating_point() else t
    return config, weights


def logits_of(folder, tokens, dtype=torch.float64) -> torch.Tensor:
    config, weights = read_folder(folder, dtype)
    return forward(config, weights, tokens).float()


def greedy(folder, prompt, steps):
    """Greedy continuation, the slow way: the whole sequence again for every token (lowest index at a tie)."""
    config, weights = read_folder(folder, torch.float64)
    tokens, out = list(prompt), []
    for _ in range(steps):
        nxt = int(torch.argmax(forward(config, weights, tokens)[-1]))
        out.append(nxt)
        tokens.append(nxt)
    return out
