"""A plain, slow implementation of the Dugudra decoder: one function per mechanism, whole sequences, no cache, no
kernels, token-by-token loops where the design is a recurrence.  It shares no code with the engine and is what the
engine's parts and models are compared with.  ``w`` is a dict of tensors by checkpoint name, ``cfg`` the contents of
config.json.  Everything runs in the type of the tensors handed in (float64 for a sharp comparison).
"""
import json
import math
import struct
from pathlib import Path

import torch


# ---------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------
def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def stretched_rates(dims, base, scaling):
    """(turning rate of pair i for i < dims / 2, factor on cos and sin).  Without ``scaling``: base**(-2i/dims) and 1.
    With it, pairs that turn often over the ``original`` length keep their rate, pairs that turn rarely are slowed by
    ``factor``, with a linear ramp between the pairs that make ``fast`` and ``slow`` turns over that length."""
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


def rotate_neighbours(x, positions, rates, magnitude):
    """x [T, ..., dims]: values 2i and 2i + 1 form a pair that is turned by position * rates[i] and stretched."""
    T = x.shape[0]
    angle = positions.to(x.dtype).reshape(T, *([1] * (x.dim() - 1))) * torch.tensor(rates, dtype=x.dtype)
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * cos - v * sin
    out[..., 1::2] = v * cos + u * sin
    return out


def windowed_softmax(scores, window, sink):
    """scores [H, T, T] (query, key): weights over the keys 0 <= i - j < window; with ``sink`` the denominator also
    holds exp(0), a term without key or value."""
    T = scores.shape[-1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) & (i - j < window) if window is not None else (j <= i)
    scores = scores.masked_fill(~seen, float("-inf"))
    top = scores.max(-1, keepdim=True).values
    if sink:
        top = torch.clamp(top, min=0.0)
    e = torch.exp(scores - top)
    den = e.sum(-1, keepdim=True)
    if sink:
        den = den + torch.exp(-top)
    return e / den


# ---------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------
def mixer_attention(h, w, p, m, eps):
    """Grouped heads, every head of q and k normalised, no positions, a window, a sink of score 0."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms((h @ w[p + "q"].T).view(T, H, D), eps) * w[p + "q.norm"]
    k = rms((h @ w[p + "k"].T).view(T, G, D), eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).view(T, G, Dv)
    group = H // G
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    window = m["mask"]["size"] if m.get("mask") else None
    weights = windowed_softmax(scores, window, sink=True)
    out = torch.einsum("hij,jhd->ihd", weights, v).reshape(T, H * Dv)
    return out @ w[p + "o"].T


def mixer_latent_attention(h, w, p, m, eps, positions):
    """Queries and keys/values through low-rank latents; a rotated key part shared by all heads."""
    T = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :C], eps) * w[p + "dkv.norm"]
    k_rot = down[:, C:]
    rot = m["rot"]
    rates, magnitude = stretched_rates(rot["dims"], rot["base"], rot.get("scaling"))
    q_rot = rotate_neighbours(q_rot, positions, rates, magnitude)
    k_rot = rotate_neighbours(k_rot, positions, rates, magnitude)
    k_plain = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, Dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    window = m["mask"]["size"] if m.get("mask") else None
    weights = windowed_softmax(scores, window, sink=False)
    out = torch.einsum("hij,jhd->ihd", weights, v).reshape(T, H * Dv)
    out = out * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def gated_linear_recurrence(q, k, v, alpha):
    """q, k, alpha [T, H, D], v [T, H, Dv]: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t; S [D, Dv] starts at zero."""
    T, H, D = q.shape
    Dv = v.shape[-1]
    S = torch.zeros(H, D, Dv, dtype=q.dtype)
    out = torch.empty(T, H, Dv, dtype=q.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def mixer_gla(h, w, p, m, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, Dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).view(T, H, D) ** (1.0 / m["tau"])
    o = gated_linear_recurrence(q, k, v, alpha)
    o = (rms(o, eps) * w[p + "norm"]).reshape(T, H * Dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def mixer(kind, h, w, p, m, eps, positions):
    if kind == "attention":
        return mixer_attention(h, w, p, m, eps)
    if kind == "latent_attention":
        return mixer_latent_attention(h, w, p, m, eps, positions)
    if kind == "gla":
        return mixer_gla(h, w, p, m, eps)
    raise ValueError(f"unknown mixer {kind!r}")


# ---------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------
def expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, router):
    """(chosen [T, top], weights [T, top]): softmax over every router output, the choice by score + correction, the
    weights the plain scores times ``scale``."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    chosen = torch.topk(choice, router["top"], dim=-1).indices
    return chosen, torch.gather(s, 1, chosen) * router["scale"]


def mixture(h, w, p, mlp):
    router = mlp["router"]
    real = router["experts"]
    chosen, weights = route(h, w, p, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(chosen[t].tolist(), weights[t]):
            if e >= real:                      # an identity expert: the token itself
                out[t] += c * h[t]
            else:
                out[t] += c * expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    return out


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------
def forward(cfg, w, tokens, return_layers=False):
    """logits [T, vocab] of one sequence (and the residual rows behind every layer)."""
    eps = cfg["norm"]["eps"]
    mult = cfg.get("residual_mult", 1.0)
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = w["embed"][tokens] * (cfg.get("embedding") or {}).get("scale", 1.0)
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, eps) * w[p + "norm1"]
        x = x + mult * mixer(layer["type"], h, w, p + "mix.", layer["mixer"], eps, positions)
        if layer.get("mlp") is not None:
            h = rms(x, eps) * w[p + "norm2"]
            x = x + mult * mixture(h, w, p + "mlp.", layer["mlp"])
        layers.append(x.clone())
    y = rms(x, eps) * w["final.norm"]
    logits = y @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(layers)) if return_layers else logits


def read_folder(folder, dtype=torch.float64):
    """(config.json, tensors by name) of a model folder; bfloat16 and float32 tensors are widened to ``dtype``."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32}
    w = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).view(*info["shape"])
        w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w


def logits_of(folder, tokens, dtype=torch.float64) -> torch.Tensor:
    cfg, w = read_folder(folder, dtype)
    return forward(cfg, w, tokens)


def greedy(folder, prompt, steps):
    cfg, w = read_folder(folder, torch.float64)
    ids = list(prompt)
    for _ in range(steps):
        ids.append(int(torch.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
