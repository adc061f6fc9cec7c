"""Tiny Dugudra configurations for the tests.  They differ from one another in every size and option: order of the three
layer kinds, layers with and without a feed-forward, head counts and groups, key and value sizes (equal, different,
multiples of 16 and not), latent sizes, size of the rotated part with and without stretched rates, windows (short,
longer than a page, none), decay exponents, numbers of experts, identity experts (none, fewer and more than are chosen)
and chosen experts, limits and scales of the experts, the factor on the residual, with and without a cap on the
logits, vocabulary, eps.  The inner size of a gla layer's decay projection stands in the configuration here
(``decay_rank``) because it is written before any weights exist."""


def yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def moe(experts, identity, top, ff, limit, scale):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}


def attention(heads, kv_heads, dim, vdim, scale, window=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, window=None, scaling=None, mlp=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling is not None:
        rot["scaling"] = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def gla(heads, dim, vdim, tau, rank, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}, "mlp": mlp}


# every kind twice, latent first; value sizes that differ from key sizes; a layer without a feed-forward
DUGUDRA_A = {
    "architecture": "Dugudra", "vocab": 150, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
    "residual_mult": 0.6, "logit_softcap": 10.0,
    "layers": [latent(3, 16, 8, 24, 20, 40, 0.2, 1000.0, 9, yarn(4.0, 64, 8.0, 2.0), moe(6, 2, 3, 40, 0.7, 2.0)),
               gla(2, 16, 8, 4.0, 6, moe(4, 1, 2, 24, 1.5, 1.0)),
               attention(4, 2, 16, 32, 0.3, 7),
               gla(4, 16, 16, 9.0, 3, moe(5, 3, 2, 16, 0.5, 0.8)),
               latent(2, 8, 8, 8, 24, 24, 0.25, 5e4, 20, None, moe(3, 0, 3, 32, 2.0, 1.3)),
               attention(2, 1, 32, 16, 0.15, 20, moe(6, 2, 3, 40, 0.7, 2.0))],
}

# sizes no fast path takes: a width that is no multiple of 8, odd head, latent and feed-forward sizes, an odd vocabulary;
# no identity experts, one chosen expert; no cap on the logits; the residual factor left out (1)
DUGUDRA_B = {
    "architecture": "Dugudra", "vocab": 97, "width": 36, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0}, "logit_softcap": None,
    "layers": [attention(3, 1, 12, 20, 0.3, 5, moe(3, 0, 1, 9, 1.0, 1.0)),
               latent(5, 6, 2, 7, 5, 11, 0.4, 10.0, 3, None, moe(5, 1, 2, 27, 0.9, 0.5)),
               gla(3, 10, 6, 1.0, 3)],
}

# sizes the tensor-core attention kernels take (64, 32; cached rows of 64), windows longer than a page and none
DUGUDRA_C = {
    "architecture": "Dugudra", "vocab": 211, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.3},
    "residual_mult": 0.8, "logit_softcap": 30.0,
    "layers": [attention(8, 2, 64, 64, 0.11, 40, moe(8, 1, 2, 48, 1.0, 1.5)),
               latent(4, 48, 16, 32, 64, 48, 0.14, 3e4, 24, yarn(16.0, 32, 16.0, 1.0), moe(4, 4, 4, 32, 3.0, 1.0)),
               gla(2, 32, 32, 16.0, 8),
               attention(4, 4, 32, 32, 0.2, None),
               latent(8, 16, 16, 16, 32, 16, 0.2, 100.0, None, yarn(2.0, 16, 4.0, 0.5), moe(8, 1, 2, 48, 1.0, 1.5))],
}

# one head everywhere, windows of two, more identity experts than real ones and every output chosen but one, a
# negative residual factor, no embedding factor
DUGUDRA_D = {
    "architecture": "Dugudra", "vocab": 53, "width": 40, "norm": {"eps": 1e-4}, "residual_mult": -0.5, "logit_softcap": 4.0,
    "layers": [gla(1, 16, 24, 2.0, 1, moe(2, 3, 4, 16, 0.25, 1.0)),
               latent(1, 8, 4, 8, 8, 12, 0.3, 50.0, 2, yarn(1.0, 8, 2.0, 1.0)),
               attention(1, 1, 8, 8, 0.5, 2, moe(2, 3, 4, 16, 0.25, 1.0))],
}

# windows that prompts of hundreds of tokens pass many times, on pages of 16 that the windows give back on the way
DUGUDRA_E = {
    "architecture": "Dugudra", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 9.8},
    "residual_mult": 0.75, "logit_softcap": 12.0,
    "layers": [attention(4, 2, 64, 64, 0.125, 70, moe(6, 2, 2, 32, 1.0, 1.5)),
               latent(4, 32, 16, 16, 48, 64, 0.14, 5e3, 150, yarn(8.0, 128, 32.0, 1.0), moe(6, 2, 2, 32, 1.0, 1.2)),
               gla(3, 32, 48, 16.0, 8)],
}

DUGUDRA_CONFIGS = {"A": DUGUDRA_A, "B": DUGUDRA_B, "C": DUGUDRA_C, "D": DUGUDRA_D}
DUGUDRA_PAGE = {"A": 8, "B": 4, "C": 16, "D": 2}
DUGUDRA_SEEDS = {"A": 35, "B": 36, "C": 37, "D": 38}
DUGUDRA_STD = {"A": 0.12, "B": 0.2, "C": 0.08, "D": 0.25}
