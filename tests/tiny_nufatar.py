"""Tiny Nufatar configurations for the tests.  They differ from one another in every size and option: order of the two
layer kinds, layers with and without a feed-forward, a repeated range of layers (in the middle, at the start, a single
layer, none), head counts and groups on both sides, key and value sizes (equal, different, multiples of 16 and not),
rotated share of a head (part, all, none) with and without stretched frequencies, windows (short, longer than a page),
rows and reach of the distance tables, taps of the convolutions (down to one), inner sizes of the low-rank
projections, scales of the sum, vocabulary, eps.  The inner sizes and the rows of the distance table stand in the
configuration here (``decay_rank``, ``gate_rank``, ``bias_rows``) because it is written before any weights exist."""


def yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def rotated(heads, kv_heads, dim, vdim, scale, rot_dims, base, scaling=None):
    """The attention of a ``parallel_2`` layer."""
    rot = {"dims": rot_dims, "base": base}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}


def windowed(heads, kv_heads, dim, scale, window, rows, far):
    """The attention of a ``parallel`` layer: its values are its keys."""
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": window},
            "bias_max": far, "bias_rows": rows}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank=None, gate_rank=None):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    if decay_rank is not None:
        d.update(decay_rank=decay_rank, gate_rank=gate_rank)
    return d


def dense(ff):
    return {"kind": "dense", "ff": ff}


def parallel(lft, rgt, mlp=None):
    return {"type": "parallel", "mixer": {"left": lft, "right": rgt}, "mlp": mlp}


def parallel_2(lft, rgt, left_scale, right_scale, mlp=None):
    return {"type": "parallel_2", "mixer": {"left": lft, "right": rgt, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


# a repeated range in the middle (three passes), keys and values of different sizes, part of a head rotated with
# stretched frequencies, grouped heads on both sides, a layer without a feed-forward
NUFATAR_A = {
    "architecture": "Nufatar", "vocab": 150, "width": 64, "norm": {"eps": 1e-5},
    "layers": [parallel_2(rotated(4, 2, 16, 32, 0.3, 8, 1000.0, yarn(4.0, 64, 8.0, 2.0)), delta(4, 2, 16, 24, 4), 0.7, 1.4, dense(48)),
               parallel(windowed(4, 2, 16, 0.22, 9, 8, 30), delta(2, 1, 16, 8, 3, 6, 5), dense(40)),
               parallel_2(rotated(2, 1, 32, 16, 0.2, 32, 5e4), delta(3, 3, 8, 16, 2), 1.2, -0.5),
               parallel(windowed(2, 2, 32, 0.15, 20, 10, 16), delta(4, 2, 8, 8, 4, 3, 7), dense(24))],
    "loop": {"start": 1, "stop": 3, "times": 3},
}

# no repeated range; sizes no fast path takes (a width that is no multiple of 8, odd head sizes, an odd vocabulary),
# a convolution of one tap (no state of its own), no rotation at all in one layer
NUFATAR_B = {
    "architecture": "Nufatar", "vocab": 97, "width": 36, "norm": {"eps": 1e-6},
    "layers": [parallel(windowed(3, 1, 12, 0.3, 5, 6, 11), delta(3, 3, 5, 7, 1, 4, 2), dense(50)),
               parallel_2(rotated(5, 5, 12, 20, 0.4, 0, 10.0), delta(2, 1, 10, 6, 5), 2.0, 0.25),
               parallel_2(rotated(3, 1, 24, 24, 0.25, 12, 123.0, yarn(2.5, 16, 4.0, 0.5)), delta(1, 1, 24, 40, 3), 1.0, 1.0, dense(27))],
}

# sizes the tensor-core attention kernels take: key = value = 64 with the whole head rotated and plain frequencies,
# 32 with a part rotated and stretched frequencies; a window longer than a page; the whole model repeated twice
NUFATAR_C = {
    "architecture": "Nufatar", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
    "layers": [parallel_2(rotated(8, 2, 64, 64, 0.11, 64, 3e5), delta(2, 2, 32, 32, 4), 1.3, 0.6, dense(96)),
               parallel(windowed(4, 1, 64, 0.1, 40, 32, 128), delta(4, 1, 32, 16, 4, 16, 8), dense(64)),
               parallel_2(rotated(4, 4, 32, 32, 0.2, 16, 2e4, yarn(16.0, 32, 16.0, 1.0)), delta(2, 1, 64, 48, 2), 0.5, 0.5)],
    "loop": {"start": 0, "stop": 3, "times": 2},
}

# a single layer repeated four times and nothing else around it but one more layer; one head everywhere; a window of
# two; a distance table of two rows
NUFATAR_D = {
    "architecture": "Nufatar", "vocab": 53, "width": 40, "norm": {"eps": 1e-4},
    "layers": [parallel(windowed(1, 1, 8, 0.5, 2, 2, 3), delta(1, 1, 16, 24, 2, 1, 1)),
               parallel_2(rotated(1, 1, 40, 8, 0.3, 4, 50.0, yarn(1.0, 8, 2.0, 1.0)), delta(5, 1, 8, 8, 7), -1.0, 0.3, dense(16))],
    "loop": {"start": 0, "stop": 1, "times": 4},
}

# windows and distance tables that prompts of hundreds of tokens pass many times, on pages of 16 that the windows give back
NUFATAR_E = {
    "architecture": "Nufatar", "vocab": 300, "width": 96, "norm": {"eps": 1e-6},
    "layers": [parallel(windowed(4, 2, 64, 0.125, 70, 16, 60), delta(2, 2, 32, 32, 4, 8, 8), dense(48)),
               parallel_2(rotated(2, 1, 32, 64, 0.18, 16, 5e5, yarn(8.0, 128, 32.0, 1.0)), delta(3, 1, 16, 48, 3), 0.8, 1.2, dense(32)),
               parallel(windowed(2, 1, 32, 0.2, 150, 24, 400), delta(3, 3, 16, 16, 4, 4, 12))],
    "loop": {"start": 1, "stop": 3, "times": 2},
}

NUFATAR_CONFIGS = {"A": NUFATAR_A, "B": NUFATAR_B, "C": NUFATAR_C, "D": NUFATAR_D}
NUFATAR_PAGE = {"A": 8, "B": 4, "C": 16, "D": 2}
NUFATAR_SEEDS = {"A": 25, "B": 26, "C": 27, "D": 28}
NUFATAR_STD = {"A": 0.12, "B": 0.2, "C": 0.08, "D": 0.25}
