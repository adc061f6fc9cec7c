"""The Dugudra configuration gate and spec builder (no GPU): what is read from where, what is refused; and the plain
implementation against itself where a mechanism can be written two ways."""
import copy
import json

import pytest
import torch

import plain_dugudra as plain
import tessweave_engine_b200 as tw
from tessweave_engine_b200.config import ConfigError, resolve, resolve_folder
from tessweave_engine_b200.models import Model
from tessweave_engine_b200.parts import FixedState, PagedKV, Runtime
from tiny_dugudra import DUGUDRA_CONFIGS, DUGUDRA_E


def meta_model(cfg):
    typed, spec = resolve(cfg)
    return typed, spec, Model(spec, Runtime(torch.device("meta"), torch.float32), config=typed)


@pytest.mark.parametrize("name", list(DUGUDRA_CONFIGS) + ["E"])
def test_tensor_names_and_shapes(name):
    cfg = {**DUGUDRA_CONFIGS, "E": DUGUDRA_E}[name]
    typed, spec, model = meta_model(cfg)
    assert len(spec.layers) == len(spec.schedule) == len(cfg["layers"])
    decls = model.weight_decls()
    names = set(decls)
    width = cfg["width"]
    assert {"embed", "final.norm", "head"} <= names
    assert decls["embed"].shape == decls["head"].shape == (cfg["vocab"], width)
    for i, layer in enumerate(cfg["layers"]):
        p, m, mlp = f"l{i}", layer["mixer"], layer["mlp"]
        assert f"{p}.norm1" in names and (f"{p}.norm2" in names) == (mlp is not None)
        mine = {n[len(p) + 5:]: decls[n].shape for n in names if n.startswith(f"{p}.mix.")}
        if layer["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            assert mine == {"q": (H * D, width), "k": (G * D, width), "v": (G * Dv, width), "o": (width, H * Dv),
                            "q.norm": (D,), "k.norm": (D,)}
        elif layer["type"] == "latent_attention":
            H, D, R, Dv, Q, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            assert mine == {"dq": (Q, width), "dq.norm": (Q,), "uq": (H * (D + R), Q), "dkv": (C + R, width), "dkv.norm": (C,),
                            "uk": (H * D, C), "uv": (H * Dv, C), "g": (H * Dv, width), "o": (width, H * Dv)}
        else:
            H, D, Dv, r = m["heads"], m["dim"], m["vdim"], m["decay_rank"]
            assert mine == {"q": (H * D, width), "k": (H * D, width), "v": (H * Dv, width), "g": (H * Dv, width),
                            "o": (width, H * Dv), "norm": (Dv,), "a1": (r, width), "a2": (H * D, r), "a2.b": (H * D,)}
        if mlp is not None:
            E, I, F = mlp["router"]["experts"], mlp["router"]["identity"], mlp["expert"]["ff"]
            assert decls[f"{p}.mlp.router"].shape == (E + I, width) and decls[f"{p}.mlp.correction"].shape == (E + I,)
            assert f"{p}.mlp.e{E - 1}.gate" in names and f"{p}.mlp.e{E}.gate" not in names     # identity experts have no tensors
            assert decls[f"{p}.mlp.e0.up"].shape == (F, width) and decls[f"{p}.mlp.e0.down"].shape == (width, F)
            assert f"{p}.mlp.router.b" not in names


def test_cache_needs():
    """An attention layer keeps keys and values of its own sizes, a latent layer one row of kv_rank + rot_dim values per
    token that serves as key and value, a gla layer a matrix per head; windows are passed on to the cache manager."""
    cfg = DUGUDRA_CONFIGS["A"]
    _, spec, model = meta_model(cfg)
    needs = [n for n, _ in model.cache_needs()]
    assert needs[0] == PagedKV(1, 48, 9, None, values_are_keys=True)
    assert needs[1] == FixedState(2 * 16 * 8)
    assert needs[2] == PagedKV(2, 16, 7, 32)
    assert needs[4] == PagedKV(1, 32, 20, None, values_are_keys=True)
    assert model.cache_bytes_per_token(2) == 2 * (48 + 2 * (16 + 32) + 32 + 1 * (32 + 16))
    assert model.state_bytes_per_request() == 4 * (2 * 16 * 8 + 4 * 16 * 16)
    _, _, c = meta_model(DUGUDRA_CONFIGS["C"])
    assert [n.window for n, _ in c.cache_needs() if isinstance(n, PagedKV)] == [40, 24, None, None]


def test_constants_reach_the_parts():
    typed, spec, model = meta_model(DUGUDRA_CONFIGS["A"])
    cfg = DUGUDRA_CONFIGS["A"]
    assert model.embedding.scale == 8.0 and model.head.softcap == 10.0
    blocks = model.blocks
    assert all(b.residual_scale == 0.6 for b in blocks)
    lat, gla, att = blocks[0].mixer, blocks[1].mixer, blocks[2].mixer
    assert (lat.scale, lat.window, lat.kv_rank, lat.rot_dim, lat.eps) == (0.2, 9, 40, 8, 1e-5)
    assert lat.position.yarn == {"factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 2.0} and blocks[4].mixer.position.yarn is None
    assert (gla.tau, gla.decay_rank, gla.eps) == (4.0, 6, 1e-5)
    assert (att.scale, att.window, att.qk_norm["eps"]) == (0.3, 7, 1e-5) and att.sink is not None and att.sink_name is None
    ff = blocks[0].feed_forward
    assert (ff.experts, ff.identity, ff.top, ff.weight_scale, ff.glu_limit, ff.glu_alpha, ff.score_all) == (6, 2, 3, 2.0, 0.7, 1.702, True)
    _, _, b = meta_model(DUGUDRA_CONFIGS["B"])
    assert b.head.softcap is None and b.blocks[0].residual_scale == 1.0
    _, _, d = meta_model(DUGUDRA_CONFIGS["D"])
    assert d.embedding.scale == 1.0 and d.blocks[0].residual_scale == -0.5


def edit(cfg, path, value):
    cfg = copy.deepcopy(cfg)
    node = cfg
    for key in path[:-1]:
        node = node[key]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "mamba", "not implemented"),
    (("layers", 0, "mixer", "rot", "dims"), 4, "rot_dim"),
    (("layers", 0, "mixer", "rot_dim"), 7, "even"),
    (("layers", 0, "mixer", "kv_rank"), 1020, "not supported"),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), 0.0, "positive"),
    (("layers", 0, "mixer", "mask", "size"), 0, "positive"),
    (("layers", 0, "mlp", "kind"), "dense", "not implemented"),
    (("layers", 0, "mlp", "router", "top"), 9, "top exceeds"),
    (("layers", 0, "mlp", "expert", "limit"), -1.0, "positive"),
    (("layers", 1, "mixer", "tau"), 0.0, "positive"),
    (("layers", 1, "mixer", "heads"), KeyError, "heads"),
    (("layers", 2, "mixer", "kv_heads"), 3, "multiple"),
    (("layers", 2, "mixer", "dim"), 1300, "not supported"),
    (("norm", "eps"), 0.0, "positive"),
    (("logit_softcap",), -2.0, "positive"),
    (("width",), 0, "positive"),
    (("layers",), [], "non-empty"),
])
def test_what_the_gate_refuses(path, value, word):
    with pytest.raises(ConfigError) as e:
        resolve(edit(DUGUDRA_CONFIGS["A"], path, value))
    assert word in str(e.value)


def test_decay_rank_comes_from_the_checkpoint(tmp_path):
    """The inner size of the decay projection is read from the checkpoint's header; a configured one that contradicts
    it is refused; without either the model cannot be described."""
    cfg = DUGUDRA_CONFIGS["B"]
    folder = tw.write_random_model(tmp_path / "m", cfg, seed=1, std=0.1)
    stored = json.loads((folder / "config.json").read_text())
    bare = edit(stored, ("layers", 2, "mixer", "decay_rank"), KeyError)
    (folder / "config.json").write_text(json.dumps(bare))
    typed, spec = resolve_folder(folder)
    assert typed.layers[2].mixer.decay_rank == 3
    with pytest.raises(ValueError):
        resolve(bare)
    (folder / "config.json").write_text(json.dumps(edit(stored, ("layers", 2, "mixer", "decay_rank"), 5)))
    with pytest.raises(ConfigError):
        resolve_folder(folder)


def test_written_weights_are_read_back(tmp_path):
    """A folder written from a configuration holds every tensor the model declares, and the plain reader sees them."""
    cfg = DUGUDRA_CONFIGS["D"]
    folder = tw.write_random_model(tmp_path / "m", cfg, seed=3, std=0.2)
    _, w = plain.read_folder(folder, torch.float64)
    _, _, model = meta_model(cfg)
    assert set(w) == set(model.weight_decls())
    logits = plain.forward(json.loads((folder / "config.json").read_text()), w, [1, 5, 2, 40, 7])
    assert logits.shape == (5, 53) and bool(torch.isfinite(logits).all()) and float(logits.abs().max()) < 4.0    # the cap


def test_plain_latent_attention_in_the_latent_space():
    """The plain mixer expands every head's keys and values; scoring the queries against the latents themselves and
    applying the value map afterwards is the same function."""
    m = DUGUDRA_CONFIGS["A"]["layers"][0]["mixer"]
    H, D, R, Dv, Q, C, width, T = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"], 64, 31
    g = torch.Generator().manual_seed(5)
    shapes = {"dq": (Q, width), "dq.norm": (Q,), "uq": (H * (D + R), Q), "dkv": (C + R, width), "dkv.norm": (C,), "uk": (H * D, C),
              "uv": (H * Dv, C), "g": (H * Dv, width), "o": (width, H * Dv)}
    w = {"p." + k: torch.randn(s, generator=g, dtype=torch.float64) * 0.3 for k, s in shapes.items()}
    h = torch.randn(T, width, generator=g, dtype=torch.float64)
    pos = torch.arange(T)
    want = plain.mixer_latent_attention(h, w, "p.", m, 1e-5, pos)
    cq = plain.rms(h @ w["p.dq"].T, 1e-5) * w["p.dq.norm"]
    q = (cq @ w["p.uq"].T).view(T, H, D + R)
    down = h @ w["p.dkv"].T
    c = plain.rms(down[:, :C], 1e-5) * w["p.dkv.norm"]
    rates, mag = plain.stretched_rates(R, m["rot"]["base"], m["rot"]["scaling"])
    qr = plain.rotate_neighbours(q[..., D:], pos, rates, mag)
    kr = plain.rotate_neighbours(down[:, C:], pos, rates, mag)
    ql = torch.einsum("thd,hdc->thc", q[..., :D], w["p.uk"].view(H, D, C))
    scores = (torch.einsum("ihc,jc->hij", ql, c) + torch.einsum("ihr,jr->hij", qr, kr)) * m["scale"]
    p = plain.windowed_softmax(scores, m["mask"]["size"], sink=False)
    mixed = torch.einsum("hij,jc->ihc", p, c)
    out = torch.einsum("ihc,hvc->ihv", mixed, w["p.uv"].view(H, Dv, C)).reshape(T, H * Dv)
    got = (out * torch.sigmoid(h @ w["p.g"].T)) @ w["p.o"].T
    assert float((got - want).abs().max()) < 1e-10


def test_plain_windowed_softmax_with_sink():
    s = torch.tensor([[[0.0, 9.0, 9.0], [1.0, 2.0, 9.0], [5.0, -1.0, 0.5]]], dtype=torch.float64)
    p = plain.windowed_softmax(s, 2, sink=True)
    assert torch.allclose(p[0, 0], torch.tensor([0.5, 0.0, 0.0], dtype=torch.float64))
    e1, e2 = torch.exp(torch.tensor(1.0, dtype=torch.float64)), torch.exp(torch.tensor(2.0, dtype=torch.float64))
    assert torch.allclose(p[0, 1], torch.stack([e1, e2, torch.tensor(0.0, dtype=torch.float64)]) / (1 + e1 + e2))
    assert float(p[0, 2, 0]) == 0.0 and abs(float(p[0, 2].sum()) - (1 - 1 / (1 + torch.exp(torch.tensor(-1.0)) + torch.exp(torch.tensor(0.5))))) < 1e-6
