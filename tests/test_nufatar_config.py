"""The Nufatar configuration gate and spec builder (no GPU): what is read from where, what is refused."""
import copy
import json

import pytest
import torch

import plain_nufatar as plain
import tessweave_engine_b200 as tw
from tessweave_engine_b200.config import ConfigError, resolve, resolve_folder
from tessweave_engine_b200.models import Model
from tessweave_engine_b200.parts import FixedState, PagedKV, Runtime, SeveralNeeds
from tessweave_engine_b200.parts.attention import GQAAttention
from tiny_nufatar import NUFATAR_CONFIGS, NUFATAR_E


def meta_model(cfg):
    typed, spec = resolve(cfg)
    return typed, spec, Model(spec, Runtime(torch.device("meta"), torch.float32), config=typed)


@pytest.mark.parametrize("name", list(NUFATAR_CONFIGS) + ["E"])
def test_tensor_names_and_schedule(name):
    cfg = {**NUFATAR_CONFIGS, "E": NUFATAR_E}[name]
    typed, spec, model = meta_model(cfg)
    runs = plain.layer_runs(cfg)
    assert len(spec.layers) == len(cfg["layers"]) and len(spec.schedule) == len(runs)
    for entry, (layer, new_pass) in zip(spec.schedule, runs):
        assert (entry.layer, entry.add_vector, entry.cache_of) == (layer, new_pass, None)
    names = set(model.weight_decls())
    assert {"embed", "final.norm"} <= names and ("loop.step" in names) == ("loop" in cfg)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        assert f"{p}.norm1" in names and f"{p}.norm2" not in names
        assert ({f"{p}.mlp.gate", f"{p}.mlp.up", f"{p}.mlp.down"} <= names) == (layer["mlp"] is not None)
        assert {f"{p}.mix.left.q", f"{p}.mix.left.k", f"{p}.mix.left.o", f"{p}.mix.right.q.conv", f"{p}.mix.right.k.conv",
                f"{p}.mix.right.v.conv", f"{p}.mix.right.b", f"{p}.mix.right.A_log", f"{p}.mix.right.dt_bias",
                f"{p}.mix.right.norm", f"{p}.mix.right.o"} <= names
        windowed = layer["type"] == "parallel"
        for tensor in ("left.rel", "left.sink", "left.out", "right.out", "right.a1", "right.a2", "right.g1", "right.g2"):
            assert (f"{p}.mix.{tensor}" in names) == windowed, tensor
        for tensor in ("left.v", "right.a", "right.g"):
            assert (f"{p}.mix.{tensor}" in names) == (not windowed), tensor
    decls = model.weight_decls()
    if "loop" in cfg:
        assert decls["loop.step"].shape == (cfg["loop"]["times"], cfg["width"])
    i = next(i for i, layer in enumerate(cfg["layers"]) if layer["type"] == "parallel")
    m = cfg["layers"][i]["mixer"]
    assert decls[f"l{i}.mix.left.rel"].shape == (m["left"]["bias_rows"], m["left"]["heads"])
    assert decls[f"l{i}.mix.right.dt_bias"].shape == (m["right"]["heads"] * m["right"]["dim"],)
    assert decls[f"l{i}.mix.right.a2"].shape == (m["right"]["heads"] * m["right"]["dim"], m["right"]["decay_rank"])


def test_cache_needs_of_every_run():
    """Every run of a repeated layer has pages and a state slot of its own; values that are the keys cost no pages
    of their own; the state holds the matrices and, behind them, the convolutions' last inputs."""
    cfg = NUFATAR_CONFIGS["A"]
    _, spec, model = meta_model(cfg)
    needs = [n for n, _ in model.cache_needs()]
    assert len(needs) == len(spec.schedule) == 1 + 3 * 2 + 1
    assert needs[0] == SeveralNeeds((PagedKV(2, 16, None, 32), FixedState(4 * 16 * 24 + (2 * 2 * 16 + 4 * 24) * 3)))
    windowed = SeveralNeeds((PagedKV(2, 16, 9, None, values_are_keys=True), FixedState(2 * 16 * 8 + (2 * 16 + 2 * 8) * 2)))
    assert needs[1] == needs[3] == needs[5] == windowed
    assert needs[2] == needs[4] == needs[6] == SeveralNeeds((PagedKV(1, 32, None, 16), FixedState(3 * 8 * 16 + (2 * 3 * 8 + 3 * 16))))
    per_token = 2 * (16 + 32) + 3 * 2 * 16 + 3 * (32 + 16) + 2 * 32
    assert model.cache_bytes_per_token(2) == 2 * per_token
    assert model.state_bytes_per_request() == 4 * sum(n.needs[1].numel for n in needs)


def test_a_convolution_of_one_tap_keeps_nothing():
    _, _, model = meta_model(NUFATAR_CONFIGS["B"])
    needs = [n for n, _ in model.cache_needs()]
    assert needs[0].needs[1] == FixedState(3 * 5 * 7)


def test_sizes_the_file_lacks_come_from_the_checkpoint(tmp_path):
    cfg = copy.deepcopy(NUFATAR_CONFIGS["A"])
    folder = tw.write_random_model(tmp_path / "m", cfg, seed=1)
    written = json.loads((folder / "config.json").read_text())
    for key in ("decay_rank", "gate_rank"):
        del written["layers"][1]["mixer"]["right"][key]
    del written["layers"][1]["mixer"]["left"]["bias_rows"]
    (folder / "config.json").write_text(json.dumps(written))
    typed, _ = resolve_folder(folder)
    assert (typed.layers[1].mixer.right.decay_rank, typed.layers[1].mixer.right.gate_rank) == (6, 5)
    assert typed.layers[1].mixer.left.bias_rows == 8
    with pytest.raises(ValueError):
        resolve(written)                                     # neither the keys nor a checkpoint
    written["layers"][1]["mixer"]["left"]["bias_rows"] = 9
    (folder / "config.json").write_text(json.dumps(written))
    with pytest.raises(ConfigError):
        resolve_folder(folder)


def test_an_empty_or_absent_loop_runs_every_layer_once():
    cfg = copy.deepcopy(NUFATAR_CONFIGS["A"])
    cfg["loop"] = {"start": 2, "stop": 2, "times": 5}
    _, spec, model = meta_model(cfg)
    assert [(e.layer, e.add_vector) for e in spec.schedule] == [(i, None) for i in range(4)]
    assert model.weight_decls()["loop.step"].shape == (5, cfg["width"])      # in the file, read by nothing
    del cfg["loop"]
    _, spec, model = meta_model(cfg)
    assert len(spec.schedule) == 4 and "loop.step" not in model.weight_decls()
    cfg["loop"] = {"start": 0, "stop": 4, "times": 1}
    _, spec, _ = meta_model(cfg)
    assert [(e.layer, e.add_vector) for e in spec.schedule] == [(0, 0), (1, None), (2, None), (3, None)]


@pytest.mark.parametrize("rows,far", [(16, 120), (8, 30), (2, 3), (6, 11), (32, 128), (10, 16), (24, 400), (7, 9.5), (5, 1000)])
def test_distance_buckets(rows, far):
    """One row per distance below half the table, then rows that widen; everything from ``far`` on reads the last."""
    half = rows // 2
    got = [GQAAttention.distance_bucket(n, rows, far) for n in range(int(far) * 3 + 5)]
    assert got == [plain.distance_bucket(n, rows, far) for n in range(len(got))]
    assert got[:half] == list(range(half)) and got[half] == half
    assert all(b >= a for a, b in zip(got, got[1:])) and got[-1] == rows - 1
    assert all(b == rows - 1 for n, b in enumerate(got) if n >= far)


def broken(change):
    cfg = copy.deepcopy(NUFATAR_CONFIGS["A"])
    change(cfg)
    return cfg


@pytest.mark.parametrize("change", [
    lambda c: c["layers"][0].update(type="parallel_3"),
    lambda c: c["layers"][0]["mlp"].update(kind="moe"),
    lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18),
    lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7),
    lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("fast"),
    lambda c: c["layers"][0]["mixer"]["left"].update(mask={"size": 4}),          # a window is not part of this kind
    lambda c: c["layers"][0]["mixer"].pop("left_scale"),
    lambda c: c["layers"][0]["mixer"]["right"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"]["right"].update(conv=0),
    lambda c: c["layers"][1]["mixer"]["left"].pop("mask"),
    lambda c: c["layers"][1]["mixer"]["left"].update(vdim=24),                   # the values are the keys
    lambda c: c["loop"].update(stop=5),
    lambda c: c["loop"].update(times=0),
    lambda c: c["norm"].update(eps=0.0),
    lambda c: c.pop("width"),
])
def test_the_gate_refuses(change):
    with pytest.raises(ConfigError):
        resolve(broken(change))


def test_heads_beyond_the_kernels_are_refused():
    with pytest.raises(ValueError):
        meta_model(broken(lambda c: c["layers"][1]["mixer"]["left"].update(bias_max=2)))      # not beyond half the table
    with pytest.raises(ConfigError):
        resolve(broken(lambda c: c["layers"][0]["mixer"]["right"].update(dim=512)))
    with pytest.raises(ConfigError):
        resolve(broken(lambda c: c["layers"][0]["mixer"]["left"].update(dim=260, rot={"dims": 0, "base": 10.0})))
