"""The Nufatar decoder as a ``ModelSpec``.

Every layer has one norm whose output both of its sub-layers read (block kind ``parallel_pre_norm``):
``x += mixer(norm(x)) + feed_forward(norm(x))``, the feed-forward optional.  A mixer puts softmax attention
(``gqa_attention``: windowed with a distance bias, a sink and keys as values, or causal with a partly rotated head
and YaRN-scaled frequencies) beside a gated delta rule (``gated_delta``) and sums the two (``weighted_sum``, with
each side normalised first in the one kind).  A range of layers may run several times in a row on the same tensors:
the schedule then names those layers again, each run with a cache and state of its own, and a learned vector per pass
(``loop.step``) is added to the stream ahead of the pass.  The norms' weights are stored around zero
(``x / rms * (1 + w)``); the output matrix is the embedding matrix.  Tensor names: ``embed``, ``final.norm``,
``loop.step``, and per layer i ``l<i>.norm1``, ``l<i>.mix.left|right.*``, ``l<i>.mlp.gate|up|down``.
"""
from __future__ import annotations

from ..config.nufatar_config import DeltaRuleConfig, NufatarConfig, NufatarLayer, SoftmaxAttentionConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry

NUFATAR_LAYER_NAMES = {"norm1": "norm1", "mixer": "mix", "feed_forward": "mlp"}
NO_POSITION_LIMIT = 2 ** 31 - 1        # the design has no table of positions; int32 positions bound a request


def attention_spec(cfg: NufatarConfig, m: SoftmaxAttentionConfig, where: str) -> PartSpec:
    params = {"hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "qkv_bias": False,
              "scale": m.scale, "window": m.window, "names": {"q": "q", "k": "k", "v": "v", "o": "o"}}
    if m.values_are_keys:
        params["values_are_keys"] = True
    else:
        params["v_head_dim"] = m.vdim
    if m.sink:
        params["sink"] = "sink"
    if m.bias_max is not None:
        if m.bias_rows is None:
            raise ValueError(f"{where}: the rows of the distance table are known neither from 'bias_rows' nor from a checkpoint")
        params["distance_bias"] = {"name": "rel", "rows": m.bias_rows, "far": m.bias_max}
    if m.rot is None:
        params["position"] = PartSpec("none", {})
    else:
        s = m.rot.scaling
        yarn = None if s is None else {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
        params["position"] = PartSpec("rope", {"theta": m.rot.base, "dims": m.rot.dims, "yarn": yarn})
    return PartSpec("gqa_attention", params)


def delta_rule_spec(cfg: NufatarConfig, m: DeltaRuleConfig, where: str) -> PartSpec:
    if m.channel_decay and m.decay_rank is None:
        raise ValueError(f"{where}: the inner size of the decay projection is known neither from 'decay_rank' nor from a checkpoint")
    if m.low_rank_gate and m.gate_rank is None:
        raise ValueError(f"{where}: the inner size of the gate projection is known neither from 'gate_rank' nor from a checkpoint")
    return PartSpec("gated_delta", {
        "hidden": cfg.width, "n_heads": m.heads, "n_qk_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim,
        "conv_taps": m.conv, "channel_decay": m.channel_decay, "decay_rank": m.decay_rank, "gate": m.gate,
        "gate_rank": m.gate_rank if m.low_rank_gate else None, "eps": cfg.norm_eps})


def mixer_spec(cfg: NufatarConfig, layer: NufatarLayer, where: str) -> PartSpec:
    m = layer.mixer
    params = {"hidden": cfg.width, "members": (
        ("left", attention_spec(cfg, m.left, f"{where}.left"), m.left_scale),
        ("right", delta_rule_spec(cfg, m.right, f"{where}.right"), m.right_scale))}
    if m.normalised:
        params.update(member_norm_eps=cfg.norm_eps, member_norm_name="out")
    return PartSpec("weighted_sum", params)


def nufatar_spec(cfg: NufatarConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": "", "unit_offset": True})
    layers = []
    for i, layer in enumerate(cfg.layers):
        params = {"hidden": cfg.width, "norm1": norm, "mixer": mixer_spec(cfg, layer, f"layers[{i}].mixer"),
                  "names": NUFATAR_LAYER_NAMES}
        if layer.mlp is not None:
            params["feed_forward"] = PartSpec("swiglu", {"hidden": cfg.width, "intermediate": layer.mlp.ff,
                                                         "names": ("gate", "up", "down")})
        layers.append(LayerSpec(PartSpec("parallel_pre_norm", params), f"l{i}"))
    n, loop = len(layers), cfg.loop
    if loop is None or loop.stop <= loop.start:      # (an empty range: the pass vectors are loaded and nothing reads them)
        schedule = [ScheduleEntry(i) for i in range(n)]
    else:
        schedule = [ScheduleEntry(i) for i in range(loop.start)]
        for t in range(loop.times):
            schedule += [ScheduleEntry(i, add_vector=t if i == loop.start else None) for i in range(loop.start, loop.stop)]
        schedule += [ScheduleEntry(i) for i in range(loop.stop, n)]
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
        schedule=tuple(schedule),
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "weight_name": ""}),
        embedding_prefix="embed", final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.width}), head_prefix="head",
        tie_word_embeddings=True, max_position_embeddings=NO_POSITION_LIMIT, eos_token_ids=cfg.eos_token_ids,
        pass_vectors=None if loop is None else ("loop.step", loop.times))


register_architecture("Nufatar", NufatarConfig, nufatar_spec)
