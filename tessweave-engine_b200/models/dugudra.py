"""The Dugudra decoder as a ``ModelSpec``.

Pre-norm layers that differ from one another and join the residual stream through one constant factor; a layer's
mixer is ``gqa_attention`` with normalised heads, no positions and a constant sink, ``latent_attention`` with a
stretched rotation of neighbouring pairs, or ``gla``; its feed-forward, where it has one, is ``routed_experts`` with
scores over every router output, a correction of the choice, identity experts and the clamped activation.  The
embedding rows are scaled and the logits capped.  Tensor names: ``embed``, ``final.norm``, ``head``, and per layer i
``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.router|correction|e<j>.gate|up|down``.
"""
from __future__ import annotations

from ..config.dugudra_config import (DugudraConfig, DugudraLayer, ExpertsConfig, GlaConfig, LatentAttentionConfig,
                                     NormedAttentionConfig)
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry

DUGUDRA_LAYER_NAMES = {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp"}
ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o"}
EXPERT_SWISH = 1.702                   # the design's constant in an expert's activation
NO_POSITION_LIMIT = 2 ** 31 - 1        # the design has no table of positions; int32 positions bound a request


def mixer_spec(cfg: DugudraConfig, layer: DugudraLayer, where: str) -> PartSpec:
    m = layer.mixer
    if isinstance(m, NormedAttentionConfig):
        return PartSpec("gqa_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
            "qkv_bias": False, "scale": m.scale, "window": m.window, "names": ATTENTION_NAMES, "position": PartSpec("none"),
            "sink_value": 0.0, "qk_norm": {"q": "q.norm", "k": "k.norm", "eps": cfg.norm_eps}})
    if isinstance(m, LatentAttentionConfig):
        position = PartSpec("rope_interleaved", {"theta": m.rot_base, "dims": m.rot_dim,
                                                 "yarn": None if m.stretch is None else m.stretch.as_dict()})
        return PartSpec("latent_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
            "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "window": m.window,
            "position": position, "output_gate": True})
    if isinstance(m, GlaConfig):
        if m.decay_rank is None:
            raise ValueError(f"{where}: the inner size of the decay projection is known neither from 'decay_rank' nor from a checkpoint")
        return PartSpec("gla", {"hidden": cfg.width, "n_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
                                "decay_rank": m.decay_rank, "tau": m.tau, "eps": cfg.norm_eps})
    raise TypeError(f"no part for mixer configuration {m!r}")


def experts_spec(cfg: DugudraConfig, mlp: ExpertsConfig) -> PartSpec:
    return PartSpec("routed_experts", {
        "hidden": cfg.width, "experts": mlp.experts, "top": mlp.top, "intermediate": mlp.ff, "router_bias": False,
        "score_all": True, "correction": "correction", "weight_scale": mlp.scale, "identity": mlp.identity,
        "activation": {"kind": "clamped", "limit": mlp.limit, "alpha": EXPERT_SWISH}})


def dugudra_spec(cfg: DugudraConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": ""})
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        params = {"hidden": cfg.width, "norm1": norm, "mixer": mixer_spec(cfg, layer, f"layers[{i}]"),
                  "names": DUGUDRA_LAYER_NAMES, "residual_scale": cfg.residual_mult}
        if layer.mlp is not None:
            params["norm2"] = norm
            params["feed_forward"] = experts_spec(cfg, layer.mlp)
        layers.append(LayerSpec(PartSpec("pre_norm", params), f"l{i}"))
        schedule.append(ScheduleEntry(i))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
        schedule=tuple(schedule),
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "weight_name": "",
                                               "scale": cfg.embedding_scale}),
        embedding_prefix="embed", final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.width, "weight_name": "",
                                      "softcap": cfg.logit_softcap}), head_prefix="head",
        tie_word_embeddings=False, max_position_embeddings=NO_POSITION_LIMIT, eos_token_ids=cfg.eos_token_ids)


register_architecture("Dugudra", DugudraConfig, dugudra_spec)
