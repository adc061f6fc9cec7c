"""Typed view of a Dugudra ``config.json``.

The file names the design under ``architecture`` and gives the residual width, the vocabulary, the norms' eps, the
factor on the embedding rows, the factor with which every sub-layer joins the residual stream (``residual_mult``),
the cap of the logits, and a list of layers.  A layer names its mixer by ``type`` -- ``attention`` (grouped heads,
normalised queries and keys, no positions, a window, one added to the softmax's denominator), ``latent_attention``
(queries and keys/values through low-rank latents, a rotated key part shared by the heads, stretched rotation rates,
a window, a sigmoid output gate) or ``gla`` (gated linear attention with a decay per key channel) -- with the mixer's
sizes and constants under ``mixer``, and its feed-forward under ``mlp`` (``moe`` or null).  Every size and constant
comes from here; the one size the file does not give, the inner size of a gla layer's decay projection, is read from
the checkpoint's tensor shapes (or from the key ``decay_rank`` where a configuration is written before its weights
exist).  Anything this engine does not implement is refused before a weight is read.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, replace
from pathlib import Path

from .linurax_config import _finite, _need, _positive_int
from .model_config import ConfigError
from .sapatar_config import safetensors_shapes

MAX_HEAD = 1024         # the attention kernels' largest head (above 256: the exact kernel alone)


def _window(d: dict, where: str) -> int | None:
    mask = d.get("mask")
    return None if mask is None else _positive_int(_need(mask, "size", f"{where}.mask"), f"{where}.mask.size")


@dataclass(frozen=True)
class NormedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "NormedAttentionConfig":
        cfg = cls(heads=_positive_int(_need(d, "heads", where), f"{where}.heads"),
                  kv_heads=_positive_int(_need(d, "kv_heads", where), f"{where}.kv_heads"),
                  dim=_positive_int(_need(d, "dim", where), f"{where}.dim"),
                  vdim=_positive_int(_need(d, "vdim", where), f"{where}.vdim"),
                  scale=_finite(_need(d, "scale", where), f"{where}.scale"), window=_window(d, where))
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}: heads must be a multiple of kv_heads")
        if max(cfg.dim, cfg.vdim) > MAX_HEAD:
            raise ConfigError(f"config.json: {where}: head sizes above {MAX_HEAD} are not supported")
        return cfg


@dataclass(frozen=True)
class StretchConfig:
    factor: float
    original: float
    fast: float
    slow: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "StretchConfig":
        cfg = cls(*(_finite(_need(d, k, where), f"{where}.{k}") for k in ("factor", "original", "fast", "slow")))
        if min(cfg.factor, cfg.original, cfg.fast, cfg.slow) <= 0:
            raise ConfigError(f"config.json: {where}: factor, original, fast and slow must be positive")
        return cfg

    def as_dict(self) -> dict:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int | None
    rot_base: float
    stretch: StretchConfig | None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "LatentAttentionConfig":
        rot = _need(d, "rot", where)
        rot_dim = _need(d, "rot_dim", where)
        if isinstance(rot_dim, bool) or not isinstance(rot_dim, int) or rot_dim <= 0 or rot_dim % 2:
            raise ConfigError(f"config.json: {where}.rot_dim must be a positive even integer, got {rot_dim!r}")
        if _need(rot, "dims", f"{where}.rot") != rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims must equal rot_dim: the rotated part is rotated as a whole")
        scaling = rot.get("scaling")
        cfg = cls(heads=_positive_int(_need(d, "heads", where), f"{where}.heads"),
                  dim=_positive_int(_need(d, "dim", where), f"{where}.dim"), rot_dim=rot_dim,
                  vdim=_positive_int(_need(d, "vdim", where), f"{where}.vdim"),
                  q_rank=_positive_int(_need(d, "q_rank", where), f"{where}.q_rank"),
                  kv_rank=_positive_int(_need(d, "kv_rank", where), f"{where}.kv_rank"),
                  scale=_finite(_need(d, "scale", where), f"{where}.scale"), window=_window(d, where),
                  rot_base=_finite(_need(rot, "base", f"{where}.rot"), f"{where}.rot.base"),
                  stretch=None if scaling is None else StretchConfig.from_dict(scaling, f"{where}.rot.scaling"))
        if not cfg.rot_base > (1 if cfg.stretch is not None else 0):
            raise ConfigError(f"config.json: {where}.rot.base must be positive (above 1 with scaling)")
        if cfg.kv_rank + cfg.rot_dim > MAX_HEAD:
            raise ConfigError(f"config.json: {where}: kv_rank + rot_dim above {MAX_HEAD} is not supported (a cached row is one key)")
        return cfg


@dataclass(frozen=True)
class GlaConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int | None      # None until the checkpoint's shapes have been seen

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "GlaConfig":
        rank = d.get("decay_rank")
        cfg = cls(heads=_positive_int(_need(d, "heads", where), f"{where}.heads"),
                  dim=_positive_int(_need(d, "dim", where), f"{where}.dim"),
                  vdim=_positive_int(_need(d, "vdim", where), f"{where}.vdim"),
                  tau=_finite(_need(d, "tau", where), f"{where}.tau"),
                  decay_rank=None if rank is None else _positive_int(rank, f"{where}.decay_rank"))
        if not cfg.tau > 0:
            raise ConfigError(f"config.json: {where}.tau must be positive")
        if cfg.dim > 256 or cfg.vdim > 255:
            raise ConfigError(f"config.json: {where}: a head of {cfg.dim} x {cfg.vdim} does not fit the recurrence kernel")
        return cfg


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    identity: int
    top: int
    scale: float
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "ExpertsConfig":
        router = _need(d, "router", where)
        expert = _need(d, "expert", where)
        identity = router.get("identity", 0)
        if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
            raise ConfigError(f"config.json: {where}.router.identity must be a non-negative integer")
        cfg = cls(experts=_positive_int(_need(router, "experts", f"{where}.router"), f"{where}.router.experts"),
                  identity=identity, top=_positive_int(_need(router, "top", f"{where}.router"), f"{where}.router.top"),
                  scale=_finite(router.get("scale", 1.0), f"{where}.router.scale"),
                  ff=_positive_int(_need(expert, "ff", f"{where}.expert"), f"{where}.expert.ff"),
                  limit=_finite(_need(expert, "limit", f"{where}.expert"), f"{where}.expert.limit"))
        if cfg.top > cfg.experts + cfg.identity:
            raise ConfigError(f"config.json: {where}.router: top exceeds the number of router outputs")
        if not cfg.limit > 0:
            raise ConfigError(f"config.json: {where}.expert.limit must be positive")
        return cfg


MIXERS = {"attention": NormedAttentionConfig, "latent_attention": LatentAttentionConfig, "gla": GlaConfig}


@dataclass(frozen=True)
class DugudraLayer:
    type: str
    mixer: NormedAttentionConfig | LatentAttentionConfig | GlaConfig
    mlp: ExpertsConfig | None


@dataclass(frozen=True)
class DugudraConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    logit_softcap: float | None
    layers: tuple[DugudraLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: dict) -> "DugudraConfig":
        raw_layers = _need(d, "layers", "the top level")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, layer in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r} is not implemented (known: {', '.join(sorted(MIXERS))})")
            mixer = MIXERS[kind].from_dict(_need(layer, "mixer", where), f"{where}.mixer")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", f"{where}.mlp") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp: feed-forward kind {mlp['kind']!r} is not implemented (known: moe)")
                mlp = ExpertsConfig.from_dict(mlp, f"{where}.mlp")
            layers.append(DugudraLayer(kind, mixer, mlp))
        cap = d.get("logit_softcap")
        embedding = d.get("embedding") or {}
        cfg = cls(architecture=str(d.get("architecture", "Dugudra")),
                  vocab=_positive_int(_need(d, "vocab", "the top level"), "vocab"),
                  width=_positive_int(_need(d, "width", "the top level"), "width"),
                  norm_eps=_finite(_need(_need(d, "norm", "the top level"), "eps", "norm"), "norm.eps"),
                  embedding_scale=_finite(embedding.get("scale", 1.0), "embedding.scale"),
                  residual_mult=_finite(d.get("residual_mult", 1.0), "residual_mult"),
                  logit_softcap=None if cap is None else _finite(cap, "logit_softcap"),
                  layers=tuple(layers))
        if not cfg.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if cfg.logit_softcap is not None and not cfg.logit_softcap > 0:
            raise ConfigError("config.json: logit_softcap must be positive or null")
        return cfg

    def with_tensor_shapes(self, shapes: dict[str, tuple]) -> "DugudraConfig":
        """Fill the size only the checkpoint gives (the inner size of a gla layer's decay projection, from
        ``l<i>.mix.a1``) and refuse a configured one that the checkpoint contradicts."""
        layers = list(self.layers)
        for i, layer in enumerate(layers):
            if not isinstance(layer.mixer, GlaConfig):
                continue
            shape = shapes.get(f"l{i}.mix.a1")
            rank = layer.mixer.decay_rank
            if shape is not None:
                if len(shape) != 2 or (rank is not None and rank != shape[0]):
                    raise ConfigError(f"config.json: layers[{i}].mixer.decay_rank {rank} contradicts l{i}.mix.a1 {list(shape)}")
                rank = int(shape[0])
            layers[i] = replace(layer, mixer=replace(layer.mixer, decay_rank=rank))
        return replace(self, layers=tuple(layers))

    @classmethod
    def read(cls, folder) -> "DugudraConfig":
        folder = Path(folder)
        cfg = cls.from_dict(json.loads((folder / "config.json").read_text()))
        return cfg.with_tensor_shapes(safetensors_shapes(folder))
