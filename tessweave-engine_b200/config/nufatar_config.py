"""Typed view of a Nufatar ``config.json``.

The file names the design under ``architecture`` and gives the residual width, the vocabulary, the norms' eps, a
list of layers and optionally a ``loop`` (``start``, ``stop``, ``times``: the layers ``start .. stop - 1`` run
``times`` times in a row on the same tensors, every pass on a cache and state of its own).  A layer names its mixer
by ``type``; both kinds put softmax attention (``left``) beside a gated delta rule (``right``) on the same input:

* ``parallel``: attention over a sliding window without rotation, whose values are its keys, with a learned bias by
  bucketed distance and a learned sink in the softmax; a delta rule with one decay per key channel (through a
  low-rank projection) and a sigmoid output gate (low-rank too); the two results are normalised and averaged.
* ``parallel_2``: causal attention with partly rotated heads (YaRN-scaled frequencies), keys and values of their own
  sizes; a delta rule with one decay per head and a silu output gate; the two results are added with two scales.

``mlp`` is a dense gated feed-forward (``kind: dense``, ``ff``) or null.  Every size and constant comes from here; the
sizes the file does not give (the inner sizes of the low-rank projections, the rows of the distance table) are read
from the checkpoint's tensor shapes, or from the keys ``decay_rank`` / ``gate_rank`` / ``bias_rows`` where a
configuration is written before its weights exist.  Anything this engine does not implement is refused before a weight
is read.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, replace
from pathlib import Path

from .linurax_config import _finite, _need, _positive_int
from .model_config import ConfigError
from .sapatar_config import safetensors_shapes


@dataclass(frozen=True)
class YarnConfig:
    factor: float
    original: float
    fast: float
    slow: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "YarnConfig":
        cfg = cls(*(_finite(_need(d, key, where), f"{where}.{key}") for key in ("factor", "original", "fast", "slow")))
        if min(cfg.factor, cfg.original, cfg.fast, cfg.slow) <= 0:
            raise ConfigError(f"config.json: {where}: factor, original, fast and slow must be positive")
        return cfg


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    scaling: YarnConfig | None

    @classmethod
    def from_dict(cls, d: dict, where: str, head_dim: int) -> "RotaryConfig":
        dims = _need(d, "dims", where)
        base = _finite(_need(d, "base", where), f"{where}.base")
        if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > head_dim or not base > 1:
            raise ConfigError(f"config.json: {where}: dims must be even and at most the head size {head_dim}, base above 1")
        scaling = d.get("scaling")
        return cls(dims, base, None if scaling is None else YarnConfig.from_dict(scaling, f"{where}.scaling"))


@dataclass(frozen=True)
class SoftmaxAttentionConfig:
    """``window`` None: causal over everything.  ``rot`` None: no rotation.  ``bias_max`` set: a table of biases by
    bucketed distance (``bias_rows`` rows, from the checkpoint) and a sink per head, and the values are the keys."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None
    rot: RotaryConfig | None
    bias_max: float | None
    bias_rows: int | None
    sink: bool
    values_are_keys: bool

    @classmethod
    def from_dict(cls, d: dict, where: str, kind: str) -> "SoftmaxAttentionConfig":
        heads = _positive_int(_need(d, "heads", where), f"{where}.heads")
        kv_heads = _positive_int(_need(d, "kv_heads", where), f"{where}.kv_heads")
        dim = _positive_int(_need(d, "dim", where), f"{where}.dim")
        vdim = _positive_int(_need(d, "vdim", where), f"{where}.vdim")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: heads must be a multiple of kv_heads")
        if max(dim, vdim) > 256:
            raise ConfigError(f"config.json: {where}: head sizes above 256 are not supported")
        scale = _finite(_need(d, "scale", where), f"{where}.scale")
        if kind == "parallel":
            window = _positive_int(_need(_need(d, "mask", where), "size", f"{where}.mask"), f"{where}.mask.size")
            bias_max = _finite(_need(d, "bias_max", where), f"{where}.bias_max")
            rows = d.get("bias_rows")
            if vdim != dim:
                raise ConfigError(f"config.json: {where}: the values are the keys, so vdim must equal dim")
            if "rot" in d and d["rot"] is not None:
                raise ConfigError(f"config.json: {where}: a rotation is not part of a 'parallel' layer's attention")
            return cls(heads, kv_heads, dim, vdim, scale, window, None, bias_max,
                       None if rows is None else _positive_int(rows, f"{where}.bias_rows"), True, True)
        for key in ("mask", "bias_max"):
            if d.get(key) is not None:
                raise ConfigError(f"config.json: {where}: {key!r} is not part of a 'parallel_2' layer's attention")
        rot = RotaryConfig.from_dict(_need(d, "rot", where), f"{where}.rot", dim)
        return cls(heads, kv_heads, dim, vdim, scale, None, rot, None, None, False, False)


@dataclass(frozen=True)
class DeltaRuleConfig:
    """``channel_decay``: one decay per head and key channel through a low-rank projection of inner size
    ``decay_rank`` (else one per head, projected directly); ``gate``: the output gate's activation, through a low-rank
    projection of inner size ``gate_rank`` where ``low_rank_gate``."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    channel_decay: bool
    decay_rank: int | None
    gate: str
    low_rank_gate: bool
    gate_rank: int | None

    @classmethod
    def from_dict(cls, d: dict, where: str, kind: str) -> "DeltaRuleConfig":
        heads = _positive_int(_need(d, "heads", where), f"{where}.heads")
        kv_heads = _positive_int(_need(d, "kv_heads", where), f"{where}.kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: heads must be a multiple of kv_heads")
        dim = _positive_int(_need(d, "dim", where), f"{where}.dim")
        vdim = _positive_int(_need(d, "vdim", where), f"{where}.vdim")
        if dim > 256 or vdim > 255:
            raise ConfigError(f"config.json: {where}: heads of {dim} x {vdim} exceed the recurrence's 256 x 255")
        conv = _positive_int(_need(d, "conv", where), f"{where}.conv")
        if conv > 16:
            raise ConfigError(f"config.json: {where}.conv: more than 16 taps are not supported")
        low = kind == "parallel"
        ranks = [None if d.get(k) is None else _positive_int(d[k], f"{where}.{k}") for k in ("decay_rank", "gate_rank")]
        return cls(heads, kv_heads, dim, vdim, conv, low, ranks[0] if low else None, "sigmoid" if low else "silu", low,
                   ranks[1] if low else None)


@dataclass(frozen=True)
class MixerConfig:
    left: SoftmaxAttentionConfig
    right: DeltaRuleConfig
    left_scale: float
    right_scale: float
    normalised: bool          # each side's result is RMS-normed with a weight of its own before the sum

    @classmethod
    def from_dict(cls, d: dict, where: str, kind: str) -> "MixerConfig":
        left = SoftmaxAttentionConfig.from_dict(_need(d, "left", where), f"{where}.left", kind)
        right = DeltaRuleConfig.from_dict(_need(d, "right", where), f"{where}.right", kind)
        if kind == "parallel":
            return cls(left, right, 0.5, 0.5, True)
        return cls(left, right, _finite(_need(d, "left_scale", where), f"{where}.left_scale"),
                   _finite(_need(d, "right_scale", where), f"{where}.right_scale"), False)


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class NufatarLayer:
    type: str
    mixer: MixerConfig
    mlp: DenseConfig | None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


MIXER_TYPES = ("parallel", "parallel_2")


@dataclass(frozen=True)
class NufatarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[NufatarLayer, ...]
    loop: LoopConfig | None
    eos_token_ids: tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: dict) -> "NufatarConfig":
        raw_layers = _need(d, "layers", "the top level")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, layer in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r} is not implemented (known: {', '.join(MIXER_TYPES)})")
            mixer = MixerConfig.from_dict(_need(layer, "mixer", where), f"{where}.mixer", kind)
            mlp = layer.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", f"{where}.mlp") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp: feed-forward kind {mlp['kind']!r} is not implemented (known: dense)")
                mlp = DenseConfig(_positive_int(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff"))
            layers.append(NufatarLayer(kind, mixer, mlp))
        loop = d.get("loop")
        if loop is not None:
            start, stop, times = (_need(loop, key, "loop") for key in ("start", "stop", "times"))
            for value in (start, stop, times):
                if isinstance(value, bool) or not isinstance(value, int):
                    raise ConfigError("config.json: loop.start, loop.stop and loop.times must be integers")
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"config.json: loop: 0 <= start <= stop <= {len(layers)} and times >= 1 are required")
            loop = LoopConfig(start, stop, times)
        cfg = cls(architecture=str(d.get("architecture", "Nufatar")),
                  vocab=_positive_int(_need(d, "vocab", "the top level"), "vocab"),
                  width=_positive_int(_need(d, "width", "the top level"), "width"),
                  norm_eps=_finite(_need(_need(d, "norm", "the top level"), "eps", "norm"), "norm.eps"),
                  layers=tuple(layers), loop=loop)
        if not cfg.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg

    def with_tensor_shapes(self, shapes: dict[str, tuple]) -> "NufatarConfig":
        """Fill the sizes only the checkpoint gives (``l<i>.mix.right.a1`` / ``.g1``: the inner sizes of the low-rank
        projections; ``l<i>.mix.left.rel``: the rows of the distance table) and refuse a configured one that the
        checkpoint contradicts."""
        def settle(configured, shape, what):
            if shape is None:
                return configured
            if len(shape) != 2 or (configured is not None and configured != shape[0]):
                raise ConfigError(f"config.json: {what} {configured} contradicts the checkpoint's {list(shape)}")
            return int(shape[0])

        layers = []
        for i, layer in enumerate(self.layers):
            left, right = layer.mixer.left, layer.mixer.right
            if right.channel_decay:
                right = replace(right, decay_rank=settle(right.decay_rank, shapes.get(f"l{i}.mix.right.a1"), f"layers[{i}].mixer.right.decay_rank"))
            if right.low_rank_gate:
                right = replace(right, gate_rank=settle(right.gate_rank, shapes.get(f"l{i}.mix.right.g1"), f"layers[{i}].mixer.right.gate_rank"))
            if left.bias_max is not None:
                left = replace(left, bias_rows=settle(left.bias_rows, shapes.get(f"l{i}.mix.left.rel"), f"layers[{i}].mixer.left.bias_rows"))
            layers.append(replace(layer, mixer=replace(layer.mixer, left=left, right=right)))
        return replace(self, layers=tuple(layers))

    @classmethod
    def read(cls, folder) -> "NufatarConfig":
        folder = Path(folder)
        cfg = cls.from_dict(json.loads((folder / "config.json").read_text()))
        return cfg.with_tensor_shapes(safetensors_shapes(folder))
