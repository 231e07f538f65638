"""Typed configuration of the Lazilorn decoder, read from config.json keys.

A Lazilorn model is a list of pre-norm layers, each with one token mixer and an optional dense feed-forward,
of which a run of consecutive layers may be passed several times in a row.  config.json carries:

* ``architecture`` "Lazilorn", ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_scale``;
* ``loop`` (optional): ``start``, ``stop``, ``times``: layers start..stop-1 run ``times`` times with the same
  weights and a cache of their own each time;
* ``layers``: per layer ``type`` ("parallel" or "delta"), ``mixer`` (its sizes and constants) and ``mlp``
  (null, or ``kind`` "dense" with ``ff``).

Mixer "parallel": ``left`` (softmax attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``mask.size``, ``mask.keep_first``), ``right`` (matrix memory: ``heads``, ``dim``, ``vdim``, ``gate_cap``),
``left_scale``, ``right_scale``.  Mixer "delta" (gated delta rule): ``heads``, ``kv_heads``, ``dim``, ``vdim``,
``conv`` (taps of the short convolution).

Every size and constant comes from here; this module is the only place that knows the key names.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .model_config import ConfigError
from .zisesun_config import _count, _get


def _number(raw: dict[str, Any], key: str, where: str) -> float:
    return float(_get(raw, key, (int, float), where))


@dataclass(frozen=True)
class WindowedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int            # size of a query / key head
    vdim: int           # size of a value head
    scale: float        # multiplies q.k
    window: int         # keys a query sees, itself included; 0: every earlier key
    keep_first: int     # first keys of a request that stay visible behind the window

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "WindowedAttentionConfig":
        heads, kv_heads = _count(raw, "heads", where), _count(raw, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
        mask = raw.get("mask")
        window = keep_first = 0
        if mask is not None:
            window = _count(mask, "size", where + ".mask")
            keep_first = int(_get(mask, "keep_first", int, where + ".mask")) if "keep_first" in mask else 0
            if keep_first < 0:
                raise ConfigError(f"config.json: {where}.mask: 'keep_first' must not be negative")
        return cls(heads, kv_heads, _count(raw, "dim", where), _count(raw, "vdim", where),
                   _number(raw, "scale", where), window, keep_first)

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                                   scale=self.scale)
        if self.window:
            raw["mask"] = dict(size=self.window, keep_first=self.keep_first)
        return raw


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "MatrixMemoryConfig":
        cap = _number(raw, "gate_cap", where)
        if not cap > 0:
            raise ConfigError(f"config.json: {where}: 'gate_cap' must be positive, got {cap}")
        return cls(_count(raw, "heads", where), _count(raw, "dim", where), _count(raw, "vdim", where), cap)

    def to_dict(self) -> dict[str, Any]:
        return dict(heads=self.heads, dim=self.dim, vdim=self.vdim, gate_cap=self.gate_cap)


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowedAttentionConfig
    right: MatrixMemoryConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "ParallelMixerConfig":
        return cls(WindowedAttentionConfig.from_dict(_get(raw, "left", dict, where), where + ".left"),
                   MatrixMemoryConfig.from_dict(_get(raw, "right", dict, where), where + ".right"),
                   _number(raw, "left_scale", where), _number(raw, "right_scale", where))

    def to_dict(self) -> dict[str, Any]:
        return dict(left=self.left.to_dict(), right=self.right.to_dict(), left_scale=self.left_scale,
                    right_scale=self.right_scale)


@dataclass(frozen=True)
class GatedDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int           # taps of the short convolution

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "GatedDeltaConfig":
        heads, kv_heads = _count(raw, "heads", where), _count(raw, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
        return cls(heads, kv_heads, _count(raw, "dim", where), _count(raw, "vdim", where), _count(raw, "conv", where))

    def to_dict(self) -> dict[str, Any]:
        return dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, conv=self.conv)


@dataclass(frozen=True)
class DenseConfig:
    ff: int

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "DenseConfig":
        kind = raw.get("kind", "dense")
        if kind != "dense":
            raise ConfigError(f"config.json: {where}: feed-forward kind {kind!r} is not built (only 'dense')")
        return cls(_count(raw, "ff", where))

    def to_dict(self) -> dict[str, Any]:
        return dict(kind="dense", ff=self.ff)


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int

    def to_dict(self) -> dict[str, Any]:
        return dict(start=self.start, stop=self.stop, times=self.times)


@dataclass(frozen=True)
class LazilornLayerConfig:
    type: str                                            # "parallel" | "delta"
    mixer: ParallelMixerConfig | GatedDeltaConfig
    mlp: DenseConfig | None

    def to_dict(self) -> dict[str, Any]:
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp is not None else None)


MIXERS = {"parallel": ParallelMixerConfig, "delta": GatedDeltaConfig}


@dataclass(frozen=True)
class LazilornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    loop: LoopConfig | None
    layers: tuple[LazilornLayerConfig, ...]
    architecture: str = "Lazilorn"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "LazilornConfig":
        where = "Lazilorn"
        eps = _number(_get(raw, "norm", dict, where), "eps", where + ".norm")
        if eps < 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {eps}")
        entries = _get(raw, "layers", list, where)
        if not entries:
            raise ConfigError("config.json: 'layers' is empty")
        layers: list[LazilornLayerConfig] = []
        for index, entry in enumerate(entries):
            here = f"layers[{index}]"
            kind = _get(entry, "type", str, here)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {here}: mixer type {kind!r} is not built (known: {sorted(MIXERS)})")
            mixer = MIXERS[kind].from_dict(_get(entry, "mixer", dict, here), here + ".mixer")
            mlp = entry.get("mlp")
            layers.append(LazilornLayerConfig(kind, mixer, DenseConfig.from_dict(mlp, here + ".mlp") if mlp is not None else None))
        loop = raw.get("loop")
        if loop is not None:
            start = int(_get(loop, "start", int, "loop"))
            stop, times = _count(loop, "stop", "loop"), _count(loop, "times", "loop")
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop: layers {start}..{stop - 1} do not lie within the {len(layers)} layers")
            loop = LoopConfig(start, stop, times)
        embedding = raw.get("embedding") or {}
        return cls(vocab=_count(raw, "vocab", where), width=_count(raw, "width", where), norm_eps=eps,
                   embedding_scale=_number(embedding, "scale", "embedding") if "scale" in embedding else 1.0,
                   logit_scale=_number(raw, "logit_scale", where) if "logit_scale" in raw else 1.0,
                   loop=loop, layers=tuple(layers), architecture=str(raw.get("architecture", "Lazilorn")))

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(architecture=self.architecture, vocab=self.vocab, width=self.width,
                                   norm=dict(eps=self.norm_eps), embedding=dict(scale=self.embedding_scale),
                                   logit_scale=self.logit_scale, layers=[layer.to_dict() for layer in self.layers])
        if self.loop is not None:
            raw["loop"] = self.loop.to_dict()
        return raw
