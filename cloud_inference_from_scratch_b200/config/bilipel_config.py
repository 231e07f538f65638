"""Typed configuration of the Bilipel decoder, read from config.json keys.

A Bilipel model is a list of pre-norm layers (layer norm with gain and bias), each with one token mixer and
an optional feed-forward, every sublayer's result multiplied by one constant before it joins the stream; a run
of consecutive layers may be passed several times in a row.  config.json carries:

* ``architecture`` "Bilipel", ``vocab``, ``width``, ``norm.eps``, ``residual_mult``;
* ``loop`` (optional): ``start``, ``stop``, ``times``: layers start..stop-1 run ``times`` times with the same
  weights and a cache of their own each time;
* ``layers``: per layer ``type`` ("attention", "latent_attention" or "gla"), ``mixer`` (its sizes and
  constants) and ``mlp`` (null; ``kind`` "dense" with ``ff``; or ``kind`` "moe" with ``expert.ff``,
  ``router.experts`` and ``router.top``).

Mixer "attention": ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` (``base``, ``dims``, optional
``scaling`` with ``factor``, ``original``, ``fast``, ``slow``).  Mixer "latent_attention": ``heads``, ``dim``,
``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``rot`` (``base``; ``dims`` equals ``rot_dim``), optional
``mask.size``.  Mixer "gla": ``heads``, ``dim``, ``vdim``, ``tau``; the inner width of its decay projection is a
tensor's shape (``decay_rank`` may name it, and is written for random models).

Every size and constant comes from here; this module is the only place that knows the key names.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .lazilorn_config import LoopConfig, _number
from .model_config import ConfigError
from .zisesun_config import _count, _get


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int                                                  # rotated elements of a head
    scaling: tuple[float, float, float, float] | None          # factor, original, fast, slow

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str, dims: int | None = None) -> "RotationConfig":
        base = _number(raw, "base", where)
        if not base > 1:
            raise ConfigError(f"config.json: {where}: 'base' must be above 1, got {base}")
        own = _count(raw, "dims", where) if "dims" in raw or dims is None else dims
        if dims is not None and own != dims:
            raise ConfigError(f"config.json: {where}: 'dims' ({own}) must equal the rotated part's size ({dims})")
        if own % 2:
            raise ConfigError(f"config.json: {where}: 'dims' must be even, got {own}")
        scaling = raw.get("scaling")
        if scaling is not None:
            here = where + ".scaling"
            scaling = tuple(_number(scaling, key, here) for key in ("factor", "original", "fast", "slow"))
            if min(scaling) <= 0:
                raise ConfigError(f"config.json: {here}: factor, original, fast and slow must be positive")
        return cls(base, own, scaling)

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(base=self.base, dims=self.dims)
        if self.scaling is not None:
            raw["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return raw


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotationConfig

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "SinkAttentionConfig":
        heads, kv_heads = _count(raw, "heads", where), _count(raw, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
        dim = _count(raw, "dim", where)
        rot = RotationConfig.from_dict(_get(raw, "rot", dict, where), where + ".rot")
        if rot.dims > dim:
            raise ConfigError(f"config.json: {where}.rot: 'dims' ({rot.dims}) is more than a head has ({dim})")
        return cls(heads, kv_heads, dim, _count(raw, "vdim", where), _number(raw, "scale", where), rot)

    def to_dict(self) -> dict[str, Any]:
        return dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale,
                    rot=self.rot.to_dict())


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int            # unrotated query / key elements of a head
    rot_dim: int        # rotated elements of a head (one key part for all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotationConfig
    window: int         # keys a query sees, itself included; 0: every earlier key

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "LatentMixerConfig":
        rot_dim = _count(raw, "rot_dim", where)
        mask = raw.get("mask")
        return cls(_count(raw, "heads", where), _count(raw, "dim", where), rot_dim, _count(raw, "vdim", where),
                   _count(raw, "kv_rank", where), _number(raw, "scale", where),
                   RotationConfig.from_dict(_get(raw, "rot", dict, where), where + ".rot", dims=rot_dim),
                   _count(mask, "size", where + ".mask") if mask is not None else 0)

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim,
                                   kv_rank=self.kv_rank, scale=self.scale, rot=self.rot.to_dict())
        if self.window:
            raw["mask"] = dict(size=self.window)
        return raw


@dataclass(frozen=True)
class GlaConfig:
    heads: int
    dim: int
    vdim: int
    tau: float          # the decay is sigmoid(z)^(1 / tau)
    decay_rank: int | None = None   # None: the shape of the stored tensor says

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "GlaConfig":
        tau = _number(raw, "tau", where)
        if not tau > 0:
            raise ConfigError(f"config.json: {where}: 'tau' must be positive, got {tau}")
        rank = raw.get("decay_rank")
        return cls(_count(raw, "heads", where), _count(raw, "dim", where), _count(raw, "vdim", where), tau,
                   None if rank is None else _count(raw, "decay_rank", where))

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(heads=self.heads, dim=self.dim, vdim=self.vdim, tau=self.tau)
        if self.decay_rank is not None:
            raw["decay_rank"] = self.decay_rank
        return raw


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str           # "dense" | "moe"
    ff: int             # inner size (of every expert, for "moe")
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "FeedForwardConfig":
        kind = _get(raw, "kind", str, where)
        if kind == "dense":
            return cls("dense", _count(raw, "ff", where))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}: feed-forward kind {kind!r} is not built (known: dense, moe)")
        router = _get(raw, "router", dict, where)
        experts, top = _count(router, "experts", where + ".router"), _count(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router: 'top' ({top}) is more than 'experts' ({experts})")
        return cls("moe", _count(_get(raw, "expert", dict, where), "ff", where + ".expert"), experts, top)

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return dict(kind="dense", ff=self.ff)
        return dict(kind="moe", expert=dict(ff=self.ff), router=dict(experts=self.experts, top=self.top))


MIXERS = {"attention": SinkAttentionConfig, "latent_attention": LatentMixerConfig, "gla": GlaConfig}


@dataclass(frozen=True)
class BilipelLayerConfig:
    type: str
    mixer: SinkAttentionConfig | LatentMixerConfig | GlaConfig
    mlp: FeedForwardConfig | None

    def to_dict(self) -> dict[str, Any]:
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp is not None else None)


@dataclass(frozen=True)
class BilipelConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    loop: LoopConfig | None
    layers: tuple[BilipelLayerConfig, ...]
    architecture: str = "Bilipel"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "BilipelConfig":
        where = "Bilipel"
        eps = _number(_get(raw, "norm", dict, where), "eps", where + ".norm")
        if eps < 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {eps}")
        entries = _get(raw, "layers", list, where)
        if not entries:
            raise ConfigError("config.json: 'layers' is empty")
        layers: list[BilipelLayerConfig] = []
        for index, entry in enumerate(entries):
            here = f"layers[{index}]"
            kind = _get(entry, "type", str, here)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {here}: mixer type {kind!r} is not built (known: {sorted(MIXERS)})")
            mixer = MIXERS[kind].from_dict(_get(entry, "mixer", dict, here), here + ".mixer")
            mlp = entry.get("mlp")
            layers.append(BilipelLayerConfig(
                kind, mixer, FeedForwardConfig.from_dict(mlp, here + ".mlp") if mlp is not None else None))
        loop = raw.get("loop")
        if loop is not None:
            start = int(_get(loop, "start", int, "loop"))
            stop, times = _count(loop, "stop", "loop"), _count(loop, "times", "loop")
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop: layers {start}..{stop - 1} do not lie within the {len(layers)} layers")
            loop = LoopConfig(start, stop, times)
        return cls(vocab=_count(raw, "vocab", where), width=_count(raw, "width", where), norm_eps=eps,
                   residual_mult=_number(raw, "residual_mult", where) if "residual_mult" in raw else 1.0,
                   loop=loop, layers=tuple(layers), architecture=str(raw.get("architecture", "Bilipel")))

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(architecture=self.architecture, vocab=self.vocab, width=self.width,
                                   norm=dict(eps=self.norm_eps), residual_mult=self.residual_mult,
                                   layers=[layer.to_dict() for layer in self.layers])
        if self.loop is not None:
            raw["loop"] = self.loop.to_dict()
        return raw
