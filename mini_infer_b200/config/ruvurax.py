"""Typed configuration of the ``Ruvurax`` architecture.

``config.json`` gives ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and a list ``layers``;
every entry names its mixer (``type``: ``"rglru"`` or ``"parallel"``), the mixer's sizes (``mixer``)
and its feed-forward (``mlp``: a mixture of experts, or null for none).  Layers may differ from one
another in everything.  Nothing here has a default that stands for a size: a missing key is an error.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .registry import ConfigError


def _need(m: Mapping[str, Any], key: str, where: str):
    if not isinstance(m, Mapping) or key not in m or m[key] is None:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return m[key]


def _positive(m: Mapping[str, Any], key: str, where: str) -> int:
    v = _need(m, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class RecurrentUnitConfig:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int | None
    rot_base: float
    rot_dims: int
    scale: float


@dataclass(frozen=True)
class LinearAttentionConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int | None = None    # rows of the decay's first matrix; None: whatever the checkpoint has


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: LinearAttentionConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: int            # 0: no shared expert
    shared_limit: float


@dataclass(frozen=True)
class RuvuraxLayer:
    type: str
    mixer: RecurrentUnitConfig | ParallelMixerConfig
    mlp: ExpertsConfig | None


@dataclass(frozen=True)
class RuvuraxConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: tuple[RuvuraxLayer, ...]

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "RuvuraxConfig":
        layers = _need(raw, "layers", "the top level")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        return cls(
            vocab=_positive(raw, "vocab", "the top level"),
            width=_positive(raw, "width", "the top level"),
            embedding_scale=float(_need(_need(raw, "embedding", "the top level"), "scale", "embedding")),
            eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            layers=tuple(_layer(l, f"layers[{i}]") for i, l in enumerate(layers)),
        )


def _layer(raw: Mapping[str, Any], where: str) -> RuvuraxLayer:
    kind = _need(raw, "type", where)
    m = _need(raw, "mixer", where)
    if kind == "rglru":
        mixer = RecurrentUnitConfig(width=_positive(m, "width", where + ".mixer"),
                                    blocks=_positive(m, "blocks", where + ".mixer"),
                                    conv=_positive(m, "conv", where + ".mixer"))
        if mixer.width % mixer.blocks:
            raise ConfigError(f"config.json: {where}: {mixer.width} channels are no {mixer.blocks} equal parts")
    elif kind == "parallel":
        l, r = _need(m, "left", where + ".mixer"), _need(m, "right", where + ".mixer")
        lw, rw = where + ".mixer.left", where + ".mixer.right"
        rot = l.get("rot")
        mask = l.get("mask")
        dim = _positive(l, "dim", lw)
        left = WindowAttentionConfig(
            heads=_positive(l, "heads", lw), kv_heads=_positive(l, "kv_heads", lw), dim=dim,
            vdim=_positive(l, "vdim", lw),
            window=_positive(mask, "size", lw + ".mask") if mask else None,
            rot_base=float(_need(rot, "base", lw + ".rot")) if rot else 0.0,
            rot_dims=int(_need(rot, "dims", lw + ".rot")) if rot else 0,
            scale=float(_need(l, "scale", lw)),
        )
        if left.heads % left.kv_heads:
            raise ConfigError(f"config.json: {lw}: {left.heads} heads cannot share {left.kv_heads} key/value heads")
        if left.rot_dims % 2 or not 0 <= left.rot_dims <= dim:
            raise ConfigError(f"config.json: {lw}.rot.dims={left.rot_dims} must be even and at most dim={dim}")
        right = LinearAttentionConfig(heads=_positive(r, "heads", rw), dim=_positive(r, "dim", rw),
                                      vdim=_positive(r, "vdim", rw), tau=float(_need(r, "tau", rw)),
                                      rank=_positive(r, "rank", rw) if r.get("rank") else None)
        mixer = ParallelMixerConfig(left, right, float(_need(m, "left_scale", where + ".mixer")),
                                    float(_need(m, "right_scale", where + ".mixer")))
    else:
        raise ConfigError(f"config.json: {where}.type {kind!r} is neither 'rglru' nor 'parallel'")
    mlp = raw.get("mlp")
    experts = None
    if mlp is not None:
        if mlp.get("kind", "moe") != "moe":
            raise ConfigError(f"config.json: {where}.mlp.kind {mlp.get('kind')!r} is not 'moe'")
        router, expert = _need(mlp, "router", where + ".mlp"), _need(mlp, "expert", where + ".mlp")
        shared = mlp.get("shared")
        experts = ExpertsConfig(
            experts=_positive(router, "experts", where + ".mlp.router"),
            top=_positive(router, "top", where + ".mlp.router"),
            ff=_positive(expert, "ff", where + ".mlp.expert"),
            limit=float(_need(expert, "limit", where + ".mlp.expert")),
            shared_ff=_positive(shared, "ff", where + ".mlp.shared") if shared else 0,
            shared_limit=float(_need(shared, "limit", where + ".mlp.shared")) if shared else 0.0,
        )
        if experts.top > experts.experts:
            raise ConfigError(f"config.json: {where}.mlp.router: top={experts.top} of {experts.experts} experts")
    return RuvuraxLayer(kind, mixer, experts)
