"""Typed configuration of the ``Lilulix`` architecture.

``config.json`` gives ``vocab``, ``width``, ``norm.eps``, the hashed token-pair embedding
(``embedding.bigram``: ``buckets``, ``mul_prev``, ``mul_cur``), a list ``layers`` and, optionally, ``loop``
(``start``, ``stop``, ``times``: layers ``start .. stop - 1`` run ``times`` times in a row).  Every entry of
``layers`` names its mixer (``type``: ``"latent_attention"`` or ``"attention"``), the mixer's sizes
(``mixer``) and its feed-forward (``mlp``: ``{"kind": "dense", "ff": ...}``, or null for none).  Layers
may differ from one another in everything.  Nothing here has a default that stands for a size: a
missing key is an error.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .registry import ConfigError
from .ruvurax import _need, _positive


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int          # unrotated query/key dimensions per head
    rot_dim: int      # rotated query/key dimensions per head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    rot_base: float
    rot_dims: int     # how many of the rot_dim dimensions turn
    scale: float


@dataclass(frozen=True)
class BiasedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class LilulixLayer:
    type: str
    mixer: LatentAttentionConfig | BiasedAttentionConfig
    mlp: DenseMlpConfig | None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class LilulixConfig:
    vocab: int
    width: int
    eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: tuple[LilulixLayer, ...]
    loop: LoopConfig | None

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "LilulixConfig":
        layers = _need(raw, "layers", "the top level")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        big = _need(_need(raw, "embedding", "the top level"), "bigram", "embedding")
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            start, stop = _need(lp, "start", "loop"), _need(lp, "stop", "loop")
            loop = LoopConfig(int(start), int(stop), _positive(lp, "times", "loop"))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop {loop.start} .. {loop.stop} does not lie within {len(layers)} layers")
        for key in ("mul_prev", "mul_cur"):
            v = _need(big, key, "embedding.bigram")
            if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                raise ConfigError(f"config.json: embedding.bigram.{key} must be a non-negative integer, got {v!r}")
        return cls(
            vocab=_positive(raw, "vocab", "the top level"),
            width=_positive(raw, "width", "the top level"),
            eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            buckets=_positive(big, "buckets", "embedding.bigram"),
            mul_prev=int(big["mul_prev"]),
            mul_cur=int(big["mul_cur"]),
            layers=tuple(_layer(l, f"layers[{i}]") for i, l in enumerate(layers)),
            loop=loop,
        )


def _layer(raw: Mapping[str, Any], where: str) -> LilulixLayer:
    kind = _need(raw, "type", where)
    m = _need(raw, "mixer", where)
    mw = where + ".mixer"
    if kind == "latent_attention":
        rot = _need(m, "rot", mw)
        rot_dim = _need(m, "rot_dim", mw)
        if isinstance(rot_dim, bool) or not isinstance(rot_dim, int) or rot_dim < 0:
            raise ConfigError(f"config.json: {mw}.rot_dim must be a non-negative integer, got {rot_dim!r}")
        mixer = LatentAttentionConfig(
            heads=_positive(m, "heads", mw), dim=_positive(m, "dim", mw), rot_dim=rot_dim,
            vdim=_positive(m, "vdim", mw), kv_rank=_positive(m, "kv_rank", mw),
            rot_base=float(_need(rot, "base", mw + ".rot")), rot_dims=int(_need(rot, "dims", mw + ".rot")),
            scale=float(_need(m, "scale", mw)))
        if mixer.rot_dims % 2 or not 0 <= mixer.rot_dims <= mixer.rot_dim:
            raise ConfigError(f"config.json: {mw}.rot.dims={mixer.rot_dims} must be even and at most rot_dim={mixer.rot_dim}")
    elif kind == "attention":
        dim = _positive(m, "dim", mw)
        mixer = BiasedAttentionConfig(heads=_positive(m, "heads", mw), kv_heads=_positive(m, "kv_heads", mw), dim=dim,
                                      vdim=_positive(m, "vdim", mw) if m.get("vdim") is not None else dim,
                                      scale=float(_need(m, "scale", mw)))
        if mixer.heads % mixer.kv_heads:
            raise ConfigError(f"config.json: {mw}: {mixer.heads} heads cannot share {mixer.kv_heads} key/value heads")
        if mixer.vdim != mixer.dim:
            raise ConfigError(f"config.json: {mw}: the values are the keys, so vdim={mixer.vdim} must equal dim={mixer.dim}")
    else:
        raise ConfigError(f"config.json: {where}.type {kind!r} is neither 'latent_attention' nor 'attention'")
    mlp = raw.get("mlp")
    dense = None
    if mlp is not None:
        if _need(mlp, "kind", where + ".mlp") != "dense":
            raise ConfigError(f"config.json: {where}.mlp.kind {mlp.get('kind')!r} is not 'dense'")
        dense = DenseMlpConfig(ff=_positive(mlp, "ff", where + ".mlp"))
    return LilulixLayer(kind, mixer, dense)
