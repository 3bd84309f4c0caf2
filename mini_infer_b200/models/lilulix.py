"""``Lilulix``: a decoder whose layers add a mixer and a dense gated feed-forward to the stream in
parallel, both reading one RMS norm (``x += mixer(n) + ff(n)``, ``n = norm1(x)``).  A layer's mixer is
either attention in a low-rank latent space (learned sink per head, sigmoid gate on the heads) or
grouped attention with a distance bias whose values are its keys.  The embedding adds a hashed
token-pair row; a stretch of layers may run several times with the same weights, each pass with a
cache of its own, the embedding's output and a learned vector per pass being added to the stream
before it; the head is the embedding table.

This file is the only place that knows the architecture: it turns a ``LilulixConfig`` into a
``ModelSpec`` of generic parts and names the checkpoint tensors (``embed``, ``bigram``, ``loop.step``,
``l{i}.norm1``, ``l{i}.mix.*``, ``l{i}.mlp.gate`` / ``up`` / ``down``, ``final.norm``).
"""

from __future__ import annotations

from ..config.lilulix import LatentAttentionConfig, LilulixConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _rms_norm(H: int, eps: float, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"hidden_size": H, "eps": eps}, rename={"weight": name})


def assemble(cfg: LilulixConfig) -> ModelSpec:
    H = cfg.width
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, LatentAttentionConfig):
            mixer = PartSpec("latent_attention",
                             {"hidden_size": H, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
                              "value_dim": m.vdim, "kv_rank": m.kv_rank, "theta": m.rot_base, "rotary_dim": m.rot_dims,
                              "scale": m.scale, "eps": cfg.eps, "sink": "learned", "gate": "sigmoid"},
                             prefix=p + "mix.")
        else:
            mixer = PartSpec("distance_bias_attention",
                             {"hidden_size": H, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                              "scale": m.scale, "qk_bias": True, "qk_norm": True, "eps": cfg.eps,
                              "values_are_keys": True, "slope_span": 8.0, "sink": "zero"}, prefix=p + "mix.")
        if layer.mlp is None:
            feed_forward, ff_norm = PartSpec("no_feed_forward"), PartSpec("no_norm")
        else:
            feed_forward = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": layer.mlp.ff,
                                                  "activation": "gelu_tanh"},
                                    rename={"gate_proj.weight": p + "mlp.gate", "up_proj.weight": p + "mlp.up",
                                            "down_proj.weight": p + "mlp.down"})
            ff_norm = PartSpec("same_norm")
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, mixer_norm=_rms_norm(H, cfg.eps, p + "norm1"),
                                feed_forward_norm=ff_norm, position=None, arrangement="parallel"))

    # the run order: a looped stretch runs `times` times, every pass with cache layers of its own and
    # a restart of the stream before its first layer
    n = len(cfg.layers)
    order: list[tuple[int, int | None]] = []
    if cfg.loop is None:
        order = [(i, None) for i in range(n)]
    else:
        lp = cfg.loop
        order = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            order += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        order += [(i, None) for i in range(lp.stop, n)]
    schedule = []
    for cache_layer, (i, pass_no) in enumerate(order):
        before = None
        if pass_no is not None:
            before = PartSpec("stream_restart", {"hidden_size": H, "rows": cfg.loop.times, "row": pass_no,
                                                 "add_embedding": pass_no > 0}, rename={"table": "loop.step"})
        schedule.append(ScheduleEntry(layer=i, cache=cache_layer, writes_cache=True, before=before))
    return ModelSpec(
        hidden_size=H,
        vocab_size=cfg.vocab,
        embedding=PartSpec("pair_hash_embedding", {"vocab_size": cfg.vocab, "hidden_size": H, "buckets": cfg.buckets,
                                                   "mul_prev": cfg.mul_prev, "mul_cur": cfg.mul_cur},
                           rename={"weight": "embed", "pair": "bigram"}),
        layers=tuple(layers),
        final_norm=_rms_norm(H, cfg.eps, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": H, "tied": True}),
        schedule=tuple(schedule),
        max_positions=None,
    )


register_architecture("Lilulix", LilulixConfig.from_json, assemble, replace=True)
