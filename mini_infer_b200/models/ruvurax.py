"""``Ruvurax``: a decoder whose layers run a mixer and a mixture of experts in parallel on the same
stream (``x += mixer(norm1(x)) + experts(norm2(x))``, layer norms with bias), where a layer's mixer
is either a real-gated linear recurrent unit or, side by side, a gated sliding-window attention and
a gated linear attention.  The embedding is scaled; a final layer norm and an untied head follow.

This file is the only place that knows the architecture: it turns a ``RuvuraxConfig`` into a
``ModelSpec`` of generic parts and names the checkpoint tensors (``embed``, ``l{i}.norm1`` / ``.b``,
``l{i}.mix.*``, ``l{i}.mlp.*``, ``final.norm`` / ``.b``, ``head``).
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.ruvurax import ParallelMixerConfig, RecurrentUnitConfig, RuvuraxConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def _layer_norm(H: int, eps: float, name: str) -> PartSpec:
    return PartSpec("layernorm", {"hidden_size": H, "eps": eps}, rename={"weight": name, "bias": name + ".b"})


def assemble(cfg: RuvuraxConfig) -> ModelSpec:
    H = cfg.width
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        position = None
        if isinstance(m, RecurrentUnitConfig):
            mixer = PartSpec("rglru", {"hidden_size": H, "width": m.width, "blocks": m.blocks, "conv_taps": m.conv,
                                       "decay_scale": 8.0}, prefix=p + "mix.")
        else:
            assert isinstance(m, ParallelMixerConfig)
            L, R = m.left, m.right
            left = PartSpec("gated_window_attention",
                            {"hidden_size": H, "num_heads": L.heads, "num_kv_heads": L.kv_heads, "head_dim": L.dim,
                             "value_dim": L.vdim, "window": L.window, "scale": L.scale, "qk_unit_norm": True,
                             "eps": cfg.eps, "gate": "sigmoid"}, prefix="left.")
            right = PartSpec("gated_linear_attention",
                             {"hidden_size": H, "num_heads": R.heads, "key_dim": R.dim, "value_dim": R.vdim,
                              "tau": R.tau, "decay_rank": R.rank, "eps": cfg.eps}, prefix="right.")
            mixer = PartSpec("side_by_side", {"left": left, "right": right, "left_scale": m.left_scale,
                                              "right_scale": m.right_scale}, prefix=p + "mix.")
            if L.rot_dims:
                position = PartSpec("rotary_interleaved", {"head_dim": L.dim, "theta": L.rot_base,
                                                           "rotary_dim": L.rot_dims})
        if layer.mlp is None:
            feed_forward, ff_norm = PartSpec("no_feed_forward"), PartSpec("no_norm")
        else:
            e = layer.mlp
            feed_forward = PartSpec("routed_experts",
                                    {"hidden_size": H, "experts": e.experts, "top": e.top, "expert_ff": e.ff,
                                     "limit": e.limit, "alpha": 1.702, "shared_ff": e.shared_ff,
                                     "shared_limit": e.shared_limit}, prefix=p + "mlp.")
            ff_norm = _layer_norm(H, cfg.eps, p + "norm2")
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, mixer_norm=_layer_norm(H, cfg.eps, p + "norm1"),
                                feed_forward_norm=ff_norm, position=position, arrangement="parallel"))
    return ModelSpec(
        hidden_size=H,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": H,
                                               "scale": cfg.embedding_scale}, rename={"weight": "embed"}),
        layers=tuple(layers),
        final_norm=_layer_norm(H, cfg.eps, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": H, "tied": False},
                      rename={"weight": "head"}),
        max_positions=None,
    )


register_architecture("Ruvurax", RuvuraxConfig.from_json, assemble, replace=True)
