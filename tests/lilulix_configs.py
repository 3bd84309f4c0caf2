"""Small Lilulix configurations and random weights for tests (none of them a real model's sizes).

The configurations differ from one another in every size: one head and several, grouped and
ungrouped key/value heads, value sizes below and above the key size, sizes that are no multiple of
4, a rotated part that turns whole or in part, a loop at the start, in the middle and up to the last
layer, one pass and several, layers with and without a feed-forward, and no loop at all; some take
the tensor-core attention kernel in bfloat16 (D, E), the others the CUDA-core one.
"""

from __future__ import annotations

import torch


def latent(*, heads, dim, rot_dim, vdim, kv_rank, base, dims, scale, ff):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "rot": {"base": base, "dims": dims}, "scale": scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def biased(*, heads, kv_heads, dim, scale, ff):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, *, vocab, width, eps, buckets, mul_prev, mul_cur, loop):
    cfg = {"architecture": "Lilulix", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


CONFIGS = {
    # a loop over the first two layers, three passes; value size below the key size; grouped heads
    "A": config([latent(heads=3, dim=12, rot_dim=8, vdim=10, kv_rank=20, base=100.0, dims=8, scale=0.22, ff=24),
                 biased(heads=4, kv_heads=2, dim=16, scale=0.25, ff=None),
                 latent(heads=2, dim=8, rot_dim=4, vdim=16, kv_rank=30, base=5000.0, dims=4, scale=0.3, ff=40)],
                vocab=61, width=40, eps=1e-6, buckets=37, mul_prev=7, mul_cur=3, loop=(0, 2, 3)),
    # a loop up to the last layer; one head; a rotated part of which only some dimensions turn; large multipliers
    "B": config([biased(heads=6, kv_heads=6, dim=8, scale=0.35, ff=32),
                 latent(heads=1, dim=16, rot_dim=6, vdim=24, kv_rank=32, base=30.0, dims=4, scale=0.2, ff=None),
                 biased(heads=2, kv_heads=1, dim=20, scale=0.2, ff=16)],
                vocab=53, width=64, eps=1e-5, buckets=101, mul_prev=1000003, mul_cur=999983, loop=(1, 3, 2)),
    # no loop; odd sizes everywhere
    "C": config([latent(heads=5, dim=7, rot_dim=6, vdim=9, kv_rank=13, base=1000.0, dims=6, scale=0.27, ff=20),
                 biased(heads=3, kv_heads=3, dim=10, scale=0.3, ff=28)],
                vocab=47, width=36, eps=1e-5, buckets=5, mul_prev=2, mul_cur=9, loop=None),
    # a loop of one pass in the middle
    "D": config([biased(heads=2, kv_heads=2, dim=32, scale=0.18, ff=24),
                 latent(heads=4, dim=16, rot_dim=32, vdim=8, kv_rank=64, base=20000.0, dims=32, scale=0.17, ff=48),
                 biased(heads=8, kv_heads=2, dim=12, scale=0.28, ff=24)],
                vocab=80, width=48, eps=1e-6, buckets=64, mul_prev=13, mul_cur=1, loop=(1, 2, 1)),
    # many heads over one key/value head (several blocks of heads per token in the tensor-core kernel),
    # sizes that kernel takes, a loop over everything
    "E": config([latent(heads=16, dim=8, rot_dim=16, vdim=12, kv_rank=32, base=500.0, dims=16, scale=0.2, ff=32),
                 biased(heads=32, kv_heads=1, dim=32, scale=0.15, ff=None),
                 biased(heads=8, kv_heads=4, dim=64, scale=0.12, ff=32)],
                vocab=70, width=64, eps=1e-5, buckets=11, mul_prev=5, mul_cur=6, loop=(0, 3, 2)),
}

PAGE_SIZE = {"A": 16, "B": 8, "C": 16, "D": 32, "E": 16}


def random_state(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random weights as a checkpoint would hold them (values that bfloat16 represents exactly, so
    that both engine dtypes and the float64 plain implementation start from the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    H = cfg["width"]

    def mat(*shape, std=None):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.1):
        return (mean + torch.randn(n, generator=g) * std).to(torch.bfloat16)

    big = cfg["embedding"]["bigram"]
    st = {"embed": mat(cfg["vocab"], H, std=1.0), "bigram": mat(big["buckets"] + 1, H, std=0.5),
          "final.norm": vec(H, 1.0)}
    if cfg.get("loop"):
        st["loop.step"] = mat(cfg["loop"]["times"], H, std=0.5)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        st[p + "norm1"] = vec(H, 1.0)
        m = layer["mixer"]
        q = p + "mix."
        if layer["type"] == "latent_attention":
            n, R = m["heads"], m["kv_rank"]
            st.update({q + "q": mat(n * (m["dim"] + m["rot_dim"]), H, std=2.0 * H ** -0.5),
                       q + "dkv": mat(R + m["rot_dim"], H, std=2.0 * H ** -0.5), q + "dkv.norm": vec(R, 1.0),
                       q + "uk": mat(n * m["dim"], R, std=2.0 * R ** -0.5), q + "uv": mat(n * m["vdim"], R),
                       q + "sink": vec(n, 0.0, 1.5), q + "g": mat(n * m["vdim"], H, std=2.0 * H ** -0.5),
                       q + "o": mat(H, n * m["vdim"])})
        else:
            nq, nkv, d = m["heads"], m["kv_heads"], m["dim"]
            st.update({q + "q": mat(nq * d, H, std=2.0 * H ** -0.5), q + "q.b": vec(nq * d, 0.0, 0.3),
                       q + "k": mat(nkv * d, H, std=2.0 * H ** -0.5), q + "k.b": vec(nkv * d, 0.0, 0.3),
                       q + "q.norm": vec(d, 1.5, 0.3), q + "k.norm": vec(d, 1.5, 0.3), q + "o": mat(H, nq * d)})
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            st.update({p + "mlp.gate": mat(ff, H, std=2.0 * H ** -0.5), p + "mlp.up": mat(ff, H),
                       p + "mlp.down": mat(H, ff)})
    return st


def prompt(cfg: dict, n: int, salt: int) -> list[int]:
    g = torch.Generator().manual_seed(2000 + salt)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
