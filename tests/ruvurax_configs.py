"""Small Ruvurax configurations and random weights for tests (none of them a real model's sizes).

The configurations differ from one another in every size: heads against key/value heads, key
against value size, sizes that are no multiple of 4 or 16, partial and full rotation, windows of
1, 9 and 40, one block and several, two and five convolution taps, one expert per token and all
of them, layers with and without experts, with and without a shared expert.
"""

from __future__ import annotations

import torch


def experts(n, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": n, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": shared}


def rglru(width, blocks, conv, mlp):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def parallel(*, heads, kv_heads, dim, vdim, window, rot_dims, rot_base, scale, r_heads, r_dim, r_vdim, tau,
             left_scale, right_scale, mlp):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                               "mask": {"size": window}, "rot": {"base": rot_base, "dims": rot_dims}, "scale": scale},
                      "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": tau},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def config(layers, *, vocab, width, scale, eps):
    return {"architecture": "Ruvurax", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # recurrent layers only: one without experts, one with a single expert per token and no shared one
    "R": config([rglru(40, 1, 2, None), rglru(36, 3, 5, experts(3, 1, 20, 0.8))],
                vocab=61, width=48, scale=2.0, eps=1e-5),
    # parallel layers: grouped heads, key and value sizes that differ, partial rotation, a short window
    "P": config([parallel(heads=4, kv_heads=2, dim=24, vdim=16, window=9, rot_dims=8, rot_base=100.0, scale=0.3,
                          r_heads=3, r_dim=20, r_vdim=24, tau=4.0, left_scale=0.7, right_scale=1.2,
                          mlp=experts(5, 2, 24, 0.7, {"ff": 40, "limit": 1.3})),
                 parallel(heads=1, kv_heads=1, dim=32, vdim=32, window=40, rot_dims=32, rot_base=5000.0, scale=0.2,
                          r_heads=1, r_dim=16, r_vdim=8, tau=9.0, left_scale=1.0, right_scale=0.5,
                          mlp=experts(4, 4, 16, 2.0))],
                vocab=53, width=40, scale=0.25, eps=1e-6),
    # both kinds mixed, odd sizes, a window that sees the token itself only
    "M": config([parallel(heads=3, kv_heads=3, dim=10, vdim=14, window=1, rot_dims=6, rot_base=30.0, scale=0.5,
                          r_heads=2, r_dim=12, r_vdim=36, tau=2.0, left_scale=0.9, right_scale=0.9, mlp=None),
                 rglru(24, 2, 3, experts(6, 3, 12, 1.0, {"ff": 8, "limit": 0.5})),
                 parallel(heads=6, kv_heads=2, dim=16, vdim=8, window=17, rot_dims=16, rot_base=1000.0, scale=0.25,
                          r_heads=2, r_dim=8, r_vdim=16, tau=16.0, left_scale=0.5, right_scale=1.5,
                          mlp=experts(2, 1, 32, 1.5, {"ff": 16, "limit": 1.0}))],
                vocab=47, width=36, scale=1.0, eps=1e-5),
}

PAGE_SIZE = {"R": 16, "P": 8, "M": 16}
DECAY_RANK = {"R": 4, "P": 5, "M": 3}


def random_state(cfg: dict, seed: int, rank: int = 4) -> dict[str, torch.Tensor]:
    """Random weights as a checkpoint would hold them (values that bfloat16 represents exactly, so
    that both engine dtypes and the float64 plain implementation start from the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    H = cfg["width"]

    def mat(*shape, std=None):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.1):
        return (mean + torch.randn(n, generator=g) * std).to(torch.bfloat16)

    st = {"embed": mat(cfg["vocab"], H, std=1.0), "head": mat(cfg["vocab"], H),
          "final.norm": vec(H, 1.0), "final.norm.b": vec(H)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        st[p + "norm1"], st[p + "norm1.b"] = vec(H, 1.0), vec(H)
        m = layer["mixer"]
        if layer["type"] == "rglru":
            C, B = m["width"], m["blocks"]
            bw = C // B
            st.update({p + "mix.y": mat(C, H), p + "mix.y.b": vec(C), p + "mix.x": mat(C, H), p + "mix.x.b": vec(C),
                       p + "mix.conv": mat(C, m["conv"], std=0.5), p + "mix.conv.b": vec(C),
                       p + "mix.ra": mat(B, bw, bw), p + "mix.ra.b": vec(B * bw).reshape(B, bw),
                       p + "mix.ri": mat(B, bw, bw), p + "mix.ri.b": vec(B * bw).reshape(B, bw),
                       p + "mix.lam": vec(C, -1.0, 1.0), p + "mix.o": mat(H, C)})
        else:
            L, R = m["left"], m["right"]
            q = p + "mix.left."
            st.update({q + "q": mat(L["heads"] * L["dim"], H), q + "k": mat(L["kv_heads"] * L["dim"], H),
                       q + "v": mat(L["kv_heads"] * L["vdim"], H), q + "g": mat(L["heads"] * L["vdim"], H),
                       q + "o": mat(H, L["heads"] * L["vdim"])})
            q = p + "mix.right."
            hk, hv = R["heads"] * R["dim"], R["heads"] * R["vdim"]
            st.update({q + "q": mat(hk, H), q + "k": mat(hk, H), q + "v": mat(hv, H), q + "g": mat(hv, H),
                       q + "o": mat(H, hv), q + "norm": vec(R["vdim"], 1.0), q + "a1": mat(rank, H),
                       q + "a2": mat(hk, rank), q + "a2.b": vec(hk, 1.0, 1.0)})
        mlp = layer.get("mlp")
        if mlp:
            st[p + "norm2"], st[p + "norm2.b"] = vec(H, 1.0), vec(H)
            q = p + "mlp."
            ff = mlp["expert"]["ff"]
            st[q + "router"] = mat(mlp["router"]["experts"], H, std=2.0 * H ** -0.5)
            for e in range(mlp["router"]["experts"]):
                st.update({f"{q}e{e}.gate": mat(ff, H, std=0.4), f"{q}e{e}.up": mat(ff, H, std=0.4),
                           f"{q}e{e}.down": mat(H, ff)})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                st.update({q + "shared.gate": mat(sf, H, std=0.4), q + "shared.up": mat(sf, H, std=0.4),
                           q + "shared.down": mat(H, sf)})
    return st


def prompt(cfg: dict, n: int, salt: int) -> list[int]:
    g = torch.Generator().manual_seed(1000 + salt)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
