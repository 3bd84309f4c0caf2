"""A plain, slow implementation of the Lilulix decoder, for tests only.

Whole sequences, no cache, no batching, loops over heads and positions, one function per
mechanism, sharing no code with the package under test.  Everything runs on the CPU in the dtype
of the tensors it is given (tests use float64).

Notation: ``h`` is a sublayer's input ``[T, width]``; ``W x`` for a stored ``[out, in]`` matrix is
written ``x @ W.T``.  ``W`` is a dict of one sublayer's tensors by their local names.
"""

from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------------------- small pieces


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps) * w`` over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def bigram_rows(ids, buckets: int, mul_prev: int, mul_cur: int) -> list[int]:
    """Row of the bigram table for every token: a hash of (previous, current); the first token of
    a sequence takes the table's last row."""
    rows = []
    for t, cur in enumerate(ids):
        rows.append(buckets if t == 0 else (int(ids[t - 1]) * mul_prev + int(cur) * mul_cur) % buckets)
    return rows


def embed(table: torch.Tensor, bigram: torch.Tensor, ids, buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    tok = table[torch.as_tensor(list(ids), dtype=torch.long)]
    return tok + bigram[torch.as_tensor(bigram_rows(ids, buckets, mul_prev, mul_cur), dtype=torch.long)]


# ------------------------------------------------------------------------------- rotary


def rotate_half(x: torch.Tensor, positions, base: float, dims: int) -> torch.Tensor:
    """``x [T, ..., d]``: among the first ``dims`` dimensions, ``i`` pairs with ``i + dims/2`` and
    the pair turns by the angle ``p * base^(-2i/dims)``; the other dimensions pass."""
    out = x.clone()
    p = torch.as_tensor(list(positions), dtype=x.dtype)
    half = dims // 2
    shape = [x.shape[0]] + [1] * (x.dim() - 2)
    for i in range(half):
        ang = p * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


# ------------------------------------------------------------------------------- softmax with a sink


def sink_softmax(s: torch.Tensor, sink) -> torch.Tensor:
    """Weights ``exp(s_j) / (exp(sink) + sum_k exp(s_k))``: the sink takes part in the denominator
    only."""
    m = max(float(s.max()), float(sink))
    e = torch.exp(s - m)
    return e / (e.sum() + math.exp(float(sink) - m))


# ------------------------------------------------------------------------------- mixers


def latent_attention(h: torch.Tensor, W: dict, positions, *, heads: int, dim: int, rot_dim: int, vdim: int,
                     kv_rank: int, rot_base: float, rot_dims: int, scale: float, eps: float) -> torch.Tensor:
    """Attention whose keys and values are expanded from a low-rank latent: per token a latent
    ``c`` (normed) and one rotated key part shared by the heads; per head an unrotated key
    ``W_uk c`` and a value ``W_uv c``.  Causal, a learned sink per head in the softmax, a sigmoid
    gate on the heads' outputs."""
    T = h.shape[0]
    q = (h @ W["q"].T).reshape(T, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate_half(q[..., dim:], positions, rot_base, rot_dims)
    down = h @ W["dkv"].T
    c = rms_norm(down[:, :kv_rank], W["dkv.norm"], eps)
    k_rot = rotate_half(down[:, kv_rank:], positions, rot_base, rot_dims)          # [T, rot_dim]
    k_plain = (c @ W["uk"].T).reshape(T, heads, dim)
    v = (c @ W["uv"].T).reshape(T, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for hd in range(heads):
        for i in range(T):
            s = (k_plain[:i + 1, hd] @ q_plain[i, hd] + k_rot[:i + 1] @ q_rot[i, hd]) * scale
            out[i, hd] = sink_softmax(s, W["sink"][hd]) @ v[:i + 1, hd]
    gate = torch.sigmoid(h @ W["g"].T)
    return (out.reshape(T, heads * vdim) * gate) @ W["o"].T


def biased_attention(h: torch.Tensor, W: dict, *, heads: int, kv_heads: int, dim: int, scale: float,
                     eps: float) -> torch.Tensor:
    """Grouped attention without rotation whose values are the projected keys: queries and keys
    with biases and a per-head RMS norm (the values stay un-normed), scores lowered by
    ``slope_h * distance`` with ``slope_h = 2^(-8 (h + 1) / heads)``, causal, and one added to the
    softmax's denominator."""
    T = h.shape[0]
    q = (h @ W["q"].T + W["q.b"]).reshape(T, heads, dim)
    k = (h @ W["k"].T + W["k.b"]).reshape(T, kv_heads, dim)
    v = k
    q, k = rms_norm(q, W["q.norm"], eps), rms_norm(k, W["k.norm"], eps)
    per = heads // kv_heads
    out = torch.zeros(T, heads, dim, dtype=h.dtype)
    for hd in range(heads):
        g = hd // per
        slope = 2.0 ** (-8.0 * (hd + 1) / heads)
        for i in range(T):
            dist = torch.arange(i, -1, -1, dtype=h.dtype)
            s = (k[:i + 1, g] @ q[i, hd]) * scale - slope * dist
            out[i, hd] = sink_softmax(s, 0.0) @ v[:i + 1, g]
    return out.reshape(T, heads * dim) @ W["o"].T


# ------------------------------------------------------------------------------- feed-forward


def gated_mlp(h: torch.Tensor, W: dict) -> torch.Tensor:
    return (gelu_tanh(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


# ------------------------------------------------------------------------------- the model


def sub(weights: dict, prefix: str) -> dict:
    return {n[len(prefix):]: t for n, t in weights.items() if n.startswith(prefix)}


def run_order(n_layers: int, loop) -> list[tuple[int, int | None]]:
    """``(layer, pass number or None)``: a pass number stands at the first layer of each pass of
    the looped stretch."""
    if not loop:
        return [(i, None) for i in range(n_layers)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n_layers)]


def layer(cfg: dict, i: int, x: torch.Tensor, weights: dict, positions) -> torch.Tensor:
    spec, eps = cfg["layers"][i], cfg["norm"]["eps"]
    m = spec["mixer"]
    h = rms_norm(x, weights[f"l{i}.norm1"], eps)
    W = sub(weights, f"l{i}.mix.")
    if spec["type"] == "latent_attention":
        mixed = latent_attention(h, W, positions, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"],
                                 vdim=m["vdim"], kv_rank=m["kv_rank"], rot_base=m["rot"]["base"],
                                 rot_dims=m["rot"]["dims"], scale=m["scale"], eps=eps)
    elif spec["type"] == "attention":
        mixed = biased_attention(h, W, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], scale=m["scale"],
                                 eps=eps)
    else:
        raise ValueError(spec["type"])
    if spec.get("mlp") is None:
        return x + mixed
    return x + (mixed + gated_mlp(h, sub(weights, f"l{i}.mlp.")))


def forward(cfg: dict, weights: dict, ids, return_layers: bool = False):
    """Logits ``[T, vocab]`` of one sequence (and, on request, the stream after every layer run)."""
    big = cfg["embedding"]["bigram"]
    x0 = embed(weights["embed"], weights["bigram"], ids, big["buckets"], big["mul_prev"], big["mul_cur"])
    positions = list(range(len(ids)))
    x = x0
    seen = []
    for i, pass_no in run_order(len(cfg["layers"]), cfg.get("loop")):
        if pass_no is not None:
            if pass_no > 0:
                x = x + x0
            x = x + weights["loop.step"][pass_no]
        x = layer(cfg, i, x, weights, positions)
        seen.append(x)
    logits = rms_norm(x, weights["final.norm"], cfg["norm"]["eps"]) @ weights["embed"].T
    return (logits, torch.stack(seen)) if return_layers else logits
