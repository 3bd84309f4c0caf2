"""A plain, slow implementation of the Ruvurax decoder, for tests only.

Whole sequences, no cache, no batching, token-by-token loops where the mathematics is a
recurrence, one function per mechanism, sharing no code with the package under test.
Everything runs on the CPU in the dtype of the tensors it is given (tests use float64).

Notation: ``h`` is a mixer's or feed-forward's input ``[T, width]``; ``W x`` for a stored
``[out, in]`` matrix is written ``x @ W.T``.
"""

from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------------------- small pieces


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def embed(table: torch.Tensor, ids, scale: float) -> torch.Tensor:
    return table[torch.as_tensor(ids, dtype=torch.long)] * scale


# ------------------------------------------------------------------------------- rotary


def rotate_interleaved(x: torch.Tensor, positions, base: float, dims: int) -> torch.Tensor:
    """``x [T, heads, d]``: the first ``dims`` dimensions are rotated in pairs ``(2i, 2i+1)`` by
    the angle ``p * base^(-2i/dims)``; the others pass."""
    out = x.clone()
    p = torch.as_tensor(positions, dtype=x.dtype)
    for i in range(dims // 2):
        ang = p * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ------------------------------------------------------------------------------- mixers


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Per channel: ``out[t, c] = b[c] + sum_j w[c, j] x[t - (taps - 1 - j), c]``, zeros before
    the start (the last column of ``w`` meets the current token)."""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        acc = b.clone()
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                acc = acc + w[:, j] * x[src]
        out[t] = acc
    return out


def rglru_mixer(h: torch.Tensor, W: dict, blocks: int) -> torch.Tensor:
    """The gated linear recurrent block: ``y = gelu(W_y h + b)``, ``u = conv(W_x h + b)``,
    per block gates ``r, i``, ``a = exp(-8 r softplus(lam))``,
    ``S_t = a S_(t-1) + sqrt(1 - a^2) i u``, output ``W_o (S * y)``."""
    y = gelu_tanh(h @ W["y"].T + W["y.b"])
    u = causal_conv(h @ W["x"].T + W["x.b"], W["conv"], W["conv.b"])
    T, C = u.shape
    bw = C // blocks
    r = torch.empty_like(u)
    g = torch.empty_like(u)
    for b in range(blocks):
        ub = u[:, b * bw:(b + 1) * bw]
        r[:, b * bw:(b + 1) * bw] = torch.sigmoid(ub @ W["ra"][b].T + W["ra.b"][b])
        g[:, b * bw:(b + 1) * bw] = torch.sigmoid(ub @ W["ri"][b].T + W["ri.b"][b])
    log_a = -8.0 * r * torch.nn.functional.softplus(W["lam"])
    a = torch.exp(log_a)
    S = torch.zeros(C, dtype=h.dtype)
    out = torch.empty_like(u)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * g[t] * u[t]
        out[t] = S * y[t]
    return out @ W["o"].T


def windowed_attention(h: torch.Tensor, W: dict, positions, *, heads: int, kv_heads: int, dim: int,
                       vdim: int, rot_base: float, rot_dims: int, scale: float, window: int,
                       eps: float) -> torch.Tensor:
    """Softmax attention with a sliding window (``0 <= i - j < window``), rotary positions of the
    interleaved layout, unit-RMS queries and keys, and a sigmoid gate on the heads' output."""
    T = h.shape[0]
    q = (h @ W["q"].T).reshape(T, heads, dim)
    k = (h @ W["k"].T).reshape(T, kv_heads, dim)
    v = (h @ W["v"].T).reshape(T, kv_heads, vdim)
    q = unit_rms(rotate_interleaved(q, positions, rot_base, rot_dims), eps)
    k = unit_rms(rotate_interleaved(k, positions, rot_base, rot_dims), eps)
    per = heads // kv_heads
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for hd in range(heads):
        g = hd // per
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, hd]) * scale
            p = torch.softmax(s, dim=0)
            out[i, hd] = p @ v[lo:i + 1, g]
    gate = torch.sigmoid(h @ W["g"].T)
    return (out.reshape(T, heads * vdim) * gate) @ W["o"].T


def gated_linear_attention(h: torch.Tensor, W: dict, *, heads: int, dim: int, vdim: int, tau: float,
                           eps: float) -> torch.Tensor:
    """Per head ``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` with
    ``alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau)``; each head's output gets an RMS norm with a
    shared weight, the heads are gated by ``silu(W_g h)`` and projected."""
    T = h.shape[0]
    q = (h @ W["q"].T).reshape(T, heads, dim) * dim ** -0.5
    k = (h @ W["k"].T).reshape(T, heads, dim)
    v = (h @ W["v"].T).reshape(T, heads, vdim)
    z = ((h @ W["a1"].T) @ W["a2"].T + W["a2.b"]).reshape(T, heads, dim)
    alpha = torch.sigmoid(z) ** (1.0 / tau)
    S = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    o = torch.empty(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = unit_rms(o, eps) * W["norm"]
    gate = torch.nn.functional.silu(h @ W["g"].T)
    return (o.reshape(T, heads * vdim) * gate) @ W["o"].T


def sub(W: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def parallel_mixer(h: torch.Tensor, W: dict, positions, m: dict, eps: float) -> torch.Tensor:
    L, R = m["left"], m["right"]
    left = windowed_attention(h, sub(W, "left."), positions, heads=L["heads"], kv_heads=L["kv_heads"],
                              dim=L["dim"], vdim=L["vdim"], rot_base=L["rot"]["base"], rot_dims=L["rot"]["dims"],
                              scale=L["scale"], window=L["mask"]["size"], eps=eps)
    right = gated_linear_attention(h, sub(W, "right."), heads=R["heads"], dim=R["dim"], vdim=R["vdim"],
                                   tau=R["tau"], eps=eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ------------------------------------------------------------------------------- feed-forward


def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
                   limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def moe(h: torch.Tensor, W: dict, mlp: dict, margins: list | None = None) -> torch.Tensor:
    """Every token: the ``top`` experts with the largest router logits, weighted by the softmax
    over those logits alone, plus a shared expert.  ``margins`` collects, per token, how far the
    last chosen logit lies above the first one left out (a test must not rest on a close call)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ W["router"].T
    if margins is not None and top < E:
        ordered = torch.sort(z, dim=-1, descending=True).values
        margins.append(ordered[:, top - 1] - ordered[:, top])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        vals, idx = torch.topk(z[t], top)
        wts = torch.softmax(vals, dim=0)
        for wgt, e in zip(wts, idx.tolist()):
            out[t] += wgt * clamped_expert(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"],
                                           mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, W["shared.gate"], W["shared.up"], W["shared.down"], mlp["shared"]["limit"])
    return out


# ------------------------------------------------------------------------------- the model


def ruvurax_forward(state: dict, cfg: dict, tokens, dtype=torch.float64, return_layers: bool = False,
                    margins: list | None = None):
    """Logits ``[T, vocab]`` of one sequence from position 0 (and, on request, the residual stream
    after every layer)."""
    W = {k: v.to(dtype) for k, v in state.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = list(range(T))
    x = embed(W["embed"], tokens, cfg["embedding"]["scale"])
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        if layer["type"] == "rglru":
            mix = rglru_mixer(a, sub(W, p + "mix."), layer["mixer"]["blocks"])
        elif layer["type"] == "parallel":
            mix = parallel_mixer(a, sub(W, p + "mix."), positions, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            b = layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps)
            mix = mix + moe(b, sub(W, p + "mlp."), layer["mlp"], margins)
        x = x + mix
        streams.append(x)
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    if return_layers:
        return logits, torch.stack(streams)
    return logits
