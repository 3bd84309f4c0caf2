"""Parts around attention in a latent space and attention with a distance bias: two mixers, an
embedding that adds a hashed token-pair row, and a stream part that restarts the stream between
two stretches of layers.

``LatentAttention`` keeps, per token, one low-rank latent and one rotated key part shared by all
heads, and computes attention in the latent's space: a head's query is mapped through that head's
key expansion once (``W_uk^T q``), scores are taken against the cached latents directly, the
weighted sum of latents is expanded to the head's value afterwards (``W_uv``).  Nothing but the
latent and the shared key part is ever cached or expanded per key.

``DistanceBiasAttention`` is grouped-query attention without rotation: scores fall linearly with
the distance between query and key, with a slope per head.

Both take a *sink*: a score per head that joins the softmax's denominator without a key or a
value (``"learned"``: a tensor; ``"zero"``: one is added to the denominator).
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import (KVNeed, LayerCache, ParamDecl, Part, PlanNeeds, StateNeed, StepContext, StreamPart, BranchSum,
                   register_embedding, register_mixer, register_stream_part)
from .builtin import _as_compute
from .mixers import ProjectedMixer, _f32


def _sink_kind(value) -> str | None:
    if value not in (None, "learned", "zero"):
        raise ValueError(f"unknown sink {value!r}: None, 'learned' or 'zero'")
    return value


class LatentAttention(ProjectedMixer):
    """Causal attention over keys and values that are linear expansions of a latent ``c`` of ``kv_rank``
    numbers per token: with ``H`` heads, per head ``head_dim`` unrotated and ``rot_dim`` rotated
    query/key dimensions and values of ``value_dim``,

    ``q = W_q h`` (per head ``[unrotated, rotated]``), ``[c_raw, r_raw] = W_dkv h``,
    ``c = rmsnorm(c_raw) * g``, ``r = rotate(r_raw)`` (one key part for all heads),
    ``score_h(i, j) = (q_h,un(i) . W_uk,h c(j) + rotate(q_h,rot(i)) . r(j)) * scale``,
    ``out_h(i) = sum_j p_h(i, j) W_uv,h c(j)``, heads gated by ``sigmoid(W_g h)`` (``gate``), then ``W_o``.

    The rotation is the half layout on the first ``rotary_dim`` of the ``rot_dim`` dimensions with base
    ``theta``.  The cache holds ``[c, r]`` per token and nothing else; the kernel reads a key's value
    from the key's own row.  Scores, softmax and sums are fp32 for either dtype.

    params: ``hidden_size``, ``num_heads``, ``head_dim``, ``rot_dim``, ``value_dim``, ``kv_rank``, ``theta``,
    ``rotary_dim``, ``scale``, ``eps``; optional ``sink`` (None, ``"learned"``, ``"zero"``), ``gate`` (None or
    ``"sigmoid"`` / ``"silu"``).
    tensors: ``q``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``o`` and, as asked, ``sink``, ``g``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        g = self.spec.params.get
        self.hidden = int(self.param("hidden_size"))
        self.heads = int(self.param("num_heads"))
        self.d, self.rd = int(self.param("head_dim")), int(self.param("rot_dim"))
        self.dv, self.rank = int(self.param("value_dim")), int(self.param("kv_rank"))
        self.theta = float(self.param("theta"))
        self.rot = int(g("rotary_dim") if g("rotary_dim") is not None else self.rd)
        self.scale = float(self.param("scale"))
        self.eps = float(self.param("eps"))
        self.sink = _sink_kind(g("sink"))
        self.gate = g("gate")
        if self.gate not in (None, "sigmoid", "silu"):
            raise ValueError(f"unknown gate {self.gate!r}")
        if self.rot % 2 or not 0 <= self.rot <= self.rd:
            raise ValueError(f"{self.rot} rotated dimensions of a part of {self.rd}")
        if min(self.heads, self.d, self.dv, self.rank) <= 0 or self.rd < 0:
            raise ValueError("a latent attention needs positive sizes")
        self.qh = self.d + self.rd                      # a head's columns of the query projection
        self.c_off = self.heads * self.qh
        self.g_off = self.c_off + self.rank + self.rd
        self.in_width = self.g_off + (self.heads * self.dv if self.gate else 0)
        self.out_width = self.heads * self.dv

    def param_decls(self):
        H, n = self.hidden, self.heads
        decls = {"q": ParamDecl((n * self.qh, H)), "dkv": ParamDecl((self.rank + self.rd, H)),
                 "dkv.norm": ParamDecl((self.rank,), "gain"), "uk": ParamDecl((n * self.d, self.rank)),
                 "uv": ParamDecl((n * self.dv, self.rank)), "o": ParamDecl((H, n * self.dv))}
        if self.sink == "learned":
            decls["sink"] = ParamDecl((n,), "table")
        if self.gate:
            decls["g"] = ParamDecl((n * self.dv, H))
        return decls

    def cache_need(self):
        return KVNeed(1, self.rank + self.rd, None, 0)     # keys only: the latent is key and value

    def plan_needs(self):
        tiles = {ops.ATTENTION_TILE_TOKENS} | ops.rows_attention_tile_sizes(self.heads, 1, self.rank + self.rd, self.rank, True)
        return PlanNeeds(frozenset(tiles))

    def bind(self, tensors, dtype, device):
        names = ["q", "dkv"] + (["g"] if self.gate else [])
        self.w_in = torch.cat([_as_compute(tensors[n], dtype) for n in names], dim=0).contiguous()
        self.w_out = _as_compute(tensors["o"], dtype).contiguous()
        n = self.heads
        # per head: W_uk^T [rank, head_dim] maps a query into the latent's space, W_uv [value_dim, rank]
        # expands a weighted sum of latents to the head's value
        self.uk_t = _as_compute(tensors["uk"], dtype).reshape(n, self.d, self.rank).transpose(1, 2).contiguous()
        self.uv = _as_compute(tensors["uv"], dtype).reshape(n, self.dv, self.rank).contiguous()
        self.c_gain = _f32(tensors["dkv.norm"])
        self.sinks = None
        if self.sink == "learned":
            self.sinks = _f32(tensors["sink"])
        elif self.sink == "zero":
            self.sinks = torch.zeros(n, dtype=torch.float32, device=device)
        i = torch.arange(self.rot // 2, dtype=torch.float64)
        self.freq = (self.theta ** (-2.0 * i / max(self.rot, 1))).to(device)
        self.finish_bind()

    def mix(self, proj, out, out_scale, ctx: StepContext, cache: LayerCache, position):
        if position is not None:
            raise ValueError("a latent attention rotates by itself and takes no position part")
        n, rank, dk = self.heads, self.rank, self.rank + self.rd
        M = ctx.n_tokens
        qfull = torch.empty((M, n, dk), dtype=proj.dtype, device=proj.device)
        group = ctx.groups[cache.group]
        ops.latent_prepare(proj, 0, n, self.qh, self.d, self.c_off, rank, self.rd, self.rot,
                           positions=ctx.positions, freq=self.freq, c_gain=self.c_gain, eps=self.eps, qfull=qfull,
                           slots=group.slots if cache.writes else None, kcache=cache.k if cache.writes else None)
        q_un = proj[:, :n * self.qh].unflatten(1, (n, self.qh))[:, :, :self.d]
        ops.batched_linear(q_un, self.uk_t, qfull[:, :, :rank])
        latent = torch.empty((M, n * rank), dtype=proj.dtype, device=proj.device)
        ops.attention_ext(qfull.view(M, n * dk), latent, cache, ctx, n, 1, dk, rank, self.scale, sinks=self.sinks,
                          values_in_keys=True)
        heads = torch.empty((M, n, self.dv), dtype=proj.dtype, device=proj.device)
        ops.batched_linear(latent.view(M, n, rank), self.uv, heads)
        heads = heads.view(M, n * self.dv)
        if self.gate:
            ops.gate_mul(heads, proj[:, self.g_off:self.g_off + n * self.dv], out, self.gate, out_scale)
        elif out_scale == 1.0:
            out.copy_(heads)
        else:
            raise ValueError("an ungated attention cannot scale its output")


def distance_slopes(heads: int, exponent_span: float = 8.0) -> torch.Tensor:
    """``2^(-span (h + 1) / heads)`` for head ``h = 0 .. heads - 1`` (fp32, rounded once from float64)."""
    h = torch.arange(1, heads + 1, dtype=torch.float64)
    return (2.0 ** (-exponent_span * h / heads)).to(torch.float32)


class DistanceBiasAttention(ProjectedMixer):
    """Causal grouped-query attention without rotation: ``score_h(i, j) = q_h(i) . k(j) * scale -
    slope_h * (i - j)`` with ``slope_h = 2^(-slope_span (h + 1) / heads)``.  Queries and keys may have
    biases (``qk_bias``) and an RMS norm over the head with one gain shared by the heads
    (``qk_norm``).  With ``values_are_keys`` there is no value projection: a key's value is the key as
    projected (with its bias), before the norm.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``; optional ``value_dim``
    (default ``head_dim``), ``qk_bias`` and ``qk_norm`` (default False) with ``eps``, ``values_are_keys``
    (default False), ``slope_span`` (default 8; None: no distance bias), ``sink`` (None, ``"learned"``, ``"zero"``).
    tensors: ``q``, ``k``, ``o``; as asked ``v``, ``q.b``, ``k.b``, ``q.norm``, ``k.norm``, ``sink``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        g = self.spec.params.get
        self.hidden = int(self.param("hidden_size"))
        self.nq, self.nkv = int(self.param("num_heads")), int(self.param("num_kv_heads"))
        self.d = int(self.param("head_dim"))
        self.values_are_keys = bool(g("values_are_keys", False))
        self.dv = int(g("value_dim") or self.d)
        self.scale = float(self.param("scale"))
        self.qk_bias, self.qk_norm = bool(g("qk_bias", False)), bool(g("qk_norm", False))
        self.eps = float(g("eps", 0.0))
        span = g("slope_span", 8.0)
        self.slope_span = None if span is None else float(span)
        self.sink = _sink_kind(g("sink"))
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads cannot share {self.nkv} key/value heads")
        if self.values_are_keys and self.dv != self.d:
            raise ValueError(f"values that are the keys have the keys' size {self.d}, not {self.dv}")
        if not (0 < self.d <= 256 and 0 < self.dv <= 256):
            raise ValueError(f"head sizes {self.d} and {self.dv} must lie in [1, 256]")
        self.q_off, self.k_off = 0, self.nq * self.d
        self.v_off = self.k_off + self.nkv * self.d
        self.in_width = self.v_off + (0 if self.values_are_keys else self.nkv * self.dv)
        self.out_width = self.nq * self.dv

    def param_decls(self):
        H, nq, nkv, d, dv = self.hidden, self.nq, self.nkv, self.d, self.dv
        decls = {"q": ParamDecl((nq * d, H)), "k": ParamDecl((nkv * d, H)), "o": ParamDecl((H, nq * dv))}
        if not self.values_are_keys:
            decls["v"] = ParamDecl((nkv * dv, H))
        if self.qk_bias:
            decls["q.b"], decls["k.b"] = ParamDecl((nq * d,), "table"), ParamDecl((nkv * d,), "table")
        if self.qk_norm:
            decls["q.norm"], decls["k.norm"] = ParamDecl((d,), "gain"), ParamDecl((d,), "gain")
        if self.sink == "learned":
            decls["sink"] = ParamDecl((nq,), "table")
        return decls

    def cache_need(self):
        return KVNeed(self.nkv, self.d, None, None if self.dv == self.d else self.dv)

    def plan_needs(self):
        tiles = {ops.ATTENTION_TILE_TOKENS} | ops.rows_attention_tile_sizes(self.nq, self.nkv, self.d, self.dv, False)
        if self.d == self.dv and self.d in (64, 128):      # sizes the tcgen05 prefill kernel takes
            tiles.add(ops.prefill_tc_tile_tokens(self.nq // self.nkv))
        return PlanNeeds(frozenset(tiles))

    def bind(self, tensors, dtype, device):
        names = ["q", "k"] + ([] if self.values_are_keys else ["v"])
        self.w_in = torch.cat([_as_compute(tensors[n], dtype) for n in names], dim=0).contiguous()
        self.w_out = _as_compute(tensors["o"], dtype).contiguous()
        self.q_bias = _f32(tensors["q.b"]) if self.qk_bias else None
        self.k_bias = _f32(tensors["k.b"]) if self.qk_bias else None
        self.q_gain = _f32(tensors["q.norm"]) if self.qk_norm else None
        self.k_gain = _f32(tensors["k.norm"]) if self.qk_norm else None
        self.slopes = None if self.slope_span is None else distance_slopes(self.nq, self.slope_span).to(device)
        self.sinks = None
        if self.sink == "learned":
            self.sinks = _f32(tensors["sink"])
        elif self.sink == "zero":
            self.sinks = torch.zeros(self.nq, dtype=torch.float32, device=device)
        self.finish_bind()

    def mix(self, proj, out, out_scale, ctx: StepContext, cache: LayerCache, position):
        if position is not None:
            raise ValueError("this attention takes no position part: positions enter through the distance bias")
        if out_scale != 1.0:
            raise ValueError("this attention cannot scale its output")
        nq, nkv, d, dv = self.nq, self.nkv, self.d, self.dv
        group = ctx.groups[cache.group]
        ops.qk_bias_norm_store(proj, self.q_off, self.k_off, self.v_off, nq, nkv, d, dv,
                               q_bias=self.q_bias, k_bias=self.k_bias, q_gain=self.q_gain, k_gain=self.k_gain,
                               eps=self.eps, values_are_keys=self.values_are_keys,
                               slots=group.slots if cache.writes else None,
                               kcache=cache.k if cache.writes else None, vcache=cache.v if cache.writes else None)
        ops.attention_ext(proj[:, self.q_off:self.q_off + nq * d], out, cache, ctx, nq, nkv, d, dv, self.scale,
                          sinks=self.sinks, slopes=self.slopes)


# ----------------------------------------------------------------------------- embedding


class PairHashEmbedding(Part):
    """``h0 = E[token] + P[row]`` in fp32, which is then the residual stream itself: ``row = (previous
    token * mul_prev + token * mul_cur) mod buckets`` of a second table ``P [buckets + 1, hidden]``,
    whose last row stands for "no previous token" (a sequence's first token).  The previous token of
    a portion's first token is per-request state (int32, one number), kept by the cache manager.

    params: ``vocab_size``, ``hidden_size``, ``buckets``, ``mul_prev``, ``mul_cur``.
    tensors: ``weight [vocab, hidden]``, ``pair [buckets + 1, hidden]``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.buckets = int(self.param("buckets"))
        self.mul_prev, self.mul_cur = int(self.param("mul_prev")), int(self.param("mul_cur"))
        if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("a pair hash needs a positive bucket count and non-negative multipliers")

    def param_decls(self):
        V, H = int(self.param("vocab_size")), int(self.param("hidden_size"))
        return {"weight": ParamDecl((V, H)), "pair": ParamDecl((self.buckets + 1, H))}

    def state_need(self):
        return StateNeed((1,), torch.int32)

    def bind(self, tensors, dtype, device):
        self.weight = _as_compute(tensors["weight"], dtype).contiguous()
        self.pair = _as_compute(tensors["pair"], dtype).contiguous()

    def forward(self, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        if cache.state is None:
            raise ValueError("this embedding needs its per-request state (the previous token)")
        return ops.embedding_pair_hash(self.weight, self.pair, ctx, cache.state, self.buckets, self.mul_prev,
                                       self.mul_cur)


# ----------------------------------------------------------------------------- stream part


class StreamRestart(StreamPart):
    """Before a stretch of layers: the embedding's output is added to the stream once more
    (``add_embedding``) and so is row ``row`` of a table ``[rows, hidden]``.  Nothing is launched: both
    ride, unrounded, on what the next norm adds to the fp32 stream.

    params: ``hidden_size``, ``rows``, ``row``, ``add_embedding``.  tensors: ``table [rows, hidden]``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.row, self.rows = int(self.param("row")), int(self.param("rows"))
        self.needs_embedding = bool(self.spec.params.get("add_embedding", False))
        if not 0 <= self.row < self.rows:
            raise ValueError(f"row {self.row} of a table of {self.rows}")

    def param_decls(self):
        return {"table": ParamDecl((self.rows, int(self.param("hidden_size"))), "table")}

    def bind(self, tensors, dtype, device):
        self.vector = _f32(tensors["table"][self.row])

    def forward(self, x, residual, ctx, embedded):
        if residual is None:                 # before the first layer: the embedding's output is the stream
            if isinstance(x, BranchSum) or x.dtype != torch.float32:
                raise ValueError("a stream part before the first layer needs an fp32 embedding output")
            residual, parts = x, ()
        else:
            parts = tuple(x) if isinstance(x, BranchSum) else (x,)
            if isinstance(x, BranchSum) and (x.stream_add is not None or x.row_add is not None):
                raise ValueError("two stream parts in a row")
        pending = BranchSum(parts)
        pending.row_add = self.vector
        if self.needs_embedding:
            if embedded is None:
                raise ValueError("the embedding's output was not kept")
            pending.stream_add = embedded
        return pending, residual


register_mixer("latent_attention", LatentAttention, replace=True)
register_mixer("distance_bias_attention", DistanceBiasAttention, replace=True)
register_embedding("pair_hash_embedding", PairHashEmbedding, replace=True)
register_stream_part("stream_restart", StreamRestart, replace=True)
