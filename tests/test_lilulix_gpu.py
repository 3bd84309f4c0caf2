"""The Lilulix architecture in the engine against the plain implementation (``plain_lilulix``):
every mechanism alone at the kernel level, then whole models of four small configurations under
every way of cutting the work, in float32 and bfloat16, long decoding with captured steps, and
greedy generation through the scheduler.  Weights and inputs are made so that a fault shows: a key
that stands out hundreds of tokens back and at a page's border, a sink that takes nearly all the
weight, caches filled with NaN where nothing was written, slots that are used again."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_lilulix as P
import trace_util as T
from lilulix_configs import CONFIGS, PAGE_SIZE, prompt, random_state

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LENGTHS = {"A": [1, 2, 37, 70], "B": [3, 19, 64, 90, 41], "C": [50, 5, 33, 81], "D": [66, 1, 45], "E": [130, 7, 65, 64]}


def ops():
    from mini_infer_b200.csrc import ops as o
    return o


def requests_for(which):
    return {f"r{i}": prompt(CONFIGS[which], n, salt=i) for i, n in enumerate(LENGTHS[which])}


_plain_cache = {}


def plain_for(which):
    if which not in _plain_cache:
        cfg = CONFIGS[which]
        state = random_state(cfg, seed=17)
        wide = {k: v.double() for k, v in state.items()}
        logits = {rid: P.forward(cfg, wide, toks).numpy() for rid, toks in requests_for(which).items()}
        _plain_cache[which] = (state, wide, logits)
    return _plain_cache[which]


def make_runner(which, dtype, steps=None, num_blocks=None, max_requests=4, cuda_graph=False):
    from mini_infer_b200.engine import ModelRunner

    state, _, _ = plain_for(which)
    ps = PAGE_SIZE[which]
    if num_blocks is None:
        num_blocks = T.max_tokens_needed(steps) // ps
    runner = ModelRunner.from_state_dict(CONFIGS[which], state, dtype=dtype, block_size=ps, num_blocks=num_blocks,
                                         max_requests=max_requests, cuda_graph=cuda_graph)
    for st in runner.cache.storage:
        st.fill_(float("nan"))            # a slot that was never written must never be read
    for arena in runner.cache.state_arenas.values():
        arena.fill_(-12345)               # the previous token of a sequence's first token must never be read
    return runner


def compare(which, dtype, got):
    _, _, want = plain_for(which)
    scale = max(float(np.abs(w).max()) for w in want.values())
    tol = T.tolerance(dtype, scale)
    for rid, w in want.items():
        assert got[rid].shape == w.shape
        assert np.isfinite(got[rid]).all(), f"{rid}: non-finite logits"
        bad = T.first_bad(got[rid], w, tol)
        assert bad is None, f"{which} {dtype} {rid}: position {bad} differs by " \
                            f"{np.abs(got[rid][bad] - w[bad]).max():.3g} (bound {float(tol):.3g})"


CUTTINGS = {"whole": T.cut_whole, "last_decoded": T.cut_last_decoded, "portions": T.cut_portions,
            "mixed": T.cut_mixed}


@pytest.mark.parametrize("cutting", list(CUTTINGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(CONFIGS))
def test_engine_matches_plain_under_every_cutting(which, dtype, cutting):
    """Whole prompts, prefill then token-by-token decoding, portions down to two tokens, and mixed
    batches of unequal requests in which slots and pages are freed and used again."""
    requests = requests_for(which)
    steps = CUTTINGS[cutting](requests)
    runner = make_runner(which, dtype, steps)
    got = T.collect(steps, T.replay_in_process(runner, steps), CONFIGS[which]["vocab"])
    runner.cache.check()
    assert runner.cache.num_requests == 0
    for gi, pool in enumerate(runner.cache.pools):
        assert runner.cache.num_free_pages(gi) == pool.num_pages
    compare(which, dtype, got)


@pytest.mark.parametrize("which", list(CONFIGS))
def test_float32_logits_do_not_depend_on_the_cutting(which):
    """In float32 every sum runs in an order that depends on the position alone: the logits of a
    position are the same bits whole, in portions, decoded, or beside other requests."""
    requests = requests_for(which)
    results = {}
    for name, cut in CUTTINGS.items():
        steps = cut(requests)
        runner = make_runner(which, "float32", steps)
        results[name] = T.collect(steps, T.replay_in_process(runner, steps), CONFIGS[which]["vocab"])
    for name in ("last_decoded", "portions", "mixed"):
        for rid in requests:
            assert np.array_equal(results[name][rid], results["whole"][rid]), f"{which} {name} {rid}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_kernel_by_kernel_and_as_captured_steps(dtype):
    """A short prompt, then 150 tokens one by one across many pages, kernel by kernel and as
    captured graphs (the previous token and every cache row come from device memory)."""
    from mini_infer_b200.engine import StepEntry

    which = "A"
    cfg = CONFIGS[which]
    _, wide, _ = plain_for(which)
    toks = prompt(cfg, 156, salt=77)
    want = P.forward(cfg, wide, toks).numpy()
    tol = T.tolerance(dtype, float(np.abs(want).max()))
    for graph in (False, True):
        runner = make_runner(which, dtype, num_blocks=12, cuda_graph=graph)
        runner.add_request("a")
        rows = [runner.step([StepEntry("a", toks[:6], list(range(6)))]).logits.cpu().numpy()]
        for t in toks[6:]:
            rows.append(runner.step([StepEntry("a", [t], [0])]).logits.cpu().numpy())
        got = np.concatenate(rows)
        assert T.first_bad(got, want, tol) is None
        if graph:
            assert any(s.replays > 100 for s in runner.stepper._graphs.values())
        runner.free_request("a")
        runner.cache.check()


def test_greedy_generation_through_the_scheduler():
    """Greedy tokens from the engine's own entry point (scheduler, sampler, cache) equal the plain
    implementation's, fed its own tokens, for several prompts generated together."""
    from mini_infer_b200.engine import ContinuousScheduler, Request
    from mini_infer_b200.sampling import SamplingParams

    which = "B"
    cfg = CONFIGS[which]
    _, wide, _ = plain_for(which)
    prompts = [prompt(cfg, n, salt=200 + i) for i, n in enumerate([4, 21, 9])]
    n_new = 12
    runner = make_runner(which, "float32", num_blocks=32)
    sched = ContinuousScheduler(runner, max_concurrent=3, max_tokens_per_step=16)
    results = sched.generate([Request(prompt=p, sampling_params=SamplingParams(), max_tokens=n_new) for p in prompts])
    sched.stop()
    for p, r in zip(prompts, results):
        assert len(r.tokens) == n_new
        seq = list(p)
        for tok in r.tokens:
            logits = P.forward(cfg, wide, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) > 1e-3:     # the plain choice is not a close call
                assert tok == int(logits.argmax()), f"after {len(seq)} tokens"
            seq.append(tok)
    runner.cache.check()
    assert runner.cache.num_requests == 0


# ----------------------------------------------------------------------------- mechanisms alone


def rnd(*shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def i32(a):
    return torch.tensor(np.asarray(a, dtype=np.int32), device=DEV)


def ctx_for(q_lens, slots, tokens, positions):
    starts = np.concatenate([[0], np.cumsum(q_lens)[:-1]]).astype(np.int32)
    return SimpleNamespace(q_start=i32(starts), q_len=i32(q_lens), state_slot=i32(slots), n_requests=len(q_lens),
                           token_ids=i32(tokens), positions=i32(positions))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_hash_embedding_carries_the_previous_token(dtype):
    """Two sequences fed in portions of 1, 2 and more tokens that share launches: the row of the pair
    table follows the previous token across portions, the first token takes the last row whatever
    the slot held before, and products beyond 32 bits are hashed exactly."""
    V, H, buckets, mp, mc = 50021, 24, 97, 1000003, 999983
    table, pair = rnd(V, H, seed=1).to(dtype), rnd(buckets + 1, H, seed=2).to(dtype)
    seqs = {0: [50020, 49999, 3, 50020, 50020, 7, 41234, 0, 12], 1: [5, 50001, 50001, 9, 30000]}
    want = {r: P.embed(table.double(), pair.double(), s, buckets, mp, mc) for r, s in seqs.items()}
    state = torch.full((4, 1), 31337, dtype=torch.int32, device=DEV)       # left over from earlier requests
    slots = {0: 3, 1: 1}
    cuts = [(1, 2), (2, 1), (1, 0), (3, 1), (2, 1)]
    done = {0: 0, 1: 0}
    got = {0: [], 1: []}
    for n0, n1 in cuts:
        who = [r for r, n in ((0, n0), (1, n1)) if n]
        lens = [n for n in (n0, n1) if n]
        toks = sum((seqs[r][done[r]:done[r] + n] for r, n in zip(who, lens)), [])
        pos = sum((list(range(done[r], done[r] + n)) for r, n in zip(who, lens)), [])
        ctx = ctx_for(lens, [slots[r] for r in who], toks, pos)
        out = ops().embedding_pair_hash(table.to(DEV), pair.to(DEV), ctx, state, buckets, mp, mc)
        assert out.dtype == torch.float32
        row = 0
        for r, n in zip(who, lens):
            got[r].append(out[row:row + n].cpu().double())
            row += n
            done[r] += n
    for r in seqs:
        assert done[r] == len(seqs[r])
        assert torch.allclose(torch.cat(got[r]), want[r], atol=1e-6), f"sequence {r}"
    assert state[3, 0].item() == seqs[0][-1] and state[1, 0].item() == seqs[1][-1]
    assert state[0, 0].item() == 31337 and state[2, 0].item() == 31337       # other slots are never touched


@pytest.mark.parametrize("dtype,bound", [(torch.float32, 2e-6), (torch.bfloat16, 1 / 128)])
def test_rms_norm_of_a_stream_with_several_addends(dtype, bound):
    M, H = 7, 50
    stream, x0, row = rnd(M, H, seed=1, scale=3.0), rnd(M, H, seed=8), rnd(H, seed=9)
    a1, a2 = rnd(M, H, seed=2, dtype=dtype), rnd(M, H, seed=3, dtype=dtype)
    gain = rnd(H, seed=4) + 1
    r = stream.double() + a1.double() + a2.double() + x0.double() + row.double()
    before = stream.to(DEV).clone()
    s = before.clone()
    out, new = ops().add_rmsnorm_multi(s, [a1.to(DEV), a2.to(DEV)], gain.to(DEV), 1e-5, dtype, add32=x0.to(DEV),
                                       row_add=row.to(DEV))
    assert torch.equal(s, before)                                    # the stream that came in is left alone
    assert torch.allclose(new.cpu().double(), r, atol=2e-6)
    want = P.rms_norm(r, gain.double(), 1e-5)
    assert (out.cpu().double() - want).abs().max() <= bound * max(1.0, want.abs().max())
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out, none = ops().add_rmsnorm_multi(s, [a1.to(DEV)], gain.to(DEV), 1e-5, dtype, rows=rows)
    want = P.rms_norm((stream.double() + a1.double())[[5, 0, 5]], gain.double(), 1e-5)
    assert none is None and (out.cpu().double() - want).abs().max() <= bound * max(1.0, want.abs().max())
    out, new = ops().add_rmsnorm_multi(s, [], gain.to(DEV), 1e-5, dtype, row_add=row.to(DEV))      # a restart before layer 0
    assert torch.allclose(new.cpu().double(), stream.double() + row.double(), atol=1e-6)


@pytest.mark.parametrize("M,I,H", [(3, 24, 40), (16, 64, 64), (40, 20, 36), (200, 256, 128)])
@pytest.mark.parametrize("dtype,bound", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_gated_feed_forward_with_the_tanh_gelu(M, I, H, dtype, bound):
    """Both routes of the gate/up product (the streaming product's epilogue for few rows, a kernel of
    its own behind the library product otherwise) against the plain feed-forward."""
    from mini_infer_b200.parts.base import build_part
    from mini_infer_b200.parts.spec import PartSpec

    W = {"gate": rnd(I, H, seed=1, scale=0.5).to(dtype), "up": rnd(I, H, seed=2, scale=0.3).to(dtype),
         "down": rnd(H, I, seed=3, scale=0.2).to(dtype)}
    x = rnd(M, H, seed=4, scale=1.5).to(dtype)
    part = build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I,
                                                            "activation": "gelu_tanh"}))
    part.bind({"gate_proj.weight": W["gate"].to(DEV), "up_proj.weight": W["up"].to(DEV),
               "down_proj.weight": W["down"].to(DEV)}, dtype, torch.device(DEV))
    got = part.forward(x.to(DEV), None).cpu().double()
    want = P.gated_mlp(x.double(), {k: v.double() for k, v in W.items()})
    assert (got - want).abs().max() <= bound * max(1.0, want.abs().max())
    g = rnd(M, 2 * I, seed=5, scale=2.0).to(dtype)
    got = ops().glu_mul_pairs(g.to(DEV), "gelu_tanh").cpu().double()
    want = P.gelu_tanh(g.double()[:, 0::2]) * g.double()[:, 1::2]
    assert (got - want).abs().max() <= (1e-6 if dtype == torch.float32 else 1 / 128) * max(1.0, want.abs().max())


@pytest.mark.parametrize("d,nq,nkv", [(16, 4, 2), (10, 3, 3), (48, 2, 1), (7, 1, 1), (256, 2, 2)])
def test_query_key_bias_norm_and_values_that_are_keys(d, nq, nkv):
    """Bias, then an RMS norm per head with a shared gain, written back in place; the key page holds
    the normed key, the value page the key as projected (with its bias), before the norm."""
    M, page = 9, 4
    width = (nq + nkv) * d + 3
    packed = rnd(M, width, seed=8)
    qb, kb = rnd(nq * d, seed=9, scale=0.3), rnd(nkv * d, seed=10, scale=0.3)
    qg, kg = rnd(d, seed=11, scale=0.2) + 1.5, rnd(d, seed=12, scale=0.2) + 1.5
    kc = torch.full((5, nkv, page, d), float("nan"), device=DEV)
    vc = torch.full((5, nkv, page, d), float("nan"), device=DEV)
    slots = [17, 2, 3, 0, 9, 10, 11, 4, 19]
    dev = packed.to(DEV).clone()
    ops().qk_bias_norm_store(dev, 0, nq * d, 0, nq, nkv, d, d, q_bias=qb.to(DEV), k_bias=kb.to(DEV), q_gain=qg.to(DEV),
                             k_gain=kg.to(DEV), eps=1e-5, values_are_keys=True, slots=i32(slots), kcache=kc, vcache=vc)
    got = dev.cpu().double()
    x = packed.double()
    q_raw = (x[:, :nq * d] + qb.double()).reshape(M, nq, d)
    k_raw = (x[:, nq * d:(nq + nkv) * d] + kb.double()).reshape(M, nkv, d)
    q_want, k_want = P.rms_norm(q_raw, qg.double(), 1e-5), P.rms_norm(k_raw, kg.double(), 1e-5)
    assert torch.allclose(got[:, :nq * d], q_want.reshape(M, -1), atol=2e-5)
    assert torch.allclose(got[:, nq * d:(nq + nkv) * d], k_want.reshape(M, -1), atol=2e-5)
    assert torch.equal(got[:, (nq + nkv) * d:], x[:, (nq + nkv) * d:])
    keys, values = ops().unpack_cache_pages(kc).cpu().double(), ops().unpack_cache_pages(vc).cpu().double()
    for t, s in enumerate(slots):
        assert torch.allclose(keys[s], k_want[t], atol=2e-5) and torch.allclose(values[s], k_raw[t], atol=2e-6)
    untouched = [s for s in range(20) if s not in slots]
    assert torch.isnan(keys[untouched]).all() and torch.isnan(values[untouched]).all()


@pytest.mark.parametrize("n,d,rd,rot,rank", [(3, 12, 8, 8, 20), (1, 16, 6, 4, 32), (5, 7, 6, 6, 13), (2, 64, 32, 32, 96)])
def test_latent_rows_and_rotated_query_parts(n, d, rd, rot, rank):
    """The latent's norm, the half-layout rotation of the shared key part and of every head's rotated
    part at small and large positions, and the cache row ``[latent, rotated key part]``."""
    M, page, base = 7, 4, 300.0
    qh = d + rd
    width = n * qh + rank + rd + 5
    packed = rnd(M, width, seed=8)
    gain = rnd(rank, seed=9, scale=0.2) + 1.0
    pos = [0, 1, 2, 100, 4095, 7, 70000]
    slots = [3, 4, 5, 0, 13, 14, 8]
    kc = torch.full((4, 1, page, rank + rd), float("nan"), device=DEV)
    qfull = torch.full((M, n, rank + rd), float("nan"), device=DEV)
    freq = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).to(DEV)
    dev = packed.to(DEV).clone()
    ops().latent_prepare(dev, 0, n, qh, d, n * qh, rank, rd, rot, positions=i32(pos), freq=freq, c_gain=gain.to(DEV),
                         eps=1e-5, qfull=qfull, slots=i32(slots), kcache=kc)
    assert torch.equal(dev.cpu(), packed)                            # the projection itself is only read
    x = packed.double()
    c = P.rms_norm(x[:, n * qh:n * qh + rank], gain.double(), 1e-5)
    kr = P.rotate_half(x[:, n * qh + rank:n * qh + rank + rd], pos, base, rot)
    qr = P.rotate_half(x[:, :n * qh].reshape(M, n, qh)[..., d:], pos, base, rot)
    rows = ops().unpack_cache_pages(kc).cpu().double()[:, 0]
    for t, s in enumerate(slots):
        assert torch.allclose(rows[s, :rank], c[t], atol=2e-5) and torch.allclose(rows[s, rank:], kr[t], atol=2e-5)
    assert torch.allclose(qfull[:, :, rank:].cpu().double(), qr, atol=2e-5)
    assert torch.isnan(qfull[:, :, :rank]).all()                     # the caller fills the latent part


def attention_fixture(nq, nkv, d, n_tokens, page, portions, latent_rank=0, dtype="float32"):
    """A runner with one attention layer, a request fed in ``portions``, and per portion the step's
    context and the layer's cache, so that a test can put rows of its own into the pages."""
    from mini_infer_b200.engine import ModelRunner
    from lilulix_configs import biased, config, latent

    if latent_rank:
        layer = latent(heads=nq, dim=4, rot_dim=d - latent_rank, vdim=4, kv_rank=latent_rank, base=10.0,
                       dims=d - latent_rank, scale=1.0, ff=None)
    else:
        layer = biased(heads=nq, kv_heads=nkv, dim=d, scale=1.0, ff=None)
    cfg = config([layer], vocab=8, width=16, eps=1e-6, buckets=3, mul_prev=1, mul_cur=1, loop=None)
    runner = ModelRunner.from_state_dict(cfg, random_state(cfg, seed=3), dtype=dtype, block_size=page,
                                         num_blocks=-(-n_tokens // page) + 1, max_requests=2)
    for st in runner.cache.storage:
        st.fill_(float("nan"))
    runner.add_request("filler")          # so that the request under test does not sit in slot 0
    runner.add_request("a")
    return runner


def plain_scores_attention(q, k, v, scale, slopes, sinks):
    T_, nq, _ = q.shape
    per = nq // k.shape[1]
    out = torch.zeros(T_, nq, v.shape[2], dtype=torch.float64)
    for h in range(nq):
        for i in range(T_):
            dist = torch.arange(i, -1, -1, dtype=torch.float64)
            s = (k[:i + 1, h // per] @ q[i, h]) * scale - slopes[h] * dist
            out[i, h] = P.sink_softmax(s, sinks[h]) @ v[:i + 1, h // per]
    return out


@pytest.mark.parametrize("portions,page", [((700,), 16), ((3, 2, 250, 1, 1, 2, 441), 8), ((699, 1), 32)])
def test_distance_bias_sink_and_a_key_far_back(portions, page):
    """Random queries and keys through prompts and single tokens against the plain softmax with a
    distance bias and a sink; then one key is made to stand out 690 tokens back and at page borders:
    the head without a slope returns its value; a sink far above every score leaves nothing."""
    from mini_infer_b200.engine import StepEntry

    nq, nkv, d, n = 4, 2, 12, 700
    runner = attention_fixture(nq, nkv, d, n, page, portions)
    o = ops()
    q, k = rnd(n, nq, d, seed=1), rnd(n, nkv, d, seed=2)
    slopes = torch.tensor([0.0, 0.05, 0.5, 0.003], dtype=torch.float64)
    sinks = torch.tensor([0.0, 2.0, -30.0, 40.0], dtype=torch.float64)       # the last one takes nearly everything
    marked = [9, 16 * 3 - 1, 16 * 3]                                          # inside, a page's last and first slot
    for mk in marked:
        k[mk, :, :] = 0.0
        k[mk, :, 0] = 12.0
    q[650:, 0, :] = 0.0
    q[650:, 0, 0] = 4.0                                                       # head 0, late queries: along the marked keys
    want = plain_scores_attention(q.double(), k.double(), k.double(), 0.7, slopes, sinks)
    got, t0 = [], 0
    for cnt in portions:
        ctx, caches, _, _ = runner.stepper.plan([StepEntry("a", [0] * cnt, [])])
        runner.stepper.apply_table_updates(ctx)
        cache = caches[0]
        packed = torch.cat([q[t0:t0 + cnt].reshape(cnt, -1), k[t0:t0 + cnt].reshape(cnt, -1)], dim=1).to(DEV)
        o.qk_bias_norm_store(packed, 0, nq * d, 0, nq, nkv, d, d, q_bias=None, k_bias=None, q_gain=None, k_gain=None,
                             eps=0.0, values_are_keys=True, slots=ctx.groups[cache.group].slots, kcache=cache.k,
                             vcache=cache.v)
        out = torch.empty(cnt, nq * d, device=DEV)
        o.attention_ext(packed[:, :nq * d], out, cache, ctx, nq, nkv, d, d, 0.7, sinks=sinks.float().to(DEV),
                        slopes=slopes.float().to(DEV))
        got.append(out.cpu().double())
        t0 += cnt
    got = torch.cat(got).reshape(n, nq, d)
    assert (got - want).abs().max() <= 2e-5 * max(1.0, want.abs().max())
    # head 0 (no slope, sink 0) at the late queries: the three marked keys share the weight, their value is the key
    assert torch.allclose(got[650:, 0, 0], torch.full((50,), 12.0, dtype=torch.float64), atol=1e-3)
    # head 2 (steep slope) at the same distance: the marked keys are out of reach
    assert (want[650:, 2] - got[650:, 2]).abs().max() < 1e-4
    assert got[:9, 3].abs().max() < 1e-6                                      # before any marked key the sink of 40 swallows head 3


@pytest.mark.parametrize("portions,page", [((300,), 16), ((5, 1, 1, 2, 290, 1), 8)])
def test_values_read_from_the_keys_rows(portions, page):
    """A cache layer with keys only: the value of a key is the first ``dv`` numbers of its row.  With
    one key standing out far back, its leading numbers come back."""
    from mini_infer_b200.engine import StepEntry

    nq, dk, dv, n = 3, 20, 14, 300
    runner = attention_fixture(nq, 1, dk, n, page, portions, latent_rank=dv)
    o = ops()
    q, k = rnd(n, nq, dk, seed=5), rnd(n, 1, dk, seed=6)
    sinks = torch.tensor([0.5, -2.0, 1.0], dtype=torch.float64)
    k[7] = 0.0
    k[7, 0, dk - 1] = 25.0                       # the marked key stands out in a column that is no value
    k[7, 0, :dv] = torch.arange(dv, dtype=torch.float32)
    q[200:, 1] = 0.0
    q[200:, 1, dk - 1] = 2.0
    want = plain_scores_attention(q.double(), k.double(), k.double()[:, :, :dv], 0.5, torch.zeros(nq), sinks)
    got, t0 = [], 0
    for cnt in portions:
        ctx, caches, _, _ = runner.stepper.plan([StepEntry("a", [0] * cnt, [])])
        runner.stepper.apply_table_updates(ctx)
        cache = caches[0]
        assert cache.v is None
        slots = ctx.groups[cache.group].slots.cpu().tolist()
        by_slot = o.unpack_cache_pages(cache.k)
        by_slot[slots] = k[t0:t0 + cnt].to(DEV)
        cache.k.copy_(o.pack_cache_pages(by_slot, page))
        out = torch.empty(cnt, nq * dv, device=DEV)
        o.attention_ext(q[t0:t0 + cnt].reshape(cnt, -1).to(DEV), out, cache, ctx, nq, 1, dk, dv, 0.5,
                        sinks=sinks.float().to(DEV), values_in_keys=True)
        got.append(out.cpu().double())
        t0 += cnt
    got = torch.cat(got).reshape(n, nq, dv)
    assert (got - want).abs().max() <= 2e-5 * max(1.0, want.abs().max())
    assert torch.allclose(got[200:, 1], torch.arange(dv, dtype=torch.float64).expand(100, dv), atol=1e-3)


def test_configurations_take_both_attention_kernels():
    """The tensor-core kernel takes D's and E's sizes, the CUDA-core kernel the others'."""
    o = ops()
    taken = {}
    for which, cfg in CONFIGS.items():
        flags = []
        for layer in cfg["layers"]:
            m = layer["mixer"]
            if layer["type"] == "latent_attention":
                flags.append(o.rows_attention_supported(m["heads"], 1, m["kv_rank"] + m["rot_dim"], m["kv_rank"], True))
            else:
                flags.append(o.rows_attention_supported(m["heads"], m["kv_heads"], m["dim"], m["dim"], False))
        taken[which] = flags
    assert taken["D"] == [True, True, False] and taken["E"] == [True, True, True]
    assert not any(taken["A"] + taken["B"] + taken["C"])


@pytest.mark.parametrize("nq,nkv,d,dv,prefix", [(4, 2, 32, 32, False), (16, 1, 48, 32, True), (32, 2, 64, 64, False),
                                                (8, 1, 576, 512, True), (1, 1, 16, 32, False), (2, 1, 144, 96, True),
                                                (8, 8, 128, 256, False)])
@pytest.mark.parametrize("portions,page,mode", [((333,), 16, "rows64"), ((3, 2, 120, 1, 1, 2, 70, 1), 8, "rows16"),
                                                ((64, 64, 1), 64, "rows64"), ((200, 1, 1, 67, 1), 16, "runs"),
                                                ((3, 250, 2, 1, 77), 16, "rows32")])
def test_tensor_core_attention_against_the_plain_softmax(nq, nkv, d, dv, prefix, portions, page, mode):
    """bfloat16 on the tensor-core kernel: random rows through prompts and single tokens, sinks and
    slopes per head, values of their own size or read from the keys' rows, against the plain softmax
    computed from the same bfloat16 rows; one key stands out far back, at a page's border."""
    o = ops()
    assert o.rows_attention_supported(nq, nkv, d, dv, prefix)
    n = sum(portions)
    q = rnd(n, nq, d, seed=1, scale=d ** -0.25).bfloat16()
    k = rnd(n, nkv, d, seed=2, scale=d ** -0.25).bfloat16()
    v = k[:, :, :dv] if prefix else rnd(n, nkv, dv, seed=3).bfloat16()
    if prefix:
        k = k.clone()
    marked = page - 1                               # the last slot of the request's first page
    k[marked] = 0.0
    k[marked, :, d - 1] = 6.0
    if not prefix:
        v = v.clone()
        v[marked] = 3.0
    q[n - 20:, 0] = 0.0
    q[n - 20:, 0, d - 1] = 5.0                      # head 0's late queries point at the marked key
    slopes = torch.linspace(0.0, 0.2, nq, dtype=torch.float64)
    slopes[0] = 0.0
    sinks = torch.linspace(-3.0, 3.0, nq, dtype=torch.float64)
    vals = k.double()[:, :, :dv] if prefix else v.double()
    want = plain_scores_attention(q.double(), k.double(), vals, 0.9, slopes, sinks)
    G = nq // nkv
    # blocks of 16 rows, blocks of 64 rows, or 16 rows with every tile's keys cut into runs that are merged
    tt16, tt64 = o.rows_attention_tile_tokens(G, 16), o.rows_attention_tile_tokens(G, 64)
    tt32 = o.rows_attention_tile_tokens(G, 32)
    tt = tt64 if mode == "rows64" and tt64 else tt32 if mode == "rows32" and tt32 else tt16
    kc = torch.full((-(-n // page) + 1, nkv, page, d), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = None if prefix else torch.full((kc.shape[0], nkv, page, dv), float("nan"), dtype=torch.bfloat16, device=DEV)
    pages = list(range(kc.shape[0] - 1, 0, -1))                   # pages handed out from the far end
    table = torch.full((3, len(pages)), -1, dtype=torch.int32, device=DEV)
    table[2, :len(pages)] = i32(pages)
    got, t0 = [], 0
    for cnt in portions:
        slots = [pages[p // page] * page + p % page for p in range(t0, t0 + cnt)]
        by_slot = o.unpack_cache_pages(kc)
        by_slot[slots] = k[t0:t0 + cnt].to(DEV)
        kc.copy_(o.pack_cache_pages(by_slot, page))
        if vc is not None:
            by_slot = o.unpack_cache_pages(vc)
            by_slot[slots] = v[t0:t0 + cnt].to(DEV)
            vc.copy_(o.pack_cache_pages(by_slot, page))
        tiles = {}
        for size in {tt, tt16}:
            firsts = list(range(0, cnt, size))
            tiles[size] = (i32([0] * len(firsts)), i32(firsts), len(firsts))
        ctx = SimpleNamespace(
            groups=[SimpleNamespace(block_table=table, page_size=page, table_rows=i32([2]))],
            q_start=i32([0]), q_len=i32([cnt]), kv_len=i32([t0 + cnt]), tiles=tiles,
            decode_only=mode == "runs", max_kv_len=t0 + cnt)
        ctx.q_tiles = lambda size, _c=ctx: _c.tiles[size]
        cache = SimpleNamespace(group=0, k=kc, v=vc)
        out = torch.full((cnt, nq * dv), float("nan"), dtype=torch.bfloat16, device=DEV)
        before = o.launch_count
        o.attention_ext(q[t0:t0 + cnt].reshape(cnt, -1).to(DEV), out, cache, ctx, nq, nkv, d, dv, 0.9,
                        sinks=sinks.float().to(DEV), slopes=slopes.float().to(DEV), values_in_keys=prefix)
        splits = o._rows_attention_plan(ctx, nq, nkv, d, dv, prefix, torch.device(DEV))[2]
        assert splits == 1 or mode == "runs"
        assert o.launch_count == before + (2 if splits > 1 else 1) and "attention_rows" in o._configured
        got.append(out.cpu().double())
        t0 += cnt
    got = torch.cat(got).reshape(n, nq, dv)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= 2e-2 * max(1.0, want.abs().max())
    late = got[n - 20:, 0]
    target = k.double()[marked, 0, :dv] if prefix else torch.full((dv,), 3.0, dtype=torch.float64)
    assert (late - target).abs().max() <= 2e-2 * max(1.0, target.abs().max())


@pytest.mark.parametrize("nq,nkv,d", [(8, 2, 128), (4, 4, 64), (16, 1, 64)])
@pytest.mark.parametrize("portions,page", [((333,), 16), ((3, 130, 2, 70, 1, 1, 40), 8)])
def test_prompt_portions_on_the_tcgen05_kernel_with_sinks_and_slopes(nq, nkv, d, portions, page):
    """bfloat16 heads of 64 and 128 whose values have the keys' size: prompt portions run on the tcgen05
    prefill kernel, single tokens on the kernel of rows, both with the distance bias and the sink; one
    key stands out far back at a page's last slot."""
    from mini_infer_b200.engine import StepEntry

    n = sum(portions)
    runner = attention_fixture(nq, nkv, d, n, page, portions, dtype="bfloat16")
    o = ops()
    q = rnd(n, nq, d, seed=1, scale=d ** -0.25).bfloat16()
    k = rnd(n, nkv, d, seed=2, scale=d ** -0.25).bfloat16()
    marked = page - 1
    k[marked] = 0.0
    k[marked, :, d - 1] = 6.0
    q[n - 20:, 0] = 0.0
    q[n - 20:, 0, d - 1] = 5.0
    slopes = torch.linspace(0.0, 0.2, nq, dtype=torch.float64)
    sinks = torch.linspace(-3.0, 3.0, nq, dtype=torch.float64)
    want = plain_scores_attention(q.double(), k.double(), k.double(), 0.9, slopes, sinks)
    got, t0, used_tc = [], 0, False
    for cnt in portions:
        ctx, caches, _, _ = runner.stepper.plan([StepEntry("a", [0] * cnt, [])])
        runner.stepper.apply_table_updates(ctx)
        cache = caches[0]
        packed = torch.cat([q[t0:t0 + cnt].reshape(cnt, -1), k[t0:t0 + cnt].reshape(cnt, -1)], dim=1).to(DEV)
        o.qk_bias_norm_store(packed, 0, nq * d, 0, nq, nkv, d, d, q_bias=None, k_bias=None, q_gain=None, k_gain=None,
                             eps=0.0, values_are_keys=True, slots=ctx.groups[cache.group].slots, kcache=cache.k,
                             vcache=cache.v)
        out = torch.full((cnt, nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        before = set(o._configured)
        o.attention_ext(packed[:, :nq * d], out, cache, ctx, nq, nkv, d, d, 0.9, sinks=sinks.float().to(DEV),
                        slopes=slopes.float().to(DEV))
        if cnt > 1:
            used_tc = used_tc or "attention_tc" in o._configured
        else:
            assert "attention_rows" in o._configured
        got.append(out.cpu().double())
        t0 += cnt
    assert used_tc and o.attention_tc_status() == 0
    got = torch.cat(got).reshape(n, nq, d)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= 2e-2 * max(1.0, want.abs().max())
    assert (got[n - 20:, 0] - k.double()[marked, 0]).abs().max() <= 2e-2 * 6.0
