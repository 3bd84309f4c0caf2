"""The Ruvurax architecture in the engine against the plain implementation (``plain_ruvurax``):
every mechanism alone at the kernel level, then whole models of three small configurations
under every way of cutting the work, in float32 and bfloat16, and greedy generation through the
scheduler.  Weights and inputs are made so that a fault shows: a key that stands out just inside
and just outside a window and at a page's border, states that must be zeroed when a slot is used
again, caches filled with NaN where nothing was written."""

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_ruvurax as P
import trace_util as T
from ruvurax_configs import CONFIGS, DECAY_RANK, PAGE_SIZE, prompt, random_state

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LENGTHS = {"R": [1, 2, 37, 70], "P": [3, 19, 64, 90, 41], "M": [50, 5, 33, 81]}
# A router logit this close to the first one left out is a close call (bfloat16 activations move a
# logit by about 0.01): the other expert is as good an answer, and through keys, values and states it
# reaches the tokens behind, so a request is compared up to its first close call.  Where only the
# last layer routes, a close call stays in its own row.
CLOSE_CALL = {"float32": 1e-3, "bfloat16": 0.05}
MIN_CHECKED = {"float32": 0.5, "bfloat16": 0.2}
ROW_LOCAL = {"R"}


def ops():
    from mini_infer_b200.csrc import ops as o
    return o


def requests_for(which):
    return {f"r{i}": prompt(CONFIGS[which], n, salt=i) for i, n in enumerate(LENGTHS[which])}


_plain_cache = {}


def plain_for(which):
    """float64 logits of every request, and per request the position of its first close router call."""
    if which not in _plain_cache:
        cfg = CONFIGS[which]
        state = random_state(cfg, seed=11, rank=DECAY_RANK[which])
        logits, margins = {}, {}
        for rid, toks in requests_for(which).items():
            m = []
            logits[rid] = P.ruvurax_forward(state, cfg, toks, torch.float64, margins=m).numpy()
            margins[rid] = torch.stack(m).min(dim=0).values.numpy() if m else np.full(len(toks), np.inf)
        _plain_cache[which] = (state, logits, margins)
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
        arena.fill_(float("nan"))         # a state must be zeroed when its slot is handed out
    return runner


def compare(which, dtype, got):
    _, want, margins = plain_for(which)
    scale = max(float(np.abs(w).max()) for w in want.values())
    tol = T.tolerance(dtype, scale)
    checked = total = 0
    for rid, w in want.items():
        assert got[rid].shape == w.shape
        close = margins[rid] < CLOSE_CALL[dtype]
        if which in ROW_LOCAL:
            keep = np.nonzero(~close)[0]
        else:
            keep = np.arange(int(np.nonzero(close)[0][0]) if close.any() else len(w))
        total += len(w)
        checked += len(keep)
        assert np.isfinite(got[rid]).all(), f"{rid}: non-finite logits"
        bad = T.first_bad(got[rid][keep], w[keep], tol)
        assert bad is None, f"{which} {dtype} {rid}: position {keep[bad]} differs by " \
                            f"{np.abs(got[rid][keep[bad]] - w[keep[bad]]).max():.3g} (bound {float(tol):.3g})"
    assert checked >= MIN_CHECKED[dtype] * total, f"only {checked} of {total} rows were compared"


CUTTINGS = {"whole": T.cut_whole, "last_decoded": T.cut_last_decoded, "portions": T.cut_portions,
            "mixed": T.cut_mixed}


@pytest.mark.parametrize("cutting", list(CUTTINGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["R", "P", "M"])
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


@pytest.mark.parametrize("which", ["R", "P", "M"])
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


def test_long_decoding_past_the_window_and_captured_steps():
    """One short prompt, then 150 tokens one by one (windows of 9 and 40 pass over decoded tokens,
    pages leave the window and come back to the pool), kernel by kernel and as captured graphs."""
    which = "P"
    cfg = CONFIGS[which]
    state, _, _ = plain_for(which)
    toks = prompt(cfg, 156, salt=77)
    m = []
    want = P.ruvurax_forward(state, cfg, toks, torch.float64, margins=m).numpy()
    margin = torch.stack(m).min(dim=0).values.numpy()
    from mini_infer_b200.engine import StepEntry
    for graph in (False, True):
        runner = make_runner(which, "float32", num_blocks=12, cuda_graph=graph)   # 96 slots for 156 tokens
        runner.add_request("a")
        rows = [runner.step([StepEntry("a", toks[:6], list(range(6)))]).logits.cpu().numpy()]
        for t in toks[6:]:
            rows.append(runner.step([StepEntry("a", [t], [0])]).logits.cpu().numpy())
        got = np.concatenate(rows)
        close = np.nonzero(margin < CLOSE_CALL["float32"])[0]
        upto = int(close[0]) if close.size else len(toks)
        assert upto > 100
        tol = T.tolerance("float32", float(np.abs(want).max()))
        assert T.first_bad(got[:upto], want[:upto], tol) is None
        runner.free_request("a")
        runner.cache.check()


def test_greedy_generation_through_the_scheduler():
    """Greedy tokens from the engine's own entry point (scheduler, sampler, cache) equal the plain
    implementation's, fed its own tokens, for several prompts generated together."""
    from mini_infer_b200.engine import ContinuousScheduler, Request
    from mini_infer_b200.sampling import SamplingParams

    which = "M"
    cfg = CONFIGS[which]
    state, _, _ = plain_for(which)
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
            logits = P.ruvurax_forward(state, cfg, seq, torch.float64)[-1]
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


def ctx_for(q_lens, slots):
    """The part of a step context the state kernels read."""
    starts = np.concatenate([[0], np.cumsum(q_lens)[:-1]]).astype(np.int32)
    i32 = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device=DEV)
    return SimpleNamespace(q_start=i32(starts), q_len=i32(q_lens), state_slot=i32(slots), n_requests=len(q_lens),
                           decode_only=all(n == 1 for n in q_lens), host_q_len=list(q_lens))


@pytest.mark.parametrize("dtype,bound", [(torch.float32, 2e-6), (torch.bfloat16, 1 / 64)])
def test_layer_norm_pair_with_branch_sum(dtype, bound):
    M, H = 7, 50
    stream = rnd(M, H, seed=1, scale=3.0)
    a1, a2 = rnd(M, H, seed=2, dtype=dtype), rnd(M, H, seed=3, dtype=dtype)
    w = [(rnd(H, seed=4) + 1, rnd(H, seed=5)), (rnd(H, seed=6) + 1, rnd(H, seed=7))]
    r = stream.double() + a1.double() + a2.double()
    s = stream.to(DEV).clone()
    outs = ops().add_layernorm(s, [a1.to(DEV), a2.to(DEV)], [(g.to(DEV), b.to(DEV)) for g, b in w], 1e-5, dtype)
    assert torch.allclose(s.cpu().double(), r, atol=1e-6)          # the stream is updated in place, in fp32
    for out, (g, b) in zip(outs, w):
        want = P.layer_norm(r, g.double(), b.double(), 1e-5)
        assert (out.cpu().double() - want).abs().max() <= bound * max(1.0, want.abs().max())
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    before = s.clone()
    out, = ops().add_layernorm(s, [a1.to(DEV)], [(w[0][0].to(DEV), w[0][1].to(DEV))], 1e-5, dtype, rows=rows)
    want = P.layer_norm((before.cpu().double() + a1.double())[[5, 0, 5]], w[0][0].double(), w[0][1].double(), 1e-5)
    assert (out.cpu().double() - want).abs().max() <= bound * max(1.0, want.abs().max())
    assert torch.equal(s, before)                                  # a gathered norm leaves the stream alone


@pytest.mark.parametrize("d,dv,rot", [(24, 16, 8), (10, 14, 6), (64, 64, 64), (7, 3, 2)])
def test_interleaved_rotation_unit_norm_and_store(d, dv, rot):
    """Rotation of pairs (2i, 2i+1) on the first ``rot`` dimensions, unit RMS over the head, and keys
    and values landing where the attention kernel looks for them (checked through attention itself
    in the model tests; here: q and k in place, against the plain functions)."""
    M, nq, nkv = 9, 4, 2
    width = nq * d + nkv * d + nkv * dv + 5          # some columns behind, which must stay untouched
    packed = rnd(M, width, seed=8)
    pos = [0, 1, 2, 3, 100, 101, 4095, 7, 8]
    base = 300.0
    inv = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float()
    dev = packed.to(DEV).clone()
    ops().rope_norm_store(dev, 0, nq * d, (nq + nkv) * d, nq, nkv, d, dv,
                          positions=torch.tensor(pos, dtype=torch.int32, device=DEV), inv_freq=inv.to(DEV), rot=rot,
                          unit_norm=True, eps=1e-6)
    got = dev.cpu().double()
    x = packed.double()
    for off, n in ((0, nq), (nq * d, nkv)):
        heads = x[:, off:off + n * d].reshape(M, n, d)
        want = P.unit_rms(P.rotate_interleaved(heads, pos, base, rot), 1e-6).reshape(M, n * d)
        # the angle is an fp32 product: its rounding grows with the position
        bound = 2e-5 + 2e-6 * torch.tensor(pos, dtype=torch.float64)[:, None]
        assert ((got[:, off:off + n * d] - want).abs() <= bound).all()
    assert torch.equal(got[:, (nq + nkv) * d:], x[:, (nq + nkv) * d:])  # values and the rest are not touched


SHORT_CUTS = ({0: 23, 1: 9}, [(1, 2), (2, 1), (7, 0), (1, 1), (3, 5), (9, 0)])
LONG_CUTS = ({0: 331, 1: 70}, [(130, 65), (1, 0), (200, 5)])     # long portions: chunks walked side by side


@pytest.mark.parametrize("dtype,bound,plan", [(torch.float32, 1e-5, SHORT_CUTS), (torch.bfloat16, 2e-2, SHORT_CUTS),
                                              (torch.float32, 1e-5, LONG_CUTS), (torch.bfloat16, 2e-2, LONG_CUTS)])
def test_recurrent_unit_carries_its_state_across_portions(dtype, bound, plan):
    """Convolution tail and recurrent state through portions of 1, 2 and more tokens, two requests
    in one launch, against the plain recurrence over the whole sequence."""
    C, blocks, taps, H = 24, 3, 4, 16
    bw = C // blocks
    total, cuts = plan
    W = {"y": rnd(C, H, seed=20, scale=0.3), "y.b": rnd(C, seed=21, scale=0.1), "x": rnd(C, H, seed=22, scale=0.3),
         "x.b": rnd(C, seed=23, scale=0.1), "conv": rnd(C, taps, seed=24, scale=0.5), "conv.b": rnd(C, seed=25, scale=0.1),
         "ra": rnd(blocks, bw, bw, seed=26, scale=0.4), "ra.b": rnd(blocks, bw, seed=27, scale=0.1),
         "ri": rnd(blocks, bw, bw, seed=28, scale=0.4), "ri.b": rnd(blocks, bw, seed=29, scale=0.1),
         "lam": rnd(C, seed=30) - 1.0, "o": torch.eye(C)}
    W = {k: v.to(dtype).float() for k, v in W.items()}
    hs = {r: rnd(n, H, seed=40 + r).to(dtype).float() for r, n in total.items()}
    want = {r: P.rglru_mixer(hs[r].double(), {k: v.double() for k, v in W.items()}, blocks) for r in total}
    state = torch.full((4, taps, C), float("nan"), device=DEV)
    slots = {0: 2, 1: 0}
    for s in slots.values():
        state[s].zero_()
    gates_w = torch.cat([W["ra"], W["ri"]], dim=1).to(dtype).to(DEV).contiguous()
    f32 = lambda t: t.float().to(DEV).contiguous()
    done = {0: 0, 1: 0}
    got = {r: [] for r in total}
    for n0, n1 in cuts:
        lens = [n for n in (n0, n1) if n]
        who = [r for r, n in ((0, n0), (1, n1)) if n]
        h = torch.cat([hs[r][done[r]:done[r] + n] for r, n in zip(who, lens)])
        proj = (h.double() @ torch.cat([W["y"], W["x"]]).double().T).to(dtype).to(DEV)     # [M, 2C]
        ctx = ctx_for(lens, [slots[r] for r in who])
        y, x = proj[:, :C], proj[:, C:]
        u = torch.empty((h.shape[0], C), dtype=dtype, device=DEV)
        ops().causal_conv(x, f32(W["x.b"]), f32(W["conv"]), f32(W["conv.b"]), state, ctx, u)
        gates = ops().block_diagonal_gates(u, gates_w)
        out = torch.empty_like(u)
        ops().rglru_scan(gates, f32(W["ra.b"]).reshape(-1), f32(W["ri.b"]).reshape(-1), f32(W["lam"]), 8.0, u, y,
                         f32(W["y.b"]), x, f32(W["x.b"]), taps, state, ctx, out)
        row = 0
        for r, n in zip(who, lens):
            got[r].append(out[row:row + n].cpu().double())
            row += n
            done[r] += n
    for r in total:
        assert done[r] == total[r]
        g = torch.cat(got[r])
        assert (g - want[r]).abs().max() <= bound * max(1.0, want[r].abs().max()), f"request {r}"
    assert torch.isnan(state[1]).all() and torch.isnan(state[3]).all()      # other slots are never touched


@pytest.mark.parametrize("heads,dk,dv,dtype,portions", [
    (2, 12, 36, torch.float32, (1, 17, 2, 1, 1, 20, 3)), (1, 64, 32, torch.float32, (1, 17, 2, 1, 1, 20, 3)),
    (3, 9, 5, torch.float32, (1, 17, 2, 1, 1, 20, 3)),
    (2, 24, 40, torch.bfloat16, (300, 1, 140, 129)), (1, 128, 64, torch.bfloat16, (513,))])   # chunks side by side
def test_gated_linear_attention_state(heads, dk, dv, dtype, portions):
    """The matrix state through portions and decoded tokens against the plain token loop, with decays
    near 1 and near 0, and a head's output norm and gate."""
    Tn, tau = sum(portions), 3.0
    stride = heads * (2 * dk + dv) + 3
    stride += (-stride) % 8
    packed = rnd(Tn, stride, seed=50).to(dtype)
    z = rnd(Tn, heads * dk, seed=51, scale=3.0)
    zb = rnd(heads * dk, seed=52)
    q, k = packed[:, :heads * dk], packed[:, heads * dk:2 * heads * dk]
    v = packed[:, 2 * heads * dk:2 * heads * dk + heads * dv]
    alpha = torch.sigmoid((z + zb).double()) ** (1.0 / tau)
    S = torch.zeros(heads, dk, dv, dtype=torch.float64)
    want = torch.empty(Tn, heads, dv, dtype=torch.float64)
    for t in range(Tn):
        kt, vt = k[t].double().reshape(heads, dk), v[t].double().reshape(heads, dv)
        S = alpha[t].reshape(heads, dk)[:, :, None] * S + kt[:, :, None] * vt[:, None, :]
        want[t] = torch.einsum("hkv,hk->hv", S, q[t].double().reshape(heads, dk) * dk ** -0.5)
    state = torch.full((3, heads, dk, dv), float("nan"), device=DEV)
    state[1].zero_()
    dev = packed.to(DEV)
    got, t0 = [], 0
    for n in portions:
        ctx = ctx_for([n], [1])
        sl = dev[t0:t0 + n]
        o = ops().gla_scan(sl[:, :heads * dk], sl[:, heads * dk:2 * heads * dk],
                           sl[:, 2 * heads * dk:2 * heads * dk + heads * dv], z[t0:t0 + n].to(DEV).contiguous(),
                           zb.to(DEV), tau, dk ** -0.5, heads, dk, dv, state, ctx)
        got.append(o.cpu().double())
        t0 += n
    got = torch.cat(got).reshape(Tn, heads, dv)
    assert (got - want).abs().max() <= 2e-5 * max(1.0, want.abs().max())
    assert (state[1].cpu().double() - S).abs().max() <= 2e-5 * max(1.0, S.abs().max())
    gain, gate = rnd(dv, seed=53) + 1, rnd(Tn, heads * dv, seed=54)
    out = torch.empty(Tn, heads * dv, device=DEV)
    ops().headnorm_gate(got.reshape(Tn, heads * dv).float().to(DEV), gain.to(DEV), gate.to(DEV), out, heads, dv, 1e-5,
                        "silu", 0.7)
    ref = (P.unit_rms(got, 1e-5) * gain.double()).reshape(Tn, heads * dv) * torch.nn.functional.silu(gate.double()) * 0.7
    assert (out.cpu().double() - ref).abs().max() <= 1e-5 * max(1.0, ref.abs().max())


@pytest.mark.parametrize("E,top,ff,H,M", [(5, 2, 24, 40, 33), (3, 1, 20, 48, 5), (4, 4, 16, 36, 70), (12, 3, 72, 64, 200),
                                          (6, 2, 24, 40, 7), (3, 3, 16, 64, 8), (16, 1, 8, 264, 100)])
@pytest.mark.parametrize("dtype,bound", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_routed_experts(E, top, ff, H, M, dtype, bound):
    """Router choice and weights, the clamped activation, and the weighted sum, against the plain
    token loop; the inputs are scaled so that both clamps bite."""
    x = rnd(M, H, seed=60).to(dtype)
    W = {"router": rnd(E, H, seed=61, scale=0.5).to(dtype)}
    for e in range(E):
        W[f"e{e}.gate"] = rnd(ff, H, seed=100 + e, scale=0.4).to(dtype)
        W[f"e{e}.up"] = rnd(ff, H, seed=200 + e, scale=0.4).to(dtype)
        W[f"e{e}.down"] = rnd(H, ff, seed=300 + e, scale=0.2).to(dtype)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": 0.9}}
    margins = []
    want = P.moe(x.double(), {k: v.double() for k, v in W.items()}, mlp, margins)
    dx = x.to(DEV)
    ids, wts = ops().moe_route(dx, W["router"].to(DEV), top)
    z = x.double() @ W["router"].double().T
    ok = torch.ones(M, dtype=torch.bool) if not margins else margins[0] > 1e-3
    vals, idx = torch.topk(z, top, dim=-1)
    assert torch.equal(ids.cpu().long()[ok], idx[ok])
    assert (wts.cpu().double()[ok] - torch.softmax(vals, dim=-1)[ok]).abs().max() < 1e-5
    gate_up = torch.stack([torch.cat([W[f"e{e}.gate"], W[f"e{e}.up"]]) for e in range(E)]).to(DEV).contiguous()
    down = torch.stack([W[f"e{e}.down"] for e in range(E)]).to(DEV).contiguous()
    shared = rnd(M, H, seed=62).to(dtype)
    out = ops().moe_experts(dx, ids, wts, gate_up, down, 0.9, 1.702, shared.to(DEV))
    ref = want + shared.double()
    assert (out.cpu().double() - ref)[ok].abs().max() <= bound * max(1.0, ref.abs().max())


def test_window_edges_page_borders_and_far_keys():
    """One key is made to stand out (its direction is the queries', ten times longer in value): a
    query whose window still holds it returns its value, the next one does not; the key sits at a
    page's last slot, at a page's first slot, and hundreds of tokens back with no window at all."""
    from mini_infer_b200.engine import ModelRunner, StepEntry
    from mini_infer_b200.parts.base import LayerCache

    def run(window, n_tokens, marked, page):
        nq, nkv, d, dv = 2, 1, 16, 12
        cfg = {"architecture": "Ruvurax", "vocab": 8, "width": 16, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
               "layers": [{"type": "parallel", "mlp": None,
                           "mixer": {"left": {"heads": nq, "kv_heads": nkv, "dim": d, "vdim": dv,
                                              "mask": {"size": window} if window else None,
                                              "rot": None, "scale": 4.0},
                                     "right": {"heads": 1, "dim": 4, "vdim": 4, "tau": 2.0},
                                     "left_scale": 1.0, "right_scale": 1.0}}]}
        state = random_state(cfg, seed=3, rank=2)
        runner = ModelRunner.from_state_dict(cfg, state, dtype="float32", block_size=page,
                                             num_blocks=-(-n_tokens // page) + 1, max_requests=2)
        for st in runner.cache.storage:
            st.fill_(float("nan"))
        runner.add_request("a")
        ctx, caches, _, _ = runner.stepper.plan([StepEntry("a", [0] * n_tokens, [])])
        runner.stepper.apply_table_updates(ctx)
        cache = caches[0]
        # packed q | k | v: every query and key points along e0; the marked key is as long as the others
        # (unit norm equalises them anyway) but all other keys point along e1, so only it scores high
        packed = torch.zeros(n_tokens, (nq + nkv) * d + nkv * dv)
        packed[:, 0:nq * d:d] = 1.0                          # q heads: e0
        packed[:, nq * d + 1] = 1.0                          # keys: e1
        packed[marked, nq * d + 1] = 0.0
        packed[marked, nq * d] = 1.0                         # the marked key: e0
        packed[:, (nq + nkv) * d:] = 1.0                     # values: ones ...
        packed[marked, (nq + nkv) * d:] = 10.0               # ... the marked value: tens
        dev = packed.to(DEV)
        ops().rope_norm_store(dev, 0, nq * d, (nq + nkv) * d, nq, nkv, d, dv, positions=None, inv_freq=None, rot=0,
                              unit_norm=True, eps=1e-6, slots=ctx.groups[cache.group].slots, kcache=cache.k,
                              vcache=cache.v)
        out = torch.empty(n_tokens, nq * dv, device=DEV)
        ops().attention_kv(dev[:, :nq * d], out, cache, ctx, nq, nkv, d, dv, 4.0, window or 0)
        return out.cpu()

    # score of the marked key: q.k * scale = 16 * 4 = 64 above the others: its weight is 1 to fp32 precision
    for page, marked in ((8, 15), (8, 16), (16, 31), (4, 13)):       # last slot of a page, first slot, inside
        window = 11
        out = run(window, 64, marked, page)
        for i in range(64):
            sees = 0 <= i - marked < window
            assert torch.allclose(out[i], torch.full_like(out[i], 10.0 if sees else 1.0), atol=1e-4), (page, marked, i)
    out = run(None, 700, 3, 16)                                      # no window: a key 696 tokens back
    assert torch.allclose(out[3:], torch.full_like(out[3:], 10.0), atol=1e-4)
    assert torch.allclose(out[:3], torch.full_like(out[:3], 1.0), atol=1e-4)
