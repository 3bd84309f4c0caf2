"""Lilulix on the CPU: configuration, tensor names and shapes, the run order of a looped stretch,
what the cache is asked to keep, and properties of the plain implementation itself."""

import copy

import pytest
import torch

import plain_lilulix as P
from lilulix_configs import CONFIGS, prompt, random_state
from mini_infer_b200.cache.manager import CacheManager
from mini_infer_b200.config.registry import ConfigError, load_config
from mini_infer_b200.parts.model import DecoderModel
from mini_infer_b200.weights.loader import WeightLoadError, check_names


def build(which):
    arch, cfg = load_config(CONFIGS[which])
    return cfg, DecoderModel(arch.assemble(cfg))


@pytest.mark.parametrize("which", list(CONFIGS))
def test_tensor_names_and_shapes_fit_a_checkpoint(which):
    _, model = build(which)
    state = random_state(CONFIGS[which], seed=1)
    check_names(model, {n: tuple(t.shape) for n, t in state.items()})
    extra = dict(state, **{"l0.mix.v": torch.zeros(2, 2)})
    with pytest.raises(WeightLoadError) as e:
        check_names(model, {n: tuple(t.shape) for n, t in extra.items()})
    assert e.value.unexpected == ["l0.mix.v"]
    del state["final.norm"]
    with pytest.raises(WeightLoadError) as e:
        check_names(model, {n: tuple(t.shape) for n, t in state.items()})
    assert e.value.missing == ["final.norm"]


def test_run_order_of_a_looped_stretch():
    cfg, model = build("A")          # layers 0, 1 three times, then layer 2
    assert [e.layer for e in model.schedule] == [0, 1, 0, 1, 0, 1, 2]
    assert [e.cache for e in model.schedule] == list(range(7))       # every pass has a cache of its own
    restarts = [(i, p.row, p.needs_embedding) for i, p in enumerate(model.before) if p is not None]
    assert restarts == [(0, 0, False), (2, 1, True), (4, 2, True)]
    assert [e.layer for e in build("B")[1].schedule] == [0, 1, 2, 1, 2]
    assert all(p is None for p in build("C")[1].before)
    assert [e.layer for e in build("D")[1].schedule] == [0, 1, 2]
    assert [p is not None for p in build("D")[1].before] == [False, True, False]
    assert P.run_order(3, CONFIGS["A"]["loop"]) == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None)]


def test_cache_needs_latent_rows_keys_only_and_the_previous_token():
    cfg, model = build("A")
    needs = model.cache_needs()
    assert len(needs) == 8                                   # seven cache layers and the embedding's state
    assert needs[0].kv.kv_heads == 1 and needs[0].kv.head_dim == 20 + 8 and needs[0].kv.value_dim == 0
    assert needs[1].kv.kv_heads == 2 and needs[1].kv.head_dim == 16 and needs[1].kv.value_dim is None
    assert needs[7].kv is None and needs[7].state.dtype == torch.int32 and needs[7].state.shape == (1,)
    cm = CacheManager(needs, page_size=8, num_pages=4, max_requests=2)
    assert [g.layers for g in cm.groups] == [(0, 2, 4), (1, 3, 5), (6,)]
    assert [g.value_dim for g in cm.groups] == [0, None, 0]


def test_configuration_errors():
    for path, value in ((("layers", 0, "type"), "convolution"), (("layers", 1, "mixer", "kv_heads"), 3),
                        (("layers", 0, "mixer", "rot", "dims"), 3), (("loop", "stop"), 9),
                        (("layers", 1, "mixer", "vdim"), 8), (("embedding", "bigram", "buckets"), 0)):
        raw = copy.deepcopy(CONFIGS["A"])
        node = raw
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            load_config(raw)
    raw = copy.deepcopy(CONFIGS["A"])
    del raw["layers"][0]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError):
        load_config(raw)


def test_plain_pair_rows_and_first_token():
    assert P.bigram_rows([4, 9, 9, 0], 5, 2, 9) == [5, (4 * 2 + 9 * 9) % 5, (9 * 2 + 81) % 5, (18 + 0) % 5]


def test_plain_is_causal_and_the_sink_takes_weight():
    cfg = CONFIGS["C"]
    state = {k: v.double() for k, v in random_state(cfg, seed=2).items()}
    toks = prompt(cfg, 14, salt=1)
    full = P.forward(cfg, state, toks)
    part = P.forward(cfg, state, toks[:9])
    assert torch.allclose(full[:9], part, atol=1e-12)
    s = torch.tensor([0.3, -1.0, 2.0], dtype=torch.float64)
    p = P.sink_softmax(s, 1.0)
    assert abs(float(p.sum()) - float(torch.exp(s).sum() / (torch.exp(s).sum() + torch.e))) < 1e-12
    assert float(P.sink_softmax(s, -1e9).sum()) == pytest.approx(1.0)


def test_plain_latent_attention_equals_its_expanded_form():
    """Scores against the latent through ``W_uk^T q`` equal scores against the expanded keys."""
    torch.manual_seed(0)
    T, H, n, d, rd, dv, R = 6, 10, 2, 4, 2, 3, 5
    W = {"q": torch.randn(n * (d + rd), H), "dkv": torch.randn(R + rd, H), "dkv.norm": torch.rand(R) + 0.5,
         "uk": torch.randn(n * d, R), "uv": torch.randn(n * dv, R), "sink": torch.randn(n),
         "g": torch.randn(n * dv, H), "o": torch.randn(H, n * dv)}
    W = {k: v.double() for k, v in W.items()}
    h = torch.randn(T, H, dtype=torch.float64)
    want = P.latent_attention(h, W, range(T), heads=n, dim=d, rot_dim=rd, vdim=dv, kv_rank=R, rot_base=50.0,
                              rot_dims=2, scale=0.4, eps=1e-5)
    q = (h @ W["q"].T).reshape(T, n, d + rd)
    down = h @ W["dkv"].T
    c = P.rms_norm(down[:, :R], W["dkv.norm"], 1e-5)
    kr = P.rotate_half(down[:, R:], range(T), 50.0, 2)
    qr = P.rotate_half(q[..., d:], range(T), 50.0, 2)
    out = torch.zeros(T, n, dv, dtype=torch.float64)
    for hd in range(n):
        q_lat = q[:, hd, :d] @ W["uk"][hd * d:(hd + 1) * d]          # [T, R]
        for i in range(T):
            s = (c[:i + 1] @ q_lat[i] + kr[:i + 1] @ qr[i, hd]) * 0.4
            out[i, hd] = W["uv"][hd * dv:(hd + 1) * dv] @ (P.sink_softmax(s, W["sink"][hd]) @ c[:i + 1])
    got = (out.reshape(T, n * dv) * torch.sigmoid(h @ W["g"].T)) @ W["o"].T
    assert torch.allclose(got, want, atol=1e-10)
