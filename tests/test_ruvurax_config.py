"""CPU checks of the Ruvurax architecture: configuration reader, assembly into parts, tensor names
and shapes against a checkpoint's, what the cache manager is asked to keep, and the plain
implementation's own consistency."""

import copy

import pytest
import torch

import plain_ruvurax as P
from ruvurax_configs import CONFIGS, DECAY_RANK, prompt, random_state

from mini_infer_b200.cache.manager import CacheManager
from mini_infer_b200.config import ConfigError, load_config
from mini_infer_b200.parts import DecoderModel, KVNeed, StateNeed
from mini_infer_b200.weights.loader import WeightLoadError, check_names


def build(which):
    arch, cfg = load_config(CONFIGS[which])
    return cfg, DecoderModel(arch.assemble(cfg))


@pytest.mark.parametrize("which", list(CONFIGS))
def test_names_and_shapes_fit_a_checkpoint(which):
    cfg, model = build(which)
    state = random_state(CONFIGS[which], seed=1, rank=DECAY_RANK[which])
    check_names(model, {n: tuple(t.shape) for n, t in state.items()})
    assert len(model.blocks) == len(cfg.layers)
    assert model.graph_safe()
    # the decay's rank is the checkpoint's: any rank fits, another shape does not
    other = random_state(CONFIGS[which], seed=1, rank=DECAY_RANK[which] + 2)
    check_names(model, {n: tuple(t.shape) for n, t in other.items()})
    broken = {n: tuple(t.shape) for n, t in state.items()}
    broken["head"] = broken["head"][::-1]
    del broken["final.norm.b"]
    broken["surplus"] = (1,)
    with pytest.raises(WeightLoadError) as e:
        check_names(model, broken)
    assert e.value.missing == ["final.norm.b"] and e.value.unexpected == ["surplus"]
    assert [m[0] for m in e.value.mismatched] == ["head"]


def test_what_the_cache_keeps():
    _, model = build("M")
    needs = model.cache_needs()
    assert needs[0].kv == KVNeed(3, 10, 1, 14) and needs[0].state == StateNeed((2, 12, 36), torch.float32)
    assert needs[1].kv is None and needs[1].state == StateNeed((3, 24), torch.float32)
    assert needs[2].kv == KVNeed(2, 16, 17, 8)
    cm = CacheManager(needs, page_size=16, num_pages=4, max_requests=2)
    assert [(g.head_dim, g.value_dim, g.window) for g in cm.groups] == [(10, 14, 1), (16, 8, 17)]
    _, model = build("P")          # second layer: keys and values of one size form an ordinary group
    cm = CacheManager(model.cache_needs(), page_size=8, num_pages=4, max_requests=2)
    assert [(g.head_dim, g.value_dim) for g in cm.groups] == [(24, 16), (32, None)]


def test_windowed_groups_give_pages_back_as_the_window_moves():
    _, model = build("P")
    cm = CacheManager(model.cache_needs(), page_size=8, num_pages=7, max_requests=2)   # windows 9 and 40
    cm.add_request("a")
    cm.plan_append([("a", 30)])
    for _ in range(200):
        cm.plan_append([("a", 1)])
        cm.check()
    assert cm.num_free_pages(0) >= 4 and cm.num_free_pages(1) >= 0
    cm.free_request("a")
    assert [cm.num_free_pages(g) for g in range(2)] == [7, 7]


@pytest.mark.parametrize("edit,words", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0].update(type="other"), "neither"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "cannot share"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("tau"), "tau"),
])
def test_configurations_that_are_refused(edit, words):
    raw = copy.deepcopy(CONFIGS["P"])
    edit(raw)
    with pytest.raises(ConfigError, match=words):
        load_config(raw)


def test_plain_implementation_is_causal_and_its_window_is_a_window():
    cfg = CONFIGS["P"]
    state = random_state(cfg, seed=5, rank=3)
    toks = prompt(cfg, 30, salt=9)
    full = P.ruvurax_forward(state, cfg, toks)
    assert torch.allclose(P.ruvurax_forward(state, cfg, toks[:13]), full[:13], atol=1e-12)
    # the attention alone: a token further back than the window does not reach the output
    L = cfg["layers"][0]["mixer"]["left"]
    W = P.sub(P.sub({k: v.double() for k, v in state.items()}, "l0.mix."), "left.")
    h = torch.randn(20, cfg["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    kw = dict(heads=L["heads"], kv_heads=L["kv_heads"], dim=L["dim"], vdim=L["vdim"], rot_base=L["rot"]["base"],
              rot_dims=L["rot"]["dims"], scale=L["scale"], window=L["mask"]["size"], eps=1e-6)
    a = P.windowed_attention(h, W, list(range(20)), **kw)
    h2 = h.clone()
    h2[5] += 1.0
    b = P.windowed_attention(h2, W, list(range(20)), **kw)
    w = L["mask"]["size"]
    changed = (a - b).abs().max(dim=1).values > 1e-9
    assert changed[5:5 + w].all() and not changed[5 + w:].any() and not changed[:5].any()
