"""Mobunex without a GPU: the configuration reader, the model as data, what its mixers keep in the
cache, and the plain implementation's mechanisms against closed forms."""
import copy
import math

import pytest
import torch

from paged_batch_engine_b200.config import ConfigError, load_config
from paged_batch_engine_b200.engine.runner import build_model
from paged_batch_engine_b200.parts import CompositeNeed, PagedNeed, StateNeed
from paged_batch_engine_b200.parts.latent_attention import yarn_frequencies
from tests.helpers import MOB_A, MOB_B, MOB_C
from tests.plain import plain_mobunex as pm


# ---------------------------------------------------------------- configuration
def test_architecture_and_constants_come_from_the_configuration():
    arch, cfg = load_config(MOB_A)
    assert arch.name == "Mobunex" and cfg.width == 64 and cfg.alpha == 1.5 and cfg.eps == 1e-5
    spec = cfg.model_spec()
    assert spec.depth_stack == "mix" and spec.embedding_norm.kind == "scalar_rmsnorm" and spec.lm_head_name == "head"
    assert [b.args["alpha"] for b in spec.blocks] == [1.5] * 4
    assert [b.args["depth_index"] for b in spec.blocks] == [0, 1, 2, 3]
    assert load_config(MOB_B)[1].model_spec().blocks[0].args["alpha"] == 1.0


def test_model_as_data_names_and_shapes():
    _, cfg = load_config(MOB_A)
    spec = cfg.model_spec()
    assert [b.kind for b in spec.blocks] == ["postnorm"] * 4
    assert [b.mixer.kind for b in spec.blocks] == ["masked_attention", "gated_linear_recurrence", "latent_attention",
                                                   "gated_linear_recurrence"]
    assert [b.feed_forward.kind if b.feed_forward else None for b in spec.blocks] == \
        ["swiglu", "routed_experts", None, "swiglu"]
    model = build_model(cfg, torch.float32, "cpu")
    names = {p.name: tuple(p.shape) for p in model.param_specs() if not p.optional}
    assert names["embed"] == (300, 64) and names["head"] == (300, 64)
    assert names["embed.norm"] == () and names["final.norm"] == () and names["l0.norm1"] == () and names["l0.norm2"] == ()
    assert [names[f"l{i}.dwa"] for i in range(4)] == [(2,), (3,), (4,), (5,)]
    assert names["l0.mix.q"] == (64, 64) and names["l0.mix.k"] == (32, 64) and names["l0.mix.v"] == (48, 64)
    assert names["l0.mix.q.b"] == (64,) and names["l0.mix.v.b"] == (48,) and names["l0.mix.temp"] == (4,)
    assert names["l0.mix.o"] == (64, 96) and "l0.mix.o.b" not in names and "l0.mix.q.norm" not in names
    assert names["l0.mlp.gate"] == (96, 64) and names["l0.mlp.down"] == (64, 96)
    assert names["l1.mix.y"] == (48, 64) and names["l1.mix.x.b"] == (48,) and names["l1.mix.conv"] == (48, 4)
    assert names["l1.mix.ra"] == (3, 16, 16) and names["l1.mix.ri.b"] == (3, 16) and names["l1.mix.lam"] == (48,)
    assert names["l1.mlp.router"] == (6, 64) and names["l1.mlp.correction"] == (6,)
    assert names["l1.mlp.e5.gate"] == (40, 64) and names["l1.mlp.shared.down"] == (64, 24)
    assert names["l2.mix.dq"] == (24, 64) and names["l2.mix.uq"] == (3 * 24, 24) and names["l2.mix.dkv"] == (48, 64)
    assert names["l2.mix.g"] == (72, 64) and names["l2.mix.o"] == (64, 72) and "l2.mix.sink" not in names
    assert not any(n.startswith("l2.mlp") or n.startswith("l2.norm2") for n in names)
    assert "l1.mlp.shared.gate" in names
    b = build_model(load_config(MOB_B)[1], torch.float32, "cpu")
    assert not any("shared" in p.name for p in b.param_specs())


def test_what_the_mixers_keep():
    model = build_model(load_config(MOB_C)[1], torch.float32, "cpu")
    win, lat, rec, one, small = model.cache_needs
    assert isinstance(win, PagedNeed) and [(t.name, t.heads, t.width) for t in win.tensors] == [("k", 1, 64), ("v", 1, 64)]
    assert win.window == 17 and one.window == 1
    assert [(t.name, t.heads, t.width) for t in lat.tensors] == [("latent", 1, 64)] and lat.window == 33
    assert isinstance(rec, CompositeNeed) and dict(rec.parts) == {"rec": StateNeed((144,), torch.float32),
                                                                 "conv": StateNeed((2, 144), torch.float32)}
    assert dict(small.parts)["conv"] == StateNeed((1, 40), torch.float32)
    single_tap = build_model(load_config(MOB_B)[1], torch.float32, "cpu").cache_needs[0]
    assert dict(single_tap.parts) == {"rec": StateNeed((96,), torch.float32)}
    assert model.decode_capturable()


def test_a_layer_without_a_mask_keeps_every_token():
    cfg = copy.deepcopy(MOB_A)
    del cfg["layers"][0]["mixer"]["mask"], cfg["layers"][0]["mixer"]["kv_heads"], cfg["layers"][2]["mixer"]["mask"]
    model = build_model(load_config(cfg)[1], torch.float32, "cpu")
    assert model.cache_needs[0].window is None and model.cache_needs[2].window is None
    assert [(t.name, t.heads) for t in model.cache_needs[0].tensors] == [("k", 4), ("v", 4)]
    assert torch.equal(pm.window_mask(torch.arange(4), None), torch.tril(torch.ones(4, 4, dtype=torch.bool)))


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "attention_9", "unknown layer type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "multiple of kv_heads"),
    (("layers", 1, "mixer", "blocks"), 5, "multiple of blocks"),
    (("layers", 1, "mixer", "conv"), 17, "taps"),
    (("layers", 2, "mixer", "rot_dim"), 7, "even"),
    (("layers", 2, "mixer", "rot", "dims"), 10, "at most rot_dim"),
    (("layers", 2, "mixer", "rot", "scaling", "factor"), 0.5, "at least 1"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4, "keep <= count"),
    (("layers", 1, "mlp", "router", "top"), 5, "at least `top`"),
    (("layers", 0, "mlp", "kind"), "sparse", "not supported"),
    (("norm", "eps"), 0.0, "positive"),
])
def test_configurations_that_are_refused(path, value, word):
    cfg = copy.deepcopy(MOB_A)
    d = cfg
    for key in path[:-1]:
        d = d[key]
    d[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        load_config(cfg)


@pytest.mark.parametrize("key", ["postln_alpha", "width", "vocab", "layers", "norm"])
def test_missing_keys_are_named(key):
    cfg = copy.deepcopy(MOB_A)
    del cfg[key]
    with pytest.raises(ConfigError, match=key):
        load_config(cfg)


# ---------------------------------------------------------------- the oracle's mechanisms by hand
def test_norm_with_one_number_and_the_scaled_skip():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    got = pm.post_norm(x, y, 2.0, torch.tensor(0.5, dtype=torch.float64), 0.0)
    v = torch.tensor([7.0, 6.0], dtype=torch.float64)
    assert torch.allclose(got[0], 0.5 * v / math.sqrt((49 + 36) / 2))


def test_depth_mix_is_a_weighted_sum_of_all_results():
    xs = [torch.full((2, 3), float(i + 1), dtype=torch.float64) for i in range(3)]
    got = pm.depth_mix(xs, torch.tensor([0.5, -1.0, 2.0], dtype=torch.float64))
    assert torch.allclose(got, torch.full((2, 3), 0.5 - 2.0 + 6.0, dtype=torch.float64))


def test_window_of_one_sees_itself_only_and_the_edge_is_exclusive():
    pos = torch.arange(6)
    assert torch.equal(pm.window_mask(pos, 1), torch.eye(6, dtype=torch.bool))
    m = pm.window_mask(pos, 3)
    assert m[5, 3] and not m[5, 2] and not m[2, 3]


def test_recurrence_closed_forms():
    # r = 0 everywhere: a = 1, nothing enters, the state stays zero
    T, C = 5, 3
    u = torch.ones(T, C, dtype=torch.float64)
    S = pm.gated_recurrence(u, torch.zeros(T, C, dtype=torch.float64), torch.ones(T, C, dtype=torch.float64),
                            torch.zeros(C, dtype=torch.float64))
    assert torch.allclose(S, torch.zeros_like(S))
    # constant gates: a geometric sum; the first token gets sqrt(1 - a^2) i u like every other
    r = torch.full((T, C), 0.5, dtype=torch.float64)
    lam = torch.tensor([0.0, 1.0, -1.0], dtype=torch.float64)
    a = torch.exp(-8.0 * 0.5 * torch.log1p(torch.exp(lam)))
    b = torch.sqrt(1 - a * a) * 0.25 * 2.0
    S = pm.gated_recurrence(2 * u, r, torch.full((T, C), 0.25, dtype=torch.float64), lam)
    assert torch.allclose(S[0], b)
    assert torch.allclose(S[4], b * (1 - a ** 5) / (1 - a))


def test_block_gates_read_their_own_part_only():
    u = torch.randn(4, 6, dtype=torch.float64)
    mat = torch.randn(2, 3, 3, dtype=torch.float64)
    bias = torch.randn(2, 3, dtype=torch.float64)
    got = pm.block_gates(u, mat, bias)
    assert torch.allclose(got[:, 3:], torch.sigmoid(u[:, 3:] @ mat[1].t() + bias[1]))
    u2 = u.clone()
    u2[:, :3] += 1.0
    assert torch.equal(pm.block_gates(u2, mat, bias)[:, 3:], got[:, 3:])


def test_last_tap_is_on_the_current_token():
    u = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64)
    w = torch.tensor([[0.0, 0.0, 1.0]], dtype=torch.float64)
    assert torch.equal(pm.causal_conv(u, w, torch.zeros(1, dtype=torch.float64)), u)
    w = torch.tensor([[1.0, 0.0, 0.0]], dtype=torch.float64)
    assert torch.equal(pm.causal_conv(u, w, torch.zeros(1, dtype=torch.float64)).flatten(),
                       torch.tensor([0.0, 0.0, 1.0], dtype=torch.float64))


def test_stretched_frequencies_by_hand():
    rot = dict(base=100.0, dims=8, scaling=dict(factor=4.0, original=64, fast=8.0, slow=1.0))
    f, mag = pm.yarn_frequencies(rot)
    dim = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(dim(8.0)), 0), min(math.ceil(dim(1.0)), 7)
    assert (lo, hi) == (0, 3)
    base = [100.0 ** (-2 * i / 8) for i in range(4)]
    ramp = [min(max((i - lo) / (hi - lo), 0), 1) for i in range(4)]
    want = [b / 4 * r + b * (1 - r) for b, r in zip(base, ramp)]
    assert torch.allclose(f, torch.tensor(want, dtype=torch.float64)) and mag == pytest.approx(0.1 * math.log(4.0) + 1)
    # the engine's table is the same, also without scaling and with lo == hi
    for sc in (rot["scaling"], None, dict(factor=2.0, original=8, fast=1.0, slow=1.0)):
        ef, em = yarn_frequencies(8, 100.0, sc)
        pf, pmag = pm.yarn_frequencies(dict(base=100.0, dims=8, scaling=sc))
        assert torch.allclose(ef, pf, rtol=1e-14) and em == pytest.approx(pmag)


def test_rotation_pairs_neighbours_and_scales_both_parts():
    x = torch.tensor([[1.0, 0.0, 5.0, 7.0]], dtype=torch.float64)
    got = pm.rotate_pairs(x, torch.tensor([2]), torch.tensor([0.25], dtype=torch.float64), 1.5)
    assert torch.allclose(got[0], torch.tensor([1.5 * math.cos(0.5), 1.5 * math.sin(0.5), 5.0, 7.0], dtype=torch.float64))


def test_routing_by_hand():
    """Four groups of two, two kept, three chosen.  Choice scores by group: (0.9, 0.1) -> 1.0,
    (0.6, 0.6) -> 1.2, (0.95, -0.5) -> 0.45, (0.3, 0.3) -> 0.6: groups 1 and 0 are kept, although
    group 2 holds the single best expert; the chosen are 0 (0.9), 2 and 3 (0.6 each, the lower
    index first); the weights come from the scores without the correction."""
    s = torch.tensor([[0.8, 0.2, 0.5, 0.7, 0.9, 0.4, 0.3, 0.2]], dtype=torch.float64)
    corr = torch.tensor([0.1, -0.1, 0.1, -0.1, 0.05, -0.9, 0.0, 0.1], dtype=torch.float64)
    logits = torch.log(s / (1 - s))
    h = torch.eye(8, dtype=torch.float64)[:1]
    w_router = torch.zeros(8, 8, dtype=torch.float64)
    w_router[:, 0] = logits[0]
    picked, weights = pm.route(h, w_router, corr, dict(experts=8, top=3, groups=dict(count=4, keep=2)))
    assert sorted(picked[0].tolist()) == [0, 2, 3]
    by = dict(zip(picked[0].tolist(), weights[0].tolist()))
    assert by[0] == pytest.approx(0.8 / 2.0) and by[2] == pytest.approx(0.5 / 2.0) and by[3] == pytest.approx(0.7 / 2.0)
    # barred experts count as minus infinity, not zero: with every kept score negative the
    # barred (positive) ones still stay out
    corr2 = torch.tensor([-5.0, -5.0, -5.0, -5.0, 0.0, 0.0, -9.0, -9.0], dtype=torch.float64)
    picked, _ = pm.route(h, w_router, corr2, dict(experts=8, top=3, groups=dict(count=4, keep=2)))
    assert set(picked[0].tolist()) <= {0, 1, 2, 3, 4, 5} and {4, 5} <= set(picked[0].tolist())


def test_the_shared_expert_is_added_unweighted():
    g = torch.Generator().manual_seed(0)
    W, F, E = 8, 4, 4
    w = {"m.router": torch.randn(E, W, generator=g, dtype=torch.float64), "m.correction": torch.zeros(E, dtype=torch.float64)}
    for name in [f"e{e}" for e in range(E)] + ["shared"]:
        w[f"m.{name}.gate"] = torch.randn(F, W, generator=g, dtype=torch.float64)
        w[f"m.{name}.up"] = torch.randn(F, W, generator=g, dtype=torch.float64)
        w[f"m.{name}.down"] = torch.randn(W, F, generator=g, dtype=torch.float64)
    x = torch.randn(3, W, generator=g, dtype=torch.float64)
    mlp = dict(router=dict(experts=E, top=2), expert=dict(ff=F))
    without = pm.routed_ff(x, w, "m.", mlp)
    with_shared = pm.routed_ff(x, w, "m.", dict(mlp, shared=dict(ff=F)))
    assert torch.allclose(with_shared - without, pm.gated_ff(x, w, "m.shared."))
