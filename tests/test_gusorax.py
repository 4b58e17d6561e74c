"""Gusorax without a GPU: the configuration reader, the model as data, the order the layers run in,
what the mixers keep in the cache, and the plain implementation's mechanisms against closed forms."""
import copy
import math

import pytest
import torch

from paged_batch_engine_b200.config import ConfigError, load_config
from paged_batch_engine_b200.engine.runner import build_model
from paged_batch_engine_b200.parts import PagedNeed
from paged_batch_engine_b200.parts.masked_attention import log_bucket
from tests.helpers import GUS_A, GUS_B, GUS_C
from tests.plain import plain_gusorax as pg

F64 = torch.float64


# ---------------------------------------------------------------- configuration
def test_architecture_and_constants_come_from_the_configuration():
    arch, cfg = load_config(GUS_A)
    assert arch.name == "Gusorax" and cfg.width == 64 and cfg.embedding_scale == 3.0 and cfg.residual_mult == 0.5
    spec = cfg.model_spec()
    assert spec.embedding_scale == 3.0 and spec.position_table_name == "pos" and spec.max_position == 512
    _, b = load_config(GUS_B)
    assert b.loop is None and b.residual_mult == 1.0 and b.eps == 1e-6


def test_model_as_data_names_and_shapes():
    _, cfg = load_config(GUS_A)
    spec = cfg.model_spec()
    assert [b.kind for b in spec.blocks] == ["parallel"] * 4
    assert [b.mixer.kind for b in spec.blocks] == ["masked_attention"] * 4
    assert [b.mixer.args["mask"] for b in spec.blocks] == ["window", "chunk", "window", "chunk"]
    assert [b.mixer.args.get("unit_sink", False) for b in spec.blocks] == [False, True, False, True]
    assert [b.feed_forward.kind if b.feed_forward else None for b in spec.blocks] == \
        ["swiglu", "routed_experts", None, "swiglu"]
    assert all(b.norm_feed_forward is None and b.args["branch_scale"] == 0.5 for b in spec.blocks)
    model = build_model(cfg, torch.float32, "cpu")
    names = {p.name: tuple(p.shape) for p in model.param_specs() if not p.optional}
    assert names["embed"] == (300, 64) and names["pos"] == (512, 64) and names["loop.in"] == (64, 128)
    assert names["final.norm"] == (64,) and names["head"] == (300, 64) and names["l0.norm1"] == (64,)
    assert names["l0.mix.q"] == (72, 64) and names["l0.mix.k"] == (24, 64) and names["l0.mix.v"] == (40, 64)
    assert names["l0.mix.o"] == (64, 120) and names["l0.mix.q.norm"] == (24,) and names["l0.mix.rel"] == (12, 3)
    assert "l0.mix.g" not in names and "l0.mix.q.b" not in names and "l1.mix.rel" not in names
    assert names["l1.mix.g"] == (80, 64) and names["l1.mix.q.b"] == (96,) and names["l1.mix.v.b"] == (40,)
    assert names["l1.mix.o.b"] == (64,) and names["l1.mlp.router"] == (6, 64) and names["l1.mlp.e5.up"] == (48, 64)
    assert names["l0.mlp.gate"] == (96, 64) and names["l0.mlp.down"] == (64, 96)
    assert not any(n.startswith("l2.mlp") or ".norm2" in n for n in names)


def test_looped_layers_run_in_a_row_with_a_cache_layer_for_every_run():
    _, cfg = load_config(GUS_A)                    # a layer, then layers 1 and 2 twice, then a layer
    order = cfg.run_order()
    assert [s.block for s in order] == [0, 1, 2, 1, 2, 3]
    assert [s.cache_layer for s in order] == list(range(6))
    assert [s.input_mix for s in order] == [None, "loop.in", None, "loop.in", None, None]
    assert pg.run_order(GUS_A) == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    _, c = load_config(GUS_C)                      # the loop covers every layer
    assert [s.block for s in c.run_order()] == [0, 1] * 3
    assert [s.input_mix for s in c.run_order()] == ["loop.in", None] * 3
    _, b = load_config(GUS_B)                      # no loop: no input mix and no such tensor
    assert [s.input_mix for s in b.run_order()] == [None] * 4
    names = {p.name for p in build_model(b, torch.float32, "cpu").param_specs() if not p.optional}
    assert "loop.in" not in names
    once = copy.deepcopy(GUS_A)
    once["loop"] = dict(start=2, stop=4, times=1)  # one pass still mixes the embedding output in
    assert [s.input_mix for s in load_config(once)[1].run_order()] == [None, None, "loop.in", None]


def test_what_the_mixers_keep():
    model = build_model(load_config(GUS_A)[1], torch.float32, "cpu")
    needs = model.cache_needs
    assert len(needs) == 6 and all(isinstance(n, PagedNeed) for n in needs)
    first = needs[0]
    assert [(t.name, t.heads, t.width) for t in first.tensors] == [("k", 1, 24), ("v", 1, 40)]
    assert [n.window for n in needs] == [21, 13, 50, 13, 50, 30]      # pages behind the mask are given back
    assert model.decode_capturable()


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "attention_3", "unknown layer type"),
    (("layers", 0, "mixer", "kv_heads"), 2, "multiple of kv_heads"),
    (("layers", 1, "mixer", "dim"), 300, "at most 256"),
    (("layers", 0, "mixer", "bias_max"), 0, "bias_max"),
    (("layers", 1, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "expert", "limit"), -1.0, "limit"),
    (("layers", 0, "mlp", "kind"), "glu", "not supported"),
    (("loop", "stop"), 9, "start < stop"),
    (("loop", "times"), 0, "loop.times"),
    (("norm", "eps"), 0.0, "positive"),
])
def test_configurations_that_cannot_run_are_refused(path, value, word):
    cfg = copy.deepcopy(GUS_A)
    d = cfg
    for key in path[:-1]:
        d = d[key]
    d[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        load_config(cfg)


@pytest.mark.parametrize("path", [("residual_mult",), ("embedding", "scale"), ("layers", 1, "mixer", "scale"),
                                  ("layers", 0, "mixer", "mask"), ("layers", 2, "mixer", "bias_max"),
                                  ("max_positions",)])
def test_a_missing_key_is_named(path):
    cfg = copy.deepcopy(GUS_A)
    d = cfg
    for key in path[:-1]:
        d = d[key]
    del d[path[-1]]
    with pytest.raises(ConfigError, match=path[-1]):
        load_config(cfg)


# ---------------------------------------------------------------- the distance buckets
def test_buckets_by_hand():
    # eight rows up to a distance of 32: 0..3 one by one, then four rows over 4..32 on a logarithmic
    # axis (row edges at 4 * 8^(k/4): 4, 6.73, 11.3, 19.0), everything from 32 on in the last row
    want = {0: 0, 1: 1, 3: 3, 4: 4, 5: 4, 6: 4, 7: 5, 11: 5, 12: 6, 19: 6, 20: 7, 31: 7, 32: 7, 33: 7, 5000: 7}
    for n, row in want.items():
        assert log_bucket(n, 8, 32.0) == row, n
        assert pg.distance_bucket(n, 8, 32.0) == row, n


@pytest.mark.parametrize("rows, far", [(12, 37.0), (4, 9.0), (20, 300.0), (16, 450.0), (2, 5.0), (7, 11.5)])
def test_buckets_never_decrease_and_end_in_the_last_row(rows, far):
    got = [log_bucket(n, rows, far) for n in range(int(far) + 50)]
    assert got[: rows // 2] == list(range(rows // 2))
    assert all(b >= a for a, b in zip(got, got[1:])) and max(got) == rows - 1
    assert all(g == rows - 1 for g in got[math.ceil(far):])
    assert got == [pg.distance_bucket(n, rows, far) for n in range(len(got))]


# ---------------------------------------------------------------- the plain mechanisms against closed forms
def test_window_and_chunk_masks_by_hand():
    w = pg.window_mask(6, 3)
    assert w[5].tolist() == [False, False, False, True, True, True] and w[1].tolist() == [True, True] + [False] * 4
    assert pg.window_mask(4, 1).tolist() == torch.eye(4, dtype=torch.bool).tolist()
    c = pg.chunk_mask(7, 3)
    assert c[2].tolist() == [True, True, True, False, False, False, False]
    assert c[3].tolist() == [False, False, False, True, False, False, False]       # the first of a chunk sees itself only
    assert c[6].tolist() == [False] * 6 + [True]


def test_unit_sink_halves_a_lone_zero_score():
    """One visible key with a score of 0: the sink's e^0 takes half; without it the key takes all.
    With scores far below 0 nearly everything goes to the sink and the output vanishes."""
    q = torch.zeros(1, 1, 4, dtype=F64)
    k = torch.ones(1, 1, 4, dtype=F64)
    v = torch.tensor([[[2.0, -4.0]]], dtype=F64)
    mask = torch.ones(1, 1, dtype=torch.bool)
    assert torch.allclose(pg.softmax_attention(q, k, v, mask, 1.0, None, True), v / 2)
    assert torch.allclose(pg.softmax_attention(q, k, v, mask, 1.0, None, False), v)
    far_down = pg.softmax_attention(q - 5.0, k, v, mask, 1.0, None, True)             # score -20
    assert float(far_down.abs().max()) < 1e-7


def test_capped_expert_by_hand():
    eye = torch.eye(3, dtype=F64)
    w = {"e.gate": eye, "e.up": eye, "e.down": eye}
    h = torch.tensor([[5.0, -5.0, 0.5]], dtype=F64)
    y = pg.capped_expert(h, w, "e.", 2.0)
    sg = lambda z: 1 / (1 + math.exp(-1.702 * z))
    # gate capped from above only; linear part clamped on both sides, plus one
    want = [2.0 * sg(2.0) * (2.0 + 1.0), -5.0 * sg(-5.0) * (-2.0 + 1.0), 0.5 * sg(0.5) * (0.5 + 1.0)]
    assert torch.allclose(y[0], torch.tensor(want, dtype=F64))


def test_router_weights_are_the_softmax_over_the_chosen_alone():
    z = torch.tensor([[1.0, 3.0, 2.0, -1.0]], dtype=F64)
    chosen, weights = pg.route(z, torch.eye(4, dtype=F64), 2)
    assert sorted(chosen[0].tolist()) == [1, 2]
    e = math.exp(3.0) + math.exp(2.0)
    assert torch.allclose(weights[0].sort().values, torch.tensor([math.exp(2.0) / e, math.exp(3.0) / e], dtype=F64))


def test_one_norm_feeds_both_branches_and_the_sum_is_scaled():
    """A layer whose mixer and feed-forward are both known linear maps of the normed input."""
    cfg = dict(width=4, vocab=5, norm=dict(eps=1e-6), embedding=dict(scale=2.0), residual_mult=0.25,
               layers=[dict(type="attention", mixer=dict(heads=1, kv_heads=1, dim=4, vdim=4, scale=1.0, mask=dict(size=1),
                                                         bias_max=3.0), mlp=None)])
    g = torch.Generator().manual_seed(0)
    w = {"embed": torch.randn(5, 4, generator=g), "pos": torch.randn(8, 4, generator=g), "l0.norm1": torch.randn(4, generator=g) * 0.1,
         "l0.mix.q": torch.randn(4, 4, generator=g), "l0.mix.k": torch.randn(4, 4, generator=g), "l0.mix.v": torch.eye(4),
         "l0.mix.q.norm": torch.ones(4), "l0.mix.k.norm": torch.ones(4), "l0.mix.rel": torch.zeros(2, 1),
         "l0.mix.o": torch.eye(4) * 3.0, "final.norm": torch.zeros(4), "head": torch.eye(5, 4)}
    res = []
    pg.forward(cfg, w, [1, 4, 2], residuals=res)
    e = w["embed"].double()[[1, 4, 2]] * 2.0 + w["pos"].double()[:3]
    n = pg.norm_one_plus(e, w["l0.norm1"].double(), 1e-6)
    # a window of one token: every row's attention returns its own value, here the normed input itself
    assert torch.allclose(res[0], e + 0.25 * 3.0 * n)
