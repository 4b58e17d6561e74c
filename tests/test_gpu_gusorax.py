"""Gusorax on the GPU against the plain implementation: every mechanism alone, then whole models
under every way of cutting and batching (whole, last tokens decoded, portions down to two tokens,
mixed batches with pages and request slots used again), long decoding, captured decode steps,
generation through the entry point, and the trace runner itself; float32 and bfloat16, three tiny
configurations."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import replay_util as ru
from tests.helpers import GUSORAX, load_plain, make_gusorax_folder
from tests.plain import plain_gusorax as pg

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
DEV = "cuda:0"
TOL_F32_REL = 3e-5          # max |dlogit| over the largest logit: summation order only
# bfloat16: a row's root-mean-square difference over the root mean square of all logits.  A router
# may choose another expert for a token whose logits lie within the rounding of 16-bit activations
# (the float32 runs are the sharp test of every schedule), so a few rows may lie beyond the bound.
TOL_BF16_RMS_MEAN = 0.03
TOL_BF16_RMS = 0.12
BF16_ROWS_BEYOND = 0.03


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_gusorax_folder(tmp_path_factory.mktemp(f"gus_{name}"), cfg, seed)
            for name, (cfg, seed, _) in GUSORAX.items()}


def _ops():
    from paged_batch_engine_b200.csrc import ops
    return ops


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


# ================================================================ mechanisms alone
@pytest.mark.parametrize("W, dt, scale", [(64, torch.float32, 3.0), (200, torch.bfloat16, 1.0), (37, torch.float32, 0.25)])
def test_scaled_embedding_with_position_rows(W, dt, scale):
    ops = _ops()
    g = torch.Generator().manual_seed(W)
    table, pos = torch.randn(50, W, generator=g).to(dt), torch.randn(30, W, generator=g).to(dt)
    ids, where = [7, 0, 49, 7, 12], [0, 29, 3, 3, 1]
    out = torch.empty(5, W, dtype=torch.float32, device=DEV)
    ops.embedding_positions(out, table.to(DEV), i32(ids), scale, pos.to(DEV), i32(where))
    want = table.double()[ids] * scale + pos.double()[where]
    assert torch.allclose(out.cpu().double(), want, atol=1e-5, rtol=1e-6)
    ops.embedding_positions(out, table.to(DEV), i32(ids), scale, None, None)
    assert torch.allclose(out.cpu().double(), table.double()[ids] * scale, atol=1e-5, rtol=1e-6)


@pytest.mark.parametrize("W, dt, m", [(64, torch.float32, 0.5), (200, torch.bfloat16, 1.0), (37, torch.float32, 0.3)])
def test_scaled_branch_sum_one_norm_and_the_pass_input(W, dt, m):
    """x + m (a + b) in float32, its norm with a gain of one plus the stored weight, and the row
    [x + m (a + b) ; first] that the input mix of a pass multiplies."""
    ops = _ops()
    g = torch.Generator().manual_seed(W + 1)
    T = 6
    x, first = torch.randn(T, W, generator=g) * 3, torch.randn(T, W, generator=g)
    a, b = torch.randn(T, W, generator=g).to(dt), torch.randn(T, W, generator=g).to(dt)
    stored = torch.randn(W, generator=g) * 0.3
    total = x.double() + m * (a.double() + b.double())
    res = x.to(DEV)
    o, none = ops.add2_rmsnorm2(res, a.to(DEV), b.to(DEV), (1.0 + stored).to(DEV), None, 1e-5, torch.float32,
                                delta_scale=m)
    assert none is None and torch.allclose(res.cpu().double(), total, atol=1e-5)
    assert torch.allclose(o.cpu().double(), pg.norm_one_plus(total, stored.double(), 1e-5), atol=3e-5, rtol=1e-5)
    pair = ops.fold_pair(x.to(DEV), a.to(DEV), b.to(DEV), m, first.to(DEV), torch.float32)
    assert torch.allclose(pair.cpu().double(), torch.cat([total, first.double()], dim=1), atol=1e-5)
    pair = ops.fold_pair(x.to(DEV), None, None, m, first.to(DEV), torch.float32)
    assert torch.equal(pair.cpu(), torch.cat([x, first], dim=1))


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("limit, alpha", [(1.2, 1.702), (0.4, 1.0), (50.0, 1.702)])
def test_capped_gate_and_clamped_linear_part(limit, alpha, dt):
    ops = _ops()
    g = torch.Generator().manual_seed(int(limit * 10))
    rows, F = 9, 52
    gu = (torch.randn(rows, 2 * F, generator=g) * 2).to(dt)
    out = torch.empty(rows, F, dtype=dt, device=DEV)
    ops.gated_activation(gu.to(DEV), out, "capped_swish", limit, alpha)
    gd, ud = gu.double()[:, :F].clamp(max=limit), gu.double()[:, F:].clamp(-limit, limit)
    want = gd * torch.sigmoid(alpha * gd) * (ud + 1.0)
    tol = 1e-5 if dt == torch.float32 else 1e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol * float(want.abs().max()), rtol=tol)


@pytest.mark.parametrize("E, top", [(6, 2), (5, 1), (3, 3), (40, 6)])
def test_router_weights_are_the_softmax_over_the_chosen(E, top):
    ops = _ops()
    g = torch.Generator().manual_seed(E * 10 + top)
    h = torch.randn(33, 24, generator=g)
    wr = torch.randn(E, 24, generator=g) * 3
    z = (h @ wr.t()).contiguous()
    chosen, weights = ops.route(z.to(DEV), top, 1, 1, 1.0)
    want_c, want_w = pg.route(h.double(), wr.double(), top)
    order = chosen.cpu().long().argsort(dim=1)
    worder = want_c.argsort(dim=1)
    assert torch.equal(chosen.cpu().long().gather(1, order), want_c.gather(1, worder))
    assert torch.allclose(weights.cpu().double().gather(1, order), want_w.gather(1, worder), atol=2e-6)


def test_router_rows_that_are_not_numbers_choose_experts_that_exist():
    """Padding rows of a captured step carry whatever their memory held: the router still returns
    indices inside the table for them, and the rows beside them are not touched."""
    ops = _ops()
    z = torch.randn(5, 7)
    z[1] = float("nan")
    z[3, 2] = float("nan")
    chosen, weights = ops.route(z.to(DEV), 3, 1, 1, 1.0)
    c = chosen.cpu().long()
    assert int(c.min()) >= 0 and int(c.max()) < 7
    for row in (0, 2, 4):
        want_c, want_w = pg.route(z[row:row + 1].double(), torch.eye(7, dtype=torch.float64), 3)
        assert sorted(c[row].tolist()) == sorted(want_c[0].tolist())
        assert torch.allclose(weights[row].cpu().double().sort().values, want_w[0].sort().values, atol=2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W, F, E, top, limit", [(64, 48, 6, 2, 0.7), (100, 24, 9, 4, 1.5), (40, 130, 3, 1, 30.0)])
def test_capped_experts_by_rows_and_sorted_by_expert(W, F, E, top, limit, dtype):
    """The routed experts with the capped activation, a few rows (every row reads its experts) and
    many (rows sorted by expert), against the plain loop over tokens and experts."""
    from paged_batch_engine_b200.parts import RoutedExperts
    g = torch.Generator().manual_seed(W + F)
    part = RoutedExperts(W, F, E, top, dtype, DEV, activation="capped_swish", limit=limit, alpha=1.702)
    w = {"m.router": torch.randn(E, W, generator=g) * 2}
    for e in range(E):
        w[f"m.e{e}.gate"] = torch.randn(F, W, generator=g) * 0.4
        w[f"m.e{e}.up"] = torch.randn(F, W, generator=g) * 0.4
        w[f"m.e{e}.down"] = torch.randn(W, F, generator=g) * 0.3
    w = {k: v.to(dtype) for k, v in w.items()}
    part.load({k: v.to(DEV) for k, v in w.items()}, "m.")
    wd = {k: v.double() for k, v in w.items()}
    mlp = dict(router=dict(experts=E, top=top), expert=dict(ff=F, limit=limit))
    for rows in (5, 300):
        x = torch.randn(rows, W, generator=g).to(dtype)
        got = part.forward(x.to(DEV), None).float().cpu().double()
        want = pg.routed_ff(x.double(), wd, "m.", mlp)
        tol = (2e-5 if dtype == torch.float32 else 3e-2) * float(want.abs().max())
        err = (got - want).abs().max(dim=1).values
        # a router may choose otherwise for a row whose logits tie within 16-bit rounding of the products
        beyond = int((err > tol).sum())
        assert beyond <= (0 if dtype == torch.float32 else max(1, rows // 50)), (rows, beyond, float(err.max()), tol)


# ================================================================ the masked attention part
def _masked_part(kind, H, G, D, E, size, hidden, dtype, seed, scale, rows=8, far=None):
    """The part with weights made so that every query looks along the first key coordinate and
    only input column 1 reaches that coordinate: a token with a large column 1 is a key that every
    query scores far above all others (after the head norms, which leave directions only)."""
    from paged_batch_engine_b200.parts import MaskedAttention
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g)
    window = kind == "window"
    part = MaskedAttention(hidden, H, G, D, E, scale, 1e-5, dtype, DEV, mask=kind, mask_size=size,
                           distance_bias=dict(rows=rows, far=far) if window else None, unit_sink=not window,
                           out_gate=not window, proj_bias=not window)
    w = {"p.q": rnd(H * D, hidden) * 0.05, "p.k": rnd(G * D, hidden) * 0.3, "p.v": rnd(G * E, hidden) * 0.3,
         "p.o": rnd(hidden, H * E) * 0.3, "p.q.norm": 1 + 0.2 * rnd(D), "p.k.norm": 1 + 0.2 * rnd(D)}
    w["p.q.norm"][0] = w["p.k.norm"][0] = 1.5
    # input column 0 is a constant that every query head's first coordinate reads; column 1 goes into
    # every key head's first coordinate and nothing else does
    w["p.q"].view(H, D, hidden)[:, 0, :] = 0
    w["p.q"].view(H, D, hidden)[:, 0, 0] = 2.0
    w["p.k"].view(G, D, hidden)[:, 0, :] = 0
    w["p.k"].view(G, D, hidden)[:, 0, 1] = 1.0
    w["p.k"][:, 0] = 0
    if window:
        w["p.rel"] = rnd(rows, H) * 0.5
    else:
        w.update({"p.g": rnd(H * E, hidden) * 0.5, "p.q.b": rnd(H * D) * 0.02, "p.k.b": rnd(G * D) * 0.02,
                  "p.v.b": rnd(G * E) * 0.3, "p.o.b": rnd(hidden) * 0.3})
        w["p.q.b"].view(H, D)[:, 0] = 0
        w["p.k.b"].view(G, D)[:, 0] = 0
    w = {k: v.to(dtype if v.dim() == 2 and not k.endswith("rel") else torch.float32) for k, v in w.items()}
    part.load({k: v.to(DEV) for k, v in w.items()}, "p.")
    m = dict(heads=H, kv_heads=G, dim=D, vdim=E, scale=scale, mask=dict(size=size), bias_max=far)
    return part, m, {k: v.double() for k, v in w.items()}


def _plain_part(kind, x, w, m):
    return (pg.attention_mixer if kind == "window" else pg.attention_2_mixer)(x, w, "p.", m, 1e-5)


def _stand_out_input(T, hidden, mark, g):
    x = torch.randn(T, hidden, generator=g) * 0.5
    x[:, 0] = 3.0                          # every query looks along the first key coordinate
    x[:, 1] = 0.02 * torch.randn(T, generator=g)
    x[mark, 1] = 30.0                      # the stand-out key: all of its direction is that coordinate
    x[mark, 2:] = 2.0                      # and a value that shows
    return x


def _run_part(part, x, cuts, page, num_pages, dtype, storage=None, handle=None):
    """Feeds rows x of one request through the part in portions of the given sizes."""
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    st = storage or CacheStorage([part.cache_need()], page, num_pages, 2, dtype, DEV, poison=True)
    keys = [(st.layer(0).group,) + k for k in part.work_keys()]
    h = st.manager.add_request() if handle is None else handle
    outs, i = [], 0
    for n in cuts:
        assert st.manager.reserve(h, n)
        ctx = StepContext(st.manager, [StepEntry(h, [0] * n, [])], torch.device(DEV), keys)
        outs.append(part.forward(x[i:i + n].to(DEV).to(dtype), ctx, st.layer(0)).float().cpu())
        st.manager.commit(h, n)
        i += n
    st.manager.check_invariants()
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind, H, G, D, E, size, page, T", [
    ("window", 3, 1, 24, 40, 21, 8, 90),       # float32-arithmetic kernel in both dtypes; a window off the page grid
    ("window", 8, 2, 32, 16, 64, 16, 200),     # tensor-core kernel for bfloat16; a window of four whole pages
    ("window", 4, 4, 16, 48, 600, 16, 1300),   # a far key among hundreds, over the edge of a key split
    ("chunk", 4, 2, 24, 20, 13, 8, 90),
    ("chunk", 6, 1, 64, 32, 48, 16, 210),
    ("chunk", 2, 2, 16, 16, 520, 8, 1100),
    ("window", 2, 1, 256, 256, 40, 16, 130),   # the widest heads: key tiles of 32 on the tensor-core path
    ("chunk", 4, 2, 192, 96, 50, 8, 130),
    ("window", 2, 1, 16, 16, 1, 4, 30),        # a row sees itself only
    ("chunk", 2, 1, 16, 16, 1, 4, 30),
])
def test_masked_attention_with_a_stand_out_key(kind, H, G, D, E, size, page, T, dtype):
    """One key that every query scores far above all others, placed in turn where a fault would
    show: the first tokens, a page's edges, so that the last row that sees it and the first that
    does not fall in the prompt portion or among the tokens decoded alone, and far back among
    hundreds.  A mask that is one token off moves that key in or out of a row's sight."""
    hidden = 40
    part, m, w = _masked_part(kind, H, G, D, E, size, hidden, dtype, T + H, scale=6.0 / D, far=max(size * 0.8 + 3, 6.0))
    g = torch.Generator().manual_seed(T)
    tail = 14 if T < 500 else 40
    head = T - tail
    if kind == "window":
        # the key leaves sight at mark + size: in the prompt portion, at its last row, among the decoded, never
        marks = {0, 1, page - 1, page, head - size - 5, head - size - 1, head - size, head - size + 6, T - size,
                 T - size - 1, T - 3}
    else:
        # the last and first token of a chunk, in the prompt portion and among the decoded
        c_head, c_tail = (head // size) * size, ((T - 1) // size) * size
        marks = {0, 1, page, c_head - size, c_head - size + 1, c_head - 1, c_head, c_tail - 1, c_tail, T - 2,
                 max(0, c_tail - size)}
    marks = sorted(x for x in marks if 0 <= x < T)
    for mark in marks[:: (1 if dtype == torch.float32 and T < 500 else 3)]:
        x = _stand_out_input(T, hidden, mark, g)
        want = _plain_part(kind, x.to(dtype).double(), w, m)
        cuts = ([head] if T < 500 else [500, head - 500]) + [1] * tail
        got = _run_part(part, x, cuts, page, (T + page - 1) // page + 3, dtype).double()
        tol = (3e-5 if dtype == torch.float32 else 4e-2) * float(want.abs().max())
        err = (got - want).abs().max(dim=1).values
        assert float(err.max()) <= tol, (mark, int(err.argmax()), float(err.max()), tol)
        # the test would see a mask that is one off: the rows around the edge differ by far more than the tolerance
        if kind == "window" and mark + size < T and size > 1:
            assert float((want[mark + size] - want[mark + size - 1]).abs().max()) > 5 * tol


@pytest.mark.parametrize("kind", ["window", "chunk"])
def test_masked_attention_in_portions_of_two_and_other_requests_beside(kind):
    """Portions of two tokens across window, chunk and page edges, and two requests of unequal
    length in one step (a prompt portion beside a single token, then the other way round) against
    each alone; the second request's pages were the first's in an earlier life."""
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    H, G, D, E, size, hidden, page = 6, 2, 24, 20, 11, 40, 8
    part, m, w = _masked_part(kind, H, G, D, E, size, hidden, torch.float32, 3, scale=0.3, far=14.0)
    g = torch.Generator().manual_seed(9)
    xa, xb = torch.randn(61, hidden, generator=g), torch.randn(30, hidden, generator=g)
    want_a, want_b = _plain_part(kind, xa.double(), w, m), _plain_part(kind, xb.double(), w, m)
    got = _run_part(part, xa, [2] * 20 + [7, 2, 3, 2, 5, 2], page, 12, torch.float32).double()
    assert float((got - want_a).abs().max()) <= 3e-5 * float(want_a.abs().max())
    st = CacheStorage([part.cache_need()], page, 12, 2, torch.float32, DEV, poison=True)
    keys = [(st.layer(0).group,) + k for k in part.work_keys()]
    # an earlier request fills the pool's pages and leaves
    h0 = st.manager.add_request()
    _run_part(part, xa[:40], [40], page, 0, torch.float32, storage=st, handle=h0)
    st.manager.free(h0)
    ha, hb = st.manager.add_request(), st.manager.add_request()
    done, outs = {ha: 0, hb: 0}, {ha: [], hb: []}
    for na, nb in [(40, 1), (1, 17), (20, 12)]:
        entries, rows = [], []
        for h, n, x in ((ha, na, xa), (hb, nb, xb)):
            assert st.manager.reserve(h, n)
            entries.append(StepEntry(h, [0] * n, []))
            rows.append(x[done[h]:done[h] + n])
        ctx = StepContext(st.manager, entries, torch.device(DEV), keys)
        y = part.forward(torch.cat(rows).to(DEV), ctx, st.layer(0)).cpu()
        outs[ha].append(y[:na]); outs[hb].append(y[na:])
        for h, n in ((ha, na), (hb, nb)):
            st.manager.commit(h, n)
            done[h] += n
    for h, want in ((ha, want_a), (hb, want_b)):
        got = torch.cat(outs[h]).double()
        assert float((got - want).abs().max()) <= 3e-5 * float(want.abs().max())
    st.manager.check_invariants()


# ================================================================ whole models
# A: windows of 21 and 50, chunks of 13 and 30; B: a window of 77 and chunks of 64; C: a window of 600
# (the longest request passes it by more than a page) and chunks of 40
LENGTHS = {"A": [3, 41, 97, 150], "B": [1, 30, 75, 161], "C": [2, 52, 110, 640]}


def requests_for(name, vocab):
    g = torch.Generator().manual_seed(sum(map(ord, name)) + 277)
    return {f"{name}{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[name])}


_plain_cache = {}


def plain_logits(folder, reqs):
    cfg, w = load_plain(folder)
    out = {}
    for rid, toks in reqs.items():
        key = (folder, tuple(toks))
        if key not in _plain_cache:
            _plain_cache[key] = pg.forward(cfg, w, toks).float()
        out[rid] = _plain_cache[key]
    return out


def make_runner(folder, dtype, page, pool_tokens, max_requests=4):
    from paged_batch_engine_b200.engine.runner import ModelRunner
    return ModelRunner.from_folder(folder, dtype=dtype, device=DEV, page_tokens=page,
                                   max_cache_tokens=pool_tokens, max_requests=max_requests, poison=True)


def check(got, want, dtype, label):
    worst, where, scale = ru.max_error(got, want)
    rms_all = float(torch.cat([v.flatten() for v in want.values()]).pow(2).mean().sqrt())
    per_row = sorted(float((row - want[rid][pos]).pow(2).mean().sqrt()) / rms_all for rid, rows in got.items()
                     for pos, row in rows.items())
    print(f"\n[gusorax] {label} {dtype}: max|dlogit| = {worst:.3e} at {where}, max|logit| = {scale:.3f}, "
          f"row rms / logit rms: worst {per_row[-1]:.3e}, mean {sum(per_row) / len(per_row):.3e}")
    assert sum(len(v) for v in got.values()) == sum(v.shape[0] for v in want.values()), label
    if dtype == "float32":
        tol = TOL_F32_REL * max(scale, 1.0)
        assert worst <= tol, (label, worst, where, "first beyond tolerance:", ru.first_wrong(got, want, tol))
        return
    beyond = sum(1 for e in per_row if not e <= TOL_BF16_RMS)
    assert beyond <= max(1, int(BF16_ROWS_BEYOND * len(per_row))), (label, beyond, len(per_row), per_row[-5:])
    kept = per_row[:len(per_row) - beyond]
    assert sum(kept) / len(kept) <= TOL_BF16_RMS_MEAN, (label, sum(kept) / len(kept))


def test_the_residual_after_every_layer_run(folders):
    """Layer by layer in float32: the residual stream after each run of a layer (a looped layer
    counts every time) against the plain implementation's."""
    from paged_batch_engine_b200.engine.batch import StepEntry
    cfg, _, page = GUSORAX["A"]
    c, w = load_plain(folders["A"])
    toks = requests_for("A", cfg["vocab"])["A2"]
    want = []
    pg.forward(c, w, toks, residuals=want)
    from paged_batch_engine_b200.parts.norm import DeltaSum
    runner = make_runner(folders["A"], "float32", page, 128)
    got = []
    for block in runner.model.blocks:
        def forward(residual, delta, ctx, cache, inner=block.forward):
            # a block leaves its branches still to be added: residual + scale * (a + b)
            residual, delta = inner(residual, delta, ctx, cache)
            x = residual.double().cpu()
            if isinstance(delta, DeltaSum):
                x = x + delta.scale * (delta.a.double().cpu() + (delta.b.double().cpu() if delta.b is not None else 0))
            elif delta is not None:
                x = x + delta.double().cpu()
            got.append(x)
            return residual, delta
        block.forward = forward
    h = runner.cache.add_request()
    assert runner.cache.reserve(h, len(toks))
    runner.step([StepEntry(h, toks, [len(toks) - 1])])
    assert len(got) == len(want) == 6
    for i, (a, b) in enumerate(zip(got, want)):
        assert float((a - b).abs().max()) <= 3e-5 * max(1.0, float(b.abs().max())), i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_schedules_agree_with_plain(folders, name, dtype):
    cfg, _, page = GUSORAX[name]
    folder = folders[name]
    reqs = requests_for(name, cfg["vocab"])
    want = plain_logits(folder, reqs)
    schedules = {"whole": ru.whole(reqs), "tail": ru.tail_decoded(reqs, 40), "portions": ru.portions(reqs),
                 "mixed": ru.mixed(reqs, max_live=3, seed=5)}
    for label, recs in schedules.items():
        # the smallest pool the trace may be given and three request slots: pages of finished
        # requests are used again (the pool is poisoned with NaN at the start)
        runner = make_runner(folder, dtype, page, ru.pool_tokens_needed(recs), max_requests=3)
        got = ru.run_records(runner, recs)
        check(got, want, dtype, f"{name}/{label}")
        runner.cache.check_invariants()
        assert runner.cache.num_live_requests == 0
        for gi in range(len(runner.cache.groups)):
            assert runner.cache.num_free_pages(gi) == runner.cache.pools[gi].num_pages


def test_batch_of_unequal_requests_equals_each_alone_and_pages_are_used_again(folders):
    """Eight requests through two request slots, two at a time, against each alone: a page that
    kept something of its former owner would show."""
    cfg, _, page = GUSORAX["A"]
    folder = folders["A"]
    g = torch.Generator().manual_seed(1)
    reqs = {f"s{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
            for i, n in enumerate([50, 9, 33, 64, 2, 71, 18, 40])}
    want = plain_logits(folder, reqs)
    recs = ru.mixed(reqs, max_live=2, seed=9)
    runner = make_runner(folder, "float32", page, ru.pool_tokens_needed(recs), max_requests=2)
    check(ru.run_records(runner, recs), want, "float32", "A/two slots")


def test_many_rows_take_the_experts_sorted_path(folders):
    """A prompt long enough that its routed feed-forward sorts the rows by expert, whole and cut
    so that one portion is below that size."""
    cfg, _, page = GUSORAX["B"]
    g = torch.Generator().manual_seed(12)
    toks = torch.randint(0, cfg["vocab"], (300,), generator=g).tolist()
    want = plain_logits(folders["B"], {"r": toks})
    for cuts in ([300], [200, 37, 63]):
        recs, at = [], 0
        for i, n in enumerate(cuts):
            recs.append({"step": i, "entries": [{"id": "r", "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
            at += n
        runner = make_runner(folders["B"], "float32", page, 320)
        check(ru.run_records(runner, recs), want, "float32", f"B/{cuts}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_token_by_token(folders, name):
    """Every token decoded alone from the first on: windows pass over decoded tokens only, chunks
    begin and end among them, and the cache grows a token at a time over many pages while the
    pages behind the masks go back to the pool."""
    cfg, _, page = GUSORAX[name]
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg["vocab"], (170,), generator=g).tolist()
    want = plain_logits(folders[name], {"r": toks})
    recs = [{"step": i, "entries": [{"id": "r", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    runner = make_runner(folders[name], "float32", page, 192)
    check(ru.run_records(runner, recs), want, "float32", f"{name}/all decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_captured_decode_steps(folders, name, dtype):
    """Steps of single tokens through the captured decode step (a replayed CUDA graph), with
    request counts that leave padding rows (3 live in a step of 4, then fewer as they end)."""
    cfg, _, page = GUSORAX[name]
    g = torch.Generator().manual_seed(6)
    reqs = {f"g{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate([70, 45, 58])}
    want = plain_logits(folders[name], reqs)
    recs = ru.batch_decode(reqs, decode_tokens=30, prefill_group=3, portion=24)
    runner = make_runner(folders[name], dtype, page, 256, max_requests=4)
    from paged_batch_engine_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(runner, decode_graphs=True)
    got = ru.run_records(runner, recs, replayer=rp)
    assert rp.graph_steps >= 30
    check(got, want, dtype, f"{name}/captured decode")


def test_greedy_generation_through_the_entry_point(folders):
    from paged_batch_engine_b200.engine.engine import Engine
    from paged_batch_engine_b200.sampling.params import SamplingParams
    cfg, _, page = GUSORAX["A"]
    c, w = load_plain(folders["A"])
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (5, 37, 60)]
    eng = Engine(folders["A"], dtype="float32", device=DEV, page_size=page, num_pages=64, max_num_seqs=2,
                 max_num_batched_tokens=48, prefill_chunk_cap=24)
    res = eng.generate(prompts, SamplingParams(max_new_tokens=30, temperature=0.0, ignore_eos=True))
    for p, r in zip(prompts, res):
        toks = list(p)
        for _ in range(30):
            lg = pg.forward(c, w, toks)[-1]
            top2 = lg.topk(2).values
            nxt = int(lg.argmax())
            got = r.output_tokens[len(toks) - len(p)]
            if float(top2[0] - top2[1]) > 1e-4:
                assert got == nxt, (len(toks), got, nxt)
            toks.append(got)


def test_command_line_generates_greedily(folders):
    cfg, _, page = GUSORAX["B"]
    c, w = load_plain(folders["B"])
    prompt = [7, 100, 33, 2, 150, 9, 81, 64, 5, 199, 12]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "pbe-qwen"), folders["B"], "--prompt-ids",
                        ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", "float32", "--ignore-eos",
                        "--page-size", str(page), "--kv-cache-blocks-per-layer", "32", "--max-num-seqs", "2"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")][0]
    toks = list(prompt)
    for got in line["output_ids"]:
        lg = pg.forward(c, w, toks)[-1]
        top2 = lg.topk(2).values
        if float(top2[0] - top2[1]) > 1e-4:
            assert got == int(lg.argmax()), (len(toks), got, int(lg.argmax()))
        toks.append(got)
    assert len(line["output_ids"]) == 6


def test_trace_runner_program(folders, tmp_path):
    cfg, _, page = GUSORAX["A"]
    reqs = requests_for("A", cfg["vocab"])
    want = plain_logits(folders["A"], reqs)
    recs = ru.mixed(reqs, max_live=4, seed=2)
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(ru.pool_tokens_needed(recs))],
                       input="\n".join(json.dumps(r) for r in recs) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {r['step']}" for r in recs]
    progress, worst = {}, 0.0
    for r in recs:
        rows = np.fromfile(out / f"{r['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        i = 0
        for e in r["entries"]:
            base = progress.get(e["id"], 0)
            for wpos in e["want"]:
                worst = max(worst, float(np.abs(rows[i] - want[e["id"]][base + wpos].numpy()).max()))
                i += 1
            progress[e["id"]] = base + len(e["tokens"])
    assert worst <= TOL_F32_REL * max(1.0, max(float(v.abs().max()) for v in want.values()))
