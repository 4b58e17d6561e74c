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
