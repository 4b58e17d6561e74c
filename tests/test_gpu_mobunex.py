"""Mobunex on the GPU against the plain implementation: every mechanism alone, then whole models
under every way of cutting and batching (whole, last tokens decoded, portions down to two tokens,
mixed batches with pages and state slots used again), long decoding, captured decode steps,
generation through the entry point, and the trace runner itself; float32 and bfloat16, three tiny
configurations."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import replay_util as ru
from tests.helpers import MOBUNEX, load_plain, make_mobunex_folder
from tests.plain import plain_mobunex as pm

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
DEV = "cuda:0"
TOL_F32_REL = 3e-5          # max |dlogit| over the largest logit: summation order only
# bfloat16: a row's root-mean-square difference over the root mean square of all logits.  A router
# may choose another expert for a token whose scores lie within the rounding of 16-bit activations
# (the float32 runs are the sharp test of every schedule), so a few rows may lie beyond the bound.
TOL_BF16_RMS_MEAN = 0.03
TOL_BF16_RMS = 0.12
BF16_ROWS_BEYOND = 0.03


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_mobunex_folder(tmp_path_factory.mktemp(f"mob_{name}"), cfg, seed)
            for name, (cfg, seed, _) in MOBUNEX.items()}


def _ops():
    from paged_batch_engine_b200.csrc import ops
    return ops


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


# ================================================================ mechanisms alone
@pytest.mark.parametrize("W, dt, alpha", [(64, torch.float32, 2.0), (200, torch.bfloat16, 1.0), (37, torch.float32, 0.25)])
def test_norm_after_the_scaled_sum_with_one_gain(W, dt, alpha):
    ops = _ops()
    g = torch.Generator().manual_seed(W)
    T = 6
    x = torch.randn(T, W, generator=g) * 3
    a, b = torch.randn(T, W, generator=g).to(dt), torch.randn(T, W, generator=g).to(dt)
    gain = torch.tensor([0.7])
    want = pm.post_norm(x.double(), a.double() + b.double(), alpha, gain.double(), 1e-5)
    normed = torch.empty(T, W, device=DEV)
    lp = ops.unit_norm(x.to(DEV), a.to(DEV), b.to(DEV), alpha, gain.to(DEV), 1e-5, dt, normed=normed)
    assert torch.allclose(normed.cpu().double(), want, atol=3e-6, rtol=1e-5)
    assert torch.equal(lp.cpu(), normed.cpu().to(dt))
    # one branch, none; gathered rows; the sum written back for a plain residual add
    one = pm.post_norm(x.double(), a.double(), alpha, gain.double(), 1e-5)
    n1 = torch.empty(T, W, device=DEV)
    assert ops.unit_norm(x.to(DEV), None, a.to(DEV), alpha, gain.to(DEV), 1e-5, None, normed=n1) is None
    assert torch.allclose(n1.cpu().double(), one, atol=3e-6, rtol=1e-5)
    rows = i32([4, 0, 4])
    got = ops.unit_norm(x.to(DEV), None, None, 1.0, gain.to(DEV), 1e-5, torch.float32, rows=rows)
    assert torch.allclose(got.cpu().double(), (pm.rms_unit(x.double(), 1e-5) * 0.7)[[4, 0, 4]], atol=3e-6, rtol=1e-5)
    res = x.to(DEV)
    ops.unit_norm(res, a.to(DEV), None, 1.0, gain.to(DEV), 1e-5, dt, sum_out=res)
    assert torch.allclose(res.cpu().double(), x.double() + a.double(), atol=1e-6)


@pytest.mark.parametrize("W, n_prev, dt", [(64, 1, torch.float32), (100, 4, torch.bfloat16), (33, 6, torch.float32)])
def test_mix_over_depth_in_the_norm_launch(W, n_prev, dt):
    ops = _ops()
    g = torch.Generator().manual_seed(W + n_prev)
    T = 5
    stack = torch.randn(n_prev + 3, T, W, generator=g)
    x, y = torch.randn(T, W, generator=g), torch.randn(T, W, generator=g).to(dt)
    mix = torch.randn(n_prev + 1, generator=g)
    gain = torch.tensor([1.3])
    n = pm.post_norm(x.double(), y.double(), 2.0, gain.double(), 1e-6)
    want = pm.depth_mix([stack[j].double() for j in range(n_prev)] + [n], mix.double())
    dev_stack = stack.to(DEV)
    mixed = torch.empty(T, W, device=DEV)
    lp = ops.unit_norm(x.to(DEV), y.to(DEV), None, 2.0, gain.to(DEV), 1e-6, dt, normed=dev_stack[n_prev],
                       stack=dev_stack, n_prev=n_prev, mix=mix.to(DEV), mixed=mixed)
    assert torch.allclose(dev_stack[n_prev].cpu().double(), n, atol=3e-6, rtol=1e-5)
    assert torch.allclose(mixed.cpu().double(), want, atol=1e-5, rtol=1e-5)
    assert torch.equal(lp.cpu(), mixed.cpu().to(dt))
    assert torch.equal(dev_stack[n_prev + 1:].cpu(), stack[n_prev + 1:])


@pytest.mark.parametrize("W, dt", [(64, torch.float32), (200, torch.bfloat16), (37, torch.bfloat16)])
def test_normed_embedding_rows(W, dt):
    ops = _ops()
    g = torch.Generator().manual_seed(W)
    table = (torch.randn(50, W, generator=g) * 4).to(dt)
    ids = [3, 49, 0, 3, 17]
    out = torch.empty(5, W, device=DEV)
    lp = ops.embedding_unit_norm(out, table.to(DEV), i32(ids), torch.tensor([1.2], device=DEV), 1e-5, torch.bfloat16)
    want = pm.rms_unit(table.double()[ids], 1e-5) * 1.2
    assert torch.allclose(out.cpu().double(), want, atol=3e-6, rtol=1e-5)
    assert torch.equal(lp.cpu(), out.cpu().to(torch.bfloat16))


def _gate_weights(C, B, g, dt):
    n = C // B
    return dict(ra=(torch.randn(B, n, n, generator=g) * 0.4).to(dt), ri=(torch.randn(B, n, n, generator=g) * 0.4).to(dt),
                rab=torch.randn(B, n, generator=g), rib=torch.randn(B, n, generator=g),
                lam=torch.randn(C, generator=g) * 1.5 - 0.5)


def _plain_coefficients(u, w):
    r = pm.block_gates(u, w["ra"].double(), w["rab"].double())
    i = pm.block_gates(u, w["ri"].double(), w["rib"].double())
    return r, i


@pytest.mark.parametrize("C, B, dt", [(48, 3, torch.float32), (160, 1, torch.bfloat16), (70, 7, torch.float32),
                                      (66, 1, torch.float32), (256, 2, torch.bfloat16)])
def test_recurrence_gates_and_coefficients(C, B, dt):
    ops = _ops()
    g = torch.Generator().manual_seed(C + B)
    T = 37
    wide = torch.randn(T, C + 5, generator=g).to(dt)
    u = wide[:, 3:3 + C]
    w = _gate_weights(C, B, g, dt)
    r, i = _plain_coefficients(u.double(), w)
    log_a = -8.0 * r * pm.softplus(w["lam"].double())
    a_want = torch.exp(log_a)
    b_want = torch.sqrt(-torch.expm1(2 * log_a)) * i * u.double()
    a, b = ops.recurrence_gates(wide.to(DEV)[:, 3:3 + C], w["ra"].to(DEV), w["ri"].to(DEV),
                                w["rab"].reshape(-1).to(DEV), w["rib"].reshape(-1).to(DEV), w["lam"].to(DEV), 8.0)
    assert torch.allclose(a.cpu().double(), a_want, atol=2e-6, rtol=2e-5)
    assert torch.allclose(b.cpu().double(), b_want, atol=2e-6, rtol=3e-5)


@pytest.mark.parametrize("C, B", [(48, 3), (160, 1), (70, 7), (256, 2), (40, 5)])
def test_gates_on_the_tensor_cores_and_coefficients_formed_in_the_scan(C, B):
    """bfloat16 input and maps: the products on the tensor cores are sums of exact products, so the
    scan that forms a and b from them equals the recurrence on float64 gates of the same numbers."""
    ops = _ops()
    g = torch.Generator().manual_seed(C * 3 + B)
    lens, starts, slots = [50, 1, 13], [0, 50, 51], [2, 0, 1]
    T = sum(lens)
    wide = torch.randn(T, 2 * C + 5, generator=g).to(torch.bfloat16)
    u, y = wide[:, 3:3 + C], wide[:, 3 + C:3 + 2 * C]
    w = _gate_weights(C, B, g, torch.bfloat16)
    r, i = _plain_coefficients(u.double(), w)
    want = torch.cat([pm.gated_recurrence(u[s:s + n].double(), r[s:s + n], i[s:s + n], w["lam"].double())
                      for s, n in zip(starts, lens)]) * pm.gelu_tanh(y.double())
    dev = wide.to(DEV)
    du, dy = dev[:, 3:3 + C], dev[:, 3 + C:3 + 2 * C]
    z = ops.gate_products(du, torch.cat([w["ra"], w["ri"]], dim=1).contiguous().to(DEV))
    n = C // B
    zr = torch.einsum("tbi,boi->tbo", u.double().reshape(T, B, n), w["ra"].double())
    assert torch.allclose(z[:, :, :n].cpu().double(), zr, atol=1e-5, rtol=1e-5)
    state = torch.zeros(4, C, device=DEV)
    gates = (z, du, w["rab"].reshape(-1).to(DEV), w["rib"].reshape(-1).to(DEV), w["lam"].to(DEV), 8.0)
    got = ops.gated_scan(None, None, dy, state, i32(starts), i32(lens), i32(slots), 3, torch.bfloat16, gates=gates)
    assert torch.allclose(got.float().cpu().double(), want, atol=2e-2, rtol=2e-2)
    # S itself, in float32, is the sharper comparison
    state.zero_()
    S = ops.gated_scan(None, None, None, state, i32(starts), i32(lens), i32(slots), 3, torch.bfloat16, activation=None,
                       gates=gates)
    del S
    ends = torch.stack([pm.gated_recurrence(u[s:s + n_].double(), r[s:s + n_], i[s:s + n_], w["lam"].double())[-1]
                        for s, n_ in zip(starts, lens)])
    assert torch.allclose(state[slots].cpu().double(), ends, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("C, dt", [(48, torch.float32), (130, torch.bfloat16)])
def test_gated_scan_carries_its_state(C, dt):
    """Unequal requests in one launch equal each alone; a request cut into launches equals it whole;
    a reused state row holds nothing of its former owner; long portions as chunks of 5 and 16 rows
    beside a request in progress."""
    ops = _ops()
    g = torch.Generator().manual_seed(C)
    lens = [11, 1, 75]
    starts = [0, 11, 12]
    T = sum(lens)
    a = torch.rand(T, C, generator=g) * 0.6 + 0.39
    b = torch.randn(T, C, generator=g)
    wide = torch.randn(T, C + 4, generator=g).to(dt)
    y = wide[:, 2:2 + C]

    def plain(rows, S0=None):
        S = torch.zeros(C, dtype=torch.float64) if S0 is None else S0
        out = []
        for t in rows:
            S = a[t].double() * S + b[t].double()
            out.append(S * pm.gelu_tanh(y[t].double()))
        return torch.stack(out), S
    want = torch.cat([plain(range(s, s + n))[0] for s, n in zip(starts, lens)])
    tol = 2e-5 if dt == torch.float32 else 2e-2
    state = torch.full((5, C), float("nan"), device=DEV)
    slots = [3, 0, 4]
    state[slots] = 0
    dev_y = wide.to(DEV)[:, 2:2 + C]
    got = ops.gated_scan(a.to(DEV), b.to(DEV), dev_y, state, i32(starts), i32(lens), i32(slots), 3, dt)
    assert torch.allclose(got.float().cpu().double(), want, atol=tol, rtol=tol)
    assert torch.allclose(state[4].cpu().double(), plain(range(12, T))[1], atol=1e-5, rtol=1e-5)
    # the third request again, in pieces, in the row the first one used
    state[3] = 0
    outs, at = [], 12
    for n in [1, 2, 1, 30, 1, 40]:
        outs.append(ops.gated_scan(a[at:at + n].to(DEV), b[at:at + n].to(DEV), dev_y[at:at + n], state, i32([0]),
                                   i32([n]), i32([3]), 1, dt))
        at += n
    assert torch.allclose(torch.cat(outs).float().cpu().double(), want[12:], atol=tol, rtol=tol)
    assert torch.allclose(state[3].cpu(), state[4].cpu(), atol=1e-6, rtol=1e-5)
    # chunks side by side: the long request starts from a state it carried in
    from paged_batch_engine_b200.engine.batch import RecurrencePlan, recurrence_plan_arrays
    for chunk in (5, 16):
        state[slots] = 0
        carried = torch.randn(C, generator=g)
        state[4] = carried.to(DEV)
        first, scan, second, entries = recurrence_plan_arrays(starts, lens, slots, chunk)
        assert entries > 0
        dev = i32(first + scan + second)
        n1, n2 = len(first), len(first) + len(scan)
        plan = RecurrencePlan(entries, dev[:n1], n1, dev[n1:n2], len(scan), dev[n2:], len(second))
        got = ops.gated_scan(a.to(DEV), b.to(DEV), dev_y, state, i32(starts), i32(lens), i32(slots), 3, dt, plan=plan)
        long_want, S_end = plain(range(12, T), carried.double())
        assert torch.allclose(got[:12].float().cpu().double(), want[:12], atol=tol, rtol=tol)
        assert torch.allclose(got[12:].float().cpu().double(), long_want, atol=tol, rtol=tol)
        assert torch.allclose(state[4].cpu().double(), S_end, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("E, top, count, keep", [(8, 3, 4, 2), (6, 2, 3, 2), (12, 4, 3, 2), (8, 1, 8, 3), (130, 6, 13, 5),
                                                (5, 5, 1, 1), (64, 8, 64, 40)])
def test_router_with_sigmoid_scores_correction_and_group_ranks(E, top, count, keep):
    ops = _ops()
    g = torch.Generator().manual_seed(E * 7 + top)
    T = 200
    logits = torch.randn(T, E, generator=g) * 2
    corr = torch.randn(E, generator=g) * 0.6 - 0.8          # most choice scores are negative
    h = torch.eye(E, dtype=torch.float64)
    picked, weights = pm.route(logits.double(), h, corr.double(), dict(experts=E, top=top, groups=dict(count=count, keep=keep)))
    chosen, w = ops.route(logits.to(DEV), top, count, keep, 1.0, score="sigmoid", correction=corr.to(DEV),
                          group_rank="top2_sum")
    got = {(t, int(e)): float(x) for t in range(T) for e, x in zip(chosen[t].cpu(), w[t].cpu())}
    want = {(t, int(e)): float(x) for t in range(T) for e, x in zip(picked[t], weights[t])}
    assert set(got) == set(want)
    assert max(abs(got[k] - want[k]) for k in want) <= 2e-6


def test_router_rows_that_are_not_numbers_choose_experts_that_exist():
    ops = _ops()
    logits = torch.full((3, 8), float("nan"))
    logits[1] = torch.randn(8)
    chosen, w = ops.route(logits.to(DEV), 3, 4, 2, 1.0, score="sigmoid", correction=torch.zeros(8, device=DEV),
                          group_rank="top2_sum")
    assert int(chosen.min()) >= 0 and int(chosen.max()) < 8
    assert all(len(set(row.tolist())) == 3 for row in chosen.cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W, F, E, top, count, keep, shared", [(64, 48, 6, 2, 3, 2, 24), (100, 24, 9, 4, 3, 2, None),
                                                               (40, 130, 4, 1, 4, 2, 56)])
def test_routed_experts_with_a_shared_expert(W, F, E, top, count, keep, shared, dtype):
    """A few rows (every row reads its experts) and many (rows sorted by expert), against the plain
    loop over tokens and experts."""
    from paged_batch_engine_b200.parts import RoutedExperts
    g = torch.Generator().manual_seed(W + F)
    part = RoutedExperts(W, F, E, top, dtype, DEV, groups=count, keep=keep, router_score="sigmoid", correction=True,
                         group_rank="top2_sum", shared_size=shared)
    w = {"m.router": torch.randn(E, W, generator=g) * 0.5, "m.correction": torch.randn(E, generator=g) * 0.4}
    for name, f in [(f"e{e}", F) for e in range(E)] + ([("shared", shared)] if shared else []):
        w[f"m.{name}.gate"] = torch.randn(f, W, generator=g) * 0.4
        w[f"m.{name}.up"] = torch.randn(f, W, generator=g) * 0.4
        w[f"m.{name}.down"] = torch.randn(W, f, generator=g) * 0.3
    w = {k: v.to(dtype if v.dim() == 2 else torch.float32) for k, v in w.items()}
    part.load({k: v.to(DEV) for k, v in w.items()}, "m.")
    wd = {k: v.double() for k, v in w.items()}
    mlp = dict(router=dict(experts=E, top=top, groups=dict(count=count, keep=keep)), expert=dict(ff=F),
               shared=dict(ff=shared) if shared else None)
    for rows in (5, 300):
        x = torch.randn(rows, W, generator=g).to(dtype)
        got = part.forward(x.to(DEV), None).float().cpu().double()
        want = pm.routed_ff(x.double(), wd, "m.", mlp)
        tol = (2e-5 if dtype == torch.float32 else 3e-2) * float(want.abs().max())
        err = (got - want).abs().max(dim=1).values
        # a router may choose otherwise for a row whose scores tie within 16-bit rounding of the products
        beyond = int((err > tol).sum())
        assert beyond <= (0 if dtype == torch.float32 else max(1, rows // 50)), (rows, beyond, float(err.max()), tol)


# ================================================================ the mixers with a stand-out key
def _run_part(part, x, cuts, page, num_pages, dtype, requests=2):
    """Feeds rows x of one request through the part in portions of the given sizes."""
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    st = CacheStorage([part.cache_need()], page, num_pages, requests, dtype, DEV, poison=True)
    keys = [(st.layer(0).group,) + k for k in part.work_keys()]
    h = st.manager.add_request()
    outs, i = [], 0
    for n in cuts:
        assert st.manager.reserve(h, n)
        ctx = StepContext(st.manager, [StepEntry(h, [0] * n, [])], torch.device(DEV), keys)
        outs.append(part.forward(x[i:i + n].to(DEV).to(dtype), ctx, st.layer(0)).float().cpu())
        st.manager.commit(h, n)
        i += n
    st.manager.check_invariants()
    return torch.cat(outs)


def _stand_out_input(T, hidden, mark, g):
    x = torch.randn(T, hidden, generator=g) * 0.5
    x[:, 0] = 3.0                          # every query looks along the first key coordinate
    x[:, 1] = 0.02 * torch.randn(T, generator=g)
    x[mark, 1] = 30.0                      # the stand-out key: all of its direction is that coordinate
    x[mark, 2:] = 2.0                      # and a value that shows
    return x


def _window_part(H, G, D, E, size, hidden, dtype, seed, scale):
    """Weights made so that every query looks along the first key coordinate and only input column 1
    reaches that coordinate: a token with a large column 1 is a key that every query scores far above
    all others (the unit norms leave directions only)."""
    from paged_batch_engine_b200.parts import MaskedAttention
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g)
    part = MaskedAttention(hidden, H, G, D, E, scale, 1e-5, dtype, DEV, mask="window", mask_size=size, qk_norm="unit",
                           proj_bias="qkv", head_temperature=True)
    w = {"p.q": rnd(H * D, hidden) * 0.05, "p.k": rnd(G * D, hidden) * 0.3, "p.v": rnd(G * E, hidden) * 0.3,
         "p.o": rnd(hidden, H * E) * 0.3, "p.q.b": rnd(H * D) * 0.02, "p.k.b": rnd(G * D) * 0.02,
         "p.v.b": rnd(G * E) * 0.3, "p.temp": 0.6 + torch.rand(H, generator=g)}
    w["p.q"].view(H, D, hidden)[:, 0, :] = 0
    w["p.q"].view(H, D, hidden)[:, 0, 0] = 2.0
    w["p.k"].view(G, D, hidden)[:, 0, :] = 0
    w["p.k"].view(G, D, hidden)[:, 0, 1] = 1.0
    w["p.k"][:, 0] = 0
    w["p.q.b"].view(H, D)[:, 0] = 0
    w["p.k.b"].view(G, D)[:, 0] = 0
    w = {k: v.to(dtype if v.dim() == 2 else torch.float32) for k, v in w.items()}
    part.load({k: v.to(DEV) for k, v in w.items()}, "p.")
    m = dict(heads=H, kv_heads=G, dim=D, vdim=E, scale=scale, mask=dict(size=size))
    return part, (lambda x: pm.window_attention_mixer(x, {k: v.double() for k, v in w.items()}, "p.", m, 1e-5))


def _latent_part(H, D, R, dims, V, kv, qr, size, hidden, dtype, seed, scale, scaling):
    """The same idea through the latents: latent coordinate 0 of the keys reads input column 1 only,
    key coordinate 0 of every head reads latent coordinate 0 only, and every head's first query
    coordinate reads the constant column 0 through the query latent."""
    from paged_batch_engine_b200.parts import LatentAttention
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g)
    rot = dict(base=1000.0, dims=dims)
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    part = LatentAttention(hidden, H, D, R, V, kv, qr, scale, 1e-5, dtype, DEV, rotary=rot, sink=False, out_gate="each",
                           window=size)
    w = {"p.dq": rnd(qr, hidden) * 0.05, "p.dq.norm": 1 + 0.1 * rnd(qr), "p.uq": rnd(H * (D + R), qr) * 0.05,
         "p.dkv": rnd(kv + R, hidden) * 0.2, "p.dkv.norm": 1 + 0.1 * rnd(kv), "p.uk": rnd(H * D, kv) * 0.1,
         "p.uv": rnd(H * V, kv) * 0.3, "p.g": rnd(H * V, hidden) * 0.3, "p.o": rnd(hidden, H * V) * 0.3}
    w["p.dq"][0, :] = 0
    w["p.dq"][0, 0] = 2.0                  # query latent 0 = the constant column
    w["p.uq"].view(H, D + R, qr)[:, 0, :] = 0
    w["p.uq"].view(H, D + R, qr)[:, 0, 0] = 1.0
    w["p.dkv"][0, :] = 0
    w["p.dkv"][0, 1] = 1.0                 # key latent 0 = input column 1
    w["p.dkv"][:, 1] = 0
    w["p.dkv"][0, 1] = 1.0
    w["p.uk"].view(H, D, kv)[:, 0, :] = 0
    w["p.uk"].view(H, D, kv)[:, 0, 0] = 1.0
    w["p.uk"][:, 0] = 0
    w["p.uk"].view(H, D, kv)[:, 0, 0] = 1.0
    w["p.dq.norm"][0] = w["p.dkv.norm"][0] = 1.0
    w = {k: v.to(dtype if v.dim() == 2 else torch.float32) for k, v in w.items()}
    part.load({k: v.to(DEV) for k, v in w.items()}, "p.")
    m = dict(heads=H, dim=D, rot_dim=R, vdim=V, kv_rank=kv, q_rank=qr, scale=scale, mask=dict(size=size), rot=rot)
    return part, (lambda x: pm.latent_attention_mixer(x, {k: v.double() for k, v in w.items()}, "p.", m, 1e-5))


def _window_marks(T, head, size, page):
    # the key leaves sight at mark + size: in the prompt portion, at its last row, among the decoded, never
    marks = {0, 1, page - 1, page, head - size - 5, head - size - 1, head - size, head - size + 6, T - size,
             T - size - 1, T - 3}
    return sorted(x for x in marks if 0 <= x < T)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind, shape, size, page, T", [
    ("window", (3, 1, 24, 40), 21, 8, 90),            # float32-arithmetic kernel in both dtypes; a window off the page grid
    ("window", (8, 2, 32, 16), 64, 16, 200),          # tensor-core kernel for bfloat16; a window of four whole pages
    ("window", (4, 4, 16, 48), 600, 16, 1300),        # a far key among hundreds, over the edge of a key split
    ("window", (2, 1, 16, 16), 1, 4, 30),             # a row sees itself only
    ("latent", (3, 16, 8, 8, 24, 40, 24, (8.0, 64, 16.0, 2.0)), 21, 8, 90),
    ("latent", (20, 8, 4, 2, 8, 28, 16, None), 64, 16, 200),
    ("latent", (4, 32, 16, 16, 56, 48, 40, (2.5, 32, 16.0, 2.0)), 600, 16, 1300),
    ("latent", (2, 16, 4, 4, 16, 12, 8, None), 1, 4, 30),
])
def test_attention_with_a_stand_out_key(kind, shape, size, page, T, dtype):
    """One key that every query scores far above all others, placed in turn where a fault would
    show: the first tokens, a page's edges, so that the last row that sees it and the first that
    does not fall in the prompt portion or among the tokens decoded alone, and far back among
    hundreds.  A window that is one token off moves that key in or out of a row's sight."""
    hidden = 40
    if kind == "window":
        H, G, D, E = shape
        part, plain = _window_part(H, G, D, E, size, hidden, dtype, T + H, scale=6.0 / D)
    else:
        H, D, R, dims, V, kv, qr, scaling = shape
        part, plain = _latent_part(H, D, R, dims, V, kv, qr, size, hidden, dtype, T + H, 0.4, scaling)
    g = torch.Generator().manual_seed(T)
    tail = 14 if T < 500 else 40
    head = T - tail
    marks = _window_marks(T, head, size, page)
    edge_seen = False
    for mark in marks[:: (1 if dtype == torch.float32 and T < 500 else 3)]:
        x = _stand_out_input(T, hidden, mark, g)
        want = plain(x.to(dtype).double())
        cuts = ([head] if T < 500 else [500, head - 500]) + [1] * tail
        got = _run_part(part, x, cuts, page, (T + page - 1) // page + 3, dtype).double()
        scale = float(want.abs().max())
        tol = (3e-5 if dtype == torch.float32 else 4e-2) * scale
        err = (got - want).abs().max(dim=1).values
        assert float(err.max()) <= tol, (kind, mark, int(err.argmax()), float(err.max()), tol)
        last = mark + size - 1
        if size > 1 and last + 1 < T:
            # the rows on both sides of the window's edge differ by far more than the tolerance
            edge_seen = edge_seen or float((want[last] - want[last + 1]).abs().max()) > 5 * tol
    assert edge_seen or size == 1 or size >= T


@pytest.mark.parametrize("kind", ["window", "latent", "recurrence"])
def test_mixers_in_portions_of_two_and_other_requests_beside(kind):
    """Two unequal requests in the same steps, one of them in portions of two tokens, on pages
    (or in a state row) that another request used before."""
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    from paged_batch_engine_b200.parts import GatedLinearRecurrence
    hidden, dtype = 40, torch.float32
    g = torch.Generator().manual_seed(5)
    if kind == "window":
        part, plain = _window_part(4, 2, 16, 24, 9, hidden, dtype, 3, 0.4)
    elif kind == "latent":
        part, plain = _latent_part(3, 16, 8, 8, 24, 40, 24, 9, hidden, dtype, 3, 0.4, (8.0, 64, 16.0, 2.0))
    else:
        C, B, taps = 48, 3, 4
        part = GatedLinearRecurrence(hidden, C, B, taps, dtype, DEV)
        gw = _gate_weights(C, B, g, dtype)
        w = {"p.y": torch.randn(C, hidden, generator=g) * 0.3, "p.y.b": torch.randn(C, generator=g) * 0.3,
             "p.x": torch.randn(C, hidden, generator=g) * 0.3, "p.x.b": torch.randn(C, generator=g) * 0.3,
             "p.conv": torch.randn(C, taps, generator=g) * 0.5, "p.conv.b": torch.randn(C, generator=g) * 0.2,
             "p.ra": gw["ra"], "p.ra.b": gw["rab"], "p.ri": gw["ri"], "p.ri.b": gw["rib"], "p.lam": gw["lam"],
             "p.o": torch.randn(hidden, C, generator=g) * 0.3}
        part.load({k: v.to(DEV) for k, v in w.items()}, "p.")
        plain = lambda x: pm.rglru_mixer(x, {k: v.double() for k, v in w.items()}, "p.", dict(width=C, blocks=B, conv=taps))
    xa, xb, xc = (torch.randn(n, hidden, generator=g) for n in (61, 30, 25))
    page = 4
    st = CacheStorage([part.cache_need()], page, 40, 2, dtype, DEV, poison=True)
    keys = [(st.layer(0).group,) + k for k in part.work_keys()]

    def step(pairs):
        entries, rows = [], []
        for h, x in pairs:
            assert st.manager.reserve(h, x.shape[0])
            entries.append(StepEntry(h, [0] * x.shape[0], []))
            rows.append(x)
        ctx = StepContext(st.manager, entries, torch.device(DEV), keys)
        y = part.forward(torch.cat(rows).to(DEV), ctx, st.layer(0)).cpu()
        out, at = [], 0
        for h, x in pairs:
            out.append(y[at:at + x.shape[0]])
            at += x.shape[0]
            st.manager.commit(h, x.shape[0])
        return out

    def zero_state(h):
        st.zero_state([st.manager.state_slot(h)])

    hc = st.manager.add_request()
    zero_state(hc)
    step([(hc, xc)])                        # someone else's keys and state, then given back
    st.manager.free(hc)
    ha, hb = st.manager.add_request(), st.manager.add_request()
    zero_state(ha), zero_state(hb)
    outs = {ha: [], hb: []}
    done_a = done_b = 0
    plan = [(2, 7), (2, 1), (2, 1), (31, 1), (2, 12), (2, 1), (20, 7)]
    for na, nb in plan:
        oa, ob = step([(ha, xa[done_a:done_a + na]), (hb, xb[done_b:done_b + nb])])
        outs[ha].append(oa), outs[hb].append(ob)
        done_a, done_b = done_a + na, done_b + nb
    assert done_a == 61 and done_b == 30
    for h, x in ((ha, xa), (hb, xb)):
        want = plain(x.double())
        got = torch.cat(outs[h]).double()
        assert float((got - want).abs().max()) <= 3e-5 * float(want.abs().max()), kind


# ================================================================ whole models
LENGTHS = {"A": [3, 41, 97, 150], "B": [1, 30, 75, 131], "C": [2, 52, 110, 171]}


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
            _plain_cache[key] = pm.forward(cfg, w, toks).float()
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
    print(f"\n[mobunex] {label} {dtype}: max|dlogit| = {worst:.3e} at {where}, max|logit| = {scale:.3f}, "
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


def test_what_every_layer_hands_on(folders):
    """The stream after every layer (after its mix over depth) against the plain implementation's."""
    cfg, _, page = MOBUNEX["C"]
    c, w = load_plain(folders["C"])
    toks = requests_for("C", cfg["vocab"])["C1"]
    want = []
    pm.forward(c, w, toks, residuals=want)
    runner = make_runner(folders["C"], "float32", page, 64)
    seen = []
    for b in runner.model.blocks:
        def wrapped(residual, delta, ctx, cache, inner=b.forward):
            out = inner(residual, delta, ctx, cache)
            seen.append(out[0].current.clone())
            return out
        b.forward = wrapped
    ru.run_records(runner, ru.whole({"r": toks}))
    assert len(seen) == len(want) == 5
    for i, (a, b) in enumerate(zip(seen, want)):
        assert float((a.cpu().double() - b).abs().max()) <= 2e-5 * max(1.0, float(b.abs().max())), i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_schedules_agree_with_plain(folders, name, dtype):
    cfg, _, page = MOBUNEX[name]
    folder = folders[name]
    reqs = requests_for(name, cfg["vocab"])
    want = plain_logits(folder, reqs)
    schedules = {"whole": ru.whole(reqs), "tail": ru.tail_decoded(reqs, 40), "portions": ru.portions(reqs),
                 "mixed": ru.mixed(reqs, max_live=3, seed=5)}
    for label, recs in schedules.items():
        # the smallest pool the trace may be given and three request slots: pages and state rows
        # of finished requests are used again (the pool is poisoned with NaN at the start)
        runner = make_runner(folder, dtype, page, ru.pool_tokens_needed(recs), max_requests=3)
        got = ru.run_records(runner, recs)
        check(got, want, dtype, f"{name}/{label}")
        runner.cache.check_invariants()
        assert runner.cache.num_live_requests == 0
        for gi in range(len(runner.cache.groups)):
            assert runner.cache.num_free_pages(gi) == runner.cache.pools[gi].num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_of_real_widths(tmp_path, dtype):
    """Heads of 128 (+ 64 rotated) over a latent of 512, windowed heads of 128 on one key head, a
    recurrence of 512 channels in blocks of 256, sixteen experts: the widths at which the tensor-core
    kernels run with their full tiles; a prompt, then tokens decoded past every window."""
    from tests.helpers import _mlat, _mmoe, _mrec, _mwin
    cfg = dict(architecture="Mobunex", width=512, vocab=640, norm=dict(eps=1e-6), postln_alpha=1.2, layers=[
        dict(type="latent_attention", mixer=_mlat(4, 128, 64, 64, 128, 512, 384, 1000000.0, 192 ** -0.5, 100,
                                                  (8.0, 128, 32.0, 1.0)), mlp=dict(kind="dense", ff=768)),
        dict(type="attention", mixer=_mwin(4, 1, 128, 128, 90, 128 ** -0.5), mlp=_mmoe(128, 16, 4, 4, 2, shared=128)),
        dict(type="rglru", mixer=_mrec(512, 2, 4), mlp=None),
    ])
    folder = make_mobunex_folder(tmp_path / "real", cfg, 61, gain=0.4)
    g = torch.Generator().manual_seed(8)
    reqs = {"r": torch.randint(0, cfg["vocab"], (190,), generator=g).tolist()}
    want = plain_logits(folder, reqs)
    recs = ru.tail_decoded(reqs, 30)
    runner = make_runner(folder, dtype, 16, 256)
    check(ru.run_records(runner, recs), want, dtype, "real widths")


def test_layers_without_a_mask_see_every_earlier_token(tmp_path):
    """A configuration whose attention layers name no mask (and no number of key heads)."""
    import copy
    cfg = copy.deepcopy(MOBUNEX["A"][0])
    del cfg["layers"][0]["mixer"]["mask"], cfg["layers"][0]["mixer"]["kv_heads"], cfg["layers"][2]["mixer"]["mask"]
    folder = make_mobunex_folder(tmp_path / "nomask", cfg, 71)
    g = torch.Generator().manual_seed(9)
    reqs = {"r": torch.randint(0, cfg["vocab"], (120,), generator=g).tolist()}
    want = plain_logits(folder, reqs)
    runner = make_runner(folder, "float32", 8, 128)
    check(ru.run_records(runner, ru.tail_decoded(reqs, 30)), want, "float32", "no masks")


def test_batch_of_unequal_requests_equals_each_alone_and_slots_are_used_again(folders):
    """Eight requests through two request slots, two at a time, against each alone: a state row
    or a page that kept something of its former owner would show."""
    cfg, _, page = MOBUNEX["A"]
    folder = folders["A"]
    g = torch.Generator().manual_seed(1)
    reqs = {f"s{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
            for i, n in enumerate([50, 9, 33, 64, 2, 71, 18, 40])}
    want = plain_logits(folder, reqs)
    recs = ru.mixed(reqs, max_live=2, seed=9)
    runner = make_runner(folder, "float32", page, ru.pool_tokens_needed(recs), max_requests=2)
    check(ru.run_records(runner, recs), want, "float32", "A/two slots")
    assert runner.cache.state_slot_assignments == 8


def test_long_prompts_take_the_chunked_recurrence_and_the_sorted_experts(folders):
    """A prompt long enough that the recurrence runs as chunks side by side and the routed
    feed-forward sorts the rows by expert, whole and cut so that one portion is below those sizes."""
    cfg, _, page = MOBUNEX["A"]
    g = torch.Generator().manual_seed(12)
    toks = torch.randint(0, cfg["vocab"], (300,), generator=g).tolist()
    want = plain_logits(folders["A"], {"r": toks})
    for cuts in ([300], [200, 37, 63]):
        recs, at = [], 0
        for i, n in enumerate(cuts):
            recs.append({"step": i, "entries": [{"id": "r", "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
            at += n
        runner = make_runner(folders["A"], "float32", page, 320)
        check(ru.run_records(runner, recs), want, "float32", f"A/{cuts}")


@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_token_by_token(folders, name):
    """Every token decoded alone from the first on: the convolution starts from its zeros, the
    states and the cache grow a token at a time over many pages, every window passes over
    decoded tokens."""
    cfg, _, page = MOBUNEX[name]
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg["vocab"], (140,), generator=g).tolist()
    want = plain_logits(folders[name], {"r": toks})
    recs = [{"step": i, "entries": [{"id": "r", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    runner = make_runner(folders[name], "float32", page, 192)
    check(ru.run_records(runner, recs), want, "float32", f"{name}/all decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_captured_decode_steps(folders, name, dtype):
    """Steps of single tokens through the captured decode step (a replayed CUDA graph), with
    request counts that leave padding rows (3 live in a step of 4, then fewer as they end)."""
    cfg, _, page = MOBUNEX[name]
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
    cfg, _, page = MOBUNEX["C"]
    c, w = load_plain(folders["C"])
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (5, 37, 60)]
    eng = Engine(folders["C"], dtype="float32", device=DEV, page_size=page, num_pages=64, max_num_seqs=2,
                 max_num_batched_tokens=48, prefill_chunk_cap=24)
    res = eng.generate(prompts, SamplingParams(max_new_tokens=24, temperature=0.0, ignore_eos=True))
    for p, r in zip(prompts, res):
        toks = list(p)
        for _ in range(24):
            lg = pm.forward(c, w, toks)[-1]
            top2 = lg.topk(2).values
            nxt = int(lg.argmax())
            got = r.output_tokens[len(toks) - len(p)]
            if float(top2[0] - top2[1]) > 1e-4:
                assert got == nxt, (len(toks), got, nxt)
            toks.append(got)


def test_command_line_generates_greedily(folders):
    cfg, _, page = MOBUNEX["B"]
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
        lg = pm.forward(c, w, toks)[-1]
        top2 = lg.topk(2).values
        if float(top2[0] - top2[1]) > 1e-4:
            assert got == int(lg.argmax()), (len(toks), got, int(lg.argmax()))
        toks.append(got)
    assert len(line["output_ids"]) == 6


def test_trace_runner_program(folders, tmp_path):
    cfg, _, page = MOBUNEX["A"]
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
