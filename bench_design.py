#!/usr/bin/env python3
"""A design beside the engine's closest existing model at equal layer sizes (random weights).

    python bench.py --design gebadra|bavetar|gusorax|mobunex [--steps K] [--warmup W] [--sizes 2048,4096]

For each size: prefill (one 2,048-token prompt in one step) and decode (batch 8 from 2,048-token
contexts, the captured decode step) throughput of a few layers of the design and of a Qwen2 model
with the same width, heads, key/value heads, feed-forward width, vocabulary and number of
layers (Mobunex stands beside Bavetar, the engine's closest model: latent attention, a recurrent
layer behind a short convolution, routed experts); and the device time of the design's own kernels in one prompt step and one decode step,
each beside the like kernel of the Qwen2 model, with the fraction of its roofline (the slower of
algorithmic bytes over the measured copy bandwidth and algorithmic FLOPs over the measured bf16
GEMM rate).  Times are CUDA events on the launching stream after warm-up; the per-kernel times
bracket every launch of that kernel in an eager step.  Prints ONE JSON line.
"""
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT = 2048
BATCH = 8
LAYERS = 4


def gebadra_config(width: int) -> dict:
    heads, kv, dim, ff = width // 128, max(1, width // 512), 128, {2048: 5632, 4096: 11008}.get(width, width * 11 // 4)
    decay = [1.0 - 2.0 ** (-5 - 5 * h / max(1, heads - 1)) for h in range(heads)]
    lin = dict(heads=heads, dim=dim, vdim=dim, decay=decay)
    par = dict(left=dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, mask=dict(size=1024, pool=64),
                         rot=dict(base=500000.0, dims=64, scaling=dict(factor=8.0)), scale=dim ** -0.5),
               right=dict(heads=heads, dim=dim // 2, vdim=dim, decay=decay))
    mlp = dict(kind="dense", ff=ff)
    kinds = ["lightning", "parallel", "lightning", "lightning"][:LAYERS]
    layers = [dict(type=k, mixer=lin if k == "lightning" else par, mlp=mlp) for k in kinds]
    return dict(architecture="Gebadra", width=width, vocab=32000, streams=2, norm=dict(eps=1e-6), layers=layers)


def bavetar_config(width: int) -> dict:
    """Four layers at the sizes of a real model of this kind: heads of 128 + 64 rotated, a latent of
    512, state-space heads of 64 with a state of 128, 32 experts of a quarter of the dense width."""
    heads, ff = width // 128, {2048: 5632, 4096: 11008}.get(width, width * 11 // 4)
    lat = dict(heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=width * 3 // 4, scale=192 ** -0.5,
               rot=dict(base=1000000.0, dims=64))
    ssm = dict(heads=width // 32, vdim=64, state=128, groups=8, conv=4, norm_groups=8)
    dense = dict(kind="dense", ff=ff)
    moe = dict(kind="moe", expert=dict(ff=ff // 4), router=dict(experts=32, top=4, scale=2.5, groups=dict(count=4, keep=2)))
    layers = [dict(type="latent_attention", mixer=lat, mlp=dense), dict(type="latent_attention", mixer=lat, mlp=moe),
              dict(type="mamba2", mixer=ssm, mlp=dense), dict(type="latent_attention", mixer=lat, mlp=moe)][:LAYERS]
    return dict(architecture="Bavetar", width=width, vocab=32000, norm=dict(eps=1e-6), logit_scale=1.0,
                logit_softcap=30.0, layers=layers)


def gusorax_config(width: int) -> dict:
    """Four layer runs at the sizes of a real model of this kind: a windowed layer with a dense
    feed-forward that runs twice (the loop), a chunked layer and a windowed layer with 32 experts of a
    quarter of the dense width; heads of 128, an eighth as many key/value heads, a window of 1,024 and
    chunks of 512, a bias table of 32 rows."""
    heads, ff = width // 128, {2048: 5632, 4096: 11008}.get(width, width * 11 // 4)
    kv = max(1, heads // 8)
    win = dict(heads=heads, kv_heads=kv, dim=128, vdim=128, scale=128 ** -0.5, mask=dict(size=1024), bias_max=1024,
               bias_rows=32)
    chunk = dict(heads=heads, kv_heads=kv, dim=128, vdim=128, scale=128 ** -0.5, mask=dict(size=512))
    dense = dict(kind="dense", ff=ff)
    moe = dict(kind="moe", expert=dict(ff=ff // 4, limit=7.0), router=dict(experts=32, top=4))
    layers = [dict(type="attention", mixer=win, mlp=dense), dict(type="attention_2", mixer=chunk, mlp=moe),
              dict(type="attention", mixer=win, mlp=moe)]
    return dict(architecture="Gusorax", width=width, vocab=32000, max_positions=8192, norm=dict(eps=1e-6),
                embedding=dict(scale=float(width) ** 0.5), residual_mult=0.5, loop=dict(start=0, stop=1, times=2),
                layers=layers)


def mobunex_config(width: int) -> dict:
    """Four layers at the sizes of a real model of this kind: latent attention (heads of 128 + 64
    rotated, a latent of 512, YaRN-stretched rotation), windowed attention with an eighth as many
    key/value heads, a gated linear recurrence as wide as the model in blocks of 256 with 4 taps; a
    window of 1,024 everywhere; 32 experts of a quarter of the dense width, 4 chosen from the best 2 of
    4 groups, and a shared expert of the same width."""
    heads, ff = width // 128, {2048: 5632, 4096: 11008}.get(width, width * 11 // 4)
    lat = dict(heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=width * 3 // 4, scale=192 ** -0.5,
               mask=dict(size=1024), rot=dict(base=1000000.0, dims=64,
                                              scaling=dict(factor=8.0, original=4096, fast=32.0, slow=1.0)))
    win = dict(heads=heads, kv_heads=max(1, heads // 8), dim=128, vdim=128, scale=128 ** -0.5, mask=dict(size=1024))
    rec = dict(width=width, blocks=max(1, width // 256), conv=4)
    dense = dict(kind="dense", ff=ff)
    moe = dict(kind="moe", expert=dict(ff=ff // 4), router=dict(experts=32, top=4, groups=dict(count=4, keep=2)),
               shared=dict(ff=ff // 4))
    layers = [dict(type="latent_attention", mixer=lat, mlp=dense), dict(type="attention", mixer=win, mlp=moe),
              dict(type="rglru", mixer=rec, mlp=moe), dict(type="latent_attention", mixer=lat, mlp=moe)][:LAYERS]
    return dict(architecture="Mobunex", width=width, vocab=32000, norm=dict(eps=1e-6), postln_alpha=1.5, layers=layers)


def qwen_config(width: int, design: str = "gebadra") -> dict:
    if design == "gusorax":
        g = gusorax_config(width)
        heads, kv, ff = g["layers"][0]["mixer"]["heads"], g["layers"][0]["mixer"]["kv_heads"], g["layers"][0]["mlp"]["ff"]
    elif design == "bavetar":       # as many query heads; the usual eight times fewer key/value heads
        heads, kv, ff = width // 128, max(1, width // 1024), bavetar_config(width)["layers"][0]["mlp"]["ff"]
    else:
        g = gebadra_config(width)
        heads, kv, ff = g["layers"][0]["mixer"]["heads"], g["layers"][1]["mixer"]["left"]["kv_heads"], \
            g["layers"][0]["mlp"]["ff"]
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=width, num_hidden_layers=LAYERS,
                num_attention_heads=heads, num_key_value_heads=kv, head_dim=128,
                intermediate_size=ff, vocab_size=32000, rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=False, max_position_embeddings=32768, use_sliding_window=False, hidden_act="silu",
                eos_token_id=31999)


class OpTimer:
    """Brackets every call of the named functions of ``ops`` with CUDA events."""

    def __init__(self, names):
        from paged_batch_engine_b200.csrc import ops
        self.ops, self.names, self.saved, self.events = ops, names, {}, []
        self.spin = 800000          # cycles (about 0.4 ms) the device spins before every bracket

    def __enter__(self):
        import torch
        for n in self.names:
            fn = getattr(self.ops, n)
            self.saved[n] = fn

            def timed(*a, _fn=fn, _n=n, **kw):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                # the device idles ahead of the bracket while the host enqueues what is inside it, so
                # that the bracket holds device time and not the interpreter's
                torch.cuda._sleep(self.spin)
                s.record()
                out = _fn(*a, **kw)
                e.record()
                self.events.append((_n, s, e))
                return out
            setattr(self.ops, n, timed)
        return self

    def __exit__(self, *exc):
        for n, fn in self.saved.items():
            setattr(self.ops, n, fn)

    def totals(self):
        import torch
        torch.cuda.synchronize()
        out = {}
        for n, s, e in self.events:
            ms, calls = out.get(n, (0.0, 0))
            out[n] = (ms + s.elapsed_time(e), calls + 1)
        return out


def _prefill(runner, tokens, want_ops=None):
    import torch
    from paged_batch_engine_b200.engine.batch import StepEntry
    cache = runner.cache
    g = torch.Generator().manual_seed(5)
    vocab = runner.model.spec.vocab_size
    times, per_op = [], None
    for i in range(5):
        prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()
        h = cache.add_request()
        assert cache.reserve(h, tokens)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if want_ops and i == 4:
            with OpTimer(want_ops) as t:
                runner.step([StepEntry(h, prompt, [tokens - 1])])
                per_op = t.totals()
        else:
            start.record()
            runner.step([StepEntry(h, prompt, [tokens - 1])])
            stop.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(start.elapsed_time(stop))
        cache.free(h)
    times.sort()
    return times[len(times) // 2], per_op


def _decode(runner, batch, context, steps, warmup, want_ops=None):
    import torch
    from paged_batch_engine_b200.csrc import ops
    from paged_batch_engine_b200.engine.batch import StepEntry
    cache = runner.cache
    g = torch.Generator().manual_seed(6)
    vocab = runner.model.spec.vocab_size
    handles = []
    for _ in range(batch):
        h = cache.add_request()
        assert cache.reserve(h, context)
        runner.step([StepEntry(h, torch.randint(0, vocab, (context,), generator=g).tolist(), [])])
        handles.append(h)
    feed = torch.randint(0, vocab, (steps + warmup + 1, batch), generator=g).tolist()
    out_ids = torch.empty(batch, dtype=torch.int32, device=runner.device)

    def one(i, graph=True):
        entries = [StepEntry(h, [feed[i][j]], [0]) for j, h in enumerate(handles)]
        for e in entries:
            assert cache.reserve(e.handle, 1)
        ops.argmax(runner.step(entries, decode_graph=graph), out_ids)
    for i in range(warmup):
        one(i)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    per_op = None
    if want_ops:
        with OpTimer(want_ops) as t:
            one(warmup + steps, graph=False)
            per_op = t.totals()
    captured = runner.graphs is not None and runner.graphs.replays > 0
    for h in handles:
        cache.free(h)
    return ms, per_op, captured


def rooflines_bavetar(width: int, pk: dict):
    """Algorithmic bytes and FLOPs of the compared kernels for the two workloads, per launch."""
    b = bavetar_config(width)
    lat, ssm = b["layers"][0]["mixer"], b["layers"][2]["mixer"]
    H, D, Rr, V, rank, qr = lat["heads"], lat["dim"], lat["rot_dim"], lat["vdim"], lat["kv_rank"], lat["q_rank"]
    dk = rank + Rr
    SH, P, N, G = ssm["heads"], ssm["vdim"], ssm["state"], ssm["groups"]
    chan = SH * P + 2 * G * N
    ff = b["layers"][0]["mlp"]["ff"]
    r = b["layers"][1]["mlp"]
    E, top, eff = r["router"]["experts"], r["router"]["top"], r["expert"]["ff"]
    q = qwen_config(width, "bavetar")
    QH, QG = q["num_attention_heads"], q["num_key_value_heads"]
    T, R, C = PROMPT, BATCH, PROMPT

    def t_us(by, fl):
        return max(by / (pk["hbm_gbs"] * 1e9), fl / (pk["bf16_tflops"] * 1e12)) * 1e6

    def both(rows, keys_total, keys_read):
        return {
            # queries (float32) in, cached rows read once, float32 latent-space outputs; scores over dk and
            # weighted sums over rank for every (row, head, visible key)
            "latent_attention": t_us(4 * rows * H * dk + 2 * keys_read * dk + 4 * rows * H * rank,
                                     2 * H * (dk + rank) * keys_total),
            "head_product": t_us(2 * rows * H * (D + Rr) + 2 * H * D * rank + 4 * rows * H * dk, 2 * rows * H * D * rank),
            "latent_prepare": t_us(2 * rows * (qr + dk) * 2, 0),
            "add2_rmsnorm2": t_us(rows * width * (2 * 4 + 2 * 2 + 2 * 2), 0),
            "linear_attention": t_us(2 * rows * chan + 4 * rows * SH * (P + 2) + 8 * (R if rows == R else 1) * SH * N * P,
                                     4 * rows * SH * N * P),
            "short_conv": t_us(2 * rows * chan * 2, 0),
            "gated_rms": t_us(rows * SH * P * (4 + 2 + 2), 0),
            "relu_squared": t_us(rows * ff * 4, 0),
            "expert_rows": t_us(2 * min(E, rows * top) * 3 * eff * width, 6 * rows * top * eff * width),
            "route": t_us(rows * E * 4, 0),
            "paged_attention": t_us(2 * (2 * rows * QH * 128) + 2 * keys_read * QG * 2 * 128, 4 * QH * 128 * keys_total),
            "attention_decode_fused": t_us(2 * keys_read * QG * 2 * 128, 4 * QH * 128 * keys_total),
            "add_rmsnorm": t_us(rows * width * (2 * 4 + 2 + 2), 0),
            "rope_kv_write": t_us(2 * rows * (QH + 2 * QG) * 128 * 2, 0),
            "silu_mul": t_us(rows * ff * 6, 0),
        }
    return {"prefill": both(T, T * (T + 1) // 2, T), "decode": both(R, R * (C + 1), R * (C + 1))}


def rooflines_gusorax(width: int, pk: dict):
    """Algorithmic bytes and FLOPs of the compared kernels for the two workloads, per launch (the
    attention's figures are those of the windowed layer, the wider of the two masks)."""
    g = gusorax_config(width)
    m = g["layers"][0]["mixer"]
    H, G, D, E, W = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"]
    ff = g["layers"][0]["mlp"]["ff"]
    r = g["layers"][1]["mlp"]
    NE, top, eff = r["router"]["experts"], r["router"]["top"], r["expert"]["ff"]
    T, R, C = PROMPT, BATCH, PROMPT

    def t_us(by, fl):
        return max(by / (pk["hbm_gbs"] * 1e9), fl / (pk["bf16_tflops"] * 1e12)) * 1e6

    def both(rows, keys_total, keys_read, qwen_total, qwen_read):
        proj = (H * D + G * (D + E)) * 2
        return {
            # queries in, the visible keys and values read once, outputs; a score over D and a weighted sum over E
            # for every (row, head, visible key)
            "masked_attention": t_us(2 * rows * H * D + 2 * keys_read * G * (D + E) + 2 * rows * H * E,
                                     2 * H * (D + E) * keys_total),
            "head_norm_write": t_us(rows * proj + 2 * rows * H * D + 2 * rows * G * (D + E), 0),
            "add2_rmsnorm2": t_us(rows * width * (2 * 4 + 2 * 2 + 2), 0),
            "fold_pair": t_us(rows * width * (2 * 4 + 2 * 2 + 2 * 2), 0),
            "embedding_positions": t_us(rows * width * (2 + 2 + 4), 0),
            "gated_activation": t_us(rows * ff * 6, 0),
            "expert_rows": t_us(2 * min(NE, rows * top) * 3 * eff * width, 6 * rows * top * eff * width),
            "route": t_us(rows * NE * 4, 0),
            "paged_attention": t_us(2 * (2 * rows * H * 128) + 2 * qwen_read * G * 2 * 128, 4 * H * 128 * qwen_total),
            "attention_decode_fused": t_us(2 * qwen_read * G * 2 * 128, 4 * H * 128 * qwen_total),
            "add_rmsnorm": t_us(rows * width * (2 * 4 + 2 + 2), 0),
            "rope_kv_write": t_us(2 * rows * (H + 2 * G) * 128 * 2, 0),
            "silu_mul": t_us(rows * ff * 6, 0),
        }
    keys_prefill = sum(min(t + 1, W) for t in range(T))
    return {"prefill": both(T, keys_prefill, T, T * (T + 1) // 2, T),
            "decode": both(R, R * min(C + 1, W), R * min(C + 1, W), R * (C + 1), R * (C + 1))}


def rooflines_mobunex(width: int, pk: dict):
    """Algorithmic bytes and FLOPs of the compared kernels for the two workloads, per launch; Bavetar's
    kernels (the model beside it) come from ``rooflines_bavetar``.  ``unit_norm`` is the mean over a
    step's launches: a norm between the sublayers moves 12 bytes an element, a layer's last norm also
    reads every earlier layer's result for the mix over depth and writes the mix."""
    m = mobunex_config(width)
    lat, win, rec = m["layers"][0]["mixer"], m["layers"][1]["mixer"], m["layers"][2]["mixer"]
    H, D, Rr, rank = lat["heads"], lat["dim"], lat["rot_dim"], lat["kv_rank"]
    dk = rank + Rr
    WH, WG, WD, WE, Wn = win["heads"], win["kv_heads"], win["dim"], win["vdim"], win["mask"]["size"]
    C, n = rec["width"], rec["width"] // rec["blocks"]
    ff = m["layers"][0]["mlp"]["ff"]
    r = m["layers"][1]["mlp"]
    E, top, eff = r["router"]["experts"], r["router"]["top"], r["expert"]["ff"]
    T, R, Cx = PROMPT, BATCH, PROMPT
    base = rooflines_bavetar(width, pk)

    def t_us(by, fl):
        return max(by / (pk["hbm_gbs"] * 1e9), fl / (pk["bf16_tflops"] * 1e12)) * 1e6

    def both(rows, keys_total, keys_read, requests):
        norm_bytes, launches = 0, 0
        for i, layer in enumerate(m["layers"]):
            if layer["mlp"] is not None:
                norm_bytes += rows * width * (4 + 2 + 4 + 2)
                launches += 1
            norm_bytes += rows * width * (4 + 2 + 4 + 4 * (i + 1) + 4 + 2)
            launches += 1
        norm_bytes += R * width * (4 + 2) if rows == R else width * (4 + 2)      # the final norm's few rows
        launches += 1
        proj = (WH * WD + WG * (WD + WE)) * 2
        return {
            "unit_norm": t_us(norm_bytes / launches, 0),
            "embedding_unit_norm": t_us(rows * width * (2 + 4 + 2), 0),
            # the gates: two block-diagonal products in 32-bit arithmetic, and the coefficients out
            "recurrence_gates": t_us(2 * rows * C + 2 * 2 * C * n + 8 * rows * C, 4 * rows * C * n),
            # the gates' float32 pre-activations (two a channel), the input and the branch in, the product out
            "gated_scan": t_us(rows * C * (8 + 2 + 2 + 2) + 8 * requests * C, 0),
            "short_conv": t_us(2 * rows * C * 2, 0),
            "masked_attention": t_us(2 * rows * WH * WD + 2 * keys_read * WG * (WD + WE) + 2 * rows * WH * WE,
                                     2 * WH * (WD + WE) * keys_total),
            "head_norm_write": t_us(rows * proj + 2 * rows * WH * WD + 2 * rows * WG * (WD + WE), 0),
            "latent_attention": t_us(4 * rows * H * dk + 2 * keys_read * dk + 4 * rows * H * rank,
                                     2 * H * (dk + rank) * keys_total),
            "latent_prepare": base["prefill" if rows == T else "decode"]["latent_prepare"],
            "silu_mul": t_us(rows * ff * 6, 0),
            "expert_rows": t_us(2 * min(E, rows * top) * 3 * eff * width, 6 * rows * top * eff * width),
            "route": t_us(rows * E * 4, 0),
        }
    keys_prefill = sum(min(t + 1, Wn) for t in range(T))
    out = {"prefill": both(T, keys_prefill, T, 1), "decode": both(R, R * min(Cx + 1, Wn), R * min(Cx + 1, Wn), R)}
    for phase in out:
        for k, v in base[phase].items():
            out[phase].setdefault(k, v)
    return out


def rooflines(width: int, pk: dict):
    """Algorithmic bytes and FLOPs of the compared kernels for the two workloads, per launch."""
    g = gebadra_config(width)
    lin, left = g["layers"][0]["mixer"], g["layers"][1]["mixer"]["left"]
    H, D, E = lin["heads"], lin["dim"], lin["vdim"]
    G, W, P = left["kv_heads"], left["mask"]["size"], left["mask"]["pool"]
    T, R, C = PROMPT, BATCH, PROMPT
    keys_prefill = sum(min(t + 1, W) + max(0, (t - W + 1) // P) for t in range(T))
    keys_decode = min(C + 1, W) + max(0, (C - W + 1) // P)

    def t_us(b, f):
        return max(b / (pk["hbm_gbs"] * 1e9), f / (pk["bf16_tflops"] * 1e12)) * 1e6
    return {
        "prefill": {
            "linear_attention": t_us(2 * T * H * (2 * D + E) + 4 * T * H * E + 8 * H * D * E, 4 * T * H * D * E),
            "pooled_attention": t_us(2 * (T * H * (D + E) + T * G * (D + E) * (1 + 1 / P)), 2 * H * (D + E) * keys_prefill),
            "stream_norm": t_us(T * width * (2 * 4 * 2 + 2 + 2), 0),
            "paged_attention": t_us(2 * (2 * T * H * 128 + 2 * T * G * 128), 4 * H * 128 * T * (T + 1) / 2),
            "add_rmsnorm": t_us(T * width * (2 * 4 + 2 + 2), 0),
        },
        "decode": {
            "linear_attention": t_us(2 * R * H * (2 * D + E) + 4 * R * H * E + 8 * R * H * D * E, 4 * R * H * D * E),
            "pooled_attention": t_us(2 * R * keys_decode * G * (D + E), 2 * R * H * (D + E) * keys_decode),
            "stream_norm": t_us(R * width * (2 * 4 * 2 + 2 + 2), 0),
            "attention_decode_fused": t_us(2 * R * C * G * 2 * 128, 4 * R * H * 128 * C),
            "paged_attention": t_us(2 * R * C * G * 2 * 128, 4 * R * H * 128 * C),
            "add_rmsnorm": t_us(R * width * (2 * 4 + 2 + 2), 0),
        },
    }


def run(design: str, steps: int, warmup: int, sizes=(2048, 4096)) -> dict:
    import gc
    import torch
    from bench import ClockSampler, peaks
    from paged_batch_engine_b200.config import load_config
    from paged_batch_engine_b200.engine.runner import ModelRunner
    if design not in ("gebadra", "bavetar", "gusorax", "mobunex"):
        raise SystemExit(f"unknown design {design!r}; known: gebadra, bavetar, gusorax, mobunex")
    os.environ["PBE_EXEC"] = "python"        # per-kernel times need every launch to come through ops
    pk = peaks()
    page = 16
    pool = BATCH * (PROMPT + steps + warmup + 64) + PROMPT + 64
    own = ["linear_attention", "pooled_attention", "stream_norm", "gated_rms", "qk_prepare", "pool_blocks",
           "branch_rms_mean"]
    theirs = ["paged_attention", "attention_decode_fused", "add_rmsnorm", "rope_kv_write"]
    if design == "bavetar":
        own = ["latent_attention", "head_product", "latent_prepare", "add2_rmsnorm2", "linear_attention", "short_conv",
               "step_sizes", "gated_rms", "relu_squared", "route", "expert_rows", "expert_places", "expert_gather",
               "expert_scatter", "grouped_heads", "grouped_runs", "run_tiles"]
        theirs = theirs + ["silu_mul"]
    if design == "gusorax":
        own = ["masked_attention", "head_norm_write", "add2_rmsnorm2", "fold_pair", "embedding_positions",
               "gated_activation", "silu_mul", "route", "expert_rows", "expert_places", "expert_gather", "expert_scatter",
               "grouped_runs", "run_tiles"]
        theirs = theirs + ["silu_mul"]
    bavetar_ops = ["latent_attention", "head_product", "latent_prepare", "add2_rmsnorm2", "linear_attention",
                   "short_conv", "step_sizes", "gated_rms", "relu_squared", "route", "expert_rows", "expert_places",
                   "expert_gather", "expert_scatter", "grouped_heads", "grouped_runs", "run_tiles"]
    beside, beside_config = "qwen2", lambda width: qwen_config(width, design)
    if design == "mobunex":
        own = ["unit_norm", "embedding_unit_norm", "recurrence_gates", "gated_scan", "short_conv", "masked_attention",
               "head_norm_write", "latent_attention", "latent_prepare", "grouped_heads", "silu_mul", "route",
               "expert_rows", "expert_places", "expert_gather", "expert_scatter", "grouped_runs", "run_tiles"]
        theirs = bavetar_ops
        beside, beside_config = "bavetar", bavetar_config
    design_config = {"bavetar": bavetar_config, "gusorax": gusorax_config, "mobunex": mobunex_config}.get(
        design, gebadra_config)
    roofs = {"bavetar": rooflines_bavetar, "gusorax": rooflines_gusorax, "mobunex": rooflines_mobunex}.get(
        design, rooflines)
    sampler = ClockSampler(0)
    sampler.active = True
    out = {}
    for width in sizes:
        roof = roofs(width, pk)
        row = {}
        for name, cfg, names in ((design, design_config(width), own), (beside, beside_config(width), theirs)):
            _, typed = load_config(cfg)
            runner = ModelRunner.from_random(typed, seed=0, dtype="bfloat16", page_tokens=page, max_cache_tokens=pool,
                                             max_requests=BATCH + 1)
            ms_p, ops_p = _prefill(runner, PROMPT, names)
            ms_d, ops_d, captured = _decode(runner, BATCH, PROMPT, steps, warmup, names)
            kernels = {}
            for phase, per_op in (("prefill", ops_p), ("decode", ops_d)):
                for op, (ms, calls) in sorted((per_op or {}).items()):
                    us = ms * 1e3 / calls
                    entry = {"us": round(us, 1), "calls": calls}
                    if op in roof[phase]:
                        entry["roofline_us"] = round(roof[phase][op], 2)
                        entry["frac"] = round(roof[phase][op] / us, 4)
                    kernels[f"{phase}.{op}"] = entry
            row[name] = {"prefill_tok_s": round(PROMPT * 1e3 / ms_p, 1), "prefill_ms": round(ms_p, 3),
                         "decode_tok_s": round(BATCH * 1e3 / ms_d, 1), "decode_ms_per_step": round(ms_d, 4),
                         "decode_captured": bool(captured), "kernels": kernels}
            del runner
            gc.collect()
            torch.cuda.empty_cache()
        out[str(width)] = row
    sampler.active = False
    return {"design": design,
            "beside": f"{beside} at equal width, heads, feed-forward, vocabulary and layers"
            + (", key/value heads" if beside == "qwen2" else ""),
            "layers": LAYERS, "prompt_tokens": PROMPT, "decode_batch": BATCH, "decode_context": PROMPT,
            "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic (random weights)",
            "peaks": {"source": pk["source"], "hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"]},
            "sizes": out, "clocks": sampler.summary()}


if __name__ == "__main__":
    print(json.dumps(run("gebadra", 32, 5)))
