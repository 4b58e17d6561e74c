"""Plain, slow implementation of the Gusorax decoder: the tests' oracle for that design.

Whole sequences, no cache, no paging, one function for each mechanism, elementary torch
arithmetic on the CPU in the dtype it is asked for (float32 or float64).  It shares no code
with the engine: ``config.json`` is a plain dict and the weights a plain ``{name: tensor}``
dict with the checkpoint's own names.

The design in this file's notation (t: position in the sequence, counted from 0):

* e_t = embed[token_t] * s + pos[t]: a scaled token embedding plus a learned position row;
* layers ``loop.start .. loop.stop - 1`` run ``loop.times`` times in a row with the same
  tensors, then the remaining layers; right before the first layer of every such pass
  (the first one too) the residual is replaced by W_in [x ; e] (x first);
* a layer has ONE norm n (RMS, gain 1 + w) and adds both branches computed from it,
  scaled: x <- x + m (mixer(n(x)) + ff(n(x)));
* mixer ``attention``: grouped-query softmax attention, RMS norm per head on queries and
  keys (a gain over the head width, shared by the heads), no rotation, a learned bias per
  head and distance bucket added to the scaled score, a sliding window;
* mixer ``attention_2``: the same skeleton with projection biases, no distance bias, a
  chunked mask (a row sees the earlier rows of its own chunk of the sequence), one added to
  the softmax's denominator, and a sigmoid gate on the concatenated heads;
* feed-forwards: dense silu-gated, and routed experts whose gate is capped from above and
  whose linear part is clamped on both sides, y = g sigmoid(1.702 g) (u + 1); the router's
  weights are the softmax over the chosen logits alone.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

Tensor = torch.Tensor


def rms_unit(x: Tensor, eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x: Tensor, w: Tensor, eps: float) -> Tensor:
    """The layers' norm: its stored weight lies around zero, the gain is 1 + w."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(x: Tensor) -> Tensor:
    return x * torch.sigmoid(x)


# ---------------------------------------------------------------------------- masks and bias
def distance_bucket(n: int, rows: int, far: float) -> int:
    """The row of the bias table for a distance n >= 0: the first half of the rows stands for the
    distances 0 .. rows/2 - 1 one by one, the other rows cut the distances up to ``far`` evenly
    on a logarithmic axis; everything beyond falls into the last row."""
    half = rows // 2
    if n < half:
        return n
    step = math.log(n / half) / math.log(far / half) * (rows - half)
    return min(rows - 1, half + int(math.floor(step)))


def window_mask(T: int, size: int) -> Tensor:
    """[T, T] bool: row i sees column j when 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def chunk_mask(T: int, size: int) -> Tensor:
    """[T, T] bool: row i sees column j <= i of its own chunk, chunks counted from position 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def bias_matrix(rel: Tensor, T: int, far: float) -> Tensor:
    """[H, T, T]: rel[bucket(i - j), h] for j <= i, 0 elsewhere (masked anyway)."""
    rows, H = rel.shape
    by_distance = torch.stack([rel[distance_bucket(n, rows, far)] for n in range(T)])      # [T, H]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    d = (i - j).clamp(min=0)
    return by_distance[d].permute(2, 0, 1)


# ---------------------------------------------------------------------------- the mixers
def head_norm(x: Tensor, gain: Tensor, eps: float) -> Tensor:
    """x [T, heads, dim]: RMS norm over dim with one gain for all heads (plain gain)."""
    return rms_unit(x, eps) * gain


def softmax_attention(q: Tensor, k: Tensor, v: Tensor, mask: Tensor, scale: float, bias: Optional[Tensor],
                      unit_sink: bool) -> Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, E] -> [T, H, E].  Query head h reads key/value head
    h // (H / G).  ``unit_sink``: the denominator gets one more term e^0 that carries no value."""
    T, H, D = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].t()) * scale
        if bias is not None:
            s = s + bias[h]
        s = s.masked_fill(~mask, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        if unit_sink:
            m = m.clamp(min=0.0)
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if unit_sink:
            den = den + torch.exp(-m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def attention_mixer(h: Tensor, w: Dict[str, Tensor], p: str, m: dict, eps: float) -> Tensor:
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].t()).reshape(T, H, D)
    k = (h @ w[p + "k"].t()).reshape(T, G, D)
    v = (h @ w[p + "v"].t()).reshape(T, G, E)
    q = head_norm(q, w[p + "q.norm"], eps)
    k = head_norm(k, w[p + "k.norm"], eps)
    bias = bias_matrix(w[p + "rel"], T, float(m["bias_max"]))
    o = softmax_attention(q, k, v, window_mask(T, m["mask"]["size"]), float(m["scale"]), bias, False)
    return o.reshape(T, H * E) @ w[p + "o"].t()


def attention_2_mixer(h: Tensor, w: Dict[str, Tensor], p: str, m: dict, eps: float) -> Tensor:
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].t() + w[p + "q.b"]).reshape(T, H, D)
    k = (h @ w[p + "k"].t() + w[p + "k.b"]).reshape(T, G, D)
    v = (h @ w[p + "v"].t() + w[p + "v.b"]).reshape(T, G, E)
    q = head_norm(q, w[p + "q.norm"], eps)
    k = head_norm(k, w[p + "k.norm"], eps)
    o = softmax_attention(q, k, v, chunk_mask(T, m["mask"]["size"]), float(m["scale"]), None, True)
    gate = torch.sigmoid(h @ w[p + "g"].t())
    return (o.reshape(T, H * E) * gate) @ w[p + "o"].t() + w[p + "o.b"]


# ---------------------------------------------------------------------------- feed-forwards
def dense_ff(h: Tensor, w: Dict[str, Tensor], p: str) -> Tensor:
    return (silu(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


def capped_expert(h: Tensor, w: Dict[str, Tensor], p: str, limit: float) -> Tensor:
    g = torch.clamp(h @ w[p + "gate"].t(), max=limit)
    u = torch.clamp(h @ w[p + "up"].t(), min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].t()


def route(h: Tensor, w_router: Tensor, top: int):
    """(chosen [T, top], weights [T, top]): the largest logits, softmax over them alone."""
    z = h @ w_router.t()
    best = z.topk(top, dim=-1)
    return best.indices, torch.softmax(best.values, dim=-1)


def routed_ff(h: Tensor, w: Dict[str, Tensor], p: str, mlp: dict) -> Tensor:
    chosen, weights = route(h, w[p + "router"], mlp["router"]["top"])
    limit = float(mlp["expert"]["limit"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            out[t] = out[t] + g * capped_expert(h[t:t + 1], w, f"{p}e{e}.", limit)[0]
    return out


# ---------------------------------------------------------------------------- the model
def run_order(config: dict) -> List[tuple]:
    """(layer, starts a pass) in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, i == 0) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    order += [(i, False) for i in range(b, n)]
    return order


def forward(config: dict, weights: Dict[str, Tensor], tokens, dtype=torch.float64,
            residuals: Optional[List[Tensor]] = None) -> Tensor:
    """Logits [T, vocab] of one whole sequence; ``residuals`` (a list) receives the residual after
    every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    mult = float(config["residual_mult"])
    T = len(tokens)
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(config["embedding"]["scale"]) + w["pos"][:T]
    x = x0
    for i, opens_pass in run_order(config):
        layer = config["layers"][i]
        p = f"l{i}."
        if opens_pass and config.get("loop"):
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].t()
        h = norm_one_plus(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "attention_2":
            y = attention_2_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp))
        x = x + mult * y
        if residuals is not None:
            residuals.append(x.clone())
    x = norm_one_plus(x, w["final.norm"], eps)
    return x @ w["head"].t()
