"""Plain, slow implementation of the Mobunex decoder: the tests' oracle for that design.

Whole sequences, no cache, no paging, one function for each mechanism, elementary torch
arithmetic on the CPU in the dtype of the tensors it is given (float32 or float64).  It
shares no code with the engine: ``config.json`` is a plain dict and the weights a plain
``{name: tensor}`` dict with the checkpoint's own names.

The design in this file's notation (t: position in the sequence, counted from 0; n(.) divides
a row by sqrt(mean of squares + eps)):

* X_0 = g_e n(embed[token]); a norm here has ONE learned number g for all coordinates;
* a layer normalises after each sum, and its sublayers read the stream itself:
  x <- g_1 n(alpha x + mixer(x)), then x <- g_2 n(alpha x + ff(x)); its result is X_(i+1);
* what the next layer (or the head) reads is a learned mix over depth, sum_j d_i[j] X_j for
  j = 0 .. i+1;
* three mixers: ``attention`` (grouped-query softmax attention in a sliding window, biases on
  q, k, v, unit-RMS queries and keys, a learned temperature per head, no rotation), ``rglru``
  (a gated diagonal linear recurrence behind a short causal convolution, times a gelu branch)
  and ``latent_attention`` (keys and values expanded from one latent per token plus a rotated
  key part shared by the heads, YaRN-scaled rotation, sliding window, a sigmoid gate on every
  output coordinate);
* two feed-forwards: dense silu-gated, and routed experts (sigmoid scores, a correction added
  for the choice only, groups ranked by the sum of their two best, weights normalised over
  the chosen) plus a shared expert;
* logits = head (g_f n(x)).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

Tensor = torch.Tensor


def rms_unit(x: Tensor, eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x: Tensor) -> Tensor:
    return x * torch.sigmoid(x)


def gelu_tanh(z: Tensor) -> Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z * z * z)))


def softplus(x: Tensor) -> Tensor:
    """log(1 + exp(x)), written so that large x does not overflow."""
    return torch.where(x > 20, x, torch.log1p(torch.exp(torch.clamp(x, max=20))))


def window_mask(positions: Tensor, size: Optional[int]) -> Tensor:
    """[T, T] bool: row i sees column j when 0 <= p_i - p_j < size (no size: every earlier j)."""
    d = positions[:, None] - positions[None, :]
    return (d >= 0) & (d < size) if size else (d >= 0)


def mask_size(m: dict) -> Optional[int]:
    return int(m["mask"]["size"]) if m.get("mask") else None


def masked_softmax(scores: Tensor, mask: Tensor) -> Tensor:
    """Softmax over the last axis among the entries the mask allows; scores [H, T, T]."""
    s = scores.masked_fill(~mask[None], float("-inf"))
    e = torch.exp(s - s.max(dim=-1, keepdim=True).values)
    return e / e.sum(dim=-1, keepdim=True)


# ---------------------------------------------------------------------------- depth
def depth_mix(history: List[Tensor], d: Tensor) -> Tensor:
    """sum_j d[j] X_j over everything computed so far (the embedding output first)."""
    assert d.numel() == len(history)
    out = torch.zeros_like(history[0])
    for j, X in enumerate(history):
        out = out + d[j] * X
    return out


def post_norm(x: Tensor, y: Tensor, alpha: float, g: Tensor, eps: float) -> Tensor:
    """g n(alpha x + y), g one number."""
    return rms_unit(alpha * x + y, eps) * g


# ---------------------------------------------------------------------------- attention
def window_attention_mixer(h: Tensor, w: Dict[str, Tensor], p: str, m: dict, eps: float,
                           positions: Optional[Tensor] = None) -> Tensor:
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    T = h.shape[0]
    positions = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].t() + w[p + "q.b"]).reshape(T, H, D)
    k = (h @ w[p + "k"].t() + w[p + "k.b"]).reshape(T, G, D)
    v = (h @ w[p + "v"].t() + w[p + "v.b"]).reshape(T, G, V)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    per = H // G
    k = k.repeat_interleave(per, dim=1)          # head h reads key/value head h // per
    v = v.repeat_interleave(per, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"] * w[p + "temp"][:, None, None]
    wts = masked_softmax(scores, window_mask(positions, mask_size(m)))
    out = torch.einsum("hij,jhv->ihv", wts, v).reshape(T, H * V)
    return out @ w[p + "o"].t()


# ---------------------------------------------------------------------------- gated linear recurrence
def causal_conv(u: Tensor, w: Tensor, b: Tensor) -> Tensor:
    """y[t, c] = b[c] + sum_j w[c, j] u[t - (taps - 1) + j, c], inputs before the start are zero;
    u [T, C], w [C, taps]: the last column multiplies the current token."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = b.expand(T, C).clone()
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


def block_gates(u: Tensor, mat: Tensor, bias: Tensor) -> Tensor:
    """sigmoid(M_b u_b + c_b) for each of the B equal parts u_b of the last axis; mat [B, n, n]
    ([out, in]), bias [B, n]."""
    T, C = u.shape
    B, n = mat.shape[0], mat.shape[1]
    ub = u.reshape(T, B, n)
    z = torch.einsum("tbi,boi->tbo", ub, mat) + bias
    return torch.sigmoid(z).reshape(T, C)


def gated_recurrence(u: Tensor, r: Tensor, i: Tensor, lam: Tensor) -> Tensor:
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0, with a_t = exp(-8 r_t softplus(lam));
    returns every S_t, [T, C]."""
    T, C = u.shape
    log_a = -8.0 * r * softplus(lam)
    a = torch.exp(log_a)
    b = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(C, dtype=u.dtype)
    out = torch.zeros_like(u)
    for t in range(T):
        S = a[t] * S + b[t]
        out[t] = S
    return out


def rglru_mixer(h: Tensor, w: Dict[str, Tensor], p: str, m: dict) -> Tensor:
    y = gelu_tanh(h @ w[p + "y"].t() + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].t() + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    r = block_gates(u, w[p + "ra"], w[p + "ra.b"])
    i = block_gates(u, w[p + "ri"], w[p + "ri.b"])
    S = gated_recurrence(u, r, i, w[p + "lam"])
    return (S * y) @ w[p + "o"].t()


# ---------------------------------------------------------------------------- latent attention
def yarn_frequencies(rot: dict, dtype=torch.float64):
    """(frequency of every pair [dims/2], the factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turns_to_dim(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turns_to_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turns_to_dim(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: Tensor, positions: Tensor, freq: Tensor, magnitude: float) -> Tensor:
    """Neighbouring pairs (2i, 2i+1) of the first 2 * len(freq) dimensions of the last axis turn by
    p * freq_i, cos and sin both times ``magnitude``; the other dimensions pass.  x [T, ..., d]."""
    dims = 2 * freq.numel()
    out = x.clone()
    ang = positions.to(x.dtype)[:, None] * freq.to(x.dtype)[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = (torch.cos(ang) * magnitude).reshape(shape), (torch.sin(ang) * magnitude).reshape(shape)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_attention_mixer(h: Tensor, w: Dict[str, Tensor], p: str, m: dict, eps: float,
                           positions: Optional[Tensor] = None) -> Tensor:
    H, D, R, V, kv = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    positions = torch.arange(T) if positions is None else positions
    freq, mag = yarn_frequencies(m["rot"], h.dtype)
    cq = rms_unit(h @ w[p + "dq"].t(), eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].t()).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], positions, freq, mag)
    ckr = h @ w[p + "dkv"].t()
    c = rms_unit(ckr[:, :kv], eps) * w[p + "dkv.norm"]
    k_rot = rotate_pairs(ckr[:, kv:], positions, freq, mag)                  # [T, R], one for all heads
    k_plain = (c @ w[p + "uk"].t()).reshape(T, H, D)
    v = (c @ w[p + "uv"].t()).reshape(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    wts = masked_softmax(scores, window_mask(positions, mask_size(m)))
    out = torch.einsum("hij,jhv->ihv", wts, v).reshape(T, H * V)
    out = out * torch.sigmoid(h @ w[p + "g"].t())                            # a gate per output coordinate
    return out @ w[p + "o"].t()


# ---------------------------------------------------------------------------- feed-forwards
def gated_ff(h: Tensor, w: Dict[str, Tensor], p: str) -> Tensor:
    return (silu(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


def route(h: Tensor, w_router: Tensor, correction: Tensor, r: dict):
    """(chosen experts [T, top], their weights [T, top]).  s = sigmoid(router logits); the choice
    is made on s + correction: a group's rank is the sum of its two largest such values, experts
    outside the ``keep`` best groups cannot be chosen, the ``top`` largest of the rest are; the
    weights are the chosen s (without the correction) over their sum."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w_router.t())
    choice = s + correction
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        rank = choice.reshape(-1, n, per).topk(min(2, per), dim=-1).values.sum(dim=-1)
        kept = rank.topk(keep, dim=-1).indices
        gmask = torch.zeros_like(rank, dtype=torch.bool).scatter_(1, kept, True)
        allowed = gmask[:, :, None].expand(-1, n, per).reshape(-1, E)
        choice = choice.masked_fill(~allowed, float("-inf"))
    picked = choice.topk(top, dim=-1).indices
    chosen = s.gather(1, picked)
    return picked, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20)


def routed_ff(h: Tensor, w: Dict[str, Tensor], p: str, mlp: dict) -> Tensor:
    picked, weights = route(h, w[p + "router"], w[p + "correction"], mlp["router"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(picked[t].tolist(), weights[t]):
            out[t] = out[t] + g * gated_ff(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_ff(h, w, p + "shared.")
    return out


# ---------------------------------------------------------------------------- the model
def forward(config: dict, weights: Dict[str, Tensor], tokens, dtype=torch.float64,
            residuals: Optional[List[Tensor]] = None) -> Tensor:
    """Logits [T, vocab] of one whole sequence; ``residuals`` (a list) receives what every layer
    hands on (after the mix over depth)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, alpha = float(config["norm"]["eps"]), float(config["postln_alpha"])
    x = rms_unit(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], eps) * w["embed.norm"]
    history = [x]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            y = window_attention_mixer(x, w, p + "mix.", m, eps)
        elif kind == "rglru":
            y = rglru_mixer(x, w, p + "mix.", m)
        elif kind == "latent_attention":
            y = latent_attention_mixer(x, w, p + "mix.", m, eps)
        else:
            raise ValueError(kind)
        x = post_norm(x, y, alpha, w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            f = gated_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(x, w, p + "mlp.", mlp)
            x = post_norm(x, f, alpha, w[p + "norm2"], eps)
        history.append(x)
        x = depth_mix(history, w[p + "dwa"])
        if residuals is not None:
            residuals.append(x.clone())
    x = rms_unit(x, eps) * w["final.norm"]
    return x @ w["head"].t()
