"""Softmax attention whose keys and values are expanded from one small latent per token."""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import CacheTensor, Mixer, PagedNeed, register_part


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict] = None):
    """(the turn per position of every rotated pair, float64 [dims / 2]; the factor on cos and sin).
    Pair i turns by f_i = base^(-2i / dims).  ``scaling`` = dict(factor, original, fast, slow): with
    dim(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(dim(fast)), 0) and hi =
    min(ceil(dim(slow)), dims - 1), the ramp r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) takes
    pair i from f_i (r = 0) to f_i / factor (r = 1); cos and sin are multiplied by 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if not factor >= 1.0 or not original > 0:
        raise ValueError("rotary scaling: factor >= 1 and original > 0")

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class LatentAttention(Mixer):
    """Per token the cache holds c (``kv_rank`` values, RMS-normed) and kr (``rot_dim`` values,
    rotated): head h's key is [U_k,h c | kr] and its value U_v,h c.  The query goes through a latent
    of its own, c_q = RMSnorm(W_dq x), q = W_uq c_q, per head [``head_dim`` plain | ``rot_dim``
    rotated].  Score = (q_plain . U_k,h c + rope(q_rot) . kr) * ``scale``; causal softmax, with
    (``sink``) a learned logit per head in the denominator that has no key and no value; head h's
    output is multiplied (``out_gate``) by sigmoid(W_g x)_h (``out_gate`` "each": W_g is [H*V, hidden]
    and every output value has a gate of its own); then the output projection.

    Keys and values are never expanded here: U_k,h^T is applied to q_plain (the score becomes a
    product with c) and U_v,h to the attention's output over c, so attention reads the cached rows
    alone.  Rotation: pairs (2i, 2i + 1) of the first ``rotary["dims"]`` values of the rotated
    part turn by position * base^(-2i / dims).  ``rotary["scaling"]`` = dict(factor, original, fast,
    slow) stretches the slow pairs (``yarn_frequencies``) and multiplies cos and sin by 0.1 ln(factor)
    + 1; ``scale`` is used as given.

    Checkpoint tensors under the prefix: dq [q_rank, hidden], dq.norm [q_rank], uq [H*(D+R),
    q_rank], dkv [kv_rank + R, hidden], dkv.norm [kv_rank], uk [H*D, kv_rank], uv [H*V, kv_rank],
    sink [H], g [H, hidden], o [hidden, H*V] (``tensor_names`` renames them)."""
    TENSOR_NAMES = dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv",
                        sink="sink", g="g", o="o")
    decode_capturable = True      # stepped from the step's device arrays alone
    # steps of at most this many rows keep the per-head products in float32 FMAs (0: bfloat16 runs
    # always take the tensor-core products: 0.88 -> 0.82 ms for a decode step of 8 rows)
    FEW_ROWS = int(os.environ.get("PBE_LATENT_FEW_ROWS", "0"))

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 q_rank: int, scale: float, eps: float, dtype, device, rotary: Optional[dict] = None,
                 sink: bool = True, out_gate: bool = True, window: Optional[int] = None,
                 tensor_names: Optional[dict] = None):
        unknown = set(tensor_names or {}) - set(self.TENSOR_NAMES)
        if unknown:
            raise ValueError(f"tensor_names knows {sorted(self.TENSOR_NAMES)}; got {sorted(unknown)}")
        if rot_dim % 2:
            raise ValueError("the rotated part is even")
        if kv_rank > 512:
            raise ValueError("kv_rank is at most 512")
        self.names = dict(self.TENSOR_NAMES, **(tensor_names or {}))
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = hidden_size, num_heads, head_dim, rot_dim
        self.value_dim, self.kv_rank, self.q_rank = value_dim, kv_rank, q_rank
        self.scale, self.eps, self.sink, self.out_gate = float(scale), float(eps), bool(sink), out_gate
        self.window = int(window) if window else None
        self.dtype, self.device = dtype, device
        self.rot_dims, self.inv_freq, self.rot_scale = 0, None, 1.0
        if out_gate not in (True, False, "each"):
            raise ValueError('out_gate is True (a gate per head), "each" (per output value) or False')
        if rotary is not None and rot_dim:
            dims, base = int(rotary["dims"]), float(rotary["base"])
            if dims % 2 or not 0 < dims <= rot_dim:
                raise ValueError(f"rotary dims must be even and in (0, rot_dim], got {dims}")
            freq, self.rot_scale = yarn_frequencies(dims, base, rotary.get("scaling"))
            self.inv_freq = freq.to(torch.float32).to(device)
            self.rot_dims = dims
        self.tile_rows = ops.latent_tile_rows(num_heads)
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = None
        self.q_gain = self.c_gain = self.sink_logits = None

    # ---- what it keeps: one row [c | kr] per token, shared by all heads
    def cache_need(self):
        return PagedNeed((CacheTensor("latent", 1, self.kv_rank + self.rot_dim),), window=self.window)

    def work_keys(self):
        return [(self.num_heads, self.tile_rows, self.window)]

    def kernel_libraries(self, dtype):
        tiled = [("grouped_gemm", None)] if dtype == torch.bfloat16 else []
        return [("latent_attention", None)] + tiled + ops.gemm_libraries(dtype)

    # ---- tensors
    def param_specs(self, prefix):
        n, w = self.names, self.hidden_size
        H, D, R, V = self.num_heads, self.head_dim, self.rot_dim, self.value_dim
        specs = [ParamSpec(prefix + n["dq"], (self.q_rank, w)), ParamSpec(prefix + n["dq_norm"], (self.q_rank,)),
                 ParamSpec(prefix + n["uq"], (H * (D + R), self.q_rank)),
                 ParamSpec(prefix + n["dkv"], (self.kv_rank + R, w)), ParamSpec(prefix + n["dkv_norm"], (self.kv_rank,)),
                 ParamSpec(prefix + n["uk"], (H * D, self.kv_rank)), ParamSpec(prefix + n["uv"], (H * V, self.kv_rank)),
                 ParamSpec(prefix + n["o"], (w, H * V))]
        if self.sink:
            specs.append(ParamSpec(prefix + n["sink"], (H,)))
        if self.out_gate:
            specs.append(ParamSpec(prefix + n["g"], (H * V if self.out_gate == "each" else H, w)))
        return specs

    def load(self, tensors, prefix):
        n = self.names
        # the projections that read the layer's input are one product: [query latent | c | kr | gate]
        ws = [tensors.pop(prefix + n["dq"]), tensors.pop(prefix + n["dkv"])]
        if self.out_gate:
            ws.append(tensors.pop(prefix + n["g"]))
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_down = torch.cat(ws, dim=0).contiguous()
        del ws
        self.w_uq = tensors.pop(prefix + n["uq"]).contiguous()
        self.w_uk = tensors.pop(prefix + n["uk"]).contiguous()      # [H, D, kv_rank]: applied to q as it lies
        self.w_uv = tensors.pop(prefix + n["uv"]).contiguous()      # [H, V, kv_rank]
        self.w_o = tensors.pop(prefix + n["o"]).contiguous()
        self.q_gain = tensors.pop(prefix + n["dq_norm"]).to(torch.float32).contiguous()
        self.c_gain = tensors.pop(prefix + n["dkv_norm"]).to(torch.float32).contiguous()
        if self.sink:
            self.sink_logits = tensors.pop(prefix + n["sink"]).to(torch.float32).contiguous()

    # ---- compute
    def forward(self, x, ctx, cache):
        T = x.shape[0]
        H, D, R, V, rank, qr = self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank, self.q_rank
        dk = rank + R
        down = ops.linear(x, self.w_down, None, out_dtype=self.dtype, kind=1)
        group = ctx.group(cache.group)
        pages = cache.tensors["latent"]
        q_lat = ops.latent_prepare(down, 0, qr, qr, rank, qr + rank, R, self.q_gain, self.c_gain, self.inv_freq,
                                   self.rot_dims, ctx.positions, group.slots if cache.writes else None,
                                   pages if cache.writes else None, self.eps, rot_scale=self.rot_scale)
        q = ops.linear(q_lat, self.w_uq, None, out_dtype=self.dtype, kind=16)           # [T, H * (D + R)]
        # the heads' key maps applied to the queries, the rotated part behind: float32 [T, H, rank + R]
        q_full = torch.empty((T, H, dk), dtype=torch.float32, device=x.device)
        # bfloat16 steps of more than a few rows: the per-head products on the tensor cores
        product = ops.grouped_heads if (T > self.FEW_ROWS and self.w_uk.dtype == torch.bfloat16
                                        and q.dtype == torch.bfloat16) else ops.head_product
        product(q, H * (D + R), D + R, D, self.w_uk, D * rank, rank, 1, rank, q_full, H * dk, dk, T, H,
                rot=R, rot_dims=self.rot_dims, inv_freq=self.inv_freq, positions=ctx.positions,
                rot_scale=self.rot_scale)
        meta = ctx.attention_work(cache.group, H, self.tile_rows, self.window, H, rank)
        mixed = ops.latent_attention(q_full, pages, self.sink_logits, meta, H, rank, self.scale, self.window,
                                     ctx.page_tokens)                                   # float32 [T, H, rank]
        # the heads' value maps applied to the attention's output, times the heads' gates
        out = torch.empty((T, H * V), dtype=self.dtype, device=x.device)
        gate = down[:, qr + dk:] if self.out_gate else None
        product(mixed, H * rank, rank, rank, self.w_uv, V * rank, 1, rank, V, out, H * V, V, T, H, gate=gate,
                gate_each=self.out_gate == "each")
        return ops.linear(out, self.w_o, None, out_dtype=self.dtype, kind=2)


register_part("mixer", "latent_attention", LatentAttention, replace=True)
