"""Grouped-query softmax attention with per-head query/key norms and a choice of mask, score
bias, sink and gate."""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import CacheTensor, Mixer, PagedNeed, register_part


def log_bucket(distance: int, rows: int, far: float) -> int:
    """The row of a distance-bias table with ``rows`` rows: the first half of the rows stands for
    the distances 0 .. rows/2 - 1 one by one; the others cut the distances from rows/2 up to
    ``far`` evenly on a logarithmic axis, and every larger distance falls into the last row."""
    half = rows // 2
    if distance < half:
        return distance
    step = math.log(distance / half) / math.log(far / half) * (rows - half)
    return min(rows - 1, half + int(math.floor(step)))


class MaskedAttention(Mixer):
    """q, k, v (and the gate) = x W^T as one fused product; an RMS norm over each query and key
    head with one gain vector per projection, shared by the heads (``qk_norm``; "unit": the heads
    are divided by their root mean square and there are no gain tensors); no rotation;
    score = q . k * ``scale`` (times a learned number per query head, ``head_temperature``: tensor
    ``temp`` [H]) (+ a learned bias by head and distance bucket, ``distance_bias``);
    softmax over the keys the mask lets the row see; output projection.

    Options, all constants of the part:
    ``mask`` "window": a row at position i sees j with 0 <= i - j < ``mask_size``; "chunk": j <= i of
    the same chunk, floor(i / mask_size) == floor(j / mask_size), chunks counted from position 0 of
    the sequence; None: every j <= i.
    ``distance_bias`` dict(far=D, rows=B): a table ``rel`` [B, H]; the score of (i, j) gets
    rel[bucket(i - j), h] with ``log_bucket``; the scale does not multiply it.  B is the checkpoint
    tensor's own first size (``rows`` only says how many to make when weights are drawn at random).
    ``unit_sink``: the softmax's denominator has one more term e^0 that carries no value.
    ``out_gate``: the concatenated heads are multiplied by sigmoid(W_g x) element by element.
    ``proj_bias``: q, k, v and the output projection have biases (``<name>.b``); "qkv": only q, k and v.
    Keys are ``key_dim`` wide and values ``value_dim``.

    What a row can see always lies within the last ``mask_size`` positions, so the pages behind
    them are given back (a chunk is a subset of the window of its size).

    Checkpoint tensors under the prefix: q [H*D, hidden], k [G*D, hidden], v [G*E, hidden], o
    [hidden, H*E], q.norm / k.norm [D], rel [B, H], g [H*E, hidden], and ``.b`` beside q, k, v, o
    (``tensor_names`` renames them)."""
    TENSOR_NAMES = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", rel="rel", g="g",
                        temp="temp", bias_suffix=".b")
    decode_capturable = True      # stepped from the step's device arrays alone

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, eps: float, dtype, device, mask: Optional[str] = None,
                 mask_size: Optional[int] = None, qk_norm: bool = True, distance_bias: Optional[dict] = None,
                 unit_sink: bool = False, out_gate: bool = False, proj_bias=False,
                 head_temperature: bool = False, tensor_names: Optional[dict] = None):
        unknown = set(tensor_names or {}) - set(self.TENSOR_NAMES)
        if unknown:
            raise ValueError(f"tensor_names knows {sorted(self.TENSOR_NAMES)}; got {sorted(unknown)}")
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if mask not in (None, "window", "chunk"):
            raise ValueError(f"unknown mask {mask!r}; known: window, chunk")
        if mask is not None and (not mask_size or mask_size < 1):
            raise ValueError("a mask needs its size")
        if key_dim > 256 or value_dim > 256:
            raise ValueError("heads are at most 256 wide")
        self.names = dict(self.TENSOR_NAMES, **(tensor_names or {}))
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale, self.eps = float(scale), float(eps)
        self.mask, self.mask_size = mask, (int(mask_size) if mask is not None else None)
        if qk_norm not in (True, False, "unit") or proj_bias not in (True, False, "qkv"):
            raise ValueError('qk_norm is True, False or "unit"; proj_bias True, False or "qkv"')
        self.qk_norm, self.unit_sink, self.out_gate = qk_norm, bool(unit_sink), bool(out_gate)
        self.proj_bias, self.head_temperature = proj_bias, bool(head_temperature)
        if self.head_temperature and not qk_norm:
            raise ValueError("a temperature per head rides on the head norm")
        self.bias_rows = self.bias_far = None
        if distance_bias is not None:
            self.bias_rows, self.bias_far = int(distance_bias.get("rows") or 16), float(distance_bias["far"])
            if mask != "window":
                raise ValueError("a distance bias is tabulated over a window's distances")
        self.dtype, self.device = dtype, device
        self.tile_rows = ops.masked_tile_rows(dtype, key_dim, value_dim)
        self.w_in = self.b_in = self.w_o = self.b_o = self.q_gain = self.k_gain = self.bias_by_distance = None
        self.q_head_scale = None

    # ---- what it keeps
    def cache_need(self):
        G = self.num_kv_heads
        return PagedNeed((CacheTensor("k", G, self.key_dim), CacheTensor("v", G, self.value_dim)),
                         window=self.mask_size)

    def work_keys(self):
        return [(self.num_heads // self.num_kv_heads, self.tile_rows, self.mask_size)]

    def kernel_libraries(self, dtype):
        return ops.masked_libraries(dtype, self.key_dim, self.value_dim) + ops.gemm_libraries(dtype)

    # ---- tensors
    def _columns(self):
        H, G, D, E = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        q_off, k_off, v_off = 0, H * D, H * D + G * D
        return q_off, k_off, v_off, v_off + G * E

    def param_specs(self, prefix):
        n, w = self.names, self.hidden_size
        H, G, D, E = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        b = n["bias_suffix"]
        specs = [ParamSpec(prefix + n["q"], (H * D, w)), ParamSpec(prefix + n["k"], (G * D, w)),
                 ParamSpec(prefix + n["v"], (G * E, w)), ParamSpec(prefix + n["o"], (w, H * E))]
        if self.proj_bias:
            specs += [ParamSpec(prefix + n["q"] + b, (H * D,)), ParamSpec(prefix + n["k"] + b, (G * D,)),
                      ParamSpec(prefix + n["v"] + b, (G * E,))]
            if self.proj_bias is True:
                specs.append(ParamSpec(prefix + n["o"] + b, (w,)))
        if self.qk_norm is True:
            specs += [ParamSpec(prefix + n["q_norm"], (D,)), ParamSpec(prefix + n["k_norm"], (D,))]
        if self.head_temperature:
            specs.append(ParamSpec(prefix + n["temp"], (H,)))
        if self.bias_rows:
            specs.append(ParamSpec(prefix + n["rel"], (self.bias_rows, H), free_dims=(0,)))
        if self.out_gate:
            specs.append(ParamSpec(prefix + n["g"], (H * E, w)))
        return specs

    def load(self, tensors, prefix):
        n = self.names
        b = n["bias_suffix"]
        # the projections that read the layer's input are one product: [q | k | v | gate]
        ws = [tensors.pop(prefix + n[x]) for x in "qkv"]
        if self.out_gate:
            ws.append(tensors.pop(prefix + n["g"]))
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        del ws
        self.w_o = tensors.pop(prefix + n["o"]).contiguous()
        if self.proj_bias:
            self.b_in = torch.cat([tensors.pop(prefix + n[x] + b).to(torch.float32) for x in "qkv"]).contiguous()
            if self.proj_bias is True:
                self.b_o = tensors.pop(prefix + n["o"] + b).to(torch.float32).contiguous()
        if self.qk_norm is True:
            self.q_gain = tensors.pop(prefix + n["q_norm"]).to(torch.float32).contiguous()
            self.k_gain = tensors.pop(prefix + n["k_norm"]).to(torch.float32).contiguous()
        elif self.qk_norm == "unit":
            self.q_gain = self.k_gain = torch.ones(self.key_dim, dtype=torch.float32, device=self.w_in.device)
        if self.head_temperature:
            self.q_head_scale = tensors.pop(prefix + n["temp"]).to(torch.float32).contiguous()
        if self.bias_rows:
            rel = tensors.pop(prefix + n["rel"]).to(torch.float32)
            self.bias_rows = int(rel.shape[0])
            if self.bias_rows < 2 or not self.bias_far > self.bias_rows // 2:
                raise ValueError("a distance bias has at least two rows and reaches beyond its one-by-one half")
            # the table by distance: a row never reads a key further back than its window
            rows = torch.tensor([log_bucket(d, self.bias_rows, self.bias_far) for d in range(self.mask_size)],
                                dtype=torch.long, device=rel.device)
            self.bias_by_distance = rel[rows].t().contiguous()      # [H, mask_size]

    # ---- compute
    def forward(self, x, ctx, cache):
        H, G, D, E = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        q_off, k_off, v_off, g_off = self._columns()
        proj = ops.linear(x, self.w_in, None, out_dtype=self.dtype, kind=1)
        group = ctx.group(cache.group)
        writes = cache.writes
        q = ops.head_norm_write(proj, q_off, k_off, v_off, self.b_in, self.q_gain, self.k_gain,
                                group.slots if writes else None, cache.k if writes else None,
                                cache.v if writes else None, H, G, D, E, ctx.page_tokens, self.eps,
                                q_head_scale=self.q_head_scale)
        meta = ctx.attention_work(cache.group, H // G, self.tile_rows, self.mask_size, H, E)
        gate = proj[:, g_off:] if self.out_gate else None
        out = ops.masked_attention(q, cache.k, cache.v, meta, H, G, self.scale, self.mask, self.mask_size,
                                   ctx.page_tokens, bias=self.bias_by_distance, unit_sink=self.unit_sink, gate=gate)
        return ops.linear(out, self.w_o, self.b_o, out_dtype=self.dtype, kind=2)


register_part("mixer", "masked_attention", MaskedAttention, replace=True)
