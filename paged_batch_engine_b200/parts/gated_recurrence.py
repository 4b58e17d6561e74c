"""A gated diagonal linear recurrence behind a short causal convolution, times an activated branch."""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import CompositeNeed, Mixer, StateNeed, register_part


class GatedLinearRecurrence(Mixer):
    """Two branches of ``width`` channels from the layer's input: y = act(W_y x + b_y) and
    u = conv(W_x x + b_x), a causal convolution per channel (``conv_taps`` taps, bias, the last tap on
    the current token, no activation).  The channels form ``blocks`` equal parts; in part b
    r = sigmoid(R_b u_b + c_r) and i = sigmoid(I_b u_b + c_i) with square maps R_b, I_b.  Per channel

        a_t = exp(-``rate`` * r_t * softplus(lam)),   S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t

    from S = 0 (no special case for the first token); the output is W_o (S * y).  S is float32, kept
    per request, as are the convolution's last taps - 1 inputs; gates, decays and the recurrence are
    float32.  ``activation``: "gelu_tanh".

    In bfloat16 runs the gates' products run on the tensor cores (``ops.gate_products``: products of
    two bfloat16 numbers are exact in float32, the sums are float32) and the scan forms a and b from
    the pre-activations on its way; float32 runs take ``ops.recurrence_gates`` (float32 FMAs).
    ``PBE_GATES=fma`` keeps bfloat16 runs on the latter too.

    Checkpoint tensors under the prefix (names in ``tensor_names``): y, x [width, hidden] with biases
    ``.b``, conv [width, taps], conv.b, ra, ri [blocks, width/blocks, width/blocks] ([out, in]) with
    biases ``.b`` [blocks, width/blocks], lam [width], o [hidden, width]."""
    TENSOR_NAMES = dict(y="y", x="x", conv="conv", conv_bias="conv.b", gate_a="ra", gate_i="ri", lam="lam", o="o",
                        bias_suffix=".b")
    decode_capturable = True      # stepped from the step's device arrays alone

    def __init__(self, hidden_size: int, width: int, blocks: int, conv_taps: int, dtype, device, rate: float = 8.0,
                 activation: str = "gelu_tanh", tensor_names: Optional[dict] = None):
        unknown = set(tensor_names or {}) - set(self.TENSOR_NAMES)
        if unknown:
            raise ValueError(f"tensor_names knows {sorted(self.TENSOR_NAMES)}; got {sorted(unknown)}")
        if blocks < 1 or width % blocks:
            raise ValueError("the channels divide into equal blocks")
        if not 1 <= conv_taps <= 16:
            raise ValueError("the convolution has 1 to 16 taps")
        if activation not in ops.SCAN_ACTIVATIONS or activation is None:
            raise ValueError(f"unknown branch activation {activation!r}")
        self.names = dict(self.TENSOR_NAMES, **(tensor_names or {}))
        self.hidden_size, self.width, self.blocks, self.conv_taps = hidden_size, width, blocks, conv_taps
        self.rate, self.activation = float(rate), activation
        self.dtype, self.device = dtype, device
        self.w_in = self.b_in = self.w_o = self.conv_w = self.conv_wt = self.conv_b = None
        self.w_r = self.w_i = self.b_r = self.b_i = self.lam = self.w_gates = None

    def cache_need(self):
        need = dict(rec=StateNeed((self.width,), torch.float32))
        if self.conv_taps > 1:
            need["conv"] = StateNeed((self.conv_taps - 1, self.width), torch.float32)
        return CompositeNeed.of(**need)

    def kernel_libraries(self, dtype):
        tiled = [("grouped_gemm", None)] if dtype == torch.bfloat16 else []
        return [("short_conv", None), ("gated_recurrence", None)] + tiled + ops.gemm_libraries(dtype)

    def param_specs(self, prefix):
        n, w, C, B = self.names, self.hidden_size, self.width, self.blocks
        b = n["bias_suffix"]
        return [ParamSpec(prefix + n["y"], (C, w)), ParamSpec(prefix + n["y"] + b, (C,)),
                ParamSpec(prefix + n["x"], (C, w)), ParamSpec(prefix + n["x"] + b, (C,)),
                ParamSpec(prefix + n["conv"], (C, self.conv_taps)), ParamSpec(prefix + n["conv_bias"], (C,)),
                ParamSpec(prefix + n["gate_a"], (B, C // B, C // B)), ParamSpec(prefix + n["gate_a"] + b, (B, C // B)),
                ParamSpec(prefix + n["gate_i"], (B, C // B, C // B)), ParamSpec(prefix + n["gate_i"] + b, (B, C // B)),
                ParamSpec(prefix + n["lam"], (C,)), ParamSpec(prefix + n["o"], (w, C))]

    def load(self, tensors, prefix):
        n = self.names
        b = n["bias_suffix"]
        f32 = lambda name: tensors.pop(prefix + name).to(torch.float32).contiguous()
        # the two projections that read the layer's input are one product: [y | x]
        ws = [tensors.pop(prefix + n["y"]), tensors.pop(prefix + n["x"])]
        if ws[0].dtype != ws[1].dtype:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        del ws
        self.b_in = torch.cat([f32(n["y"] + b), f32(n["x"] + b)]).contiguous()
        self.w_o = tensors.pop(prefix + n["o"]).contiguous()
        self.conv_w, self.conv_b = f32(n["conv"]), f32(n["conv_bias"])
        self.conv_wt = self.conv_w.t().contiguous()        # [taps, C]: the layout the eight-channel kernel reads
        self.w_r = tensors.pop(prefix + n["gate_a"]).contiguous()
        self.w_i = tensors.pop(prefix + n["gate_i"]).contiguous()
        if self.w_r.dtype != self.w_i.dtype:
            self.w_r, self.w_i = self.w_r.to(torch.float32), self.w_i.to(torch.float32)
        self.b_r = f32(n["gate_a"] + b).reshape(-1).contiguous()
        self.b_i = f32(n["gate_i"] + b).reshape(-1).contiguous()
        self.lam = f32(n["lam"])
        if self.w_r.dtype == torch.bfloat16 and os.environ.get("PBE_GATES", "").strip().lower() != "fma":
            # a block's recurrence-gate rows followed by its input-gate rows: one product gives both
            self.w_gates = torch.cat([self.w_r, self.w_i], dim=1).contiguous()

    def chunk_rows(self, rows: int) -> int:
        """Rows of a chunk when a long portion's recurrence runs as chunks side by side: so long that
        the chunks of all channel slices fill the GPU a few times over, a power of two, 32 to 256."""
        want = rows * ((self.width + 127) // 128) // 2048
        chunk = 32
        while chunk < want and chunk < 256:
            chunk *= 2
        return chunk

    def forward(self, x, ctx, cache):
        C = self.width
        proj = ops.linear(x, self.w_in, self.b_in, out_dtype=self.dtype, kind=1)
        y, x_in = proj[:, :C], proj[:, C:]
        if self.conv_taps > 1:
            conv_state = cache.sub["conv"].state
        else:
            conv_state = torch.empty((1, 0, C), dtype=torch.float32, device=x.device)
        u = ops.short_conv(x_in, self.conv_w, self.conv_b, conv_state, ctx.request_of_row, ctx.q_start, ctx.q_len,
                           ctx.state_slots, ctx.num_requests, silu=False, update_state=cache.writes,
                           weight_t=self.conv_wt)
        if self.w_gates is not None and u.dtype == torch.bfloat16:
            a = b = None
            gates = (ops.gate_products(u, self.w_gates), u, self.b_r, self.b_i, self.lam, self.rate)
        else:
            a, b = ops.recurrence_gates(u, self.w_r, self.w_i, self.b_r, self.b_i, self.lam, self.rate)
            gates = None
        captured = getattr(ctx, "captured", False)
        plan = None if captured else ctx.recurrence_plan(self.chunk_rows(ctx.num_tokens))
        state = cache.sub["rec"].state
        if not cache.writes:
            state = state.clone()
        out = ops.gated_scan(a, b, y, state, ctx.q_start, ctx.q_len, ctx.state_slots, ctx.num_requests, self.dtype,
                             self.activation, plan, zero_out=captured, gates=gates)
        return ops.linear(out, self.w_o, None, out_dtype=self.dtype, kind=2)


register_part("mixer", "gated_linear_recurrence", GatedLinearRecurrence, replace=True)
