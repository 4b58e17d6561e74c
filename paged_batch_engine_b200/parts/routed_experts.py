"""A feed-forward of many small gated experts, of which a router picks a few per token."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import FeedForward, register_part
from .mlp import SwiGLU


class RoutedExperts(FeedForward):
    """m_t = sum over the chosen experts e of g_{t,e} W_down,e (silu(W_gate,e x_t) * (W_up,e x_t)).

    The router: logits z = W_router x in float32, scores s = softmax(z) over all experts; the
    experts form ``groups`` equal groups of neighbours, a group's score is its largest score and
    only experts of the ``keep`` best groups can be chosen (``groups`` 1: all can); the ``top``
    allowed experts with the largest scores are chosen; g = s / (sum of the chosen s + 1e-20) *
    ``scale`` (with one group and scale 1 that is the softmax over the chosen logits alone).
    ``router_score`` "sigmoid": s = sigmoid(z) per expert instead of the softmax.  ``correction``: a
    learned vector (tensor ``correction`` [E]) added to s for the choice only (groups and experts are
    ranked by s + correction; the weights use s).  ``group_rank`` "top2_sum": a group's score is the
    sum of its two largest choice scores.  ``shared_size`` F_s: one more expert of that width (tensors
    ``shared.gate``, ``shared.up``, ``shared.down``) runs for every token and is added, unweighted.
    Experts have no biases.  ``activation``: "silu" as above, or "capped_swish" with ``limit`` L and
    ``alpha`` a: g <- min(W_gate x, L), u <- clamp(W_up x, -L, L), hidden = g sigmoid(a g) (u + 1).

    Steps of few rows stream each (row, chosen expert) pair's matrices; steps of many rows sort the
    rows by expert.  In bfloat16 every expert's run is padded to whole row tiles and one launch per
    projection multiplies each tile with its expert's matrix on the tensor cores, all on the
    device.  In float32 one product per expert and projection runs over its rows (``many_rows``:
    from how many rows on; such steps read the experts' row counts on the host and are never
    captured).
    Checkpoint tensors under the prefix: ``router`` [E, hidden]; per expert i ``e<i>.gate``,
    ``e<i>.up`` [inter, hidden] and ``e<i>.down`` [hidden, inter]."""
    decode_capturable = True
    MANY_ROWS_TILED = 16       # bfloat16 steps of at least this many rows take the tiled products

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, dtype, device,
                 groups: int = 1, keep: Optional[int] = None, scale: float = 1.0, many_rows: int = 64,
                 router_name: str = "router", expert_prefix: str = "e", activation: str = "silu",
                 limit: float = 0.0, alpha: float = 1.0, router_score: str = "softmax", correction: bool = False,
                 group_rank: str = "max", shared_size: Optional[int] = None, shared_prefix: str = "shared."):
        keep = groups if keep is None else keep
        if num_experts % groups or not 1 <= keep <= groups or not 1 <= top <= keep * (num_experts // groups):
            raise ValueError("experts divide into equal groups, 1 <= keep <= groups, and the kept groups hold "
                             "at least `top` experts")
        if num_experts > 512 or top > 32 or groups > 64:
            raise ValueError("at most 512 experts, 32 chosen per token and 64 groups")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top, self.groups, self.keep = num_experts, top, groups, keep
        self.scale, self.many_rows = float(scale), int(many_rows)
        self.router_name, self.expert_prefix = router_name, expert_prefix
        if activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"unknown expert activation {activation!r}; known: {', '.join(ops.GLU_ACTIVATIONS)}")
        if activation == "capped_swish" and not limit > 0:
            raise ValueError("the capped activation needs a positive limit")
        self.activation, self.limit, self.alpha = activation, float(limit), float(alpha)
        if router_score not in ops.ROUTER_SCORES or group_rank not in ops.GROUP_RANKS:
            raise ValueError(f"router scores: {sorted(ops.ROUTER_SCORES)}; group ranks: {sorted(ops.GROUP_RANKS)}")
        self.router_score, self.group_rank, self.has_correction = router_score, group_rank, bool(correction)
        self.dtype, self.device = dtype, device
        self.w_router = self.w_gate_up = self.w_down = self.correction = None
        self.shared, self.shared_prefix = None, shared_prefix
        if shared_size:
            if activation != "silu":
                raise ValueError("the shared expert is silu-gated")
            self.shared = SwiGLU(hidden_size, int(shared_size), dtype, device,
                                 tensor_names=dict(gate="gate", up="up", down="down"), weight_suffix="")

    def kernel_libraries(self, dtype):
        tiled = [("grouped_gemm", None)] if dtype == torch.bfloat16 else []
        shared = self.shared.kernel_libraries(dtype) if self.shared is not None else []
        return [("routed_experts", None), ("elementwise", None)] + tiled + ops.gemm_libraries(dtype) + shared

    def param_specs(self, prefix):
        i, h = self.intermediate_size, self.hidden_size
        specs = [ParamSpec(prefix + self.router_name, (self.num_experts, h))]
        if self.has_correction:
            specs.append(ParamSpec(prefix + "correction", (self.num_experts,)))
        if self.shared is not None:
            specs += self.shared.param_specs(prefix + self.shared_prefix)
        for e in range(self.num_experts):
            p = f"{prefix}{self.expert_prefix}{e}."
            specs += [ParamSpec(p + "gate", (i, h)), ParamSpec(p + "up", (i, h)), ParamSpec(p + "down", (h, i))]
        return specs

    def load(self, tensors, prefix):
        self.w_router = tensors.pop(prefix + self.router_name).contiguous()
        if self.has_correction:
            self.correction = tensors.pop(prefix + "correction").to(torch.float32).contiguous()
        if self.shared is not None:
            self.shared.load(tensors, prefix + self.shared_prefix)
        names = [f"{prefix}{self.expert_prefix}{e}." for e in range(self.num_experts)]
        # an expert's gate rows followed by its up rows: one product gives both
        self.w_gate_up = torch.stack([torch.cat([tensors.pop(p + "gate"), tensors.pop(p + "up")], dim=0)
                                      for p in names]).contiguous()
        self.w_down = torch.stack([tensors.pop(p + "down") for p in names]).contiguous()

    def forward(self, x, ctx):
        T = x.shape[0]
        logits = ops.linear(x, self.w_router, None, out_dtype=torch.float32)
        chosen, weights = ops.route(logits, self.top, self.groups, self.keep, self.scale, self.router_score,
                                    self.correction, self.group_rank)
        # the shared expert's output rides into the launch that adds a token's experts up
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        if x.dtype == torch.bfloat16 and self.w_gate_up.dtype == torch.bfloat16:
            if T < min(self.many_rows, self.MANY_ROWS_TILED):
                return self._rows(x, chosen, weights, shared)
            return self._tiled(x, chosen, weights, shared)
        if T < self.many_rows or getattr(ctx, "captured", False):
            return self._rows(x, chosen, weights, shared)
        return self._sorted(x, chosen, weights, shared)

    def _rows(self, x, chosen, weights, shared=None):
        return ops.expert_rows(x, self.w_gate_up, self.w_down, chosen, weights, self.activation, self.limit,
                               self.alpha, addend=shared)

    def _tiled(self, x, chosen, weights, shared=None):
        """bfloat16: rows sorted by expert, every expert's run padded to whole row tiles, and one
        launch per projection that multiplies every tile with its expert's matrix on the tensor
        cores.  Nothing is read on the host."""
        T = x.shape[0]
        counts, place = ops.expert_places(chosen, self.num_experts)
        max_tiles = (T * self.top + ops.GROUP_TILE_ROWS - 1) // ops.GROUP_TILE_ROWS + self.num_experts
        start, tiles = ops.run_tiles(counts, max_tiles)
        rows = ops.expert_gather(x, chosen, place, start, total_rows=max_tiles * ops.GROUP_TILE_ROWS)
        gu = ops.grouped_runs(rows, self.w_gate_up, tiles, self.dtype)
        hidden = torch.empty((rows.shape[0], self.intermediate_size), dtype=self.dtype, device=x.device)
        ops.gated_activation(gu, hidden, self.activation, self.limit, self.alpha)
        out = ops.grouped_runs(hidden, self.w_down, tiles, self.dtype)
        return ops.expert_scatter(out, chosen, place, start, weights, T, addend=shared)

    def _sorted(self, x, chosen, weights, shared=None):
        """Rows sorted by expert, one product per expert and projection over its run of rows."""
        T = x.shape[0]
        counts, place = ops.expert_places(chosen, self.num_experts)
        ends = torch.cumsum(counts, 0, dtype=torch.int32)
        start = (ends - counts).contiguous()
        rows = ops.expert_gather(x, chosen, place, start)
        bounds = ends.tolist()                       # the experts' runs, known on the host
        hidden = torch.empty((rows.shape[0], self.intermediate_size), dtype=self.dtype, device=x.device)
        out = torch.empty_like(rows)
        lo = 0
        for e, hi in enumerate(bounds):
            if hi > lo:
                gu = ops.linear(rows[lo:hi], self.w_gate_up[e], None, out_dtype=self.dtype)
                ops.gated_activation(gu, hidden[lo:hi], self.activation, self.limit, self.alpha)
                out[lo:hi] = ops.linear(hidden[lo:hi], self.w_down[e], None, out_dtype=self.dtype)
            lo = hi
        return ops.expert_scatter(out, chosen, place, start, weights, T, addend=shared)


register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
