"""Norms fused with the residual add that precedes them."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    """y = (w * x) * rsqrt(mean(x^2) + eps) on x = residual + delta, all in float32.

    The reference runs the add (add_kernel.cu:6-15) and the norm (rmsnorm_kernel.cu:9-41)
    as two launches and rounds the residual stream to the run dtype in between; here it is
    one launch and the residual stream stays float32.

    ``one_plus``: the checkpoint stores the gain around zero, w = 1 + stored (formed once at load,
    in float32)."""

    def __init__(self, size: int, eps: float, dtype, device, weight_name: str = "weight", one_plus: bool = False):
        self.size, self.eps, self.dtype, self.device = int(size), float(eps), dtype, device
        self.weight_name, self.one_plus = weight_name, bool(one_plus)
        self.gain = None

    def param_specs(self, prefix):
        return [ParamSpec(prefix + self.weight_name, (self.size,))]

    def load(self, tensors, prefix):
        self.gain = tensors[prefix + self.weight_name].to(torch.float32).contiguous()
        if self.one_plus:
            self.gain = (self.gain + 1.0).contiguous()

    def add_norm(self, residual, delta, rows=None, out_dtype=None):
        if isinstance(delta, DeltaSum):
            return ops.add2_rmsnorm2(residual, delta.a, delta.b, self.gain, None, self.eps,
                                     out_dtype or self.dtype, rows, delta_scale=delta.scale)[0]
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype or self.dtype, device=residual.device)
        return ops.add_rmsnorm(residual, delta, self.gain, out, self.eps, rows)

    def add_norm_pair(self, other: "RMSNorm", residual, delta, out_dtype=None):
        """This norm and ``other`` of the same summed row (residual += delta first): the two differ
        in their gains only, so one launch and one root mean square serve both."""
        if other.size != self.size or other.eps != self.eps:
            raise ValueError("two norms of one row share its width and eps")
        a, b, scale = (delta.a, delta.b, delta.scale) if isinstance(delta, DeltaSum) else (delta, None, 1.0)
        return ops.add2_rmsnorm2(residual, a, b, self.gain, other.gain, self.eps, out_dtype or self.dtype,
                                 delta_scale=scale)


class ScalarRMSNorm(Norm):
    """y = g * x / sqrt(mean(x^2) + eps) with ONE learned number g for all coordinates (the checkpoint
    tensor has no axes), all in float32.  As a norm after a plain residual add it behaves like
    ``RMSNorm`` (residual += delta, then the norm); layers that normalise after the sum call
    ``norm_sum`` instead."""

    def __init__(self, size: int, eps: float, dtype, device, weight_name: str = "weight"):
        self.size, self.eps, self.dtype, self.device = int(size), float(eps), dtype, device
        self.weight_name = weight_name
        self.gain = None

    def param_specs(self, prefix):
        return [ParamSpec(prefix + self.weight_name, ())]

    def load(self, tensors, prefix):
        self.gain = tensors[prefix + self.weight_name].to(torch.float32).reshape(1).contiguous()

    def kernel_libraries(self, dtype):
        return [("unit_norm", None)]

    def add_norm(self, residual, delta, rows=None, out_dtype=None):
        if isinstance(delta, DeltaSum):
            if delta.scale != 1.0:
                raise ValueError("a norm with one gain adds unscaled branches")
            a, b = delta.a, delta.b
        else:
            a, b = delta, None
        write_back = rows is None and (a is not None or b is not None)
        return ops.unit_norm(residual, a, b, 1.0, self.gain, self.eps, out_dtype or self.dtype, rows=rows,
                             sum_out=residual if write_back else None)

    def norm_sum(self, x, y, alpha, lp_dtype, normed=None, stack=None, n_prev=0, mix=None, mixed=None):
        """g * n(alpha * x + y) (``y`` a tensor, a ``DeltaSum`` of two, or None): float32 into ``normed``;
        with ``mix`` the learned mix over ``stack[:n_prev]`` and this result into ``mixed``; the last of
        these also returned in ``lp_dtype`` (None: not)."""
        a, b = (y.a, y.b) if isinstance(y, DeltaSum) else (y, None)
        return ops.unit_norm(x, a, b, alpha, self.gain, self.eps, lp_dtype, normed=normed, stack=stack, n_prev=n_prev,
                             mix=mix, mixed=mixed)

    def embed(self, out, table, ids, lp_dtype):
        """The norm of gathered embedding rows, float32 into ``out``; a copy in ``lp_dtype`` returned."""
        return ops.embedding_unit_norm(out, table, ids, self.gain, self.eps, lp_dtype)


class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b on x = residual + delta, all
    in float32 (the variance from the deviations, in a second pass over the row).

    ``residual`` is float32 [T, W], or [T, S, W] for S residual streams: the norm then reads
    their sum.  ``delta`` is a tensor [T, W] (the plain residual add; one stream), or a
    ``PendingUpdate`` of a block with several streams, folded in by the same launch.
    Checkpoint tensors: ``prefix + weight_name`` and ``prefix + bias_name`` (None: no bias)."""

    def __init__(self, size: int, eps: float, dtype, device, weight_name: str = "weight",
                 bias_name: Optional[str] = "bias"):
        self.size, self.eps, self.dtype, self.device = int(size), float(eps), dtype, device
        self.weight_name, self.bias_name = weight_name, bias_name
        self.gain = self.bias = None
        self._ones = {}

    def param_specs(self, prefix):
        specs = [ParamSpec(prefix + self.weight_name, (self.size,))]
        if self.bias_name is not None:
            specs.append(ParamSpec(prefix + self.bias_name, (self.size,)))
        return specs

    def load(self, tensors, prefix):
        self.gain = tensors[prefix + self.weight_name].to(torch.float32).contiguous()
        if self.bias_name is not None:
            self.bias = tensors[prefix + self.bias_name].to(torch.float32).contiguous()

    def identity(self, streams: int, device):
        """(mix, beta, alpha) of a plain residual add: the streams unchanged, the delta added to each."""
        got = self._ones.get(streams)
        if got is None:
            got = self._ones[streams] = (torch.eye(streams, dtype=torch.float32, device=device).contiguous(),
                                         torch.ones(streams, dtype=torch.float32, device=device))
        return got

    def norm_streams(self, streams, pending, alpha, rows=None, out_dtype=None):
        """The norm of sum_j alpha_j r_j after ``pending`` (a ``PendingUpdate`` or None) is folded in."""
        n = streams.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype or self.dtype, device=streams.device)
        eye, ones = self.identity(streams.shape[1], streams.device)
        if pending is None:
            y, mix, beta = None, eye, ones
        else:
            y, mix, beta = pending.y, pending.mix, pending.beta
        return ops.stream_norm(streams, y, mix, beta, ones if alpha is None else alpha, self.gain, self.bias, out,
                               self.eps, rows)

    def as_pending(self, delta, streams):
        """A plain delta (added to every stream) as a ``PendingUpdate``."""
        eye, ones = self.identity(streams.shape[1], streams.device)
        return PendingUpdate(delta, eye, ones)

    def add_norm(self, residual, delta, rows=None, out_dtype=None):
        streams = residual if residual.dim() == 3 else residual.view(residual.shape[0], 1, residual.shape[1])
        if delta is not None and not isinstance(delta, PendingUpdate):
            delta = self.as_pending(delta, streams)
        return self.norm_streams(streams, delta, None, rows, out_dtype)

    def kernel_libraries(self, dtype):
        return [("streams", None)]


class DeltaSum:
    """Two branch outputs of one layer that are not yet added to the residual: x' = x + scale *
    (a + b) (``b`` may be None).  The next norm's launch adds them."""
    __slots__ = ("a", "b", "scale")

    def __init__(self, a, b, scale: float = 1.0):
        self.a, self.b, self.scale = a, b, float(scale)


class PendingUpdate:
    """A sublayer's output that is not yet folded into the residual streams: r'_j = sum_s
    mix[s, j] r_s + beta[j] y.  The next norm's launch does it."""
    __slots__ = ("y", "mix", "beta")

    def __init__(self, y, mix, beta):
        self.y, self.mix, self.beta = y, mix, beta


register_part("norm", "rmsnorm", RMSNorm, replace=True)
register_part("norm", "layernorm", LayerNorm, replace=True)
register_part("norm", "scalar_rmsnorm", ScalarRMSNorm, replace=True)
