"""Arrangements of norms, mixer and feed-forward in a layer."""
from __future__ import annotations

import torch

from ..config.specs import BlockSpec
from .base import Block, build_part, register_part
from ..weights.loader import ParamSpec
from .norm import DeltaSum


class PreNormBlock(Block):
    """x -> norm -> mixer -> +x -> norm -> feed-forward -> +x  (reference:
    infMain/source/model/qwen2_batch.cpp:600-601, 753-759, 780).  Each add is carried as
    ``delta`` into the next norm so that add and norm are one kernel."""

    def __init__(self, spec: BlockSpec, dtype, device):
        self.spec = spec
        self.prefix = spec.prefix
        n = spec.names
        self.p_mixer = self.prefix + n.get("mixer", "mixer.")
        self.p_ffn = self.prefix + n.get("feed_forward", "feed_forward.")
        self.p_norm1 = self.prefix + n.get("norm_mixer", "norm_mixer.")
        self.p_norm2 = self.prefix + n.get("norm_feed_forward", "norm_feed_forward.")
        self.norm1 = build_part("norm", spec.norm_mixer, dtype, device)
        self.mixer = build_part("mixer", spec.mixer, dtype, device)
        self.norm2 = build_part("norm", spec.norm_feed_forward, dtype, device)
        self.ffn = build_part("feed_forward", spec.feed_forward, dtype, device)

    def parts(self):
        return [(self.norm1, self.p_norm1), (self.mixer, self.p_mixer), (self.norm2, self.p_norm2),
                (self.ffn, self.p_ffn)]

    def param_specs(self, prefix=""):
        out = []
        for part, p in self.parts():
            out += part.param_specs(p)
        return out

    def load(self, tensors, prefix=""):
        for part, p in self.parts():
            part.load(tensors, p)

    def kernel_libraries(self, dtype):
        out = []
        for part, _ in self.parts():
            out += part.kernel_libraries(dtype)
        return out

    def forward(self, residual, delta, ctx, cache):
        h = self.norm1.add_norm(residual, delta)
        a = self.mixer.forward(h, ctx, cache)
        f = self.norm2.add_norm(residual, a)
        m = self.ffn.forward(f, ctx)
        return residual, m


class ParallelBlock(PreNormBlock):
    """x -> x + mixer(norm1(x)) + feed_forward(norm2(x)): both branches read norms of the same
    residual, which differ in their gains only (one launch makes both), and their outputs travel
    together as a ``DeltaSum`` into the next layer's norms, where x + (a + b) is formed in
    float32.  A layer without feed-forward has the mixer branch alone.

    A layer with a feed-forward but no norm of its own for it (``norm_feed_forward`` None) has ONE
    norm whose output both branches read: x -> x + mixer(n(x)) + feed_forward(n(x)).
    ``args["branch_scale"]`` m scales the branches before the residual sum: x + m * (a + b)."""

    def __init__(self, spec: BlockSpec, dtype, device):
        self.spec = spec
        self.prefix = spec.prefix
        n = spec.names
        self.p_mixer = self.prefix + n.get("mixer", "mixer.")
        self.p_ffn = self.prefix + n.get("feed_forward", "feed_forward.")
        self.p_norm1 = self.prefix + n.get("norm_mixer", "norm_mixer.")
        self.p_norm2 = self.prefix + n.get("norm_feed_forward", "norm_feed_forward.")
        self.norm1 = build_part("norm", spec.norm_mixer, dtype, device)
        self.mixer = build_part("mixer", spec.mixer, dtype, device)
        self.norm2 = self.ffn = None
        self.branch_scale = float(spec.args.get("branch_scale", 1.0))
        if spec.feed_forward is not None:
            if spec.norm_feed_forward is not None:
                self.norm2 = build_part("norm", spec.norm_feed_forward, dtype, device)
            self.ffn = build_part("feed_forward", spec.feed_forward, dtype, device)
        if not hasattr(self.norm1, "add_norm_pair"):
            raise TypeError("a parallel block needs norms that can be taken in pairs (RMSNorm)")

    def parts(self):
        out = [(self.norm1, self.p_norm1), (self.mixer, self.p_mixer)]
        if self.norm2 is not None:
            out.append((self.norm2, self.p_norm2))
        if self.ffn is not None:
            out.append((self.ffn, self.p_ffn))
        return out

    def forward(self, residual, delta, ctx, cache):
        m = self.branch_scale
        if self.ffn is None:
            a = self.mixer.forward(self.norm1.add_norm(residual, delta), ctx, cache)
            return residual, (a if m == 1.0 else DeltaSum(a, None, m))
        if self.norm2 is None:
            h1 = h2 = self.norm1.add_norm(residual, delta)
        else:
            h1, h2 = self.norm1.add_norm_pair(self.norm2, residual, delta)
        a = self.mixer.forward(h1, ctx, cache)
        return residual, DeltaSum(a, self.ffn.forward(h2, ctx), m)


class DepthStack:
    """The residual of a model whose layers hand on a learned mix over everything computed so far:
    ``results`` float32 [runs + 1, T, W] holds X_0 (the embedding output) and every layer run's own
    result X_(i+1); ``current`` (float32 [T, W]) is what the next layer reads, ``current_lp`` the
    same in the run dtype for the products (``current`` itself in float32 runs).  Without a mix a
    layer's result is what the next one reads and ``results`` keeps two rows that take turns."""

    def __init__(self, runs: int, tokens: int, width: int, run_dtype, device, mixes: bool):
        self.mixes = bool(mixes)
        self.results = torch.empty(((runs + 1) if mixes else 2, tokens, width), dtype=torch.float32, device=device)
        self.mixed = torch.empty((2, tokens, width), dtype=torch.float32, device=device) if mixes else None
        self.filled = 0
        self.run_dtype = run_dtype
        self.current = self.current_lp = None

    def lp_dtype(self):
        return None if self.run_dtype == torch.float32 else self.run_dtype

    def first(self):
        """Where the embedding output goes."""
        return self.results[0]

    def start(self, lp):
        self.filled = 1
        self.current = self.results[0]
        self.current_lp = lp if lp is not None else self.current

    def next_result(self):
        return self.results[self.filled if self.mixes else self.filled & 1]

    def next_mixed(self):
        return self.mixed[self.filled & 1] if self.mixes else None

    def push(self, mixed, lp):
        """The layer run's result is in ``next_result()`` (and its mix over depth in ``mixed``)."""
        result = self.next_result()
        self.filled += 1
        self.current = mixed if mixed is not None else result
        self.current_lp = lp if lp is not None else self.current


class PostNormBlock(Block):
    """Norm after the sum, sublayers reading the stream itself: x <- n1(alpha x + mixer(x)), then
    (with a feed-forward) x <- n2(alpha x + feed_forward(x)); ``args["alpha"]`` scales the skip path.
    The stream is float32; the products read its rounding to the run dtype, which the norm's launch
    leaves beside it.  ``args["depth_mix"]``: the layer hands on sum_j d[j] X_j over the embedding
    output and every layer result so far, its own last, with d the tensor ``<prefix>dwa``
    [``args["depth_index"]`` + 2]; the mix is part of the last norm's launch.  The residual such
    blocks pass along is a ``DepthStack``."""

    def __init__(self, spec: BlockSpec, dtype, device):
        self.spec = spec
        self.prefix = spec.prefix
        n = spec.names
        self.dtype = dtype
        self.p_mixer = self.prefix + n.get("mixer", "mixer.")
        self.p_ffn = self.prefix + n.get("feed_forward", "feed_forward.")
        self.p_norm1 = self.prefix + n.get("norm_mixer", "norm_mixer.")
        self.p_norm2 = self.prefix + n.get("norm_feed_forward", "norm_feed_forward.")
        self.p_mix = self.prefix + n.get("depth_mix", "dwa")
        self.norm1 = build_part("norm", spec.norm_mixer, dtype, device)
        self.mixer = build_part("mixer", spec.mixer, dtype, device)
        self.norm2 = self.ffn = None
        if spec.feed_forward is not None:
            self.norm2 = build_part("norm", spec.norm_feed_forward, dtype, device)
            self.ffn = build_part("feed_forward", spec.feed_forward, dtype, device)
        for norm in (self.norm1, self.norm2):
            if norm is not None and not hasattr(norm, "norm_sum"):
                raise TypeError("a post-norm block needs norms that take the scaled sum (ScalarRMSNorm)")
        self.alpha = float(spec.args.get("alpha", 1.0))
        self.depth_mix = bool(spec.args.get("depth_mix", False))
        self.depth_index = int(spec.args.get("depth_index", 0))
        self.mix_weights = None

    def parts(self):
        out = [(self.norm1, self.p_norm1), (self.mixer, self.p_mixer)]
        if self.ffn is not None:
            out += [(self.norm2, self.p_norm2), (self.ffn, self.p_ffn)]
        return out

    def param_specs(self, prefix=""):
        out = []
        for part, p in self.parts():
            out += part.param_specs(p)
        if self.depth_mix:
            out.append(ParamSpec(self.p_mix, (self.depth_index + 2,)))
        return out

    def load(self, tensors, prefix=""):
        for part, p in self.parts():
            part.load(tensors, p)
        if self.depth_mix:
            self.mix_weights = tensors.pop(self.p_mix).to(torch.float32).contiguous()

    def kernel_libraries(self, dtype):
        out = []
        for part, _ in self.parts():
            out += part.kernel_libraries(dtype)
        return out

    def forward(self, residual, delta, ctx, cache):
        if not isinstance(residual, DepthStack) or delta is not None:
            raise TypeError("post-norm blocks pass a DepthStack along and leave nothing pending")
        st = residual
        if self.depth_mix and st.filled != self.depth_index + 1:
            raise ValueError(f"the depth mix of layer run {self.depth_index} needs {self.depth_index + 1} earlier "
                             f"results, the stack holds {st.filled}")
        lp = st.lp_dtype()
        last = dict(normed=st.next_result())
        if self.depth_mix:
            last.update(stack=st.results, n_prev=st.filled, mix=self.mix_weights, mixed=st.next_mixed())
        y = self.mixer.forward(st.current_lp, ctx, cache)
        if self.ffn is None:
            out_lp = self.norm1.norm_sum(st.current, y, self.alpha, lp, **last)
        else:
            x1 = torch.empty_like(st.current)
            x1_lp = self.norm1.norm_sum(st.current, y, self.alpha, lp, normed=x1)
            f = self.ffn.forward(x1_lp if x1_lp is not None else x1, ctx)
            out_lp = self.norm2.norm_sum(x1, f, self.alpha, lp, **last)
        st.push(last.get("mixed"), out_lp)
        return st, None


register_part("block", "postnorm", lambda spec, dtype, device: PostNormBlock(spec, dtype, device), replace=True)
register_part("block", "prenorm", lambda spec, dtype, device: PreNormBlock(spec, dtype, device),
              replace=True)
register_part("block", "parallel", lambda spec, dtype, device: ParallelBlock(spec, dtype, device),
              replace=True)
