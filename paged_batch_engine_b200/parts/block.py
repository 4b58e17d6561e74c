"""Arrangements of norms, mixer and feed-forward in a layer."""
from __future__ import annotations

from ..config.specs import BlockSpec
from .base import Block, build_part, register_part
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


register_part("block", "prenorm", lambda spec, dtype, device: PreNormBlock(spec, dtype, device),
              replace=True)
register_part("block", "parallel", lambda spec, dtype, device: ParallelBlock(spec, dtype, device),
              replace=True)
