"""The generic decoder: embedding, blocks in their run order, final norm, LM head.

Built from a ``ModelSpec`` alone.  Which blocks exist, what each is made of and in which
order they run (a block may run twice, a layer may read another layer's cache) is data of
the spec; this class holds no architecture-specific name or constant.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.specs import ModelSpec
from ..csrc import ops
from ..csrc.build import compile_many
from ..parts.base import build_block, build_part
from ..weights.loader import ParamSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"run dtype must be float32 or bfloat16, got {dtype}")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.blocks = [build_block(b, dtype, self.device) for b in spec.blocks]
        self._native = None       # the blocks' descriptors for the host library (False: not this model)
        self.final_norm = build_part("norm", spec.final_norm, dtype, self.device)
        self.embedding_norm = None
        if spec.embedding_norm is not None:
            self.embedding_norm = build_part("norm", spec.embedding_norm, dtype, self.device)
            if not hasattr(self.embedding_norm, "embed"):
                raise TypeError("the embedding's norm must be able to norm gathered rows (ScalarRMSNorm)")
        if spec.depth_stack not in (None, "mix", "plain"):
            raise ValueError(f"unknown depth_stack {spec.depth_stack!r}")
        if spec.depth_stack is not None and (spec.residual_streams != 1 or spec.embedding_scale != 1.0
                                             or spec.position_table_name is not None
                                             or any(st.input_mix for st in spec.run_order)):
            raise ValueError("a depth stack goes with one residual stream, an unscaled embedding and no input mixes")
        self.embed = None
        self.lm_head = None
        self.position_table = None
        self.input_mixes: Dict[str, torch.Tensor] = {}
        # a cache layer's need is stated by the run step that writes it
        needs: List[object] = [None] * spec.num_cache_layers
        for step in spec.run_order:
            if step.writes_cache:
                needs[step.cache_layer] = self.blocks[step.block].mixer.cache_need()
        self.cache_needs = needs

    # ------------------------------------------------------------------ tensors
    def param_specs(self) -> List[ParamSpec]:
        s = self.spec
        specs = [ParamSpec(s.embedding_name, (s.vocab_size, s.hidden_size))]
        if s.position_table_name is not None:
            specs.append(ParamSpec(s.position_table_name, (s.max_position, s.hidden_size)))
        for name in dict.fromkeys(st.input_mix for st in s.run_order if st.input_mix is not None):
            specs.append(ParamSpec(name, (s.hidden_size, 2 * s.hidden_size)))
        if self.embedding_norm is not None:
            specs += self.embedding_norm.param_specs(s.embedding_norm_name)
        for b in self.blocks:
            specs += b.param_specs()
        specs += self.final_norm.param_specs(s.final_norm_name)
        if s.lm_head_name is not None:
            specs.append(ParamSpec(s.lm_head_name, (s.vocab_size, s.hidden_size)))
        else:
            specs.append(ParamSpec("lm_head.weight", (s.vocab_size, s.hidden_size), optional=True))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        tensors = dict(tensors)
        self.embed = tensors.pop(s.embedding_name).contiguous()
        if s.position_table_name is not None:
            self.position_table = tensors.pop(s.position_table_name).to(self.embed.dtype).contiguous()
        for name in dict.fromkeys(st.input_mix for st in s.run_order if st.input_mix is not None):
            self.input_mixes[name] = tensors.pop(name).contiguous()
        if self.embedding_norm is not None:
            self.embedding_norm.load(tensors, s.embedding_norm_name)
        for b in self.blocks:
            b.load(tensors)
        self.final_norm.load(tensors, s.final_norm_name)
        if s.lm_head_name is not None:
            self.lm_head = tensors.pop(s.lm_head_name).contiguous()
        else:
            self.lm_head = self.embed     # tied: the head is the embedding table

    def kernel_libraries(self):
        from ..csrc import ops
        jobs = [("elementwise", None)] + ops.gemm_libraries(self.dtype)
        for b in self.blocks:
            jobs += b.kernel_libraries(self.dtype)
        for norm in (self.embedding_norm, self.final_norm):
            if norm is not None:
                jobs += norm.kernel_libraries(self.dtype)
        seen, out = set(), []
        for name, defines in jobs:
            key = (name, tuple(sorted((defines or {}).items())))
            if key not in seen:
                seen.add(key)
                out.append((name, defines))
        return out

    def build_kernels(self):
        """Compile, side by side, the kernels this model launches (no-op when built)."""
        compile_many(self.kernel_libraries())

    def decode_capturable(self) -> bool:
        """True when every mixer says it can step decoded tokens inside a captured CUDA graph
        (``Mixer.decode_capturable``)."""
        return all(getattr(b.mixer, "decode_capturable", False) for b in self.blocks)

    # ------------------------------------------------------------------ what a step needs
    def work_keys(self, storage):
        keys = []
        for step in self.spec.run_order:
            mixer = self.blocks[step.block].mixer
            lc = storage.layer(step.cache_layer)
            for gsize, tile_rows, window in mixer.work_keys():
                key = (lc.group, gsize, tile_rows, window)
                if key not in keys:
                    keys.append(key)
        return keys

    # ------------------------------------------------------------------ compute
    def _native_descs(self, ctx):
        """The blocks' descriptors for the host library's block executor, or None when this
        model or this step stays with the Python parts: a block of other parts, a run order that
        reads another layer's cache, a mixer with state of its own, a captured step (its launches
        are recorded once and replayed, the interpreter's cost does not recur)."""
        from ..csrc import native_exec
        if self.dtype != torch.bfloat16 or not native_exec.enabled() or getattr(ctx, "captured", False):
            return None
        if ctx.position_ids.dim() != 1:        # several axes: only a position encoding of its own reads them
            return None
        if self._native is None:
            descs = [native_exec.block_desc(b) for b in self.blocks]
            ok = all(d is not None for d in descs) and all(st.writes_cache and st.input_mix is None
                                                           for st in self.spec.run_order)
            ok = ok and self.spec.embedding_scale == 1.0 and self.spec.position_table_name is None
            ok = ok and self.spec.embedding_norm is None and self.spec.depth_stack is None
            self._native = descs if ok else False
        return self._native or None

    def _forward_native(self, descs, ctx, storage, residual):
        from ..csrc import native_exec
        s = self.spec
        T = residual.shape[0]
        buffers, steps = {}, {}
        deltas = [torch.empty((T, s.hidden_size), dtype=self.dtype, device=self.device) for _ in range(2)]
        delta_in = None
        for i, step in enumerate(s.run_order):
            block = self.blocks[step.block]
            cache = storage.layer(step.cache_layer, step.writes_cache)
            m = block.mixer
            key = (cache.group, m.num_heads, m.num_kv_heads, m.head_dim, m.tile_rows, m.window, m.kernel_kind)
            sd = steps.get(key)
            if sd is None:
                sd = steps[key] = native_exec.step_desc(block, ctx, cache, residual, buffers)
            fns = native_exec.exec_fns(m.head_dim, m.kernel_kind == "tc5", native_exec.block_streams(block))
            delta_out = deltas[i & 1]
            native_exec.run_block(descs[step.block], fns, sd, delta_in, delta_out, cache.k, cache.v)
            delta_in = delta_out
        return delta_in

    def _mix_input(self, mix, residual, delta, first):
        """x <- M [x ; e]: the pending branch outputs are folded into x while the operand is formed
        (float32 sum, rounded once to the run dtype); the product's float32 result is the new
        residual, in a buffer of its own (``first`` may be the old one)."""
        from ..parts.norm import DeltaSum
        if isinstance(delta, DeltaSum):
            a, b, scale = delta.a, delta.b, delta.scale
        else:
            a, b, scale = delta, None, 1.0
        if residual.dim() != 2:
            raise ValueError("an input mix reads one residual stream")
        operand = ops.fold_pair(residual, a, b, scale, first, self.dtype)
        return ops.linear(operand, mix, None, out_dtype=torch.float32)

    def forward(self, ctx, storage) -> torch.Tensor:
        """Runs the step's rows through every run step; returns float32 logits at the
        wanted rows, [wanted, vocab]."""
        s = self.spec
        T = ctx.num_tokens
        stack = None
        if s.depth_stack is not None:
            from ..parts.block import DepthStack
            stack = DepthStack(len(s.run_order), T, s.hidden_size, self.dtype, self.device, s.depth_stack == "mix")
            residual = stack.first()
        else:
            residual = torch.empty((T, s.hidden_size), dtype=torch.float32, device=self.device)
        first_lp = None
        if self.embedding_norm is not None:
            first_lp = self.embedding_norm.embed(residual, self.embed, ctx.token_ids,
                                                 stack.lp_dtype() if stack is not None else None)
        elif s.embedding_scale != 1.0 or self.position_table is not None:
            # a learned position row follows the token's place in the sequence
            ops.embedding_positions(residual, self.embed, ctx.token_ids, s.embedding_scale, self.position_table,
                                    ctx.positions)
        else:
            ops.embedding(residual, self.embed, ctx.token_ids)
        first = None
        if self.input_mixes:
            # the embedding output, which input mixes read again: a copy unless the first run step
            # replaces the residual at once (the norms add into the residual in place)
            first = residual if s.run_order[0].input_mix is not None else residual.clone()
        if s.residual_streams > 1:
            # several residual streams, [T, S, W]: every one starts as the embedding
            residual = residual.unsqueeze(1).expand(T, s.residual_streams, s.hidden_size).contiguous()
        if stack is not None:
            if first_lp is None and stack.lp_dtype() is not None:
                first_lp = residual.to(stack.lp_dtype())
            stack.start(first_lp)
            residual = stack
        delta = None
        native = self._native_descs(ctx)
        if native is not None:
            delta = self._forward_native(native, ctx, storage, residual)
        else:
            from ..engine.metrics import nvtx_enabled, nvtx_range
            traced = nvtx_enabled()
            for i, step in enumerate(s.run_order):
                block = self.blocks[step.block]
                cache = storage.layer(step.cache_layer, step.writes_cache)
                if step.input_mix is not None:
                    residual, delta = self._mix_input(self.input_mixes[step.input_mix], residual, delta, first), None
                if traced:
                    with nvtx_range(f"layer.{i}"):
                        residual, delta = block.forward(residual, delta, ctx, cache)
                else:
                    residual, delta = block.forward(residual, delta, ctx, cache)
        if ctx.num_wanted == 0:
            return torch.empty((0, s.vocab_size), dtype=torch.float32, device=self.device)
        if stack is not None:
            residual = stack.current
        h = self.final_norm.add_norm(residual, delta, rows=ctx.want_rows)
        logits = ops.linear(h, self.lm_head, None, out_dtype=torch.float32)
        if s.logit_scale != 1.0 or s.logit_softcap:
            ops.scale_softcap(logits, s.logit_scale, s.logit_softcap)
        return logits
