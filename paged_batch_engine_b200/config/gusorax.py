"""Typed configuration of the Gusorax design and its model as data.

config.json keys: ``architecture`` ("Gusorax"), ``width``, ``vocab``, ``max_positions``,
``norm.eps``, ``embedding.scale``, ``residual_mult``, ``loop`` (``start``, ``stop``, ``times``;
absent or null: every layer runs once) and ``layers``, a list of entries with ``type``
("attention" or "attention_2"), ``mixer`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``mask.size``, and for "attention" ``bias_max``; the rows of the bias table are the checkpoint
tensor's, ``bias_rows`` only says how many to make when weights are drawn at random) and ``mlp`` (``{"kind": "dense", "ff": n}``,
``{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}}`` or null).

Tensors: ``embed``, ``pos``, ``loop.in``, ``final.norm``, ``head``; per layer ``l<i>.norm1``,
``l<i>.mix.*`` and ``l<i>.mlp.*``.

The token's embedding row is scaled and a learned position row added.  The layers ``start`` ..
``stop - 1`` run ``times`` times in a row with the same tensors and a cache of their own for every
pass; right before the first layer of each pass the residual x becomes W_in [x ; e], e being the
embedding output.  A layer has one RMS norm n (gain 1 + w) and adds both branches scaled:
x + m (mixer(n(x)) + mlp(n(x))).  attention: grouped-query softmax attention with an RMS norm per
query and key head, a learned bias by head and distance bucket, and a sliding window.  attention_2:
projection biases, a chunked mask, one added to the softmax's denominator, a sigmoid gate on the
concatenated heads.  Feed-forwards: dense silu-gated, or routed experts with a capped gate and a
clamped linear part, weighted by the softmax over the chosen router logits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .specs import BlockSpec, ConfigError, ModelSpec, PartSpec, RunStep

_LAYER_TYPES = ("attention", "attention_2")
_MLP_KINDS = ("dense", "moe")
DEFAULT_BIAS_ROWS = 16          # rows of a bias table made at random when the configuration names none
EXPERT_GATE_SLOPE = 1.702       # the experts' gate is g * sigmoid(1.702 g): the design fixes it


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"{where} lacks {key!r}")
    return d[key]


def _positive(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


@dataclass
class GusoraxConfig:
    width: int
    vocab: int
    max_positions: int
    eps: float
    embedding_scale: float
    residual_mult: float
    loop: Optional[Dict[str, int]]
    layers: List[dict]
    raw: Dict[str, Any]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GusoraxConfig":
        loop = d.get("loop")
        cfg = cls(width=_positive(_need(d, "width", "config.json"), "width"),
                  vocab=_positive(_need(d, "vocab", "config.json"), "vocab"),
                  max_positions=_positive(_need(d, "max_positions", "config.json"), "max_positions"),
                  eps=float(_need(_need(d, "norm", "config.json"), "eps", "norm")),
                  embedding_scale=float(_need(_need(d, "embedding", "config.json"), "scale", "embedding")),
                  residual_mult=float(_need(d, "residual_mult", "config.json")),
                  loop=dict(loop) if loop else None,
                  layers=list(_need(d, "layers", "config.json")), raw=dict(d))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps!r}")
        if not self.layers:
            raise ConfigError("layers is empty")
        if self.loop is not None:
            start, stop = _need(self.loop, "start", "loop"), _need(self.loop, "stop", "loop")
            times = _positive(_need(self.loop, "times", "loop"), "loop.times")
            if not (isinstance(start, int) and isinstance(stop, int) and 0 <= start < stop <= len(self.layers)):
                raise ConfigError(f"loop: 0 <= start < stop <= {len(self.layers)} layers, got {start!r}, {stop!r}")
            del times
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in _LAYER_TYPES:
                raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {', '.join(_LAYER_TYPES)}")
            m = _need(layer, "mixer", where)
            mw = where + ".mixer"
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _positive(_need(m, key, mw), f"{mw}.{key}")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{mw}: heads must be a multiple of kv_heads")
            if m["dim"] > 256 or m["vdim"] > 256:
                raise ConfigError(f"{mw}: heads are at most 256 wide")
            _need(m, "scale", mw)
            _positive(_need(_need(m, "mask", mw), "size", mw + ".mask"), f"{mw}.mask.size")
            if kind == "attention" and not float(_need(m, "bias_max", mw)) > 0:
                raise ConfigError(f"{mw}.bias_max must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                mk = mlp.get("kind", "dense")
                if mk not in _MLP_KINDS:
                    raise ConfigError(f"{where}.mlp.kind {mk!r} is not supported; known: {', '.join(_MLP_KINDS)}")
                if mk == "dense":
                    _positive(_need(mlp, "ff", where + ".mlp"), f"{where}.mlp.ff")
                else:
                    ex = _need(mlp, "expert", where + ".mlp")
                    _positive(_need(ex, "ff", where + ".mlp.expert"), "expert.ff")
                    if not float(_need(ex, "limit", where + ".mlp.expert")) > 0:
                        raise ConfigError(f"{where}.mlp.expert.limit must be positive")
                    r = _need(mlp, "router", where + ".mlp")
                    E = _positive(_need(r, "experts", where + ".mlp.router"), "router.experts")
                    top = _positive(_need(r, "top", where + ".mlp.router"), "router.top")
                    if top > E:
                        raise ConfigError(f"{where}.mlp.router: top is at most experts")

    # ------------------------------------------------------------------ the model as data
    def _mixer(self, layer: dict) -> PartSpec:
        m = layer["mixer"]
        args = dict(hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                    key_dim=int(m["dim"]), value_dim=int(m["vdim"]), scale=float(m["scale"]), eps=self.eps,
                    mask_size=int(m["mask"]["size"]), qk_norm=True)
        if layer["type"] == "attention":
            args.update(mask="window", distance_bias=dict(rows=int(m.get("bias_rows", DEFAULT_BIAS_ROWS)),
                                                          far=float(m["bias_max"])))
        else:
            args.update(mask="chunk", unit_sink=True, out_gate=True, proj_bias=True)
        return PartSpec("masked_attention", args)

    def _mlp(self, mlp: Optional[dict]) -> Optional[PartSpec]:
        if mlp is None:
            return None
        if mlp.get("kind", "dense") == "dense":
            return PartSpec("swiglu", dict(hidden_size=self.width, intermediate_size=int(mlp["ff"]),
                                           tensor_names=dict(gate="gate", up="up", down="down"), weight_suffix=""))
        r = mlp["router"]
        return PartSpec("routed_experts", dict(
            hidden_size=self.width, intermediate_size=int(mlp["expert"]["ff"]), num_experts=int(r["experts"]),
            top=int(r["top"]), groups=1, keep=1, scale=1.0, activation="capped_swish",
            limit=float(mlp["expert"]["limit"]), alpha=EXPERT_GATE_SLOPE))

    def run_order(self):
        """The layers in the order they run, every run with a cache layer of its own; the first
        layer of each pass over the looped layers takes the input mix."""
        n = len(self.layers)
        if self.loop is None:
            layers = [(i, None) for i in range(n)]
        else:
            a, b, times = int(self.loop["start"]), int(self.loop["stop"]), int(self.loop["times"])
            layers = [(i, None) for i in range(a)]
            for _ in range(times):
                layers += [(i, "loop.in" if i == a else None) for i in range(a, b)]
            layers += [(i, None) for i in range(b, n)]
        return tuple(RunStep(block=i, cache_layer=c, input_mix=mix) for c, (i, mix) in enumerate(layers))

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", dict(size=self.width, eps=self.eps, weight_name="", one_plus=True))
        blocks = []
        for i, layer in enumerate(self.layers):
            blocks.append(BlockSpec(
                kind="parallel", mixer=self._mixer(layer), feed_forward=self._mlp(layer.get("mlp")),
                norm_mixer=norm, norm_feed_forward=None, prefix=f"l{i}.",
                names=dict(mixer="mix.", feed_forward="mlp.", norm_mixer="norm1"),
                args=dict(branch_scale=self.residual_mult)))
        return ModelSpec(
            architecture="Gusorax", hidden_size=self.width, vocab_size=self.vocab, blocks=tuple(blocks),
            run_order=self.run_order(), final_norm=norm, embedding_name="embed", final_norm_name="final.norm",
            lm_head_name="head", max_position=self.max_positions, eos_token_ids=(),
            embedding_scale=self.embedding_scale, position_table_name="pos")
