"""Typed configuration of the Mobunex design and its model as data.

config.json keys: ``architecture`` ("Mobunex"), ``width``, ``vocab``, ``norm.eps``,
``postln_alpha`` and ``layers``, a list of entries with ``type`` ("attention", "rglru" or
"latent_attention"), ``mixer`` (the mixer's sizes and constants) and ``mlp`` (``{"kind":
"dense", "ff": n}``, ``{"kind": "moe", "expert": {"ff": n}, "router": {"experts", "top",
"groups": {"count", "keep"}}, "shared": {"ff": n}}`` or null).

Tensors: ``embed``, ``embed.norm``, ``final.norm``, ``head``; per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.dwa``, ``l<i>.mix.*`` and ``l<i>.mlp.*``.

Every norm of the stack is an RMS norm with one learned number as its gain.  The embedding row is
normed.  A layer normalises after each sum and its sublayers read the stream itself:
x <- n1(alpha x + mixer(x)), x <- n2(alpha x + mlp(x)); what it hands on is a learned mix of the
embedding output and every layer's result so far (``dwa``).  attention: grouped-query softmax
attention in a sliding window, biases on q, k, v, unit-RMS queries and keys, a learned
temperature per head, no rotation.  rglru: a gated diagonal linear recurrence (decay rate 8)
behind a short convolution, times a gelu branch.  latent_attention: softmax attention over a
compressed latent per token with a rotated key part shared by the heads (YaRN-scaled), a sliding
window and a sigmoid gate on every output value.  The routed feed-forward scores its experts
with a sigmoid, corrects the scores for the choice only, ranks groups by their two best, and adds
a shared expert.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .specs import BlockSpec, ConfigError, ModelSpec, PartSpec, RunStep

_LAYER_TYPES = ("attention", "rglru", "latent_attention")
_MLP_KINDS = ("dense", "moe")
RGLRU_RATE = 8.0          # log a = -RGLRU_RATE * r * softplus(lam): fixed by the design


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"{where} lacks {key!r}")
    return d[key]


def _positive(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


@dataclass
class MobunexConfig:
    width: int
    vocab: int
    eps: float
    alpha: float
    layers: List[dict]
    raw: Dict[str, Any]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MobunexConfig":
        cfg = cls(width=_positive(_need(d, "width", "config.json"), "width"),
                  vocab=_positive(_need(d, "vocab", "config.json"), "vocab"),
                  eps=float(_need(_need(d, "norm", "config.json"), "eps", "norm")),
                  alpha=float(_need(d, "postln_alpha", "config.json")),
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
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in _LAYER_TYPES:
                raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {', '.join(_LAYER_TYPES)}")
            m = _need(layer, "mixer", where)
            mw = where + ".mixer"
            if kind == "rglru":
                for key in ("width", "blocks", "conv"):
                    _positive(_need(m, key, mw), f"{mw}.{key}")
                if m["width"] % m["blocks"]:
                    raise ConfigError(f"{mw}: width must be a multiple of blocks")
                if m["conv"] > 16:
                    raise ConfigError(f"{mw}: at most 16 convolution taps are supported")
            elif kind == "attention":
                for key in ("heads", "dim", "vdim"):
                    _positive(_need(m, key, mw), f"{mw}.{key}")
                if m["heads"] % _positive(m.get("kv_heads", m["heads"]), f"{mw}.kv_heads"):
                    raise ConfigError(f"{mw}: heads must be a multiple of kv_heads")
                if m["dim"] > 256 or m["vdim"] > 256:
                    raise ConfigError(f"{mw}: heads are at most 256 wide")
                _need(m, "scale", mw)
                if m.get("mask") is not None:
                    _positive(_need(m["mask"], "size", mw + ".mask"), "mask.size")
            else:
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
                    _positive(_need(m, key, mw), f"{mw}.{key}")
                if m["rot_dim"] % 2:
                    raise ConfigError(f"{mw}.rot_dim must be even")
                if m["kv_rank"] > 512:
                    raise ConfigError(f"{mw}.kv_rank is at most 512")
                _need(m, "scale", mw)
                if m.get("mask") is not None:
                    _positive(_need(m["mask"], "size", mw + ".mask"), "mask.size")
                rot = _need(m, "rot", mw)
                dims = _positive(_need(rot, "dims", mw + ".rot"), "rot.dims")
                if dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"{mw}.rot.dims must be even and at most rot_dim")
                if not float(_need(rot, "base", mw + ".rot")) > 1:
                    raise ConfigError("rot.base must be larger than 1")
                sc = rot.get("scaling")
                if sc:
                    for key in ("factor", "original", "fast", "slow"):
                        if not float(_need(sc, key, mw + ".rot.scaling")) > 0:
                            raise ConfigError(f"rot.scaling.{key} must be positive")
                    if float(sc["factor"]) < 1:
                        raise ConfigError("rot.scaling.factor must be at least 1")
            mlp = layer.get("mlp")
            if mlp is not None:
                mk = mlp.get("kind", "dense")
                if mk not in _MLP_KINDS:
                    raise ConfigError(f"{where}.mlp.kind {mk!r} is not supported; known: {', '.join(_MLP_KINDS)}")
                if mk == "dense":
                    _positive(_need(mlp, "ff", where + ".mlp"), f"{where}.mlp.ff")
                else:
                    _positive(_need(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert"), "expert.ff")
                    r = _need(mlp, "router", where + ".mlp")
                    E = _positive(_need(r, "experts", where + ".mlp.router"), "router.experts")
                    top = _positive(_need(r, "top", where + ".mlp.router"), "router.top")
                    g = r.get("groups") or {}
                    count = _positive(g.get("count", 1), "router.groups.count")
                    keep = _positive(g.get("keep", count), "router.groups.keep")
                    if E % count or keep > count or top > keep * (E // count):
                        raise ConfigError(f"{where}.mlp.router: experts divide into equal groups, keep <= count, "
                                          "and the kept groups hold at least `top` experts")
                    if E > 512 or top > 32 or count > 64:
                        raise ConfigError(f"{where}.mlp.router: at most 512 experts, 32 chosen and 64 groups")
                    if mlp.get("shared"):
                        _positive(_need(mlp["shared"], "ff", where + ".mlp.shared"), "shared.ff")

    # ------------------------------------------------------------------ the model as data
    def _mixer(self, layer: dict) -> PartSpec:
        m = layer["mixer"]
        if layer["type"] == "rglru":
            return PartSpec("gated_linear_recurrence", dict(
                hidden_size=self.width, width=int(m["width"]), blocks=int(m["blocks"]), conv_taps=int(m["conv"]),
                rate=RGLRU_RATE, activation="gelu_tanh"))
        window = int(m["mask"]["size"]) if m.get("mask") is not None else None     # no mask: every earlier token
        if layer["type"] == "attention":
            return PartSpec("masked_attention", dict(
                hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m.get("kv_heads", m["heads"])),
                key_dim=int(m["dim"]), value_dim=int(m["vdim"]), scale=float(m["scale"]), eps=self.eps,
                mask="window" if window else None, mask_size=window, qk_norm="unit", proj_bias="qkv",
                head_temperature=True))
        rot = m["rot"]
        rotary = dict(base=float(rot["base"]), dims=int(rot["dims"]))
        if rot.get("scaling"):
            rotary["scaling"] = {k: float(rot["scaling"][k]) for k in ("factor", "original", "fast", "slow")}
        return PartSpec("latent_attention", dict(
            hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
            value_dim=int(m["vdim"]), kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), scale=float(m["scale"]),
            eps=self.eps, rotary=rotary, sink=False, out_gate="each", window=window))

    def _mlp(self, mlp: Optional[dict]) -> Optional[PartSpec]:
        if mlp is None:
            return None
        if mlp.get("kind", "dense") == "dense":
            return PartSpec("swiglu", dict(hidden_size=self.width, intermediate_size=int(mlp["ff"]),
                                           tensor_names=dict(gate="gate", up="up", down="down"), weight_suffix=""))
        r = mlp["router"]
        g = r.get("groups") or {}
        count = int(g.get("count", 1))
        shared = mlp.get("shared")
        return PartSpec("routed_experts", dict(
            hidden_size=self.width, intermediate_size=int(mlp["expert"]["ff"]), num_experts=int(r["experts"]),
            top=int(r["top"]), groups=count, keep=int(g.get("keep", count)), scale=1.0, router_score="sigmoid",
            correction=True, group_rank="top2_sum", shared_size=int(shared["ff"]) if shared else None))

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("scalar_rmsnorm", dict(size=self.width, eps=self.eps, weight_name=""))
        blocks = []
        for i, layer in enumerate(self.layers):
            ffn = self._mlp(layer.get("mlp"))
            blocks.append(BlockSpec(
                kind="postnorm", mixer=self._mixer(layer), feed_forward=ffn, norm_mixer=norm,
                norm_feed_forward=norm if ffn is not None else None, prefix=f"l{i}.",
                names=dict(mixer="mix.", feed_forward="mlp.", norm_mixer="norm1", norm_feed_forward="norm2",
                           depth_mix="dwa"),
                args=dict(alpha=self.alpha, depth_mix=True, depth_index=i)))
        run = tuple(RunStep(block=i, cache_layer=i) for i in range(len(self.layers)))
        return ModelSpec(
            architecture="Mobunex", hidden_size=self.width, vocab_size=self.vocab, blocks=tuple(blocks),
            run_order=run, final_norm=norm, embedding_name="embed", final_norm_name="final.norm",
            lm_head_name="head", max_position=1 << 30, eos_token_ids=(),
            embedding_norm=norm, embedding_norm_name="embed.norm", depth_stack="mix")
