"""Shared test data: tiny configurations and model-folder helpers."""
import json
import os

import torch

# Tiny configurations of the architecture that differ in every size and option.
TINY_A = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=64,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=160,
              vocab_size=320, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=4096, use_sliding_window=False, hidden_act="silu",
              eos_token_id=319)
TINY_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=192,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, intermediate_size=512,
              vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=2048, use_sliding_window=False, hidden_act="silu",
              eos_token_id=[998, 999])
# head_dim given and unequal to hidden/heads, three kv heads, a window on layers 1.., sizes
# that are no power of two
TINY_C = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=88,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
              intermediate_size=208, vocab_size=517, rope_theta=50000.0, rms_norm_eps=3e-6,
              tie_word_embeddings=False, max_position_embeddings=1024, use_sliding_window=True,
              sliding_window=24, max_window_layers=1, hidden_act="silu", eos_token_id=516)
# head size 64 (in bfloat16 its prompt portions run on the tcgen05 attention kernel), three
# query heads on one key/value head, a window on the second layer
TINY_D = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=96,
              num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=1, head_dim=64,
              intermediate_size=144, vocab_size=411, rope_theta=20000.0, rms_norm_eps=2e-6,
              tie_word_embeddings=True, max_position_embeddings=2048, use_sliding_window=True,
              sliding_window=150, max_window_layers=1, hidden_act="silu", eos_token_id=410)
TINY = {"A": (TINY_A, 0, 16, 8.0), "B": (TINY_B, 1, 8, 4.0), "C": (TINY_C, 2, 8, 6.0), "D": (TINY_D, 3, 16, 5.0)}


def make_model_folder(path, cfg: dict, seed: int, sharpen: float = 1.0, dtype=torch.bfloat16) -> str:
    """A model folder with seeded random weights through the engine's random-weights mode;
    ``sharpen`` scales the query and key projections so that attention is far from uniform
    and a wrong, missing or extra key changes the logits visibly."""
    from paged_batch_engine_b200.config import load_config
    from paged_batch_engine_b200.engine.runner import build_model
    from paged_batch_engine_b200.weights import write_random_model
    _, typed = load_config(cfg)
    model = build_model(typed, torch.float32, "cpu")
    write_random_model(str(path), typed, model.param_specs(), seed, dtype)
    if sharpen != 1.0:
        from safetensors.torch import load_file, save_file
        f = os.path.join(str(path), "model.safetensors")
        w = load_file(f)
        for k in list(w):
            if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
                w[k] = (w[k].float() * sharpen).to(w[k].dtype)
        save_file(w, f)
    return str(path)


def load_plain(folder: str):
    """config.json as a dict and the weights as float32 tensors, read without the engine."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, w




# ---------------------------------------------------------------- Gebadra: tiny configurations
def _lin(heads, dim, vdim, decay):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))


def _soft(heads, kv, dim, vdim, window, pool, rot_dims, base, factor, scale):
    rot = dict(base=base, dims=rot_dims)
    if factor is not None:
        rot["scaling"] = dict(factor=factor)
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, mask=dict(size=window, pool=pool), rot=rot,
                scale=scale)


# three residual streams, one key/value head, a rotation on half of each head, a layer that runs
# another's tensors (of each type), widths that differ between keys and values
GEB_A = dict(
    architecture="Gebadra", width=64, vocab=300, streams=3, norm=dict(eps=1e-5),
    layers=[
        dict(type="lightning", mixer=_lin(2, 16, 24, [0.9, 0.99]), mlp=dict(kind="dense", ff=96)),
        dict(type="parallel", mixer=dict(left=_soft(4, 1, 32, 16, 20, 4, 16, 10000.0, 2.0, 0.2),
                                         right=_lin(2, 16, 32, [0.8, 0.97])), mlp=dict(kind="dense", ff=80)),
        dict(type="lightning", mixer=_lin(2, 16, 24, [0.9, 0.99]), mlp=dict(kind="dense", ff=96), weights_of=0),
        dict(type="parallel", mixer=dict(left=_soft(4, 1, 32, 16, 20, 4, 16, 10000.0, 2.0, 0.2),
                                         right=_lin(2, 16, 32, [0.8, 0.97])), mlp=dict(kind="dense", ff=80),
             weights_of=1),
    ])
# the plain residual sum (no streams key), a window shorter than a block, as many key/value heads as
# heads, no scaling of the rotation, a layer without feed-forward, one head
GEB_B = dict(
    architecture="Gebadra", width=96, vocab=211, norm=dict(eps=1e-6),
    layers=[
        dict(type="parallel", mixer=dict(left=_soft(3, 3, 24, 40, 7, 8, 24, 500.0, None, 0.3),
                                         right=_lin(3, 40, 8, [0.5, 0.9, 0.999])), mlp=dict(kind="dense", ff=64)),
        dict(type="lightning", mixer=_lin(1, 48, 64, [0.95]), mlp=None),
    ])
# one stream with its own connection tensors, blocks as long as a page, keys wider than 128 in the
# recurrence, a window that is no multiple of anything
GEB_C = dict(
    architecture="Gebadra", width=128, vocab=257, streams=1, norm=dict(eps=1e-6),
    layers=[
        dict(type="lightning", mixer=_lin(2, 160, 16, [0.9, 0.98]), mlp=dict(kind="dense", ff=72)),
        dict(type="parallel", mixer=dict(left=_soft(6, 2, 64, 64, 33, 16, 32, 100000.0, 4.0, 0.125),
                                         right=_lin(4, 24, 40, [0.7, 0.9, 0.97, 0.995])),
             mlp=dict(kind="dense", ff=72)),
    ])
GEBADRA = {"A": (GEB_A, 11, 8), "B": (GEB_B, 12, 8), "C": (GEB_C, 13, 16)}     # config, seed, page tokens


def make_gebadra_folder(path, cfg: dict, seed: int, dtype=torch.bfloat16) -> str:
    """A model folder with seeded random weights through the engine's random-weights mode, then
    reshaped so that no mechanism is a near-identity: projections large enough for sharp softmaxes
    and gates away from one half, stream mixtures and head mixtures with off-diagonal weight."""
    from paged_batch_engine_b200.config import load_config
    from paged_batch_engine_b200.engine.runner import build_model
    from paged_batch_engine_b200.weights import write_random_model
    from safetensors.torch import load_file, save_file
    _, typed = load_config(cfg)
    model = build_model(typed, torch.float32, "cpu")
    write_random_model(str(path), typed, model.param_specs(), seed, dtype)
    f = os.path.join(str(path), "model.safetensors")
    w = load_file(f)
    g = torch.Generator().manual_seed(seed)
    for k in list(w):
        t = w[k].float()
        leaf = k.split(".")[-1]
        if k.endswith(".mix") and ".hc" in k:
            t = torch.eye(t.shape[0]) * 0.8 + torch.randn(t.shape, generator=g) * 0.15
        elif leaf in ("in", "out") and ".hc" in k:
            t = 0.6 + 0.3 * torch.rand(t.shape, generator=g)
        elif leaf == "talk":
            t = torch.eye(t.shape[0]) * 0.7 + torch.randn(t.shape, generator=g) * 0.2
        elif leaf in ("q", "k") and t.dim() == 2:
            t = t * 6.0
        elif leaf in ("v", "g", "o", "gate", "up", "down") and t.dim() == 2:
            t = t * 1.5
        elif leaf == "b":
            t = torch.randn(t.shape, generator=g) * 0.1
        elif k == "head":
            t = t * 5.0
        w[k] = t.to(w[k].dtype)
    save_file(w, f)
    return str(path)


# ---------------------------------------------------------------- Bavetar: tiny configurations
def _lat(heads, dim, rot_dim, rot_dims, vdim, kv_rank, q_rank, base, scale):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale,
                rot=dict(base=base, dims=rot_dims))


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def _moe(ff, experts, top, count, keep, scale):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale,
                                                            groups=dict(count=count, keep=keep)))


# three heads (the rows of a tile straddle tokens), all head widths different, only half of the rotated
# part turns, one group of experts (no restriction), a layer without feed-forward, one state group and
# as many as heads, two and four convolution taps
BAV_A = dict(
    architecture="Bavetar", width=64, vocab=300, norm=dict(eps=1e-5), logit_scale=0.7, logit_softcap=9.0,
    layers=[
        dict(type="latent_attention", mixer=_lat(3, 16, 8, 4, 24, 40, 24, 10000.0, 0.25), mlp=dict(kind="dense", ff=96)),
        dict(type="mamba2", mixer=_ssm(4, 16, 24, 1, 4, 4), mlp=_moe(48, 6, 2, 1, 1, 1.0)),
        dict(type="latent_attention", mixer=_lat(3, 16, 8, 4, 24, 40, 24, 10000.0, 0.25), mlp=None),
        dict(type="mamba2", mixer=_ssm(2, 40, 80, 2, 2, 1), mlp=dict(kind="dense", ff=72)),
    ])
# twenty heads (more than a block's packed rows), five groups of two experts of which two are kept,
# a state-space layer without feed-forward, three taps, no cap on the logits
BAV_B = dict(
    architecture="Bavetar", width=96, vocab=211, norm=dict(eps=1e-6), logit_scale=2.0,
    layers=[
        dict(type="mamba2", mixer=_ssm(6, 8, 16, 3, 3, 2), mlp=None),
        dict(type="latent_attention", mixer=_lat(20, 8, 4, 4, 8, 20, 16, 500.0, 0.3), mlp=_moe(40, 10, 3, 5, 2, 1.5)),
        dict(type="latent_attention", mixer=_lat(20, 8, 4, 4, 8, 20, 16, 500.0, 0.3), mlp=dict(kind="dense", ff=64)),
    ])
# one expert chosen from the one kept group, a state wider than 128, a single tap (no convolution
# state), eight norm groups, a value wider than the latent
BAV_C = dict(
    architecture="Bavetar", width=128, vocab=257, norm=dict(eps=1e-6), logit_scale=1.0, logit_softcap=30.0,
    layers=[
        dict(type="latent_attention", mixer=_lat(8, 32, 16, 16, 56, 48, 40, 100000.0, 0.15), mlp=_moe(24, 8, 1, 4, 1, 2.5)),
        dict(type="mamba2", mixer=_ssm(8, 8, 130, 4, 1, 8), mlp=dict(kind="dense", ff=72)),
        dict(type="mamba2", mixer=_ssm(4, 24, 32, 4, 4, 2), mlp=_moe(32, 9, 4, 3, 2, 1.0)),
    ])
BAVETAR = {"A": (BAV_A, 21, 8), "B": (BAV_B, 22, 16), "C": (BAV_C, 23, 8)}     # config, seed, page tokens


def make_bavetar_folder(path, cfg: dict, seed: int, dtype=torch.bfloat16) -> str:
    """A model folder with seeded random weights through the engine's random-weights mode, then
    reshaped so that no mechanism is a near-identity: projections large enough for sharp softmaxes,
    decisive routers and gates away from one half; sinks, decay rates, step-size biases and skip
    terms spread over a range."""
    from paged_batch_engine_b200.config import load_config
    from paged_batch_engine_b200.engine.runner import build_model
    from paged_batch_engine_b200.weights import write_random_model
    from safetensors.torch import load_file, save_file
    _, typed = load_config(cfg)
    model = build_model(typed, torch.float32, "cpu")
    write_random_model(str(path), typed, model.param_specs(), seed, dtype)
    f = os.path.join(str(path), "model.safetensors")
    w = load_file(f)
    g = torch.Generator().manual_seed(seed)
    for k in list(w):
        t = w[k].float()
        leaf = k.split("mix.")[-1] if ".mix." in k else k.split(".")[-1]
        latent = k.split(".")[0] + ".mix.uv" in w
        if leaf in ("dq", "dkv", "uq", "uk", "in") and t.dim() == 2:
            t = t * 6.0
        elif leaf in ("uv", "o", "g") and t.dim() == 2:
            t = t * (12.0 if latent else 4.0)
        elif leaf in ("up", "down", "gate") and t.dim() == 2:
            t = t * 4.5
        elif leaf == "router":
            t = t * 40.0
        elif leaf == "sink":
            t = torch.randn(t.shape, generator=g) * 2.0
        elif leaf == "A_log":
            t = torch.log(0.05 + 2.0 * torch.rand(t.shape, generator=g))
        elif leaf == "dt_bias":
            t = torch.randn(t.shape, generator=g) * 1.5 - 1.0
        elif leaf == "D":
            t = torch.randn(t.shape, generator=g)
        elif leaf == "conv":
            t = torch.randn(t.shape, generator=g) * 0.6
        elif leaf == "conv.b":
            t = torch.randn(t.shape, generator=g) * 0.2
        elif k == "embed":
            t = t * 30.0
        w[k] = t.to(w[k].dtype)
    save_file(w, f)
    return str(path)
# one kind of layer only: a model without any paged cache, and one without any state row
BAV_STATE_ONLY = dict(
    architecture="Bavetar", width=48, vocab=150, norm=dict(eps=1e-5), logit_scale=1.5, logit_softcap=20.0,
    layers=[dict(type="mamba2", mixer=_ssm(3, 8, 12, 3, 2, 3), mlp=dict(kind="dense", ff=40)),
            dict(type="mamba2", mixer=_ssm(2, 16, 20, 1, 5, 1), mlp=None)])
BAV_LATENT_ONLY = dict(
    architecture="Bavetar", width=56, vocab=170, norm=dict(eps=1e-5), logit_scale=1.0, logit_softcap=12.0,
    layers=[dict(type="latent_attention", mixer=_lat(2, 12, 6, 6, 20, 26, 10, 3000.0, 0.2), mlp=None),
            dict(type="latent_attention", mixer=_lat(5, 8, 8, 8, 8, 16, 12, 3000.0, 0.3), mlp=_moe(16, 4, 2, 2, 1, 1.0))])


# ---------------------------------------------------------------- Gusorax: tiny configurations
def _win(heads, kv, dim, vdim, size, far, rows, scale):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, mask=dict(size=size), bias_max=far,
                bias_rows=rows)


def _chk(heads, kv, dim, vdim, size, scale):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, mask=dict(size=size))


def _gmoe(ff, limit, experts, top):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))


# a layer ahead of the loop and one after it, the loop runs two layers twice; three query heads on one
# key/value head (a block's rows straddle tokens); head widths that are no multiples of 16 (the
# float32-arithmetic kernel in bfloat16 too); windows and chunks that are no multiples of the page; a
# layer without feed-forward; a bias table whose far end lies beyond the window
GUS_A = dict(
    architecture="Gusorax", width=64, vocab=300, max_positions=512, norm=dict(eps=1e-5), embedding=dict(scale=3.0),
    residual_mult=0.5, loop=dict(start=1, stop=3, times=2),
    layers=[
        dict(type="attention", mixer=_win(3, 1, 24, 40, 21, 37.0, 12, 0.2), mlp=dict(kind="dense", ff=96)),
        dict(type="attention_2", mixer=_chk(4, 2, 24, 20, 13, 0.25), mlp=_gmoe(48, 1.2, 6, 2)),
        dict(type="attention", mixer=_win(6, 3, 8, 8, 50, 30.0, 8, 0.35), mlp=None),
        dict(type="attention_2", mixer=_chk(2, 2, 40, 24, 30, 0.15), mlp=dict(kind="dense", ff=72)),
    ])
# no loop at all; as many key/value heads as query heads; head widths on the tensor-core path with
# unequal key and value widths; a window of one token (a row sees itself only) and chunks of one; one
# expert chosen; multiplier one
GUS_B = dict(
    architecture="Gusorax", width=96, vocab=211, max_positions=400, norm=dict(eps=1e-6), embedding=dict(scale=1.0),
    residual_mult=1.0,
    layers=[
        dict(type="attention", mixer=_win(4, 4, 32, 16, 1, 9.0, 4, 0.3), mlp=_gmoe(40, 0.8, 5, 1)),
        dict(type="attention_2", mixer=_chk(5, 5, 16, 48, 64, 0.3), mlp=dict(kind="dense", ff=64)),
        dict(type="attention_2", mixer=_chk(2, 1, 32, 32, 1, 0.2), mlp=None),
        dict(type="attention", mixer=_win(8, 2, 16, 32, 77, 300.0, 20, 0.25), mlp=_gmoe(24, 2.0, 4, 4)),
    ])
# the loop covers every layer and runs three times; sixteen query heads on two key/value heads; a
# window longer than any test sequence; heads of 80 and 128 (unequal, tensor cores); every expert chosen
GUS_C = dict(
    architecture="Gusorax", width=128, vocab=257, max_positions=640, norm=dict(eps=3e-6), embedding=dict(scale=11.0),
    residual_mult=0.25, loop=dict(start=0, stop=2, times=3),
    layers=[
        dict(type="attention", mixer=_win(16, 2, 80, 128, 600, 450.0, 16, 0.11), mlp=_gmoe(32, 3.0, 3, 3)),
        dict(type="attention_2", mixer=_chk(8, 1, 48, 16, 40, 0.14), mlp=dict(kind="dense", ff=80)),
    ])
GUSORAX = {"A": (GUS_A, 41, 8), "B": (GUS_B, 42, 16), "C": (GUS_C, 43, 8)}     # config, seed, page tokens


def make_gusorax_folder(path, cfg: dict, seed: int, dtype=torch.bfloat16) -> str:
    """A model folder with seeded random weights through the engine's random-weights mode, then
    reshaped so that no mechanism is a near-identity: query and key projections large enough for
    sharp softmaxes, bias tables that matter beside the scores, gains away from one, projection
    biases and gates away from one half, decisive routers, experts that reach their limits."""
    from paged_batch_engine_b200.config import load_config
    from paged_batch_engine_b200.engine.runner import build_model
    from paged_batch_engine_b200.weights import write_random_model
    from safetensors.torch import load_file, save_file
    _, typed = load_config(cfg)
    model = build_model(typed, torch.float32, "cpu")
    write_random_model(str(path), typed, model.param_specs(), seed, dtype)
    f = os.path.join(str(path), "model.safetensors")
    w = load_file(f)
    g = torch.Generator().manual_seed(seed)
    for k in list(w):
        t = w[k].float()
        leaf = k.split(".mix.")[-1] if ".mix." in k else k.split(".")[-1]
        if leaf in ("q", "k") and t.dim() == 2:
            t = t * 5.0
        elif leaf in ("q.norm", "k.norm"):
            t = 2.5 + 0.8 * torch.randn(t.shape, generator=g)
        elif leaf == "rel":
            t = torch.randn(t.shape, generator=g) * 2.0
        elif leaf in ("v", "o", "g") and t.dim() == 2:
            t = t * 4.0
        elif leaf == "b" or k.endswith(".b"):
            t = torch.randn(t.shape, generator=g) * 0.7
        elif leaf in ("up", "down", "gate") and t.dim() == 2:
            t = t * 4.5
        elif leaf == "router":
            t = t * 40.0
        elif leaf in ("norm1", "norm"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif k == "pos":
            t = torch.randn(t.shape, generator=g) * 0.5
        elif k == "embed":
            t = t * 20.0
        elif k == "loop.in":
            t = t * 3.0
        w[k] = t.to(w[k].dtype)
    save_file(w, f)
    return str(path)


# ---------------------------------------------------------------- Mobunex: tiny configurations
def _mwin(heads, kv, dim, vdim, size, scale):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, mask=dict(size=size))


def _mlat(heads, dim, rot_dim, rot_dims, vdim, kv_rank, q_rank, base, scale, size, scaling=None):
    rot = dict(base=base, dims=rot_dims)
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale,
                mask=dict(size=size), rot=rot)


def _mrec(width, blocks, conv):
    return dict(width=width, blocks=blocks, conv=conv)


def _mmoe(ff, experts, top, count, keep, shared=None):
    d = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, groups=dict(count=count, keep=keep)))
    if shared:
        d["shared"] = dict(ff=shared)
    return d


# four query heads on two key heads with values wider than keys and a window off the page grid; three
# gate blocks and four taps; three groups of two experts of which two are kept, with a shared expert; a
# latent layer without feed-forward whose slow pairs are stretched eightfold; one gate block, two taps
MOB_A = dict(
    architecture="Mobunex", width=64, vocab=300, norm=dict(eps=1e-5), postln_alpha=1.5,
    layers=[
        dict(type="attention", mixer=_mwin(4, 2, 16, 24, 21, 0.3), mlp=dict(kind="dense", ff=96)),
        dict(type="rglru", mixer=_mrec(48, 3, 4), mlp=_mmoe(40, 6, 2, 3, 2, shared=24)),
        dict(type="latent_attention", mixer=_mlat(3, 16, 8, 8, 24, 40, 24, 10000.0, 0.25, 40, (8.0, 64, 16.0, 2.0)),
             mlp=None),
        dict(type="rglru", mixer=_mrec(80, 1, 2), mlp=dict(kind="dense", ff=72)),
    ])
# alpha 1; a recurrent layer first, with a single tap (no convolution state) and no feed-forward; twenty
# latent heads, only half of whose rotated part turns, no frequency scaling, a window of four whole
# pages; five groups of two experts, no shared expert; as many key heads as query heads and a window
# longer than any request
MOB_B = dict(
    architecture="Mobunex", width=96, vocab=211, norm=dict(eps=1e-6), postln_alpha=1.0,
    layers=[
        dict(type="rglru", mixer=_mrec(96, 6, 1), mlp=None),
        dict(type="latent_attention", mixer=_mlat(20, 8, 4, 2, 8, 20, 16, 500.0, 0.3, 64), mlp=_mmoe(40, 10, 3, 5, 2)),
        dict(type="attention", mixer=_mwin(6, 6, 32, 16, 600, 0.2), mlp=dict(kind="dense", ff=64)),
    ])
# eight query heads on one key head, heads of 64 (the tensor-core path in bfloat16), a window of 17;
# groups of ONE expert and one expert chosen; a value wider than the latent; nine experts in three
# groups, four chosen from two; five layers, so the depth mix reaches six terms
MOB_C = dict(
    architecture="Mobunex", width=128, vocab=257, norm=dict(eps=1e-6), postln_alpha=3.0,
    layers=[
        dict(type="attention", mixer=_mwin(8, 1, 64, 64, 17, 0.11), mlp=_mmoe(24, 8, 1, 8, 3, shared=48)),
        dict(type="latent_attention", mixer=_mlat(8, 32, 16, 16, 56, 48, 40, 100000.0, 0.15, 33, (2.5, 32, 16.0, 2.0)),
             mlp=_mmoe(32, 9, 4, 3, 2, shared=16)),
        dict(type="rglru", mixer=_mrec(144, 4, 3), mlp=dict(kind="dense", ff=72)),
        dict(type="attention", mixer=_mwin(2, 2, 24, 40, 1, 0.5), mlp=None),
        dict(type="rglru", mixer=_mrec(40, 5, 2), mlp=None),
    ])
MOBUNEX = {"A": (MOB_A, 51, 8), "B": (MOB_B, 52, 16), "C": (MOB_C, 53, 8)}     # config, seed, page tokens


def make_mobunex_folder(path, cfg: dict, seed: int, dtype=torch.bfloat16, gain: float = 1.0) -> str:
    """A model folder with seeded random weights through the engine's random-weights mode, then
    reshaped so that no mechanism is a near-identity: projections large enough that every sublayer
    matters beside the skip path, sharp softmaxes, temperatures, gate biases and decay rates spread
    over a range, routers that decide and corrections that change the choice, depth mixes far from
    "the last result only".  ``gain`` scales the matrices' factors (wide models need less)."""
    from paged_batch_engine_b200.config import load_config
    from paged_batch_engine_b200.engine.runner import build_model
    from paged_batch_engine_b200.weights import write_random_model
    from safetensors.torch import load_file, save_file
    _, typed = load_config(cfg)
    model = build_model(typed, torch.float32, "cpu")
    write_random_model(str(path), typed, model.param_specs(), seed, dtype)
    f = os.path.join(str(path), "model.safetensors")
    w = load_file(f)
    g = torch.Generator().manual_seed(seed)
    for k in list(w):
        t = w[k].float()
        leaf = k.split(".mix.")[-1] if ".mix." in k else k.split(".")[-1]
        if k.endswith(".b"):
            t = torch.randn(t.shape, generator=g) * 0.5
        elif leaf in ("q", "k", "dq", "dkv", "uq", "uk", "x", "y") and t.dim() == 2:
            t = t * 6.0 * gain
        elif leaf in ("v", "o", "g", "uv") and t.dim() == 2:
            t = t * 6.0 * gain
        elif leaf in ("ra", "ri"):
            t = t * 12.0 * gain
        elif leaf == "temp":
            t = 0.5 + 1.5 * torch.rand(t.shape, generator=g)
        elif leaf == "lam":
            t = torch.randn(t.shape, generator=g) * 1.5 - 1.0
        elif leaf == "conv":
            t = torch.randn(t.shape, generator=g) * 0.6
        elif leaf in ("up", "down", "gate") and t.dim() == 2:
            t = t * 4.5 * gain
        elif leaf == "router":
            t = t * 12.0 * gain
        elif leaf == "correction":
            t = torch.randn(t.shape, generator=g) * 0.3
        elif leaf == "dwa":
            t = torch.randn(t.shape, generator=g) * 0.6
            t[-1] = 1.0
        elif k == "head":
            t = t * 8.0
        w[k] = t.to(w[k].dtype)
    save_file(w, f)
    return str(path)
