"""Python faces of the CUDA entry points: each takes torch tensors on a CUDA device,
checks what the kernel assumes, and launches on the current stream.

There is no CPU path and no library stand-in for any of these: a tensor that is not on
a CUDA device is an error, and so is a failed build of the kernel library.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else c_void_p(t.data_ptr())


def _stream():
    # the raw handle of the current stream, without building a torch.cuda.Stream object per launch
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("this engine runs on CUDA devices only: got a tensor on " + str(t.device))


def _need_contiguous(*tensors):
    for t in tensors:
        if t is not None and not t.is_contiguous():
            raise KernelError("kernel operands must be contiguous")


_launches = 0


def launch_count() -> int:
    """Kernel launches of this package issued from Python so far (a captured graph's
    launches count once, at capture)."""
    return _launches


def count_launches(n: int) -> None:
    """Launches made on this package's behalf by the host library."""
    global _launches
    _launches += int(n)


def _check(code: int, what: str):
    global _launches
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")
    _launches += 1




_fns = {}


def _fn(lib_name, fn_name, argtypes, defines=None):
    key = (lib_name, fn_name, tuple(sorted(defines.items())) if defines else None)
    fn = _fns.get(key)
    if fn is None:
        lib = load_library(lib_name, defines)
        fn = getattr(lib, fn_name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _fns[key] = fn
    return fn


# ------------------------------------------------------------------ elementwise
def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] as float32.  ids: int32 [T]."""
    _need_cuda(out, table, ids)
    _need_contiguous(out, table, ids)
    if out.dtype != torch.float32 or ids.dtype != torch.int32:
        raise KernelError("embedding writes float32 rows from int32 ids")
    T, d = out.shape
    if table.shape[1] != d or ids.numel() != T:
        raise KernelError("embedding: shapes do not agree")
    fn = _fn("elementwise", "pbe_embedding",
             [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(out), _ptr(table), _dtype_code(table), _ptr(ids), T, d, table.shape[0], _stream()),
           "embedding")
    return out


def embedding_positions(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float,
                        pos_table: Optional[torch.Tensor], positions: Optional[torch.Tensor]) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] * scale + pos_table[positions[t], :] as float32 (the position row is
    not scaled; ``pos_table`` None: no position row)."""
    _need_cuda(out, table, ids, pos_table, positions)
    _need_contiguous(out, table, ids, pos_table, positions)
    if out.dtype != torch.float32 or ids.dtype != torch.int32:
        raise KernelError("embedding writes float32 rows from int32 ids")
    T, d = out.shape
    if table.shape[1] != d or ids.numel() != T:
        raise KernelError("embedding: shapes do not agree")
    if pos_table is not None and (pos_table.dtype != table.dtype or pos_table.shape[1] != d or positions is None
                                  or positions.dtype != torch.int32 or positions.numel() != T):
        raise KernelError("embedding: the position table has the embedding's dtype and width, positions are int32 [T]")
    fn = _fn("elementwise", "pbe_embedding_pos",
             [c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(out), _ptr(table), _dtype_code(table), _ptr(ids), float(scale), _ptr(pos_table), _ptr(positions),
              pos_table.shape[0] if pos_table is not None else 0, T, d, table.shape[0], _stream()), "embedding_pos")
    return out


def fold_pair(residual: torch.Tensor, delta_a: Optional[torch.Tensor], delta_b: Optional[torch.Tensor],
              delta_scale: float, first: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """[residual + delta_scale * (delta_a + delta_b) | first] as rows of twice the width in ``out_dtype``
    (either delta may be None); residual and ``first`` are float32 [T, W]."""
    _need_cuda(residual, delta_a, delta_b, first)
    _need_contiguous(residual, delta_a, delta_b, first)
    if residual.dtype != torch.float32 or first.dtype != torch.float32 or first.shape != residual.shape \
            or residual.dim() != 2:
        raise KernelError("fold_pair: the residual and the first rows are float32 [T, W]")
    deltas = [x for x in (delta_a, delta_b) if x is not None]
    for x in deltas:
        if x.shape != residual.shape or x.dtype != deltas[0].dtype:
            raise KernelError("fold_pair: the deltas have the residual's shape and one dtype")
    T, d = residual.shape
    out = torch.empty((T, 2 * d), dtype=out_dtype, device=residual.device)
    fn = _fn("elementwise", "pbe_fold_pair", [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int,
                                              c_int, c_int, c_void_p])
    _check(fn(_ptr(residual), _ptr(delta_a), _ptr(delta_b), _dtype_code(deltas[0]) if deltas else F32,
              float(delta_scale), _ptr(first), _ptr(out), _dtype_code(out), T, d, _stream()), "fold_pair")
    return out


GLU_ACTIVATIONS = {"silu": 0, "capped_swish": 1}


def gated_activation(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu", limit: float = 0.0,
                     alpha: float = 1.0) -> torch.Tensor:
    """out[r, c] = act(gate_up[r, c], gate_up[r, inter + c]).  "silu": silu(g) * u.  "capped_swish":
    g <- min(g, limit), u <- clamp(u, -limit, limit), g * sigmoid(alpha * g) * (u + 1)."""
    if activation == "silu":
        return silu_mul(gate_up, out)
    _need_cuda(gate_up, out)
    _need_contiguous(gate_up, out)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("gated_activation: shapes or dtypes do not agree")
    fn = _fn("elementwise", "pbe_glu_act", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p])
    _check(fn(_ptr(gate_up), _ptr(out), _dtype_code(out), rows, two_i // 2, GLU_ACTIVATIONS[activation], float(limit),
              float(alpha), _stream()), "gated_activation")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor,
                out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual += delta (float32, in place) and out = rmsnorm(residual) * gain.

    With ``rows`` (int32 [n]) output row i is made from batch row rows[i] and the residual
    is not written."""
    _need_cuda(residual, delta, gain, out, rows)
    _need_contiguous(residual, delta, gain, out, rows)
    if residual.dtype != torch.float32 or gain.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream and the gain are float32")
    d = residual.shape[-1]
    n = out.shape[0] if out.dim() == 2 else 1
    if gain.numel() != d or out.shape[-1] != d or (delta is not None and delta.shape != residual.shape):
        raise KernelError("add_rmsnorm: shapes do not agree")
    if rows is None and n != residual.shape[0]:
        raise KernelError("add_rmsnorm: output rows do not match the batch")
    if rows is not None and (rows.dtype != torch.int32 or rows.numel() != n):
        raise KernelError("add_rmsnorm: rows must be int32, one per output row")
    if d * 4 > 200 * 1024:
        raise KernelError(f"add_rmsnorm: a row of {d} floats does not fit in shared memory")
    fn = _fn("elementwise", "pbe_add_rmsnorm",
             [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float,
              c_void_p])
    _check(fn(_ptr(residual), _ptr(delta), _dtype_code(delta) if delta is not None else F32,
              _ptr(gain), _ptr(out), _dtype_code(out), _ptr(rows), n, d, float(eps), _stream()),
           "add_rmsnorm")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, inter + c]."""
    _need_cuda(gate_up, out)
    _need_contiguous(gate_up, out)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("silu_mul: shapes or dtypes do not agree")
    fn = _fn("elementwise", "pbe_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(gate_up), _ptr(out), _dtype_code(out), rows, two_i // 2, _stream()), "silu_mul")
    return out


# ------------------------------------------------------------------ residual streams, norms of branches
def stream_norm(streams: torch.Tensor, y: Optional[torch.Tensor], mix: torch.Tensor, beta: torch.Tensor,
                alpha: torch.Tensor, gain: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, rms: bool = False) -> torch.Tensor:
    """Folds the pending sublayer output ``y`` into the residual streams (float32 [T, S, W], in
    place: r'_j = sum_s mix[s, j] r_s + beta[j] y), collapses them with ``alpha`` and writes the
    LayerNorm (``gain``, ``bias``) or RMSNorm (``rms``) of the collapsed rows to ``out``.  With
    ``rows`` (int32 [n]) output row i is made from batch row rows[i] and the streams are left
    alone.  ``y`` None: nothing is folded in."""
    _need_cuda(streams, y, mix, beta, alpha, gain, bias, out, rows)
    _need_contiguous(streams, y, mix, beta, alpha, gain, bias, out, rows)
    if streams.dtype != torch.float32 or streams.dim() != 3:
        raise KernelError("stream_norm: the residual streams are float32 [T, S, W]")
    T, S, W = streams.shape
    n = out.shape[0]
    for name, t, size in (("mix", mix, S * S), ("beta", beta, S), ("alpha", alpha, S), ("gain", gain, W)):
        if t.dtype != torch.float32 or t.numel() != size:
            raise KernelError(f"stream_norm: {name} must be float32 with {size} elements")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != W):
        raise KernelError("stream_norm: bias must be float32 [W]")
    if out.shape[-1] != W or (y is not None and tuple(y.shape) != (T, W)):
        raise KernelError("stream_norm: shapes do not agree")
    if rows is None and n != T:
        raise KernelError("stream_norm: output rows do not match the batch")
    if rows is not None and (rows.dtype != torch.int32 or rows.numel() != n):
        raise KernelError("stream_norm: rows must be int32, one per output row")
    if S > 8 or W * 4 > 200 * 1024:
        raise KernelError(f"stream_norm takes at most 8 streams and rows of at most 51,200 floats (got {S}, {W})")
    fn = _fn("streams", "pbe_stream_norm",
             [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
              c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_ptr(streams), _ptr(y), _dtype_code(y) if y is not None else F32, _ptr(mix), _ptr(beta), _ptr(alpha),
              _ptr(gain), _ptr(bias), _ptr(out), _dtype_code(out), _ptr(rows), n, S, W, float(eps),
              1 if rms else 0, _stream()), "stream_norm")
    return out


def branch_rms_mean(branches, gains, eps: float) -> torch.Tensor:
    """mean over the branches of x_b / rms(x_b) * gain_b, row by row; up to four branches of
    equal shape [T, W] and dtype; gains float32 [W]."""
    n = len(branches)
    if not 1 <= n <= 4 or len(gains) != n:
        raise KernelError("branch_rms_mean takes one to four branches and a gain for each")
    _need_cuda(*branches, *gains)
    _need_contiguous(*branches, *gains)
    T, W = branches[0].shape
    for x, g in zip(branches, gains):
        if x.shape != (T, W) or x.dtype != branches[0].dtype or g.dtype != torch.float32 or g.numel() != W:
            raise KernelError("branch_rms_mean: shapes or dtypes do not agree")
    out = torch.empty_like(branches[0])
    xs = (c_void_p * 4)(*[x.data_ptr() for x in branches])
    gs = (c_void_p * 4)(*[g.data_ptr() for g in gains])
    fn = _fn("streams", "pbe_branch_rms_mean", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float,
                                                c_void_p])
    _check(fn(ctypes.addressof(xs), ctypes.addressof(gs), n, _ptr(out), _dtype_code(out), T, W, float(eps),
              _stream()), "branch_rms_mean")
    return out


def gated_rms(o: torch.Tensor, gate: torch.Tensor, gain: Optional[torch.Tensor], heads: int, eps: float,
              per_head: bool, gate_act: str, out_dtype: torch.dtype, gate_first: bool = False) -> torch.Tensor:
    """out = o / rms(o) (* gain) * act(gate): ``o`` float32 [T, heads * E]; the root mean square
    over the whole row or over each head's E values; ``gate`` a column slice [T, heads * E] of a
    wider matrix (unit column stride); ``gate_act`` "sigmoid" or "silu".  ``gate_first``: out =
    u / rms(u) (* gain) with u = o * act(gate), the gate inside the norm."""
    _need_cuda(o, gate, gain)
    _need_contiguous(o, gain)
    T, N = o.shape
    if o.dtype != torch.float32 or N % heads or tuple(gate.shape) != (T, N) or gate.stride(1) != 1:
        raise KernelError("gated_rms: shapes, strides or dtypes do not agree")
    if gate.dtype != out_dtype:
        raise KernelError("gated_rms: the gate has the output's dtype")
    if gain is not None and (gain.dtype != torch.float32 or gain.numel() != N):
        raise KernelError("gated_rms: gain must be float32 [heads * E]")
    if gate_act not in ("sigmoid", "silu"):
        raise KernelError(f"gated_rms: unknown gate activation {gate_act!r}")
    out = torch.empty((T, N), dtype=out_dtype, device=o.device)
    fn = _fn("streams", "pbe_gated_rms", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_float, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(o), _ptr(gate), gate.stride(0) if T > 1 else N, _ptr(gain), _ptr(out), _dtype_code(out), T, heads,
              N // heads, float(eps), 1 if per_head else 0, 1 if gate_act == "silu" else 0, 1 if gate_first else 0,
              _stream()), "gated_rms")
    return out


# ------------------------------------------------------------------ linear attention (decayed recurrence)
def _column_slice(x: torch.Tensor, what: str):
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError(f"{what}: operands are column slices of a row-major matrix")


def linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, decay: torch.Tensor,
                     q_start: torch.Tensor, q_len: torch.Tensor, slots: torch.Tensor, num_requests: int,
                     heads: int, k_scale: float = 1.0, silu: bool = False, plan=None,
                     tok_decay: Optional[torch.Tensor] = None, tok_scale: Optional[torch.Tensor] = None,
                     skip: Optional[torch.Tensor] = None, kq_share: int = 1) -> torch.Tensor:
    """o_t = S_t^T q_t with S_t = decay_h S_{t-1} + k_t v_t^T per head, request by request over
    the rows each brings (``q_start``, ``q_len`` int32 [R]); ``state`` float32 [slots, H, D, E]
    is read at ``slots[r]`` and left updated.  q, k [T, H*D] and v [T, H*E] are column slices of
    one projection matrix (equal row stride).  ``plan`` (a ``RecurrencePlan`` of the step): long
    portions are cut into chunks that run side by side, their start states made by a scan over
    the chunks' own contributions.  The selective form: ``tok_decay`` float32 [T, H] replaces the
    heads' constant decays (``decay`` may then be None), ``tok_scale`` float32 [T, H] multiplies v
    as it enters the state, ``skip`` float32 [H] adds skip_h v_t to the output, and ``kq_share``
    neighbouring heads read one q and k (q, k are then [T, H / kq_share * D]).
    Returns float32 [T, H*E]."""
    _need_cuda(q, k, v, state, decay, q_start, q_len, slots, tok_decay, tok_scale, skip)
    _need_contiguous(tok_decay, tok_scale, skip)
    for x in (q, k, v):
        _column_slice(x, "linear_attention")
    T = q.shape[0]
    ld = q.stride(0) if T > 1 else max(q.stride(0), q.shape[1])
    if T > 1 and (k.stride(0) != ld or v.stride(0) != ld):
        raise KernelError("linear_attention: q, k and v must share a row stride")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise KernelError("linear_attention: q, k and v share a dtype")
    if kq_share < 1 or heads % kq_share:
        raise KernelError("linear_attention: kq_share must divide the head count")
    kq_heads = heads // kq_share
    D, E = q.shape[1] // kq_heads, v.shape[1] // heads
    if q.shape[1] != kq_heads * D or k.shape[1] != kq_heads * D or v.shape[1] != heads * E:
        raise KernelError("linear_attention: widths are not multiples of the head count")
    for name, x, shape in (("tok_decay", tok_decay, (T, heads)), ("tok_scale", tok_scale, (T, heads)),
                           ("skip", skip, (heads,))):
        if x is not None and (x.dtype != torch.float32 or tuple(x.shape) != shape):
            raise KernelError(f"linear_attention: {name} must be float32 {list(shape)}")
    if decay is None and tok_decay is None:
        raise KernelError("linear_attention: give the heads' decays or the tokens'")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, D, E) or not state.is_contiguous():
        raise KernelError("linear_attention: the state is float32 [slots, heads, D, E]")
    if decay is not None and (decay.dtype != torch.float32 or decay.numel() != heads):
        raise KernelError("linear_attention: decay is float32 [heads]")
    for x in (q_start, q_len, slots):
        if x.dtype != torch.int32 or x.numel() < num_requests:
            raise KernelError("linear_attention: request arrays are int32 [R]")
    if D > 512:
        raise KernelError(f"linear_attention: key width {D} per head is beyond 512")
    out = torch.empty((T, heads * E), dtype=torch.float32, device=q.device)
    fn = _fn("linear_attention", "pbe_linear_attention",
             [c_void_p, c_void_p, c_void_p, c_int, c_int] + [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_float, c_int,
                                                                             c_void_p, c_void_p, c_void_p, c_int,
                                                                             c_void_p, c_void_p])
    chunk_decay = None

    def launch(result, items, scratch, n):
        _check(fn(_ptr(q), _ptr(k), _ptr(v), ld, _dtype_code(q), _ptr(result), _ptr(state), _ptr(decay), _ptr(q_start),
                  _ptr(q_len), _ptr(slots), _ptr(items), _ptr(scratch), n, heads, D, E, float(k_scale),
                  1 if silu else 0, _ptr(tok_decay), _ptr(tok_scale), _ptr(skip), int(kq_share), _ptr(chunk_decay),
                  _stream()), "linear_attention")
    if plan is None or plan.num_chunks == 0:
        launch(out, None, None, num_requests)
        return out
    scratch = torch.empty((plan.num_chunks, heads, D, E), dtype=torch.float32, device=q.device)
    if tok_decay is not None:       # the chunks' decay products, left by the pass that makes their contributions
        chunk_decay = torch.empty((plan.num_chunks, heads), dtype=torch.float32, device=q.device)
    launch(None, plan.first_pass, scratch, plan.num_first_pass)          # the chunks' own contributions
    scan = _fn("linear_attention", "pbe_linear_attention_scan",
               [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(scan(_ptr(state), _ptr(scratch), _ptr(decay), _ptr(plan.scan), plan.num_scan, heads, D, E,
                _ptr(chunk_decay), _stream()), "linear_attention_scan")
    launch(out, plan.second_pass, scratch, plan.num_second_pass)         # every chunk from its start state
    return out


# ------------------------------------------------------------------ window + pooled blocks attention
def _pa_defines(dtype: torch.dtype) -> dict:
    """The pooled attention library of a dtype (one library per dtype, built when first asked for)."""
    return {"PBE_PA_F32": 1 if dtype == torch.float32 else 0}


def qk_prepare(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_gain: Optional[torch.Tensor],
               k_gain: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rotary_dim: int,
               positions: torch.Tensor, slots: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
               v_pages: Optional[torch.Tensor], heads: int, kv_heads: int, eps: float, page_tokens: int) -> torch.Tensor:
    """RMS norm over the whole query projection and over the whole key projection (gains float32,
    None: no norm), rotary encoding of neighbouring pairs on the first ``rotary_dim`` dimensions of
    every head, keys and values into the token pages; returns the queries [T, heads * D].
    q, k, v are column slices of one projection matrix."""
    _need_cuda(q, k, v, q_gain, k_gain, inv_freq, positions, slots, k_pages, v_pages)
    for x in (q, k, v):
        _column_slice(x, "qk_prepare")
    T = q.shape[0]
    D, E = q.shape[1] // heads, v.shape[1] // kv_heads
    if q.shape[1] != heads * D or k.shape[1] != kv_heads * D or v.shape[1] != kv_heads * E or D % 2:
        raise KernelError("qk_prepare: widths do not agree with the head counts (and the key width is even)")
    ld = q.stride(0) if T > 1 else q.shape[1] + k.shape[1] + v.shape[1]
    if T > 1 and (k.stride(0) != ld or v.stride(0) != ld):
        raise KernelError("qk_prepare: q, k and v must share a row stride")
    if positions.dtype != torch.int32 or positions.numel() != T:
        raise KernelError("qk_prepare: positions must be int32 [T]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() * 2 != rotary_dim
                                 or rotary_dim > D):
        raise KernelError("qk_prepare: inv_freq must be float32 [rotary_dim / 2], rotary_dim <= D")
    if k_pages is not None:
        if slots is None or slots.dtype != torch.int32 or slots.numel() != T:
            raise KernelError("qk_prepare: slots must be int32 [T]")
        if tuple(k_pages.shape[1:]) != (kv_heads, page_tokens, D) or tuple(v_pages.shape[1:]) != (kv_heads, page_tokens, E) \
                or k_pages.dtype != q.dtype or v_pages.dtype != q.dtype:
            raise KernelError("qk_prepare: pages must be [page, kv_head, page_tokens, width] in the activations' dtype")
    q_out = torch.empty((T, heads * D), dtype=q.dtype, device=q.device)
    fn = _fn("pooled_attention", "pbe_qk_prepare", [c_void_p, c_void_p, c_void_p, c_int] + [c_void_p] * 8 +
             [c_int] * 7 + [c_float, c_int, c_void_p], _pa_defines(q.dtype))
    _check(fn(_ptr(q), _ptr(k), _ptr(v), ld, _ptr(q_gain), _ptr(k_gain), _ptr(inv_freq), _ptr(positions), _ptr(slots),
              _ptr(q_out), _ptr(k_pages), _ptr(v_pages), T, heads, kv_heads, D, E,
              rotary_dim if inv_freq is not None else 0, page_tokens, float(eps), _dtype_code(q), _stream()),
           "qk_prepare")
    return q_out


def pool_blocks(k_tok, v_tok, k_pool, v_pool, positions, request_of_row, bt_tok, bt_pool, pool: int,
                page_tokens: int) -> None:
    """For every row whose position closes a block of ``pool`` tokens: the means of the block's
    keys and values, as the token pages hold them, into the block's entry of the pooled pages."""
    _need_cuda(k_tok, v_tok, k_pool, v_pool, positions, request_of_row, bt_tok, bt_pool)
    _need_contiguous(k_tok, v_tok, k_pool, v_pool, positions, request_of_row, bt_tok, bt_pool)
    T = positions.numel()
    G, D, E = k_tok.shape[1], k_tok.shape[3], v_tok.shape[3]
    if tuple(k_pool.shape[1:]) != tuple(k_tok.shape[1:]) or tuple(v_pool.shape[1:]) != tuple(v_tok.shape[1:]) \
            or k_tok.shape[2] != page_tokens or len({k_tok.dtype, v_tok.dtype, k_pool.dtype, v_pool.dtype}) != 1:
        raise KernelError("pool_blocks: token pages and pooled pages differ in geometry or dtype")
    fn = _fn("pooled_attention", "pbe_pool_blocks", [c_void_p] * 7 + [c_int, c_void_p] + [c_int] * 8 + [c_void_p],
             _pa_defines(k_tok.dtype))
    _check(fn(_ptr(k_tok), _ptr(v_tok), _ptr(k_pool), _ptr(v_pool), _ptr(positions), _ptr(request_of_row),
              _ptr(bt_tok), bt_tok.shape[1], _ptr(bt_pool), bt_pool.shape[1], T, G, D, E, page_tokens, int(pool),
              _dtype_code(k_tok), _stream()), "pool_blocks")


def pooled_attention_tile_rows(heads: int, value_dim: int, want: int, dtype: torch.dtype = torch.bfloat16) -> int:
    fn = _fn("pooled_attention", "pbe_pooled_attention_tile_rows", [c_int, c_int, c_int], _pa_defines(dtype))
    rows = fn(heads, value_dim, want)
    if rows <= 0:
        raise KernelError(f"pooled attention: {heads} heads x {value_dim} values a row are beyond the kernel")
    return rows


# key tiles a block of the split form walks at least (8 rows over 1,040 keys: 92 us with 1, 86 with 2, 135 with 4)
PA_SPLIT_TILES = int(os.environ.get("PBE_PA_SPLIT_TILES", "2"))
PA_MAX_SPLITS = 64        # blocks per row tile at most
PA_FEW_TILES = 96         # row tiles below which the keys are split over more blocks


def pooled_attention_splits(num_tiles: int, tile_rows: int, most_keys: int, heads: int, kv_heads: int, key_dim: int,
                            value_dim: int, dtype: torch.dtype = torch.bfloat16):
    """(blocks per row tile, key tiles a block walks): (1, 0) when the step's row tiles fill the
    GPU by themselves, else the longest row's key tiles in groups of at least ``PA_SPLIT_TILES``,
    at most ``PA_MAX_SPLITS`` groups."""
    if num_tiles >= PA_FEW_TILES:
        return 1, 0
    fn = _fn("pooled_attention", "pbe_pooled_attention_key_tile", [c_int] * 5, _pa_defines(dtype))
    bn = fn(tile_rows, heads, kv_heads, key_dim, value_dim)
    tiles = (most_keys + bn - 1) // bn + 2           # pooled and token tiles round up separately
    per = max(PA_SPLIT_TILES, (tiles + PA_MAX_SPLITS - 1) // PA_MAX_SPLITS)
    return max(1, (tiles + per - 1) // per), per


def pooled_attention(q, k_tok, v_tok, k_pool, v_pool, talk, tiles, num_tiles: int, tile_rows: int, q_start, q_len,
                     seq_len, bt_tok, bt_pool, heads: int, kv_heads: int, scale: float, window: int, pool: int,
                     page_tokens: int, splits: int = 1, split_tiles: int = 0) -> torch.Tensor:
    """Softmax attention of every row over the tokens of its window and the pooled blocks before
    it (one softmax), the probabilities mixed across heads by ``talk`` (float32 [H, H], row h
    weighs the heads' probabilities for head h; None: no mixing).  ``splits`` > 1: the keys of a
    row tile are cut over that many blocks (statistics per split, their combination, the
    normalised shares of the output, their sum).  Returns [T, heads * E]."""
    _need_cuda(q, k_tok, v_tok, k_pool, v_pool, talk, tiles, q_start, q_len, seq_len, bt_tok, bt_pool)
    _need_contiguous(q, k_tok, v_tok, k_pool, v_pool, talk, tiles, q_start, q_len, seq_len, bt_tok, bt_pool)
    T = q.shape[0]
    D, E = k_tok.shape[3], v_tok.shape[3]
    if q.shape[1] != heads * D or k_tok.shape[1] != kv_heads or k_tok.dtype != q.dtype or v_tok.dtype != q.dtype:
        raise KernelError("pooled_attention: shapes or dtypes do not agree")
    if talk is not None and (talk.dtype != torch.float32 or tuple(talk.shape) != (heads, heads)):
        raise KernelError("pooled_attention: the mixing matrix is float32 [heads, heads]")
    if pool and (k_pool is None or bt_pool is None):
        raise KernelError("pooled_attention: pooled blocks need their pages and block table")
    out = torch.empty((T, heads * E), dtype=q.dtype, device=q.device)
    part_ml = stats = part_o = None
    if splits > 1:
        per = tile_rows * heads
        part_ml = torch.empty((num_tiles, splits, per, 2), dtype=torch.float32, device=q.device)
        stats = torch.empty((num_tiles, per, 2), dtype=torch.float32, device=q.device)
        part_o = torch.empty((num_tiles, splits, per * E), dtype=torch.float32, device=q.device)
    fn = _fn("pooled_attention", "pbe_pooled_attention",
             [c_void_p] * 8 + [c_int, c_int] + [c_void_p] * 4 + [c_int, c_void_p, c_int] + [c_int] * 7 +
             [c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p], _pa_defines(q.dtype))
    _check(fn(_ptr(q), _ptr(k_tok), _ptr(v_tok), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(talk), _ptr(tiles),
              num_tiles, tile_rows, _ptr(q_start), _ptr(q_len), _ptr(seq_len), _ptr(bt_tok), bt_tok.shape[1],
              _ptr(bt_pool), bt_pool.shape[1] if bt_pool is not None else 0, heads, kv_heads, D, E, page_tokens,
              int(window), int(pool or 0), float(scale), _dtype_code(q), int(splits), int(split_tiles), _ptr(part_ml),
              _ptr(stats), _ptr(part_o), _stream()), "pooled_attention")
    return out


# ------------------------------------------------------------------ rope + cache write
def rope_kv_write(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  positions: torch.Tensor, slots: Optional[torch.Tensor],
                  inv_freq: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                  head_dim: int, rotary_dim: int, page_tokens: int, interleaved: bool = False):
    """q_out = rope(q + b); cache[slot] = rope(k + b), v + b.  k_cache / v_cache are one
    layer's pages [page, kv_head, page_tokens, head_dim]; None: nothing is written."""
    _need_cuda(qkv, bias, q_out, k_cache, v_cache, positions, slots, inv_freq)
    _need_contiguous(qkv, bias, q_out, k_cache, v_cache, positions, slots, inv_freq)
    T = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width or q_out.shape != (T, num_heads * head_dim) or q_out.dtype != qkv.dtype:
        raise KernelError("rope_kv_write: shapes or dtypes do not agree")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != width):
        raise KernelError("rope_kv_write: bias must be float32 of the fused width")
    if positions.dtype != torch.int32 or positions.numel() != T:
        raise KernelError("rope_kv_write: positions must be int32 [T]")
    if k_cache is not None:
        if slots is None or slots.dtype != torch.int32 or slots.numel() != T:
            raise KernelError("rope_kv_write: slots must be int32 [T]")
        for c in (k_cache, v_cache):
            if c is None or c.dtype != qkv.dtype or tuple(c.shape[1:]) != (num_kv_heads, page_tokens, head_dim):
                raise KernelError("rope_kv_write: cache pages must be [page, kv_head, page_tokens, head_dim] "
                                  "in the activations' dtype")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_kv_write: inv_freq must be float32 [rotary_dim / 2]")
    fn = _fn("rope_kv", "pbe_rope_kv_write",
             [c_void_p] * 8 + [c_int] * 8 + [c_void_p])
    _check(fn(_ptr(qkv), _ptr(bias), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(positions),
              _ptr(slots), _ptr(inv_freq), T, num_heads, num_kv_heads, head_dim,
              rotary_dim if inv_freq is not None else 0, page_tokens, 1 if interleaved else 0,
              _dtype_code(qkv), _stream()), "rope_kv_write")
    return q_out


# ------------------------------------------------------------------ matrix products
def sgemm_nt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor):
    """out = x @ w.T (+ bias) in true float32 arithmetic; w float32 [N, K]."""
    _need_cuda(x, w, bias, out)
    _need_contiguous(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    if w.dtype != torch.float32 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError("sgemm_nt: shapes or dtypes do not agree")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("sgemm_nt: bias must be float32 [N]")
    if x.dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("sgemm_nt: float32 rows give float32 rows (bfloat16 rows give either)")
    need = _fn("sgemm", "pbe_sgemm_scratch_floats", [c_int, c_int, c_int, c_void_p])
    need.restype = c_ll
    n_tickets = c_int(0)
    floats = int(need(M, N, K, ctypes.byref(n_tickets)))
    scratch = tickets = None
    if floats > 0:
        # partial sums of the K slices, and the tickets by which the last block or warp of a group
        # of outputs learns that it is the one to add them up (zeroed once, left at zero by every call)
        scratch = torch.empty(floats, dtype=torch.float32, device=x.device)
        tickets = _sgemm_tickets.get(x.device)
        if tickets is None or tickets.numel() < n_tickets.value:
            tickets = _sgemm_tickets[x.device] = torch.zeros(max(8192, 2 * n_tickets.value), dtype=torch.int32,
                                                             device=x.device)
    fn = _fn("sgemm", "pbe_sgemm_nt",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
              c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(x), _dtype_code(x), _ptr(w), _ptr(bias), _ptr(out), _dtype_code(out), M, N, K, K, N,
              _ptr(scratch), _ptr(tickets), _stream()), "sgemm_nt")
    return out


_sgemm_tickets = {}      # per device: zeroed int32 tickets shared by the float32 products of the stream


SKINNY_MAX_ROWS = int(os.environ.get('PBE_SKINNY_ROWS', '8'))      # batches of at most this many rows take the weight-streaming kernel (0: never); with 9 to
                         # 16 rows its two-tile instance loses to the library GEMM (4.39 against 3.48 ms a step)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, swiglu: bool = False) -> torch.Tensor:
    """y = x w^T (+ b) for at most 16 rows, bfloat16 operands, weights streamed once.
    ``swiglu``: w is [gate; up] stacked and y = silu(x gate^T) * (x up^T), [M, N/2]."""
    _need_cuda(x, w, bias)
    _need_contiguous(x, w, bias)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError("gemm_skinny takes bfloat16 x [M, K] and w [N, K]")
    if M > 16 or K % 8 != 0:
        raise KernelError(f"gemm_skinny takes at most 16 rows and K a multiple of 8 (got M={M}, K={K})")
    if swiglu and (N % 2 or bias is not None):
        raise KernelError("gemm_skinny: the SwiGLU epilogue needs an even N and no bias")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_skinny: bias must be float32 [N]")
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    fn = _fn("gemm_skinny", "pbe_gemm_skinny",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _dtype_code(out), M, N, K, 1 if swiglu else 0,
              _stream()), "gemm_skinny")
    return out


_tc5_err = {}        # per device: the GEMM's flag
_tc5_attn_err = {}   # per device: the attention kernel's flag (element 0) and room for a debugging trace


TC5_PAIR = os.environ.get("PBE_TC5_PAIR", "0") == "1"


def gemm_tc5(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
             swiglu: bool = False, check: bool = False, pair: Optional[bool] = None) -> torch.Tensor:
    """y = x w^T for many rows on the tcgen05 tensor cores (TMA-fed, accumulator in tensor
    memory).  ``swiglu``: w is [gate; up] stacked and y = silu(x gate^T) * (x up^T), [M, N/2].
    ``pair``: two-SM tiles (a cluster of two blocks a 256 x 256 tile) from 256 rows on; None
    takes PBE_TC5_PAIR from the environment (off unless it is 1).
    ``check`` synchronises and raises if a bounded wait inside the kernel ran out."""
    _need_cuda(x, w)
    _need_contiguous(x, w)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError("gemm_tc5 takes bfloat16 x [M, K] and w [N, K]")
    if K % 8 != 0:
        raise KernelError(f"gemm_tc5 needs K to be a multiple of 8 (rows on 16-byte boundaries), got {K}")
    out_dtype = out_dtype or torch.bfloat16
    if swiglu and (N % 2 or out_dtype != torch.bfloat16):
        raise KernelError("gemm_tc5: the SwiGLU epilogue needs an even N and bfloat16 output")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    err = _tc5_err.get(x.device)
    if err is None:
        err = _tc5_err[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    fn = _fn("gemm_tc5", "pbe_gemm_tc5",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    mode = (1 if swiglu else 0) | (2 if (TC5_PAIR if pair is None else pair) else 0)
    _check(fn(_ptr(x), _ptr(w), _ptr(out), _dtype_code(out), M, N, K, mode, _ptr(err), _stream()), "gemm_tc5")
    if check and int(err.item()) != 0:
        err.zero_()
        raise KernelError("gemm_tc5: a wait inside the kernel ran out; the result is invalid")
    return out


_stream_state = {}     # per device: (scratch floats, zeroed tickets) of the K-split products


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                swiglu: bool = False, check: bool = False) -> torch.Tensor:
    """y = x w^T for up to 64 rows on the tcgen05 tensor cores with the weights as the streamed
    operand (TMA-fed ring, accumulator in tensor memory, K split over blocks where the matrix has
    few rows).  ``swiglu``: w is [gate; up] stacked and y = silu(x gate^T) * (x up^T), [M, N/2].
    ``check`` synchronises and raises if a bounded wait inside the kernel ran out."""
    _need_cuda(x, w)
    _need_contiguous(x, w)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError("gemm_stream takes bfloat16 x [M, K] and w [N, K]")
    if M > STREAM_KERNEL_ROWS or K % 8 != 0:
        raise KernelError(f"gemm_stream takes at most {STREAM_KERNEL_ROWS} rows and K a multiple of 8 (got M={M}, K={K})")
    out_dtype = out_dtype or torch.bfloat16
    if swiglu and (N % 2 or out_dtype != torch.bfloat16):
        raise KernelError("gemm_stream: the SwiGLU epilogue needs an even N and bfloat16 output")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    scratch, tickets, err = gemm_stream_buffers(x.device)
    fn = _fn("gemm_stream", "pbe_gemm_stream",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(x), _ptr(w), _ptr(out), _dtype_code(out), M, N, K, 1 if swiglu else 0, _ptr(scratch), _ptr(tickets),
              _ptr(err), _stream()), "gemm_stream")
    if check and int(err.item()) != 0:
        err.zero_()
        raise KernelError("gemm_stream: a wait inside the kernel ran out; the result is invalid")
    return out


def gemm_stream_buffers(device):
    """(scratch, tickets, flag) of ``gemm_stream`` on this device, made on first use: partial tiles
    of at most one block a multiprocessor (128 weight rows x 64 batch rows of float32, twice that
    for gate and up), the tiles' tickets, zeroed once and left at zero by every launch, and the flag
    that a bounded wait sets."""
    device = torch.device(device)
    st = _stream_state.get(device)
    if st is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        st = _stream_state[device] = (torch.empty(sms * 128 * 128, dtype=torch.float32, device=device),
                                      torch.zeros(1024, dtype=torch.int32, device=device))
    err = _tc5_err.get(device)
    if err is None:
        err = _tc5_err[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return st[0], st[1], err


# Which projections of a decode step go through gemm_stream, as bits (1 QKV, 2 output, 4 gate/up
# with SwiGLU, 8 down, 16 LM head and others): STREAM_MASK_FEW for steps of at most SKINNY_MAX_ROWS
# rows (the rest of such a step is gemm_skinny's), STREAM_MASK for steps of more rows up to
# STREAM_MID_ROWS and STREAM_MASK_MANY beyond that up to STREAM_MAX_ROWS (the rest is the
# library's).  Measured in the captured decode step of the 7B shape, ms a step: 1 / 2 / 4 / 8 rows
# with gate/up on it 2.91 / 2.93 / 2.98 / 3.12-3.14 against 2.95 / 2.99 / 3.05 / 3.19 on gemm_skinny
# (down on it as well: 3.14 at 8 rows, down alone 3.22); 16 rows 3.52 -> 3.37 with gate/up and
# down, 3.40 with all four; 24 / 32 / 48 / 64 rows with gate/up alone 3.67 / 3.76 / 4.18 / 4.52
# against 3.75 / 3.84 / 4.26 / 4.58 on the library GEMM and silu_mul (with down as well: level at 24
# and 32, 4.77 at 64).  So: gate/up everywhere up to 64 rows, down as well from 9 to 16.  The
# PBE_STREAM_FEW, PBE_STREAM and PBE_STREAM_MANY masks (0: never) and PBE_STREAM_ROWS /
# PBE_STREAM_MAX_ROWS override the choice.
STREAM_KERNEL_ROWS = 64
STREAM_MID_ROWS = int(os.environ.get("PBE_STREAM_ROWS", "16"))
STREAM_MAX_ROWS = min(STREAM_KERNEL_ROWS, int(os.environ.get("PBE_STREAM_MAX_ROWS", "64")))
STREAM_MASK_FEW = int(os.environ.get("PBE_STREAM_FEW", "4"))
STREAM_MASK = int(os.environ.get("PBE_STREAM", "12"))
STREAM_MASK_MANY = int(os.environ.get("PBE_STREAM_MANY", "4"))
# ... and only matrices of at least this many elements: below it (the 1.5B shape's 27.5 M and 13.8 M)
# the library's product is the shorter one (21.4 against 24.5 us, 19.5 against 20.5 us at 16 rows)
STREAM_MIN_WEIGHT = int(os.environ.get("PBE_STREAM_MIN_WEIGHT", str(48 << 20)))


def stream_mask(rows: int) -> int:
    if rows <= SKINNY_MAX_ROWS:
        return STREAM_MASK_FEW
    if rows <= STREAM_MID_ROWS:
        return STREAM_MASK
    return STREAM_MASK_MANY if rows <= STREAM_MAX_ROWS else 0


def stream_applies(x: torch.Tensor, w: torch.Tensor, bit: int) -> bool:
    return (stream_mask(x.shape[0]) & bit != 0 and x.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and w.numel() >= STREAM_MIN_WEIGHT)


# Projections of many rows (prompt portions): which of them take gemm_tc5 instead of the vendor
# GEMM library, as bits (1 QKV, 2 output, 4 gate/up with the SwiGLU epilogue, 8 down, 16 others).
# PBE_GEMM in the environment: "tc5" all of them, "library" none, or the mask as a number.
def _tc5_mask() -> int:
    e = os.environ.get("PBE_GEMM", "").strip().lower()
    if e == "tc5":
        return 31
    if e == "library":
        return 0
    return int(e) if e.isdigit() else TC5_DEFAULT_MASK


TC5_DEFAULT_MASK = 0
TC5_MIN_ROWS = 128
TC5_MASK = _tc5_mask()


def tc5_applies(x: torch.Tensor, w: torch.Tensor, bit: int = 16) -> bool:
    return (TC5_MASK & bit != 0 and x.shape[0] >= TC5_MIN_ROWS and x.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0)


def stream_wanted(largest_weight: int) -> bool:
    """True when a matrix of that many elements would go through gemm_stream at some step size."""
    return bool(STREAM_MASK or STREAM_MASK_FEW or STREAM_MASK_MANY) and largest_weight >= STREAM_MIN_WEIGHT


def gemm_libraries(dtype: torch.dtype, largest_weight: int = 0):
    """The matrix-product libraries a part of this dtype launches whose largest matrix has that
    many elements (for parallel builds)."""
    if dtype == torch.float32:
        return [("sgemm", None)]
    return [("gemm_skinny", None)] + ([("gemm_stream", None)] if stream_wanted(largest_weight) else []) + \
        ([("gemm_tc5", None)] if TC5_MASK else [])


def skinny_applies(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (0 < x.shape[0] <= SKINNY_MAX_ROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.shape[1] % 8 == 0)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, kind: int = 16) -> torch.Tensor:
    """y = x w^T (+ b).  A float32 weight takes the true-float32 kernel of this package; a
    bfloat16 weight takes the package's weight-streaming kernels for few rows and otherwise the
    vendor GEMM library with float32 accumulation, as the reference does for every projection
    (matmul_kernel_batch.cu:39-208).  ``kind``: which projection this is, a bit of STREAM_MASK."""
    _need_cuda(x, w, bias)
    out_dtype = out_dtype or x.dtype
    if w.dtype == torch.float32:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
        return sgemm_nt(x, w, bias, out)
    if x.dtype != torch.bfloat16:
        raise KernelError("a bfloat16 weight takes bfloat16 activations")
    if bias is None and stream_applies(x, w, kind):
        return gemm_stream(x, w, out_dtype)
    if skinny_applies(x, w):
        return gemm_skinny(x, w, bias, out_dtype)
    if tc5_applies(x, w, kind) and bias is None:
        return gemm_tc5(x, w, out_dtype)
    if out_dtype == torch.float32:
        y = torch.mm(x, w.t(), out_dtype=torch.float32)
    else:
        y = torch.mm(x, w.t())
    if bias is not None:
        y += bias.to(y.dtype)
    return y


# ------------------------------------------------------------------ attention
class AttnParams(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("out", c_void_p),
                ("part_o", c_void_p), ("part_ml", c_void_p), ("q_start", c_void_p),
                ("q_len", c_void_p), ("seq_len", c_void_p), ("block_table", c_void_p),
                ("work", c_void_p), ("tok_split_row", c_void_p),
                ("bt_stride", c_int), ("num_heads", c_int), ("num_kv_heads", c_int),
                ("page_tokens", c_int), ("window", c_int), ("split_keys", c_int),
                ("max_splits", c_int), ("tile_rows", c_int), ("scale", c_float), ("kinds", c_int),
                ("num_pages", c_int)]


class AttnMergeParams(ctypes.Structure):
    _fields_ = [("part_o", c_void_p), ("part_ml", c_void_p), ("out", c_void_p),
                ("split_tokens", c_void_p), ("split_counts", c_void_p),
                ("num_heads", c_int), ("head_dim", c_int), ("max_splits", c_int)]


SIMPLE_TILE_ROWS = 16   # packed rows per block of the plain attention kernel
SIMPLE_KEY_TILE = 32


def attention_kernel_config(head_dim: int, dtype: torch.dtype, kind: Optional[str] = None):
    """(kind, tile_rows, key_tile) of the attention kernel used for a head size and dtype."""
    if head_dim % 16 != 0 or head_dim <= 0 or head_dim > 256:
        raise KernelError(f"attention kernels take head sizes 16, 32, ..., 256; got {head_dim}")
    if kind is None and dtype == torch.bfloat16 and head_dim in (64, 128) and _attention_choice() != "mma" \
            and _tc5_available():
        kind = "tc5"
    kind = kind or ("mma" if dtype == torch.bfloat16 and _mma_available() else "simple")
    if kind == "simple":
        return "simple", SIMPLE_TILE_ROWS, SIMPLE_KEY_TILE
    if kind == "tc5":
        return "tc5", 128, 128
    return "mma", (128 if head_dim <= 128 else 64), MMA_KEY_TILE


MMA_KEY_TILE = 64


def _attention_choice() -> str:
    """Prompt portions of bfloat16 models with head size 64 or 128 run on the tcgen05
    attention kernel; PBE_ATTN=mma keeps them on the mma.sync kernel."""
    return os.environ.get("PBE_ATTN", "").strip().lower()


def _tc5_available() -> bool:
    from .build import KERNEL_DIR
    return os.path.isfile(os.path.join(KERNEL_DIR, "attention_tc5.cu"))


def _mma_available() -> bool:
    from .build import KERNEL_DIR
    return os.path.isfile(os.path.join(KERNEL_DIR, "attention_mma.cu"))


def paged_attention(q, k_cache, v_cache, out, meta, num_heads, num_kv_heads, head_dim, scale, window,
                    page_tokens, kind="simple"):
    """Causal attention of every row of the batch over the paged cache.

    ``meta`` carries the step's device arrays for this (group, head grouping, tile size,
    window): q_start, q_len, seq_len, block_table [R, stride], work [n, 4], tok_split_row,
    split_tokens, split_counts, max_splits, split_keys, part_o, part_ml."""
    _need_cuda(q, k_cache, v_cache, out)
    _need_contiguous(q, k_cache, v_cache, out)
    if q.dtype != k_cache.dtype or q.dtype != out.dtype:
        raise KernelError("attention: q, cache and output must share one dtype")
    if kind == "mma" and q.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention kernel takes bfloat16")
    lib = "attention_simple" if kind == "simple" else "attention_mma"
    defines = {"PBE_HEAD_DIM": int(head_dim)}
    tc5 = kind == "tc5"
    if tc5:
        if q.dtype != torch.bfloat16 or head_dim not in (64, 128):
            raise KernelError("the tcgen05 attention kernel takes bfloat16 and head sizes 64 and 128")
        # its page loads need pages of 8 tokens or more that divide the key tile of 64 or are a
        # multiple of it; with other page sizes the mma.sync kernel (same work list, same tile
        # rows) does the tiles
        tc5 = tc5_attention_applies(head_dim, page_tokens)
        kind = "mma"
    p = AttnParams(
        q=q.data_ptr(), k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr(), out=out.data_ptr(),
        part_o=meta.part_o.data_ptr() if meta.part_o is not None else None,
        part_ml=meta.part_ml.data_ptr() if meta.part_ml is not None else None,
        q_start=meta.q_start.data_ptr(), q_len=meta.q_len.data_ptr(), seq_len=meta.seq_len.data_ptr(),
        block_table=meta.block_table.data_ptr(), work=meta.work.data_ptr(),
        tok_split_row=meta.tok_split_row.data_ptr(), bt_stride=int(meta.bt_stride),
        num_heads=int(num_heads), num_kv_heads=int(num_kv_heads), page_tokens=int(page_tokens),
        window=int(window or 0), split_keys=int(meta.split_keys), max_splits=int(meta.max_splits),
        tile_rows=int(meta.tile_rows), scale=float(scale), kinds=int(getattr(meta, "kinds", 0)),
        num_pages=int(k_cache.shape[0]))
    if tc5:
        # prompt-portion tiles on the tcgen05 kernel; the decode instances below take the rest
        err = tc5_attention_error_buffer(q.device)
        tfn = _fn("attention_tc5", "pbe_attn_tc5", [ctypes.POINTER(AttnParams), c_int, c_int, c_void_p, c_void_p],
                  defines)
        if (p.kinds & 3) == 0 or (p.kinds & 2):
            _check(tfn(ctypes.byref(p), int(meta.num_work), int(k_cache.shape[0]), _ptr(err), _stream()),
                   "paged_attention (tcgen05)")
        p.kinds = (p.kinds | 8) if (p.kinds & 3) else (1 | 8)
    fn = _fn(lib, "pbe_attn_" + kind, [ctypes.POINTER(AttnParams), c_int, c_int, c_void_p], defines)
    if kind == "mma":
        _mma_flag_heads.add(int(head_dim))
    _check(fn(ctypes.byref(p), int(meta.num_work), _dtype_code(q), _stream()), "paged_attention")
    if meta.num_split_rows > 0:
        mp = AttnMergeParams(part_o=meta.part_o.data_ptr(), part_ml=meta.part_ml.data_ptr(),
                             out=out.data_ptr(), split_tokens=meta.split_tokens.data_ptr(),
                             split_counts=meta.split_counts.data_ptr(), num_heads=int(num_heads),
                             head_dim=int(head_dim), max_splits=int(meta.max_splits))
        mfn = _fn("attention_simple", "pbe_attn_merge",
                  [ctypes.POINTER(AttnMergeParams), c_int, c_int, c_void_p], defines)
        _check(mfn(ctypes.byref(mp), int(meta.num_split_rows), _dtype_code(out), _stream()),
               "attention merge")
    return out


# The block-cooperative instance of the decode attention kernel (four warps share each key tile)
# is the shortest path through one work item; it pays while all its blocks (work items x kv
# heads) are resident at once, three a multiprocessor.  Beyond that the persistent instance,
# in which every warp streams whole work items, is faster (measured crossover between 256 and
# 512 items on 148 multiprocessors).
DECODE_BLOCK_ITEMS_PER_SM = 3


_sm_counts = {}


def decode_block_max_items(device) -> int:
    sms = _sm_counts.get(device)
    if sms is None:
        try:
            sms = torch.cuda.get_device_properties(device).multi_processor_count
        except (RuntimeError, AssertionError):
            sms = 148
        _sm_counts[device] = sms
    return DECODE_BLOCK_ITEMS_PER_SM * sms


class AttnFusedParams(ctypes.Structure):
    _fields_ = [("qkv", c_void_p), ("bias", c_void_p), ("positions", c_void_p), ("slots", c_void_p),
                ("inv_freq", c_void_p), ("num_requests", c_int)]


FUSED_DECODE_MAX_KEYS_PER_BLOCK = 32768   # beyond that the other path takes the step


def fused_decode_splits(num_requests: int, num_kv_heads: int, longest_keys: int, device) -> int:
    """Blocks per (request, key/value head) of the fused decode attention kernel: the largest of
    8, 4, 2, 1 with which every block of the step is resident at once; 1 for steps too large for
    that (their blocks run in waves: batch 128 at 2,048 tokens 16,900 -> 20,600 tok/s against the
    separate kernels); 0 when a block would get more keys than the kernel is meant for."""
    cap = decode_block_max_items(device)
    for splits in (8, 4, 2, 1):
        blocks = num_requests * num_kv_heads * splits
        if blocks <= cap:
            per_block = (longest_keys + splits - 1) // splits
            if not 0 < per_block <= FUSED_DECODE_MAX_KEYS_PER_BLOCK:
                return 0
            # a few dozen blocks with thousands of keys each (one or two requests with very long
            # contexts) stream better as many small work items on the other path
            if per_block > 1536 and blocks <= 64:
                return 0
            return splits
    return 1 if 0 < longest_keys <= FUSED_DECODE_MAX_KEYS_PER_BLOCK else 0


def fused_decode_attention_applies(dtype: torch.dtype, head_dim: int, group_size: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and group_size <= 16
            and _mma_available() and os.environ.get("PBE_DECODE_FUSED", "1") != "0")


def attention_decode_fused(qkv, bias, k_cache, v_cache, out, meta, positions, slots, inv_freq, num_requests,
                           num_heads, num_kv_heads, head_dim, scale, window, page_tokens, splits=8):
    """A step of decoded tokens only (one row a request): bias and rotary position encoding of
    the new token's query, key and value, the cache write, attention over the pages and the
    merge of the key splits in ONE launch (clusters of 8 blocks, one per request and key/value
    head).  ``qkv``: the fused projection's output [T, (H + 2 KV) hd]; ``out``: [T, H hd];
    row r of both belongs to request r (a step of decoded tokens has its rows in that order)."""
    _need_cuda(qkv, bias, k_cache, v_cache, out, positions, slots, inv_freq)
    _need_contiguous(qkv, k_cache, v_cache, out)
    if qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the fused decode attention kernel takes bfloat16")
    p = AttnParams(
        q=None, k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr(), out=out.data_ptr(),
        part_o=None, part_ml=None,
        q_start=meta.q_start.data_ptr(), q_len=meta.q_len.data_ptr(), seq_len=meta.seq_len.data_ptr(),
        block_table=meta.block_table.data_ptr(), work=None, tok_split_row=None, bt_stride=int(meta.bt_stride),
        num_heads=int(num_heads), num_kv_heads=int(num_kv_heads), page_tokens=int(page_tokens),
        window=int(window or 0), split_keys=int(meta.split_keys), max_splits=int(splits),
        tile_rows=int(meta.tile_rows), scale=float(scale), kinds=1, num_pages=int(k_cache.shape[0]))
    f = AttnFusedParams(qkv=qkv.data_ptr(), bias=bias.data_ptr() if bias is not None else None,
                        positions=positions.data_ptr(), slots=slots.data_ptr(), inv_freq=inv_freq.data_ptr(),
                        num_requests=int(num_requests))
    fn = _fn("attention_mma", "pbe_attn_decode_fused",
             [ctypes.POINTER(AttnParams), ctypes.POINTER(AttnFusedParams), c_int, c_int, c_void_p],
             {"PBE_HEAD_DIM": int(head_dim)})
    _mma_flag_heads.add(int(head_dim))
    _check(fn(ctypes.byref(p), ctypes.byref(f), _dtype_code(qkv), int(splits), _stream()), "attention_decode_fused")
    return out


def tc5_attention_error_buffer(device) -> torch.Tensor:
    """Element 0: set by the tcgen05 attention kernel when a bounded wait ran out."""
    err = _tc5_attn_err.get(device)
    if err is None:
        err = _tc5_attn_err[device] = torch.zeros(1024, dtype=torch.int32, device=device)
    return err


def tc5_attention_applies(head_dim: int, page_tokens: int) -> bool:
    return head_dim in (64, 128) and page_tokens >= 8 and page_tokens % 8 == 0 and \
        (64 % page_tokens == 0 or page_tokens % 64 == 0)


def tc5_error_flag(device) -> int:
    """1 if a bounded wait inside a tcgen05 kernel ran out since the last call (then reset)."""
    err = _tc5_attn_err.get(torch.device(device))
    if err is None:
        return 0
    v = int(err[0].item())
    if v:
        err[:1].zero_()
    return v


def attention_mma_wait_flag(head_dim: int) -> int:
    """1 once a bounded wait for a key tile ran out inside the mma.sync attention kernels of this
    head size (never in a correct run; the launch's results are not valid then)."""
    fn = _fn("attention_mma", "pbe_attn_mma_wait_gave_up", [], {"PBE_HEAD_DIM": int(head_dim)})
    return int(fn())


# ------------------------------------------------------------------ the kernels' status word
_STATUS_NAMES = {}      # device -> names of the flags, in bit order
_status_state = {}      # device -> (addresses on the device, number of flags, key of the sources)
_mma_flag_heads = set() # head sizes whose mma.sync attention library this process has launched


def _status_sources(device):
    """(name, device address) of every flag a bounded wait of this package's kernels can set
    on ``device``, in a fixed order."""
    device = torch.device(device)
    out = []
    err = _tc5_attn_err.get(device)
    if err is not None:
        out.append(("tcgen05 attention", err.data_ptr()))
    err = _tc5_err.get(device)
    if err is not None:
        out.append(("tcgen05 GEMM", err.data_ptr()))
    for hd in sorted(_mma_flag_heads):
        fn = _fns.get(("attention_mma", "pbe_attn_mma_wait_flag_address", (("PBE_HEAD_DIM", hd),)))
        if fn is None:
            lib = load_library("attention_mma", {"PBE_HEAD_DIM": hd})
            fn = lib.pbe_attn_mma_wait_flag_address
            fn.argtypes, fn.restype = [], ctypes.c_ulonglong
            _fns[("attention_mma", "pbe_attn_mma_wait_flag_address", (("PBE_HEAD_DIM", hd),))] = fn
        with torch.cuda.device(device):
            addr = int(fn())
        if addr:
            out.append((f"mma.sync attention (head size {hd})", addr))
    return out[:32]


def collect_status(out: torch.Tensor) -> torch.Tensor:
    """Launches a kernel that writes into ``out`` (int32, one element, on the device) a word
    with bit i set when flag i of ``status_names(device)`` was set, and clears those flags.
    A flag is set by a kernel whose bounded wait ran out: the results of that launch are not
    valid.  Costs one launch of one thread; nothing waits."""
    _need_cuda(out)
    device = out.device
    # the flags' addresses are looked up again only when a new flag has come into being
    key = (device in _tc5_attn_err, device in _tc5_err, len(_mma_flag_heads))
    st = _status_state.get(device)
    if st is None or st[2] != key:
        import numpy as np
        src = _status_sources(device)
        addrs = torch.from_numpy(np.array([a for _, a in src] + [0], dtype=np.uint64).view(np.int64)).to(device)
        st = _status_state[device] = (addrs, len(src), key)
        _STATUS_NAMES[device] = [n for n, _ in src]
    fn = _fn("elementwise", "pbe_collect_status", [c_void_p, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(st[0]), st[1], _ptr(out), _stream()), "collect_status")
    return out


def status_message(device, word: int) -> str:
    names = _STATUS_NAMES.get(torch.device(device), [])
    hit = [names[i] if i < len(names) else f"flag {i}" for i in range(32) if (int(word) >> i) & 1]
    return ("a bounded wait ran out inside: " + ", ".join(hit) +
            "; the results of that step are not valid (the flags have been cleared)")


def raise_on_kernel_status(device) -> None:
    """Synchronises, reads the kernels' flags and raises KernelError if one was set."""
    out = torch.zeros(1, dtype=torch.int32, device=device)
    word = int(collect_status(out).item())
    if word:
        raise KernelError(status_message(device, word))


def attention_libraries(head_dim: int, dtype: torch.dtype):
    """The (library, defines) pairs a model with this head size needs, for parallel builds."""
    jobs = [("attention_simple", {"PBE_HEAD_DIM": int(head_dim)})]
    if dtype == torch.bfloat16 and _mma_available():
        jobs.append(("attention_mma", {"PBE_HEAD_DIM": int(head_dim)}))
        if head_dim in (64, 128) and _attention_choice() != "mma" and _tc5_available():
            jobs.append(("attention_tc5", {"PBE_HEAD_DIM": int(head_dim)}))
    return jobs


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy token per row; ties go to the lowest id."""
    _need_cuda(logits, out)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax takes float32 logits with unit column stride")
    n, V = logits.shape
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    fn = _fn("sampling", "pbe_argmax", [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), n, V, _ptr(out), _stream()), "argmax")
    return out


def sample(logits, temperature, top_k, top_p, uniform, out=None) -> torch.Tensor:
    """One token per row with per-row temperature (float32), top_k (int32), top_p (float32)
    and uniform draw (float32)."""
    _need_cuda(logits, temperature, top_k, top_p, uniform, out)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample takes float32 logits with unit column stride")
    n, V = logits.shape
    for t, dt in ((temperature, torch.float32), (top_k, torch.int32), (top_p, torch.float32),
                  (uniform, torch.float32)):
        if t.dtype != dt or t.numel() != n or not t.is_contiguous():
            raise KernelError("sample: per-row parameters must be contiguous, one per row")
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    fn = _fn("sampling", "pbe_sample", [c_void_p, c_ll, c_int, c_int] + [c_void_p] * 6)
    _check(fn(_ptr(logits), logits.stride(0), n, V, _ptr(temperature), _ptr(top_k), _ptr(top_p),
              _ptr(uniform), _ptr(out), _stream()), "sample")
    return out


def seen_mark(seen: torch.Tensor, tokens: torch.Tensor, slots: Optional[torch.Tensor] = None, slot: int = -1) -> None:
    """seen[slots[i], tokens[i]] = 1 (``slots`` None: all in row ``slot``).  seen: uint8
    [slots, ld], tokens and slots int32 on the device; slots below 0 are skipped."""
    _need_cuda(seen, tokens, slots)
    if seen.dtype != torch.uint8 or tokens.dtype != torch.int32 or (slots is not None and slots.dtype != torch.int32):
        raise KernelError("seen_mark: a uint8 table, int32 tokens and slots")
    fn = _fn("sampling", "pbe_seen_mark", [c_void_p, c_ll, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(seen), seen.stride(0), seen.shape[1], _ptr(slots), int(slot), _ptr(tokens), tokens.numel(),
              _stream()), "seen_mark")


def penalty_seen(logits: torch.Tensor, seen: torch.Tensor, slots: torch.Tensor, penalties: torch.Tensor) -> torch.Tensor:
    """The repetition penalty from the table of seen tokens: row r of ``logits`` takes the
    tokens marked in seen[slots[r]] (slot below 0: the row is left alone)."""
    _need_cuda(logits, seen, slots, penalties)
    n, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or seen.dtype != torch.uint8 or \
            slots.dtype != torch.int32 or penalties.dtype != torch.float32 or slots.numel() != n or penalties.numel() != n:
        raise KernelError("penalty_seen: wrong dtypes or sizes")
    fn = _fn("sampling", "pbe_penalty_seen", [c_void_p, c_ll, c_int, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), n, V, _ptr(seen), seen.stride(0), _ptr(slots), _ptr(penalties),
              _stream()), "penalty_seen")
    return logits


def sample_set_mode(mode: int) -> None:
    """0 (default): the sampling kernel's binned selection with the radix descent behind it; 1: the
    radix descent only.  Both give the same token; the switch is for tests that compare them."""
    _fn("sampling", "pbe_sample_set_mode", [c_int])(int(mode))


def apply_penalty(logits, rows, tokens, penalties):
    """logits[rows[i], tokens[i]] is divided by penalties[i] when positive, multiplied
    otherwise; every (row, token) pair appears once."""
    _need_cuda(logits, rows, tokens, penalties)
    n = rows.numel()
    if logits.dtype != torch.float32 or rows.dtype != torch.int32 or tokens.dtype != torch.int32 \
            or penalties.dtype != torch.float32 or tokens.numel() != n or penalties.numel() != n:
        raise KernelError("apply_penalty: wrong dtypes or sizes")
    fn = _fn("sampling", "pbe_apply_penalty", [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), logits.shape[1], _ptr(rows), _ptr(tokens),
              _ptr(penalties), n, _stream()), "apply_penalty")
    return logits


# ------------------------------------------------------------------ two branches on one residual
def add2_rmsnorm2(residual: torch.Tensor, delta_a: Optional[torch.Tensor], delta_b: Optional[torch.Tensor],
                  gain1: torch.Tensor, gain2: Optional[torch.Tensor], eps: float,
                  out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, delta_scale: float = 1.0):
    """residual += delta_scale * (delta_a + delta_b) (float32, in place; either may be None), then the two RMS
    norms of the same row, out_i = gain_i * x * rsqrt(mean(x^2) + eps).  ``gain2`` None: one norm.
    With ``rows`` (int32 [n]) output row i is made from batch row rows[i] and the residual is left
    alone.  Returns (out1, out2 or None)."""
    _need_cuda(residual, delta_a, delta_b, gain1, gain2, rows)
    _need_contiguous(residual, delta_a, delta_b, gain1, gain2, rows)
    d = residual.shape[-1]
    if residual.dtype != torch.float32 or residual.dim() != 2:
        raise KernelError("add2_rmsnorm2: the residual stream is float32 [T, W]")
    for g in (gain1, gain2):
        if g is not None and (g.dtype != torch.float32 or g.numel() != d):
            raise KernelError("add2_rmsnorm2: gains are float32 [W]")
    deltas = [x for x in (delta_a, delta_b) if x is not None]
    for x in deltas:
        if x.shape != residual.shape or x.dtype != deltas[0].dtype:
            raise KernelError("add2_rmsnorm2: the deltas have the residual's shape and one dtype")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("add2_rmsnorm2: rows must be int32")
    if d * 4 > 200 * 1024:
        raise KernelError(f"add2_rmsnorm2: a row of {d} floats does not fit in shared memory")
    n = residual.shape[0] if rows is None else rows.numel()
    out1 = torch.empty((n, d), dtype=out_dtype, device=residual.device)
    out2 = torch.empty((n, d), dtype=out_dtype, device=residual.device) if gain2 is not None else None
    fn = _fn("elementwise", "pbe_add2_rmsnorm2",
             [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
              c_float, c_float, c_void_p])
    _check(fn(_ptr(residual), _ptr(delta_a), _ptr(delta_b), _dtype_code(deltas[0]) if deltas else F32, _ptr(gain1),
              _ptr(gain2), _ptr(out1), _ptr(out2), _dtype_code(out1), _ptr(rows), n, d, float(eps),
              float(delta_scale), _stream()), "add2_rmsnorm2")
    return out1, out2


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    """relu(x)^2 element by element (float32 arithmetic, rounded once)."""
    _need_cuda(x)
    _need_contiguous(x)
    out = torch.empty_like(x)
    fn = _fn("elementwise", "pbe_relu_squared", [c_void_p, c_void_p, c_int, c_ll, c_void_p])
    _check(fn(_ptr(x), _ptr(out), _dtype_code(x), x.numel(), _stream()), "relu_squared")
    return out


def scale_softcap(logits: torch.Tensor, scale: float, cap: Optional[float]) -> torch.Tensor:
    """logits <- logits * scale, then (with a cap) cap * tanh(logits / cap); float32, in place."""
    _need_cuda(logits)
    _need_contiguous(logits)
    if logits.dtype != torch.float32:
        raise KernelError("scale_softcap: logits are float32")
    fn = _fn("elementwise", "pbe_scale_softcap", [c_void_p, c_ll, c_float, c_float, c_void_p])
    _check(fn(_ptr(logits), logits.numel(), float(scale), float(cap or 0.0), _stream()), "scale_softcap")
    return logits


# ------------------------------------------------------------------ short convolution, step sizes
def short_conv(u: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
               request_of_row: torch.Tensor, q_start: torch.Tensor, q_len: torch.Tensor, slots: torch.Tensor,
               num_requests: int, silu: bool = True, update_state: bool = True,
               weight_t: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal convolution per channel over each request's rows: ``u`` [T, C] a column slice of a
    projection, ``weight`` float32 [C, taps] (last column: the current token), ``state`` float32
    [slots, taps - 1, C] holding each request's last inputs (read, then moved on).  ``weight_t``:
    the same weights as float32 [taps, C], for the kernel that takes eight channels a thread.
    Returns [T, C] in u's dtype."""
    _need_cuda(u, weight, bias, state, request_of_row, q_start, q_len, slots, weight_t)
    _need_contiguous(weight, bias, state, weight_t)
    if weight_t is not None and (weight_t.dtype != torch.float32 or tuple(weight_t.shape) != (weight.shape[1], u.shape[1])):
        raise KernelError("short_conv: weight_t is float32 [taps, C]")
    _column_slice(u, "short_conv")
    T, C = u.shape
    taps = weight.shape[1]
    if weight.dtype != torch.float32 or weight.shape[0] != C or (bias is not None and (bias.dtype != torch.float32
                                                                                     or bias.numel() != C)):
        raise KernelError("short_conv: weight is float32 [C, taps], bias float32 [C]")
    if taps > 16:
        raise KernelError(f"short_conv: at most 16 taps, got {taps}")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (taps - 1, C):
        raise KernelError("short_conv: the state is float32 [slots, taps - 1, C]")
    for x in (request_of_row, q_start, q_len, slots):
        if x.dtype != torch.int32:
            raise KernelError("short_conv: the step's arrays are int32")
    out = torch.empty((T, C), dtype=u.dtype, device=u.device)
    ld = u.stride(0) if T > 1 else max(u.stride(0), C)
    fn = _fn("short_conv", "pbe_short_conv",
             [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    global _launches
    _check(fn(_ptr(u), ld, _dtype_code(u), _ptr(weight), _ptr(weight_t), _ptr(bias), _ptr(state), _ptr(out), _ptr(request_of_row),
              _ptr(q_start), _ptr(q_len), _ptr(slots), T, int(num_requests), C, taps, 1 if silu else 0,
              1 if update_state else 0, _stream()), "short_conv")
    if update_state and taps > 1:
        _launches += 1
    return out


def step_sizes(u: torch.Tensor, bias: torch.Tensor, rate_log: torch.Tensor):
    """(dt, decay), float32 [T, H]: dt = softplus(u + bias_h), decay = exp(-exp(rate_log_h) * dt);
    ``u`` [T, H] is a column slice of a projection."""
    _need_cuda(u, bias, rate_log)
    _column_slice(u, "step_sizes")
    T, H = u.shape
    if bias.dtype != torch.float32 or rate_log.dtype != torch.float32 or bias.numel() != H or rate_log.numel() != H:
        raise KernelError("step_sizes: bias and rate_log are float32 [H]")
    dt = torch.empty((T, H), dtype=torch.float32, device=u.device)
    decay = torch.empty((T, H), dtype=torch.float32, device=u.device)
    ld = u.stride(0) if T > 1 else max(u.stride(0), H)
    fn = _fn("short_conv", "pbe_step_sizes", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                              c_int, c_void_p])
    _check(fn(_ptr(u), ld, _dtype_code(u), _ptr(bias), _ptr(rate_log), _ptr(dt), _ptr(decay), T, H, _stream()),
           "step_sizes")
    return dt, decay


# ------------------------------------------------------------------ attention over a compressed latent
LATENT_TILE = 16     # packed rows (row x head) a block of the latent attention kernel takes
# bfloat16 caches whose rows are a multiple of 16 values wide run on the tensor-core kernel;
# PBE_LATENT=fma keeps them on the float32-arithmetic kernel (which every other case takes)
LATENT_FMA = os.environ.get("PBE_LATENT", "").strip().lower() == "fma"
LATENT_SUB = max(1, int(os.environ.get("PBE_LATENT_SUB", "4")))     # blocks that share a key split of a decode step


LATENT_WIDE_TILE = 64    # packed rows a block takes in steps with prompt portions (four groups of 16)


def latent_tile_rows(num_heads: int) -> int:
    """Packed rows of a row tile of the work list: all heads of a row lie in one tile, and a tile
    is whole blocks of either size."""
    return LATENT_WIDE_TILE * ((num_heads + LATENT_WIDE_TILE - 1) // LATENT_WIDE_TILE)


def latent_prepare(proj: torch.Tensor, q_off: int, q_rank: int, c_off: int, rank: int, r_off: int, rot: int,
                   q_gain: Optional[torch.Tensor], c_gain: torch.Tensor, inv_freq: Optional[torch.Tensor],
                   rot_dims: int, positions: torch.Tensor, slots: Optional[torch.Tensor],
                   cache: Optional[torch.Tensor], eps: float, rot_scale: float = 1.0) -> Optional[torch.Tensor]:
    """From the fused down projection [T, ld]: the RMS-normed query latent (returned, [T, q_rank];
    None when q_rank is 0) and, written into ``cache`` ([page, 1, page_tokens, rank + rot]) at
    ``slots``: the RMS-normed latent c followed by the rotated shared key part (cos and sin of the
    rotation both times ``rot_scale``)."""
    _need_cuda(proj, q_gain, c_gain, inv_freq, positions, slots, cache)
    _need_contiguous(proj, q_gain, c_gain, inv_freq, positions, slots, cache)
    T = proj.shape[0]
    if cache is not None and (cache.dtype != proj.dtype or cache.shape[-1] != rank + rot or cache.shape[1] != 1):
        raise KernelError("latent_prepare: cache pages are [page, 1, page_tokens, rank + rot] in the activations' dtype")
    if c_gain.dtype != torch.float32 or c_gain.numel() != rank or (q_rank and (q_gain.dtype != torch.float32
                                                                              or q_gain.numel() != q_rank)):
        raise KernelError("latent_prepare: gains are float32 of the latents' widths")
    if rot_dims and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2):
        raise KernelError("latent_prepare: inv_freq is float32 [rot_dims / 2]")
    if rot_dims > rot or rot % 2 or rot_dims % 2:
        raise KernelError("latent_prepare: the rotated part is even and at least rot_dims wide")
    q_lat = torch.empty((T, q_rank), dtype=proj.dtype, device=proj.device) if q_rank else None
    fn = _fn("latent_attention", "pbe_latent_prepare",
             [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
              c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p])
    _check(fn(_ptr(proj), proj.stride(0), _dtype_code(proj), q_off, q_rank, c_off, rank, r_off, rot, _ptr(q_gain),
              _ptr(c_gain), _ptr(inv_freq), int(rot_dims), float(rot_scale), _ptr(positions), _ptr(slots), _ptr(q_lat), _ptr(cache),
              float(eps), T, _stream()), "latent_prepare")
    return q_lat


def head_product(a: torch.Tensor, lda: int, head_stride: int, K: int, w: torch.Tensor, w_head_stride: int,
                 wk: int, wn: int, N: int, out: torch.Tensor, ldo: int, out_head_stride: int, T: int, H: int,
                 rot: int = 0, rot_dims: int = 0, inv_freq: Optional[torch.Tensor] = None,
                 positions: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                 rot_scale: float = 1.0, gate_each: bool = False) -> torch.Tensor:
    """out[t, h, n] = sum_k a[t, h, k] * w[h][k * wk + n * wn] for n < N, per head, float32 sums in
    k order.  ``rot`` > 0: out[t, h, N : N + rot] = the rotation of a[t, h, K : K + rot] by the rows'
    positions (pairs (2i, 2i + 1) of its first ``rot_dims`` values; cos and sin both times
    ``rot_scale``).  ``gate`` [T, >= H] (a column slice in the weights' dtype): the result is
    multiplied by sigmoid(gate[t, h]); with ``gate_each`` the gate is [T, >= H * N] and has a value
    for every output, sigmoid(gate[t, h * N + n])."""
    _need_cuda(a, w, out, inv_freq, positions, gate)
    if gate is not None and (gate.stride(1) != 1 or gate.dtype != w.dtype):
        raise KernelError("head_product: the gate is a column slice in the weights' dtype")
    fn = _fn("latent_attention", "pbe_head_product",
             [c_void_p, c_int, c_int, c_int, c_void_p, c_ll, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
              c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p])
    ldg = 0
    if gate is not None:
        ldg = gate.stride(0) if T > 1 else max(gate.stride(0), H * (N if gate_each else 1))
    _check(fn(_ptr(a), int(lda), int(head_stride), _dtype_code(a), _ptr(w), int(w_head_stride), int(wk), int(wn),
              _dtype_code(w), _ptr(out), int(ldo), int(out_head_stride), _dtype_code(out), int(T), int(H), int(K),
              int(N), int(rot), int(rot_dims), _ptr(inv_freq), _ptr(positions), _ptr(gate), int(ldg),
              float(rot_scale), 1 if gate_each else 0, _stream()),
           "head_product")
    return out


def latent_attention(q: torch.Tensor, cache: torch.Tensor, sink: Optional[torch.Tensor], meta, num_heads: int,
                     value_width: int, scale: float, window, page_tokens: int) -> torch.Tensor:
    """Causal attention of every row over its request's cached rows, all heads sharing them:
    ``q`` float32 [T, H, dk], ``cache`` [page, 1, page_tokens, dk] whose first ``value_width``
    values of a row are the value; ``sink`` float32 [H] joins each head's softmax denominator.
    ``meta``: the step's work list for (group, H heads a group, ``latent_tile_rows(H)``, window).
    Returns float32 [T, H, value_width]."""
    _need_cuda(q, cache, sink)
    _need_contiguous(q, cache, sink)
    T, H, dk = q.shape
    if q.dtype != torch.float32 or H != num_heads or cache.shape[-1] != dk or cache.shape[1] != 1:
        raise KernelError("latent_attention: q is float32 [T, H, dk], the cache [page, 1, page_tokens, dk]")
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != H):
        raise KernelError("latent_attention: the sink is float32 [H]")
    if value_width > 512 or value_width > dk:
        raise KernelError("latent_attention: the value is at most 512 wide and a prefix of the cached row")
    if (dk * 16 + (dk | 1) * 32) * 4 > 200 * 1024:
        raise KernelError(f"latent_attention: cached rows of {dk} values do not fit in shared memory")
    out = torch.empty((T, H, value_width), dtype=torch.float32, device=q.device)
    mode = 0 if (LATENT_FMA or cache.dtype != torch.bfloat16 or dk % 16) else (1 if meta.decode_rows > 0 else 2)
    # steps of decoded tokens in which every row's keys are split: four blocks share each split, so
    # that few long requests still fill the GPU (8 requests at 2,048 keys: 64 -> 256 blocks)
    sub = LATENT_SUB if (mode == 1 and meta.num_split_rows == T and meta.split_keys % (LATENT_SUB * 32) == 0) else 1
    slots = meta.max_splits * sub
    part_o = part_ml = None
    if meta.num_split_rows:
        part_o, part_ml = meta.part_o, meta.part_ml       # the step's buffers, when they have this shape
        if part_o is None or tuple(part_o.shape) != (meta.num_split_rows, H, slots, value_width):
            part_o = torch.empty((meta.num_split_rows, H, slots, value_width), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((meta.num_split_rows, H, slots, 2), dtype=torch.float32, device=q.device)
    p = AttnParams(
        q=q.data_ptr(), k_cache=cache.data_ptr(), v_cache=cache.data_ptr(), out=out.data_ptr(),
        part_o=part_o.data_ptr() if part_o is not None else None,
        part_ml=part_ml.data_ptr() if part_ml is not None else None,
        q_start=meta.q_start.data_ptr(), q_len=meta.q_len.data_ptr(), seq_len=meta.seq_len.data_ptr(),
        block_table=meta.block_table.data_ptr(), work=meta.work.data_ptr(),
        tok_split_row=meta.tok_split_row.data_ptr(), bt_stride=int(meta.bt_stride),
        num_heads=int(H), num_kv_heads=1, page_tokens=int(page_tokens),
        window=int(window or 0), split_keys=int(meta.split_keys), max_splits=int(meta.max_splits),
        tile_rows=int(meta.tile_rows), scale=float(scale), kinds=0, num_pages=int(cache.shape[0]))
    fn = _fn("latent_attention", "pbe_latent_attention",
             [ctypes.POINTER(AttnParams), c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(ctypes.byref(p), _ptr(sink), dk, int(value_width), int(meta.num_work), _dtype_code(cache),
              mode, sub, _stream()), "latent_attention")
    if meta.num_split_rows > 0:
        mp = AttnMergeParams(part_o=part_o.data_ptr(), part_ml=part_ml.data_ptr(), out=out.data_ptr(),
                             split_tokens=meta.split_tokens.data_ptr(), split_counts=meta.split_counts.data_ptr(),
                             num_heads=int(H), head_dim=int(value_width), max_splits=int(slots))
        mfn = _fn("latent_attention", "pbe_latent_merge", [ctypes.POINTER(AttnMergeParams), c_void_p, c_int, c_int,
                                                           c_void_p])
        _check(mfn(ctypes.byref(mp), _ptr(sink), sub, int(meta.num_split_rows), _stream()), "latent_merge")
    return out


# ------------------------------------------------------------------ masked attention (head norms, bias, sink, gate)
MASKED_TILE_ROWS = 16     # packed rows (row x head of a key/value group) a block of the float32 masked attention takes
MASKED_MMA_TILE_ROWS = 64  # and a block of the tensor-core one
MASK_KINDS = {None: 0, "causal": 0, "window": 1, "chunk": 2}


def masked_mma_applies(dtype: torch.dtype, key_dim: int, value_dim: int) -> bool:
    """bfloat16 pages with head widths that are multiples of 16 run the masked attention on the tensor
    cores; PBE_MASKED=plain keeps them on the float32-arithmetic kernel."""
    return (dtype == torch.bfloat16 and key_dim % 16 == 0 and value_dim % 16 == 0 and 16 <= key_dim <= 256
            and 16 <= value_dim <= 256 and os.environ.get("PBE_MASKED", "").strip().lower() != "plain")


def masked_tile_rows(dtype: torch.dtype, key_dim: int, value_dim: int) -> int:
    """Packed rows a work item of ``masked_attention`` takes for these pages."""
    return MASKED_MMA_TILE_ROWS if masked_mma_applies(dtype, key_dim, value_dim) else MASKED_TILE_ROWS


def masked_libraries(dtype: torch.dtype, key_dim: int, value_dim: int):
    """The (library, defines) pairs of the masked attention for these pages (for parallel builds)."""
    jobs = [("masked_attention", None)]
    if masked_mma_applies(dtype, key_dim, value_dim):
        jobs.append(("masked_attention_mma", {"PBE_MA_D": int(key_dim), "PBE_MA_E": int(value_dim)}))
    return jobs


def head_norm_write(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, bias: Optional[torch.Tensor],
                    q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                    k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], num_heads: int,
                    num_kv_heads: int, key_dim: int, value_dim: int, page_tokens: int, eps: float,
                    q_head_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """From a fused projection [T, ld] (queries at column ``q_off``, keys at ``k_off``, values at
    ``v_off``): ``bias`` (float32, indexed like the columns) added, an RMS norm over each query and
    key head's ``key_dim`` elements with the gains ``q_gain`` / ``k_gain`` (float32 [key_dim], shared
    by the heads; None: no norm), all in float32; ``q_head_scale`` (float32 [H]) multiplies head h's
    normed query (a temperature per head).  Returns the queries, float32 [T, H * D]; keys go to
    ``k_pages`` [page, G, page_tokens, D] and values to ``v_pages`` [page, G, page_tokens, E] at
    ``slots`` (None or a negative slot: nothing is written)."""
    _need_cuda(proj, bias, q_gain, k_gain, slots, k_pages, v_pages, q_head_scale)
    _need_contiguous(bias, q_gain, k_gain, slots, k_pages, v_pages, q_head_scale)
    if q_head_scale is not None and (q_head_scale.dtype != torch.float32 or q_head_scale.numel() != num_heads):
        raise KernelError("head_norm_write: the heads' factors are float32 [H]")
    if proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("head_norm_write: the projection is [T, ld] with unit column stride")
    T = proj.shape[0]
    H, G, D, E = num_heads, num_kv_heads, key_dim, value_dim
    if D > 256:
        raise KernelError("head_norm_write: heads are at most 256 wide")
    for g in (q_gain, k_gain):
        if g is not None and (g.dtype != torch.float32 or g.numel() != D):
            raise KernelError("head_norm_write: gains are float32 [key_dim]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() < max(q_off + H * D, k_off + G * D,
                                                                              v_off + G * E)):
        raise KernelError("head_norm_write: the bias is float32 and covers the projection's columns")
    if k_pages is not None and (k_pages.dtype != proj.dtype or tuple(k_pages.shape[1:]) != (G, page_tokens, D)
                                or v_pages is None or tuple(v_pages.shape[1:]) != (G, page_tokens, E)):
        raise KernelError("head_norm_write: pages are [page, G, page_tokens, D] and [page, G, page_tokens, E]")
    q = torch.empty((T, H * D), dtype=torch.float32, device=proj.device)
    fn = _fn("masked_attention", "pbe_head_norm_write",
             [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_ptr(proj), proj.stride(0), int(q_off), int(k_off), int(v_off), _ptr(bias), _ptr(q_gain), _ptr(k_gain),
              _ptr(q_head_scale), _ptr(slots if k_pages is not None else None), _ptr(q), _ptr(k_pages), _ptr(v_pages), T, H, G, D, E,
              int(page_tokens), float(eps), _dtype_code(proj), _stream()), "head_norm_write")
    return q


def masked_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, meta, num_heads: int,
                     num_kv_heads: int, scale: float, mask: Optional[str], mask_size: Optional[int],
                     page_tokens: int, bias: Optional[torch.Tensor] = None, unit_sink: bool = False,
                     gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax attention of every row over its request's pages.  ``q`` float32 [T, H * D]; pages
    [page, G, page_tokens, D] and [page, G, page_tokens, E].  ``mask``: None / "causal" (every earlier
    key), "window" (the last ``mask_size`` keys) or "chunk" (the earlier keys of the row's own chunk of
    ``mask_size`` positions).  ``bias`` float32 [H, rows]: bias[h, min(distance, rows - 1)] is added to
    the scaled score.  ``unit_sink``: one more term e^0 in the denominator.  ``gate`` [T, >= H * E] (a
    column slice in the pages' dtype): the output times its sigmoid.  ``meta``: the step's work list
    for (group, H / G, ``masked_tile_rows(dtype, D, E)``, ``mask_size``).  Returns [T, H * E] in the
    pages' dtype.  Arithmetic is float32 throughout; on the tensor-core path the float32 queries and
    softmax weights enter the products as two bfloat16 numbers each."""
    _need_cuda(q, k_pages, v_pages, bias, gate)
    _need_contiguous(q, k_pages, v_pages, bias)
    T = q.shape[0]
    H, G = num_heads, num_kv_heads
    D, E = k_pages.shape[-1], v_pages.shape[-1]
    if q.dtype != torch.float32 or q.shape[1] != H * D or k_pages.dtype != v_pages.dtype:
        raise KernelError("masked_attention: q is float32 [T, H * D]; the pages share a dtype")
    if mask not in MASK_KINDS or (MASK_KINDS[mask] and not mask_size):
        raise KernelError(f"masked_attention: unknown mask {mask!r}, or a mask without its size")
    if bias is not None and (bias.dtype != torch.float32 or bias.dim() != 2 or bias.shape[0] != H):
        raise KernelError("masked_attention: the bias is float32 [H, rows]")
    if gate is not None and (gate.dtype != k_pages.dtype or gate.stride(1) != 1 or gate.shape[1] < H * E):
        raise KernelError("masked_attention: the gate is a column slice [T, H * E] in the pages' dtype")
    if E > 256:
        raise KernelError("masked_attention: values are at most 256 wide")
    out = torch.empty((T, H * E), dtype=k_pages.dtype, device=q.device)
    part_o = part_ml = None
    if meta.num_split_rows:
        part_o, part_ml = meta.part_o, meta.part_ml
        if part_o is None or tuple(part_o.shape) != (meta.num_split_rows, H, meta.max_splits, E):
            part_o = torch.empty((meta.num_split_rows, H, meta.max_splits, E), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((meta.num_split_rows, H, meta.max_splits, 2), dtype=torch.float32, device=q.device)
    ldg = 0
    if gate is not None:
        ldg = gate.stride(0) if T > 1 else max(gate.stride(0), H * E)
    p = AttnParams(
        q=q.data_ptr(), k_cache=k_pages.data_ptr(), v_cache=v_pages.data_ptr(), out=out.data_ptr(),
        part_o=part_o.data_ptr() if part_o is not None else None,
        part_ml=part_ml.data_ptr() if part_ml is not None else None,
        q_start=meta.q_start.data_ptr(), q_len=meta.q_len.data_ptr(), seq_len=meta.seq_len.data_ptr(),
        block_table=meta.block_table.data_ptr(), work=meta.work.data_ptr(),
        tok_split_row=meta.tok_split_row.data_ptr(), bt_stride=int(meta.bt_stride),
        num_heads=int(H), num_kv_heads=int(G), page_tokens=int(page_tokens),
        window=int(mask_size or 0), split_keys=int(meta.split_keys), max_splits=int(meta.max_splits),
        tile_rows=int(meta.tile_rows), scale=float(scale), kinds=0, num_pages=int(k_pages.shape[0]))
    if masked_mma_applies(k_pages.dtype, D, E):
        fn = _fn("masked_attention_mma", "pbe_masked_attention_mma",
                 [ctypes.POINTER(AttnParams), c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p],
                 {"PBE_MA_D": int(D), "PBE_MA_E": int(E)})
        _check(fn(ctypes.byref(p), _ptr(bias), bias.shape[1] if bias is not None else 0, MASK_KINDS[mask],
                  1 if unit_sink else 0, _ptr(gate), int(ldg), int(meta.num_work), _stream()), "masked_attention_mma")
    else:
        fn = _fn("masked_attention", "pbe_masked_attention",
                 [ctypes.POINTER(AttnParams), c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int,
                  c_int, c_void_p])
        _check(fn(ctypes.byref(p), int(D), int(E), _ptr(bias), bias.shape[1] if bias is not None else 0,
                  MASK_KINDS[mask], 1 if unit_sink else 0, _ptr(gate), int(ldg), int(meta.num_work),
                  _dtype_code(k_pages), _stream()), "masked_attention")
    if meta.num_split_rows > 0:
        mp = AttnMergeParams(part_o=part_o.data_ptr(), part_ml=part_ml.data_ptr(), out=out.data_ptr(),
                             split_tokens=meta.split_tokens.data_ptr(), split_counts=meta.split_counts.data_ptr(),
                             num_heads=int(H), head_dim=int(E), max_splits=int(meta.max_splits))
        mfn = _fn("masked_attention", "pbe_masked_merge",
                  [ctypes.POINTER(AttnMergeParams), c_int, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(mfn(ctypes.byref(mp), 1 if unit_sink else 0, _ptr(gate), int(ldg), int(meta.num_split_rows),
                   _dtype_code(k_pages), _stream()), "masked_merge")
    return out


# ------------------------------------------------------------------ routed experts
ROUTER_SCORES = {"softmax": 0, "sigmoid": 1}
GROUP_RANKS = {"max": 1, "top2_sum": 2}


def route(logits: torch.Tensor, top: int, groups: int, keep: int, scale: float, score: str = "softmax",
          correction: Optional[torch.Tensor] = None, group_rank: str = "max"):
    """(chosen int32 [T, top], weights float32 [T, top]) from float32 router logits [T, E]: scores
    by ``score`` ("softmax" over the experts or "sigmoid" of each logit); the choice is made on the
    scores plus ``correction`` (float32 [E], optional): experts outside the ``keep`` best of
    ``groups`` neighbouring groups barred (a group ranks by ``group_rank``: its "max" or its
    "top2_sum"), the top ones chosen; weights = score (uncorrected) / (sum of the chosen + 1e-20) *
    scale."""
    _need_cuda(logits, correction)
    _need_contiguous(logits, correction)
    if score not in ROUTER_SCORES or group_rank not in GROUP_RANKS:
        raise KernelError(f"route: scores are one of {sorted(ROUTER_SCORES)}, group ranks one of {sorted(GROUP_RANKS)}")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != logits.shape[1]):
        raise KernelError("route: the correction is float32 [E]")
    T, E = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("route: router logits are float32")
    if E > 512 or top > 32 or groups > 64:
        raise KernelError("route: at most 512 experts, 32 chosen and 64 groups")
    chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    fn = _fn("routed_experts", "pbe_route", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                            c_int, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(logits), _ptr(chosen), _ptr(weights), T, E, int(top), int(groups), int(keep), float(scale),
              ROUTER_SCORES[score], _ptr(correction), GROUP_RANKS[group_rank], _stream()), "route")
    return chosen, weights


def expert_rows(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                chosen: torch.Tensor, weights: torch.Tensor, activation: str = "silu", limit: float = 0.0,
                alpha: float = 1.0, addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = (addend[t], optional) + sum_k weights[t, k] * W_down[e] act(W_gate[e] x_t, W_up[e] x_t), e = chosen[t, k]:
    a block per (row, chosen expert) streams that expert's matrices; for few rows.  ``w_gate_up``
    [E, 2F, W]: an expert's gate rows followed by its up rows; ``w_down`` [E, W, F].  ``activation``:
    one of ``GLU_ACTIVATIONS`` (see ``gated_activation``)."""
    _need_cuda(x, w_gate_up, w_down, chosen, weights)
    _need_contiguous(x, w_gate_up, w_down, chosen, weights)
    T, W = x.shape
    E, F2, _ = w_gate_up.shape
    F = F2 // 2
    top = chosen.shape[1]
    if F2 % 2 or tuple(w_down.shape) != (E, W, F) or w_gate_up.shape[2] != W:
        raise KernelError("expert_rows: gate/up is [E, 2F, W], down is [E, W, F]")
    if not (x.dtype == w_gate_up.dtype == w_down.dtype):
        raise KernelError("expert_rows: rows and expert matrices share a dtype")
    if (W + F) * 4 > 200 * 1024:
        raise KernelError("expert_rows: a row and an expert's hidden units do not fit in shared memory")
    hidden = torch.empty((T * top, F), dtype=torch.float32, device=x.device)
    part = torch.empty((T, top, W), dtype=torch.float32, device=x.device)
    out = torch.empty((T, W), dtype=x.dtype, device=x.device)
    if addend is not None and (addend.shape != x.shape or addend.dtype != x.dtype or not addend.is_cuda
                               or not addend.is_contiguous()):
        raise KernelError("expert_rows: the addend has the rows' shape and dtype")
    fn = _fn("routed_experts", "pbe_expert_rows", [c_void_p] * 3 + [c_ll] + [c_void_p] * 6 + [c_int] * 6 +
             [c_float, c_float, c_void_p, c_void_p])
    global _launches
    up = c_void_p(w_gate_up.data_ptr() + F * W * w_gate_up.element_size())
    _check(fn(_ptr(x), _ptr(w_gate_up), up, 2 * F * W, _ptr(w_down), _ptr(chosen), _ptr(weights), _ptr(hidden),
              _ptr(part), _ptr(out), _dtype_code(x), T, W, F, top, GLU_ACTIVATIONS[activation], float(limit),
              float(alpha), _ptr(addend), _stream()), "expert_rows")
    _launches += 2
    return out


def expert_places(chosen: torch.Tensor, num_experts: int):
    """(counts int32 [E], place int32 [T * top]): how many (row, k) pairs chose each expert, and each
    pair's place inside its expert's run, in pair order."""
    _need_cuda(chosen)
    _need_contiguous(chosen)
    pairs = chosen.numel()
    counts = torch.empty(num_experts, dtype=torch.int32, device=chosen.device)
    place = torch.empty(pairs, dtype=torch.int32, device=chosen.device)
    fn = _fn("routed_experts", "pbe_expert_places", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(chosen), pairs, int(num_experts), _ptr(counts), _ptr(place), _stream()), "expert_places")
    return counts, place


def expert_gather(x: torch.Tensor, chosen: torch.Tensor, place: torch.Tensor, start: torch.Tensor,
                  total_rows: Optional[int] = None) -> torch.Tensor:
    """The rows of x once per chosen expert, sorted by expert: row start[e] + place[pair] = x[t].
    ``total_rows``: rows of the result when the experts' runs are padded (rows between the runs are
    left as they are)."""
    _need_cuda(x, chosen, place, start)
    _need_contiguous(x, chosen, place, start)
    T, W = x.shape
    top = chosen.shape[1]
    out = torch.empty((total_rows or T * top, W), dtype=x.dtype, device=x.device)
    fn = _fn("routed_experts", "pbe_expert_gather", [c_void_p] * 5 + [c_int] * 4 + [c_void_p])
    _check(fn(_ptr(x), _ptr(chosen), _ptr(place), _ptr(start), _ptr(out), _dtype_code(x), T, top, W, _stream()),
           "expert_gather")
    return out


def expert_scatter(y: torch.Tensor, chosen: torch.Tensor, place: torch.Tensor, start: torch.Tensor,
                   weights: torch.Tensor, T: int, addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_k weights[t, k] * y[start[e] + place[(t, k)]], e = chosen[t, k], in k order, plus
    ``addend`` [T, W] (optional, y's dtype)."""
    _need_cuda(y, chosen, place, start, weights, addend)
    _need_contiguous(y, chosen, place, start, weights, addend)
    if addend is not None and (tuple(addend.shape) != (T, y.shape[1]) or addend.dtype != y.dtype):
        raise KernelError("expert_scatter: the addend is [T, W] in the rows' dtype")
    W = y.shape[1]
    top = chosen.shape[1]
    out = torch.empty((T, W), dtype=y.dtype, device=y.device)
    fn = _fn("routed_experts", "pbe_expert_scatter", [c_void_p] * 6 + [c_int] * 4 + [c_void_p, c_void_p])
    _check(fn(_ptr(y), _ptr(chosen), _ptr(place), _ptr(start), _ptr(weights), _ptr(out), _dtype_code(y), T, top, W,
              _ptr(addend), _stream()), "expert_scatter")
    return out


# ------------------------------------------------------------------ many small products in one launch
GROUP_TILE_ROWS = 64     # rows of a tile of the grouped product (runs of rows are padded to it)


def _grouped(a, lda, a_group, w, w_group, wk, wn, out, ldo, out_group, T, K, N, groups, tiles, num_tiles,
             gate=None, rot=0, rot_dims=0, inv_freq=None, positions=None, rot_scale=1.0, gate_each=False):
    _need_cuda(a, w, out, tiles, gate, inv_freq, positions)
    if w.dtype != torch.bfloat16 or (gate is not None and (gate.dtype != torch.bfloat16 or gate.stride(1) != 1)):
        raise KernelError("grouped product: weights (and the gate) are bfloat16")
    fn = _fn("grouped_gemm", "pbe_grouped_gemm",
             [c_void_p, c_int, c_int, c_ll, c_void_p, c_ll, c_int, c_int, c_void_p, c_int, c_int, c_ll, c_int, c_int, c_int,
              c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p])
    ldg = 0
    if gate is not None:
        ldg = gate.stride(0) if T > 1 else max(gate.stride(0), groups * (N if gate_each else 1))
    _check(fn(_ptr(a), _dtype_code(a), int(lda), int(a_group), _ptr(w), int(w_group), int(wk), int(wn), _ptr(out),
              _dtype_code(out), int(ldo), int(out_group), int(T), int(K), int(N), int(groups), _ptr(tiles),
              int(num_tiles), _ptr(gate), int(ldg), int(rot), int(rot_dims), _ptr(inv_freq), _ptr(positions),
              float(rot_scale), 1 if gate_each else 0, _stream()), "grouped_gemm")
    return out


def grouped_heads(a: torch.Tensor, lda: int, head_stride: int, K: int, w: torch.Tensor, w_head_stride: int,
                  wk: int, wn: int, N: int, out: torch.Tensor, ldo: int, out_head_stride: int, T: int, H: int,
                  rot: int = 0, rot_dims: int = 0, inv_freq: Optional[torch.Tensor] = None,
                  positions: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                  rot_scale: float = 1.0, gate_each: bool = False) -> torch.Tensor:
    """``head_product`` on the tensor cores: the same arguments and result; ``a`` bfloat16 or float32
    (rounded to bfloat16 as an operand), ``w`` and ``gate`` bfloat16, float32 sums."""
    return _grouped(a, lda, head_stride, w, w_head_stride, wk, wn, out, ldo, out_head_stride, T, K, N, H, None, 0,
                    gate, rot, rot_dims, inv_freq, positions, rot_scale, gate_each)


def run_tiles(counts: torch.Tensor, max_tiles: int):
    """(start int32 [G], tiles int32 [max_tiles, 3]) for rows sorted by group with every group's run
    padded to whole tiles of ``GROUP_TILE_ROWS``: a group's first row, and per tile (group, first
    row, rows), idle tiles with group -1."""
    _need_cuda(counts)
    G = counts.numel()
    start = torch.empty(G, dtype=torch.int32, device=counts.device)
    tiles = torch.empty((max_tiles, 3), dtype=torch.int32, device=counts.device)
    fn = _fn("grouped_gemm", "pbe_run_tiles", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(counts), G, int(max_tiles), _ptr(start), _ptr(tiles), _stream()), "run_tiles")
    return start, tiles


def grouped_runs(a: torch.Tensor, w: torch.Tensor, tiles: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """out[row] = W[g] a[row] for the rows of every tile (group g): ``a`` [rows, K] sorted by group,
    ``w`` bfloat16 [G, N, K], ``tiles`` from ``run_tiles``."""
    _need_contiguous(a, w, tiles)
    rows, K = a.shape
    G, N, _ = w.shape
    if w.shape[2] != K:
        raise KernelError("grouped_runs: the weights are [G, N, K]")
    out = torch.empty((rows, N), dtype=out_dtype, device=a.device)
    return _grouped(a, K, 0, w, N * K, 1, K, out, N, 0, rows, K, N, G, tiles, tiles.shape[0])


# ------------------------------------------------------------------ norms with one learned number, mix over depth
def unit_norm(x: torch.Tensor, y1: Optional[torch.Tensor], y2: Optional[torch.Tensor], alpha: float, gain: torch.Tensor,
              eps: float, lp_dtype: Optional[torch.dtype] = None, normed: Optional[torch.Tensor] = None,
              stack: Optional[torch.Tensor] = None, n_prev: int = 0, mix: Optional[torch.Tensor] = None,
              mixed: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
              sum_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """n = g * v / sqrt(mean(v^2) + eps) with v = alpha * x + y1 + y2 (float32; ``gain`` holds the one
    number g; y1, y2 optional, in one dtype).  ``normed`` (float32 [T, W]) receives n, ``sum_out``
    (float32 [T, W]) receives v.  With ``mix`` (float32 [n_prev + 1]) and ``stack`` (float32
    [>= n_prev, T, W], the earlier results), ``mixed`` receives sum_j mix[j] stack[j] + mix[n_prev] n.
    Returns a copy of the last of these (the mix if there is one, else n) in ``lp_dtype``, or None
    when ``lp_dtype`` is None.  With ``rows`` (int32 [n]) output row i is made from row rows[i]."""
    _need_cuda(x, y1, y2, gain, normed, stack, mix, mixed, rows, sum_out)
    _need_contiguous(x, y1, y2, normed, stack, mix, mixed, rows, sum_out)
    if x.dtype != torch.float32 or x.dim() != 2 or gain.dtype != torch.float32 or gain.numel() != 1:
        raise KernelError("unit_norm: x is float32 [T, W], the gain one float32 number")
    T, d = x.shape
    ys = [y for y in (y1, y2) if y is not None]
    for y in ys:
        if y.shape != x.shape or y.dtype != ys[0].dtype:
            raise KernelError("unit_norm: the branch outputs have x's shape and one dtype")
    if y1 is None and y2 is not None:
        y1, y2 = y2, None
    n = T if rows is None else rows.numel()
    if rows is not None and (rows.dtype != torch.int32 or sum_out is not None):
        raise KernelError("unit_norm: rows are int32, and gathered rows write no sum back")
    for o in (normed, mixed):
        if o is not None and (o.dtype != torch.float32 or tuple(o.shape) != (n, d)):
            raise KernelError("unit_norm: float32 outputs are [rows, W]")
    if sum_out is not None and (sum_out.dtype != torch.float32 or sum_out.shape != x.shape):
        raise KernelError("unit_norm: the sum is float32 [T, W]")
    stride = 0
    if mix is not None:
        if mix.dtype != torch.float32 or mix.numel() != n_prev + 1:
            raise KernelError("unit_norm: the mix is float32 [n_prev + 1]")
        if n_prev > 0:
            if stack is None or stack.dtype != torch.float32 or stack.dim() != 3 or stack.shape[0] < n_prev or \
                    tuple(stack.shape[1:]) != (T, d):
                raise KernelError("unit_norm: the stack is float32 [>= n_prev, T, W]")
            stride = stack.stride(0)
    if d * 4 > 200 * 1024:
        raise KernelError(f"unit_norm: a row of {d} floats does not fit in shared memory")
    lp = torch.empty((n, d), dtype=lp_dtype, device=x.device) if lp_dtype is not None else None
    fn = _fn("unit_norm", "pbe_unit_norm",
             [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_ll, c_int,
              c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(y1), _ptr(y2), _dtype_code(ys[0]) if ys else F32, float(alpha), _ptr(gain), float(eps),
              _ptr(sum_out), _ptr(normed), _ptr(stack if mix is not None and n_prev > 0 else None), int(stride),
              int(n_prev), _ptr(mix), _ptr(mixed), _ptr(lp), _dtype_code(lp) if lp is not None else F32, _ptr(rows), n, d,
              _stream()), "unit_norm")
    return lp


def embedding_unit_norm(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, gain: torch.Tensor, eps: float,
                        lp_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """out[t] = g * e / sqrt(mean(e^2) + eps), e = table[ids[t]], float32; also returned in ``lp_dtype``
    (None: no copy)."""
    _need_cuda(out, table, ids, gain)
    _need_contiguous(out, table, ids)
    T, d = out.shape
    if out.dtype != torch.float32 or ids.dtype != torch.int32 or table.shape[1] != d or ids.numel() != T:
        raise KernelError("embedding_unit_norm: float32 rows from int32 ids, widths agree")
    if gain.dtype != torch.float32 or gain.numel() != 1:
        raise KernelError("embedding_unit_norm: the gain is one float32 number")
    lp = torch.empty((T, d), dtype=lp_dtype, device=out.device) if lp_dtype is not None else None
    fn = _fn("unit_norm", "pbe_embedding_unit_norm",
             [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(out), _ptr(lp), _dtype_code(lp) if lp is not None else F32, _ptr(table), _dtype_code(table), _ptr(ids),
              _ptr(gain), T, d, table.shape[0], float(eps), _stream()), "embedding_unit_norm")
    return lp


# ------------------------------------------------------------------ gated diagonal linear recurrence
def recurrence_gates(u: torch.Tensor, w_r: torch.Tensor, w_i: torch.Tensor, b_r: torch.Tensor, b_i: torch.Tensor,
                     lam: torch.Tensor, rate: float):
    """(a, b), float32 [T, C]: with r = sigmoid(R u + b_r) and i = sigmoid(I u + b_i), R and I block
    diagonal (``w_r``, ``w_i`` [B, C/B, C/B], [out, in]), a = exp(-rate * r * softplus(lam)) and
    b = sqrt(1 - a^2) * i * u; all float32 arithmetic.  ``u`` [T, C] may be a column slice."""
    _need_cuda(u, w_r, w_i, b_r, b_i, lam)
    _need_contiguous(w_r, w_i, b_r, b_i, lam)
    _column_slice(u, "recurrence_gates")
    T, C = u.shape
    B, n = w_r.shape[0], w_r.shape[1]
    if tuple(w_r.shape) != (B, n, n) or w_i.shape != w_r.shape or B * n != C or w_i.dtype != w_r.dtype:
        raise KernelError("recurrence_gates: the gate maps are [B, C/B, C/B] in one dtype")
    for v in (b_r, b_i, lam):
        if v.dtype != torch.float32 or v.numel() != C:
            raise KernelError("recurrence_gates: gate biases and lam are float32 [C]")
    a = torch.empty((T, C), dtype=torch.float32, device=u.device)
    b = torch.empty((T, C), dtype=torch.float32, device=u.device)
    ld = u.stride(0) if T > 1 else max(u.stride(0), C)
    fn = _fn("gated_recurrence", "pbe_recurrence_gates",
             [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
              c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(u), ld, _dtype_code(u), _ptr(w_r), _ptr(w_i), _dtype_code(w_r), _ptr(b_r), _ptr(b_i), _ptr(lam),
              float(rate), _ptr(a), _ptr(b), T, C, B, _stream()), "recurrence_gates")
    return a, b


SCAN_ACTIVATIONS = {None: 0, "gelu_tanh": 1}


def gate_products(u: torch.Tensor, w_gates: torch.Tensor) -> torch.Tensor:
    """z, float32 [T, B, 2n]: per block b of the channels the pre-activations [R_b u_b | I_b u_b] of both
    gates, on the tensor cores; ``u`` bfloat16 [T, B*n] (possibly a column slice), ``w_gates`` bfloat16
    [B, 2n, n], a block's recurrence-gate rows followed by its input-gate rows.  Products of two
    bfloat16 numbers are exact in float32 and the sums are float32."""
    _need_cuda(u, w_gates)
    _need_contiguous(w_gates)
    _column_slice(u, "gate_products")
    T, C = u.shape
    B, n2, n = w_gates.shape
    if n2 != 2 * n or B * n != C or u.dtype != torch.bfloat16 or w_gates.dtype != torch.bfloat16:
        raise KernelError("gate_products: bfloat16 input [T, B*n] and maps [B, 2n, n]")
    z = torch.empty((T, B, 2 * n), dtype=torch.float32, device=u.device)
    ld = u.stride(0) if T > 1 else max(u.stride(0), C)
    return grouped_heads(u, ld, n, n, w_gates, 2 * n * n, 1, n, 2 * n, z, B * 2 * n, 2 * n, T, B)


def gated_scan(a: Optional[torch.Tensor], b: Optional[torch.Tensor], y: Optional[torch.Tensor], state: torch.Tensor,
               q_start: torch.Tensor, q_len: torch.Tensor, slots: torch.Tensor, num_requests: int,
               out_dtype: torch.dtype, activation: Optional[str] = "gelu_tanh", plan=None, zero_out: bool = False,
               gates: Optional[tuple] = None) -> torch.Tensor:
    """S_t = a_t S_(t-1) + b_t per channel over each request's rows, from and to the request's row of
    ``state`` (float32 [slots, C]); returns S_t * act(y_t) as [T, C] in ``out_dtype`` (``y`` [T, C],
    possibly a column slice, or None: S itself).  ``plan`` (a ``RecurrencePlan`` with chunks): long
    portions run as chunks side by side, in three launches.  Instead of ``a`` and ``b``, ``gates`` =
    (z, u, b_r, b_i, lam, rate) with z from ``gate_products``: the scan forms the coefficients of
    ``recurrence_gates`` itself, row by row, in float32."""
    _need_cuda(a, b, y, state, q_start, q_len, slots)
    _need_contiguous(a, b, state)
    z = u = b_r = b_i = lam = None
    rate, n, ldu = 0.0, 0, 0
    if gates is not None:
        if a is not None or b is not None:
            raise KernelError("gated_scan: coefficients or gates, not both")
        z, u, b_r, b_i, lam, rate = gates
        _need_cuda(z, u, b_r, b_i, lam)
        _need_contiguous(z, b_r, b_i, lam)
        _column_slice(u, "gated_scan")
        T, C = u.shape
        n = z.shape[2] // 2
        if z.dtype != torch.float32 or z.dim() != 3 or z.shape[0] != T or z.shape[1] * n != C or u.dtype != out_dtype:
            raise KernelError("gated_scan: z is float32 [T, B, 2n], u [T, B*n] in the output's dtype")
        for v in (b_r, b_i, lam):
            if v.dtype != torch.float32 or v.numel() != C:
                raise KernelError("gated_scan: gate biases and lam are float32 [C]")
        ldu = u.stride(0) if T > 1 else max(u.stride(0), C)
    else:
        T, C = a.shape
    if gates is None and (a.dtype != torch.float32 or b.dtype != torch.float32 or b.shape != a.shape):
        raise KernelError("gated_scan: a and b are float32 [T, C]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != C:
        raise KernelError("gated_scan: the state is float32 [slots, C]")
    if activation not in SCAN_ACTIVATIONS:
        raise KernelError(f"gated_scan: unknown activation {activation!r}")
    ldy = 0
    if y is not None:
        _column_slice(y, "gated_scan")
        if tuple(y.shape) != (T, C) or y.dtype != out_dtype:
            raise KernelError("gated_scan: y is [T, C] in the output's dtype")
        ldy = y.stride(0) if T > 1 else max(y.stride(0), C)
    dev = state.device
    out = (torch.zeros if zero_out else torch.empty)((T, C), dtype=out_dtype, device=dev)
    fn = _fn("gated_recurrence", "pbe_gated_scan",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_int,
              c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
              c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    code, act = _dtype_code(out), SCAN_ACTIVATIONS[activation]
    coeff = (_ptr(a), _ptr(b), _ptr(z), _ptr(u), int(ldu), _ptr(b_r), _ptr(b_i), _ptr(lam), float(rate), int(n))
    if plan is None or plan.num_chunks == 0:
        _check(fn(*coeff, _ptr(y), ldy, _ptr(out), code, _ptr(state), None, None, None, int(num_requests),
                  _ptr(q_start), _ptr(q_len), _ptr(slots), C, act, 0, _stream()), "gated_scan")
        return out
    scratch_s = torch.empty((plan.num_chunks, C), dtype=torch.float32, device=dev)
    scratch_p = torch.empty((plan.num_chunks, C), dtype=torch.float32, device=dev)
    if plan.num_first_pass:
        _check(fn(*coeff, None, 0, None, code, _ptr(state), _ptr(scratch_s), _ptr(scratch_p),
                  _ptr(plan.first_pass), plan.num_first_pass, None, None, None, C, act, 1, _stream()), "gated_scan")
    sfn = _fn("gated_recurrence", "pbe_chunk_starts", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(sfn(_ptr(plan.scan), plan.num_scan, _ptr(state), _ptr(scratch_s), _ptr(scratch_p), C, _stream()),
           "chunk_starts")
    _check(fn(*coeff, _ptr(y), ldy, _ptr(out), code, _ptr(state), _ptr(scratch_s), _ptr(scratch_p),
              _ptr(plan.second_pass), plan.num_second_pass, None, None, None, C, act, 2, _stream()), "gated_scan")
    return out
