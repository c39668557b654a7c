"""Typed Python faces of the exported kernels: they check devices, dtypes, shapes and strides of
torch tensors, then pass raw pointers and the current CUDA stream to the library.

Nothing here computes anything, and nothing falls back to another implementation.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from .library import KernelError, library

EPI_STORE = 0
EPI_ACCUMULATE = 1
EPI_SWIGLU = 2

FLAG_WRITE_CACHE = 1
FLAG_K_IN_PLACE = 2

STATUS_BAD_TOKEN = 1
STATUS_NO_PAGE = 2
STATUS_BAD_POSITION = 4


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 storage, not {dt}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current CUDA stream of the current device, as a handle for the launchers."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on the GPU; there is no CPU path")


def _rows_2d(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be 2-D with unit stride along the last dim, got shape "
                          f"{tuple(t.shape)} strides {t.stride()}")


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{what} must be a contiguous int32 tensor")


def convert(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A contiguous copy of ``src`` (float32 or bfloat16, on the GPU) in ``dtype``; rounding to
    bfloat16 is to nearest even."""
    _need_cuda(src)
    src = src.contiguous()
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    with torch.cuda.device(src.device):
        library("core").call("bfi_convert", _ptr(src), c_int(dtype_code(src.dtype)), _ptr(out),
                             c_int(dtype_code(dtype)), c_long(src.numel()), _stream())
    return out


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor,
               status: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """``out[t] = table[ids[t]] * scale`` into the float32 residual stream."""
    _need_cuda(table, ids, out, status)
    _rows_2d(table, "embedding table")
    _rows_2d(out, "embedding output")
    _i32(ids, "token ids")
    if out.dtype != torch.float32 or not out.is_contiguous() or out.shape != (ids.numel(), table.shape[1]):
        raise KernelError("embedding output must be contiguous float32 [tokens, width]")
    if not table.is_contiguous():
        raise KernelError("embedding table must be contiguous")
    library("core").call("bfi_embed_rows", _ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(out),
                         c_int(ids.numel()), c_int(table.shape[1]), c_int(table.shape[0]), c_float(scale), _ptr(status),
                         _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """``out[r] = norm(x[rows[r]]) * w`` (``rows`` None: every row in order)."""
    _need_cuda(x, w, out, rows)
    _rows_2d(x, "norm input")
    _rows_2d(out, "norm output")
    _i32(rows, "row indices")
    width = x.shape[1]
    n_rows = rows.numel() if rows is not None else x.shape[0]
    if w.dim() != 1 or w.shape[0] != width or not w.is_contiguous():
        raise KernelError(f"norm weight must be [{width}], got {tuple(w.shape)}")
    if out.shape != (n_rows, width):
        raise KernelError(f"norm output must be [{n_rows}, {width}], got {tuple(out.shape)}")
    library("core").call("bfi_rmsnorm", _ptr(x), c_int(dtype_code(x.dtype)), c_long(x.stride(0)), _ptr(rows),
                         _ptr(w), c_int(dtype_code(w.dtype)), _ptr(out), c_int(dtype_code(out.dtype)),
                         c_long(out.stride(0)), c_int(n_rows), c_int(width), c_float(eps), _stream())


def silu_mul(gu: torch.Tensor, out: torch.Tensor, interleaved: bool) -> None:
    _need_cuda(gu, out)
    _rows_2d(gu, "gate/up input")
    _rows_2d(out, "gated output")
    if gu.dtype != out.dtype or gu.shape[0] != out.shape[0] or gu.shape[1] != 2 * out.shape[1]:
        raise KernelError("silu_mul: input must be [rows, 2*width] and output [rows, width] of one dtype")
    library("core").call("bfi_silu_mul", _ptr(gu), c_long(gu.stride(0)), _ptr(out), c_long(out.stride(0)),
                         c_int(dtype_code(gu.dtype)), c_int(gu.shape[0]), c_int(out.shape[1]),
                         c_int(1 if interleaved else 0), _stream())


def gate_mul(gu: torch.Tensor, out: torch.Tensor, interleaved: bool, alpha: float = 1.0, limit: float = 0.0,
             shift: float = 0.0) -> None:
    """The gated activation over gate/up pairs: ``g' * sigmoid(alpha * g') * (u' + shift)`` with
    ``g' = min(g, limit)`` and ``u' = clamp(u, -limit, limit)`` (``limit`` 0: no clamping)."""
    _need_cuda(gu, out)
    _rows_2d(gu, "gate/up input")
    _rows_2d(out, "gated output")
    if gu.dtype != out.dtype or gu.shape[0] != out.shape[0] or gu.shape[1] != 2 * out.shape[1]:
        raise KernelError("gate_mul: input must be [rows, 2*width] and output [rows, width] of one dtype")
    library("core").call("bfi_gate_mul", _ptr(gu), c_long(gu.stride(0)), _ptr(out), c_long(out.stride(0)),
                         c_int(dtype_code(gu.dtype)), c_int(gu.shape[0]), c_int(out.shape[1]),
                         c_int(1 if interleaved else 0), c_float(alpha), c_float(limit), c_float(shift), _stream())


def residual_add(x: torch.Tensor, y: torch.Tensor) -> None:
    _need_cuda(x, y)
    if x.dtype != torch.float32 or not x.is_contiguous() or not y.is_contiguous() or x.shape != y.shape:
        raise KernelError("residual_add: x must be contiguous float32 and y contiguous of the same shape")
    library("core").call("bfi_residual_add", _ptr(x), _ptr(y), c_int(dtype_code(y.dtype)), c_long(x.numel()),
                         _stream())


def qk_norm_rope_cache(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                       q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                       rope_table: Optional[torch.Tensor], rot_dim: int,
                       token_pos: torch.Tensor, token_slot: torch.Tensor, kv, flags: int,
                       status: Optional[torch.Tensor] = None) -> None:
    """``kv`` is a ``KVView`` or None; ``rope_table`` is float32 ``[positions, rot_dim/2, 2]``."""
    _need_cuda(qkv, q_norm_w, k_norm_w, rope_table, token_pos, token_slot, status)
    _rows_2d(qkv, "qkv")
    _i32(token_pos, "token positions")
    _i32(token_slot, "token slots")
    n_tokens = qkv.shape[0]
    if token_pos.numel() < n_tokens or token_slot.numel() < n_tokens:
        raise KernelError("qk_norm_rope_cache: position/slot arrays shorter than the tokens")
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError(f"qkv row must hold ({n_q}+2*{n_kv})*{head_dim} values, got {qkv.shape[1]}")
    norm_dt = 0
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            if w.shape != (head_dim,) or not w.is_contiguous():
                raise KernelError(f"q/k norm weight must be [{head_dim}]")
            norm_dt = dtype_code(w.dtype)
    if q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("q and k norm weights must share a dtype")
    positions = 0
    if rope_table is not None:
        if rope_table.dtype != torch.float32 or not rope_table.is_contiguous() or rope_table.dim() != 3 \
                or rope_table.shape[1] != rot_dim // 2 or rope_table.shape[2] != 2:
            raise KernelError("rotation table must be contiguous float32 [positions, rot_dim/2, 2]")
        positions = rope_table.shape[0]
    k_pages = v_pages = table = None
    stride = 0
    if kv is not None and (flags & FLAG_WRITE_CACHE):
        if kv.k.dtype != qkv.dtype or kv.n_kv_heads != n_kv or kv.head_dim != head_dim:
            raise KernelError("cache pages do not fit the heads being written")
        k_pages, v_pages, table = kv.k, kv.v, kv.block_table
        stride = table.stride(0)
    library("core").call(
        "bfi_qk_norm_rope_cache", _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_long(qkv.stride(0)), c_int(n_tokens),
        c_int(n_q), c_int(n_kv), c_int(head_dim), _ptr(q_norm_w), _ptr(k_norm_w), c_int(norm_dt), c_float(eps),
        _ptr(rope_table), c_int(rot_dim), c_int(positions), _ptr(token_pos), _ptr(token_slot), _ptr(k_pages),
        _ptr(v_pages), _ptr(table), c_int(stride), c_int(flags), _ptr(status), _stream())


NORM_NONE, NORM_HEAD, NORM_ROW = 0, 1, 2
PAIR_HALF, PAIR_ADJACENT = 0, 1
FLAG_VALUES_ARE_KEYS = 4


def qk_prepare(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int, token_pos: torch.Tensor,
               token_slot: torch.Tensor, kv, flags: int, *, q_bias=None, k_bias=None, v_bias=None,
               q_norm_w=None, k_norm_w=None, norm_mode: int = NORM_NONE, eps: float = 1e-6, rope_table=None,
               rot_dim: int = 0, pairing: int = PAIR_HALF, residual=None, out_bias=None,
               status: Optional[torch.Tensor] = None, v_dim: Optional[int] = None) -> None:
    """Between the q/k(/v) projection and the attention, one block per token: biases, the values
    (the row's own v heads, or with ``FLAG_VALUES_ARE_KEYS`` the keys as they stand after their
    bias), a norm per head or over the whole projection, the rotation with either pairing, q back in
    place and k, v into the cache; ``out_bias`` is added to the token's row of ``residual``."""
    _need_cuda(qkv, q_bias, k_bias, v_bias, q_norm_w, k_norm_w, rope_table, token_pos, token_slot, residual, out_bias, status)
    _rows_2d(qkv, "qkv")
    _i32(token_pos, "token positions")
    _i32(token_slot, "token slots")
    n_tokens = qkv.shape[0]
    own_v = not (flags & FLAG_VALUES_ARE_KEYS)
    v_dim = head_dim if v_dim is None else int(v_dim)
    if token_pos.numel() < n_tokens or token_slot.numel() < n_tokens:
        raise KernelError("qk_prepare: position/slot arrays shorter than the tokens")
    if qkv.shape[1] != (n_q + n_kv) * head_dim + (n_kv * v_dim if own_v else 0):
        raise KernelError(f"qk_prepare: a row of {qkv.shape[1]} values does not hold the heads")
    bias_dt = norm_dt = 0
    for b, n in ((q_bias, n_q * head_dim), (k_bias, n_kv * head_dim), (v_bias, n_kv * v_dim)):
        if b is not None:
            if b.shape != (n,) or not b.is_contiguous():
                raise KernelError(f"qk_prepare: a projection bias must be [{n}]")
            bias_dt = dtype_code(b.dtype)
    if len({b.dtype for b in (q_bias, k_bias, v_bias) if b is not None}) > 1:
        raise KernelError("qk_prepare: the projection biases must share a dtype")
    for w, n in ((q_norm_w, n_q), (k_norm_w, n_kv)):
        if w is not None:
            want = head_dim if norm_mode == NORM_HEAD else n * head_dim
            if w.shape != (want,) or not w.is_contiguous():
                raise KernelError(f"qk_prepare: norm weight must be [{want}], got {tuple(w.shape)}")
            norm_dt = dtype_code(w.dtype)
    if q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("q and k norm weights must share a dtype")
    positions = 0
    if rope_table is not None:
        if rope_table.dtype != torch.float32 or not rope_table.is_contiguous() or rope_table.dim() != 3 \
                or rope_table.shape[1] != rot_dim // 2 or rope_table.shape[2] != 2:
            raise KernelError("rotation table must be contiguous float32 [positions, rot_dim/2, 2]")
        positions = rope_table.shape[0]
    k_pages = v_pages = table = None
    stride = 0
    if kv is not None and (flags & FLAG_WRITE_CACHE):
        if kv.k.dtype != qkv.dtype or kv.n_kv_heads != n_kv or kv.head_dim != head_dim or kv.value_dim != v_dim:
            raise KernelError("cache pages do not fit the heads being written")
        k_pages, v_pages, table = kv.k, kv.v, kv.block_table
        stride = table.stride(0)
    width = r_stride = ob_dt = 0
    if out_bias is not None:
        if residual is None or residual.dtype != torch.float32 or residual.dim() != 2 or residual.stride(1) != 1 \
                or residual.shape[0] < n_tokens or out_bias.shape != (residual.shape[1],) or not out_bias.is_contiguous():
            raise KernelError("qk_prepare: the output bias needs the float32 residual [tokens, width] and a bias [width]")
        width, r_stride, ob_dt = residual.shape[1], residual.stride(0), dtype_code(out_bias.dtype)
    library("core").call(
        "bfi_qk_prepare", _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_long(qkv.stride(0)), c_int(n_tokens), c_int(n_q),
        c_int(n_kv), c_int(head_dim), c_int(v_dim), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias), c_int(bias_dt), _ptr(q_norm_w),
        _ptr(k_norm_w), c_int(norm_dt), c_int(norm_mode), c_float(eps), _ptr(rope_table), c_int(rot_dim),
        c_int(positions), c_int(pairing), _ptr(token_pos), _ptr(token_slot), _ptr(k_pages), _ptr(v_pages), _ptr(table),
        c_int(stride), c_int(flags), _ptr(residual if out_bias is not None else None), c_long(r_stride), _ptr(out_bias),
        c_int(ob_dt), c_int(width), _ptr(status), _stream())


LIGHT_ACT_NONE, LIGHT_ACT_SILU = 0, 1


def lightning_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, out: torch.Tensor, state: torch.Tensor,
                   decay: torch.Tensor, cu_seqlens: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int,
                   n_heads: int, dim: int, vdim: int, act: int = LIGHT_ACT_SILU, few_tokens: bool = False,
                   single_tokens: bool = False) -> None:
    """Linear attention with a decay per head over the step's new tokens, sequence by sequence:
    ``S = decay * S + k v^T; o = S^T q`` with ``S`` float32 ``[slots, heads, dim, vdim]`` carried
    in ``state``.  q, k, v are columns ``q_off``, ``k_off``, ``v_off`` of ``proj`` (activated here
    when ``act`` says so); ``out`` is float32 ``[tokens, heads * vdim]``.  ``single_tokens``: every
    sequence of the step brings exactly one token (the kernel then keeps the state in registers)."""
    _need_cuda(proj, out, state, decay, cu_seqlens, seq_slot)
    _rows_2d(proj, "projections")
    _rows_2d(out, "recurrence output")
    _i32(cu_seqlens, "cu_seqlens")
    _i32(seq_slot, "sequence slots")
    if out.dtype != torch.float32 or out.shape[1] != n_heads * vdim:
        raise KernelError("lightning_scan: the output must be float32 [tokens, heads * vdim]")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (n_heads, dim, vdim):
        raise KernelError("lightning_scan: the state must be contiguous float32 [slots, heads, dim, vdim]")
    if decay.dtype != torch.float32 or not decay.is_contiguous() or decay.numel() != n_heads:
        raise KernelError("lightning_scan: one float32 decay per head")
    if max(q_off, k_off) + n_heads * dim > proj.shape[1] or v_off + n_heads * vdim > proj.shape[1]:
        raise KernelError("lightning_scan: the projections' row is shorter than the heads")
    library("core").call("bfi_lightning_scan", _ptr(proj), c_int(dtype_code(proj.dtype)), c_long(proj.stride(0)),
                         c_int(q_off), c_int(k_off), c_int(v_off), _ptr(out), c_long(out.stride(0)), _ptr(state),
                         _ptr(decay), _ptr(cu_seqlens), _ptr(seq_slot), c_int(n_seqs), c_int(n_heads), c_int(dim),
                         c_int(vdim), c_int(act), c_int(2 if single_tokens else (1 if few_tokens else 0)), _stream())


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """``out = x * rsqrt(mean(x^2) + eps) * w * sigmoid(gate)`` row by row; ``x`` float32, ``gate``
    (a view into the projections) and ``out`` in the activation dtype."""
    _need_cuda(x, gate, w, out)
    _rows_2d(x, "norm input")
    _rows_2d(gate, "gate")
    _rows_2d(out, "norm output")
    n, width = x.shape
    if x.dtype != torch.float32 or gate.dtype != out.dtype or gate.shape != (n, width) or out.shape != (n, width):
        raise KernelError("gated_rmsnorm: x float32 [rows, width]; gate and output [rows, width] of one dtype")
    if w.shape != (width,) or not w.is_contiguous():
        raise KernelError(f"gated_rmsnorm: weight must be [{width}]")
    library("core").call("bfi_gated_rmsnorm", _ptr(x), c_long(x.stride(0)), _ptr(gate), c_long(gate.stride(0)),
                         c_int(dtype_code(out.dtype)), _ptr(w), c_int(dtype_code(w.dtype)), _ptr(out),
                         c_long(out.stride(0)), c_int(n), c_int(width), c_float(eps), _stream())


def attention_paged(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv, cu_seqlens: torch.Tensor,
                    seq_slot: torch.Tensor, seq_start: torch.Tensor, n_seqs: int, max_tokens: int,
                    n_q: int, scale: float, sink=None) -> None:
    """``q`` is the first query element of the step (a view into the qkv buffer); token ``t``, head
    ``h`` lies at ``q + t*q_stride + h*head_dim``.  ``out`` is ``[tokens, n_q*v_dim]``.  With
    ``sink`` (a number, or a float32 tensor with one per query head) the softmax's denominator
    carries ``exp(sink)`` beside the keys' terms.  The cache view says whether the values have a
    size of their own (or are the first values of the keys) and whether a token reads only its own
    chunk of positions."""
    has_sink, sink_value, sinks = 0, 0.0, None
    if isinstance(sink, torch.Tensor):
        if sink.dtype != torch.float32 or not sink.is_contiguous() or sink.numel() != n_q or not sink.is_cuda:
            raise KernelError(f"attention: a sink per head must be contiguous float32 [{n_q}] on the GPU")
        has_sink, sinks = 2, sink
    elif sink is not None:
        has_sink, sink_value = 1, float(sink)
    _need_cuda(q, out, cu_seqlens, seq_slot, seq_start)
    _rows_2d(out, "attention output")
    _i32(cu_seqlens, "cu_seqlens")
    _i32(seq_slot, "sequence slots")
    _i32(seq_start, "sequence starts")
    if q.dtype != out.dtype or kv.k.dtype != q.dtype:
        raise KernelError("attention: q, output and cache must share a dtype")
    library("core").call(
        "bfi_attention_paged", _ptr(q), c_int(dtype_code(q.dtype)), c_long(q_stride), _ptr(out),
        c_long(out.stride(0)), _ptr(kv.k), _ptr(None if kv.values_in_keys else kv.v), _ptr(kv.block_table),
        c_int(kv.block_table.stride(0)),
        _ptr(cu_seqlens), _ptr(seq_slot), _ptr(seq_start), c_int(n_seqs), c_int(max_tokens), c_int(n_q),
        c_int(kv.n_kv_heads), c_int(kv.head_dim), c_int(kv.value_dim), c_int(kv.window or 0), c_int(kv.chunk or 0),
        c_float(scale), c_int(has_sink), c_float(sink_value), _ptr(sinks), _stream())


def latent_prepare(proj: torch.Tensor, qa: torch.Tensor, n_heads: int, dim: int, rot_dim: int, rank: int, kv_off: int,
                   norm_w: Optional[torch.Tensor], eps: float, rope_table: Optional[torch.Tensor], rot_used: int,
                   token_pos: torch.Tensor, token_slot: torch.Tensor, kv, write_cache: bool,
                   status: Optional[torch.Tensor] = None) -> None:
    """Latent attention, per token: every query head's rotated part (``rot_dim`` values behind its
    ``dim`` unrotated ones in ``proj``) turned by the position's angles and put at columns
    ``rank .. rank + rot_dim`` of the head's row in ``qa`` ``[tokens, heads * (rank + rot_dim)]``; with
    ``write_cache`` the down projection at column ``kv_off`` of ``proj`` becomes the token's cache
    row: its first ``rank`` values RMS-normed with ``norm_w``, its last ``rot_dim`` turned.
    ``rot_used`` of the rotated part's values turn (value i with value i + rot_used/2)."""
    _need_cuda(proj, qa, norm_w, rope_table, token_pos, token_slot, status)
    _rows_2d(proj, "projections")
    _rows_2d(qa, "latent queries")
    _i32(token_pos, "token positions")
    _i32(token_slot, "token slots")
    n = proj.shape[0]
    if qa.dtype != proj.dtype or qa.shape != (n, n_heads * (rank + rot_dim)):
        raise KernelError("latent_prepare: the query buffer must be [tokens, heads * (rank + rot_dim)] of the projections' dtype")
    if proj.shape[1] < n_heads * (dim + rot_dim) or token_pos.numel() < n or token_slot.numel() < n:
        raise KernelError("latent_prepare: a row is shorter than the heads, or the index arrays than the tokens")
    positions = 0
    if rot_used:
        if rope_table is None or rope_table.dtype != torch.float32 or not rope_table.is_contiguous() or rope_table.dim() != 3 \
                or rope_table.shape[1] != rot_used // 2 or rope_table.shape[2] != 2:
            raise KernelError("rotation table must be contiguous float32 [positions, rot_dim/2, 2]")
        positions = rope_table.shape[0]
    k_pages = table = None
    stride = 0
    if write_cache:
        if kv is None or kv.k.dtype != proj.dtype or kv.n_kv_heads != 1 or kv.head_dim != rank + rot_dim or not kv.k.is_contiguous():
            raise KernelError("latent_prepare: the cache must hold one contiguous row of rank + rot_dim values per token")
        if norm_w is None or norm_w.shape != (rank,) or not norm_w.is_contiguous() or proj.shape[1] < kv_off + rank + rot_dim:
            raise KernelError("latent_prepare: writing the cache needs the latent's norm weight and the down projection's columns")
        k_pages, table = kv.k, kv.block_table
        stride = table.stride(0)
    library("core").call(
        "bfi_latent_prepare", _ptr(proj), c_int(dtype_code(proj.dtype)), c_long(proj.stride(0)), _ptr(qa), c_long(qa.stride(0)),
        c_int(n), c_int(n_heads), c_int(dim), c_int(rot_dim), c_int(rank), c_int(kv_off), _ptr(norm_w),
        c_int(0 if norm_w is None else dtype_code(norm_w.dtype)), c_float(eps), _ptr(rope_table if rot_used else None),
        c_int(rot_used), c_int(positions), _ptr(token_pos), _ptr(token_slot), _ptr(k_pages), _ptr(table), c_int(stride),
        c_int(1 if write_cache else 0), _ptr(status), _stream())


def latent_absorb(proj: torch.Tensor, w_uk: torch.Tensor, qa: torch.Tensor, token_slot: torch.Tensor, n_heads: int, dim: int,
                  rot_dim: int, rank: int) -> None:
    """``qa[t, h, :rank] = W_uk_h^T q[t, h, :dim]`` with ``w_uk`` ``[heads * dim, rank]``: the unrotated
    part of every query head taken into the latent space, where it meets the cached latents."""
    _need_cuda(proj, w_uk, qa, token_slot)
    _rows_2d(proj, "projections")
    _rows_2d(qa, "latent queries")
    _i32(token_slot, "token slots")
    n = proj.shape[0]
    if w_uk.shape != (n_heads * dim, rank) or not w_uk.is_contiguous():
        raise KernelError(f"latent_absorb: the key matrices must be contiguous [{n_heads * dim}, {rank}]")
    if qa.dtype != proj.dtype or qa.shape != (n, n_heads * (rank + rot_dim)) or proj.shape[1] < n_heads * (dim + rot_dim):
        raise KernelError("latent_absorb: queries [tokens, heads * (dim + rot_dim)] in, [tokens, heads * (rank + rot_dim)] out")
    library("core").call("bfi_latent_absorb", _ptr(proj), c_int(dtype_code(proj.dtype)), c_long(proj.stride(0)), _ptr(w_uk),
                         c_int(dtype_code(w_uk.dtype)), _ptr(qa), c_long(qa.stride(0)), _ptr(token_slot), c_int(n),
                         c_int(n_heads), c_int(dim), c_int(rot_dim), c_int(rank), _stream())


def latent_expand(lat: torch.Tensor, w_uv: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor,
                  token_slot: torch.Tensor, n_heads: int, v_dim: int, rank: int) -> None:
    """``out[t, h] = (W_uv_h lat[t, h]) * sigmoid(gate[t, h])`` with ``w_uv`` ``[heads * v_dim, rank]``,
    ``lat`` ``[tokens, heads * rank]`` (the attention's weighted sums of cached latents) and ``gate`` a
    view ``[tokens, heads]`` of logits (None: no gate), or ``[tokens, heads * v_dim]``: a gate per
    output value."""
    _need_cuda(lat, w_uv, gate, out, token_slot)
    _rows_2d(lat, "latent outputs")
    _rows_2d(out, "head outputs")
    _i32(token_slot, "token slots")
    n = lat.shape[0]
    if w_uv.shape != (n_heads * v_dim, rank) or not w_uv.is_contiguous():
        raise KernelError(f"latent_expand: the value matrices must be contiguous [{n_heads * v_dim}, {rank}]")
    if lat.shape != (n, n_heads * rank) or out.shape != (n, n_heads * v_dim) or out.dtype != lat.dtype:
        raise KernelError("latent_expand: [tokens, heads * rank] in, [tokens, heads * v_dim] out, of one dtype")
    if gate is not None:
        _rows_2d(gate, "gate logits")
        if gate.shape not in ((n, n_heads), (n, n_heads * v_dim)) or gate.dtype != lat.dtype:
            raise KernelError("latent_expand: the gate must be [tokens, heads] or [tokens, heads * v_dim] of the activations' dtype")
    library("core").call("bfi_latent_expand", _ptr(lat), c_int(dtype_code(lat.dtype)), c_long(lat.stride(0)), _ptr(w_uv),
                         c_int(dtype_code(w_uv.dtype)), _ptr(gate), c_long(0 if gate is None else gate.stride(0)), _ptr(out),
                         c_long(out.stride(0)), _ptr(token_slot), c_int(n), c_int(n_heads), c_int(v_dim), c_int(rank),
                         c_int(1 if gate is not None and v_dim > 1 and gate.shape[1] == n_heads * v_dim else 0), _stream())


def bigram_add(table: torch.Tensor, ids: torch.Tensor, token_pos: torch.Tensor, token_slot: torch.Tensor,
               last_token: torch.Tensor, x: torch.Tensor, mul_prev: int, mul_cur: int, vocab: int,
               status: Optional[torch.Tensor] = None) -> None:
    """``x[t] += table[(previous token * mul_prev + token * mul_cur) mod buckets]`` with ``table``
    ``[buckets + 1, width]``; a token at position 0 takes the last row.  The previous token of a
    sequence's first token in the step is ``last_token[slot]`` (int32 ``[slots, 1]``)."""
    _need_cuda(table, ids, token_pos, token_slot, last_token, x, status)
    _rows_2d(table, "bigram table")
    for t, what in ((ids, "token ids"), (token_pos, "token positions"), (token_slot, "token slots"), (last_token, "last tokens")):
        _i32(t, what)
    n = x.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or x.shape[1] != table.shape[1] or not table.is_contiguous():
        raise KernelError("bigram_add: the residual stream must be contiguous float32 [tokens, width], the table contiguous")
    if ids.numel() < n or token_pos.numel() < n or token_slot.numel() < n or table.shape[0] < 2:
        raise KernelError("bigram_add: index arrays shorter than the tokens, or a table without buckets")
    library("core").call("bfi_bigram_add", _ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(token_pos),
                         _ptr(token_slot), _ptr(last_token), _ptr(x), c_int(n), c_int(x.shape[1]), c_int(table.shape[0] - 1),
                         c_long(int(mul_prev)), c_long(int(mul_cur)), c_int(vocab), _ptr(status), _stream())


def keep_last_tokens(ids: torch.Tensor, cu_seqlens: torch.Tensor, seq_slot: torch.Tensor, last_token: torch.Tensor,
                     n_seqs: int) -> None:
    """``last_token[slot] = `` the last token id each sequence brings in this step."""
    _need_cuda(ids, cu_seqlens, seq_slot, last_token)
    for t, what in ((ids, "token ids"), (cu_seqlens, "cu_seqlens"), (seq_slot, "sequence slots"), (last_token, "last tokens")):
        _i32(t, what)
    library("core").call("bfi_keep_last_tokens", _ptr(ids), _ptr(cu_seqlens), _ptr(seq_slot), _ptr(last_token), c_int(n_seqs),
                         _stream())


def _f32_vector(t: Optional[torch.Tensor], n: int, what: str) -> None:
    if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n or not t.is_cuda):
        raise KernelError(f"{what} must be contiguous float32 [{n}] on the GPU")


def norm_add(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, next_w: Optional[torch.Tensor] = None,
             next_eps: float = 0.0, out: Optional[torch.Tensor] = None, mult: float = 1.0,
             gate: Optional[torch.Tensor] = None, gate_bias: Optional[torch.Tensor] = None, conv=None) -> None:
    """``x[t] += mult * y[t] * rsqrt(mean(y[t]^2) + eps) * w``: a sublayer's output, normed, into the
    float32 residual stream.  With ``gate`` (logits ``[rows, width]`` of either storage type, and an
    optional ``gate_bias`` ``[width]``) ``y`` is first multiplied by ``sigmoid(gate + gate_bias)``.
    With ``next_w`` and ``out`` the next sublayer's norm of the new ``x`` is made in the same
    kernel: ``out[t] = x[t] * rsqrt(mean(x[t]^2) + next_eps) * next_w``.  ``conv`` (for steps in
    which every sequence brings one token; rows of a multiple of 4 values): ``(w, state, token_slot,
    h, plain)``, the convolution over time that stands in front of the NEXT sublayer, made from
    the row just written: ``h[t] = x[t] + conv(x)[t]`` with ``w`` ``[width, taps]`` (2 to 4 taps) and
    the kept inputs ``state`` ``[slots, taps-1, width]``, which move on by one; ``plain[t] = x[t]``; both
    outputs in one storage type."""
    _need_cuda(x, y, w, next_w, out, gate, gate_bias)
    cw = cstate = cslot = ch = cplain = None
    if conv is not None:
        cw, cstate, cslot, ch, cplain = conv
        _need_cuda(cw, cstate, cslot, ch, cplain)
        _i32(cslot, "token slots")
        _rows_2d(ch, "convolved rows")
        _rows_2d(cplain, "plain rows")
        taps = cw.shape[1] if cw.dim() == 2 else 0
        if cw.shape != (x.shape[1], taps) or not cw.is_contiguous() or not 2 <= taps <= 4:
            raise KernelError(f"norm_add: the convolution that follows takes contiguous weights [{x.shape[1]}, 2 to 4 taps]")
        if cstate.dtype != torch.float32 or not cstate.is_contiguous() or tuple(cstate.shape[1:]) != (taps - 1, x.shape[1]):
            raise KernelError("norm_add: the convolution's state must be contiguous float32 [slots, taps-1, width]")
        if ch.shape != x.shape or cplain.shape != x.shape or ch.dtype != cplain.dtype or cslot.numel() < x.shape[0]:
            raise KernelError("norm_add: the convolution's outputs have the stream's shape and one dtype; a slot per row")
    if gate is not None:
        _rows_2d(gate, "gate logits")
        if gate.shape != x.shape:
            raise KernelError("norm_add: the gate's logits must have the residual stream's shape")
        if gate_bias is not None and (gate_bias.shape != (x.shape[1],) or not gate_bias.is_contiguous()):
            raise KernelError(f"norm_add: the gate's bias must be [{x.shape[1]}]")
    elif gate_bias is not None:
        raise KernelError("norm_add: a gate bias without gate logits")
    if (next_w is None) != (out is None):
        raise KernelError("norm_add: the next norm needs both its weight and its output")
    if out is not None:
        _rows_2d(out, "norm output")
        if out.shape != x.shape or next_w.shape != (x.shape[1],) or not next_w.is_contiguous():
            raise KernelError("norm_add: the next norm's output must be [rows, width] and its weight [width]")
    _rows_2d(x, "residual stream")
    _rows_2d(y, "sublayer output")
    if x.dtype != torch.float32 or y.dtype != torch.float32 or x.shape != y.shape:
        raise KernelError("norm_add: the residual stream and the sublayer output must be float32 of one shape")
    if w.shape != (x.shape[1],) or not w.is_contiguous():
        raise KernelError(f"norm_add: weight must be [{x.shape[1]}]")
    library("core").call("bfi_norm_add", _ptr(x), c_long(x.stride(0)), _ptr(y), c_long(y.stride(0)), _ptr(w),
                         c_int(dtype_code(w.dtype)), c_int(x.shape[0]), c_int(x.shape[1]), c_float(eps), _ptr(next_w),
                         c_int(0 if next_w is None else dtype_code(next_w.dtype)), c_float(next_eps), _ptr(out),
                         c_int(0 if out is None else dtype_code(out.dtype)), c_long(0 if out is None else out.stride(0)),
                         c_float(mult), _ptr(gate), c_int(0 if gate is None else dtype_code(gate.dtype)),
                         c_long(0 if gate is None else gate.stride(0)), _ptr(gate_bias),
                         c_int(0 if gate_bias is None else dtype_code(gate_bias.dtype)), _ptr(cw),
                         c_int(0 if cw is None else dtype_code(cw.dtype)), c_int(0 if cw is None else cw.shape[1]), _ptr(cstate),
                         _ptr(cslot), _ptr(ch), c_long(0 if ch is None else ch.stride(0)), _ptr(cplain),
                         c_long(0 if cplain is None else cplain.stride(0)), c_int(0 if ch is None else dtype_code(ch.dtype)),
                         _stream())


def weighted_sum(out: torch.Tensor, y0: torch.Tensor, a: float, y1: torch.Tensor, b: float) -> None:
    """``out = a * y0 + b * y1`` over contiguous float32 tensors of one shape."""
    _need_cuda(out, y0, y1)
    for t in (out, y0, y1):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.shape != out.shape:
            raise KernelError("weighted_sum: contiguous float32 tensors of one shape")
    library("core").call("bfi_weighted_sum", _ptr(out), _ptr(y0), c_float(a), _ptr(y1), c_float(b), c_long(out.numel()),
                         _stream())


def scale_rows(x: torch.Tensor, s: float) -> None:
    """``x *= s`` over float32 rows."""
    _need_cuda(x)
    _rows_2d(x, "rows")
    if x.dtype != torch.float32:
        raise KernelError("scale_rows: float32 rows")
    library("core").call("bfi_scale_rows", _ptr(x), c_long(x.stride(0)), c_int(x.shape[0]), c_int(x.shape[1]),
                         c_float(s), _stream())


def gated_rows(out: torch.Tensor, src: torch.Tensor, g: torch.Tensor, accumulate: bool = False) -> None:
    """``out[r] (= | +=) g[r] * src[r]`` over float32 rows, one factor per row."""
    _need_cuda(out, src, g)
    _rows_2d(out, "rows")
    _rows_2d(src, "rows")
    if out.dtype != torch.float32 or src.dtype != torch.float32 or out.shape != src.shape or g.dtype != torch.float32 \
            or not g.is_contiguous() or g.numel() < out.shape[0]:
        raise KernelError("gated_rows: float32 rows of one shape and one float32 factor per row")
    library("core").call("bfi_gated_rows", _ptr(out), c_long(out.stride(0)), _ptr(src), c_long(src.stride(0)), _ptr(g),
                         c_int(out.shape[0]), c_int(out.shape[1]), c_int(1 if accumulate else 0), _stream())


DECAY_STEP, DECAY_SIGMOID = 1, 2


def decay_scan(qk: torch.Tensor, q_off: int, k_off: int, v: torch.Tensor, v_off: int, raw: torch.Tensor, r_off: int,
               out: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int,
               n_heads: int, dim: int, vdim: int, heads_per_group: int, mode: int, bias: torch.Tensor,
               rate: Optional[torch.Tensor] = None, skip: Optional[torch.Tensor] = None, q_scale: float = 1.0,
               inv_tau: float = 1.0, few_tokens: bool = False, single_tokens: bool = False, chunk_len: int = 0,
               max_chunks: int = 0,
               chunk_state: Optional[torch.Tensor] = None, chunk_decay: Optional[torch.Tensor] = None) -> None:
    """A linear recurrence whose decay depends on the token, over the step's new tokens:
    ``S = diag(a) S + k (c v)^T; o = S^T q + skip * v`` with ``S`` float32
    ``[slots, heads, dim, vdim]`` carried in ``state``.  q and k are columns of ``qk`` (group
    ``h // heads_per_group`` of head ``h``), v of ``v``, the decay's raw value of ``raw`` (rows of one
    storage type).  ``DECAY_STEP``: ``c = softplus(raw_h + bias_h)``, ``a = exp(-rate_h c)``;
    ``DECAY_SIGMOID``: ``a_d = sigmoid(raw_hd + bias_hd)^inv_tau``, ``c = 1``.  ``out`` float32.
    ``chunk_len`` > 0 runs the chunked form (chunks of a sequence side by side, then a carry over the
    chunks, then the earlier tokens' part of every output): ``chunk_state`` float32 with
    ``heads * dim * vdim`` values and ``chunk_decay`` with ``heads * dim`` for every chunk of the step;
    ``max_chunks`` is the most chunks one sequence has.  ``single_tokens``: every sequence of the
    step brings exactly one token (the state is then streamed through once)."""
    _need_cuda(qk, v, raw, out, state, cu_seqlens, seq_slot, bias, rate, skip)
    for t, what in ((qk, "q and k"), (v, "values"), (raw, "decay input"), (out, "recurrence output")):
        _rows_2d(t, what)
    _i32(cu_seqlens, "cu_seqlens")
    _i32(seq_slot, "sequence slots")
    if not (qk.dtype == v.dtype == raw.dtype):
        raise KernelError("decay_scan: q, k, v and the decay input must share a storage type")
    if out.dtype != torch.float32 or out.shape[1] != n_heads * vdim:
        raise KernelError("decay_scan: the output must be float32 [tokens, heads * vdim]")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (n_heads, dim, vdim):
        raise KernelError("decay_scan: the state must be contiguous float32 [slots, heads, dim, vdim]")
    groups = n_heads // max(1, heads_per_group)
    if max(q_off, k_off) + groups * dim > qk.shape[1] or v_off + n_heads * vdim > v.shape[1]:
        raise KernelError("decay_scan: a row is shorter than the heads")
    n_raw = n_heads if mode == DECAY_STEP else n_heads * dim
    if r_off + n_raw > raw.shape[1]:
        raise KernelError("decay_scan: the decay input's row is shorter than the heads")
    _f32_vector(bias, n_raw, "decay_scan: the decay's bias")
    _f32_vector(rate, n_heads, "decay_scan: the decay's rate")
    _f32_vector(skip, n_heads, "decay_scan: the skip factor")
    if chunk_len > 0:
        n_chunks = qk.shape[0] // chunk_len + n_seqs
        for t, per in ((chunk_state, n_heads * dim * vdim), (chunk_decay, n_heads * dim)):
            if t is None or t.dtype != torch.float32 or not t.is_contiguous() or t.numel() < n_chunks * per or not t.is_cuda:
                raise KernelError(f"decay_scan: the chunked form needs float32 scratch for {n_chunks} chunks")
    library("core").call("bfi_decay_scan", _ptr(qk), c_long(qk.stride(0)), c_int(q_off), c_int(k_off), _ptr(v),
                         c_long(v.stride(0)), c_int(v_off), _ptr(raw), c_long(raw.stride(0)), c_int(r_off),
                         c_int(dtype_code(qk.dtype)), _ptr(out), c_long(out.stride(0)), _ptr(state), _ptr(cu_seqlens),
                         _ptr(seq_slot), c_int(n_seqs), c_int(n_heads), c_int(dim), c_int(vdim), c_int(heads_per_group),
                         c_int(mode), c_float(q_scale), c_float(inv_tau), _ptr(bias), _ptr(rate), _ptr(skip),
                         c_int(2 if single_tokens else (1 if few_tokens else 0)), c_int(chunk_len), c_int(max_chunks),
                         _ptr(chunk_state),
                         _ptr(chunk_decay), _stream())


CONV_ACT_NONE, CONV_ACT_SILU = 0, 1


def causal_conv(u: torch.Tensor, u_off: int, channels: int, w: torch.Tensor, bias: Optional[torch.Tensor],
                state: torch.Tensor, y: torch.Tensor, token_slot: torch.Tensor, cu_seqlens: torch.Tensor,
                seq_slot: torch.Tensor, n_seqs: int, single_tokens: bool = False, act: int = CONV_ACT_SILU,
                add_input: bool = False, copy: Optional[torch.Tensor] = None, mix_off: int = 0,
                mix_src: Optional[torch.Tensor] = None, mix_dst: Optional[torch.Tensor] = None,
                mix_lambda: Optional[torch.Tensor] = None) -> None:
    """``y[t, c] = act(bias[c] + sum_j w[c, taps-1-j] u[t-j, u_off + c])`` within each sequence; the
    inputs before a step's first token come from ``state`` (float32 ``[slots, taps-1, channels]``,
    oldest first), which is then moved on by the step's tokens.  ``act`` is silu or none;
    ``add_input`` adds ``u[t]`` to the result; ``copy`` receives ``u[t]`` itself in the output's type.
    The input may be float32 with a bfloat16 output.  For channels from ``mix_off`` on, ``mix_src``
    (rows of ``channels - mix_off`` values in the output's type) is mixed in as
    ``(1 - lambda) y + lambda mix_src`` with ``mix_lambda`` one float32 on the device, and
    ``mix_dst`` receives the resulting values."""
    _need_cuda(u, w, bias, state, y, token_slot, cu_seqlens, seq_slot, copy, mix_src, mix_dst, mix_lambda)
    _rows_2d(u, "convolution input")
    _rows_2d(y, "convolution output")
    _i32(token_slot, "token slots")
    _i32(cu_seqlens, "cu_seqlens")
    _i32(seq_slot, "sequence slots")
    taps = w.shape[1] if w.dim() == 2 else 0
    if w.shape != (channels, taps) or not w.is_contiguous() or taps < 1:
        raise KernelError(f"causal_conv: weights must be contiguous [{channels}, taps]")
    if bias is not None and (bias.shape != (channels,) or bias.dtype != w.dtype or not bias.is_contiguous()):
        raise KernelError(f"causal_conv: bias must be [{channels}] of the weights' dtype")
    if (u.dtype != y.dtype and u.dtype != torch.float32) or y.shape != (u.shape[0], channels) or u_off + channels > u.shape[1]:
        raise KernelError("causal_conv: the output has the input's dtype (or the input is float32); output [tokens, channels]")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (max(taps - 1, 0), channels):
        raise KernelError("causal_conv: the state must be contiguous float32 [slots, taps-1, channels]")
    if copy is not None:
        _rows_2d(copy, "copy of the convolution's input")
        if copy.shape != y.shape or copy.dtype != y.dtype:
            raise KernelError("causal_conv: the copy must have the output's shape and dtype")
    mix_stride = 0
    for m in (mix_src, mix_dst):
        if m is not None:
            _rows_2d(m, "mixed channels")
            if m.shape != (u.shape[0], channels - mix_off) or m.dtype != y.dtype or mix_off < 0:
                raise KernelError(f"causal_conv: mixed channels must be [tokens, {channels - mix_off}] of the output's dtype")
            if mix_stride not in (0, m.stride(0)):
                raise KernelError("causal_conv: the two mixed buffers must share a row stride")
            mix_stride = m.stride(0)
    if mix_src is not None:
        _f32_vector(mix_lambda, 1, "causal_conv: the mixing factor")
        if mix_lambda is None:
            raise KernelError("causal_conv: mixing needs its factor")
    library("core").call("bfi_causal_conv", _ptr(u), c_long(u.stride(0)), c_int(u_off), c_int(dtype_code(u.dtype)),
                         _ptr(w), _ptr(bias), c_int(dtype_code(w.dtype)), _ptr(state), _ptr(y), c_long(y.stride(0)),
                         c_int(dtype_code(y.dtype)), _ptr(token_slot), _ptr(cu_seqlens), _ptr(seq_slot), c_int(u.shape[0]),
                         c_int(n_seqs), c_int(channels), c_int(taps), c_int(1 if single_tokens else 0), c_int(act),
                         c_int(1 if add_input else 0), _ptr(copy), c_long(0 if copy is None else copy.stride(0)),
                         c_int(mix_off), _ptr(mix_src), _ptr(mix_dst), c_long(mix_stride), _ptr(mix_lambda), _stream())


SCAN_CAND_IDENTITY, SCAN_CAND_POSITIVE = 0, 1


def gated_scan(proj: torch.Tensor, z_off: int, u_off: int, g_off: Optional[int], channels: int,
               z_bias: Optional[torch.Tensor], u_bias: Optional[torch.Tensor], y: torch.Tensor, state: torch.Tensor,
               cu_seqlens: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int, max_seq_tokens: int,
               cand: int = SCAN_CAND_POSITIVE) -> None:
    """A recurrence with one float32 state value per channel: with ``z = sigmoid(proj[z] + z_bias)``
    and ``u = proj[u] + u_bias``, ``S_t = (1 - z_t) S_(t-1) + z_t cand(u_t)`` and
    ``y_t = S_t * silu(proj[g])`` (``g_off`` None: ``y_t = S_t``).  ``cand`` is the identity or the
    positive map (``u + 1/2`` for ``u >= 0``, ``sigmoid(u)`` below).  ``state`` is ``[slots, channels]``
    and is moved on; ``max_seq_tokens`` (the most tokens a sequence brings) sizes the split over time."""
    _need_cuda(proj, z_bias, u_bias, y, state, cu_seqlens, seq_slot)
    _rows_2d(proj, "projections")
    _rows_2d(y, "recurrence output")
    _i32(cu_seqlens, "cu_seqlens")
    _i32(seq_slot, "sequence slots")
    _f32_vector(z_bias, channels, "gated_scan: the gate's bias")
    _f32_vector(u_bias, channels, "gated_scan: the candidate's bias")
    if y.dtype != proj.dtype or y.shape != (proj.shape[0], channels):
        raise KernelError("gated_scan: the output must be [tokens, channels] of the projections' dtype")
    if max(z_off, u_off, -1 if g_off is None else g_off) + channels > proj.shape[1] or min(z_off, u_off) < 0:
        raise KernelError("gated_scan: a column range lies outside the projections")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (channels,):
        raise KernelError("gated_scan: the state must be contiguous float32 [slots, channels]")
    library("core").call("bfi_gated_scan", _ptr(proj), c_long(proj.stride(0)), c_int(z_off), c_int(u_off),
                         c_int(-1 if g_off is None else g_off), c_int(dtype_code(proj.dtype)), _ptr(z_bias), _ptr(u_bias),
                         _ptr(y), c_long(y.stride(0)), _ptr(state), _ptr(cu_seqlens), _ptr(seq_slot), c_int(n_seqs),
                         c_int(channels), c_int(cand), c_int(max_seq_tokens), _stream())


def bias_act(u: torch.Tensor, bias: Optional[torch.Tensor], y: torch.Tensor, fill: Optional[torch.Tensor] = None,
             fill_bias: Optional[torch.Tensor] = None) -> None:
    """``y[t, j] = gelu_tanh(u[t, j] + bias[j])`` over rows of one storage type; with ``fill`` (float32
    rows) and ``fill_bias``, ``fill[t, :] = fill_bias`` in the same launch: the bias of a product that
    then accumulates into those rows."""
    _need_cuda(u, bias, y, fill, fill_bias)
    _rows_2d(u, "activation input")
    _rows_2d(y, "activation output")
    if y.shape != u.shape or y.dtype != u.dtype:
        raise KernelError("bias_act: input and output of one shape and dtype")
    if bias is not None and (bias.shape != (u.shape[1],) or not bias.is_contiguous()):
        raise KernelError(f"bias_act: the bias must be [{u.shape[1]}]")
    if (fill is None) != (fill_bias is None):
        raise KernelError("bias_act: rows to fill come with their bias")
    if fill is not None:
        _rows_2d(fill, "rows to fill")
        if fill.dtype != torch.float32 or fill.shape[0] != u.shape[0] or fill_bias.shape != (fill.shape[1],) \
                or not fill_bias.is_contiguous():
            raise KernelError("bias_act: the rows to fill are float32 [rows, n] and their bias [n]")
    library("core").call("bfi_bias_act", _ptr(u), c_long(u.stride(0)), c_int(dtype_code(u.dtype)), _ptr(bias),
                         c_int(0 if bias is None else dtype_code(bias.dtype)), _ptr(y), c_long(y.stride(0)), c_int(u.shape[0]),
                         c_int(u.shape[1]), _ptr(fill), c_long(0 if fill is None else fill.stride(0)), _ptr(fill_bias),
                         c_int(0 if fill_bias is None else dtype_code(fill_bias.dtype)),
                         c_int(0 if fill is None else fill.shape[1]), _stream())


def sigmoid_gate(x: torch.Tensor, g: torch.Tensor, group: int) -> None:
    """``x[t, j] *= sigmoid(g[t, j // group])`` in place, over rows of one storage type."""
    _need_cuda(x, g)
    _rows_2d(x, "rows to gate")
    _rows_2d(g, "gate logits")
    if group < 1 or x.shape[1] % group != 0 or g.shape != (x.shape[0], x.shape[1] // group) or g.dtype != x.dtype:
        raise KernelError("sigmoid_gate: logits [rows, cols / group] of the rows' dtype")
    library("core").call("bfi_sigmoid_gate", _ptr(x), c_long(x.stride(0)), _ptr(g), c_long(g.stride(0)),
                         c_int(dtype_code(x.dtype)), c_int(x.shape[0]), c_int(x.shape[1]), c_int(group), _stream())


GATE_SIGMOID, GATE_SILU = 0, 1


def gated_group_norm(x: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor, parts: int,
                     gate_first: bool, gate_act: int = GATE_SILU) -> None:
    """A row cut into ``parts`` equal parts, each divided by its own root mean square, times ``w``
    (which repeats along the row when shorter), with a gate ``act(gate)`` applied before the norm
    (``gate_first``) or after it.  ``x`` float32; ``gate`` and ``out`` in the activation dtype."""
    _need_cuda(x, gate, w, out)
    _rows_2d(x, "norm input")
    _rows_2d(gate, "gate")
    _rows_2d(out, "norm output")
    n, width = x.shape
    if x.dtype != torch.float32 or gate.dtype != out.dtype or gate.shape != (n, width) or out.shape != (n, width):
        raise KernelError("gated_group_norm: x float32 [rows, width]; gate and output [rows, width] of one dtype")
    if w.dim() != 1 or not w.is_contiguous():
        raise KernelError("gated_group_norm: the weight must be a contiguous vector")
    library("core").call("bfi_gated_group_norm", _ptr(x), c_long(x.stride(0)), _ptr(gate), c_long(gate.stride(0)),
                         c_int(dtype_code(out.dtype)), _ptr(w), c_int(dtype_code(w.dtype)), c_int(w.numel()), _ptr(out),
                         c_long(out.stride(0)), c_int(n), c_int(width), c_int(parts), c_int(1 if gate_first else 0),
                         c_int(gate_act), c_float(eps), _stream())


SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1
EXPERT_GATED_SILU, EXPERT_RELU_SQUARED = 0, 1


def moe_route(z: torch.Tensor, n_experts: int, correction: Optional[torch.Tensor], idx: torch.Tensor,
              weight: torch.Tensor, top: int, n_groups: int = 1, keep: int = 1, weight_scale: float = 1.0,
              gate: Optional[torch.Tensor] = None, score: int = SCORE_SOFTMAX, group_top: int = 1) -> None:
    """The router's decision per token from float32 logits ``z[:, :n_experts]``: scores ``s`` (the
    softmax over the experts, or with ``SCORE_SIGMOID`` each expert's own sigmoid), choice
    scores ``s + correction``, the ``keep`` best of ``n_groups`` groups (a group counts by the sum of
    its ``group_top`` largest choice scores), the ``top`` best experts of
    those; ``idx`` int32 and ``weight`` float32 ``[tokens, top]`` (the chosen ``s`` times
    ``weight_scale``).  With ``gate`` (float32 ``[tokens]``): ``sigmoid(z[:, n_experts])``."""
    _need_cuda(z, correction, idx, weight, gate)
    _rows_2d(z, "router logits")
    n = z.shape[0]
    if z.dtype != torch.float32:
        raise KernelError("moe_route: the logits must be float32")
    _f32_vector(correction, n_experts, "moe_route: the correction")
    if idx.dtype != torch.int32 or not idx.is_contiguous() or idx.shape != (n, top) or weight.dtype != torch.float32 \
            or not weight.is_contiguous() or weight.shape != (n, top):
        raise KernelError("moe_route: idx int32 and weight float32, both contiguous [tokens, top]")
    if gate is not None and (gate.dtype != torch.float32 or not gate.is_contiguous() or gate.numel() < n):
        raise KernelError("moe_route: the gate must be contiguous float32 [tokens]")
    library("core").call("bfi_moe_route", _ptr(z), c_long(z.stride(0)), _ptr(correction), _ptr(idx), _ptr(weight), _ptr(gate),
                         c_int(n), c_int(n_experts), c_int(top), c_int(n_groups), c_int(keep), c_float(weight_scale),
                         c_int(0 if gate is None else 1), c_int(score), c_int(group_top), _stream())


def moe_router(h: torch.Tensor, w_router: torch.Tensor, n_experts: int, correction: Optional[torch.Tensor],
               token_slot: torch.Tensor, idx: torch.Tensor, weight: torch.Tensor, top: int, n_groups: int = 1, keep: int = 1,
               weight_scale: float = 1.0, gate: Optional[torch.Tensor] = None, score: int = SCORE_SOFTMAX,
               group_top: int = 1) -> None:
    """``moe_route`` with the logits made in the same kernel: ``z = w_router h`` with ``w_router``
    float32 ``[n_experts (+ 1), width]`` (the extra row is the gate's, wanted with ``gate``)."""
    _need_cuda(h, w_router, correction, token_slot, idx, weight, gate)
    _rows_2d(h, "router input")
    n, width = h.shape
    rows = n_experts + (0 if gate is None else 1)
    if w_router.dtype != torch.float32 or not w_router.is_contiguous() or w_router.shape != (rows, width):
        raise KernelError(f"moe_router: the router's rows must be contiguous float32 [{rows}, {width}]")
    _f32_vector(correction, n_experts, "moe_router: the correction")
    _i32(token_slot, "token slots")
    if idx.dtype != torch.int32 or not idx.is_contiguous() or idx.shape != (n, top) or weight.dtype != torch.float32 \
            or not weight.is_contiguous() or weight.shape != (n, top):
        raise KernelError("moe_router: idx int32 and weight float32, both contiguous [tokens, top]")
    if gate is not None and (gate.dtype != torch.float32 or not gate.is_contiguous() or gate.numel() < n):
        raise KernelError("moe_router: the gate must be contiguous float32 [tokens]")
    library("core").call("bfi_moe_router", _ptr(h), c_long(h.stride(0)), c_int(dtype_code(h.dtype)), _ptr(w_router),
                         _ptr(correction), _ptr(token_slot), _ptr(idx), _ptr(weight), _ptr(gate), c_int(n), c_int(width),
                         c_int(n_experts), c_int(top), c_int(n_groups), c_int(keep), c_float(weight_scale),
                         c_int(0 if gate is None else 1), c_int(score), c_int(group_top), _stream())


def moe_gate_up(h: torch.Tensor, w_gu: torch.Tensor, n_experts: int, idx: torch.Tensor, token_slot: torch.Tensor,
                act: torch.Tensor, kind: int = EXPERT_GATED_SILU) -> None:
    """``act[t, k] = silu(gate_e h_t) * (up_e h_t)`` with ``e = idx[t, k]``; ``w_gu`` is
    ``[experts * 2 * ff, width]`` with expert e's gate row j at row ``2 (e ff + j)`` and its up row
    after it, ``act`` ``[tokens * top, ff]``.  ``EXPERT_RELU_SQUARED``: ``act[t, k] = relu(up_e h_t)^2``
    with ``w_gu`` ``[experts * ff, width]``, the experts' up matrices one after the other.  ``idx``
    None (with one expert): every token uses that expert."""
    _need_cuda(h, w_gu, idx, token_slot, act)
    _rows_2d(h, "feed-forward input")
    n, width = h.shape
    if idx is None and n_experts != 1:
        raise KernelError("moe_gate_up: without choices there is one expert")
    top = 1 if idx is None else idx.shape[1]
    per = 1 if kind == EXPERT_RELU_SQUARED else 2
    ff = w_gu.shape[0] // (per * n_experts)
    if w_gu.dim() != 2 or w_gu.shape != (n_experts * per * ff, width) or not w_gu.is_contiguous() or w_gu.dtype != h.dtype:
        raise KernelError(f"moe_gate_up: expert weights must be contiguous [experts * {per} * ff, width] of the input's dtype")
    if act.dtype != h.dtype or not act.is_contiguous() or act.shape != (n * top, ff):
        raise KernelError("moe_gate_up: the output must be contiguous [tokens * top, ff] of the input's dtype")
    _i32(idx, "expert choices")
    _i32(token_slot, "token slots")
    library("core").call("bfi_moe_gate_up", _ptr(h), c_long(h.stride(0)), c_int(dtype_code(h.dtype)), _ptr(w_gu),
                         _ptr(idx), _ptr(token_slot), _ptr(act), c_int(n), c_int(top), c_int(width), c_int(ff), c_int(kind),
                         _stream())


def moe_down(act: torch.Tensor, w_down: torch.Tensor, n_experts: int, idx: torch.Tensor, weight: torch.Tensor,
             token_slot: torch.Tensor, out: torch.Tensor, shared_out: Optional[torch.Tensor] = None,
             gate: Optional[torch.Tensor] = None, accumulate: bool = False) -> None:
    """``out[t] (= | +=) sum_k weight[t, k] * down_e act[t, k] + gate[t] * shared_out[t]`` with
    ``e = idx[t, k]`` (the last term only with ``shared_out``; ``gate`` None is 1); ``w_down`` is
    ``[width, experts * ff]`` with expert e's columns at ``e ff`` (its rows may be further apart: the
    first columns of a wider matrix), ``out`` float32 ``[tokens, width]``."""
    _need_cuda(act, w_down, idx, weight, token_slot, out, shared_out, gate)
    _rows_2d(out, "feed-forward output")
    _rows_2d(w_down, "expert down matrices")
    n, top = idx.shape
    width, ff = w_down.shape[0], w_down.shape[1] // n_experts
    if w_down.shape[1] != n_experts * ff or w_down.dtype != act.dtype:
        raise KernelError("moe_down: expert weights must be [width, experts * ff] of the activations' dtype")
    if not act.is_contiguous() or act.shape != (n * top, ff):
        raise KernelError("moe_down: the activations must be contiguous [tokens * top, ff]")
    if out.dtype != torch.float32 or out.shape != (n, width):
        raise KernelError("moe_down: the output must be float32 [tokens, width]")
    if shared_out is not None and (shared_out.dtype != torch.float32 or shared_out.shape != (n, width) or shared_out.stride(1) != 1):
        raise KernelError("moe_down: the shared output must be float32 [tokens, width]")
    library("core").call("bfi_moe_down", _ptr(act), c_int(dtype_code(act.dtype)), _ptr(w_down), _ptr(idx), _ptr(weight),
                         _ptr(token_slot), _ptr(shared_out), c_long(0 if shared_out is None else shared_out.stride(0)),
                         _ptr(gate), _ptr(out), c_long(out.stride(0)), c_int(n), c_int(top), c_int(width), c_int(ff),
                         c_long(w_down.stride(0)), c_int(1 if accumulate else 0), _stream())


def moe_weigh_dense(act: torch.Tensor, n_experts: int, idx: torch.Tensor, weight: torch.Tensor,
                    token_slot: torch.Tensor, tail: int = 0, gate: Optional[torch.Tensor] = None,
                    kind: int = EXPERT_GATED_SILU) -> None:
    """``act[t, e ff + j] *= (weight of expert e for token t, 0 if it was not chosen)`` over
    activations ``[tokens, experts * ff + tail]`` that the dense product computed for every expert;
    the last ``tail`` columns (an expert every token uses) are multiplied by ``gate[t]`` (None: 1).
    ``EXPERT_RELU_SQUARED``: the columns hold the up products themselves and become ``relu(u)^2``
    here, before their weight."""
    _need_cuda(act, idx, weight, token_slot, gate)
    _rows_2d(act, "dense expert activations")
    _i32(idx, "expert choices")
    _i32(token_slot, "token slots")
    n, top = idx.shape
    routed = act.shape[1] - tail
    if act.shape[0] != n or tail < 0 or routed <= 0 or routed % n_experts != 0 or weight.dtype != torch.float32 \
            or not weight.is_contiguous() or weight.shape != (n, top):
        raise KernelError("moe_weigh_dense: activations [tokens, experts * ff + tail], weights float32 [tokens, top]")
    if tail and kind == EXPERT_GATED_SILU and gate is None:
        raise KernelError("moe_weigh_dense: the tail needs one float32 gate per token")
    if gate is not None and (gate.dtype != torch.float32 or not gate.is_contiguous() or gate.numel() < n):
        raise KernelError("moe_weigh_dense: the gate must be contiguous float32 with one value per token")
    library("core").call("bfi_moe_weigh_dense", _ptr(act), c_long(act.stride(0)), c_int(dtype_code(act.dtype)), _ptr(idx),
                         _ptr(weight), _ptr(token_slot), c_int(n), c_int(top), c_int(n_experts), c_int(routed // n_experts),
                         c_int(tail), _ptr(gate), c_int(kind), _stream())


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """``out = a @ w.T`` on the CUDA cores in float32 arithmetic (any dtypes, any sizes)."""
    _need_cuda(a, w, out)
    _rows_2d(a, "A")
    _rows_2d(w, "W")
    _rows_2d(out, "C")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"matrix product: A is {tuple(a.shape)} but W is {tuple(w.shape)}")
    cols = n // 2 if epilogue == EPI_SWIGLU else n
    if out.shape != (m, cols):
        raise KernelError(f"matrix product: output must be [{m}, {cols}], got {tuple(out.shape)}")
    library("core").call("bfi_gemm_simt", _ptr(a), c_int(dtype_code(a.dtype)), c_long(a.stride(0)), _ptr(w),
                         c_int(dtype_code(w.dtype)), c_long(w.stride(0)), _ptr(out), c_int(dtype_code(out.dtype)),
                         c_long(out.stride(0)), c_int(m), c_int(n), c_int(k), c_int(epilogue), _stream())


def argmax_rows(logits: torch.Tensor, out: torch.Tensor, scratch: Optional[torch.Tensor] = None) -> None:
    """``scratch`` (int32 or float32, at least ``2 * rows * ceil(vocab / 8192)`` values) lets many
    blocks search each row of a large vocabulary."""
    _need_cuda(logits, out, scratch)
    _rows_2d(logits, "logits")
    _i32(out, "argmax output")
    if logits.dtype != torch.float32 or out.numel() < logits.shape[0]:
        raise KernelError("argmax: logits must be float32 and the output hold one id per row")
    n_scratch = 0
    if scratch is not None:
        if scratch.element_size() != 4 or not scratch.is_contiguous():
            raise KernelError("argmax: scratch must be a contiguous tensor of 4-byte values")
        n_scratch = scratch.numel()
    library("core").call("bfi_argmax_rows", _ptr(logits), c_long(logits.stride(0)), c_int(logits.shape[0]),
                         c_int(logits.shape[1]), _ptr(out), _ptr(scratch), c_long(n_scratch), _stream())


def sample_sorted_rows(logits: torch.Tensor, temperature: torch.Tensor, u: torch.Tensor, out: torch.Tensor,
                       probs: torch.Tensor, top_k: int = 0, top_p: float = 1.0, repeat_penalty: float = 1.0,
                       presence_penalty: float = 0.0, min_p: float = 0.0, seen: Optional[torch.Tensor] = None,
                       seen_cu: Optional[torch.Tensor] = None, work: Optional[torch.Tensor] = None) -> None:
    """Top-k / top-p sampling in the reference's order (probability descending, index ascending)
    without a sort; ``probs`` is float32 scratch ``[rows, vocab]``."""
    _need_cuda(logits, temperature, u, out, probs, seen, seen_cu, work)
    _rows_2d(logits, "logits")
    _i32(out, "sample output")
    _i32(seen, "seen ids")
    _i32(seen_cu, "seen offsets")
    rows, vocab = logits.shape
    for t, what in ((temperature, "temperature"), (u, "uniform draws")):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() < rows:
            raise KernelError(f"{what} must be contiguous float32 with one value per row")
    if logits.dtype != torch.float32 or out.numel() < rows:
        raise KernelError("sample: logits must be float32 and the output hold one id per row")
    for buf, what in ((probs, "probability"), (work, "work")):
        if buf is not None and (buf.dtype != torch.float32 or not buf.is_contiguous() or buf.numel() < rows * vocab):
            raise KernelError(f"sample: {what} buffer must be contiguous float32 [rows, vocab]")
    library("core").call("bfi_sample_sorted_rows", _ptr(logits), c_long(logits.stride(0)), _ptr(work), _ptr(probs),
                         c_int(rows), c_int(vocab), _ptr(seen), _ptr(seen_cu), _ptr(temperature), _ptr(u),
                         c_float(repeat_penalty), c_float(presence_penalty), c_int(int(top_k)), c_float(top_p),
                         c_float(min_p), _ptr(out), _stream())


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, u: torch.Tensor, out: torch.Tensor,
                repeat_penalty: float = 1.0, presence_penalty: float = 0.0, min_p: float = 0.0,
                seen: Optional[torch.Tensor] = None, seen_cu: Optional[torch.Tensor] = None,
                work: Optional[torch.Tensor] = None) -> None:
    _need_cuda(logits, temperature, u, out, seen, seen_cu, work)
    _rows_2d(logits, "logits")
    _i32(out, "sample output")
    _i32(seen, "seen ids")
    _i32(seen_cu, "seen offsets")
    rows, vocab = logits.shape
    for t, what in ((temperature, "temperature"), (u, "uniform draws")):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() < rows:
            raise KernelError(f"{what} must be contiguous float32 with one value per row")
    if logits.dtype != torch.float32 or out.numel() < rows:
        raise KernelError("sample: logits must be float32 and the output hold one id per row")
    if work is not None and (work.dtype != torch.float32 or not work.is_contiguous() or work.numel() < rows * vocab):
        raise KernelError("sample: work buffer must be contiguous float32 [rows, vocab]")
    library("core").call("bfi_sample_rows", _ptr(logits), c_long(logits.stride(0)), _ptr(work), c_int(rows),
                         c_int(vocab), _ptr(seen), _ptr(seen_cu), _ptr(temperature), _ptr(u),
                         c_float(repeat_penalty), c_float(presence_penalty), c_float(min_p), _ptr(out), _stream())
