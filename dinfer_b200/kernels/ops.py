"""Typed Python wrappers over the C ABI of the kernel libraries.

Each wrapper checks what the kernel cannot (device, dtype, contiguity of the last axis), passes
explicit strides and the live token count, and launches on torch's current stream.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .lib import KernelError, check, dtype_code, library, ptr, require_cuda, stream_handle

_sigs_done = set()


def _fn(libname: str, fname: str, argtypes):
    lib = library(libname)
    f = getattr(lib, fname)
    if (libname, fname) not in _sigs_done:
        f.argtypes = argtypes
        f.restype = c_int
        _sigs_done.add((libname, fname))
    return lib, f


def _rows_contiguous(t: torch.Tensor, what: str) -> None:
    if t.dim() < 1 or t.stride(-1) != 1:
        raise KernelError(f"{what}: last axis must be contiguous")


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
              prev: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] * scale into the f32 residual stream.  With ``prev`` (int32 [rows], the tokens
    the previous step sampled) an id -(r + 1) stands for prev[r]."""
    require_cuda(ids, table, out)
    T, h = out.shape
    if ids.dtype != torch.int32 or out.dtype != torch.float32 or not out.is_contiguous() \
            or not table.is_contiguous() or table.shape[1] != h or ids.numel() != T:
        raise KernelError("embedding: ids int32 [T], table [V, h] contiguous, out f32 [T, h] contiguous")
    if prev is not None:
        require_cuda(prev)
        if prev.dtype != torch.int32 or prev.dim() != 1 or not prev.is_contiguous():
            raise KernelError("embedding: prev int32 [rows] contiguous")
    lib, f = _fn("elementwise", "dinfer_embedding",
                 [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    check(lib, f(ptr(ids), ptr(prev) if prev is not None else None, prev.numel() if prev is not None else 0,
                 ptr(table), ptr(out), T, h, table.shape[0], dtype_code(table.dtype), float(scale), stream_handle()),
          "embedding")
    return out


def embedding_bigram(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, bigram: Optional[torch.Tensor],
                     hashing, pos_table: Optional[torch.Tensor], positions: torch.Tensor, cu_seqlens: torch.Tensor,
                     slots: torch.Tensor, fresh: torch.Tensor, last: Optional[torch.Tensor],
                     prev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[id] + bigram[(before * mul_prev + id * mul_cur) mod buckets] + pos_table[positions[t]]`` into the
    f32 residual stream; ``hashing`` = (buckets, mul_prev, mul_cur); ``before`` is the token before in the same request
    (row ``buckets`` of the bigram table for a request's first token).  The token before a step's first one comes from
    ``last[slots[b]]`` (int32, one per state slot; not read for a fresh request), which then takes the request's last
    token of this step.  ``bigram`` / ``pos_table`` None: that term is left out.  ``prev``: as in ``embedding``."""
    require_cuda(ids, table, out, bigram, pos_table, positions, cu_seqlens, slots, fresh, last, prev)
    T, h = out.shape
    if ids.dtype != torch.int32 or out.dtype != torch.float32 or not out.is_contiguous() \
            or not table.is_contiguous() or table.shape[1] != h or ids.numel() != T:
        raise KernelError("embedding_bigram: ids int32 [T], table [V, h] contiguous, out f32 [T, h] contiguous")
    buckets, mul_prev, mul_cur = (int(v) for v in hashing) if bigram is not None else (0, 0, 0)
    if bigram is not None:
        if bigram.dtype != table.dtype or not bigram.is_contiguous() or tuple(bigram.shape) != (buckets + 1, h):
            raise KernelError("embedding_bigram: the bigram table is [buckets + 1, h] of the table's dtype")
        if last is None or last.dtype != torch.int32 or not last.is_contiguous():
            raise KernelError("embedding_bigram: last int32 [state slots]")
    if pos_table is not None and (pos_table.dtype != table.dtype or not pos_table.is_contiguous() or pos_table.shape[1] != h):
        raise KernelError("embedding_bigram: the position table is [positions, h] of the table's dtype")
    for t in (positions, cu_seqlens, slots, fresh) + ((prev,) if prev is not None else ()):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("embedding_bigram: positions, offsets, slots, fresh flags and prev are contiguous int32")
    B = cu_seqlens.numel() - 1
    lib, f = _fn("elementwise", "dinfer_embedding_bigram",
                 [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(ids), ptr(prev), prev.numel() if prev is not None else 0, ptr(table), ptr(bigram), ptr(pos_table),
                 ptr(positions), ptr(cu_seqlens), ptr(slots), ptr(fresh), ptr(last), B, ptr(out), T, h, table.shape[0],
                 buckets, mul_prev, mul_cur, pos_table.shape[0] if pos_table is not None else 0, dtype_code(table.dtype),
                 stream_handle()), "embedding_bigram")
    if bigram is not None and T > 0:
        from .lib import add_launches
        add_launches(1)                                   # the kernel that stores the requests' last tokens
    return out


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap) in place (float32, contiguous): logits with a soft cap."""
    require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous() or not cap > 0:
        raise KernelError("softcap: contiguous float32 values and a positive cap")
    lib, f = _fn("elementwise", "dinfer_softcap", [c_void_p, c_int64, c_float, c_void_p])
    check(lib, f(ptr(x), x.numel(), float(cap), stream_handle()), "softcap")
    return x


def scale(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place (float32, contiguous): logits with a fixed factor."""
    require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale: contiguous float32 values")
    lib, f = _fn("elementwise", "dinfer_scale", [c_void_p, c_int64, c_float, c_void_p])
    check(lib, f(ptr(x), x.numel(), float(factor), stream_handle()), "scale")
    return x


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, group: int = 1) -> torch.Tensor:
    """``x[t, i] *= sigmoid(gate[t, i // group])`` in place: one gate per element (``group`` 1) or per ``group``
    neighbouring elements (a head).  Rows of either may have a stride."""
    require_cuda(x, gate)
    _rows_contiguous(x, "sigmoid_gate")
    _rows_contiguous(gate, "sigmoid_gate")
    T, N = x.shape
    if gate.shape[0] != T or N % group or gate.shape[1] != N // group:
        raise KernelError("sigmoid_gate: x [T, N], gate [T, N / group]")
    lib, f = _fn("elementwise", "dinfer_sigmoid_gate",
                 [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), x.stride(0), ptr(gate), gate.stride(0), T, N, int(group), dtype_code(x.dtype),
                 dtype_code(gate.dtype), stream_handle()), "sigmoid_gate")
    return x


def rmsnorm(residual: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = rmsnorm(residual[src] + delta[src]) * weight, src = rows[r] or r; the sum is written
    back to ``residual`` when ``delta`` is given and ``rows`` is not."""
    require_cuda(residual, weight, out, delta, rows)
    h = residual.shape[-1]
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("rmsnorm: residual must be contiguous float32")
    if not out.is_contiguous() or out.shape[-1] != h or weight.numel() != h or not weight.is_contiguous():
        raise KernelError("rmsnorm: out [R, h] contiguous, weight [h]")
    if delta is not None and (delta.dtype != out.dtype or delta.shape != residual.shape or not delta.is_contiguous()):
        raise KernelError("rmsnorm: delta must have the residual's shape and the output's dtype")
    if rows is not None:
        if rows.dtype != torch.int32 or rows.numel() != out.shape[0]:
            raise KernelError("rmsnorm: rows must be int32 [R]")
        n = rows.numel()
    else:
        n = residual.shape[0]
        if out.shape[0] != n:
            raise KernelError("rmsnorm: out must have the residual's row count")
    lib, f = _fn("norm", "dinfer_rmsnorm",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p])
    check(lib, f(ptr(residual), ptr(delta), ptr(rows), ptr(weight), ptr(out), n, h, float(eps),
                 dtype_code(out.dtype), dtype_code(weight.dtype), stream_handle()), "rmsnorm")
    return out


def rmsnorm_plain(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    require_cuda(x, weight, out)
    h = x.shape[-1]
    if not x.is_contiguous() or not out.is_contiguous() or out.shape != x.shape or out.dtype != x.dtype \
            or weight.numel() != h:
        raise KernelError("rmsnorm_plain: x, out contiguous of one shape and dtype; weight [h]")
    lib, f = _fn("norm", "dinfer_rmsnorm_plain",
                 [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), ptr(weight), ptr(out), x.numel() // h, h, float(eps), dtype_code(x.dtype),
                 dtype_code(weight.dtype), stream_handle()), "rmsnorm_plain")
    return out


def silu_mul(x: torch.Tensor, out: torch.Tensor, pairs: bool = False) -> torch.Tensor:
    """out[t, i] = silu(gate_i) * up_i for x [T, 2I] that holds gate and up as halves (gate_i = x[t, i],
    up_i = x[t, I + i]) or, with ``pairs``, side by side (gate_i = x[t, 2i], up_i = x[t, 2i + 1])."""
    require_cuda(x, out)
    _rows_contiguous(x, "silu_mul")
    T, two_i = x.shape
    inter = two_i // 2
    if two_i % 2 or out.shape != (T, inter) or not out.is_contiguous() or out.dtype != x.dtype:
        raise KernelError("silu_mul: x [T, 2I], out [T, I] contiguous, same dtype")
    lib, f = _fn("elementwise", "dinfer_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), ptr(out), T, inter, x.stride(0), dtype_code(x.dtype), int(bool(pairs)), stream_handle()),
          "silu_mul")
    return out


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[t, :] += bias, in place (a view with a row stride is fine)."""
    require_cuda(out, bias)
    _rows_contiguous(out, "add_bias")
    if out.dim() != 2 or bias.dim() != 1 or bias.numel() != out.shape[1] or not bias.is_contiguous():
        raise KernelError("add_bias: out [T, N], bias [N]")
    lib, f = _fn("elementwise", "dinfer_add_bias", [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(out), out.stride(0), ptr(bias), out.shape[0], out.shape[1], dtype_code(out.dtype),
                 dtype_code(bias.dtype), stream_handle()), "add_bias")
    return out


def cast(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    require_cuda(src, dst)
    if not src.is_contiguous() or not dst.is_contiguous() or src.numel() != dst.numel():
        raise KernelError("cast: contiguous tensors of one length")
    lib, f = _fn("elementwise", "dinfer_cast", [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p])
    check(lib, f(ptr(src), ptr(dst), src.numel(), dtype_code(src.dtype), dtype_code(dst.dtype),
                 stream_handle()), "cast")
    return dst


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T, 32-bit multiply-adds on the CUDA cores; each operand f32 or bf16."""
    require_cuda(a, w, out)
    for t, n in ((a, "a"), (w, "w"), (out, "out")):
        if t.dim() != 2:
            raise KernelError(f"gemm_f32: {n} must be 2-D")
        _rows_contiguous(t, "gemm_f32 " + n)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    lib, f = _fn("gemm_f32", "dinfer_gemm_f32",
                 [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int,
                  c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(a), a.stride(0), dtype_code(a.dtype), ptr(w), w.stride(0), dtype_code(w.dtype),
                 ptr(out), out.stride(0), dtype_code(out.dtype), M, N, K, stream_handle()), "gemm_f32")
    return out


def qk_post(qkv: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
            eps: float, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
            cos_sin: Optional[torch.Tensor], cache: Optional[torch.Tensor],
            slots: Optional[torch.Tensor], block_size: int, interleaved: bool = False) -> None:
    """Per-head RMSNorm of q and k, rotation (element i with i + rot/2, or with ``interleaved`` element 2i with
    2i + 1), write-back in place, k and v into the paged cache."""
    require_cuda(qkv, positions, q_weight, k_weight, cos_sin, cache, slots)
    _rows_contiguous(qkv, "qk_post")
    T = qkv.shape[0]
    if positions.dtype != torch.int32 or positions.numel() != T:
        raise KernelError("qk_post: positions int32 [T]")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_post: q and k norm weights come together")
    w_dt = q_weight.dtype if q_weight is not None else torch.float32
    if q_weight is not None and (q_weight.numel() != head_dim or k_weight.numel() != head_dim
                                 or k_weight.dtype != w_dt):
        raise KernelError("qk_post: norm weights must be [head_dim] of one dtype")
    rot = 0
    if cos_sin is not None:
        if cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous() or cos_sin.dim() != 2:
            raise KernelError("qk_post: angle table must be contiguous float32 [max_pos, rot]")
        rot = cos_sin.shape[1]
    if cache is not None:
        if cache.dtype != qkv.dtype or not cache.is_contiguous() or slots is None or slots.dtype != torch.int32 \
                or slots.numel() != T:
            raise KernelError("qk_post: cache of the activations' dtype, contiguous; slots int32 [T]")
        if tuple(cache.shape[1:]) != (2, num_kv_heads, block_size, head_dim):
            raise KernelError(f"qk_post: cache shape {tuple(cache.shape)} is not [blocks, 2, {num_kv_heads}, "
                              f"{block_size}, {head_dim}]")
    lib, f = _fn("qk_post", "dinfer_qk_post_styled",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(qkv), qkv.stride(0), ptr(positions), ptr(q_weight), ptr(k_weight), float(eps),
                 ptr(cos_sin), rot, int(bool(interleaved)), ptr(cache), ptr(slots), block_size, T, num_heads, num_kv_heads,
                 head_dim, dtype_code(qkv.dtype), dtype_code(w_dt), stream_handle()), "qk_post")


def attention_generic(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      cu_seqlens: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int,
                      head_dim: int, scale: float, window: int = 0, v_dim: Optional[int] = None,
                      sink: bool = False, slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged causal attention, plain arithmetic, any head size.  ``q`` may be a strided view (for
    instance the q columns of the qkv rows).  ``v_dim``: the values' width where it differs from the keys' (the
    cache's rows are then ``max(head_dim, v_dim)`` wide, ``out`` holds head h at ``h * v_dim``); ``sink``: one more
    term of score 0 and no value in the softmax's denominator; ``slopes`` (f32 [H]): a distance bias,
    ``score_ij - slopes[h] * (i - j)``."""
    require_cuda(q, out, cache, block_table, cu_seqlens, positions, slopes)
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.numel() != num_heads or not slopes.is_contiguous()):
        raise KernelError("attention: slopes float32 [H]")
    _rows_contiguous(q, "attention q")
    _rows_contiguous(out, "attention out")
    T = q.shape[0]
    B = cu_seqlens.numel() - 1
    v_dim = head_dim if v_dim is None else int(v_dim)
    row = max(head_dim, v_dim)
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and cache must have one dtype")
    for t, n in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (positions, "positions")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"attention: {n} must be contiguous int32")
    if block_table.dim() != 2 or block_table.shape[0] < B or positions.numel() != T:
        raise KernelError("attention: block_table [B, max_blocks], positions [T]")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != row \
            or not cache.is_contiguous():
        raise KernelError(f"attention: cache shape {tuple(cache.shape)} is not [blocks, 2, Hkv, block, {row}]")
    lib, f = _fn("attention_generic", "dinfer_attention_generic_bias",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_void_p])
    check(lib, f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cache), ptr(block_table),
                 block_table.shape[1], ptr(cu_seqlens), ptr(positions), T, B, num_heads, num_kv_heads,
                 head_dim, v_dim, row, cache.shape[3], float(scale), int(window), int(bool(sink)), ptr(slopes),
                 dtype_code(q.dtype), stream_handle()), "attention_generic")
    return out


def qkv_post_general(qkv: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                     v_dim: int, eps: float, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                     norm: bool, norm_first: bool, cos_sin: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                     slots: Optional[torch.Tensor], block_size: int, interleaved: bool = False,
                     bias: Optional[torch.Tensor] = None, q_temperature=None, v_first: Optional[torch.Tensor] = None,
                     v_lambda: float = 0.0) -> None:
    """The general q/k/v post-processing: per-head RMS norm of q and k (``norm``; the weights may be None: a norm
    without a weight) before or behind (``norm_first``) the rotation, q and k written back in place, k and v (v of
    width ``v_dim``) into a paged cache whose rows are ``max(head_dim, v_dim)`` wide.  ``bias``: f32, one per column of
    the q, k, v projections, added first (a projection whose bias has no kernel of its own).  ``q_temperature`` =
    (coef, every): q at position p times ``1 + coef * ln(floor((p + 1) / every) + 1)``.  ``v_first`` [T, Hkv * v_dim]
    (rows with a stride are fine) and ``v_lambda``: the cache gets ``(1 - v_lambda) v + v_lambda v_first``."""
    require_cuda(qkv, positions, q_weight, k_weight, cos_sin, cache, slots, bias, v_first)
    coef, every = (float(q_temperature[0]), int(q_temperature[1])) if q_temperature else (0.0, 1)
    if v_first is not None and (v_first.dtype != qkv.dtype or v_first.stride(1) != 1 or v_first.shape[0] != qkv.shape[0]
                                or v_first.shape[1] != num_kv_heads * v_dim):
        raise KernelError("qkv_post_general: v_first [T, Hkv * v_dim] of the activations' dtype")
    if bias is not None and (bias.dtype != torch.float32 or not bias.is_contiguous()
                             or bias.numel() != (num_heads + num_kv_heads) * head_dim + num_kv_heads * v_dim):
        raise KernelError("qkv_post_general: bias f32 [(H + Hkv) * D + Hkv * Dv]")
    _rows_contiguous(qkv, "qkv_post_general")
    T = qkv.shape[0]
    row = max(head_dim, v_dim)
    if positions.dtype != torch.int32 or positions.numel() != T:
        raise KernelError("qkv_post_general: positions int32 [T]")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qkv_post_general: q and k norm weights come together")
    w_dt = q_weight.dtype if q_weight is not None else torch.float32
    if q_weight is not None and (q_weight.numel() != head_dim or k_weight.numel() != head_dim or k_weight.dtype != w_dt):
        raise KernelError("qkv_post_general: norm weights must be [head_dim] of one dtype")
    rot = 0
    if cos_sin is not None:
        if cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous() or cos_sin.dim() != 2:
            raise KernelError("qkv_post_general: angle table must be contiguous float32 [max_pos, rot]")
        rot = cos_sin.shape[1]
    if cache is not None:
        if cache.dtype != qkv.dtype or not cache.is_contiguous() or slots is None or slots.dtype != torch.int32 \
                or slots.numel() != T or tuple(cache.shape[1:]) != (2, num_kv_heads, block_size, row):
            raise KernelError(f"qkv_post_general: cache [blocks, 2, {num_kv_heads}, {block_size}, {row}] of the "
                              f"activations' dtype, contiguous; slots int32 [T]")
    lib, f = _fn("qk_post", "dinfer_qkv_post_mixed",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_int,
                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_int, c_void_p,
                  c_int64, c_float, c_int, c_int, c_void_p])
    check(lib, f(ptr(qkv), qkv.stride(0), ptr(positions), ptr(q_weight), ptr(k_weight), int(bool(norm)),
                 int(bool(norm_first)), float(eps), ptr(cos_sin), rot, int(bool(interleaved)), ptr(cache), ptr(slots),
                 block_size, T, num_heads, num_kv_heads, head_dim, v_dim, row, ptr(bias), coef, every, ptr(v_first),
                 v_first.stride(0) if v_first is not None else 0, float(v_lambda), dtype_code(qkv.dtype), dtype_code(w_dt),
                 stream_handle()), "qkv_post_general")


def branch_norm(a: torch.Tensor, weight: Optional[torch.Tensor], eps: float, residual: Optional[torch.Tensor] = None,
                out32: Optional[torch.Tensor] = None, cast: Optional[torch.Tensor] = None,
                inner=None, b: Optional[torch.Tensor] = None, coef: float = 1.0, inner_eps: float = 0.0):
    """A branch output normed before it joins the residual stream: ``residual += rms(y) * weight`` (or ``out32 = ...``
    without a residual; ``weight`` None: no outer norm), ``cast = T(residual)`` on the way (T the cast's own dtype;
    the branches may be wider: 32-bit outputs of their last products).  ``y = a``, or with
    ``inner = (w_a, w_b)``: ``y = coef * (rms(a) * w_a + rms(b) * w_b)`` (``b`` None: one branch).  32-bit throughout."""
    require_cuda(a, b, weight, residual, out32, cast)
    R, h = a.shape
    wa, wb = inner if inner is not None else (None, None)
    ws = [w for w in (weight, wa, wb) if w is not None]
    w_dt = ws[0].dtype if ws else torch.float32
    for w in ws:
        _opt_vec(w, h, w_dt, "branch_norm: a weight")
    if not a.is_contiguous() or (b is not None and (b.shape != a.shape or b.dtype != a.dtype or not b.is_contiguous())):
        raise KernelError("branch_norm: branches [R, h] contiguous of one dtype")
    for t in (residual, out32, cast):
        if t is not None and (tuple(t.shape) != (R, h) or not t.is_contiguous()
                              or (t is not cast and t.dtype != torch.float32)):
            raise KernelError("branch_norm: residual / out32 f32 [R, h], cast [R, h], contiguous")
    lib, f = _fn("norm", "dinfer_branch_norm",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_float, c_void_p, c_void_p,
                  c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(a), ptr(wa), ptr(b), ptr(wb), float(coef), float(inner_eps), ptr(weight), float(eps),
                 ptr(residual), ptr(out32), ptr(cast), R, h, dtype_code(a.dtype),
                 dtype_code(cast.dtype if cast is not None else a.dtype), dtype_code(w_dt), stream_handle()),
          "branch_norm")
    return residual if residual is not None else out32


def _opt_vec(t: Optional[torch.Tensor], h: int, dt: torch.dtype, what: str) -> None:
    if t is not None and (t.numel() != h or t.dtype != dt or not t.is_contiguous()):
        raise KernelError(f"{what} must be [{h}] of {dt}, contiguous")


def layernorm(residual: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, out: torch.Tensor,
              deltas=(), rows: Optional[torch.Tensor] = None, weight2: Optional[torch.Tensor] = None,
              bias2: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None):
    """Layer norm of ``v = residual[src] + sum_i deltas[i][0][src] * deltas[i][1]`` (up to two deltas, each with a
    per-channel scale or None; src = rows[r] or r) with weight and bias; with ``out2`` a second norm of the same
    rows with its own weight and bias.  The sum is written back to ``residual`` when a delta is given and
    ``rows`` is not."""
    deltas = [d for d in deltas if d is not None]
    if len(deltas) > 2:
        raise KernelError("layernorm: at most two pending deltas")
    require_cuda(residual, weight, bias, out, rows, weight2, bias2, out2)
    h = residual.shape[-1]
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("layernorm: residual must be contiguous float32")
    wdt = weight.dtype
    for t, n in ((weight, "weight"), (bias, "bias"), (weight2, "weight2"), (bias2, "bias2")):
        _opt_vec(t, h, wdt, "layernorm: " + n)
    n = rows.numel() if rows is not None else residual.shape[0]
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("layernorm: rows must be int32")
    for o in (out, out2):
        if o is not None and (not o.is_contiguous() or tuple(o.shape) != (n, h) or o.dtype != out.dtype):
            raise KernelError("layernorm: outputs [R, h] contiguous of one dtype")
    if out2 is not None and weight2 is None:
        raise KernelError("layernorm: a second output needs its weight")
    args = []
    for d, s in deltas + [(None, None)] * (2 - len(deltas)):
        if d is not None:
            require_cuda(d, s)
            if d.dtype != out.dtype or d.shape != residual.shape or not d.is_contiguous():
                raise KernelError("layernorm: a delta must have the residual's shape and the output's dtype")
            _opt_vec(s, h, wdt, "layernorm: a delta's scale")
        args += [ptr(d), ptr(s)]
    lib, f = _fn("norm", "dinfer_layernorm", [c_void_p] * 12 + [c_int, c_int, c_float, c_int, c_int, c_void_p])
    check(lib, f(ptr(residual), *args, ptr(rows), ptr(weight), ptr(bias), ptr(out), ptr(weight2), ptr(bias2), ptr(out2),
                 n, h, float(eps), dtype_code(out.dtype), dtype_code(wdt), stream_handle()), "layernorm")
    return out if out2 is None else (out, out2)


def scaled_add(residual: torch.Tensor, deltas) -> torch.Tensor:
    """residual += sum_i deltas[i][0] * deltas[i][1] (up to two; a scale [h] or None), 32-bit, in place."""
    deltas = [d for d in deltas if d is not None and d[0] is not None]
    if not deltas:
        return residual
    if len(deltas) > 2:
        raise KernelError("scaled_add: at most two deltas")
    h = residual.shape[-1]
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("scaled_add: residual must be contiguous float32")
    adt = deltas[0][0].dtype
    wdt = next((s.dtype for _, s in deltas if s is not None), torch.float32)
    args = []
    for d, s in deltas + [(None, None)] * (2 - len(deltas)):
        if d is not None:
            require_cuda(d, s)
            if d.dtype != adt or d.shape != residual.shape or not d.is_contiguous():
                raise KernelError("scaled_add: a delta must have the residual's shape")
            _opt_vec(s, h, wdt, "scaled_add: a scale")
        args += [ptr(d), ptr(s)]
    lib, f = _fn("norm", "dinfer_scaled_add", [c_void_p] * 5 + [c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(residual), *args, residual.numel() // h, h, dtype_code(adt), dtype_code(wdt), stream_handle()),
          "scaled_add")
    return residual


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu": 2, "relu2": 3}


def gated_act(x: torch.Tensor, out: torch.Tensor, activation: str = "silu", pairs: bool = False) -> torch.Tensor:
    """out[t, i] = act(gate_i) * up_i; the layouts of ``silu_mul``; ``activation`` a key of ``GATE_ACTIVATIONS``."""
    if activation == "silu":
        return silu_mul(x, out, pairs)
    require_cuda(x, out)
    _rows_contiguous(x, "gated_act")
    T, two_i = x.shape
    inter = two_i // 2
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation {activation!r}")
    if two_i % 2 or out.shape != (T, inter) or not out.is_contiguous() or out.dtype != x.dtype:
        raise KernelError("gated_act: x [T, 2I], out [T, I] contiguous, same dtype")
    lib, f = _fn("elementwise", "dinfer_gated_act", [c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), ptr(out), T, inter, x.stride(0), dtype_code(x.dtype), int(bool(pairs)),
                 GATE_ACTIVATIONS[activation], stream_handle()), "gated_act")
    return out


def gated_act_scaled(x: torch.Tensor, out: torch.Tensor, scale: torch.Tensor, index: Optional[torch.Tensor] = None,
                     activation: str = "silu", pairs: bool = False) -> torch.Tensor:
    """``out[t, i] = act(s_t gate_i) * (s_t up_i)`` with ``s_t = scale[index[t]]`` (``scale[t]`` without an index; a row
    whose index is outside ``scale`` gives zeros); layouts and activations of ``gated_act``."""
    require_cuda(x, out, scale, index)
    _rows_contiguous(x, "gated_act_scaled")
    T, two_i = x.shape
    inter = two_i // 2
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"gated_act_scaled: unknown activation {activation!r}")
    if two_i % 2 or out.shape != (T, inter) or not out.is_contiguous() or out.dtype != x.dtype:
        raise KernelError("gated_act_scaled: x [T, 2I], out [T, I] contiguous, same dtype")
    if scale.dtype != torch.float32 or not scale.is_contiguous() or (index is None and scale.numel() < T) \
            or (index is not None and (index.dtype != torch.int32 or index.numel() != T or not index.is_contiguous())):
        raise KernelError("gated_act_scaled: scale f32 contiguous, index int32 [T]")
    lib, f = _fn("elementwise", "dinfer_gated_act_scaled",
                 [c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    check(lib, f(ptr(x), ptr(out), T, inter, x.stride(0), dtype_code(x.dtype), int(bool(pairs)),
                 GATE_ACTIVATIONS[activation], ptr(scale), ptr(index), scale.numel(), stream_handle()), "gated_act_scaled")
    return out


def gemm_f32_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[:, b, :] = a[:, b, :] @ w[b]^T for every b: a [M, B, K], w [B, N, K], out [M, B, N] (any views whose last
    axis is contiguous, e.g. the heads of a row); 32-bit multiply-adds on the CUDA cores, operands f32 or bf16."""
    require_cuda(a, w, out)
    if a.dim() != 3 or w.dim() != 3 or out.dim() != 3:
        raise KernelError("gemm_f32_batched: a [M, B, K], w [B, N, K], out [M, B, N]")
    M, B, K = a.shape
    N = w.shape[1]
    if w.shape[0] != B or w.shape[2] != K or tuple(out.shape) != (M, B, N):
        raise KernelError(f"gemm_f32_batched: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    for t in (a, w, out):
        _rows_contiguous(t, "gemm_f32_batched")
    lib, f = _fn("gemm_f32", "dinfer_gemm_f32_batched",
                 [c_void_p, c_int64, c_int64, c_int, c_void_p, c_int64, c_int64, c_int, c_void_p, c_int64, c_int64, c_int,
                  c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(a), a.stride(0), a.stride(1), dtype_code(a.dtype), ptr(w), w.stride(1), w.stride(0),
                 dtype_code(w.dtype), ptr(out), out.stride(0), out.stride(1), dtype_code(out.dtype), M, N, K, B,
                 stream_handle()), "gemm_f32_batched")
    return out


def attention_diff(q: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor], cache: torch.Tensor,
                   block_table: torch.Tensor, cu_seqlens: torch.Tensor, positions: torch.Tensor, num_heads: int,
                   num_kv_heads: int, head_dim: int, v_dim: int, scale: float, window: int, keep_first: int,
                   lam: float, eps: float, out_scale: float) -> torch.Tensor:
    """Differential attention over the paged cache, plain arithmetic, any sizes: per head two softmax maps (queries and
    keys ``[map 1 | map 2]``, ``head_dim`` each) over the same values, ``o = a1 - lam * a2``, then ``o / rms(o) *
    out_scale * sigmoid(gate[t, h])``.  A query at p sees j <= p with p - j < window or j < keep_first.  ``q`` [T, H * 2 D]
    and ``gate`` [T, H] may be strided views of one projection's rows; cache rows are ``max(2 D, v_dim)`` wide."""
    require_cuda(q, out, gate, cache, block_table, cu_seqlens, positions)
    _rows_contiguous(q, "attention_diff q")
    _rows_contiguous(out, "attention_diff out")
    T = q.shape[0]
    B = cu_seqlens.numel() - 1
    row = max(2 * head_dim, v_dim)
    if q.dtype != cache.dtype or out.dtype != q.dtype or (gate is not None and (gate.dtype != q.dtype or gate.stride(1) != 1
                                                                                or tuple(gate.shape) != (T, num_heads))):
        raise KernelError("attention_diff: q, out, gate [T, H] and cache must have one dtype")
    if q.shape[1] != num_heads * 2 * head_dim or tuple(out.shape) != (T, num_heads * v_dim):
        raise KernelError("attention_diff: q [T, H * 2 D], out [T, H * Dv]")
    for t, n in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (positions, "positions")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"attention_diff: {n} must be contiguous int32")
    if block_table.dim() != 2 or block_table.shape[0] < B or positions.numel() != T:
        raise KernelError("attention_diff: block_table [B, max_blocks], positions [T]")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != row \
            or not cache.is_contiguous():
        raise KernelError(f"attention_diff: cache shape {tuple(cache.shape)} is not [blocks, 2, Hkv, block, {row}]")
    lib, f = _fn("attention_diff", "dinfer_attention_diff",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_float, c_float, c_float,
                  c_int, c_void_p])
    check(lib, f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(gate), gate.stride(0) if gate is not None else 0,
                 ptr(cache), ptr(block_table), block_table.shape[1], ptr(cu_seqlens), ptr(positions), T, B, num_heads,
                 num_kv_heads, head_dim, v_dim, row, cache.shape[3], float(scale), int(window or 0), int(keep_first or 0),
                 float(lam), float(eps), float(out_scale), dtype_code(q.dtype), stream_handle()), "attention_diff")
    return out
