"""Wrappers of the latent-attention kernels (``csrc/latent_post.cu``, ``csrc/attention_latent.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .lib import KernelError, check, dtype_code, ptr, require_cuda, stream_handle
from .ops import _fn, _rows_contiguous


def latent_down_post(x: torch.Tensor, positions: torch.Tensor, q_weight: torch.Tensor, q_rank: int,
                     kv_weight: Optional[torch.Tensor], kv_rank: int, rope_dim: int, eps: float,
                     cos_sin: Optional[torch.Tensor], cache: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                     halves: bool = False) -> None:
    """Rows ``x`` [T, q_rank (+ kv_rank + rope_dim)] of the stacked down projections: the q latent is RMS-normed in
    place; with a kv part, the normed kv latent and the rotated shared key part (pairs (2i, 2i + 1), angles from the
    ``cos_sin`` table row of the token's position) go into the token's row ``slots[t]`` of the latent ``cache``
    [pages, page, kv_rank + rope_dim]."""
    require_cuda(x, positions, q_weight, kv_weight, cos_sin, cache, slots)
    _rows_contiguous(x, "latent_down_post")
    T = x.shape[0]
    has_kv = kv_weight is not None
    R = kv_rank if has_kv else 0
    P = rope_dim if has_kv else 0
    if x.shape[1] != q_rank + R + P or positions.dtype != torch.int32 or positions.numel() != T:
        raise KernelError("latent_down_post: x [T, q_rank (+ kv_rank + rope_dim)], positions int32 [T]")
    if q_weight.numel() != q_rank or (has_kv and (kv_weight.numel() != R or kv_weight.dtype != q_weight.dtype)):
        raise KernelError("latent_down_post: norm weights [q_rank], [kv_rank] of one dtype")
    rot = 0
    if has_kv:
        if cache is None or slots is None or cache.dtype != x.dtype or not cache.is_contiguous() \
                or cache.shape[-1] != R + P or slots.dtype != torch.int32 or slots.numel() != T:
            raise KernelError("latent_down_post: cache [..., kv_rank + rope_dim] of the activations' dtype, slots int32 [T]")
        if cos_sin is not None:
            if cos_sin.dtype != torch.float32 or cos_sin.dim() != 2 or not cos_sin.is_contiguous():
                raise KernelError("latent_down_post: angle table must be contiguous float32 [max_pos, rot]")
            rot = cos_sin.shape[1]
    lib, f = _fn("latent_post", "dinfer_latent_down_post",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                  c_int, c_int, c_float, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), x.stride(0), ptr(positions), ptr(q_weight), ptr(kv_weight), ptr(cos_sin) if has_kv else None,
                 rot, ptr(cache) if has_kv else None, ptr(slots) if has_kv else None, T, q_rank, R, P, float(eps),
                 int(bool(halves)), dtype_code(x.dtype), dtype_code(q_weight.dtype), stream_handle()), "latent_down_post")


def latent_q_rope(q: torch.Tensor, positions: torch.Tensor, cos_sin: Optional[torch.Tensor], q_lat: torch.Tensor,
                  num_heads: int, nope_dim: int, rope_dim: int, kv_rank: int, halves: bool = False) -> None:
    """The last ``rope_dim`` elements of every head of ``q`` [T, H * (nope_dim + rope_dim)], rotated by the token's
    position, into ``q_lat[t, h, kv_rank:]`` (q_lat [T, H, kv_rank + rope_dim], any token and head strides)."""
    require_cuda(q, positions, cos_sin, q_lat)
    _rows_contiguous(q, "latent_q_rope")
    T = q.shape[0]
    if q.shape[1] != num_heads * (nope_dim + rope_dim) or tuple(q_lat.shape) != (T, num_heads, kv_rank + rope_dim) \
            or q_lat.stride(2) != 1 or q_lat.dtype != q.dtype or positions.dtype != torch.int32:
        raise KernelError("latent_q_rope: q [T, H (D + P)], q_lat [T, H, R + P] (last axis contiguous) of one dtype")
    rot = 0
    if cos_sin is not None:
        if cos_sin.dtype != torch.float32 or cos_sin.dim() != 2 or not cos_sin.is_contiguous():
            raise KernelError("latent_q_rope: angle table must be contiguous float32 [max_pos, rot]")
        rot = cos_sin.shape[1]
    lib, f = _fn("latent_post", "dinfer_latent_q_rope",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int,
                  c_int, c_int, c_void_p])
    check(lib, f(ptr(q), q.stride(0), ptr(positions), ptr(cos_sin), rot, ptr(q_lat), q_lat.stride(0), q_lat.stride(1), T,
                 num_heads, nope_dim, rope_dim,
                 kv_rank, int(bool(halves)), dtype_code(q.dtype), stream_handle()), "latent_q_rope")


def _check_attention(q_lat, out, cache, block_table, cu_seqlens, kv_rank, rope_dim):
    require_cuda(q_lat, out, cache, block_table, cu_seqlens)
    if q_lat.dim() != 3 or out.dim() != 3 or q_lat.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError("attention_latent: q_lat [T, H, R + P], out [T, H, R], last axis contiguous")
    T, H, W = q_lat.shape
    if W != kv_rank + rope_dim or tuple(out.shape) != (T, H, kv_rank) or out.dtype != q_lat.dtype or cache.dtype != q_lat.dtype:
        raise KernelError("attention_latent: shapes or dtypes of q_lat, out and cache do not agree")
    if not cache.is_contiguous() or cache.shape[-1] != W or cache.dim() < 3:
        raise KernelError(f"attention_latent: cache {tuple(cache.shape)} is not [pages, ..., page, {W}] contiguous")
    for t, n in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"attention_latent: {n} must be contiguous int32")
    if block_table.dim() != 2 or block_table.shape[0] < cu_seqlens.numel() - 1:
        raise KernelError("attention_latent: block_table [B, max_blocks]")
    return T, H


def _check_sinks(sinks, H):
    if sinks is not None:
        require_cuda(sinks)
        if sinks.dtype != torch.float32 or sinks.numel() != H or not sinks.is_contiguous():
            raise KernelError("attention_latent: sinks float32 [H] contiguous")


def attention_latent_generic(q_lat: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                             cu_seqlens: torch.Tensor, positions: torch.Tensor, kv_rank: int, rope_dim: int,
                             scale: float, window: int = 0, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal multi-query attention in the absorbed form over the paged latent cache, plain arithmetic, any sizes:
    ``out[t, h] = sum_j softmax_j((q_lat[t, h] . row_j) * scale) row_j[:kv_rank]``.  ``sinks`` f32 [H]: head h's
    softmax has one more term ``exp(sinks[h])`` that carries no value."""
    T, H = _check_attention(q_lat, out, cache, block_table, cu_seqlens, kv_rank, rope_dim)
    require_cuda(positions)
    _check_sinks(sinks, H)
    if positions.dtype != torch.int32 or positions.numel() != T:
        raise KernelError("attention_latent: positions int32 [T]")
    lib, f = _fn("attention_latent", "dinfer_attention_latent_generic",
                 [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_void_p])
    check(lib, f(ptr(q_lat), q_lat.stride(0), q_lat.stride(1), ptr(out), out.stride(0), out.stride(1), ptr(cache),
                 ptr(block_table), block_table.shape[1], ptr(cu_seqlens), ptr(positions), T, cu_seqlens.numel() - 1, H,
                 kv_rank, rope_dim, cache.shape[-2], float(scale), int(window), ptr(sinks), dtype_code(q_lat.dtype),
                 stream_handle()),
          "attention_latent_generic")
    return out


def tc_supported(dtype: torch.dtype, kv_rank: int, rope_dim: int, block_size: int = 16) -> bool:
    """Sizes the tensor-core kernel takes: bfloat16, latent and rotated part in multiples of 16, a latent of at most 512."""
    return dtype == torch.bfloat16 and kv_rank % 16 == 0 and rope_dim % 16 == 0 and 0 < kv_rank <= 512 and block_size > 0


def tc_row_tile(kv_rank: int, max_rows_per_req: int) -> int:
    """Rows ((token, head) pairs) a CTA of the tensor-core kernel owns."""
    from .lib import library
    return int(library("attention_latent").dinfer_attention_latent_tc_rows(int(kv_rank), int(max_rows_per_req)))


def tc_splits(row_tiles: int, max_seq_len: int) -> int:
    """CTAs that share the keys of a row tile: enough to give every SM two CTAs' worth of tiles, each CTA at least
    two key tiles long (a step with more row tiles than that shares nothing)."""
    from .lib import num_sms
    key_tiles = (max_seq_len + 63) // 64
    want = (2 * num_sms() + row_tiles - 1) // max(1, row_tiles)
    return max(1, min(want, key_tiles // 2, 64))


def attention_latent_tc(q_lat: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                        cu_seqlens: torch.Tensor, seq_lens: torch.Tensor, kv_rank: int, rope_dim: int, scale: float,
                        window: int = 0, max_q_len: int = 1, max_seq_len: int = 1, splits: Optional[int] = None,
                        sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same attention on tensor cores (bfloat16): prompt portions and decoded tokens in one launch.  ``seq_lens`` [B]:
    tokens of each request after the step (a token's position follows from it); ``max_q_len``: the longest portion of
    the batch (chooses the row tile); ``max_seq_len``: the longest request (chooses how many CTAs share a row tile's keys
    unless ``splits`` says)."""
    T, H = _check_attention(q_lat, out, cache, block_table, cu_seqlens, kv_rank, rope_dim)
    require_cuda(seq_lens)
    _check_sinks(sinks, H)
    B = cu_seqlens.numel() - 1
    if seq_lens.dtype != torch.int32 or seq_lens.numel() < B or not seq_lens.is_contiguous():
        raise KernelError("attention_latent_tc: seq_lens int32 [B]")
    if not tc_supported(q_lat.dtype, kv_rank, rope_dim, cache.shape[-2]):
        raise KernelError("attention_latent_tc: bfloat16 with kv_rank and rope_dim in multiples of 16 only")
    rows_per_req = max(1, int(max_q_len)) * H
    bm = tc_row_tile(kv_rank, rows_per_req)
    row_tiles = (T * H + bm - 1) // bm + B
    if splits is None:
        splits = tc_splits(row_tiles, max_seq_len)
    part = ml = None
    if splits > 1:
        part = torch.empty((T * H * splits * kv_rank,), dtype=torch.float32, device=q_lat.device)
        ml = torch.empty((T * H * splits * 2,), dtype=torch.float32, device=q_lat.device)
    lib, f = _fn("attention_latent", "dinfer_attention_latent_tc",
                 [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                  c_void_p])
    check(lib, f(ptr(q_lat), q_lat.stride(0), q_lat.stride(1), ptr(out), out.stride(0), out.stride(1), ptr(cache),
                 ptr(block_table), block_table.shape[1], ptr(cu_seqlens), ptr(seq_lens), T, B, H, kv_rank, rope_dim,
                 cache.shape[-2], float(scale), int(window), rows_per_req, row_tiles, int(splits), ptr(part), ptr(ml),
                 ptr(sinks), stream_handle()), "attention_latent_tc")
    if splits > 1:
        from .lib import add_launches
        add_launches(1)                                   # the fold kernel
    return out
