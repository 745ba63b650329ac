"""Wrappers of the kernels around a layer's sublayers: the join of a sublayer with norms on both sides
(``csrc/sandwich.cu``), the short convolution on a mixer's input (``csrc/short_conv.cu``) and retention
(``csrc/retention.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .lib import KernelError, check, dtype_code, ptr, require_cuda, stream_handle
from .ops import _fn, _rows_contiguous


def gain_norm_join(a: torch.Tensor, gain, eps: float, x_in: torch.Tensor, x_out: torch.Tensor,
                   average=None, next_gain=None, next_out: Optional[torch.Tensor] = None) -> None:
    """``x_out = x_in + a / rms(a) * gain`` (32-bit rows [T, h]; ``x_out`` may be ``x_in``).  ``gain`` and ``next_gain``
    are each one number or a float32 vector [h] of per-coordinate weights.  ``average`` =
    (first [T, h], results [count, T, h], n, weights [n + 1], out [T, h]): ``out = weights[0] * first + sum_(j=1..n-1)
    weights[j] * results[j - 1] + weights[n] * x_out``.  ``next_out`` (the activations' dtype): the RMS norm with
    ``next_gain`` of the average, or of ``x_out`` without one."""
    require_cuda(a, x_in, x_out, next_out)
    _rows_contiguous(a, "gain_norm_join")
    T, h = x_in.shape

    def split(g):                                          # (the number, the vector) of a norm's weight
        if isinstance(g, torch.Tensor):
            require_cuda(g)
            if g.dtype != torch.float32 or g.numel() != h or not g.is_contiguous():
                raise KernelError("gain_norm_join: a norm's weight vector is contiguous float32 [h]")
            return 1.0, g
        return float(g or 0.0), None
    g_a, w_a = split(gain)
    g_n, w_n = split(next_gain)
    for t in (x_in, x_out):
        if t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != (T, h):
            raise KernelError("gain_norm_join: the stream is contiguous float32 [T, h]")
    if tuple(a.shape) != (T, h):
        raise KernelError("gain_norm_join: the branch is [T, h]")
    first = results = weights = out = None
    n, stride = 0, 0
    if average is not None:
        first, results, n, weights, out = average
        require_cuda(first, results, weights, out)
        if first.dtype != torch.float32 or not first.is_contiguous() or tuple(first.shape) != (T, h) \
                or out.dtype != torch.float32 or not out.is_contiguous() or tuple(out.shape) != (T, h) \
                or weights.numel() != n + 1 or not weights.is_contiguous() or n < 1:
            raise KernelError("gain_norm_join: average = (first f32 [T, h], results, n, weights [n + 1], out f32 [T, h])")
        if n > 1:
            if results.dtype != torch.float32 or results.dim() != 3 or results.shape[0] < n - 1 or results.stride(2) != 1 \
                    or results.stride(1) != h or tuple(results.shape[1:]) != (T, h):
                raise KernelError("gain_norm_join: results float32 [count >= n - 1, T, h] with contiguous [T, h]")
            stride = results.stride(0)
    if next_out is not None and (tuple(next_out.shape) != (T, h) or not next_out.is_contiguous() or next_gain is None):
        raise KernelError("gain_norm_join: next_out contiguous [T, h] with its gain")
    lib, f = _fn("sandwich", "dinfer_weight_norm_join",
                 [c_void_p, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int64, c_int,
                  c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(a), a.stride(0), g_a, ptr(w_a), ptr(x_in), ptr(x_out), float(eps), ptr(first), ptr(results), stride,
                 int(n), ptr(weights), ptr(out), g_n, ptr(w_n), ptr(next_out), T, h, dtype_code(a.dtype),
                 dtype_code(next_out.dtype if next_out is not None else torch.float32),
                 dtype_code(weights.dtype if weights is not None else torch.float32), stream_handle()), "gain_norm_join")


def _ints(*tensors) -> None:
    for t in tensors:
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("request offsets, slots and fresh flags are contiguous int32")


def short_conv_input(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor,
                     slots: torch.Tensor, fresh: torch.Tensor, out: torch.Tensor, update: bool = True) -> torch.Tensor:
    """``out[t] = x[t] + sum_j weight[:, j] * x[t - taps + 1 + j]`` within each request, inputs before the portion
    from the request's history: the first ``(taps - 1) * C`` elements of row ``slots[b]`` of ``state`` (f32 rows, any
    row stride), zeros for a fresh request.  With ``update`` the history then moves on by the portion."""
    require_cuda(x, weight, state, cu_seqlens, slots, fresh, out)
    _rows_contiguous(x, "short_conv_input")
    _rows_contiguous(out, "short_conv_input")
    _ints(cu_seqlens, slots, fresh)
    T, C = x.shape
    taps = weight.shape[1]
    if tuple(out.shape) != (T, C) or out.dtype != x.dtype or tuple(weight.shape) != (C, taps) or not weight.is_contiguous():
        raise KernelError("short_conv_input: x, out [T, C] of one dtype, weight [C, taps] contiguous")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < (taps - 1) * C:
        raise KernelError("short_conv_input: state f32 [slots, >= (taps - 1) * C]")
    B = cu_seqlens.numel() - 1
    lib, f = _fn("short_conv", "dinfer_short_conv_input",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), x.stride(0), ptr(out), out.stride(0), ptr(weight), ptr(state), state.stride(0), ptr(cu_seqlens),
                 ptr(slots), ptr(fresh), T, B, C, taps, int(bool(update)), dtype_code(x.dtype), dtype_code(weight.dtype),
                 stream_handle()), "short_conv_input")
    if update and taps > 1 and T > 0:
        from .lib import add_launches
        add_launches(1)                                   # the history kernel
    return out


# Steps whose longest portion has more tokens than this take their chunks side by side (three launches) instead of
# one after the other inside a CTA.
RETENTION_CHAIN_TOKENS = 128


RETENTION_POWERS = 65          # entries of a head's row of the table of powers (POWERS in the kernels)


def retention_powers(decay: torch.Tensor) -> torch.Tensor:
    """f32 [H, 65]: row h holds ``decay[h] ** 0 .. decay[h] ** 64``, made in 64-bit and rounded once."""
    d = decay.detach().to(torch.float64).reshape(-1, 1)
    return torch.pow(d, torch.arange(RETENTION_POWERS, dtype=torch.float64, device=decay.device)).to(torch.float32).contiguous()


def retention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
              cu_seqlens: torch.Tensor, slots: torch.Tensor, fresh: torch.Tensor, num_heads: int, key_dim: int,
              value_dim: int, k_scale: float, max_q_len: int = 0, side_by_side: Optional[bool] = None,
              powers: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``S_t = decay_h S_(t-1) + (k_scale k_t) v_t^T; o_t = S_t^T q_t`` per request and head, S [dk, dv] in the first
    ``H * dk * dv`` elements of row ``slots[b]`` of ``state`` (f32 rows, any row stride; zero for a fresh request).
    q, k [T, H * dk], v [T, H * dv]: float32 rows (views with a row stride are fine).  Returns o f32 [T, H, dv].
    ``max_q_len``: the longest portion of the step (0: not known); long portions run their chunks side by side, which
    ``side_by_side`` forces or forbids.  ``powers``: ``retention_powers(decay)``, for a caller that keeps it."""
    require_cuda(q, k, v, decay, state, cu_seqlens, slots, fresh)
    _ints(cu_seqlens, slots, fresh)
    T = q.shape[0]
    H, dk, dv = num_heads, key_dim, value_dim
    for t, n in ((q, H * dk), (k, H * dk), (v, H * dv)):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or t.shape[1] != n or t.shape[0] != T:
            raise KernelError("retention: q, k [T, H * dk], v [T, H * dv] float32 rows")
    if decay.dtype != torch.float32 or decay.numel() != H or not decay.is_contiguous():
        raise KernelError("retention: decay float32 [H]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < H * dk * dv:
        raise KernelError("retention: state f32 [slots, >= H * dk * dv]")
    out = torch.empty((T, H, dv), dtype=torch.float32, device=q.device)
    if T == 0:
        return out
    if powers is None:
        powers = retention_powers(decay)
    if powers.dtype != torch.float32 or tuple(powers.shape) != (H, RETENTION_POWERS) or not powers.is_contiguous():
        raise KernelError("retention: powers float32 [H, 65]")
    require_cuda(powers)
    B = cu_seqlens.numel() - 1
    single = max_q_len == 1 and T == B
    if side_by_side is None:
        # the chain keeps a chunk's q and k and a slice of S in shared memory: keys too wide for that go side by side
        chain_smem = 4 * (2 * 32 * (dk + 1) + dk * 32 + 2 * 32 * 32 + 32 * 33 + 33)
        side_by_side = max_q_len > RETENTION_CHAIN_TOKENS or (not single and chain_smem > 200 * 1024)
    if side_by_side:
        longest = int(max_q_len) if max_q_len > 0 else T
        lib, f = _fn("retention", "dinfer_retention_chunks",
                     [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p,
                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
        chunk = 64                                        # tokens of a chunk in the kernels (CP)
        work = torch.empty((T // chunk + B) * H * dk * dv, dtype=torch.float32, device=q.device)
        check(lib, f(ptr(q), ptr(k), ptr(v), q.stride(0), k.stride(0), v.stride(0), ptr(powers), ptr(state), state.stride(0),
                     ptr(cu_seqlens), ptr(slots), ptr(fresh), ptr(out), ptr(work), B, H, dk, dv, float(k_scale), longest,
                     stream_handle()), "retention_chunks")
        from .lib import add_launches
        add_launches(2)                                   # three launches in all
        return out
    lib, f = _fn("retention", "dinfer_retention",
                 [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    check(lib, f(ptr(q), ptr(k), ptr(v), q.stride(0), k.stride(0), v.stride(0), ptr(powers), ptr(state), state.stride(0),
                 ptr(cu_seqlens), ptr(slots), ptr(fresh), ptr(out), B, H, dk, dv, float(k_scale),
                 int(single), stream_handle()), "retention")
    return out
