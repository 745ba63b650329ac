"""Wrappers of the kernels for linear-attention mixers with a decay per key channel (``csrc/linear_state.cu``): the
general delta rule and the gate-write form share one recurrence."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional, Tuple

import torch

from .lib import KernelError, check, ptr, require_cuda, stream_handle
from .ops import _fn


def _rows(t: torch.Tensor, n: int, T: int, what: str) -> None:
    if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != T or t.shape[1] != n:
        raise KernelError(f"{what}: float32 rows [T, {n}] (a view with a row stride is fine)")


def _vec(t: torch.Tensor, n: int, what: str) -> None:
    if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
        raise KernelError(f"{what}: contiguous float32 [{n}]")


def _ints(*tensors) -> None:
    for t in tensors:
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("linear state: cu_seqlens, state slots and fresh flags must be contiguous int32")


def tanh_rows(x: torch.Tensor) -> torch.Tensor:
    """``x <- tanh(x)`` in place on float32 rows (a view of some columns of wider rows is fine)."""
    require_cuda(x)
    _rows(x, x.shape[1], x.shape[0], "tanh_rows")
    lib, f = _fn("linear_state", "dinfer_tanh_rows", [c_void_p, c_int64, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), x.stride(0), x.shape[0], x.shape[1], stream_handle()), "tanh_rows")
    return x


def general_delta_prep(k: torch.Tensor, d: torch.Tensor, a: torch.Tensor, w0: torch.Tensor, a_bias: torch.Tensor,
                       decay_scale: float, num_heads: int, key_dim: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """From the keys ``k``, the decay's logits ``d`` and the removal's logits ``a`` (float32 rows [T, H * dk]):
    ``w = exp(-decay_scale * sigmoid(d + w0))``, the unit key ``u = k / sqrt(sum(k^2) + 1e-6)`` of every head, and
    ``p = sigmoid(a + a_bias) * u``.  Returns float32 (w, u, p), each [T, H * dk]."""
    require_cuda(k, d, a, w0, a_bias)
    T, n = k.shape[0], num_heads * key_dim
    for t, what in ((k, "k"), (d, "decay logits"), (a, "removal logits")):
        _rows(t, n, T, "general_delta_prep " + what)
    _vec(w0, n, "general_delta_prep w0")
    _vec(a_bias, n, "general_delta_prep a_bias")
    w, u, p = (torch.empty((T, n), dtype=torch.float32, device=k.device) for _ in range(3))
    lib, f = _fn("linear_state", "dinfer_general_delta_prep",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                  c_void_p, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(k), k.stride(0), ptr(d), d.stride(0), ptr(a), a.stride(0), ptr(w0), ptr(a_bias), float(decay_scale),
                 ptr(w), ptr(u), ptr(p), T, num_heads, key_dim, stream_handle()), "general_delta_prep")
    return w, u, p


def gate_write_prep(xq: torch.Tensor, xf: torch.Tensor, f_bias: torch.Tensor, lower: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q = silu(xq)`` and the forget gate ``f = lower + (1 - lower) * sigmoid(xf + f_bias)`` (float32 rows [T, n] in,
    contiguous float32 [T, n] out)."""
    require_cuda(xq, xf, f_bias, lower)
    T, n = xq.shape
    _rows(xq, n, T, "gate_write_prep xq")
    _rows(xf, n, T, "gate_write_prep xf")
    _vec(f_bias, n, "gate_write_prep f_bias")
    _vec(lower, n, "gate_write_prep lower")
    q, fg = (torch.empty((T, n), dtype=torch.float32, device=xq.device) for _ in range(2))
    lib, f = _fn("linear_state", "dinfer_gate_write_prep",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    check(lib, f(ptr(xq), xq.stride(0), ptr(xf), xf.stride(0), ptr(f_bias), ptr(lower), ptr(q), ptr(fg), T, n,
                 stream_handle()), "gate_write_prep")
    return q, fg


def recurrence(r: torch.Tensor, w: torch.Tensor, v: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor,
               slots: torch.Tensor, fresh: torch.Tensor, num_heads: int, key_dim: int, value_dim: int,
               k: Optional[torch.Tensor] = None, u: Optional[torch.Tensor] = None, p: Optional[torch.Tensor] = None,
               widen: int = 0) -> torch.Tensor:
    """Token by token per request and head, S [dk, dv] in the first ``H * dk * dv`` floats of row ``slots[b]`` of
    ``state`` (zero for a fresh request), carried in place.  With ``k``, ``u``, ``p``:
    ``S <- diag(w) S - p (u^T S) + k v^T`` (both the decay and the removal read the old S); without them the
    gate-write form ``S <- diag(w) S + (1 - w) v^T``.  ``o = S^T r`` of the new S.  All inputs float32 rows (views with
    a row stride are fine): r, w, k, u, p [T, H * dk], v [T, H * dv].  Returns o float32 [T, H, dv].
    ``widen`` (0: the sizes decide; 1, 2): how many lanes share a column, which only changes the order of the sums."""
    remove = k is not None
    if remove != (u is not None) or remove != (p is not None):
        raise KernelError("linear state: k, u and p come together")
    require_cuda(r, w, v, state, cu_seqlens, slots, fresh, k, u, p)
    _ints(cu_seqlens, slots, fresh)
    T = r.shape[0]
    H, dk, dv = num_heads, key_dim, value_dim
    for t, what in ((r, "r"), (w, "w"), (k, "k"), (u, "u"), (p, "p")):
        if t is not None:
            _rows(t, H * dk, T, "linear state " + what)
    _rows(v, H * dv, T, "linear state v")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < H * dk * dv:
        raise KernelError("linear state: state f32 [slots, >= H * dk * dv]")
    out = torch.empty((T, H, dv), dtype=torch.float32, device=r.device)
    if T == 0:
        return out
    st = lambda t: t.stride(0) if t is not None else 0
    lib, f = _fn("linear_state", "dinfer_linear_state",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                  c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                  c_int, c_int, c_void_p])
    B = cu_seqlens.numel() - 1
    # a step with portions of several tokens (more rows than requests) spreads its CTAs evenly: see the kernel's launch
    check(lib, f(ptr(r), st(r), ptr(k), st(k), ptr(w), st(w), ptr(u), st(u), ptr(p), st(p), ptr(v), st(v), ptr(state),
                 state.stride(0), ptr(cu_seqlens), ptr(slots), ptr(fresh), ptr(out), B, H, dk, dv,
                 int(remove), int(widen), int(T > B), stream_handle()), "linear_state")
    return out
