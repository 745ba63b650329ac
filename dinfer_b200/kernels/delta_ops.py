"""Wrappers of the gated delta rule's kernels (``csrc/delta_rule.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional, Tuple

import torch

from .lib import KernelError, check, dtype_code, ptr, require_cuda, stream_handle
from .ops import _fn, _rows_contiguous


def _ints(*tensors) -> None:
    for t in tensors:
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("delta rule: cu_seqlens, state slots and fresh flags must be contiguous int32")


def prep(P: torch.Tensor, cols: Tuple[int, int, int, int], A: torch.Tensor, conv_w: torch.Tensor, A_log: torch.Tensor,
         dt_bias: torch.Tensor, state: torch.Tensor, hist_offset: int, cu_seqlens: torch.Tensor, slots: torch.Tensor,
         fresh: torch.Tensor, H: int, G: int, dk: int, dv: int, taps: int, per_channel: bool):
    """From the stacked projections ``P`` [T, *] (q, k, v, b at the columns ``cols``) and the decay's input ``A``
    [T, H] or [T, H * dk]: the short convolutions with silu (what lies before the step comes from the requests'
    state, whose convolution history is brought up to date afterwards), unit q and k, beta, decay.  ``state``
    [slots, S + (taps - 1) * C] f32: the matrix S of every head, then the convolution history from ``hist_offset``.
    Returns f32 (q [T, G, dk], k [T, G, dk], v [T, H, dv], beta [T, H], decay [T, H] or [T, H, dk]); the decay comes as
    ``g - 1`` (``expm1`` of its exponent), which keeps the digits of a g just below one."""
    require_cuda(P, A, conv_w, A_log, dt_bias, state, cu_seqlens, slots, fresh)
    _rows_contiguous(P, "delta prep P")
    _rows_contiguous(A, "delta prep A")
    _ints(cu_seqlens, slots, fresh)
    T = P.shape[0]
    B = cu_seqlens.numel() - 1
    C = 2 * G * dk + H * dv
    nd = H * dk if per_channel else H
    if A.dtype != P.dtype or A.shape[0] != T or A.shape[1] < nd:
        raise KernelError("delta prep: A [T, H (* dk)] of P's dtype")
    for t, n, what in ((conv_w, C * taps, "conv_w [C, taps]"), (A_log, H, "A_log [H]"), (dt_bias, nd, "dt_bias")):
        if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
            raise KernelError(f"delta prep: {what} must be contiguous float32")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 \
            or state.shape[1] < hist_offset + (taps - 1) * C:
        raise KernelError("delta prep: state f32 [slots, S + (taps - 1) * C]")
    dev = P.device
    q = torch.empty((T, G, dk), dtype=torch.float32, device=dev)
    k = torch.empty((T, G, dk), dtype=torch.float32, device=dev)
    v = torch.empty((T, H, dv), dtype=torch.float32, device=dev)
    beta = torch.empty((T, H), dtype=torch.float32, device=dev)
    decay = torch.empty((T, nd), dtype=torch.float32, device=dev)
    lib, f = _fn("delta_rule", "dinfer_delta_prep",
                 [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    hist = state.data_ptr() + 4 * hist_offset
    check(lib, f(ptr(P), P.stride(0), *[int(c) for c in cols], ptr(A), A.stride(0), ptr(conv_w), ptr(A_log),
                 ptr(dt_bias), c_void_p(hist), state.stride(0), ptr(cu_seqlens), ptr(slots), ptr(fresh), B, ptr(q),
                 ptr(k), ptr(v), ptr(beta), ptr(decay), T, H, G, dk, dv, taps, int(bool(per_channel)),
                 dtype_code(P.dtype), stream_handle()), "delta_prep")
    return q, k, v, beta, decay


def recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor,
               state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, fresh: torch.Tensor,
               per_channel: bool, widen: int = 0) -> torch.Tensor:
    """Token by token per request and head: ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` (``decay``
    holds ``g - 1``, as ``prep`` makes it), S [dk, dv]
    of head h at ``state[slot, h * dk * dv:]`` (zero for a fresh request), carried in place.  Returns o f32 [T, H, dv].
    ``widen`` (1, 2, 4; 0: the sizes decide): how far a column's rows are spread over more lanes than 16 rows a lane
    would need, which only changes the order of the sums."""
    require_cuda(q, k, v, beta, decay, state, cu_seqlens, slots, fresh)
    _ints(cu_seqlens, slots, fresh)
    T, G, dk = q.shape
    _, H, dv = v.shape
    for t in (q, k, v, beta, decay):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise KernelError("delta recurrence: contiguous float32 inputs")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < H * dk * dv:
        raise KernelError("delta recurrence: state f32 [slots, >= H * dk * dv]")
    out = torch.empty((T, H, dv), dtype=torch.float32, device=q.device)
    if T == 0:
        return out
    lib, f = _fn("delta_rule", "dinfer_delta_recurrence",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    B = cu_seqlens.numel() - 1
    # a step with portions of several tokens (more rows than requests) spreads its CTAs evenly: see the kernel's launch
    check(lib, f(ptr(q), ptr(k), ptr(v), ptr(beta), ptr(decay), ptr(state), state.stride(0), ptr(cu_seqlens),
                 ptr(slots), ptr(fresh), ptr(out), B, H, G, dk, dv, int(bool(per_channel)),
                 int(widen), int(T > B), stream_handle()), "delta_recurrence")
    return out


def post(o: torch.Tensor, weight: torch.Tensor, gate: Optional[torch.Tensor], eps: float, sigmoid_gate: bool,
         out: torch.Tensor) -> torch.Tensor:
    """``out[t, h] = o[t, h] / rms(o[t, h]) * weight * act(gate[t, h])`` with act = sigmoid or silu; o f32 [T, H, dv],
    gate [T, H * dv] (its own dtype; None: no gate) and out [T, H * dv] of the activations' dtype (views with a row
    stride are fine).  ``weight`` f32 [dv] (one row for all heads) or [H * dv] (every head its own)."""
    require_cuda(o, weight, gate, out)
    T, H, dv = o.shape
    if gate is not None:
        _rows_contiguous(gate, "delta post gate")
    _rows_contiguous(out, "delta post out")
    if o.dtype != torch.float32 or not o.is_contiguous() or weight.dtype != torch.float32 \
            or weight.numel() not in (dv, H * dv) or not weight.is_contiguous() \
            or (gate is not None and (gate.shape[0] != T or gate.shape[1] < H * dv)) or tuple(out.shape) != (T, H * dv):
        raise KernelError("delta post: o f32 [T, H, dv], weight f32 [dv] or [H * dv], gate / out [T, H * dv]")
    per_head = weight.numel() == H * dv and H > 1
    lib, f = _fn("delta_rule", "dinfer_delta_post_ex",
                 [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_float, c_int, c_int,
                  c_int, c_int, c_void_p])
    check(lib, f(ptr(o), ptr(weight), ptr(gate), gate.stride(0) if gate is not None else 0, ptr(out), out.stride(0), T, H,
                 dv, float(eps), int(bool(sigmoid_gate)), int(per_head),
                 dtype_code(gate.dtype if gate is not None else torch.float32), dtype_code(out.dtype), stream_handle()),
          "delta_post")
    return out
