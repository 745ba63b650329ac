"""Wrappers of the routed feed-forward's kernels (``csrc/moe.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional, Tuple

import torch

from .lib import KernelError, check, dtype_code, ptr, require_cuda, stream_handle
from .ops import _fn, _rows_contiguous

ACTIVATIONS = {"none": 0, "relu2": 1, "silu": 2, "gelu_tanh": 3, "relu": 4}


def route(logits: torch.Tensor, num_experts: int, top_k: int, scoring: str = "softmax", renormalize: bool = False,
          has_gate: bool = False) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """From 32-bit router logits [T, E (+ 1) or more columns]: (expert ids int32 [T, top_k], weights f32 [T, top_k], gate f32 [T] or
    None).  ``scoring`` softmax (over all experts) or sigmoid; the weights are the chosen scores, divided by their sum
    with ``renormalize``; ``has_gate``: column E holds a shared expert's gate logit, gate = its sigmoid."""
    require_cuda(logits)
    _rows_contiguous(logits, "moe route")
    T = logits.shape[0]
    if scoring not in ("softmax", "sigmoid"):
        raise KernelError(f"moe route: unknown scoring {scoring!r}")
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.shape[1] < num_experts + int(has_gate):
        raise KernelError("moe route: logits f32 [T, >= E (+ 1)]")
    ids = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    gate = torch.empty((T,), dtype=torch.float32, device=logits.device) if has_gate else None
    lib, f = _fn("moe", "dinfer_moe_route",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(logits), logits.stride(0), ptr(ids), ptr(weights), ptr(gate), T, num_experts, top_k,
                 int(scoring == "sigmoid"), int(bool(renormalize)), stream_handle()), "moe_route")
    return ids, weights, gate


def route_table(tokens: torch.Tensor, table: torch.Tensor, num_experts: int,
                prev: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Routing without a router: ``table`` [vocab, top] int32 names each token id's experts, every choice weighs
    ``1 / top``.  ``tokens`` int32 [T]; an id -(r + 1) stands for ``prev[r]``.  Returns (ids int32 [T, top], weights f32)."""
    require_cuda(tokens, table, prev)
    if tokens.dtype != torch.int32 or table.dtype != torch.int32 or table.dim() != 2 or not table.is_contiguous() \
            or not tokens.is_contiguous():
        raise KernelError("moe route_table: tokens int32 [T], table int32 [vocab, top], contiguous")
    T, top = tokens.numel(), table.shape[1]
    ids = torch.empty((T, top), dtype=torch.int32, device=tokens.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=tokens.device)
    lib, f = _fn("moe", "dinfer_moe_route_table",
                 [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(tokens), ptr(prev), prev.numel() if prev is not None else 0, ptr(table), table.shape[0], ptr(ids),
                 ptr(weights), T, num_experts, top, stream_handle()), "moe_route_table")
    return ids, weights


def router(h: torch.Tensor, w_router: torch.Tensor, top_k: int, scoring: str = "softmax", renormalize: bool = False,
           w_gate: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """The router from its input: logits by the 32-bit product (``w_router`` [E, K], and ``w_gate`` [K] as one more
    row), then ``route``."""
    from .ops import gemm_f32
    w = w_router if w_gate is None else torch.cat([w_router, w_gate.reshape(1, -1).to(w_router.dtype)])
    z = torch.empty((h.shape[0], w.shape[0]), dtype=torch.float32, device=h.device)
    gemm_f32(h, w.contiguous(), z)
    return route(z, w_router.shape[0], top_k, scoring, renormalize, w_gate is not None)


def row_tile(pairs: int, num_experts: int) -> int:
    """Rows of a tile of the grouped products: 16 while an expert gets few rows (decode steps), else 64."""
    return 16 if pairs <= 16 * num_experts else 64


# rows of a tile of the two-SM tcgen05 kernel, and the average rows per expert from which the grouped products of a
# step run on it (below, padding every expert's run to a whole tile costs more than the faster tensor path gains)
TC_ROW_TILE = 256
TC_MIN_ROWS_PER_EXPERT = 96


def tc_grouped_supported(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, pairs: int) -> bool:
    """Whether a step's grouped products can run on the tcgen05 kernel: bfloat16, rows TMA can address, and enough rows."""
    E, ff, h = w_up.shape
    return (x.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
            and h % 8 == 0 and ff % 8 == 0 and w_down.shape[2] % 8 == 0 and pairs >= TC_MIN_ROWS_PER_EXPERT * E
            and w_up.data_ptr() % 16 == 0 and w_down.data_ptr() % 16 == 0)


def gather_rows(x: torch.Tensor, sorted_: torch.Tensor, pairs: int, top_k: int) -> torch.Tensor:
    """The step's rows laid out expert by expert: a[pos] = x[sorted[pos] // top_k], zeros where the layout pads."""
    require_cuda(x, sorted_)
    _rows_contiguous(x, "moe gather")
    cap, h = sorted_.numel(), x.shape[1]
    a = torch.empty((cap, h), dtype=x.dtype, device=x.device)
    lib, f = _fn("moe", "dinfer_moe_gather", [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), x.stride(0), ptr(sorted_), ptr(a), cap, pairs, top_k, h, dtype_code(x.dtype), stream_handle()),
          "moe_gather")
    return a


def grouped_gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, sorted_: torch.Tensor, tile_expert: torch.Tensor,
                    pairs: int, mode: int, activation: str = "none", weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The grouped product on the two-SM tcgen05 kernel (bfloat16; the layout padded to ``TC_ROW_TILE`` rows per
    expert run).  a [cap, K] by position.  mode 0: ``out[pos] = act(a[pos] @ w[e]^T)`` (out [cap, N]); mode 1:
    ``out[pair] = (a[pos] @ w[e]^T) * weights[pair]`` (out [pairs, N])."""
    from . import gemm_ops
    require_cuda(a, w, out, sorted_, tile_expert, weights)
    E, N, K = w.shape
    cap = sorted_.numel()
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or not w.is_contiguous() \
            or tuple(a.shape) != (cap, K) or a.stride(1) != 1 or out.stride(1) != 1 or out.shape[1] != N \
            or cap % TC_ROW_TILE or tile_expert.numel() != cap // TC_ROW_TILE:
        raise KernelError("moe grouped_gemm_tc: bfloat16 a [cap, K], w [E, N, K], out [*, N]; cap in whole tiles")
    if (mode == 0 and out.shape[0] != cap) or (mode == 1 and (out.shape[0] != pairs or weights is None
                                                              or weights.dtype != torch.float32 or weights.numel() != pairs)):
        raise KernelError("moe grouped_gemm_tc: row counts or weights do not fit the mode")
    st = gemm_ops._state(a.device)
    lib, f = _fn("gemm_tc", "dinfer_gemm_tc_grouped",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                  c_int, c_int, c_int, c_void_p, c_void_p])
    check(lib, f(ptr(a), a.stride(0), ptr(w), ptr(out), out.stride(0), ptr(tile_expert), ptr(sorted_), ptr(weights), cap,
                 pairs, E, N, K, int(mode), ACTIVATIONS[activation], ptr(st["status"]), stream_handle()), "gemm_tc_grouped")
    return out


def align(ids: torch.Tensor, num_experts: int, tile: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The (token, choice) pairs laid out expert by expert, each expert's run padded to a multiple of ``tile``:
    (sorted int32 [cap]: pair index or ``pairs`` for padding; tile_expert int32 [cap / tile]: expert or -1)."""
    require_cuda(ids)
    if ids.dtype != torch.int32 or not ids.is_contiguous():
        raise KernelError("moe align: ids int32 contiguous")
    pairs = ids.numel()
    cap = (pairs + num_experts * (tile - 1) + tile - 1) // tile * tile
    sorted_ = torch.empty((cap,), dtype=torch.int32, device=ids.device)
    tile_expert = torch.empty((cap // tile,), dtype=torch.int32, device=ids.device)
    lib, f = _fn("moe", "dinfer_moe_align", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(ids), ptr(sorted_), ptr(tile_expert), pairs, num_experts, tile, cap, stream_handle()), "moe_align")
    return sorted_, tile_expert


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, sorted_: torch.Tensor, tile_expert: torch.Tensor,
                 pairs: int, top_k: int, tile: int, mode: int, activation: str = "none",
                 weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """mode 0: ``out[pos] = act(a[pair // top_k] @ w[e]^T)`` for every position of the layout (a [T, K], out [cap, N]);
    mode 1: ``out[pair] = (a[pos] @ w[e]^T) * weights[pair]`` (a [cap, K], out [pairs, N]).  w [E, N, K]."""
    require_cuda(a, w, out, sorted_, tile_expert, weights)
    _rows_contiguous(a, "moe gemm a")
    _rows_contiguous(out, "moe gemm out")
    E, N, K = w.shape
    cap = sorted_.numel()
    if not w.is_contiguous() or a.shape[1] != K or out.shape[1] != N or out.dtype != a.dtype:
        raise KernelError("moe gemm: w [E, N, K] contiguous, a [*, K], out [*, N] of a's dtype")
    if (mode == 0 and out.shape[0] != cap) or (mode == 1 and (a.shape[0] != cap or out.shape[0] != pairs)):
        raise KernelError("moe gemm: row counts do not fit the layout")
    if mode == 1 and (weights is None or weights.dtype != torch.float32 or weights.numel() != pairs):
        raise KernelError("moe gemm: mode 1 needs the routing weights, f32 [pairs]")
    lib, f = _fn("moe", "dinfer_moe_gemm",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(a), a.stride(0), ptr(w), ptr(out), out.stride(0), ptr(sorted_), ptr(tile_expert), ptr(weights),
                 pairs, top_k, N, K, tile, cap, mode, ACTIVATIONS[activation], dtype_code(a.dtype), dtype_code(w.dtype),
                 stream_handle()), "moe_gemm")
    return out


def combine(y: torch.Tensor, out: torch.Tensor, top_k: int, shared: Optional[torch.Tensor] = None,
            gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_k y[t * top_k + k] (+ gate[t] * shared[t]), summed in the order of the choices."""
    require_cuda(y, out, shared, gate)
    T, h = out.shape
    if tuple(y.shape) != (T * top_k, h) or not y.is_contiguous() or not out.is_contiguous() or y.dtype != out.dtype:
        raise KernelError("moe combine: y [T * top_k, h], out [T, h] contiguous of one dtype")
    if shared is not None and (tuple(shared.shape) != (T, h) or not shared.is_contiguous() or shared.dtype != out.dtype):
        raise KernelError("moe combine: shared [T, h] contiguous")
    if gate is not None and (gate.dtype != torch.float32 or gate.numel() != T):
        raise KernelError("moe combine: gate f32 [T]")
    lib, f = _fn("moe", "dinfer_moe_combine", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(y), ptr(shared), ptr(gate), ptr(out), T, top_k, h, dtype_code(out.dtype), stream_handle()),
          "moe_combine")
    return out


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """out = act(x) element by element (``out`` may be ``x``)."""
    require_cuda(x, out)
    if not x.is_contiguous() or not out.is_contiguous() or x.shape != out.shape or x.dtype != out.dtype:
        raise KernelError("activation: contiguous tensors of one shape and dtype")
    lib, f = _fn("moe", "dinfer_activation", [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), ptr(out), x.numel(), ACTIVATIONS[kind], dtype_code(x.dtype), stream_handle()), "activation")
    return out
