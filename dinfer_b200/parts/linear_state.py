"""Two recurrent mixers whose per-request state is a matrix S [key channels, value channels] per head in 32-bit with
a decay per key channel; they share one recurrence kernel (``csrc/linear_state.cu``).

``general_delta``: the generalized delta rule.  With ``r, k, v = W_r x, W_k x, W_v x``, the decay
``w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 x) + w0))``, the removal rate ``a = sigmoid(W_a x + a_b)`` and the unit
key ``u = k / sqrt(sum(k^2) + 1e-6)`` of each head:

    S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,    o_t = S_t^T r_t

Each head's o is divided by its root mean square, the heads times a weight (every head's channels their own) times
``sigmoid(W_g x)``, then the output projection.

``gate_write`` (HGRN2): linear attention in which the forget gate also says what is written.  ``q = silu(W_q x)``,
``v = W_v x``, ``f = lower + (1 - lower) * sigmoid(W_f x + f_b)``:

    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,    o_t = S_t^T q_t

Each head's o is RMS-normed with a weight shared by the heads, then the output projection.

Data flow of one step (prompt portions and decoded tokens alike): one stacked product whose result stays 32-bit (what
enters the recurrence is rounded nowhere behind x itself), a preparation kernel (32-bit), the recurrence with S in place
in the request's state row, the output norm (and gate), the output projection.  Slots and fresh flags are read from
the device only, so steps replay as CUDA graphs.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kernels import delta_ops, state_ops
from .base import MIXERS, BuildEnv, CacheBinding, Mixer, StateNeed, StepContext
from .linear import Linear
from .spec import TensorDecl


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


def _stack(mats: List[torch.Tensor]):
    """One matrix of the given ones on top of each other, each starting at a multiple of 8 rows (zero rows between):
    (matrix, the column at which each part of the product starts)."""
    dt = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
    parts, cols, at = [], [], 0
    for t in mats:
        cols.append(at)
        parts.append(t.to(dt))
        pad = _up8(t.shape[0]) - t.shape[0]
        if pad:
            parts.append(t.new_zeros((pad, t.shape[1]), dtype=dt))
        at += _up8(t.shape[0])
    return torch.cat(parts, dim=0), cols


@MIXERS.register("general_delta")
class GeneralDelta(Mixer):
    """params: ``num_heads``, ``key_dim``, ``value_dim``, ``eps`` (of the output norm), ``decay_scale`` (the factor in
    the decay's exponent; default ``exp(-1/2)``), ``out_float32`` (the output projection's result stays 32-bit, for an
    arrangement that norms it before it joins the stream), and the tensor names ``r_proj``, ``k_proj``, ``v_proj``,
    ``a_proj``, ``a_bias``, ``decay_proj`` (the two matrices of the thin projection as a pair; the width of its middle is
    ``decay_rank``, or whatever the file holds), ``decay_bias``, ``gate_proj``, ``norm``, ``o_proj``."""

    graph_capturable = True

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.hidden = env.hidden_size
        self.H, self.dk, self.dv = int(p["num_heads"]), int(p["key_dim"]), int(p.get("value_dim", p["key_dim"]))
        self.eps = float(p["eps"])
        self.decay_scale = float(p.get("decay_scale", math.exp(-0.5)))
        self.out_float32 = bool(p.get("out_float32", False))
        self.decay_rank = int(p.get("decay_rank", -1) or -1)
        if min(self.H, self.dk, self.dv) <= 0:
            raise ValueError(f"general_delta: {self.H} heads of {self.dk} x {self.dv}")
        n = lambda key, default: prefix + p.get(key, default)
        d1, d2 = p.get("decay_proj", ("w1", "w2"))
        self.names = {"r": n("r_proj", "r"), "k": n("k_proj", "k"), "v": n("v_proj", "v"), "a": n("a_proj", "a"),
                      "ab": n("a_bias", "a.b"), "w1": prefix + d1, "w2": prefix + d2, "w0": n("decay_bias", "w0"),
                      "g": n("gate_proj", "g"), "norm": n("norm", "norm"), "o": n("o_proj", "o")}
        self.nk, self.nv = self.H * self.dk, self.H * self.dv
        self.state_size = self.H * self.dk * self.dv
        self.proj: Optional[Linear] = None

    def declare(self) -> List[TensorDecl]:
        h, N, nk, nv = self.hidden, self.names, self.nk, self.nv
        return [TensorDecl(N["r"], (nk, h)), TensorDecl(N["k"], (nk, h)), TensorDecl(N["v"], (nv, h)),
                TensorDecl(N["a"], (nk, h)), TensorDecl(N["ab"], (nk,)), TensorDecl(N["w1"], (self.decay_rank, h)),
                TensorDecl(N["w2"], (nk, self.decay_rank)), TensorDecl(N["w0"], (nk,)), TensorDecl(N["g"], (nv, h)),
                TensorDecl(N["norm"], (nv,), init="ones"), TensorDecl(N["o"], (h, nv))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        N = self.names
        w1, w2 = tensors[N["w1"]], tensors[N["w2"]]
        if w1.shape[0] != w2.shape[1]:
            raise ValueError(f"{N['w1']} has {w1.shape[0]} rows, {N['w2']} has {w2.shape[1]} columns: the thin middle must agree")
        self.rank = int(w1.shape[0])
        stacked, self.col = _stack([tensors[N[x]] for x in ("r", "k", "v", "a", "g")] + [w1])
        self.proj = Linear(stacked)
        self.decay_up = Linear(w2)
        self.o = Linear(tensors[N["o"]])
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.w0, self.a_bias, self.norm_w = f32(tensors[N["w0"]]), f32(tensors[N["ab"]]), f32(tensors[N["norm"]])

    def cache_need(self):
        return StateNeed((self.state_size,), torch.float32)

    def kernel_libraries(self):
        return (["linear_state", "delta_rule", "gemm_f32"] + self.proj.kernel_libraries() + self.decay_up.kernel_libraries()
                + self.o.kernel_libraries())

    def forward(self, x, ctx: StepContext, cache: CacheBinding):
        T = x.shape[0]
        P = self.proj(x, out_dtype=torch.float32)
        cr, ck, cv, ca, cg, cw = self.col
        nk, nv = self.nk, self.nv
        d = self.decay_up(state_ops.tanh_rows(P[:, cw:cw + self.rank]))
        k = P[:, ck:ck + nk]
        w, u, p = state_ops.general_delta_prep(k, d, P[:, ca:ca + nk], self.w0, self.a_bias, self.decay_scale, self.H, self.dk)
        B = ctx.cu_seqlens.numel() - 1
        o = state_ops.recurrence(P[:, cr:cr + nk], w, P[:, cv:cv + nv], cache.state, ctx.cu_seqlens, ctx.state_slots[:B],
                                 ctx.state_fresh[:B], self.H, self.dk, self.dv, k=k, u=u, p=p)
        y = torch.empty((T, nv), dtype=x.dtype, device=x.device)
        delta_ops.post(o, self.norm_w, P[:, cg:cg + nv], self.eps, True, y)
        return self.o(y, out_dtype=torch.float32 if self.out_float32 else None)


@MIXERS.register("gate_write")
class GateWrite(Mixer):
    """params: ``num_heads``, ``key_dim``, ``value_dim``, ``eps`` (of the output norm), ``out_float32``, and the tensor
    names ``q_proj``, ``f_proj``, ``f_bias``, ``lower`` (the gate's lower bound per head and channel), ``v_proj``,
    ``norm`` (one row of ``value_dim`` shared by the heads), ``o_proj``."""

    graph_capturable = True

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.hidden = env.hidden_size
        self.H, self.dk, self.dv = int(p["num_heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.eps = float(p["eps"])
        self.out_float32 = bool(p.get("out_float32", False))
        if min(self.H, self.dk, self.dv) <= 0:
            raise ValueError(f"gate_write: {self.H} heads of {self.dk} x {self.dv}")
        n = lambda key, default: prefix + p.get(key, default)
        self.names = {"q": n("q_proj", "q"), "f": n("f_proj", "f"), "fb": n("f_bias", "f.b"), "lower": n("lower", "lower"),
                      "v": n("v_proj", "v"), "norm": n("norm", "norm"), "o": n("o_proj", "o")}
        self.nk, self.nv = self.H * self.dk, self.H * self.dv
        self.state_size = self.H * self.dk * self.dv
        self.proj: Optional[Linear] = None

    def declare(self) -> List[TensorDecl]:
        h, N, nk, nv = self.hidden, self.names, self.nk, self.nv
        return [TensorDecl(N["q"], (nk, h)), TensorDecl(N["f"], (nk, h)), TensorDecl(N["fb"], (nk,)),
                TensorDecl(N["lower"], (nk,)), TensorDecl(N["v"], (nv, h)), TensorDecl(N["norm"], (self.dv,), init="ones"),
                TensorDecl(N["o"], (h, nv))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        N = self.names
        stacked, self.col = _stack([tensors[N[x]] for x in ("q", "f", "v")])
        self.proj = Linear(stacked)
        self.o = Linear(tensors[N["o"]])
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.f_bias, self.lower, self.norm_w = f32(tensors[N["fb"]]), f32(tensors[N["lower"]]), f32(tensors[N["norm"]])

    def cache_need(self):
        return StateNeed((self.state_size,), torch.float32)

    def kernel_libraries(self):
        return ["linear_state", "delta_rule"] + self.proj.kernel_libraries() + self.o.kernel_libraries()

    def forward(self, x, ctx: StepContext, cache: CacheBinding):
        T = x.shape[0]
        P = self.proj(x, out_dtype=torch.float32)
        cq, cf, cv = self.col
        nk, nv = self.nk, self.nv
        q, f = state_ops.gate_write_prep(P[:, cq:cq + nk], P[:, cf:cf + nk], self.f_bias, self.lower)
        B = ctx.cu_seqlens.numel() - 1
        o = state_ops.recurrence(q, f, P[:, cv:cv + nv], cache.state, ctx.cu_seqlens, ctx.state_slots[:B],
                                 ctx.state_fresh[:B], self.H, self.dk, self.dv)
        y = torch.empty((T, nv), dtype=x.dtype, device=x.device)
        delta_ops.post(o, self.norm_w, None, self.eps, False, y)
        return self.o(y, out_dtype=torch.float32 if self.out_float32 else None)
