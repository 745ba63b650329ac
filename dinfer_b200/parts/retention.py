"""Retention: linear attention with one fixed decay per head, no softmax and no denominator.  Per head a matrix
S [key channels, value channels] in 32-bit is carried from token to token of a request:

    S_t = d_h S_(t-1) + k_t v_t^T,    o_t = S_t^T q_t,    k = (W_k x) dk^-1/2

Each head's o is divided by its root mean square (no weight), the heads are multiplied by ``silu(W_g x)`` and go
through the output projection.

Data flow of one step (prompt portions and decoded tokens alike):
  P = x [W_q; W_k; W_v; W_g]^T      one stacked product, its result kept 32-bit (what enters the recurrence is rounded
                                    nowhere behind x itself)
  o = retention(q, k, v, S)         32-bit, chunks of tokens, S in place in the request's state row
  y = o / rms(o) * silu(gate);  out = y W_o^T
Slots and fresh flags are read from the device only, so steps replay as CUDA graphs.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import delta_ops, stream_ops
from .base import MIXERS, BuildEnv, CacheBinding, Mixer, StateNeed, StepContext
from .linear import Linear
from .spec import TensorDecl


@MIXERS.register("retention")
class Retention(Mixer):
    """params: ``num_heads``, ``key_dim``, ``value_dim``, ``decay`` (one number per head), ``eps`` (of the output
    norm), ``out_float32`` (the output projection's result stays 32-bit, for an arrangement that norms it before it
    joins the stream), and the tensor names ``q_proj``, ``k_proj``, ``v_proj``, ``gate_proj``, ``o_proj``."""

    graph_capturable = True

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.hidden = env.hidden_size
        self.H, self.dk, self.dv = int(p["num_heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.decay_values = [float(d) for d in p["decay"]]
        self.eps = float(p["eps"])
        self.out_float32 = bool(p.get("out_float32", False))
        if min(self.H, self.dk, self.dv) <= 0 or len(self.decay_values) != self.H:
            raise ValueError(f"retention: {self.H} heads of {self.dk} x {self.dv} with {len(self.decay_values)} decays")
        n = lambda key, default: prefix + p.get(key, default)
        self.names = {"q": n("q_proj", "q"), "k": n("k_proj", "k"), "v": n("v_proj", "v"), "g": n("gate_proj", "g"),
                      "o": n("o_proj", "o")}
        self.nq, self.nv = self.H * self.dk, self.H * self.dv
        self.state_size = self.H * self.dk * self.dv
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def declare(self) -> List[TensorDecl]:
        h, N = self.hidden, self.names
        return [TensorDecl(N["q"], (self.nq, h)), TensorDecl(N["k"], (self.nq, h)), TensorDecl(N["v"], (self.nv, h)),
                TensorDecl(N["g"], (self.nv, h)), TensorDecl(N["o"], (h, self.nv))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        N = self.names
        rows = [tensors[N[x]] for x in ("q", "k", "v", "g")]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in rows) else rows[0].dtype
        self.proj = Linear(torch.cat([t.to(dt) for t in rows], dim=0))
        self.o = Linear(tensors[N["o"]])
        dev = rows[0].device
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=dev)
        self.powers = stream_ops.retention_powers(self.decay)
        self.ones = torch.ones(self.dv, dtype=torch.float32, device=dev)

    def cache_need(self):
        return StateNeed((self.state_size,), torch.float32)

    def kernel_libraries(self):
        return ["retention", "delta_rule"] + self.proj.kernel_libraries() + self.o.kernel_libraries()

    def forward(self, x, ctx: StepContext, cache: CacheBinding):
        T = x.shape[0]
        P = self.proj(x, out_dtype=torch.float32)
        nq, nv = self.nq, self.nv
        B = ctx.cu_seqlens.numel() - 1
        o = stream_ops.retention(P[:, :nq], P[:, nq:2 * nq], P[:, 2 * nq:2 * nq + nv], self.decay, cache.state,
                                 ctx.cu_seqlens, ctx.state_slots[:B], ctx.state_fresh[:B], self.H, self.dk, self.dv,
                                 float(self.dk) ** -0.5, max_q_len=ctx.max_q_len, powers=self.powers)
        y = torch.empty((T, nv), dtype=x.dtype, device=x.device)
        # the delta rule's output kernel does o / rms(o) * w * silu(gate); here w is all ones
        delta_ops.post(o, self.ones, P[:, 2 * nq + nv:], self.eps, False, y)
        return self.o(y, out_dtype=torch.float32 if self.out_float32 else None)
