"""Differential attention over the paged cache.  Every query head has two score maps: its query is ``[map 1 | map 2]``
(``head_dim`` elements each), and so is every key of its key/value head; each map is a causal softmax attention of
its own over the same values, and the head's output is their difference

    o = a_1 - lambda a_2,    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff     (one number for the layer)

followed by ``o / rms(o) * (1 - diff)`` over the head's values (no weight) and a gate ``sigmoid(W_g x)_h`` of one number
per head and token.  No position encoding.  A query at position p sees the keys j <= p with ``p - j < window`` or
``j < keep_first``: the first tokens of a request stay visible behind the window (their pages are kept).

Data flow of one step:
  [q | k | v | gate] = x [W_q; W_k; W_v; W_g]^T     one stacked product
  k, v -> cache                                      rows [map 1 | map 2] and values, ``max(2 D, Dv)`` wide
  o = attention_diff(q, cache, gate)                 both maps, the difference, the norm and the gate in one kernel:
                                                     on the tensor cores in bfloat16 where it takes the sizes (prompt
                                                     portions in tiles of rows, decoded tokens with the keys split),
                                                     else the plain-arithmetic kernel, which takes every size
  y = o W_o^T
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kernels import attention_ops, ops
from .base import MIXERS, BuildEnv, CacheBinding, KvCacheNeed, Mixer, StepContext
from .linear import Linear
from .spec import TensorDecl


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim`` (of one map), ``v_dim``, ``scale``, ``diff`` (the constant in
    lambda and in the output factor ``1 - diff``), ``eps`` (of the output norm), optional ``window``, ``keep_first``,
    ``cache_block_size``, ``out_float32``, ``decode_splits`` (key splits of decoded tokens; 0: chosen per step), and the tensor names ``q_proj``, ``k_proj``, ``v_proj``, ``gate_proj`` ([H,
    width]), ``o_proj``, ``lambda_q1``, ``lambda_k1``, ``lambda_q2``, ``lambda_k2`` ([head_dim] each)."""

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.hidden = env.hidden_size
        self.H, self.Hkv = int(p["num_heads"]), int(p["num_kv_heads"])
        self.D, self.Dv = int(p["head_dim"]), int(p["v_dim"])
        if self.H % self.Hkv or min(self.H, self.Hkv, self.D, self.Dv) <= 0:
            raise ValueError(f"differential attention: heads {self.H} / kv heads {self.Hkv} / sizes {self.D}, {self.Dv}")
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.D)))
        self.diff = float(p["diff"])
        self.eps = float(p.get("eps", 1e-6))
        self.window = p.get("window")
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.force_splits = int(p.get("decode_splits") or 0)
        self.page_size = p.get("cache_block_size")
        self.out_float32 = bool(p.get("out_float32", False))
        n = lambda key, default: prefix + p.get(key, default)
        self.names = {"q": n("q_proj", "q"), "k": n("k_proj", "k"), "v": n("v_proj", "v"), "g": n("gate_proj", "g"),
                      "o": n("o_proj", "o"), "lq1": n("lambda_q1", "lq1"), "lk1": n("lambda_k1", "lk1"),
                      "lq2": n("lambda_q2", "lq2"), "lk2": n("lambda_k2", "lk2")}
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.lam = 0.0

    def declare(self) -> List[TensorDecl]:
        H, G, D, Dv, h, N = self.H, self.Hkv, self.D, self.Dv, self.hidden, self.names
        return [TensorDecl(N["q"], (H * 2 * D, h)), TensorDecl(N["k"], (G * 2 * D, h)), TensorDecl(N["v"], (G * Dv, h)),
                TensorDecl(N["g"], (H, h)), TensorDecl(N["o"], (h, H * Dv))] + \
               [TensorDecl(N[x], (D,)) for x in ("lq1", "lk1", "lq2", "lk2")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        N = self.names
        rows = [tensors[N[x]] for x in ("q", "k", "v", "g")]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in rows) else rows[0].dtype
        gate = rows[3].to(dt)
        pad = (-gate.shape[0]) % 8                           # the product's kernels like a multiple of 8 columns
        if pad:
            gate = torch.cat([gate, gate.new_zeros((pad, gate.shape[1]))], dim=0)
        self.proj = Linear(torch.cat([rows[0].to(dt), rows[1].to(dt), rows[2].to(dt), gate], dim=0))
        self.o = Linear(tensors[N["o"]])
        dot = lambda a, b: float((tensors[N[a]].double() * tensors[N[b]].double()).sum().item())
        self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + self.diff

    def cache_need(self):
        return KvCacheNeed(self.Hkv, max(2 * self.D, self.Dv), self.window, int(self.page_size) if self.page_size else None,
                           keep_first=self.keep_first)

    def kernel_libraries(self):
        return ["qk_post", "attention_diff", "attention_diff_tc"] + self.proj.kernel_libraries() + self.o.kernel_libraries()

    def forward(self, x, ctx: StepContext, cache: CacheBinding):
        H, G, D, Dv = self.H, self.Hkv, self.D, self.Dv
        g = ctx.groups[cache.group]
        P = self.proj(x)
        nq, nk, nv = H * 2 * D, G * 2 * D, G * Dv
        if cache.write:
            # no norm, no rotation: the general q/k/v kernel only moves keys (both maps as one row) and values into the cache
            ops.qkv_post_general(P[:, :nq + nk + nv], ctx.positions, H, G, 2 * D, Dv, self.eps, None, None, False, True, None,
                                 cache.kv, g.slot_mapping, g.block_size)
        out = torch.empty((P.shape[0], H * Dv), dtype=P.dtype, device=P.device)
        q, gate, window = P[:, :nq], P[:, nq + nk + nv:nq + nk + nv + H], int(self.window or 0)
        if attention_ops.diff_tc_supported(P.dtype, D, Dv, H // G):
            # the keys a decoded token sees end at the window (and the kept first ones): no more splits than they fill
            # (inside a captured graph the count is fixed for the longest request the engine admits).  The splits are
            # counted against one wave of the CTAs of the decode shape that fit the SMs.
            longest = self.env.max_positions if ctx.decode_splits else ctx.max_seq_len
            seen = min(longest, window + self.keep_first) if window else longest
            splits = self.force_splits or attention_ops.decode_splits(ctx.num_reqs, G, seen,
                                                                      attention_ops.diff_tc_decode_ctas_per_sm(D, Dv))
            attention_ops.attention_diff_tc(q, out, gate, cache.kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, H, G, D, Dv,
                                            self.scale, window, self.keep_first, self.lam, self.eps, 1.0 - self.diff,
                                            ctx.max_q_len, ctx.any_decode, ctx.any_prefill, splits)
        else:
            ops.attention_diff(q, out, gate, cache.kv, g.block_table, ctx.cu_seqlens, ctx.positions, H, G, D, Dv,
                               self.scale, window, self.keep_first, self.lam, self.eps, 1.0 - self.diff)
        return self.o(out, out_dtype=torch.float32 if self.out_float32 else None)
