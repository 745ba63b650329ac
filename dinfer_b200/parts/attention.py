"""Grouped-query attention over the paged cache: the mixer of Qwen3 and of anything else that is
q/k/v projections, an optional per-head RMSNorm of q and k, a position encoding, causal softmax
attention (optionally over a window) and an output projection.

Data flow of one step (models/qwen3/src/model.rs:141-172,212-313):
  qkv = x Wqkv^T                       one fused product, rows laid out q heads | k heads | v heads
  q, k <- rope(headnorm(q, k)); k, v -> cache      one kernel, in place
  o = softmax(q k^T * scale + mask) v              over the cache, through the block table
  y = o Wo^T
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kernels import attention_ops, ops
from .base import (MIXERS, POSITION_ENCODINGS, BuildEnv, CacheBinding, KvCacheNeed, Mixer, StepContext,
                   build_part)
from .linear import Linear
from .spec import PartSpec, TensorDecl


@MIXERS.register("gqa_attention")
class GQAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``qk_norm`` (bool), ``eps``,
    ``position`` (a PartSpec), optional ``window``, ``scale``, ``bias`` (bool: the four projections have a bias,
    named like their weights with ``.bias``, or with ``bias_suffix`` added to the weight's name), and the tensor
    names ``q_proj``, ``k_proj``, ``v_proj``, ``o_proj``, ``q_norm``, ``k_norm`` (after the prefix).  Further:
    ``v_dim`` (the values' width where it differs from ``head_dim``), ``qk_norm_order`` ("before" the rotation, the
    default, or "after" it), ``qk_norm_weight`` (False: the head norm has no weight), ``sink`` (the softmax has one
    more term of score 0 that carries no value: ``p_j = exp(s_j) / (1 + sum exp(s_j))``), ``out_float32`` (the output
    projection's result stays 32-bit, for an arrangement that norms it before it joins the stream).
    ``q_temperature`` = (coef, every): q at position p is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``.
    ``distance_slopes``: a distance bias ``- slope_h * (i - j)`` on the scores; "geometric" (``slope_h = 2^(-8 (h + 1) /
    H)``) or one number per head.  ``value_mix`` = {"weight": tensor name of one number lambda, "key": any name}: the
    first layer of a model with this key keeps its values of the step's tokens, every later one caches
    ``(1 - lambda) v + lambda v_first`` instead of its own v (the first one's tensor is not used).  ``gate_proj``: the
    heads are multiplied by ``sigmoid(W_g x)`` before the output projection."""

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.hidden = env.hidden_size
        self.H = int(p["num_heads"])
        self.Hkv = int(p["num_kv_heads"])
        self.D = int(p["head_dim"])
        if self.H % self.Hkv:
            raise ValueError(f"heads {self.H} not divisible by kv heads {self.Hkv}")
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("eps", 1e-6))
        self.window = p.get("window")
        self.page_size = p.get("cache_block_size")           # None: the engine's page size
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.D)))
        self.bias = bool(p.get("bias", False))
        self.bias_suffix = p.get("bias_suffix")
        self.out_float32 = bool(p.get("out_float32", False))     # the output projection's result stays 32-bit
        self.Dv = int(p.get("v_dim", self.D))
        self.sink = bool(p.get("sink", False))
        self.norm_after = p.get("qk_norm_order", "before") == "after"
        self.norm_weight = bool(p.get("qk_norm_weight", True))
        if p.get("qk_norm_order", "before") not in ("before", "after") or self.Dv <= 0:
            raise ValueError("attention: qk_norm_order is before or after, v_dim positive")
        self.q_temperature = tuple(p["q_temperature"]) if p.get("q_temperature") else None
        if self.q_temperature and (float(self.q_temperature[0]) == 0.0):
            self.q_temperature = None
        slopes = p.get("distance_slopes")
        if slopes == "geometric":
            slopes = [2.0 ** (-8.0 * (h + 1) / self.H) for h in range(self.H)]
        if slopes is not None and len(slopes) != self.H:
            raise ValueError("attention: distance_slopes is 'geometric' or one number per head")
        self.slope_values = [float(v) for v in slopes] if slopes is not None else None
        self.value_mix = dict(p["value_mix"]) if p.get("value_mix") else None
        self.gate_name = prefix + p["gate_proj"] if p.get("gate_proj") else None
        # the q/k kernel with lane paths takes the usual order and equal widths; anything else takes the general one
        self.general = (self.Dv != self.D or (self.qk_norm and (self.norm_after or not self.norm_weight))
                        or self.q_temperature is not None or self.value_mix is not None)
        pos: PartSpec = p.get("position") or PartSpec("none")
        self.position = build_part(POSITION_ENCODINGS, pos, env, prefix)
        n = lambda key, default: prefix + p.get(key, default)
        self.names = {
            "q": n("q_proj", "q_proj.weight"), "k": n("k_proj", "k_proj.weight"),
            "v": n("v_proj", "v_proj.weight"), "o": n("o_proj", "o_proj.weight"),
            "qn": n("q_norm", "q_norm.weight"), "kn": n("k_norm", "k_norm.weight"),
        }
        if self.value_mix:
            self.names["vmix"] = prefix + self.value_mix["weight"]
        self.slopes = None
        self.v_lambda = 0.0
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.q_norm_w = self.k_norm_w = None

    def declare(self) -> List[TensorDecl]:
        H, Hkv, D, Dv, h = self.H, self.Hkv, self.D, self.Dv, self.hidden
        d = [TensorDecl(self.names["q"], (H * D, h)), TensorDecl(self.names["k"], (Hkv * D, h)),
             TensorDecl(self.names["v"], (Hkv * Dv, h)), TensorDecl(self.names["o"], (h, H * Dv))]
        if self.qk_norm and self.norm_weight:
            d += [TensorDecl(self.names["qn"], (D,), init="ones"), TensorDecl(self.names["kn"], (D,), init="ones")]
        if self.bias:
            d += [TensorDecl(self._bias_name(x), (n,)) for x, n in (("q", H * D), ("k", Hkv * D), ("v", Hkv * Dv), ("o", h))]
        if self.value_mix:
            d.append(TensorDecl(self.names["vmix"], ()))
        if self.gate_name:
            d.append(TensorDecl(self.gate_name, (H * Dv, h)))
        return d

    def _bias_name(self, which: str) -> str:
        name = self.names[which]
        if self.bias_suffix:
            return name + self.bias_suffix
        return (name[:-len(".weight")] if name.endswith(".weight") else name) + ".bias"

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        q, k, v = (tensors[self.names[x]] for x in ("q", "k", "v"))
        dt = torch.float32 if any(t.dtype == torch.float32 for t in (q, k, v)) else q.dtype
        # q, k, v rows stacked once at load into one [(H + 2 Hkv) D, h] matrix (model.rs:141-164)
        qkv_bias = o_bias = None
        if self.bias:
            qkv_bias = torch.cat([tensors[self._bias_name(x)].to(dt) for x in ("q", "k", "v")])
            o_bias = tensors[self._bias_name("o")]
        # with the general q/k/v kernel the projection's bias is added there, not by a kernel of its own
        self.qkv_bias32 = qkv_bias.float().contiguous() if (self.general and qkv_bias is not None) else None
        rows = [q.to(dt), k.to(dt), v.to(dt)]
        self.gate_col = 0
        if self.gate_name:                                   # the gate rides behind q, k, v, from a multiple of 8 columns on
            if self.bias:
                raise ValueError("attention: a gate beside projections with biases is not built")
            used = sum(t.shape[0] for t in rows)
            self.gate_col = (used + 7) // 8 * 8
            if self.gate_col > used:
                rows.append(q.new_zeros((self.gate_col - used, q.shape[1]), dtype=dt))
            rows.append(tensors[self.gate_name].to(dt))
        self.qkv = Linear(torch.cat(rows, dim=0), None if self.general else qkv_bias)
        if self.slope_values is not None:
            self.slopes = torch.tensor(self.slope_values, dtype=torch.float32, device=q.device)
        if self.value_mix:
            self.v_lambda = float(tensors[self.names["vmix"]].float().item())
        self.o = Linear(tensors[self.names["o"]], o_bias)
        if self.qk_norm and self.norm_weight:
            self.q_norm_w = tensors[self.names["qn"]].contiguous()
            self.k_norm_w = tensors[self.names["kn"]].to(self.q_norm_w.dtype).contiguous()

    def cache_need(self):
        return KvCacheNeed(self.Hkv, max(self.D, self.Dv), self.window, int(self.page_size) if self.page_size else None)

    def _fast(self, dtype) -> bool:
        """Whether the tensor-core kernels take this attention: keys and values of one width."""
        return self.Dv == self.D and attention_ops.tc_supported(dtype, self.D, self.H // self.Hkv)


    def kernel_libraries(self):
        att = ["attention_generic"]
        if self._fast(self.env.act_dtype):
            att = ["attention_tc"]
            if self.D in (64, 128):
                att += ["attention_decode", "attention_umma", "attention_umma64"]
        return ["qk_post"] + att + self.qkv.kernel_libraries() + self.o.kernel_libraries()

    def takes_half_normed(self, rows: int) -> bool:
        return self.qkv.fuses_norm(rows, self.env.act_dtype)

    def adds_into_residual(self, rows: int) -> bool:
        return self.o.fuses_norm(rows, self.env.act_dtype)

    def forward(self, x, ctx: StepContext, cache: CacheBinding, sink=None):
        H, Hkv, D = self.H, self.Hkv, self.D
        g = ctx.groups[cache.group]
        qkv = self.qkv(x)
        kv = cache.kv if cache.write else None
        table = self.position.fused_table()
        if self.general:
            if not self.position.fused:
                raise NotImplementedError("attention: a head norm behind the rotation, or values of another width, "
                                          "need a position encoding the q/k kernel applies")
            v_first = None
            if self.value_mix:
                # the first layer with this key leaves its values of the step's tokens for the later ones
                key = ("value_mix", self.value_mix.get("key", ""))
                owner, v_first = ctx.derived.get(key, (None, None))
                if owner is None or owner is self:          # (the same context may run twice: a graph's warm-up)
                    at = (H + Hkv) * D
                    ctx.derived[key] = (self, qkv[:, at:at + Hkv * self.Dv])
                    v_first = None
            ops.qkv_post_general(qkv, ctx.positions, H, Hkv, D, self.Dv, self.eps, self.q_norm_w, self.k_norm_w,
                                 self.qk_norm, not self.norm_after, table, kv, g.slot_mapping, g.block_size,
                                 interleaved=getattr(self.position, "interleaved", False), bias=self.qkv_bias32,
                                 q_temperature=self.q_temperature, v_first=v_first, v_lambda=self.v_lambda)
        elif self.position.fused:
            ops.qk_post(qkv, ctx.positions, H, Hkv, D, self.eps, self.q_norm_w, self.k_norm_w, table,
                        kv, g.slot_mapping, g.block_size, interleaved=getattr(self.position, "interleaved", False))
        else:
            if self.qk_norm:
                ops.qk_post(qkv, ctx.positions, H, Hkv, D, self.eps, self.q_norm_w, self.k_norm_w, None,
                            None, None, g.block_size)
            T = qkv.shape[0]
            self.position.apply(qkv[:, :H * D].unflatten(1, (H, D)),
                                qkv[:, H * D:(H + Hkv) * D].unflatten(1, (Hkv, D)), ctx)
            if kv is not None:
                ops.qk_post(qkv, ctx.positions, H, Hkv, D, self.eps, None, None, None, kv,
                            g.slot_mapping, g.block_size)
        out = torch.empty((qkv.shape[0], H * self.Dv), dtype=qkv.dtype, device=qkv.device)
        self.attend(qkv[:, :H * D], out, cache.kv, g, ctx)
        if self.gate_name:
            ops.sigmoid_gate(out, qkv[:, self.gate_col:self.gate_col + H * self.Dv])
        if sink is not None:                               # (residual, the norm behind this mixer)
            return self.o.into_residual(out, sink[0], sink[1])
        return self.o(out, out_dtype=torch.float32 if self.out_float32 else None)

    def attend(self, q, out, kv, g, ctx: StepContext) -> None:
        """Tensor-core kernels where they take the head size (bfloat16; 32, 64, 128), else the
        plain-arithmetic kernel, which takes every size."""
        window = int(self.window or 0)
        if self._fast(q.dtype):
            splits = ctx.decode_splits or attention_ops.decode_splits(ctx.num_reqs, self.Hkv, ctx.max_seq_len)
            tc_decode = ctx.any_decode
            if ctx.any_decode and attention_ops.decode_supported(q.dtype, self.D, self.H // self.Hkv, g.block_size) \
                    and (g.block_size >= 8 or not (self.sink or self.slopes is not None)):
                # decoded tokens: the kernel made for them (keys on the tile's rows, in-kernel fold)
                attention_ops.attention_decode(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, self.H,
                                               self.Hkv, self.D, self.scale, window, splits, sink=self.sink,
                                               slopes=self.slopes)
                tc_decode = False
            tc_prefill = ctx.any_prefill
            if ctx.any_prefill and attention_ops.umma_supported(q.dtype, self.D, self.H // self.Hkv, g.block_size):
                # prompt portions: tcgen05 / TMEM / TMA
                key = ("attention_umma", self.H, self.Hkv, self.D)
                shape = ctx.derived.get(key)
                if shape is None:
                    cu = ctx.cu_seqlens_host
                    lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
                    group = self.H // self.Hkv
                    shape = ctx.derived[key] = (
                        attention_ops.umma_key_splits(lens or [ctx.max_q_len], group, self.Hkv, self.D, ctx.max_seq_len),
                        attention_ops.umma_pair_bound(lens, group) if lens else 0)
                if ((ctx.max_prefill_seq_len or ctx.max_seq_len) <= attention_ops.UMMA_SHORT_CONTEXT
                        and attention_ops.umma64_supported(q.dtype, self.D, self.H // self.Hkv, g.block_size)):
                    attention_ops.attention_umma64(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, self.H,
                                                   self.Hkv, self.D, self.scale, window, ctx.max_q_len, shape[1],
                                                   sink=self.sink, slopes=self.slopes)
                else:
                    attention_ops.attention_umma(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, self.H,
                                                 self.Hkv, self.D, self.scale, window, ctx.max_q_len, shape[0], shape[1],
                                                 sink=self.sink, slopes=self.slopes)
                tc_prefill = False
            if tc_decode or tc_prefill:
                attention_ops.attention_tc(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, self.H,
                                           self.Hkv, self.D, self.scale, window, ctx.max_q_len, tc_decode,
                                           tc_prefill, splits, sink=self.sink, slopes=self.slopes)
        else:
            ops.attention_generic(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.positions, self.H, self.Hkv,
                                  self.D, self.scale, window, v_dim=self.Dv, sink=self.sink, slopes=self.slopes)
