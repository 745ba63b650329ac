"""Attention over a cached latent (multi-head latent attention), run in its absorbed form.

The design: queries go through a latent (``cq = RMSNorm(W_dq x)``, ``q = W_uq cq``, per head ``D`` unrotated and
``P`` rotated elements); keys and values come from one latent per token, ``c = RMSNorm((W_dkv x)[:R])``, plus one
rotated key part ``kr = rot((W_dkv x)[R:])`` shared by all heads: ``k_h = [W_uk[h] c | kr]``, ``v_h = W_uv[h] c``.
Only ``[c | kr]`` is cached (one row of R + P per token, pages ``[pages, 1, 1, page, R + P]``).

Absorbed: ``q_h . k_h = (W_uk[h]^T q_h[:D]) . c + q_h[D:] . kr`` and ``sum_j p_j v_hj = W_uv[h] (sum_j p_j c_j)``, so a
step never expands a cached row into per-head keys and values:

  [cq | c | kr] = x [W_dq; W_dkv]^T        one stacked product
  norm(cq), norm(c), rot(kr) -> cache      one kernel
  q = cq W_uq^T
  q_lat[:, h] = [ q[:, h, :D] W_uk[h] | rot(q[:, h, D:]) ]      batched product + one kernel
  o_lat[:, h] = softmax(q_lat[:, h] . rows * scale) rows[:, :R] multi-query attention over the latent cache
  o[:, h] = o_lat[:, h] W_uv[h]^T          batched product
  y = o W_o^T

A layer with ``own_kv`` False has no W_dkv: its schedule entry reads another entry's cache (``cache.write`` False)
with its own W_uk, W_uv and queries.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import latent_ops, ops
from ..kernels.lib import add_launches
from .base import MIXERS, POSITION_ENCODINGS, BuildEnv, CacheBinding, KvCacheNeed, Mixer, StepContext, build_part
from .linear import Linear
from .spec import PartSpec, TensorDecl


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """params: ``num_heads``, ``nope_dim`` (D), ``rope_dim`` (P), ``v_dim``, ``kv_rank`` (R), ``q_rank``, ``scale``,
    ``eps`` (of the two latent norms), ``position`` (a PartSpec of a table rotation over the ``rope_dim`` part),
    ``own_kv`` (False: no down projection for keys and values, the entry reads another entry's cache), optional
    ``window``, ``cache_block_size``, ``sink`` (tensor name of one number per head: the softmax of head h has one more
    term ``exp(sink_h)`` that carries no value and is not scaled), ``gate_proj`` (tensor name of ``W_g`` [H * v_dim,
    width]: the heads' outputs are multiplied by ``sigmoid(W_g x)`` before the output projection; it rides in the
    stacked down projection), ``out_float32``, and the tensor names ``q_down``, ``q_norm``, ``q_up``, ``kv_down``, ``kv_norm``,
    ``k_up``, ``v_up``, ``o_proj``."""

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.hidden = env.hidden_size
        self.H, self.D, self.P = int(p["num_heads"]), int(p["nope_dim"]), int(p["rope_dim"])
        self.V, self.R, self.Rq = int(p["v_dim"]), int(p["kv_rank"]), int(p["q_rank"])
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / float(self.D + self.P) ** 0.5
        self.eps = float(p.get("eps", 1e-6))
        self.own_kv = bool(p.get("own_kv", True))
        self.window = p.get("window")
        self.page_size = p.get("cache_block_size")
        pos: PartSpec = p.get("position") or PartSpec("none")
        self.position = build_part(POSITION_ENCODINGS, pos, env, prefix)
        if not self.position.fused:
            raise ValueError("latent attention rotates by a table (a position encoding its kernels apply)")
        # pairs (2i, 2i + 1), or (i, i + rot / 2) for a table rotation of the other style
        self.halves = self.position.fused_table() is not None and not getattr(self.position, "interleaved", False)
        self.sink_name = prefix + p["sink"] if p.get("sink") else None
        self.gate_name = prefix + p["gate_proj"] if p.get("gate_proj") else None
        self.out_float32 = bool(p.get("out_float32", False))
        self.sinks = None
        n = lambda key, default: prefix + p.get(key, default)
        self.names = {"dq": n("q_down", "q_down.weight"), "qn": n("q_norm", "q_norm.weight"), "uq": n("q_up", "q_up.weight"),
                      "dkv": n("kv_down", "kv_down.weight"), "kvn": n("kv_norm", "kv_norm.weight"),
                      "uk": n("k_up", "k_up.weight"), "uv": n("v_up", "v_up.weight"), "o": n("o_proj", "o_proj.weight")}
        self.down: Optional[Linear] = None
        self.uq: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.q_norm_w = self.kv_norm_w = self.uk_t = self.uv = None

    def declare(self) -> List[TensorDecl]:
        H, D, P, V, R, Rq, h = self.H, self.D, self.P, self.V, self.R, self.Rq, self.hidden
        d = [TensorDecl(self.names["dq"], (Rq, h)), TensorDecl(self.names["qn"], (Rq,), init="ones"),
             TensorDecl(self.names["uq"], (H * (D + P), Rq)), TensorDecl(self.names["uk"], (H * D, R)),
             TensorDecl(self.names["uv"], (H * V, R)), TensorDecl(self.names["o"], (h, H * V))]
        if self.own_kv:
            d += [TensorDecl(self.names["dkv"], (R + P, h)), TensorDecl(self.names["kvn"], (R,), init="ones")]
        if self.sink_name:
            d.append(TensorDecl(self.sink_name, (H,)))
        if self.gate_name:
            d.append(TensorDecl(self.gate_name, (H * V, h)))
        return d

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = {k: tensors[v] for k, v in self.names.items() if v in tensors}
        rows = [t["dq"]] + ([t["dkv"]] if self.own_kv else [])
        # the gate's rows ride behind the latents, from a multiple of 8 columns on (zero rows between)
        self.low_width = sum(x.shape[0] for x in rows)
        self.gate_at = (self.low_width + 7) // 8 * 8
        if self.gate_name:
            g = tensors[self.gate_name]
            if self.gate_at > self.low_width:
                rows.append(g.new_zeros((self.gate_at - self.low_width, g.shape[1])))
            rows.append(g)
        dt = torch.float32 if any(x.dtype == torch.float32 for x in rows) else rows[0].dtype
        self.down = Linear(torch.cat([x.to(dt) for x in rows], dim=0))           # [Rq (+ R + P) (+ H V), h], stacked once
        if self.sink_name:
            self.sinks = tensors[self.sink_name].float().contiguous()
        self.uq = Linear(t["uq"])
        self.o = Linear(t["o"])
        self.q_norm_w = t["qn"].contiguous()
        if self.own_kv:
            self.kv_norm_w = t["kvn"].to(self.q_norm_w.dtype).contiguous()
        # per head: W_uk[h] is [D, R]; the absorbing product wants it as [R, D] (out, in)
        self.uk_t = t["uk"].reshape(self.H, self.D, self.R).transpose(1, 2).contiguous()
        self.uv = t["uv"].reshape(self.H, self.V, self.R).contiguous()

    def cache_need(self):
        return KvCacheNeed(1, self.R + self.P, self.window, int(self.page_size) if self.page_size else None, planes=1)

    def kernel_libraries(self):
        return (["latent_post", "attention_latent", "gemm_f32"] + (["elementwise"] if self.gate_name else []) + self.down.kernel_libraries() + self.uq.kernel_libraries()
                + self.o.kernel_libraries())

    def forward(self, x, ctx: StepContext, cache: CacheBinding, sink=None):
        H, D, P, V, R, Rq = self.H, self.D, self.P, self.V, self.R, self.Rq
        g = ctx.groups[cache.group]
        T = x.shape[0]
        table = self.position.fused_table()
        full = self.down(x)                                              # [T, Rq (+ R + P) (+ gate)]
        low = full[:, :self.low_width]
        write = self.own_kv and cache.write
        if self.own_kv and not write:
            raise RuntimeError("a latent attention layer with its own down projection must own its cache entry")
        latent_ops.latent_down_post(low, ctx.positions, self.q_norm_w, Rq, self.kv_norm_w if write else None, R, P,
                                    self.eps, table, cache.kv if write else None, g.slot_mapping if write else None,
                                    halves=self.halves)
        q = self.uq(low[:, :Rq])                                         # [T, H (D + P)]
        # head-major storage, seen as [T, H, *]: the batched products then write whole matrices per head
        q_lat = torch.empty((H, T, R + P), dtype=q.dtype, device=q.device).transpose(0, 1)
        self.absorb(q.view(T, H, D + P)[:, :, :D], self.uk_t, q_lat[:, :, :R])
        latent_ops.latent_q_rope(q, ctx.positions, table, q_lat, H, D, P, R, halves=self.halves)
        o_lat = torch.empty((H, T, R), dtype=q.dtype, device=q.device).transpose(0, 1)
        self.attend(q_lat, o_lat, cache.kv, g, ctx)
        o = torch.empty((T, H, V), dtype=q.dtype, device=q.device)
        self.absorb(o_lat, self.uv, o)
        o = o.view(T, H * V)
        if self.gate_name:
            ops.sigmoid_gate(o, full[:, self.gate_at:self.gate_at + H * V])
        return self.o(o, out_dtype=torch.float32 if self.out_float32 else None)

    # rows up to which the per-head products run on this package's own kernel (each weight read once, 32-bit
    # multiply-adds); beyond, bfloat16 goes to the library's batched product like the other prompt-sized products
    OWN_ABSORB_ROWS = 32

    def absorb(self, a, w, out) -> None:
        """out[:, h] = a[:, h] @ w[h]^T for every head (a [T, H, K], w [H, N, K], out [T, H, N], any strides)."""
        if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] > self.OWN_ABSORB_ROWS:
            add_launches(1)
            torch.bmm(a.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
        else:
            ops.gemm_f32_batched(a, w, out)

    def attend(self, q_lat, o_lat, kv, g, ctx: StepContext) -> None:
        window = int(self.window or 0)
        if latent_ops.tc_supported(q_lat.dtype, self.R, self.P, g.block_size):
            # inside a captured graph the longest request is whatever the engine admits
            longest = self.env.max_positions if ctx.decode_splits else ctx.max_seq_len
            latent_ops.attention_latent_tc(q_lat, o_lat, kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, self.R, self.P,
                                           self.scale, window, max_q_len=ctx.max_q_len, max_seq_len=longest,
                                           sinks=self.sinks)
        else:
            latent_ops.attention_latent_generic(q_lat, o_lat, kv, g.block_table, ctx.cu_seqlens, ctx.positions, self.R,
                                                self.P, self.scale, window, sinks=self.sinks)
