"""A routed feed-forward: a 32-bit router picks ``top_k`` of ``num_experts`` small feed-forwards per token, their
outputs are summed with the router's weights, and an optional shared expert runs for every token.

Data flow of one step (nothing goes through the host; every size is fixed by the number of tokens, so the step
can be captured in a CUDA graph):
  z = x [W_r; w_g]^T                    f32 logits of the router (and of the shared expert's gate) by the engine's product
  ids, w, g = route(z)                  scores -> top-k (+ the gate's sigmoid)
  layout    = align(ids)                (token, choice) pairs expert by expert, runs padded to the row tile
  u         = act(x[pair] W_up[e]^T)    grouped product, rows gathered
  y[pair]   = (u W_down[e]^T) * w[pair] grouped product, rows scattered back
  out[t]    = sum_k y[t, k] + g[t] * shared(x[t])
The experts' matrices are stacked at load into ``[E, ff, h]`` and ``[E, h, ff]``.

Two options change the ends of that flow, not its middle.  ``routing = "table"``: no router; an integer table
[vocab, top_k] names each token id's experts and every choice weighs ``1 / top_k`` (the step's token ids come
from ``ctx.token_ids``).  ``gated``: an expert is ``down(act(gate(x)) * up(x))``; gate and up are stacked as
(gate_j, up_j) row pairs into ``[E, 2 ff, h]``, so that one grouped product feeds the gate.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import moe_ops
from .base import FEED_FORWARDS, FeedForward
from .linear import Linear
from .spec import TensorDecl


@FEED_FORWARDS.register("moe")
class MoE(FeedForward):
    """params: ``num_experts``, ``top_k``, ``expert_size``, ``activation`` (relu2, silu, gelu_tanh, relu: experts are
    ``down(act(up(x)))`` without a gate), ``scoring`` (softmax over all experts, or sigmoid), ``renormalize`` (the
    chosen scores divided by their sum), ``shared_size`` (0: no shared expert), ``shared_gate`` ("sigmoid": the
    shared expert's output times ``sigmoid(w_g . x)``; None: added as it is), and the tensor names ``router``,
    ``expert_up`` / ``expert_down`` (with ``{e}`` for the expert's index), ``shared_up``, ``shared_down``,
    ``shared_gate_proj``.  ``routing`` ("router", the default, or "table": tensor name ``table``), ``gated`` (experts
    and the shared expert have a gate matrix: names ``expert_gate``, ``shared_gate_up``).  ``weight_on`` ("output", the
    default: ``sum_k w_k expert_k(x)``; "input": ``sum_k expert_k(w_k x)``, gated experts only: the weight is applied
    to the first product's result, in 32-bit, ahead of the activation)."""

    def __init__(self, params, env, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.hidden = env.hidden_size
        self.E, self.top = int(p["num_experts"]), int(p["top_k"])
        self.ff = int(p["expert_size"])
        self.shared_ff = int(p.get("shared_size", 0) or 0)
        self.activation = str(p.get("activation", "relu2"))
        self.scoring = str(p.get("scoring", "softmax"))
        self.renormalize = bool(p.get("renormalize", False))
        self.shared_gate = p.get("shared_gate")
        self.routing = str(p.get("routing", "router"))
        self.gated = bool(p.get("gated", False))
        self.vocab = int(p.get("vocab_size", 0))
        self.weight_on_input = p.get("weight_on", "output") == "input"
        if p.get("weight_on", "output") not in ("output", "input") or (self.weight_on_input and not self.gated):
            raise ValueError("moe: weight_on is output or input, and input needs gated experts")
        self._ones = {}
        if self.routing not in ("router", "table") or (self.routing == "table" and (self.vocab <= 0 or self.shared_gate)):
            raise ValueError("moe: routing is router or table; a table needs vocab_size and takes no gate on the shared expert")
        if not (0 < self.top <= self.E):
            raise ValueError(f"moe: top_k {self.top} must be between 1 and num_experts {self.E}")
        if self.activation not in moe_ops.ACTIVATIONS or self.activation == "none":
            raise ValueError(f"moe: unknown activation {self.activation!r}")
        if self.scoring not in ("softmax", "sigmoid") or self.shared_gate not in (None, "sigmoid"):
            raise ValueError("moe: scoring is softmax or sigmoid, shared_gate sigmoid or None")
        n = lambda key, default: prefix + p.get(key, default)
        self.names = {"router": n("router", "router.weight"), "up": n("expert_up", "experts.{e}.up.weight"),
                      "down": n("expert_down", "experts.{e}.down.weight"), "s_up": n("shared_up", "shared.up.weight"),
                      "s_down": n("shared_down", "shared.down.weight"), "s_gate": n("shared_gate_proj", "shared.gate.weight"),
                      "table": n("table", "table"), "gate": n("expert_gate", "experts.{e}.gate.weight"),
                      "s_gate_up": n("shared_gate_up", "shared.gate_proj.weight")}
        self.router: Optional[Linear] = None
        self.w_up = self.w_down = None
        self.shared_up: Optional[Linear] = None
        self.shared_down: Optional[Linear] = None

    def declare(self) -> List[TensorDecl]:
        h = self.hidden
        if self.routing == "table":
            d = [TensorDecl(self.names["table"], (self.vocab, self.top), kind="int", init="choices", init_arg=self.E)]
        else:
            d = [TensorDecl(self.names["router"], (self.E, h))]
        for e in range(self.E):
            if self.gated:
                d.append(TensorDecl(self.names["gate"].format(e=e), (self.ff, h)))
            d += [TensorDecl(self.names["up"].format(e=e), (self.ff, h)),
                  TensorDecl(self.names["down"].format(e=e), (h, self.ff))]
        if self.shared_ff:
            if self.gated:
                d.append(TensorDecl(self.names["s_gate_up"], (self.shared_ff, h)))
            d += [TensorDecl(self.names["s_up"], (self.shared_ff, h)), TensorDecl(self.names["s_down"], (h, self.shared_ff))]
            if self.shared_gate:
                d.append(TensorDecl(self.names["s_gate"], (1, h)))
        return d

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.routing == "table":
            self.table = tensors[self.names["table"]].to(torch.int32).contiguous()
        else:
            router_w = tensors[self.names["router"]]
            if self.shared_ff and self.shared_gate:             # the gate's row rides behind the experts' rows
                router_w = torch.cat([router_w, tensors[self.names["s_gate"]].to(router_w.dtype).reshape(1, -1)])
            # rows padded with zeros to a multiple of 8: the product's 32-bit output rows then start on 16-byte boundaries
            pad = -router_w.shape[0] % 8
            if pad:
                router_w = torch.cat([router_w, router_w.new_zeros((pad, router_w.shape[1]))])
            self.router = Linear(router_w)
        ups = [tensors[self.names["up"].format(e=e)] for e in range(self.E)]
        downs = [tensors[self.names["down"].format(e=e)] for e in range(self.E)]
        gates = [tensors[self.names["gate"].format(e=e)] for e in range(self.E)] if self.gated else []
        dt = torch.float32 if any(t.dtype == torch.float32 for t in ups + downs + gates) else ups[0].dtype
        if self.gated:                                          # rows 2j, 2j + 1 of an expert: gate_j, up_j
            self.w_up = torch.stack([torch.stack([g.to(dt), u.to(dt)], dim=1).reshape(2 * self.ff, self.hidden)
                                     for g, u in zip(gates, ups)]).contiguous()  # [E, 2 ff, h]
        else:
            self.w_up = torch.stack([t.to(dt) for t in ups]).contiguous()      # [E, ff, h]
        self.w_down = torch.stack([t.to(dt) for t in downs]).contiguous()      # [E, h, ff]
        if self.shared_ff:
            if self.gated:
                g, u = tensors[self.names["s_gate_up"]], tensors[self.names["s_up"]]
                sdt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
                self.shared_up = Linear(torch.stack([g.to(sdt), u.to(sdt)], dim=1).reshape(2 * self.shared_ff, self.hidden))
            else:
                self.shared_up = Linear(tensors[self.names["s_up"]])
            self.shared_down = Linear(tensors[self.names["s_down"]])

    def kernel_libraries(self):
        libs = ["moe", "elementwise"] + (self.router.kernel_libraries() if self.router is not None else [])
        if self.w_up.dtype == torch.bfloat16:
            libs.append("gemm_tc")
        if self.shared_ff:
            libs += self.shared_up.kernel_libraries() + self.shared_down.kernel_libraries()
        return libs

    def forward(self, x, ctx=None, sink=None):
        T = x.shape[0]
        if self.routing == "table":
            if ctx is None or ctx.token_ids is None:
                raise RuntimeError("moe: routing by a table needs the step's token ids (StepContext.token_ids)")
            ids, weights = moe_ops.route_table(ctx.token_ids, self.table, self.E, ctx.prev_tokens)
            gate = None
        else:
            # 32-bit logits: products of the stored values summed in 32-bit (the same product that makes the model's logits)
            z = self.router(x, out_dtype=torch.float32)
            ids, weights, gate = moe_ops.route(z, self.E, self.top, self.scoring, self.renormalize,
                                               bool(self.shared_ff and self.shared_gate))
        pairs = T * self.top
        wide = self.w_up.shape[1]                            # ff, or 2 ff with a gate
        first_act = "none" if self.gated else self.activation
        if moe_ops.tc_grouped_supported(x, self.w_up, self.w_down, pairs):
            # prompt-sized steps: rows laid out expert by expert in whole 256-row tiles, both products on tcgen05
            order, tile_expert = moe_ops.align(ids, self.E, moe_ops.TC_ROW_TILE)
            a = moe_ops.gather_rows(x, order, pairs, self.top)
            u = torch.empty((order.numel(), wide), dtype=x.dtype, device=x.device)
            moe_ops.grouped_gemm_tc(a, self.w_up, u, order, tile_expert, pairs, 0, first_act)
            u, weights = self._gate(u, order, weights)
            y = torch.empty((pairs, self.hidden), dtype=x.dtype, device=x.device)
            moe_ops.grouped_gemm_tc(u, self.w_down, y, order, tile_expert, pairs, 1, weights=weights)
            return self._combine(x, y, gate)
        tile = moe_ops.row_tile(pairs, self.E)
        order, tile_expert = moe_ops.align(ids, self.E, tile)
        u = torch.empty((order.numel(), wide), dtype=x.dtype, device=x.device)
        moe_ops.grouped_gemm(x, self.w_up, u, order, tile_expert, pairs, self.top, tile, 0, first_act)
        u, weights = self._gate(u, order, weights)
        y = torch.empty((pairs, self.hidden), dtype=x.dtype, device=x.device)
        moe_ops.grouped_gemm(u, self.w_down, y, order, tile_expert, pairs, self.top, tile, 1, weights=weights)
        return self._combine(x, y, gate)

    def _gate(self, u, order, weights):
        """With a gate: the (gate, up) column pairs of the first product become act(gate) * up.  Where the routing weight
        belongs on the expert's input, both are multiplied by it first and the second product gets weights of one.
        Returns (the second product's input, its weights)."""
        if not self.gated:
            return u, weights
        from ..kernels import ops
        out = torch.empty((u.shape[0], self.ff), dtype=u.dtype, device=u.device)
        if not self.weight_on_input:
            return ops.gated_act(u, out, self.activation, pairs=True), weights
        flat = weights.reshape(-1)
        ones = self._ones.get(flat.numel())
        if ones is None:
            if len(self._ones) > 64:
                self._ones.clear()
            ones = self._ones[flat.numel()] = torch.ones_like(flat)
        return ops.gated_act_scaled(u, out, flat, order, self.activation, pairs=True), ones

    def _combine(self, x, y, gate):
        shared = None
        if self.shared_ff and self.gated:
            shared = self.shared_down(self.shared_up.gated_pairs(x, self.activation))
        elif self.shared_ff:
            s = self.shared_up(x)
            moe_ops.activation(s, s, self.activation)
            shared = self.shared_down(s)
        out = torch.empty((x.shape[0], self.hidden), dtype=x.dtype, device=x.device)
        return moe_ops.combine(y, out, self.top, shared, gate)
