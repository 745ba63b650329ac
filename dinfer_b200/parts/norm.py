"""RMSNorm over the residual stream, fused with the residual add and the gather of rows."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import NORMS, Norm
from .spec import TensorDecl


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``, ``weight`` (tensor name after the prefix), ``optional`` (the weight may be absent
    from the file: the norm of a branch the layer does not have), ``scalar`` (the weight is one number for all
    coordinates, a tensor without dimensions: kept as ``gain``, and spread over the row for the kernels that take a
    vector), ``offset`` (the file stores the weight around zero: the norm multiplies by ``offset + w``, kept in 32-bit
    so that the stored digits survive the sum).

    ``out = T(v * rsqrt(mean(v^2) + eps) * w)`` with ``v = residual (+ delta)`` in 32-bit
    (crates/kernels/cuda/norm.cu:54-115, crates/layers/src/nn.rs:78-111)."""

    def __init__(self, params, env, prefix=""):
        super().__init__(params, env, prefix)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight_name = prefix + params.get("weight", "weight")
        self.optional = bool(params.get("optional", False))
        self.scalar = bool(params.get("scalar", False))
        self.offset = float(params.get("offset", 0.0))
        self.weight: Optional[torch.Tensor] = None
        self.gain: Optional[float] = None

    def declare(self) -> List[TensorDecl]:
        return [TensorDecl(self.weight_name, () if self.scalar else (self.size,), init="normal" if self.offset else "ones",
                           optional=self.optional)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors.get(self.weight_name) if self.optional else tensors[self.weight_name]
        if w is not None and self.offset:
            w = w.to(torch.float32) + self.offset
        if w is not None and self.scalar:
            self.gain = float(w.float().item())
            w = w.reshape(1).expand(self.size)
        self.weight = None if w is None else w.contiguous()

    def kernel_libraries(self):
        return ["norm"]

    def forward(self, residual, delta=None, rows=None):
        from .base import ScaledDeltas
        if isinstance(delta, ScaledDeltas):                 # branch outputs with scales: summed by a kernel of their own
            ops.scaled_add(residual, delta.items)
            delta = None
        n = rows.numel() if rows is not None else residual.shape[0]
        out = torch.empty((n, self.size), dtype=self.env.act_dtype, device=residual.device)
        return ops.rmsnorm(residual, self.weight, self.eps, out, delta=delta, rows=rows)


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """params: ``size``, ``eps``, ``weight``, ``bias`` (tensor names after the prefix; ``bias`` None: no bias),
    ``optional`` (the tensors may be absent from the file: the norm of a branch the layer does not have).

    ``out = T((v - mean(v)) * rsqrt(mean((v - mean(v))^2) + eps) * w + b)`` over ``v = residual (+ pending)`` in
    32-bit.  ``delta`` may be a plain tensor or a ``ScaledDeltas`` (branch outputs with per-channel scales): the
    same kernel adds them.  ``forward_pair`` norms the same rows with two norms in one kernel (mean and variance
    are computed once), for layers whose mixer and feed-forward read the same ``x``."""

    def __init__(self, params, env, prefix=""):
        super().__init__(params, env, prefix)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight_name = prefix + params.get("weight", "weight")
        self.bias_name = prefix + params["bias"] if params.get("bias") else None
        self.optional = bool(params.get("optional", False))
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def declare(self) -> List[TensorDecl]:
        d = [TensorDecl(self.weight_name, (self.size,), init="ones", optional=self.optional)]
        if self.bias_name:
            d.append(TensorDecl(self.bias_name, (self.size,), optional=self.optional))
        return d

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors.get(self.weight_name) if self.optional else tensors[self.weight_name]
        if w is None:
            return
        self.weight = w.contiguous()
        if self.bias_name:
            self.bias = tensors[self.bias_name].to(self.weight.dtype).contiguous()

    def kernel_libraries(self):
        return ["norm"]

    @staticmethod
    def _deltas(delta):
        from .base import ScaledDeltas
        if delta is None:
            return ()
        return delta.items if isinstance(delta, ScaledDeltas) else ((delta, None),)

    def _deltas_for(self, delta):
        # scales travel in the dtype of this norm's weights (a file that stores some of them wider converts here)
        dt = self.weight.dtype
        return [(d, s if s is None or s.dtype == dt else s.to(dt)) for d, s in self._deltas(delta)]

    def forward(self, residual, delta=None, rows=None):
        n = rows.numel() if rows is not None else residual.shape[0]
        out = torch.empty((n, self.size), dtype=self.env.act_dtype, device=residual.device)
        return ops.layernorm(residual, self.weight, self.bias, self.eps, out, deltas=self._deltas_for(delta), rows=rows)

    def forward_pair(self, other: "LayerNorm", residual, delta=None):
        """(this norm of the rows, ``other``'s norm of the same rows); both must agree in size and eps."""
        if other.size != self.size or other.eps != self.eps:
            raise ValueError("two norms of one kernel must have the same size and eps")
        out = torch.empty((2, residual.shape[0], self.size), dtype=self.env.act_dtype, device=residual.device)
        ops.layernorm(residual, self.weight, self.bias, self.eps, out[0], deltas=self._deltas_for(delta),
                      weight2=other.weight, bias2=other.bias, out2=out[1])
        return out[0], out[1]
