"""A short causal convolution on a mixer's input: the mixer inside reads ``x + conv(x)`` instead of ``x``, where
``conv(x)_t = sum_j w[:, j] * x_(t - taps + 1 + j)`` per channel, zeros before a request's first token.

The last ``taps - 1`` inputs of a request are part of its state, so the pair keeps one fixed-size state row per request:
first the history, behind it whatever the mixer inside keeps as state (that mixer sees a view of the row's rest); a paged
cache of the mixer inside is handed through as it is.  Slots and fresh flags are read from the device only, so steps
replay as CUDA graphs whenever the mixer inside allows it."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import stream_ops
from .base import MIXERS, BuildEnv, CacheBinding, Mixer, StateNeed, StepContext, build_part, split_needs
from .spec import TensorDecl


@MIXERS.register("short_conv_input")
class ShortConvInput(Mixer):
    """params: ``inner`` (the PartSpec of the mixer that reads the result; its tensor names follow the same prefix),
    ``taps``, ``weight`` (tensor name of the taps, [width, taps])."""

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.inner: Mixer = build_part(MIXERS, p["inner"], env, prefix)
        self.taps = int(p["taps"])
        if self.taps < 1:
            raise ValueError("short_conv_input: at least one tap")
        self.width = env.hidden_size
        self.name = prefix + p.get("weight", "conv")
        self.history = (self.taps - 1) * self.width
        _, inner_state = split_needs(self.inner.cache_need())
        if inner_state is not None and (inner_state.dtype != torch.float32 or len(inner_state.shape) != 1):
            raise ValueError("short_conv_input: the mixer inside keeps its state as one row of 32-bit numbers")
        self.inner_state = inner_state.shape[0] if inner_state is not None else 0
        self.weight = None

    @property
    def graph_capturable(self):
        return self.inner_state == 0 or bool(getattr(self.inner, "graph_capturable", False))

    def declare(self) -> List[TensorDecl]:
        return self.inner.declare() + [TensorDecl(self.name, (self.width, self.taps))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.inner.bind(tensors)
        self.weight = tensors[self.name].contiguous()

    def cache_need(self):
        kv, _ = split_needs(self.inner.cache_need())
        need = [kv] if kv is not None else []
        if self.history + self.inner_state > 0:
            need.append(StateNeed((self.history + self.inner_state,), torch.float32))
        return need

    def kernel_libraries(self):
        return ["short_conv"] + self.inner.kernel_libraries()

    def forward(self, x, ctx: StepContext, cache: CacheBinding):
        inner = CacheBinding(kv=cache.kv, group=cache.group, write=cache.write,
                             state=cache.state[:, self.history:] if self.inner_state else None)
        B = ctx.cu_seqlens.numel() - 1
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        state = cache.state if cache.state is not None else torch.empty((1, 0), dtype=torch.float32, device=x.device)
        stream_ops.short_conv_input(x, self.weight, state, ctx.cu_seqlens, ctx.state_slots[:B], ctx.state_fresh[:B], y)
        return self.inner.forward(y, ctx, inner)
