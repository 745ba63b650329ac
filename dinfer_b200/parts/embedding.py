"""What turns a step's token ids into the first rows of the 32-bit residual stream.

``table``: a row of the embedding table per token, times a fixed factor.  ``hashed_bigram``: the token's row plus a row
of a second table picked by a hash of (the token before, the token), plus a learned position vector.  The token before
a step's first one is part of the request's state (one int32 per state slot), read and brought up to date on the
device, so steps replay as CUDA graphs and a step launched on placeholders of the last step's samples works too.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import EMBEDDINGS, Embedding, StateNeed, StepContext
from .spec import TensorDecl


@EMBEDDINGS.register("table")
class TableEmbedding(Embedding):
    """params: ``tensor`` (the table's name), ``vocab_size``, ``scale`` (the rows are multiplied by it; default 1)."""

    def __init__(self, params, env, prefix=""):
        super().__init__(params, env, prefix)
        self.name = prefix + self.params.get("tensor", "embed")
        self.vocab = int(self.params["vocab_size"])
        self.scale = float(self.params.get("scale", 1.0))

    def declare(self) -> List[TensorDecl]:
        return [TensorDecl(self.name, (self.vocab, self.env.hidden_size))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.name].contiguous()

    def forward(self, ids, ctx: StepContext, state=None):
        x = torch.empty((ids.numel(), self.env.hidden_size), dtype=torch.float32, device=ids.device)
        return ops.embedding(ids, self.table, x, prev=ctx.prev_tokens, scale=self.scale)


@EMBEDDINGS.register("hashed_bigram")
class HashedBigramEmbedding(Embedding):
    """params: ``tensor``, ``vocab_size``; ``bigram`` (the second table's name; None: none) with ``buckets``,
    ``mul_prev``, ``mul_cur``: row ``(before * mul_prev + token * mul_cur) mod buckets``, and row ``buckets`` (the
    table's last) for a request's first token; ``positions`` (the name of a learned position table
    [``max_positions``, h]; None: none)."""

    def __init__(self, params, env, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.name = prefix + p.get("tensor", "embed")
        self.vocab = int(p["vocab_size"])
        self.bigram_name = prefix + p["bigram"] if p.get("bigram") else None
        self.pos_name = prefix + p["positions"] if p.get("positions") else None
        self.hashing = (int(p.get("buckets", 0)), int(p.get("mul_prev", 0)), int(p.get("mul_cur", 0)))
        self.max_positions = int(p.get("max_positions", env.max_positions))
        if self.bigram_name and (self.hashing[0] <= 0 or min(self.hashing[1:]) < 0):
            raise ValueError("hashed_bigram: buckets must be positive and the multipliers not negative")
        self.table = self.bigram = self.pos_table = None

    def declare(self) -> List[TensorDecl]:
        h = self.env.hidden_size
        d = [TensorDecl(self.name, (self.vocab, h))]
        if self.bigram_name:
            d.append(TensorDecl(self.bigram_name, (self.hashing[0] + 1, h)))
        if self.pos_name:
            d.append(TensorDecl(self.pos_name, (self.max_positions, h)))
        return d

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.name].contiguous()
        dt = self.table.dtype
        if self.bigram_name:
            self.bigram = tensors[self.bigram_name].to(dt).contiguous()
        if self.pos_name:
            self.pos_table = tensors[self.pos_name].to(dt).contiguous()

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((), torch.int32) if self.bigram_name else None

    def forward(self, ids, ctx: StepContext, state=None):
        x = torch.empty((ids.numel(), self.env.hidden_size), dtype=torch.float32, device=ids.device)
        B = ctx.cu_seqlens.numel() - 1
        return ops.embedding_bigram(ids, self.table, x, self.bigram, self.hashing, self.pos_table, ctx.positions,
                                    ctx.cu_seqlens, ctx.state_slots[:B], ctx.state_fresh[:B], state, prev=ctx.prev_tokens)
