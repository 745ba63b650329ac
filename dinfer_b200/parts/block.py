"""Arrangements of a layer's four parts around the residual stream."""
from __future__ import annotations

from typing import Optional

from .base import BLOCKS, Block, CacheBinding, ResidualStream, StepContext
import torch

from .norm import RMSNorm


def norm_comes_apart(producer, norm, consumer, rows: int) -> bool:
    """Whether ``norm`` between ``producer`` and ``consumer`` can be taken apart for this many rows: the
    producer adds its output into the residual itself and hands on half-normed rows, the consumer finishes."""
    give = getattr(producer, "adds_into_residual", None)
    take = getattr(consumer, "takes_half_normed", None)
    return (isinstance(norm, RMSNorm) and norm.weight is not None and give is not None and take is not None
            and give(rows) and take(rows))


@BLOCKS.register("prenorm_residual")
class PreNormResidual(Block):
    """``x += mixer(norm1(x)); x += ffn(norm2(x))``.

    Each add is done inside the norm that follows it, and the feed-forward's output stays pending
    until the next layer's (or the model's final) norm picks it up, as the reference defers its MLP
    residual (models/qwen3/src/model.rs:700-743,772-813).  The stream itself stays 32-bit.

    Where the step asks for it (``ctx.split_norms``) and the parts on both sides of a norm can (few rows,
    bfloat16: decode steps), the norm has no kernel of its own: the part before it adds into the residual and
    leaves half-normed rows, the part behind it finishes them (``HalfNormed``).  That holds for the norm
    between mixer and feed-forward and for the first norm of the block that runs next.  Whether it pays
    depends on the sizes (two launches less against longer tails of the products), so it is an option of
    the engine (``EngineConfig.split_norms``)."""

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheBinding,
                next_block: Optional[Block] = None) -> None:
        rows = stream.x.shape[0]
        if stream.half is not None:
            if stream.half_norm is not self.mixer_norm:
                raise RuntimeError("half-normed rows were made for another norm than this block's first")
            h, stream.half, stream.half_norm = stream.half, None, None
        else:
            h = self.mixer_norm.forward(stream.x, delta=stream.pending)
            stream.pending = None
        split = bool(getattr(ctx, "split_norms", False))
        if split and norm_comes_apart(self.mixer, self.feed_forward_norm, self.feed_forward, rows):
            h = self.mixer.forward(h, ctx, cache, sink=(stream.x, self.feed_forward_norm))
        else:
            a = self.mixer.forward(h, ctx, cache)
            h = self.feed_forward_norm.forward(stream.x, delta=a)
        if split and next_block is not None and norm_comes_apart(self.feed_forward, next_block.mixer_norm, next_block.mixer, rows):
            stream.half = self.feed_forward.forward(h, ctx, sink=(stream.x, next_block.mixer_norm))
            stream.half_norm = next_block.mixer_norm
        else:
            stream.pending = self.feed_forward.forward(h, ctx)


@BLOCKS.register("parallel_residual")
class ParallelResidual(Block):
    """``x += s1 * mixer(norm1(x)) + s2 * ffn(norm2(x))``: both branches read the same ``x``.

    extras: ``mixer_scale`` / ``feed_forward_scale``: tensor names (after the layer's prefix) of per-channel
    scales [h] of the two branches (layer scale); absent = 1.  A layer may have no feed-forward (kind "none").

    Neither branch output is added by a kernel of its own: both stay pending (``ScaledDeltas``) until the next
    layer's (or the model's final) norm, whose kernel computes ``x + s1 * a + s2 * f`` in 32-bit, writes it back and
    norms it.  When the two norms are layer norms of one size they run as one kernel (one mean and variance, two
    weights and biases)."""

    def declare(self):
        from .spec import TensorDecl
        h = self.env.hidden_size
        d = []
        if self.extras.get("mixer_scale"):
            d.append(TensorDecl(self.prefix + self.extras["mixer_scale"], (h,), init="ones"))
        if self.extras.get("feed_forward_scale"):
            d.append(TensorDecl(self.prefix + self.extras["feed_forward_scale"], (h,), init="ones",
                                optional=self._no_feed_forward()))
        return d

    def _no_feed_forward(self) -> bool:
        return bool(getattr(self.feed_forward, "absent", False))

    def bind(self, tensors):
        def get(key):
            name = self.extras.get(key)
            t = tensors.get(self.prefix + name) if name else None
            return None if t is None else t.contiguous()
        self.mixer_scale, self.feed_forward_scale = get("mixer_scale"), get("feed_forward_scale")
        scales = [s for s in (self.mixer_scale, self.feed_forward_scale) if s is not None]
        if len(scales) == 2 and scales[0].dtype != scales[1].dtype:
            self.mixer_scale, self.feed_forward_scale = (s.float() for s in scales)

    def kernel_libraries(self):
        return ["norm"]

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheBinding,
                next_block: Optional[Block] = None) -> None:
        from .base import ScaledDeltas, resolve_pending
        from .norm import LayerNorm
        if stream.half is not None:
            raise RuntimeError("a parallel block does not take half-normed rows")
        n1, n2 = self.mixer_norm, self.feed_forward_norm
        if self._no_feed_forward():
            h1, h2 = n1.forward(stream.x, delta=stream.pending), None
        elif isinstance(n1, LayerNorm) and isinstance(n2, LayerNorm) and n1.size == n2.size and n1.eps == n2.eps:
            h1, h2 = n1.forward_pair(n2, stream.x, delta=stream.pending)
        else:
            h1 = n1.forward(stream.x, delta=stream.pending)
            h2 = n2.forward(stream.x)
        stream.pending = None
        a = self.mixer.forward(h1, ctx, cache)
        items = [(a, self.mixer_scale)]
        if h2 is not None:
            items.append((self.feed_forward.forward(h2, ctx), self.feed_forward_scale))
        stream.pending = ScaledDeltas(items)


@BLOCKS.register("postnorm_residual")
class PostNormResidual(Block):
    """``x += norm1(mixer(x)); x += norm2(ffn(x))``: the norm sits on the sublayer's output only, the sublayers read
    the stream itself (rounded to the activation type).

    One kernel per sublayer does the norm, the add into the 32-bit stream and the rounded copy of the new stream
    that the next sublayer's product reads (``ResidualStream.cast``).  A mixer that hands over branches which are
    each normed first and then averaged (``NormedBranches``) has that done in the same kernel.  A layer may have no
    feed-forward (kind "none")."""

    def kernel_libraries(self):
        return ["norm", "elementwise"]

    def _input(self, stream: ResidualStream):
        from ..kernels import ops
        if self.env.act_dtype == torch.float32:
            return stream.x
        if stream.cast is None:
            stream.cast = ops.cast(stream.x, torch.empty(stream.x.shape, dtype=self.env.act_dtype, device=stream.x.device))
        return stream.cast

    def _join(self, stream: ResidualStream, branch, norm) -> None:
        from ..kernels import ops
        from .base import NormedBranches
        cast = None
        if self.env.act_dtype != torch.float32:
            cast = torch.empty(stream.x.shape, dtype=self.env.act_dtype, device=stream.x.device)
        if isinstance(branch, NormedBranches):
            (a, wa), (b, wb) = branch.items if len(branch.items) == 2 else (branch.items[0], (None, None))
            ops.branch_norm(a, norm.weight, norm.eps, residual=stream.x, cast=cast, inner=(wa, wb), b=b,
                            coef=branch.coef, inner_eps=branch.eps)
        else:
            ops.branch_norm(branch, norm.weight, norm.eps, residual=stream.x, cast=cast)
        stream.cast = cast

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheBinding,
                next_block: Optional[Block] = None) -> None:
        from .base import resolve_pending
        if stream.half is not None:
            raise RuntimeError("a post-norm block does not take half-normed rows")
        if stream.pending is not None:                     # a block of another arrangement ran before this one
            from ..kernels import ops
            if isinstance(stream.pending, torch.Tensor):
                ops.scaled_add(stream.x, [(stream.pending, None)])
                stream.pending = None
            else:
                resolve_pending(stream)
            stream.cast = None
        for part, norm in ((self.mixer, self.mixer_norm), (self.feed_forward, self.feed_forward_norm)):
            if getattr(part, "absent", False):
                continue
            if not isinstance(norm, RMSNorm):
                raise TypeError("postnorm_residual: the norms are RMS norms")
            h = self._input(stream)
            branch = part.forward(h, ctx, cache) if part is self.mixer else part.forward(h, ctx)
            self._join(stream, branch, norm)


@BLOCKS.register("sandwich_residual")
class SandwichResidual(Block):
    """``x += norm1b(mixer(norm1(x))); x += norm2b(ffn(norm2(x)))``: every sublayer has a norm on its input and one on
    its output, all four RMS norms whose weight is one number or a vector kept in 32-bit (a norm with an ``offset``).
    A layer may have no feed-forward (kind "none").

    extras: ``depth_average`` (tensor name after the layer's prefix) and ``depth_index`` (how many layers ran before
    this one): with X_0 what the embedding gave and X_(j+1) the result of layer j, what leaves layer i is
    ``sum_(j=0..i+1) w[j] X_j`` with the layer's weights ``w`` [i + 2], not X_(i+1) itself.  The results live in one
    buffer of the stream (``ResidualStream.results``): layer i works in place on row i and leaves the next layer's
    input in row i + 1; X_0 stays where the embedding wrote it.

    One kernel per sublayer joins it to the stream: the output norm, the 32-bit add, after the layer's last sublayer
    the average, and the input norm of whatever reads the stream next (this layer's feed-forward, or the next layer's
    mixer when that is a block of this kind with the same eps), rounded to the activation type.

    extras also holds the PartSpecs of the two output norms, ``mixer_norm_out`` and ``feed_forward_norm_out``."""

    def configure(self, extras, env, prefix) -> None:
        from .base import NORMS, build_part
        super().configure(extras, env, prefix)
        self.mixer_norm_out = build_part(NORMS, self.extras["mixer_norm_out"], env, prefix)
        self.feed_forward_norm_out = build_part(NORMS, self.extras["feed_forward_norm_out"], env, prefix)

    def parts(self):
        return super().parts() + [self.mixer_norm_out, self.feed_forward_norm_out]

    def declare(self):
        from .spec import TensorDecl
        name = self.extras.get("depth_average")
        return [TensorDecl(self.prefix + name, (int(self.extras["depth_index"]) + 2,), init="ones")] if name else []

    def bind(self, tensors):
        name = self.extras.get("depth_average")
        self.depth_weights = tensors[self.prefix + name].contiguous() if name else None
        self.depth_index = int(self.extras.get("depth_index", 0))

    def kernel_libraries(self):
        return ["sandwich", "norm", "elementwise"]

    def _no_feed_forward(self) -> bool:
        return bool(getattr(self.feed_forward, "absent", False))

    def _gain(self, norm):
        """One number, or the norm's weight vector in 32-bit."""
        if isinstance(norm, RMSNorm) and norm.gain is not None:
            return norm.gain
        if isinstance(norm, RMSNorm) and norm.weight is not None:
            if norm.weight.dtype != torch.float32:
                norm.weight = norm.weight.to(torch.float32).contiguous()
            return norm.weight
        raise TypeError("sandwich_residual: the norms are RMS norms with a weight")

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheBinding,
                next_block: Optional[Block] = None) -> None:
        from ..kernels import ops, stream_ops
        from .base import resolve_pending
        if stream.half is not None:
            raise RuntimeError("a sandwich block does not take half-normed rows")
        if stream.pending is not None:                     # a block of another arrangement ran before this one
            if isinstance(stream.pending, torch.Tensor):
                ops.scaled_add(stream.x, [(stream.pending, None)])
                stream.pending = None
            else:
                resolve_pending(stream)
            stream.normed = None
        act = self.env.act_dtype
        T, h = stream.x.shape
        eps = self.mixer_norm.eps
        x_in = stream.x
        x_work = stream.x
        average = None
        if self.depth_weights is not None:
            i = self.depth_index
            if stream.results is None:
                if i != 0:
                    raise RuntimeError("the average over the layers' results starts at the first layer")
                stream.origin = stream.x
                # a row for every layer's result and one more for what leaves the last layer
                total = int(self.extras.get("depth_layers", 1))
                stream.results = torch.empty((total + 1, T, h), dtype=torch.float32, device=stream.x.device)
            if stream.results is None or i + 1 >= stream.results.shape[0]:
                raise RuntimeError("the average over the layers' results: more layers than the first one was told of")
            x_work = stream.results[i]
            average = (stream.origin, stream.results, i + 1, self.depth_weights, stream.results[i + 1])
        # the mixer's input: normed by the kernel that last changed the stream, or here
        if stream.normed is not None and stream.normed_by is self.mixer_norm:
            hin = stream.normed
        else:
            hin = self.mixer_norm.forward(x_in)
        stream.normed = stream.normed_by = None
        a = self.mixer.forward(hin, ctx, cache)
        last = self._no_feed_forward()
        nxt = next_block.mixer_norm if (isinstance(next_block, SandwichResidual) and next_block.mixer_norm.eps == eps
                                        and next_block.mixer_norm.weight is not None) else None

        def join(branch, norm, x_from, final: bool):
            follow = nxt if final else self.feed_forward_norm
            out = torch.empty((T, h), dtype=act, device=branch.device) if follow is not None else None
            stream_ops.gain_norm_join(branch, self._gain(norm), eps, x_from, x_work,
                                      average=average if final else None,
                                      next_gain=self._gain(follow) if follow is not None else None, next_out=out)
            return out

        out = join(a, self.mixer_norm_out, x_in, last)
        if not last:
            f = self.feed_forward.forward(out, ctx)
            out = join(f, self.feed_forward_norm_out, x_work, True)
        stream.x = average[4] if average is not None else x_work
        stream.cast = None
        if nxt is not None:
            stream.normed, stream.normed_by = out, nxt
