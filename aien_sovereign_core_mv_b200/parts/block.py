"""Arrangements of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Optional

import torch

from ..registry import register_block
from .. import kernels as K
from .base import Block, FeedForward, Mixer, Norm, Part, Prenormed, RunBinding, ScaledSum, StepContext, StreamCopy, add_to_residual


@register_block("prenorm")
class PreNormBlock(Block):
    """x -> norm -> mixer -> +x -> norm -> feed-forward -> +x
    (crates/aien-inference-abi/src/weights.rs:290-365).  Each residual sum is carried as a
    pending ``delta`` and added inside the next norm kernel; or, where the norm and the parts
    around it allow (``Norm.sink``), the product that ends a branch adds it and the product that
    follows finishes the norm, and no norm kernel runs between them."""

    norm_slots = ("norm_in", "norm_post")
    chains_norm = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norm_in: Norm, norm_post: Norm):
        self.mixer, self.feed_forward, self.norm_in, self.norm_post = mixer, feed_forward, norm_in, norm_post

    def parts(self):
        return {"norm_in": self.norm_in, "mixer": self.mixer, "norm_post": self.norm_post, "feed_forward": self.feed_forward}

    def workspace_bytes(self, lim):
        return sum(p.workspace_bytes(lim) for p in self.parts().values())

    def first_norm(self):
        return self.norm_in

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, run: RunBinding, next_norm: Optional[Norm] = None):
        h = self.norm_in.forward(ctx, x, delta)
        if isinstance(h, Prenormed) and not self.mixer.takes_prenormed:
            h = h.materialise(ctx)
        sink = self.norm_post.sink(ctx, x) if self.mixer.feeds_residual else None
        a = self.mixer.forward(ctx, h, run, sink=sink) if sink is not None else self.mixer.forward(ctx, h, run)
        h2 = self.norm_post.forward(ctx, x, a)
        if isinstance(h2, Prenormed) and not self.feed_forward.takes_prenormed:
            h2 = h2.materialise(ctx)
        sink = next_norm.sink(ctx, x) if (next_norm is not None and self.feed_forward.feeds_residual) else None
        return self.feed_forward.forward(ctx, h2, sink=sink) if sink is not None else self.feed_forward.forward(ctx, h2)


@register_block("branchnorm")
class BranchNormBlock(Block):
    """x -> x + norm_mixer(mixer(x)) -> x + norm_ff(feed_forward(x)): the sublayers read the
    stream itself and each norm stands on its sublayer's *output*.  Every sum is made here, in
    float32 (``Norm.add_normed``), so the block hands no pending sum on; it hands on the
    compute-dtype copy of the stream that the last sum's kernel wrote (``StreamCopy``), which the
    next block of this kind takes as its mixer's input.  A layer without a feed-forward is the
    kind "branchnorm_mixer"."""

    norm_slots = ("norm_mixer", "norm_ff")

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_mixer: Norm, norm_ff: Optional[Norm] = None):
        if (feed_forward is None) != (norm_ff is None):
            raise ValueError("a branch-norm block has a feed-forward and its norm, or neither")
        self.mixer, self.feed_forward, self.norm_mixer, self.norm_ff = mixer, feed_forward, norm_mixer, norm_ff

    def parts(self):
        out = {"norm_mixer": self.norm_mixer, "mixer": self.mixer}
        if self.feed_forward is not None:
            out["norm_ff"] = self.norm_ff
            out["feed_forward"] = self.feed_forward
        return out

    def workspace_bytes(self, lim):
        return sum(p.workspace_bytes(lim) for p in self.parts().values()) + 3 * (lim.max_tokens * self.norm_mixer.size * lim.itemsize + 256)

    def _stream_copy(self, ctx: StepContext, x: torch.Tensor, delta):
        if isinstance(delta, StreamCopy):
            return delta.h
        add_to_residual(ctx, x, delta)             # whatever another kind of block left pending
        if ctx.dtype == torch.float32:
            return x
        h = ctx.workspace.take(tuple(x.shape), ctx.dtype)
        K.convert(x, h)
        return h

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, run: RunBinding):
        h = self._stream_copy(ctx, x, delta)
        a = self.mixer.forward(ctx, h, run)
        h = self.norm_mixer.add_normed(ctx, x, a, want_copy=True)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(ctx, h)
            a, b = f if isinstance(f, tuple) else (f, None)          # a routed feed-forward returns (routed parts, shared output)
            h = self.norm_ff.add_normed(ctx, x, a, b, want_copy=True)
        return StreamCopy(h)


@register_block("branchnorm_mixer")
class BranchNormMixerBlock(BranchNormBlock):
    """The branch-norm block of a layer that has no feed-forward: x -> x + norm_mixer(mixer(x))."""

    norm_slots = ("norm_mixer",)

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_mixer: Norm):
        if feed_forward is not None:
            raise ValueError("the block kind 'branchnorm_mixer' takes no feed-forward")
        super().__init__(mixer, None, norm_mixer, None)


class BranchScale(Part):
    """One learned number per channel that multiplies a branch's result before the residual sum (``weight`` [hidden]),
    with a constant factor folded in when the tensor arrives (float32)."""

    def __init__(self, size: int, mult: float = 1.0):
        self.size, self.mult = int(size), float(mult)
        self.vec: Optional[torch.Tensor] = None

    def param_shapes(self):
        return {"weight": ((self.size,), "norm")}

    def bind(self, tensors):
        self.vec = (tensors["weight"].float() * self.mult).contiguous()


@register_block("prenorm_scaled")
class ScaledPreNormBlock(Block):
    """x <- x + m * s_1 * mixer(norm_in(x)); x <- x + m * s_2 * ff(norm_post(x)): the pre-norm layer with a constant
    ``residual_mult`` m and, with ``layer_scale``, a learned vector per branch (tensors ``scale_mixer.weight`` and
    ``scale_ff.weight``) that multiplies the branch's result element by element before the sum.  Every sum is float32 and
    is made by the kernel that also makes the next norm (``kernels.scaled_add_rmsnorm``); the feed-forward's sum is handed
    on as a ``ScaledSum`` for the next block's first norm.  A layer without a feed-forward is the kind
    "prenorm_scaled_mixer".  The norms are RMS norms with a plain weight."""

    norm_slots = ("norm_in", "norm_post")

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_in: Norm, norm_post: Optional[Norm] = None,
                 residual_mult: float = 1.0, layer_scale: bool = False):
        if (feed_forward is None) != (norm_post is None):
            raise ValueError("a scaled pre-norm block has a feed-forward and its norm, or neither")
        for n in (norm_in, norm_post):
            if n is not None and (not hasattr(n, "weight") or not hasattr(n, "eps") or getattr(n, "weight_offset", 0.0) != 0.0):
                raise ValueError("the norms of a scaled pre-norm block are RMS norms with a plain weight")
        self.mixer, self.feed_forward, self.norm_in, self.norm_post = mixer, feed_forward, norm_in, norm_post
        self.mult, self.layer_scale = float(residual_mult), bool(layer_scale)
        self.scale_mixer = BranchScale(norm_in.size, self.mult) if self.layer_scale else None
        self.scale_ff = BranchScale(norm_in.size, self.mult) if (self.layer_scale and feed_forward is not None) else None
        self._const: Optional[torch.Tensor] = None

    def parts(self):
        out = {"norm_in": self.norm_in, "mixer": self.mixer}
        if self.scale_mixer is not None:
            out["scale_mixer"] = self.scale_mixer
        if self.feed_forward is not None:
            out.update({"norm_post": self.norm_post, "feed_forward": self.feed_forward})
            if self.scale_ff is not None:
                out["scale_ff"] = self.scale_ff
        return out

    def workspace_bytes(self, lim):
        return sum(p.workspace_bytes(lim) for p in self.parts().values()) + 2 * (lim.max_tokens * self.norm_in.size * lim.itemsize + 256)

    def first_norm(self):
        return self.norm_in

    def _vec(self, scale: Optional[BranchScale], device) -> Optional[torch.Tensor]:
        if scale is not None:
            return scale.vec
        if self.mult == 1.0:
            return None
        if self._const is None:
            self._const = torch.full((self.norm_in.size,), self.mult, dtype=torch.float32, device=device)
        return self._const

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, run: RunBinding):
        d = vec = bias = None
        if isinstance(delta, ScaledSum):
            d, vec, bias = delta.delta, delta.vec, delta.bias
        else:
            add_to_residual(ctx, x, delta)             # whatever another kind of block left pending
        h = ctx.workspace.take(tuple(x.shape), ctx.dtype)
        K.scaled_add_rmsnorm(x, d, vec, bias, self.norm_in.weight, self.norm_in.eps, h)
        a = self.mixer.forward(ctx, h, run)
        if self.feed_forward is None:
            return ScaledSum(a, self._vec(self.scale_mixer, x.device), None)
        h2 = ctx.workspace.take(tuple(x.shape), ctx.dtype)
        K.scaled_add_rmsnorm(x, a, self._vec(self.scale_mixer, x.device), None, self.norm_post.weight, self.norm_post.eps, h2)
        f = self.feed_forward.forward(ctx, h2)
        return ScaledSum(f, self._vec(self.scale_ff, x.device), self.feed_forward.pending_bias())


@register_block("prenorm_scaled_mixer")
class ScaledPreNormMixerBlock(ScaledPreNormBlock):
    """The scaled pre-norm block of a layer that has no feed-forward."""

    norm_slots = ("norm_in",)

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_in: Norm, residual_mult: float = 1.0,
                 layer_scale: bool = False):
        if feed_forward is not None:
            raise ValueError("the block kind 'prenorm_scaled_mixer' takes no feed-forward")
        super().__init__(mixer, None, norm_in, None, residual_mult, layer_scale)
