"""RMSNorm with the residual sum fused in front of it."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_norm
from .base import Norm, NormedStream, Prenormed, ResidualSink, ScaledSum, StepContext, StreamCopy, add_to_residual

# AIEN_B200_FUSED_NORM=0 keeps every norm in its own kernel
_FUSE = __import__("os").environ.get("AIEN_B200_FUSED_NORM", "1").strip() not in ("0", "off", "no")


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """h = x * (1/sqrt(mean(x^2) + eps)) * w over the last axis
    (crates/aien-inference-abi/src/tensor.rs:94-110).  The sum of squares and the scale are
    float32; x is the float32 residual stream and is updated in place when ``delta`` is given.

    ``weight_offset``: the stored vector lies around zero and the norm multiplies by
    ``weight_offset + w``; the sum is made once, in float32, when the tensor arrives.

    Besides the norm of what a sublayer reads (``forward``) it offers the norm of what a sublayer
    returns (``add_normed``: x += norm(branch output)) and the norm of the stream in place
    (``norm_stream``: the embedding's norm)."""

    def __init__(self, size: int, eps: float, weight_offset: float = 0.0):
        self.size = int(size)
        self.eps = float(eps)
        self.weight_offset = float(weight_offset)
        self.weight: Optional[torch.Tensor] = None

    def param_shapes(self):
        return {"weight": ((self.size,), "norm_offset" if self.weight_offset != 0.0 else "norm")}

    def bind(self, tensors):
        w = tensors["weight"]
        self.weight = (w.float() + self.weight_offset).contiguous() if self.weight_offset != 0.0 else w.contiguous()

    def workspace_bytes(self, lim):
        return lim.max_tokens * self.size * lim.itemsize + 256

    def _copy_for(self, ctx: StepContext, x: torch.Tensor, want_copy: bool):
        return ctx.workspace.take(tuple(x.shape), ctx.dtype) if (want_copy and ctx.dtype != torch.float32) else None

    def add_normed(self, ctx: StepContext, x: torch.Tensor, a, b=None, want_copy: bool = False):
        h = self._copy_for(ctx, x, want_copy)
        K.branch_norm_add(x, a, self.weight, self.eps, b=b, h=h)
        return (h if h is not None else x) if want_copy else None

    def add_normed_scaled(self, ctx: StepContext, x: torch.Tensor, a, mult: float, then=None, want_copy: bool = False):
        """x += mult * norm(a) in float32, and in the same kernel what the next sublayer reads: ``then`` (a norm of this
        kind) gives then(x) in the compute dtype; ``want_copy`` the stream's compute-dtype copy (x itself in float32).
        Returns that tensor, or None when neither was asked.  A ``then`` of another kind is applied by its own kernel."""
        fused = then is not None and type(then) is RMSNorm
        h = None
        if fused or (want_copy and ctx.dtype != torch.float32):
            h = ctx.workspace.take(tuple(x.shape), ctx.dtype)
        K.post_norm_add(x, a, self.weight, self.eps, mult, then.weight if fused else None, then.eps if fused else 0.0, h)
        if fused:
            return h
        if then is not None:
            return then.forward(ctx, x, None)
        return (h if h is not None else x) if want_copy else None

    def norm_stream(self, ctx: StepContext, x: torch.Tensor, want_copy: bool = False):
        """x = norm(x) in place; with ``want_copy`` also the compute-dtype copy (x itself in float32)."""
        h = self._copy_for(ctx, x, want_copy)
        K.stream_norm_inplace(x, self.weight, self.eps, h=h)
        return (h if h is not None else x) if want_copy else None

    def sink(self, ctx: StepContext, x: torch.Tensor) -> Optional[ResidualSink]:
        if self.weight_offset != 0.0:
            return None                           # the spread-out form is kept to norms without an offset
        if not _FUSE or not K.small_step_products_fuse(ctx.dtype, ctx.num_tokens):
            return None
        return ResidualSink(x, self, self.weight, self.eps)

    def forward(self, ctx: StepContext, x: torch.Tensor, delta):
        if isinstance(delta, Prenormed):
            if delta.norm is self:
                return delta                      # the sum is in x already; the consumer finishes the norm
            delta = None                          # made for another norm: x is up to date, norm it here
        if isinstance(delta, NormedStream):
            if delta.norm is self:
                return delta.h                    # made by the kernel that wrote the last sum
            delta = None
        if isinstance(delta, StreamCopy):
            delta = None                          # nothing pending
        if isinstance(delta, ScaledSum):
            add_to_residual(ctx, x, delta)        # left by a block that scales its branches
            delta = None
        out = ctx.workspace.take(tuple(x.shape), ctx.dtype)
        K.add_rmsnorm(x, delta, self.weight, self.eps, out)
        return out
