"""A layer over several copies of the residual stream ("hyper-connections"), with an optional token shift in front of
the mixer."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_block
from .base import Block, CacheNeed, FeedForward, Mixer, Norm, Part, RunBinding, StepContext, add_to_residual


class StreamConnection(Part):
    """How one sublayer reads and writes ``streams`` copies x_1 .. x_n of the residual stream: it reads
    u = sum_s in[s] x_s and, with its output y, all copies change at once to x_t <- sum_s mix[s, t] x_s + out[t] y
    (``mix`` indexed [from, to]).  ``learned=False`` (one stream only) is the plain residual sum: in = out = mix = 1.
    The three tensors are kept as one float32 pack [in | out | mix] on the device."""

    def __init__(self, streams: int, learned: bool = True):
        self.streams, self.learned = int(streams), bool(learned)
        if not (1 <= self.streams <= 8):
            raise ValueError(f"streams {streams}: the stream kernels take 1 to 8 copies")
        if not self.learned and self.streams != 1:
            raise ValueError("several streams need their in / out / mix tensors")
        self.pack: Optional[torch.Tensor] = None

    def param_shapes(self):
        n = self.streams
        return {"in": ((n,), "norm"), "out": ((n,), "norm"), "mix": ((n, n), "near_identity")} if self.learned else {}

    def bind(self, tensors):
        self.pack = torch.cat([tensors["in"].float().reshape(-1), tensors["out"].float().reshape(-1),
                               tensors["mix"].float().reshape(-1)]).contiguous()

    def ensure(self, device) -> torch.Tensor:
        if self.pack is None:
            self.pack = torch.ones(3, dtype=torch.float32, device=device)
        return self.pack


class TokenShift(Part):
    """h <- h + (h' - h) * shift, element by element, h' being the token before's h as it was before this replacement
    (zeros for the first token of a sequence).  The last h of every request is a float32 state slot of ``size`` numbers."""

    def __init__(self, size: int):
        self.size = int(size)
        self.weight: Optional[torch.Tensor] = None

    def param_shapes(self):
        return {"weight": ((self.size,), "fraction")}

    def bind(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def state_need(self):
        return CacheNeed("state", state_shape=(self.size,), state_dtype="float32")


@dataclass
class PendingStreams:
    """What a block over several streams hands on: the output ``y`` of its last sublayer (a [T, H] tensor or float32
    partial products [P, T, H]) and the pack of that sublayer's connection; the write into the streams is still to be
    made.  The next block of this kind makes it inside its first kernel; the decoder's end asks :meth:`sum_rows`."""

    y: torch.Tensor
    pack: torch.Tensor

    def sum_rows(self, ctx: StepContext, x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
        """out[r] = the sum of the streams of row rows[r] after the pending write."""
        K.hc_sum_rows(x if x.dim() == 3 else x.unsqueeze(0), self.y, self.pack, rows, out)


@register_block("hyper")
class HyperBlock(Block):
    """Pre-norm layer over ``streams`` copies of the residual stream (float32 [streams, T, H]; [T, H] with one):
    for the mixer and then the feed-forward, u = sum_s in[s] x_s, y = sublayer(norm(u)), x_t <- sum_s mix[s, t] x_s
    + out[t] y.  With ``token_shift`` the mixer reads norm(u) shifted toward the token before (:class:`TokenShift`).
    One kernel makes the write of the sublayer before, the read u and its norm (``kernels.hc_norm``); in a step of single
    tokens it makes the shift too.  With one stream and ``learned=False`` this is the plain pre-norm layer.  A layer
    without a feed-forward is the kind "hyper_mixer"."""

    norm_slots = ("norm_in", "norm_post")
    takes_streams = True

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_in: Norm, norm_post: Optional[Norm] = None,
                 streams: int = 1, learned: bool = True, token_shift: bool = False):
        if (feed_forward is None) != (norm_post is None):
            raise ValueError("a hyper block has a feed-forward and its norm, or neither")
        for norm in (norm_in, norm_post):
            if norm is not None and (not hasattr(norm, "eps") or getattr(norm, "weight_offset", 0.0) != 0.0):
                raise ValueError("the norms of a hyper block are RMS norms with a plain weight")
        self.mixer, self.feed_forward, self.norm_in, self.norm_post = mixer, feed_forward, norm_in, norm_post
        self.streams = int(streams)
        self.hc_mixer = StreamConnection(streams, learned)
        self.hc_ff = StreamConnection(streams, learned) if feed_forward is not None else None
        self.shift = TokenShift(norm_in.size) if token_shift else None

    def parts(self):
        out = {"norm_in": self.norm_in, "mixer": self.mixer}
        if self.hc_mixer.learned:
            out["hc_mixer"] = self.hc_mixer
        if self.feed_forward is not None:
            out.update({"norm_post": self.norm_post, "feed_forward": self.feed_forward})
            if self.hc_ff.learned:
                out["hc_ff"] = self.hc_ff
        if self.shift is not None:
            out["shift"] = self.shift
        return out

    def workspace_bytes(self, lim):
        H = self.norm_in.size
        return sum(p.workspace_bytes(lim) for p in self.parts().values()) + lim.max_tokens * H * (4 + 2 * lim.itemsize) + 1024

    def first_norm(self):
        return self.norm_in

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, run: RunBinding):
        T, H = ctx.num_tokens, self.norm_in.size
        x3 = x if x.dim() == 3 else x.unsqueeze(0)
        if x3.shape[0] != self.streams:
            raise ValueError(f"the block keeps {self.streams} streams and was given {x3.shape[0]}")
        y = prev = None
        if isinstance(delta, PendingStreams):
            y, prev = delta.y, delta.pack
        elif delta is not None:
            if self.streams != 1:
                raise ValueError("a block of another kind cannot hand a pending sum to several streams")
            add_to_residual(ctx, x, delta)
        ws = ctx.workspace
        pack1 = self.hc_mixer.ensure(x.device)
        if self.shift is None:
            h = ws.take((T, H), ctx.dtype)
            K.hc_norm(x3, y, prev, pack1, self.norm_in.weight, self.norm_in.eps, h)
        else:
            state, slots = run.state_of(ctx, self.shift)
            if ctx.decode_only:                       # every row's predecessor is its request's slot: one kernel
                h = ws.take((T, H), ctx.dtype)
                K.hc_norm(x3, y, prev, pack1, self.norm_in.weight, self.norm_in.eps, h, self.shift.weight, state, slots, ctx.positions)
            else:
                hn = ws.take((T, H), torch.float32)
                K.hc_norm(x3, y, prev, pack1, self.norm_in.weight, self.norm_in.eps, hn)
                h = ws.take((T, H), ctx.dtype)
                K.token_shift(hn, self.shift.weight, state, slots, ctx.seq_of_token, ctx.q_start, ctx.positions, h)
        a = self.mixer.forward(ctx, h, run)
        if self.feed_forward is None:
            return PendingStreams(a, pack1)
        pack2 = self.hc_ff.ensure(x.device)
        h2 = ws.take((T, H), ctx.dtype)
        K.hc_norm(x3, a, pack1, pack2, self.norm_post.weight, self.norm_post.eps, h2)
        return PendingStreams(self.feed_forward.forward(ctx, h2), pack2)


@register_block("hyper_mixer")
class HyperMixerBlock(HyperBlock):
    """The hyper block of a layer that has no feed-forward."""

    norm_slots = ("norm_in",)

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_in: Norm, streams: int = 1, learned: bool = True,
                 token_shift: bool = False):
        if feed_forward is not None:
            raise ValueError("the block kind 'hyper_mixer' takes no feed-forward")
        super().__init__(mixer, None, norm_in, None, streams, learned, token_shift)
