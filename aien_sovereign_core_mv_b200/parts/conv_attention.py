"""Grouped-query attention whose projections pass a short convolution over time, with a distance bias instead of a
rotation, a temperature per head and an output gate per head."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_mixer
from .base import CacheNeed, Mixer, RunBinding, StepContext
from .linear import linear


@register_mixer("conv_gated_attention")
class ConvGatedAttention(Mixer):
    """q = W_q h, k = W_k h, v = W_v h (``num_heads`` query heads, ``num_kv_heads`` key/value heads; keys of ``head_dim``,
    values of ``value_dim`` numbers), each followed by a causal convolution over time per channel with ``taps`` taps
    (weights [channels, taps], the last column is the current token's; zeros before the sequence's start).  Then the
    whole q row and the whole k row pass an RMS norm with a plain weight of the row's size (``qk_norm``), and every value
    head is divided by its root mean square (``value_norm``); keys and values are cached in that form.  The score of
    query i of head h against key j is  q.k * ``scale`` * temp[h] - slope_h * (i - j)  with a learned temperature per
    head (``temperature``) and the fixed slopes slope_h = 2^(-``slope_exponent`` * (h + 1) / num_heads)
    (``slope_exponent`` None: no bias); i sees j with 0 <= i - j < ``window`` (0: every j <= i); ordinary softmax.  Head
    h's output is multiplied by sigmoid(W_g h)_h (``gate``: one number per head) before W_o.

    ``own_cache`` False: the mixer has no key/value tensors and attends over the planes another run wrote.
    ``cache_window``: what the cache keeps (the widest window among the runs that read it; 0: everything).

    Between steps a request keeps, beside its pages, the last taps-1 projected rows of q (and k, v) in a float32 state
    slot.  Convolution, norms, scores, softmax and the gate are float32 in both engine precisions."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: Optional[int] = None,
                 scale: Optional[float] = None, window: int = 0, cache_window: Optional[int] = None, taps: int = 1,
                 qk_norm_eps: float = 1e-6, value_norm: bool = True, slope_exponent: Optional[float] = None,
                 temperature: bool = True, gate: bool = True, own_cache: bool = True, position=None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.value_dim = int(value_dim if value_dim is not None else head_dim)
        if not (0 < self.head_dim <= 256 and 0 < self.value_dim <= 256):
            raise ValueError(f"head sizes {self.head_dim} / {self.value_dim}: the attention kernels take sizes up to 256")
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        self.window = int(window or 0)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.window < 0 or (self.cache_window and (self.window == 0 or self.window > self.cache_window)):
            raise ValueError("a mixer cannot see further back than its cache keeps")
        self.taps = int(taps)
        if not (1 <= self.taps <= 8):
            raise ValueError(f"taps {taps}: the convolution kernels take 1 to 8")
        self.eps, self.value_norm = float(qk_norm_eps), bool(value_norm)
        self.slope_exponent = None if slope_exponent is None else float(slope_exponent)
        self.temperature, self.gate, self.own_cache = bool(temperature), bool(gate), bool(own_cache)
        self.q_dim, self.k_dim, self.v_dim = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.num_kv_heads * self.value_dim
        self.o_in = self.num_heads * self.value_dim
        self.channels = self.q_dim + (self.k_dim + self.v_dim if self.own_cache else 0)
        self.w_in = self.w_o = self.head_scale = self.slopes = None
        self.conv = {}
        self.q_norm = self.k_norm = None

    # ---- tensors
    def param_shapes(self):
        H, t = self.hidden_size, self.taps
        shapes = {"q_proj": ((self.q_dim, H), "matrix"), "q_conv": ((self.q_dim, t), "matrix"), "q_norm": ((self.q_dim,), "norm"),
                  "o_proj": ((H, self.o_in), "matrix")}
        if self.own_cache:
            shapes.update({"k_proj": ((self.k_dim, H), "matrix"), "k_conv": ((self.k_dim, t), "matrix"), "k_norm": ((self.k_dim,), "norm"),
                           "v_proj": ((self.v_dim, H), "matrix"), "v_conv": ((self.v_dim, t), "matrix")})
        if self.temperature:
            shapes["temp"] = ((self.num_heads,), "norm")
        if self.gate:
            shapes["g_proj"] = ((self.num_heads, H), "matrix")
        return shapes

    def bind(self, tensors):
        rows = [tensors["q_proj"]] + ([tensors["k_proj"], tensors["v_proj"]] if self.own_cache else []) + ([tensors["g_proj"]] if self.gate else [])
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.w_in = torch.cat(rows, dim=0).contiguous()                 # rows q (| k | v) (| g)
        self.w_o = tensors["o_proj"].contiguous()
        names = ["q"] + (["k", "v"] if self.own_cache else [])
        convs = [tensors[f"{n}_conv"] for n in names]
        if len({t.dtype for t in convs}) > 1:
            convs = [t.float() for t in convs]
        self.conv = {n: t.contiguous() for n, t in zip(names, convs)}
        norms = [tensors["q_norm"]] + ([tensors["k_norm"]] if self.own_cache else [])
        if len({t.dtype for t in norms}) > 1:
            norms = [t.float() for t in norms]
        self.q_norm = norms[0].contiguous()
        self.k_norm = norms[1].contiguous() if self.own_cache else None
        dev = self.w_o.device
        self.head_scale = tensors["temp"].float().contiguous() if self.temperature else None      # the score is float32
        if self.slope_exponent is not None:
            n = self.num_heads
            self.slopes = torch.tensor([2.0 ** (-self.slope_exponent * (h + 1) / n) for h in range(n)], dtype=torch.float32, device=dev)

    def cache_need(self):
        planes = (("k", (self.num_kv_heads, self.head_dim)), ("v", (self.num_kv_heads, self.value_dim)))
        if self.cache_window > 0:
            return CacheNeed("window", self.cache_window, planes)
        return CacheNeed("full", 0, planes)

    def state_need(self):
        if self.taps == 1:
            return None
        return CacheNeed("state", state_shape=((self.taps - 1) * self.channels,), state_dtype="float32")

    def workspace_bytes(self, lim):
        n = self.w_in.shape[0] if self.w_in is not None else self.channels + self.num_heads
        return lim.max_tokens * (n * 4 + (self.q_dim + self.o_in) * lim.itemsize + self.hidden_size * 4) + 8192 + K.PARTIALS_MAX_BYTES \
            + K.biased_attention_workspace_bytes(lim, self.num_heads, self.value_dim, self.window)

    # ---- one step
    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding):
        T = ctx.num_tokens
        group = ctx.groups[run.group]
        k_cache, v_cache = group.storage["k"][run.slot], group.storage["v"][run.slot]
        proj = linear(ctx, h, self.w_in, out_dtype=torch.float32)                            # float32 into the convolution and norms
        state, slots = run.state_of(ctx, self) if self.taps > 1 else (None, ctx.q_start)
        q = ctx.workspace.take((T, self.q_dim), ctx.dtype)
        own = self.own_cache
        K.attn_conv_prepare(proj, 0, self.q_dim, self.q_dim + self.k_dim, self.q_dim, self.k_dim if own else 0, self.v_dim if own else 0,
                            self.conv["q"], self.conv.get("k"), self.conv.get("v"), self.taps, self.q_norm, self.k_norm, self.eps,
                            self.num_kv_heads, self.value_dim, self.value_norm, state, slots, ctx.seq_of_token, ctx.q_start, ctx.positions,
                            group.slot_map if own else None, k_cache if own else None, v_cache if own else None, q)
        gate = proj[:, self.channels:self.channels + self.num_heads] if self.gate else None
        out = ctx.workspace.take((T, self.o_in), ctx.dtype)
        K.biased_attention(ctx, q, k_cache, v_cache, group, out, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim,
                           self.window, self.scale, self.head_scale, self.slopes, gate)
        return linear(ctx, out, self.w_o, out_dtype=torch.float32, may_defer_sum=True)
