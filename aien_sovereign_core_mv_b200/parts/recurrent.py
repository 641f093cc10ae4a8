"""Mixers that keep a state of fixed size per request instead of keys and values."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels as K
from ..registry import register_mixer
from .base import CacheNeed, Mixer, RunBinding, StepContext
from .linear import linear


@register_mixer("decay_linear_attention")
class DecayLinearAttention(Mixer):
    """Linear attention with one decay per head: q = silu(W_q h), k = silu(W_k h) (heads x ``head_dim``), v = silu(W_v h)
    (heads x ``value_dim``); per head S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, with no other scale.  The
    heads together pass an RMS norm (plain weight ``norm``), are multiplied by sigmoid(W_g h) and projected by W_o.
    The state [heads, head_dim, value_dim] is float32, starts at zero and is carried in a state slot of the cache; the
    recurrence, its decay powers and the norm are float32 in both engine precisions.  One product makes q | k | v | g."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay: Sequence[float],
                 norm_eps: float = 1e-6, position=None):
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.decay_values = [float(d) for d in decay]
        if len(self.decay_values) != self.num_heads:
            raise ValueError(f"decay names {len(self.decay_values)} values for {self.num_heads} heads")
        if any(not (0.0 <= d <= 1.0) for d in self.decay_values):
            raise ValueError("every decay must lie in [0, 1]")
        self.norm_eps = float(norm_eps)
        self.qk_dim, self.v_dim = self.num_heads * self.head_dim, self.num_heads * self.value_dim
        self.w_in = self.w_o = self.norm_w = self.decay = None

    def param_shapes(self):
        H = self.hidden_size
        return {"q_proj": ((self.qk_dim, H), "matrix"), "k_proj": ((self.qk_dim, H), "matrix"), "v_proj": ((self.v_dim, H), "matrix"),
                "g_proj": ((self.v_dim, H), "matrix"), "o_proj": ((H, self.v_dim), "matrix"), "norm": ((self.v_dim,), "norm")}

    def bind(self, tensors):
        rows = [tensors[n] for n in ("q_proj", "k_proj", "v_proj", "g_proj")]
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.w_in = torch.cat(rows, dim=0).contiguous()                 # rows q | k | v | g
        self.w_o = tensors["o_proj"].contiguous()
        self.norm_w = tensors["norm"].contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.num_heads, self.head_dim, self.value_dim), state_dtype="float32")

    def workspace_bytes(self, lim):
        chunks = K.decay_linear_attention_scratch(lim.max_tokens, lim.max_seqs, self.num_heads, self.head_dim, self.value_dim) * 4
        return lim.max_tokens * ((2 * self.qk_dim + 2 * self.v_dim) * 4 + self.v_dim * (4 + lim.itemsize) + self.hidden_size * 4) + 8192 + chunks + K.PARTIALS_MAX_BYTES

    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding):
        T = ctx.num_tokens
        group = ctx.groups[run.group]
        state = group.storage["state"][run.slot]
        proj = linear(ctx, h, self.w_in, out_dtype=torch.float32)
        o = ctx.workspace.take((T, self.v_dim), torch.float32)
        scratch = None
        if not ctx.decode_only:                                         # portions of prompts: their chunks side by side
            n = K.decay_linear_attention_scratch(T, ctx.num_seqs, self.num_heads, self.head_dim, self.value_dim)
            scratch = ctx.workspace.take((n,), torch.float32)
        K.decay_linear_attention(proj, 0, self.qk_dim, 2 * self.qk_dim, self.decay, state, group.slot_map, ctx.q_start, ctx.positions,
                                 o, ctx.num_seqs, self.num_heads, self.head_dim, self.value_dim, scratch, single_tokens=ctx.decode_only)
        y = ctx.workspace.take((T, self.v_dim), ctx.dtype)
        K.gated_rmsnorm(o, proj[:, 2 * self.qk_dim + self.v_dim:], self.norm_w, self.norm_eps, y)
        return linear(ctx, y, self.w_o, out_dtype=torch.float32, may_defer_sum=True)     # the branch norm adds partial products


@register_mixer("gated_recurrence")
class GatedRecurrence(Mixer):
    """A gated recurrence over ``width`` channels whose gates read only the current token: z = sigmoid(W_z h + b_z),
    u = W_x h + b_x, candidate c = u + 1/2 where u >= 0 and sigmoid(u) where u < 0; S_t = (1 - z) S_(t-1) + z c element
    by element; output W_o (S_t * silu(W_g h)).  The state [width] is float32, starts at zero and is carried in a state
    slot of the cache; gates, candidate and state are float32 in both engine precisions.  One product makes z | u | g."""

    def __init__(self, hidden_size: int, width: int, bias: bool = True, position=None):
        self.hidden_size, self.width, self.bias = int(hidden_size), int(width), bool(bias)
        self.w_in = self.w_o = self.b_z = self.b_x = None

    def param_shapes(self):
        H, W = self.hidden_size, self.width
        shapes = {"z_proj": ((W, H), "matrix"), "x_proj": ((W, H), "matrix"), "g_proj": ((W, H), "matrix"), "o_proj": ((H, W), "matrix")}
        if self.bias:
            shapes.update({"z_bias": ((W,), "vector"), "x_bias": ((W,), "vector")})
        return shapes

    def bind(self, tensors):
        rows = [tensors[n] for n in ("z_proj", "x_proj", "g_proj")]
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.w_in = torch.cat(rows, dim=0).contiguous()                 # rows z | u | g
        self.w_o = tensors["o_proj"].contiguous()
        if self.bias:
            self.b_z, self.b_x = tensors["z_bias"].float().contiguous(), tensors["x_bias"].float().contiguous()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.width,), state_dtype="float32")

    def workspace_bytes(self, lim):
        return lim.max_tokens * (3 * self.width * 4 + self.width * lim.itemsize + self.hidden_size * 4) + 8192 + K.PARTIALS_MAX_BYTES

    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding):
        T, W = ctx.num_tokens, self.width
        group = ctx.groups[run.group]
        state = group.storage["state"][run.slot]
        proj = linear(ctx, h, self.w_in, out_dtype=torch.float32)
        y = ctx.workspace.take((T, W), ctx.dtype)
        K.gated_recurrence(proj, 0, W, 2 * W, self.b_z, self.b_x, state, group.slot_map, ctx.q_start, ctx.positions, y, ctx.num_seqs, W,
                           segments=not ctx.decode_only)
        return linear(ctx, y, self.w_o, out_dtype=torch.float32, may_defer_sum=True)     # the branch norm adds partial products


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    """The gated delta rule.  q = W_q h and k = W_k h (``num_qk_heads`` x ``head_dim``), v = W_v h (``num_heads`` x
    ``value_dim``; value head h uses q/k head h // (num_heads / num_qk_heads)); each passes a causal convolution over
    time per channel (``taps`` taps, weights [channels, taps], the last column the current token's) and silu; q and k
    become unit vectors per head, x / sqrt(sum x^2 + 1e-6), q also times head_dim^-1/2.  Per value head
    beta = sigmoid(W_b h) and the decay g = exp(-exp(A_log) * softplus(W_a h + dt_bias)), and then token by token
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.  Each head's o is divided by its root mean square,
    times the weight ``norm`` (``value_dim`` numbers shared by the heads), times silu(W_g h); then W_o.

    One float32 state slot per request holds the last taps-1 projected rows of q | k | v followed by S
    [num_heads, head_dim, value_dim].  Convolution, activations, unit norms, decay, beta, the recurrence and the output
    norm are float32 in both engine precisions.  One product makes q | k | v | g | b | a."""

    def __init__(self, hidden_size: int, num_heads: int, num_qk_heads: int, head_dim: int, value_dim: int, taps: int = 1,
                 norm_eps: float = 1e-6, position=None):
        self.hidden_size, self.num_heads, self.num_qk_heads = int(hidden_size), int(num_heads), int(num_qk_heads)
        self.head_dim, self.value_dim, self.taps, self.norm_eps = int(head_dim), int(value_dim), int(taps), float(norm_eps)
        if self.num_heads % self.num_qk_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_qk_heads {num_qk_heads}")
        if not (0 < self.head_dim <= 256):
            raise ValueError(f"head_dim {head_dim}: the delta-rule kernel keeps up to 256 rows of a state column in registers")
        if not (1 <= self.taps <= 8):
            raise ValueError(f"taps {taps}: the convolution kernels take 1 to 8")
        self.qk_dim, self.v_dim = self.num_qk_heads * self.head_dim, self.num_heads * self.value_dim
        self.channels = 2 * self.qk_dim + self.v_dim
        self.conv_floats = (self.taps - 1) * self.channels
        self.w_in = self.w_o = self.norm_w = self.a_log = self.dt_bias = None
        self.conv = {}

    def param_shapes(self):
        H, t, n = self.hidden_size, self.taps, self.num_heads
        return {"q_proj": ((self.qk_dim, H), "matrix"), "q_conv": ((self.qk_dim, t), "matrix"),
                "k_proj": ((self.qk_dim, H), "matrix"), "k_conv": ((self.qk_dim, t), "matrix"),
                "v_proj": ((self.v_dim, H), "matrix"), "v_conv": ((self.v_dim, t), "matrix"),
                "b_proj": ((n, H), "matrix"), "a_proj": ((n, H), "matrix"), "A_log": ((n,), "vector"), "dt_bias": ((n,), "vector"),
                "norm": ((self.value_dim,), "norm"), "g_proj": ((self.v_dim, H), "matrix"), "o_proj": ((H, self.v_dim), "matrix")}

    def bind(self, tensors):
        rows = [tensors[n] for n in ("q_proj", "k_proj", "v_proj", "g_proj", "b_proj", "a_proj")]
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.w_in = torch.cat(rows, dim=0).contiguous()                 # rows q | k | v | g | b | a
        self.w_o = tensors["o_proj"].contiguous()
        convs = [tensors[n] for n in ("q_conv", "k_conv", "v_conv")]
        if len({t.dtype for t in convs}) > 1:
            convs = [t.float() for t in convs]
        self.conv = {n: t.contiguous() for n, t in zip("qkv", convs)}
        self.norm_w = tensors["norm"].contiguous()
        self.a_log, self.dt_bias = tensors["A_log"].float().contiguous(), tensors["dt_bias"].float().contiguous()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.conv_floats + self.num_heads * self.head_dim * self.value_dim,), state_dtype="float32")

    def workspace_bytes(self, lim):
        n = 2 * self.qk_dim + 2 * self.v_dim + 2 * self.num_heads
        return lim.max_tokens * ((n + self.channels + 2 * self.num_heads + self.v_dim) * 4 + self.v_dim * lim.itemsize + self.hidden_size * 4) \
            + 8192 + K.PARTIALS_MAX_BYTES

    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding):
        T, n = ctx.num_tokens, self.num_heads
        group = ctx.groups[run.group]
        state = group.storage["state"][run.slot]                           # [slots + 1, conv | S]
        proj = linear(ctx, h, self.w_in, out_dtype=torch.float32)
        g_off = 2 * self.qk_dim + self.v_dim
        b_off = g_off + self.v_dim
        qkv = ctx.workspace.take((T, self.channels), torch.float32)
        gb = ctx.workspace.take((T, 2 * n), torch.float32)
        K.delta_conv_prepare(proj, 0, self.qk_dim, 2 * self.qk_dim, b_off, b_off + n, self.num_qk_heads, self.head_dim, n, self.value_dim,
                             self.conv["q"], self.conv["k"], self.conv["v"], self.taps, self.a_log, self.dt_bias, state, group.slot_map,
                             ctx.seq_of_token, ctx.q_start, ctx.positions, qkv, gb)
        o = ctx.workspace.take((T, self.v_dim), torch.float32)
        K.delta_rule(qkv, 0, self.qk_dim, 2 * self.qk_dim, gb, state, self.conv_floats, group.slot_map, ctx.q_start, ctx.positions, o,
                     ctx.num_seqs, n, self.num_qk_heads, self.head_dim, self.value_dim)
        y = ctx.workspace.take((T, self.v_dim), ctx.dtype)
        K.grouped_gated_rmsnorm(o, proj[:, g_off:g_off + self.v_dim], self.norm_w, self.norm_eps, y, self.value_dim, "silu")
        return linear(ctx, y, self.w_o, out_dtype=torch.float32, may_defer_sum=True)
