"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_mixer
from .base import CacheNeed, Mixer, Position, Prenormed, ResidualSink, RunBinding, StepContext
from .linear import linear, linear_into_residual, linear_prenormed


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    """q/k/v projection (one product over the stacked rows q|k|v), optional per-head RMSNorm of
    q and k before rotation, rotation, write of k and v into the token's cache slot, causal
    attention over the request's pages (optionally only the last ``window`` keys), output
    projection.  Formulas: crates/aien-inference-abi/src/transformer_backend.rs:1229-1319 and
    src/backend.rs:311-379; the stacked q|k|v rows follow src/resident.rs:284-288.

    A run that does not write its cache (``run.writes == False``) projects q only and attends
    over the planes another run filled."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position: Position,
                 qk_norm: bool = False, qk_norm_eps: float = 1e-6, window: int = 0, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take even sizes up to 256")
        if getattr(position, "pairing", "halves") != "halves":
            raise ValueError("this mixer rotates halves (i with i + d/2); interleaved pairs belong to 'chunked_sink_attention'")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.position = position
        self.qk_norm, self.qk_norm_eps = bool(qk_norm), float(qk_norm_eps)
        self.window = int(window or 0)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_dim, self.kv_dim = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    # ---- tensors
    def param_shapes(self):
        H = self.hidden_size
        shapes = {
            "q_proj": ((self.q_dim, H), "matrix"), "k_proj": ((self.kv_dim, H), "matrix"),
            "v_proj": ((self.kv_dim, H), "matrix"), "o_proj": ((H, self.q_dim), "matrix"),
        }
        if self.qk_norm:
            shapes["q_norm"] = ((self.head_dim,), "norm")
            shapes["k_norm"] = ((self.head_dim,), "norm")
        return shapes

    def bind(self, tensors):
        q, k, v = tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()       # rows q | k | v
        self.w_o = tensors["o_proj"].contiguous()
        if self.qk_norm:
            qn, kn = tensors["q_norm"], tensors["k_norm"]
            if qn.dtype != kn.dtype:
                qn, kn = qn.float(), kn.float()
            self.q_norm_w, self.k_norm_w = qn.contiguous(), kn.contiguous()

    def cache_need(self):
        return CacheNeed.keys_and_values("window" if self.window > 0 else "full", self.window, self.num_kv_heads, self.head_dim)

    def workspace_bytes(self, lim):
        return lim.max_tokens * (2 * self.q_dim + 2 * self.kv_dim + self.q_dim + self.hidden_size) * lim.itemsize + 4096 \
            + 8 * K.GEMV_MAX_ROWS * (self.q_dim + 2 * self.kv_dim + self.hidden_size) * 4 + 2 * K.PARTIALS_MAX_BYTES \
            + K.attention_workspace_bytes(lim, self.num_heads, self.head_dim) + K.FUSED_NORM_SCRATCH_BYTES(self.hidden_size)

    # ---- one step
    takes_prenormed = True
    feeds_residual = True

    def _project(self, ctx: StepContext, h, w: torch.Tensor) -> torch.Tensor:
        if isinstance(h, Prenormed):
            y = linear_prenormed(ctx, h, w)
            if y is not None:
                return y
            h = h.materialise(ctx)
        return linear(ctx, h, w, may_defer_sum=True)

    def forward(self, ctx: StepContext, h, run: RunBinding, sink: Optional[ResidualSink] = None):
        T = ctx.num_tokens
        group = ctx.groups[run.group]
        k_cache, v_cache = group.storage["k"][run.slot], group.storage["v"][run.slot]     # [tokens, nkv, hd] each
        if run.writes:
            qkv = self._project(ctx, h, self.w_qkv)
            q, k, v = qkv[..., :self.q_dim], qkv[..., self.q_dim:self.q_dim + self.kv_dim], qkv[..., self.q_dim + self.kv_dim:]
        else:
            q = self._project(ctx, h, self.w_qkv[:self.q_dim])
            k = v = None
        rot = self.position.rotary(ctx)
        cos, sin, rdim = rot if rot is not None else (None, None, 0)
        if (K._FORCE_ATTN == "fused" and ctx.decode_only and run.writes and q.dim() == 2 and rot is not None
                and K.decode_attention_supports(q, k_cache, self.num_heads, self.num_kv_heads, self.head_dim)):
            # One launch: q/k norm, rotation, cache write and attention.  Opt-in (AIEN_B200_ATTENTION=fused):
            # measured on the Qwen3-8B shape it equals the two launches at batch 1 and loses at batch 8
            # and 64, where every chunk's CTA repeats the q work.
            out = ctx.workspace.take((T, self.q_dim), ctx.dtype)
            K.paged_attention_decode_fused(ctx, q, k, v, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, cos, sin, rdim, group,
                                           k_cache, v_cache, out, self.num_heads, self.num_kv_heads, self.head_dim,
                                           self.window, self.scale)
            return linear(ctx, out, self.w_o, may_defer_sum=True)
        q_out = ctx.workspace.take((T, self.q_dim), ctx.dtype) if q.dim() == 3 else q
        K.qk_norm_rope_kv_write(q, k, v, self.head_dim, self.q_norm_w, self.k_norm_w if k is not None else None,
                                self.qk_norm_eps, cos, sin, rdim,
                                group.slot_map if k is not None else None,
                                k_cache if k is not None else None, v_cache if k is not None else None, q_out=q_out)
        if rot is None:
            self.position.apply(ctx, q_out, group, run)
        out = ctx.workspace.take((T, self.q_dim), ctx.dtype)
        K.paged_attention(ctx, q_out, k_cache, v_cache, group, out, self.num_heads, self.num_kv_heads, self.head_dim,
                          self.window, self.scale)
        return linear_into_residual(ctx, out, self.w_o, sink) or linear(ctx, out, self.w_o, may_defer_sum=True)


from .state_space import BranchMixer            # noqa: E402  (the two-products form this mixer follows)


@register_mixer("gated_capped_attention")
class GatedCappedAttention(BranchMixer):
    """Grouped-query attention with a capped score and an output gate.  q = W_q h (``num_heads`` heads of ``head_dim``),
    k = W_k h, v = W_v h (``num_kv_heads`` heads; values of ``value_dim`` numbers), no biases; q and k are rotated over the
    dimensions the position part names (halves: i with i + d/2; the rest pass unchanged); score = q.k * ``scale``, then
    (``softcap`` c > 0) c * tanh(score / c); causal, optionally only the last ``window`` keys; ordinary softmax.  The
    concatenated heads are multiplied element by element by sigmoid(W_g h) (``gate``) and projected by W_o.  One product
    makes q | k | v | g.  Rotation, scores, softmax and the gate are float32 in both engine precisions."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position: Position,
                 value_dim: Optional[int] = None, scale: Optional[float] = None, softcap: float = 0.0, window: int = 0, gate: bool = True):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.value_dim = int(value_dim if value_dim is not None else head_dim)
        if not (0 < self.head_dim <= 256 and 0 < self.value_dim <= 256):
            raise ValueError(f"head sizes {self.head_dim} / {self.value_dim}: the attention kernels take sizes up to 256")
        if getattr(position, "pairing", "halves") != "halves":
            raise ValueError("this mixer rotates halves (i with i + d/2)")
        self.position = position
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        self.softcap, self.window, self.gate = float(softcap or 0.0), int(window or 0), bool(gate)
        if self.softcap < 0.0 or self.window < 0:
            raise ValueError("softcap and window must not be negative")
        self.q_dim, self.k_dim, self.v_dim = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.num_kv_heads * self.value_dim
        self.out_cols = self.num_heads * self.value_dim
        self.in_rows = self.q_dim + self.k_dim + self.v_dim + (self.out_cols if self.gate else 0)
        self.w_in = self.w_o = None

    def param_shapes(self):
        H = self.hidden_size
        shapes = {"q_proj": ((self.q_dim, H), "matrix"), "k_proj": ((self.k_dim, H), "matrix"), "v_proj": ((self.v_dim, H), "matrix"),
                  "o_proj": ((H, self.out_cols), "matrix")}
        if self.gate:
            shapes["g_proj"] = ((self.out_cols, H), "matrix")
        return shapes

    def bind(self, tensors):
        rows = [tensors[n] for n in ("q_proj", "k_proj", "v_proj")] + ([tensors["g_proj"]] if self.gate else [])
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.w_in = torch.cat(rows, dim=0).contiguous()                 # rows q | k | v | g
        self.w_o = tensors["o_proj"].contiguous()

    def in_weight(self):
        return self.w_in

    def out_weight(self):
        return self.w_o

    def cache_need(self):
        planes = (("k", (self.num_kv_heads, self.head_dim)), ("v", (self.num_kv_heads, self.value_dim)))
        return CacheNeed("window" if self.window > 0 else "full", self.window, planes)

    def store(self, ctx, run):
        group = ctx.groups[run.group]
        return group, group.storage["k"][run.slot], group.storage["v"][run.slot]

    def core_workspace_bytes(self, lim):
        return lim.max_tokens * (self.q_dim + self.out_cols) * lim.itemsize + 1024 \
            + K.capped_attention_workspace_bytes(lim, self.num_heads, self.value_dim)

    def core(self, ctx, proj, col0, store, out, out_col0, mult):
        T = ctx.num_tokens
        group, k_cache, v_cache = store
        rot = self.position.rotary(ctx)
        cos, sin, rdim = rot if rot is not None else (None, None, 0)
        q = ctx.workspace.take((T, self.q_dim), ctx.dtype)
        K.rope_halves_value_write(proj, col0, col0 + self.q_dim, col0 + self.q_dim + self.k_dim, self.num_heads, self.num_kv_heads,
                                  self.head_dim, self.value_dim, cos, sin, rdim, group.slot_map, q, k_cache, v_cache)
        dst = out[:, out_col0:out_col0 + self.out_cols]
        gated = self.gate or mult != 1.0
        o = ctx.workspace.take((T, self.out_cols), ctx.dtype) if gated else dst
        K.capped_attention(ctx, q, k_cache, v_cache, group, o, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim,
                           self.window, self.scale, self.softcap)
        if self.gate:
            g0 = col0 + self.q_dim + self.k_dim + self.v_dim
            K.sigmoid_gate(o, proj[:, g0:g0 + self.out_cols], mult, dst)
        elif gated:
            K.scale_rows(o, mult, dst)
