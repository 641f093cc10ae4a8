"""Routed feed-forward: a router, small experts, an optional shared expert."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_feed_forward
from .base import FeedForward, StepContext
from .linear import linear


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """Every token uses ``top`` of ``num_experts`` experts.  Router logits z = W_r h and the scores
    s = softmax(z) over all experts are float32.  With ``group_count`` > 1 the experts form that
    many equal groups of neighbours, a group scores its best expert and only experts of the best
    ``group_keep`` groups can be chosen.  The chosen experts' outputs are summed with their scores
    as weights (``renormalise``: divided by the sum of the chosen scores).  An expert is
    W_down f(W_up h) without biases and without a gate, f the gelu in its erf form ("gelu") or its
    tanh form ("gelu_tanh").  ``shared_ff`` > 0: one more expert of that hidden size runs for
    every token and is added.

    ``forward`` returns ``(parts, shared)``: the weighted outputs of the chosen experts as parts
    [top, T, H], one per choice (float32, or bfloat16 from the grouped tensor-core products), and
    the shared expert's output (or None); whoever takes the branch adds them in that order, in float32.  Expert tensors are stacked [E, ...] when they arrive.

    Further, each off unless asked for: ``correction``: a stored vector, one number per router output, is added to the
    scores for the choice only (the weights use the scores without it).  ``identity_experts`` n: the router has n more
    outputs behind the experts' whose "expert" returns its input (no tensors).  ``renormalise_eps`` is added to the sum of
    the chosen scores before the division.  ``shared_gate``: the shared expert's output is multiplied by sigmoid(w_sg . h),
    one number per token (tensor ``shared.gate`` [1, hidden]; its row rides with the router's product).  ``combined``:
    ``forward`` returns the one float32 tensor [T, H] that is the feed-forward's whole result instead of the pair.  Any of
    the first four needs ``combined`` (and no expert groups)."""

    def __init__(self, hidden_size: int, expert_ff: int, num_experts: int, top: int, group_count: int = 1, group_keep: int = 1,
                 shared_ff: int = 0, act: str = "gelu", shared_act: Optional[str] = None, renormalise: bool = False,
                 correction: bool = False, identity_experts: int = 0, renormalise_eps: float = 0.0, shared_gate: bool = False,
                 combined: bool = False):
        self.hidden_size, self.expert_ff, self.num_experts, self.top = int(hidden_size), int(expert_ff), int(num_experts), int(top)
        self.group_count, self.group_keep = int(group_count or 1), int(group_keep or 1)
        self.shared_ff = int(shared_ff or 0)
        if act not in K.ACT_KINDS or (shared_act or act) not in K.ACT_KINDS:
            raise ValueError(f"expert activation {act!r} / {shared_act!r}: one of {sorted(K.ACT_KINDS)}")
        self.act, self.shared_act = K.ACT_KINDS[act], K.ACT_KINDS[shared_act or act]
        self.renormalise = bool(renormalise)
        self.correction_on, self.identity = bool(correction), int(identity_experts or 0)
        self.renormalise_eps, self.shared_gate, self.combined = float(renormalise_eps or 0.0), bool(shared_gate), bool(combined)
        self.biased = self.correction_on or self.identity > 0 or self.renormalise_eps != 0.0 or self.shared_gate
        if self.biased and (not self.combined or self.group_count != 1):
            raise ValueError("a correction, identity experts, a renormalisation eps or a shared gate need combined=True and no expert groups")
        if self.identity < 0 or (self.shared_gate and not self.shared_ff):
            raise ValueError("identity_experts must not be negative; a shared gate needs a shared expert")
        self.outputs = self.num_experts + self.identity            # what the router scores
        self.correction = None
        E, G = self.num_experts, self.group_count
        if E <= 0 or G <= 0 or E % G:
            raise ValueError(f"{E} experts do not form {G} equal groups")
        if not (0 < self.group_keep <= G):
            raise ValueError(f"group_keep {self.group_keep} of {G} groups")
        if not (0 < self.top <= self.group_keep * (E // G) + self.identity):
            raise ValueError(f"top {self.top} exceeds the {self.group_keep * (E // G) + self.identity} experts that stay eligible")
        self.w_router = self.w_up = self.w_down = self.w_shared_up = self.w_shared_down = self.expert_count = None

    def param_shapes(self):
        H, F = self.hidden_size, self.expert_ff
        shapes = {"router": ((self.outputs, H), "matrix")}
        if self.correction_on:
            shapes["correction"] = ((self.outputs,), "fraction")
        for e in range(self.num_experts):
            shapes[f"experts.{e}.up"] = ((F, H), "matrix")
            shapes[f"experts.{e}.down"] = ((H, F), "matrix")
        if self.shared_ff:
            shapes["shared.up"] = ((self.shared_ff, H), "matrix")
            shapes["shared.down"] = ((H, self.shared_ff), "matrix")
            if self.shared_gate:
                shapes["shared.gate"] = ((1, H), "matrix")
        return shapes

    def bind(self, tensors):
        # Router logits are float32 sums.  A float32 engine keeps the matrix in float32 and multiplies on the CUDA
        # cores; a bfloat16 engine multiplies the stored bfloat16 matrix by the bfloat16 copy of the stream on the
        # products it uses everywhere (every product of two bfloat16 numbers is exact in float32; the sums are float32).
        self.w_router = tensors["router"].contiguous()
        if self.shared_gate:                                            # the gate's row rides behind the router's rows
            r, g = tensors["router"], tensors["shared.gate"]
            if r.dtype != g.dtype:
                r, g = r.float(), g.float()
            self.w_router = torch.cat([r, g.reshape(1, -1)], dim=0).contiguous()
        if self.correction_on:
            self.correction = tensors["correction"].float().contiguous()
        ups = [tensors[f"experts.{e}.up"] for e in range(self.num_experts)]
        downs = [tensors[f"experts.{e}.down"] for e in range(self.num_experts)]
        if len({t.dtype for t in ups + downs}) > 1:
            ups, downs = [t.float() for t in ups], [t.float() for t in downs]
        self.w_up = torch.stack(ups, dim=0).contiguous()                # [E, F, H]
        self.w_down = torch.stack(downs, dim=0).contiguous()            # [E, H, F]
        # choices per expert: the router's kernel counts, the plan of the grouped products reads and zeroes them again
        self.expert_count = torch.zeros(self.num_experts, dtype=torch.int32, device=self.w_up.device)
        if self.shared_ff:
            self.w_shared_up = tensors["shared.up"].contiguous()
            self.w_shared_down = tensors["shared.down"].contiguous()

    def workspace_bytes(self, lim):
        T = lim.max_tokens
        return T * ((self.outputs + 1) * 4 + 4 + self.hidden_size * 4 + self.top * 8 + self.top * self.expert_ff * lim.itemsize + self.top * self.hidden_size * 4
                    + self.shared_ff * lim.itemsize + self.hidden_size * 4) + 16384 + 2 * K.PARTIALS_MAX_BYTES \
            + K.moe_workspace_bytes(lim, self.num_experts, self.top, self.hidden_size, self.expert_ff)

    def forward(self, ctx: StepContext, h: torch.Tensor):
        T, top = ctx.num_tokens, self.top
        ws = ctx.workspace
        if h.dtype == torch.bfloat16 and self.w_router.dtype == torch.bfloat16:
            z = linear(ctx, h, self.w_router, out_dtype=torch.float32)
        else:
            z = ws.take((T, self.w_router.shape[0]), torch.float32)
            K.gemm_simple(h, self.w_router, z)                          # float32 operands, float32 sums
        ids = ws.take((T, top), torch.int32)
        wts = ws.take((T, top), torch.float32)
        counts = self.expert_count if K.moe_takes_grouped(h, self.w_up, self.w_down) else None
        w_same = None
        if self.biased:
            w_same = ws.take((T,), torch.float32) if self.identity else None
            K.moe_route_biased(z, self.outputs, self.num_experts, top, self.renormalise, self.renormalise_eps, self.correction, ids, wts,
                               w_same, counts)
        else:
            K.moe_route(z, self.group_count, self.group_keep, top, self.renormalise, ids, wts, counts)
        parts = K.moe_experts(ctx, h, self.w_up, self.w_down, ids, wts, top, self.act, counts)
        shared = None
        if self.shared_ff:
            a = linear(ctx, h, self.w_shared_up, act=self.shared_act)          # the activation in the product's epilogue
            # beside bfloat16 routed parts (the grouped products) the shared expert's output is bfloat16 too; else float32
            shared = linear(ctx, a, self.w_shared_down, out_dtype=torch.bfloat16 if counts is not None else torch.float32, may_defer_sum=True)
        if self.combined:
            out = ws.take((T, self.hidden_size), torch.float32)
            K.routed_combine(parts, h if w_same is not None else None, w_same, shared, z[:, self.outputs] if self.shared_gate else None, out)
            return out
        return parts, shared
