"""State-space mixers: the selective scan with a state per channel, the state-space-duality form with a state matrix per
head, and a mixer that runs two mixers side by side on the same input."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import make_part, register_mixer
from .base import CacheNeed, Mixer, RunBinding, StepContext
from .linear import linear


def _stack(rows):
    if len({t.dtype for t in rows}) > 1:
        rows = [t.float() for t in rows]
    return torch.cat(rows, dim=0).contiguous()


class BranchMixer(Mixer):
    """A mixer of the form W_o core(W_in h) whose two products can be shared with a neighbour that reads the same h:
    ``in_weight()`` [in_rows, hidden] and ``out_weight()`` [hidden, out_cols] are the products' matrices, and
    ``core(ctx, proj, col0, store, out, out_col0, mult)`` turns columns col0 .. col0 + in_rows of the float32 rows ``proj``
    into columns out_col0 .. out_col0 + out_cols of ``out`` (compute dtype), times the constant ``mult``.  ``store(ctx,
    run)`` finds what the core keeps between steps when the mixer stands alone.  ``forward`` is the two products around
    the core."""

    in_rows = 0
    out_cols = 0

    def in_weight(self) -> torch.Tensor:
        raise NotImplementedError

    def out_weight(self) -> torch.Tensor:
        raise NotImplementedError

    def store(self, ctx: StepContext, run: RunBinding):
        raise NotImplementedError

    def core(self, ctx: StepContext, proj: torch.Tensor, col0: int, store, out: torch.Tensor, out_col0: int, mult: float) -> None:
        raise NotImplementedError

    def core_workspace_bytes(self, lim) -> int:
        return 0

    def workspace_bytes(self, lim):
        return lim.max_tokens * (self.in_rows * 4 + self.out_cols * lim.itemsize + self.hidden_size * 4) + 8192 + K.PARTIALS_MAX_BYTES \
            + self.core_workspace_bytes(lim)

    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding):
        proj = linear(ctx, h, self.in_weight(), out_dtype=torch.float32)
        y = ctx.workspace.take((ctx.num_tokens, self.out_cols), ctx.dtype)
        self.core(ctx, proj, 0, self.store(ctx, run), y, 0, 1.0)
        return linear(ctx, y, self.out_weight(), out_dtype=torch.float32, may_defer_sum=True)


def _segments(ctx: StepContext, lanes: int, parallel: int):
    """(segment length, segments, scratch) of the portion-parallel recurrences for this step; ``lanes``: state values a
    request, ``parallel``: lanes a request gives the kernel without cutting."""
    seg, nseg = K.scan_segments(ctx.num_tokens, ctx.decode_only, parallel * ctx.num_seqs)
    if not seg:
        return 0, 1, None
    return seg, nseg, ctx.workspace.take((2 * (ctx.num_tokens // seg + ctx.num_seqs) * lanes,), torch.float32)


@register_mixer("selective_scan")
class SelectiveScan(Mixer):
    """The selective scan.  W_in h = [x | z] (``inner`` channels each); x passes a causal convolution over time per
    channel (``taps`` taps, weights [inner, taps] with the current token's in the last column, a bias, zeros before the
    sequence's start) and silu; W_x x = [dt | B | C] (``dt_rank``, ``state``, ``state`` numbers); dt = softplus(W_dt dt +
    dt_bias), one per channel; A = -exp(A_log) [inner, state].  Per channel c and state n, token by token,
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n and y_c = sum_n S[c, n] C_n + D_c x_c; the output is
    W_o (y * silu(z)).

    One float32 state slot per request holds the convolution's last taps - 1 inputs followed by S; it starts from zeros.
    Step sizes, decays, the recurrence and the gate are float32 in both engine precisions."""

    def __init__(self, hidden_size: int, inner: int, state: int, dt_rank: int, taps: int = 4, position=None):
        self.hidden_size, self.inner, self.state, self.dt_rank, self.taps = int(hidden_size), int(inner), int(state), int(dt_rank), int(taps)
        if not (1 <= self.taps <= 8):
            raise ValueError(f"taps {taps}: the convolution kernels take 1 to 8")
        if not (0 < self.state <= 128):
            raise ValueError(f"state {state}: the scan keeps up to 128 state values of a channel in registers")
        if self.inner <= 0 or self.dt_rank <= 0:
            raise ValueError("inner and dt_rank must be positive")
        self.conv_floats = (self.taps - 1) * self.inner
        self.w_in = self.w_x = self.w_dt = self.w_o = self.conv = self.conv_b = self.dt_b = self.A = self.D = None

    def param_shapes(self):
        H, I, N, R = self.hidden_size, self.inner, self.state, self.dt_rank
        return {"in_proj": ((2 * I, H), "matrix"), "conv": ((I, self.taps), "matrix"), "conv_bias": ((I,), "small"),
                "x_proj": ((R + 2 * N, I), "matrix"), "dt_proj": ((I, R), "matrix"), "dt_bias": ((I,), "rate_bias"),
                "A_log": ((I, N), "log_rate"), "D": ((I,), "norm"), "o_proj": ((H, I), "matrix")}

    def bind(self, tensors):
        self.w_in, self.w_x = tensors["in_proj"].contiguous(), tensors["x_proj"].contiguous()
        self.w_dt, self.w_o = tensors["dt_proj"].contiguous(), tensors["o_proj"].contiguous()
        self.conv, self.conv_b = tensors["conv"].contiguous(), tensors["conv_bias"].float().contiguous()
        self.dt_b, self.D = tensors["dt_bias"].float().contiguous(), tensors["D"].float().contiguous()
        self.A = (-torch.exp(tensors["A_log"].float())).contiguous()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.conv_floats + self.inner * self.state,), state_dtype="float32")

    def workspace_bytes(self, lim):
        I, N, R = self.inner, self.state, self.dt_rank
        return lim.max_tokens * ((2 * I + I + (R + 2 * N) + I) * 4 + 2 * I * lim.itemsize + self.hidden_size * 4) + 16384 \
            + 2 * K.PARTIALS_MAX_BYTES + 4 * K.scan_scratch_floats(lim.max_tokens, lim.max_seqs, I * N, I * min(N, 16))

    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding):
        T, I, N, R = ctx.num_tokens, self.inner, self.state, self.dt_rank
        ws = ctx.workspace
        group = ctx.groups[run.group]
        state = group.storage["state"][run.slot]
        proj = linear(ctx, h, self.w_in, out_dtype=torch.float32)                       # x | z
        x = ws.take((T, I), torch.float32)
        # the x_proj product's operand in the compute dtype leaves the convolution's kernel beside the float32 rows
        xa = ws.take((T, I), ctx.dtype) if ctx.dtype != torch.float32 else x
        K.conv_act(proj, 0, I, self.conv, self.conv_b, self.taps, "silu", state, group.slot_map, ctx.seq_of_token, ctx.q_start,
                   ctx.positions, x, xa if xa is not x else None)
        xp = linear(ctx, xa, self.w_x, out_dtype=torch.float32)                         # dt | B | C
        dtz = linear(ctx, xp[:, :R], self.w_dt, out_dtype=torch.float32)                # float32 step sizes into the softplus
        y = ws.take((T, I), ctx.dtype)
        seg, nseg, scratch = _segments(ctx, I * N, I * min(N, 16))
        K.selective_scan(x, dtz, xp, R, R + N, proj[:, I:], self.A, self.dt_b, self.D, state, self.conv_floats, group.slot_map,
                         ctx.q_start, ctx.positions, y, ctx.num_seqs, N, seg, nseg, scratch)
        return linear(ctx, y, self.w_o, out_dtype=torch.float32, may_defer_sum=True)


@register_mixer("state_space_duality")
class StateSpaceDuality(BranchMixer):
    """The state-space-duality recurrence.  With inner = ``num_heads`` * ``value_dim``, N = ``state`` and G = ``groups``,
    W_in h = [z: inner | x: inner | B: G N | C: G N | dt: heads]; x, B and C together pass a causal convolution over time
    per channel (``taps`` taps, weights [channels, taps] with the current token's in the last column, a bias, zeros before
    the sequence's start) and silu; dt = softplus(dt + dt_bias) per head.  Head h (group h // (heads / G)) keeps S [N,
    value_dim]: S <- exp(-exp(A_log_h) dt) S + dt B x^T and y = S^T C + D_h x.  The heads together are multiplied by
    silu(z), cut into ``norm_groups`` equal parts that are each divided by their own root mean square (``norm_eps`` inside
    the root), multiplied by the weight ``norm`` and projected by W_o.

    One float32 state slot per request holds the convolution's last taps - 1 inputs followed by S as [heads, value_dim, N];
    it starts from zeros.  Step sizes, decays, the recurrence, the gate and the norm are float32 in both precisions."""

    def __init__(self, hidden_size: int, num_heads: int, value_dim: int, state: int, groups: int = 1, norm_groups: int = 1,
                 taps: int = 4, norm_eps: float = 1e-6, position=None):
        self.hidden_size, self.num_heads, self.value_dim = int(hidden_size), int(num_heads), int(value_dim)
        self.state, self.groups, self.norm_groups, self.taps, self.norm_eps = int(state), int(groups), int(norm_groups), int(taps), float(norm_eps)
        if self.num_heads <= 0 or self.groups <= 0 or self.num_heads % self.groups:
            raise ValueError(f"num_heads {num_heads} is not a positive multiple of groups {groups}")
        self.inner = self.num_heads * self.value_dim
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise ValueError(f"norm_groups {norm_groups} does not cut {self.inner} channels into equal parts")
        if not (1 <= self.taps <= 8):
            raise ValueError(f"taps {taps}: the convolution kernels take 1 to 8")
        if not (0 < self.state <= 256):
            raise ValueError(f"state {state}: the recurrence keeps up to 256 rows of a state column in registers")
        self.channels = self.inner + 2 * self.groups * self.state               # what the convolution sees: x | B | C
        self.conv_floats = (self.taps - 1) * self.channels
        self.in_rows = 2 * self.inner + 2 * self.groups * self.state + self.num_heads
        self.out_cols = self.inner
        self.w_in = self.w_o = self.conv = self.conv_b = self.dt_b = self.A = self.D = self.norm_w = None

    def param_shapes(self):
        H, n = self.hidden_size, self.num_heads
        return {"in_proj": ((self.in_rows, H), "matrix"), "conv": ((self.channels, self.taps), "matrix"),
                "conv_bias": ((self.channels,), "small"), "dt_bias": ((n,), "rate_bias"), "A_log": ((n,), "log_rate"), "D": ((n,), "norm"),
                "norm": ((self.inner,), "norm"), "o_proj": ((H, self.inner), "matrix")}

    def bind(self, tensors):
        self.w_in, self.w_o = tensors["in_proj"].contiguous(), tensors["o_proj"].contiguous()
        self.conv, self.conv_b = tensors["conv"].contiguous(), tensors["conv_bias"].float().contiguous()
        self.dt_b, self.D = tensors["dt_bias"].float().contiguous(), tensors["D"].float().contiguous()
        self.A = torch.exp(tensors["A_log"].float()).contiguous()
        self.norm_w = tensors["norm"].contiguous()

    def in_weight(self):
        return self.w_in

    def out_weight(self):
        return self.w_o

    def state_shape(self):
        return (self.conv_floats + self.num_heads * self.state * self.value_dim,)

    def cache_need(self):
        return CacheNeed("state", state_shape=self.state_shape(), state_dtype="float32")

    def store(self, ctx, run):
        group = ctx.groups[run.group]
        return group.storage["state"][run.slot], group.slot_map

    def core_workspace_bytes(self, lim):
        return lim.max_tokens * (self.channels + self.inner + 2 * self.num_heads) * 4 + 2048 \
            + 4 * K.scan_scratch_floats(lim.max_tokens, lim.max_seqs, self.num_heads * self.state * self.value_dim, self.inner * min(self.state, 32))

    def core(self, ctx, proj, col0, store, out, out_col0, mult):
        T, I, GN = ctx.num_tokens, self.inner, self.groups * self.state
        state, slots = store
        ws = ctx.workspace
        xbc = ws.take((T, self.channels), torch.float32)
        K.conv_act(proj, col0 + I, self.channels, self.conv, self.conv_b, self.taps, "silu", state, slots, ctx.seq_of_token, ctx.q_start,
                   ctx.positions, xbc)
        y = ws.take((T, I), torch.float32)
        seg, nseg, scratch = _segments(ctx, self.num_heads * self.state * self.value_dim, I * min(self.state, 32))
        steps = ws.take((T * 2 * self.num_heads,), torch.float32)
        dt0 = col0 + 2 * I + 2 * GN
        K.ssd_scan(xbc, 0, I, I + GN, proj[:, dt0:dt0 + self.num_heads], self.A, self.dt_b, self.D, state, self.conv_floats, slots,
                   ctx.q_start, ctx.positions, y, ctx.num_seqs, self.num_heads, self.value_dim, self.groups, self.state, seg, nseg, scratch, steps)
        K.gate_group_norm(y, proj[:, col0:col0 + I], self.norm_w, self.norm_eps, mult, out[:, out_col0:out_col0 + I], self.norm_groups)


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    """Two mixers side by side on the same input: y = ``left_scale`` * left(h) + ``right_scale`` * right(h).  ``left`` and
    ``right`` name registered mixers of the two-products form (:class:`BranchMixer`) as {"kind": ..., further parameters};
    their tensors are this part's ``left.<name>`` and ``right.<name>``.  Both input products are one product over the
    stacked rows, both output products one product over the two cores' outputs side by side (each already times its
    scale), so the sum of the halves is made inside that product, in float32.

    The left mixer's cache is this mixer's cache; the right mixer's is kept beside it as a state of the part."""

    def __init__(self, hidden_size: int, left: dict, right: dict, left_scale: float = 1.0, right_scale: float = 1.0, position=None):
        self.hidden_size = int(hidden_size)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        mk = lambda d: make_part("mixer", d["kind"], hidden_size=self.hidden_size, position=position,
                                 **{k: v for k, v in dict(d).items() if k != "kind"})
        self.left, self.right = mk(left), mk(right)
        for m in (self.left, self.right):
            if not isinstance(m, BranchMixer):
                raise ValueError("the halves of 'parallel_mixers' are mixers of the two-products form (BranchMixer)")
        need = self.right.cache_need()
        if need is not None and need.kind != "state":
            raise ValueError("the right half keeps a state of fixed size, or nothing")
        self.w_in = self.w_o = None

    def param_shapes(self):
        shapes = {}
        for side, m in (("left", self.left), ("right", self.right)):
            for local, spec in m.param_shapes().items():
                shapes[f"{side}.{local}"] = spec
        return shapes

    def bind(self, tensors):
        for side, m in (("left", self.left), ("right", self.right)):
            m.bind({k[len(side) + 1:]: v for k, v in tensors.items() if k.startswith(side + ".")})
        self.w_in = _stack([self.left.in_weight(), self.right.in_weight()])
        wl, wr = self.left.out_weight(), self.right.out_weight()
        if wl.dtype != wr.dtype:
            wl, wr = wl.float(), wr.float()
        self.w_o = torch.cat([wl, wr], dim=1).contiguous()

    def cache_need(self):
        return self.left.cache_need()

    def state_need(self):
        return self.right.cache_need()

    def workspace_bytes(self, lim):
        rows, cols = self.left.in_rows + self.right.in_rows, self.left.out_cols + self.right.out_cols
        return lim.max_tokens * (rows * 4 + cols * lim.itemsize + self.hidden_size * 4) + 8192 + K.PARTIALS_MAX_BYTES \
            + self.left.core_workspace_bytes(lim) + self.right.core_workspace_bytes(lim)

    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding):
        proj = linear(ctx, h, self.w_in, out_dtype=torch.float32)
        y = ctx.workspace.take((ctx.num_tokens, self.left.out_cols + self.right.out_cols), ctx.dtype)
        self.left.core(ctx, proj, 0, self.left.store(ctx, run), y, 0, self.left_scale)
        store = run.state_of(ctx, self) if self.right.cache_need() is not None else None
        self.right.core(ctx, proj, self.left.in_rows, store, y, self.left.out_cols, self.right_scale)
        return linear(ctx, y, self.w_o, out_dtype=torch.float32, may_defer_sum=True)
