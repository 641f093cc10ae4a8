"""Python face of the CUDA kernel library (``csrc/kernels``), loaded with ctypes.

Every function here takes torch tensors that already live on the device, checks what the
kernel cannot check for itself, and launches on the current CUDA stream.  Nothing falls back
to another implementation: a missing library, a refused size or a failed launch raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_long, c_size_t, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {
    -2: "unsupported dtype combination",
    -3: "a size this kernel refuses",
    -4: "pointer or stride not aligned as the kernel requires",
    -5: "library state error (tensor map / attribute)",
    -6: "a bounded wait inside the kernel ran out",
}


class KernelError(RuntimeError):
    pass


_lib: Optional[ctypes.CDLL] = None
_proxy = None
_RECORD: Optional[list] = None
_QUERIES = ("_supports", "_ranges", "_grid", "_error")     # answer a question, launch nothing


class _Entry:
    """One launching entry point.  Calls go to the ctypes function and, while a recording is on,
    into the list; every attribute (argtypes, restype, ...) is the ctypes function's own, so code
    that declares a signature on what :func:`lib` hands out declares it on the real thing."""
    __slots__ = ("_fn",)

    def __init__(self, fn):
        object.__setattr__(self, "_fn", fn)

    def __call__(self, *args):
        rc = self._fn(*args)
        if _RECORD is not None:
            _RECORD.append((self._fn, args))
        return rc

    def __getattr__(self, key):
        return getattr(self._fn, key)

    def __setattr__(self, key, value):
        setattr(self._fn, key, value)


class _Library:
    """The loaded library with its launching entry points wrapped, so that what a forward pass
    launches can be written down as (function, arguments) and issued again by
    :func:`replay_launches` without the Python that chose the arguments."""

    def __init__(self, cdll: ctypes.CDLL):
        self._cdll = cdll

    def __getattr__(self, name: str):
        fn = getattr(self._cdll, name)
        wrapped = fn if name.endswith(_QUERIES) else _Entry(fn)
        self.__dict__[name] = wrapped
        return wrapped


def lib() -> "_Library":
    global _lib, _proxy
    if _proxy is None:
        _lib = _build.load_kernels()
        _declare(_lib)
        _proxy = _Library(_lib)
    return _proxy


def begin_recording() -> None:
    """From here every launch made through this module is also written down."""
    global _RECORD
    _RECORD = []


def end_recording() -> list:
    global _RECORD
    plan, _RECORD = _RECORD or [], None
    return plan


def replay_launches(plan: list) -> None:
    """Issue a recorded list again.  Valid only while every argument still means the same: the
    same buffers at the same addresses, the same sizes, the same stream."""
    global _launches
    for fn, args in plan:
        rc = fn(*args)
        if rc != 0:
            _check(rc, getattr(fn, "__name__", "a recorded launch"))
    _launches += len(plan)


def _declare(l: ctypes.CDLL) -> None:
    P, I, L, F = c_void_p, c_int, c_long, c_float
    sigs = {
        "aien_embed_gather": [P, I, P, P, I, I, I, P],
        "aien_add_rmsnorm": [P, P, I, I, c_size_t, P, I, F, P, I, I, I, P],
        "aien_gather_add_rows": [P, P, I, I, c_size_t, P, P, I, I, P],
        "aien_swiglu": [P, P, I, I, I, I, P],
        "aien_add_residual": [P, P, I, I, c_size_t, I, I, P],
        "aien_rope_table": [P, P, P, P, I, I, P],
        "aien_qk_norm_rope_kv_write": [P, L, I, P, L, P, L, I, I, I, c_size_t, P, L, I, P, P, I, F, P, P, I, P, P, P, I, I, I, P],
        "aien_convert": [P, I, P, I, c_size_t, P],
        "aien_gemm_simple": [P, I, L, P, I, L, P, I, L, I, I, I, P],
        "aien_paged_attention_generic": [P, L, P, P, P, I, P, P, P, L, I, I, I, I, I, F, I, I, I, I, P, I, P, P, P, P, L, F, P],
        "aien_branch_norm_add": [P, P, I, I, c_size_t, P, I, I, c_size_t, P, I, F, P, I, I, I, P],
        "aien_stream_norm_inplace": [P, P, I, F, P, I, I, I, P],
        "aien_qk_rope_pairs_unit_kv_write": [P, L, I, P, L, P, L, I, I, I, c_size_t, P, L, I, I, I, F, P, P, I, P, P, P, I, I, I, P],
        "aien_moe_route": [P, I, I, I, I, I, I, P, P, P, P],
        "aien_moe_expert_up": [P, I, L, P, I, P, P, I, I, I, I, I, I, P],
        "aien_moe_expert_down": [P, I, P, I, P, P, P, I, I, I, I, P],
        "aien_act_rows": [P, I, c_size_t, I, P],
        "aien_moe_plan_rows": [P, I, I, P, P, P, P],
        "aien_moe_place_rows": [P, L, P, P, P, I, I, P, I, P, P, P],
        "aien_moe_expert_rows_bf16": [I, P, L, P, P, P, P, I, I, I, I, I, P],
        "aien_gemm_tc_grouped": [P, L, P, L, I, P, I, L, P, I, P, P, I, I, I, P],
        "aien_argmax_rows": [P, I, I, P, P],
        "aien_sample_rows": [P, I, I, P, P, P, P, P, P, P, P, P],
        "aien_sample_rows_logprob": [P, I, I, P, P, P, P, P, P, P, P, P, P],
        "aien_gemv_bf16": [P, L, P, L, P, I, L, I, I, I, I, I, c_size_t, P],
        "aien_gemv_stream_bf16": [P, L, P, L, P, I, L, I, I, I, I, I, c_size_t, P],
        "aien_gemv_stream_error": [],
        "aien_gemm_tc": [P, L, P, L, P, I, L, I, I, I, I, I, c_size_t, P],
        "aien_gemm_tc_ranges": [I, I],
        "aien_gemm_tc_m256_supports": [I, I, I, I],
        "aien_gemv_stream_scaled": [P, L, P, L, P, I, L, I, I, I, I, P, I, F, P],
        "aien_gemv_stream_residual": [P, L, P, L, P, L, P, I, P, L, P, I, I, I, P],
        "aien_gemv_stream_grid": [I],
        "aien_feed_token_ids": [P, P, P, I, P],
        "aien_copy_spans": [P, c_size_t, I, c_size_t, c_size_t, c_size_t, P],
        "aien_zero_fill": [P, c_size_t, P],
        "aien_scale_rows_ssq": [P, L, P, I, F, P, L, I, I, P],
        "aien_gemm_tc_error": [],
        "aien_attention_prefill_tc_error": [],
        "aien_paged_attention_prefill": [P, L, P, P, P, I, P, P, P, P, I, P, L, I, I, I, I, I, F, I, P, P],
        "aien_paged_attention_prefill_tc": [P, L, I, P, P, I, P, I, P, P, P, P, I, P, L, I, I, I, I, I, F, P],
        "aien_paged_attention_prefill_tc_split": [P, L, I, P, P, I, P, I, P, P, P, P, I, P, L, I, I, I, I, I, F, P, L, I, I, P],
        "aien_paged_attention_prefill_tc_supports": [I, I],
        "aien_paged_attention_prefill_tc_masked": [P, L, I, P, P, I, P, I, P, P, P, P, I, P, L, I, I, I, I, I, F, P, L, I, I, I, P, P],
        "aien_paged_attention_decode": [P, L, P, P, P, I, P, P, P, P, L, P, P, P, I, I, I, I, I, F, I, I, P],
        "aien_paged_attention_decode_masked": [P, L, P, P, P, I, P, P, P, P, L, P, P, P, I, I, I, I, I, F, I, I, I, P, P],
        "aien_paged_attention_decode_terms": [P, L, P, P, P, I, P, P, P, P, L, P, P, P, I, I, I, I, I, F, I, I, P, P, P, L, F, P],
        "aien_paged_attention_prefill_tc_terms": [P, L, I, P, P, I, P, I, P, P, P, P, I, P, L, I, I, I, I, I, F, P, L, I, I, I, P, P, P, P, L, F, P],
        "aien_paged_attention_decode_stream": [P, L, P, P, I, P, I, P, P, P, P, L, P, P, P, I, I, I, I, I, F, I, I, P],
        "aien_paged_attention_decode_stream_supports": [I, I, I, I, I],
        "aien_attention_decode_stream_error": [],
        "aien_collect_wait_errors": [P, P],
        "aien_decay_linear_attention": [P, I, L, I, I, I, P, P, P, P, P, P, L, I, I, I, I, I, P],
        "aien_gated_rmsnorm": [P, L, P, I, L, P, I, F, P, I, L, I, I, P],
        "aien_gated_recurrence": [P, I, L, I, I, I, P, P, I, P, P, P, P, P, I, L, I, I, I, P],
        "aien_decay_linear_attention_chunked": [P, I, L, I, I, I, P, P, P, P, P, P, L, P, I, I, I, I, I, P],
        "aien_latent_prepare": [P, I, L, I, P, P, I, F, P, I, L, I, I, I, I, P, P, P, P, I, I, P],
        "aien_rotate_pairs_rows": [P, I, L, L, P, I, L, L, I, I, I, I, P, P, P],
        "aien_latent_attention_tc": [P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P, I, P, P, I, P],
        "aien_head_project_tc": [P, L, L, P, P, I, L, L, I, I, I, I, P],
        "aien_latent_attention_tc_supports": [I, I],
        "aien_head_project": [P, I, L, L, P, I, L, L, P, I, L, L, I, I, I, I, P],
        "aien_latent_attention": [P, L, P, I, P, I, P, P, P, P, I, L, I, I, I, I, I, I, F, P, P],
        "aien_post_norm_add": [P, P, I, I, c_size_t, P, I, F, F, P, I, F, P, I, I, I, P],
        "aien_embed_gather_scaled": [P, I, P, P, I, I, I, F, P],
        "aien_gelu_times_table": [P, I, L, P, I, L, I, P, I, P, I, L, I, I, P],
        "aien_softcap": [P, c_size_t, F, P],
        "aien_replicate_streams": [P, c_size_t, I, P],
        "aien_hc_norm": [P, I, P, I, I, c_size_t, P, P, P, I, F, P, I, I, I, P, I, P, P, P, P],
        "aien_token_shift": [P, P, I, P, P, P, P, P, P, I, I, I, P],
        "aien_hc_sum_rows": [P, I, I, P, I, I, c_size_t, P, P, P, I, I, P],
        "aien_embed_gather_sinusoid": [P, I, P, P, P, P, I, I, I, F, P],
        "aien_attn_conv_prepare": [P, L, I, I, I, I, I, I, P, P, P, I, I, P, P, I, F, I, I, I, P, P, P, P, P, P, P, P, I, P, I, L, I, P],
        "aien_delta_conv_prepare": [P, L, I, I, I, I, I, I, I, I, I, P, P, P, I, I, P, P, I, P, c_size_t, P, P, P, P, P, L, P, L, I, P],
        "aien_delta_rule": [P, L, I, I, I, P, L, P, c_size_t, c_size_t, P, P, P, P, L, I, I, I, I, I, P],
        "aien_grouped_gated_rmsnorm": [P, L, P, I, L, P, I, F, P, I, L, I, I, I, I, P],
        "aien_paged_attention_decode_fused": [P, L, P, L, P, L, P, P, I, F, P, P, I, P, P, P, P, I, P, P, L, P, P, P,
                                              I, I, I, I, I, F, I, I, P],
        "aien_conv_act": [P, L, I, I, P, I, P, I, I, I, P, c_size_t, P, P, P, P, P, L, P, L, I, P],
        "aien_selective_scan": [P, L, P, L, P, L, I, I, P, L, P, P, P, I, P, c_size_t, c_size_t, P, P, P, P, I, L, I, I, I, I, I, I, P, P],
        "aien_ssd_scan": [P, L, I, I, I, P, L, P, P, P, I, P, c_size_t, c_size_t, P, P, P, P, L, I, I, I, I, I, I, I, I, P, P, P],
        "aien_gate_group_norm": [P, L, P, L, P, I, F, F, P, I, L, I, I, I, P],
        "aien_scaled_add_rmsnorm": [P, P, I, I, c_size_t, P, P, P, I, F, P, I, I, I, P],
        "aien_pass_input": [P, P, P, I, I, I, P],
        "aien_clamped_glu": [P, I, L, I, I, P, P, I, F, F, P, I, L, I, I, P],
        "aien_sigmoid_gate": [P, I, L, P, L, F, P, I, L, I, I, P],
        "aien_routed_combine": [P, I, I, c_size_t, P, I, L, P, P, I, I, c_size_t, P, L, P, I, I, P],
        "aien_moe_route_biased": [P, L, I, I, I, I, I, F, P, I, P, P, P, P, P],
        "aien_rope_halves_value_write": [P, L, I, I, I, I, I, I, I, P, P, I, P, P, I, L, P, P, I, I, P],
    }
    for name, args in sigs.items():
        fn = getattr(l, name)
        fn.argtypes = args
        fn.restype = c_int


def declare_optional(name: str, args) -> bool:
    """Declare a symbol that later kernel files add; returns False when the library lacks it."""
    lib()
    try:
        fn = getattr(_lib, name)
    except AttributeError:
        return False
    fn.argtypes = args
    fn.restype = c_int
    return True


_launches = 0


def launch_count() -> int:
    """Kernel launches issued through this module so far (replayed graph nodes included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(rc: int, name: str) -> None:
    global _launches
    if rc == 0:
        _launches += 1
        return
    if rc < 0:
        raise KernelError(f"{name}: {_ERRORS.get(rc, 'refused')} (code {rc})")
    raise KernelError(f"{name}: CUDA error {rc} at launch")


_STREAM: Optional[int] = None


class stream_scope:
    """Looks the current CUDA stream up once for every launch made inside the block (a step
    makes hundreds; the lookup costs more than the launch)."""

    def __enter__(self):
        global _STREAM
        self._prev = _STREAM
        _STREAM = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _STREAM
        _STREAM = self._prev
        return False


def _stream() -> int:
    return _STREAM if _STREAM is not None else torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels") from None


def _dev(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on the CUDA device (there is no CPU path)")


# ---------------------------------------------------------------------------- row-wise ops
def embed_gather(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor) -> None:
    """x[t] = table[ids[t]] as float32.  table [V,H], ids int32 [T], x float32 [T,H]."""
    _dev(table, ids, x)
    T, H = x.shape
    assert table.is_contiguous() and x.is_contiguous() and ids.dtype == torch.int32 and x.dtype == torch.float32
    assert table.shape[1] == H and ids.numel() >= T
    _check(lib().aien_embed_gather(_p(table), dt(table), _p(ids), _p(x), T, H, table.shape[0], _stream()), "embed_gather")


def _parts_of(delta: Optional[torch.Tensor], shape) -> tuple:
    """(nparts, stride in elements) of a pending sum: [T,H], or float32 partials [P,T,H]."""
    if delta is None:
        return 1, 0
    assert delta.is_contiguous()
    if delta.dim() == 3:
        assert tuple(delta.shape[1:]) == tuple(shape) and delta.dtype == torch.float32
        return delta.shape[0], delta.shape[1] * delta.shape[2]
    assert tuple(delta.shape) == tuple(shape)
    return 1, 0


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """x += delta (when given); out = rmsnorm(x) * weight.  x float32 [T,H] updated in place."""
    _dev(x, delta, weight, out)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape == x.shape
    assert weight.numel() == H and weight.is_contiguous()
    nparts, stride = _parts_of(delta, x.shape)
    _check(lib().aien_add_rmsnorm(_p(x), _p(delta), dt(delta) if delta is not None else F32, nparts, stride,
                                  _p(weight), dt(weight), float(eps), _p(out), dt(out), T, H, _stream()), "add_rmsnorm")


def gather_add_rows(x: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = x[rows[r]] + delta[rows[r]] in float32."""
    _dev(x, delta, rows, out)
    R, H = out.shape
    assert x.dtype == torch.float32 and out.dtype == torch.float32 and rows.dtype == torch.int32
    assert x.is_contiguous() and out.is_contiguous() and x.shape[1] == H and rows.numel() >= R
    nparts, stride = _parts_of(delta, x.shape)
    _check(lib().aien_gather_add_rows(_p(x), _p(delta), dt(delta) if delta is not None else F32, nparts, stride,
                                      _p(rows), _p(out), R, H, _stream()), "gather_add_rows")


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    """x += delta in float32; delta [T,H] in any kernel dtype, or float32 partial products [P,T,H]."""
    _dev(x, delta)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    nparts, stride = _parts_of(delta, x.shape)
    _check(lib().aien_add_residual(_p(x), _p(delta), dt(delta), nparts, stride, T, H, _stream()), "add_residual")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, group: int = 0) -> None:
    """out = silu(gate) * up for gate_up = [T, 2I]: gate columns first (group 0), or gate and up
    columns interleaved in runs of ``group``."""
    _dev(gate_up, out)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype
    _check(lib().aien_swiglu(_p(gate_up), _p(out), dt(out), T, I, int(group), _stream()), "swiglu")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    """cos/sin [T, half] float32 of positions[t] * inv_freq[i], the angle taken in float64."""
    _dev(positions, inv_freq, cos, sin)
    T, half = cos.shape
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float64 and inv_freq.numel() == half
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    _check(lib().aien_rope_table(_p(positions), _p(inv_freq), _p(cos), _p(sin), T, half, _stream()), "rope_table")


def qk_norm_rope_kv_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], head_dim: int,
                          q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                          cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                          slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], q_out: Optional[torch.Tensor] = None) -> None:
    """Per-head RMSNorm of q and k (when weights are given), rotation of the first
    ``rotary_dim`` values, q written to ``q_out`` (default: in place), k and v written to their
    cache slots.  q [T, nq*hd], k/v [T, nkv*hd] may be column slices of one projection output, or
    of float32 partial products [P, T, ...] that are summed on the way in (then q_out is needed)."""
    _dev(q, k, v, q_norm_w, k_norm_w, cos, sin, slot_map, k_cache, v_cache, q_out)
    nparts, part_stride = 1, 0
    if q.dim() == 3:
        assert q.dtype == torch.float32 and q_out is not None
        nparts, part_stride = q.shape[0], q.stride(0)
        if k is not None:
            assert k.dim() == 3 and v.dim() == 3 and k.stride(0) == part_stride and v.stride(0) == part_stride
    if q_out is None:
        q_out = q
    T = q.shape[-2]
    assert q.stride(-1) == 1 and q.shape[-1] % head_dim == 0 and q_out.stride(1) == 1 and q_out.shape == (T, q.shape[-1])
    nq = q.shape[-1] // head_dim
    nkv = 0
    if k is not None:
        assert v is not None and slot_map is not None and k_cache is not None and v_cache is not None
        assert k.stride(-1) == 1 and v.stride(-1) == 1 and k.dtype == q.dtype and v.dtype == q.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == v_cache.dtype
        assert slot_map.dtype == torch.int32 and slot_map.numel() >= T
        nkv = k.shape[-1] // head_dim
    wdt = F32
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            assert w.numel() == head_dim and w.is_contiguous()
            wdt = dt(w)
    if q_norm_w is not None and k_norm_w is not None:
        assert q_norm_w.dtype == k_norm_w.dtype
    if cos is not None:
        assert sin is not None and cos.shape == (T, rotary_dim // 2) and cos.is_contiguous() and sin.is_contiguous()
    _check(lib().aien_qk_norm_rope_kv_write(
        _p(q), q.stride(-2), nq, _p(k), k.stride(-2) if k is not None else 0, _p(v), v.stride(-2) if v is not None else 0,
        nkv, dt(q), nparts, part_stride, _p(q_out), q_out.stride(0), head_dim, _p(q_norm_w), _p(k_norm_w), wdt, float(eps),
        _p(cos), _p(sin), rotary_dim if cos is not None else 0, _p(slot_map), _p(k_cache), _p(v_cache),
        dt(q_out), dt(k_cache) if k_cache is not None else dt(q_out), T, _stream()), "qk_norm_rope_kv_write")


def _source(t: Optional[torch.Tensor], shape) -> tuple:
    """(pointer, dtype code, parts, part stride) of a branch output: [T,H], or float32 parts [P,T,H]."""
    if t is None:
        return 0, F32, 1, 0
    assert t.is_contiguous()
    if t.dim() == 3:                         # parts [P,T,H], float32 or (the weighted outputs of routed experts) bfloat16
        assert tuple(t.shape[1:]) == tuple(shape)
        return _p(t), dt(t), t.shape[0], t.shape[1] * t.shape[2]
    assert tuple(t.shape) == tuple(shape)
    return _p(t), dt(t), 1, 0


def branch_norm_add(x: torch.Tensor, a: torch.Tensor, weight: torch.Tensor, eps: float, b: Optional[torch.Tensor] = None,
                    h: Optional[torch.Tensor] = None) -> None:
    """x += y / sqrt(mean(y^2) + eps) * weight with y = a (+ b): the norm of a branch's output, added
    into the float32 stream.  a and b are [T,H] tensors or float32 parts [P,T,H] (added in order).
    ``h`` (optional, [T,H]) receives the updated rows in its own dtype."""
    _dev(x, a, b, weight, h)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and weight.numel() == H and weight.is_contiguous()
    if h is not None:
        assert h.is_contiguous() and tuple(h.shape) == (T, H)
    pa, da, na, sa = _source(a, x.shape)
    pb, db, nb, sb = _source(b, x.shape)
    _check(lib().aien_branch_norm_add(_p(x), pa, da, na, sa, pb, db, nb, sb, _p(weight), dt(weight), float(eps),
                                      _p(h), dt(h) if h is not None else F32, T, H, _stream()), "branch_norm_add")


def stream_norm_inplace(x: torch.Tensor, weight: torch.Tensor, eps: float, h: Optional[torch.Tensor] = None) -> None:
    """x = x / sqrt(mean(x^2) + eps) * weight in place (float32 rows); ``h`` as in branch_norm_add."""
    _dev(x, weight, h)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and weight.numel() == H and weight.is_contiguous()
    if h is not None:
        assert h.is_contiguous() and tuple(h.shape) == (T, H)
    _check(lib().aien_stream_norm_inplace(_p(x), _p(weight), dt(weight), float(eps), _p(h), dt(h) if h is not None else F32,
                                          T, H, _stream()), "stream_norm_inplace")


def qk_rope_pairs_unit_kv_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], head_dim: int,
                                value_dim: int, unit: bool, eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                                rotary_dim: int, slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                                v_cache: Optional[torch.Tensor], q_out: torch.Tensor) -> None:
    """Rotation over neighbouring pairs (2i, 2i+1) of the first ``rotary_dim`` values of every q and
    k head, then (``unit``) division by the head's root mean square; q to ``q_out``, k to its cache
    slot, and as values the first ``value_dim`` values of the k head as projected (``v`` None) or of
    the v head.  q [T, nq*hd], k [T, nkv*hd] may be column slices of one product's output, or of
    float32 partial products [P, T, ...]."""
    _dev(q, k, v, cos, sin, slot_map, k_cache, v_cache, q_out)
    nparts, part_stride = 1, 0
    if q.dim() == 3:
        assert q.dtype == torch.float32
        nparts, part_stride = q.shape[0], q.stride(0)
        assert k is None or (k.dim() == 3 and k.stride(0) == part_stride)
        assert v is None or (v.dim() == 3 and v.stride(0) == part_stride)
    T = q.shape[-2]
    assert q.stride(-1) == 1 and q.shape[-1] % head_dim == 0 and q_out.stride(1) == 1 and q_out.shape == (T, q.shape[-1])
    nq, nkv = q.shape[-1] // head_dim, 0
    if k is not None:
        assert slot_map is not None and k_cache is not None and v_cache is not None and k.stride(-1) == 1 and k.dtype == q.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == v_cache.dtype
        assert slot_map.dtype == torch.int32 and slot_map.numel() >= T
        nkv = k.shape[-1] // head_dim
        assert v is None or (v.stride(-1) == 1 and v.dtype == q.dtype and v.shape[-1] == nkv * value_dim)
    if cos is not None:
        assert sin is not None and cos.shape == (T, rotary_dim // 2) and cos.is_contiguous() and sin.is_contiguous()
    _check(lib().aien_qk_rope_pairs_unit_kv_write(
        _p(q), q.stride(-2), nq, _p(k), k.stride(-2) if k is not None else 0, _p(v), v.stride(-2) if v is not None else 0, nkv,
        dt(q), nparts, part_stride, _p(q_out), q_out.stride(0), head_dim, int(value_dim), 1 if unit else 0, float(eps),
        _p(cos), _p(sin), rotary_dim if cos is not None else 0, _p(slot_map), _p(k_cache), _p(v_cache),
        dt(q_out), dt(k_cache) if k_cache is not None else dt(q_out), T, _stream()), "qk_rope_pairs_unit_kv_write")


# ---------------------------------------------------------------------------- routed feed-forward
ACT_KINDS = {"gelu": 0, "gelu_erf": 0, "gelu_tanh": 1, "relu2": 2}      # relu2: the square of relu
ACT_IN_PRODUCT = (0, 1, 2)          # the kinds that the products' epilogues know; others would run as a kernel behind the product


def moe_route(z: torch.Tensor, groups: int, keep: int, top: int, renorm: bool, ids: torch.Tensor, wts: torch.Tensor,
              expert_count: Optional[torch.Tensor] = None) -> None:
    """From router logits z [T,E] (float32): softmax scores, the ``keep`` best of ``groups`` equal groups of
    neighbouring experts (a group scores its best expert), the ``top`` best experts of those; ids int32
    [T,top], wts float32 [T,top] = their scores (``renorm``: divided by their sum).  ``expert_count`` (int32 [E],
    zero on entry): every choice adds one to its expert's count, for the grouped products' plan, which zeroes it again."""
    _dev(z, ids, wts, expert_count)
    assert expert_count is None or (expert_count.dtype == torch.int32 and expert_count.is_contiguous() and expert_count.numel() >= z.shape[1])
    T, E = z.shape
    assert z.dtype == torch.float32 and z.is_contiguous() and ids.dtype == torch.int32 and wts.dtype == torch.float32
    assert ids.is_contiguous() and wts.is_contiguous() and ids.numel() >= T * top and wts.numel() >= T * top
    _check(lib().aien_moe_route(_p(z), T, E, int(groups), int(keep), int(top), 1 if renorm else 0, _p(ids), _p(wts), _p(expert_count),
                                _stream()), "moe_route")


def moe_expert_up(h: torch.Tensor, w_up: torch.Tensor, ids: torch.Tensor, act: torch.Tensor, top: int, act_kind: int) -> None:
    """act[t*top + c] = f(w_up[ids[t,c]] . h[t]); h [T,D], w_up [E,F,D], act [T*top, F]."""
    _dev(h, w_up, ids, act)
    T, D = h.shape
    E, Fd, D2 = w_up.shape
    assert D2 == D and h.stride(1) == 1 and w_up.is_contiguous() and act.is_contiguous() and tuple(act.shape) == (T * top, Fd)
    _check(lib().aien_moe_expert_up(_p(h), dt(h), h.stride(0), _p(w_up), dt(w_up), _p(ids), _p(act), dt(act), T, int(top), D, Fd,
                                    int(act_kind), _stream()), "moe_expert_up")


def moe_expert_down(act: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, parts: torch.Tensor, top: int) -> None:
    """parts[c, t] = wts[t,c] * (w_down[ids[t,c]] . act[t*top + c]); w_down [E,D,F], parts float32 [top,T,D]."""
    _dev(act, w_down, ids, wts, parts)
    E, D, Fd = w_down.shape
    T = act.shape[0] // top
    assert act.is_contiguous() and act.shape[1] == Fd and w_down.is_contiguous()
    assert parts.dtype == torch.float32 and parts.is_contiguous() and tuple(parts.shape) == (top, T, D)
    _check(lib().aien_moe_expert_down(_p(act), dt(act), _p(w_down), dt(w_down), _p(ids), _p(wts), _p(parts), T, int(top), D, Fd,
                                      _stream()), "moe_expert_down")


MOE_ROWS_MAX_TOKENS = 16      # steps of up to this many tokens stream the chosen experts row by row


def _moe_tiles(num_pairs: int, num_experts: int) -> int:
    """Row tiles of 128 that the pairs sorted by expert can need: every expert's run is padded to whole tiles."""
    return (num_pairs + 127) // 128 + num_experts


def moe_workspace_bytes(lim, num_experts: int, top: int, hidden: int, expert_ff: int) -> int:
    """Scratch of the grouped expert products for the largest step: the rows sorted by expert (inputs
    and hidden activations, bfloat16) and their maps."""
    tiles = _moe_tiles(lim.max_tokens * top, num_experts)
    return tiles * 128 * ((hidden + expert_ff) * 2 + 8) + tiles * 4 + num_experts * 4 + 8192


_MOE_IMPL = __import__("os").environ.get("AIEN_B200_MOE", "").strip().lower()      # "plain" pins the plain kernels


def moe_grouped_supports(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    D, Fd = w_up.shape[2], w_up.shape[1]
    return (h.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16 and D % 8 == 0
            and Fd % 8 == 0 and h.stride(1) == 1 and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0
            and w_up.data_ptr() % 16 == 0 and w_down.data_ptr() % 16 == 0)


def moe_takes_grouped(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    """Whether moe_experts runs this step on the grouped tensor-core products (the router then counts its choices per expert)."""
    return _MOE_IMPL != "plain" and h.shape[0] > MOE_ROWS_MAX_TOKENS and moe_grouped_supports(h, w_up, w_down)


def moe_experts(ctx, h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor,
                top: int, act_kind: int, expert_count: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Returns parts [top, T, D] with parts[c, t] = wts[t,c] * w_down[e] f(w_up[e] h[t]), e = ids[t,c]: the chosen
    experts of every token, weighted, one part per choice (float32; bfloat16 from the grouped products, whose
    consumer adds them in float32).  ``expert_count``: what moe_route counted; the grouped products need it.
    bfloat16: a few tokens stream their experts' rows (one warp per output value, 16-byte loads); larger
    steps place the (token, choice) pairs in rows sorted by expert and run two grouped tcgen05 products, the activation in
    the first one's epilogue, the weights and the way back to token order in the second's.  float32, and
    sizes those kernels do not take: the plain products."""
    T, D = h.shape
    E, Fd, _ = w_up.shape
    ws = ctx.workspace
    ok = _MOE_IMPL != "plain" and moe_grouped_supports(h, w_up, w_down)
    grouped = ok and T > MOE_ROWS_MAX_TOKENS
    if grouped and expert_count is None:
        raise KernelError("moe_experts: the grouped products need the per-expert counts of moe_route (expert_count)")
    parts = ws.take((top, T, D), torch.bfloat16 if grouped else torch.float32)
    if ok and T <= MOE_ROWS_MAX_TOKENS and D % 256 == 0 and Fd % 256 == 0:
        act = ws.take((T * top, Fd), torch.bfloat16)
        _check(lib().aien_moe_expert_rows_bf16(0, _p(h), h.stride(0), _p(w_up), _p(ids), _p(wts), _p(act), T, top, Fd, D,
                                               int(act_kind), _stream()), "moe_expert_rows(up)")
        _check(lib().aien_moe_expert_rows_bf16(1, _p(act), Fd, _p(w_down), _p(ids), _p(wts), _p(parts), T, top, D, Fd,
                                               int(act_kind), _stream()), "moe_expert_rows(down)")
        return parts
    if grouped:
        tiles = _moe_tiles(T * top, E)
        rows = tiles * 128
        tile_group = ws.take((tiles,), torch.int32)
        cursor = ws.take((E,), torch.int32)
        row_dest = ws.take((rows,), torch.int32)
        row_scale = ws.take((rows,), torch.float32)
        a_sorted = ws.take((rows, D), torch.bfloat16)
        act = ws.take((rows, Fd), torch.bfloat16)
        _check(lib().aien_moe_plan_rows(_p(expert_count), E, tiles, _p(cursor), _p(tile_group), _p(row_dest), _stream()), "moe_plan_rows")
        _check(lib().aien_moe_place_rows(_p(h), h.stride(0), _p(ids), _p(wts), _p(cursor), T, top, _p(a_sorted), D, _p(row_dest),
                                         _p(row_scale), _stream()), "moe_place_rows")
        _check(lib().aien_gemm_tc_grouped(_p(a_sorted), D, _p(w_up), D, E, _p(act), BF16, Fd, _p(tile_group), tiles, None, None,
                                          Fd, D, 2 + int(act_kind), _stream()), "gemm_tc_grouped(up)")
        _check(lib().aien_gemm_tc_grouped(_p(act), Fd, _p(w_down), Fd, E, _p(parts), BF16, D, _p(tile_group), tiles, _p(row_dest),
                                          _p(row_scale), D, Fd, 0, _stream()), "gemm_tc_grouped(down)")
        return parts
    act = ws.take((T * top, Fd), ctx.dtype)
    moe_expert_up(h, w_up, ids, act, top, act_kind)
    moe_expert_down(act, w_down, ids, wts, parts, top)
    return parts


def act_rows(a: torch.Tensor, act_kind: int) -> None:
    """a = f(a) in place: 0 the erf gelu, 1 the tanh gelu, 2 the square of relu."""
    _dev(a)
    assert a.is_contiguous()
    _check(lib().aien_act_rows(_p(a), dt(a), a.numel(), int(act_kind), _stream()), "act_rows")


def convert(src: torch.Tensor, dst: torch.Tensor) -> None:
    _dev(src, dst)
    assert src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel()
    _check(lib().aien_convert(_p(src), dt(src), _p(dst), dt(dst), src.numel(), _stream()), "convert")


# ---------------------------------------------------------------------------- matrix products
def gemm_simple(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] . w[N,K]^T, float32 accumulation on the CUDA cores, any sizes."""
    _dev(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib().aien_gemm_simple(_p(a), dt(a), a.stride(0), _p(w), dt(w), w.stride(0), _p(out), dt(out), out.stride(0),
                                  M, N, K, _stream()), "gemm_simple")


# ---------------------------------------------------------------------------- attention
def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                            max_blocks: int, seq_of_token: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                            num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                            scale: float, chunk: int = 0, sinks: Optional[torch.Tensor] = None, value_dim: int = 0,
                            token_list: Optional[torch.Tensor] = None, num_tokens: Optional[int] = None,
                            head_scale: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None,
                            gate: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Causal attention of T query tokens over their requests' pages.  q [T, nq*hd] (row stride
    free), caches [slots, nkv, hd], block_table int32 [S, max_blocks], out [T, nq*hd].
    ``chunk`` > 0: a token sees only the keys of its own chunk of that many positions.  ``sinks``
    (float32 [nq]): one more term exp(sink) in every head's softmax denominator.  ``value_dim``:
    size of a value when it differs from the head size (v_cache [slots, nkv, value_dim], out [T, nq*value_dim]).
    ``token_list`` (int32) with ``num_tokens``: only these tokens of the step are served.  Per head (float32 [nq]):
    ``head_scale`` multiplies the scaled score, ``slopes`` takes slope * (query position - key position) off it;
    ``gate`` (float32 [T, >= nq], row stride free): the head's output is multiplied by sigmoid(gate[t, h]).
    ``softcap`` c > 0: the scaled score s becomes c * tanh(s / c)."""
    _dev(q, k_cache, v_cache, block_table, seq_of_token, positions, out, sinks, token_list, head_scale, slopes, gate)
    for v in (head_scale, slopes):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == num_q_heads)
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[1] >= num_q_heads)
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == num_q_heads
    T = q.shape[0] if token_list is None else int(num_tokens)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == v_cache.dtype
    assert block_table.dtype == torch.int32 and seq_of_token.dtype == torch.int32 and positions.dtype == torch.int32
    assert token_list is None or (token_list.dtype == torch.int32 and token_list.numel() >= T)
    _check(lib().aien_paged_attention_generic(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), max_blocks, _p(seq_of_token), _p(positions),
        _p(out), out.stride(0), num_q_heads, num_kv_heads, head_dim, page_size, window, float(scale),
        dt(q), dt(k_cache), T, int(chunk), _p(sinks), int(value_dim), _p(token_list), _p(head_scale), _p(slopes), _p(gate),
        gate.stride(0) if gate is not None else 0, float(softcap or 0.0), _stream()), "paged_attention_generic")


# ---------------------------------------------------------------------------- sampling
def argmax_rows(logits: torch.Tensor, out_ids: torch.Tensor) -> None:
    _dev(logits, out_ids)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and out_ids.dtype == torch.int32 and out_ids.numel() >= R
    _check(lib().aien_argmax_rows(_p(logits), R, V, _p(out_ids), _stream()), "argmax_rows")


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, top_k: torch.Tensor,
                seeds: torch.Tensor, request_ids: torch.Tensor, positions: torch.Tensor, scratch: torch.Tensor,
                out_ids: torch.Tensor, out_logprob: Optional[torch.Tensor] = None) -> None:
    """One token per row; see csrc/kernels/sampling.cu for the rules.  scratch: R*V float32.
    ``out_logprob`` (float32 [R]) also receives the log-probability of each chosen token."""
    _dev(logits, temperature, top_p, top_k, seeds, request_ids, positions, scratch, out_ids, out_logprob)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and top_k.dtype == torch.int32
    assert seeds.dtype == torch.int64 and request_ids.dtype == torch.int64 and positions.dtype == torch.int32
    assert scratch.dtype == torch.float32 and scratch.numel() >= R * V and out_ids.dtype == torch.int32
    if out_logprob is not None:
        assert out_logprob.dtype == torch.float32 and out_logprob.numel() >= R and out_logprob.is_contiguous()
        _check(lib().aien_sample_rows_logprob(_p(logits), R, V, _p(temperature), _p(top_p), _p(top_k), _p(seeds), _p(request_ids),
                                              _p(positions), _p(scratch), _p(out_ids), _p(out_logprob), _stream()), "sample_rows_logprob")
        return
    _check(lib().aien_sample_rows(_p(logits), R, V, _p(temperature), _p(top_p), _p(top_k), _p(seeds), _p(request_ids),
                                  _p(positions), _p(scratch), _p(out_ids), _stream()), "sample_rows")


# ---------------------------------------------------------------------------- decode product
GEMV_MAX_ROWS = 16          # what the decode products take
# Up to how many rows a step's products go to them: beyond 8 rows (their second token tile) the
# tensor-core tile kernel with 32 rows of A per stage is faster (Qwen3-8B shape, batch 9 / 12 / 16:
# 4.15 / 4.19 / 4.21 ms a step against 3.59 / 3.68 / 3.75 ms).
GEMV_ROUTE_ROWS = 8
# "stream": persistent TMA-fed kernel; "direct": loads straight from global memory into fragments
GEMV_IMPL = __import__("os").environ.get("AIEN_B200_GEMV", "stream").strip().lower()


def gemv_supports(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    K_ = a.shape[1]
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] <= GEMV_MAX_ROWS and K_ % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(-1) == 1)


def gemv_splits(N: int, K_: int) -> int:
    """How many ranges K is cut into across CTAs, from the weight's shape alone (never from the
    batch): enough CTAs to fill the GPU when the matrix has few rows."""
    if GEMV_IMPL == "stream" and K_ % 64 == 0:
        return 1                     # the persistent kernel balances itself; no partial products needed
    tiles = (N + 15) // 16
    return max(1, min(8, 1184 // tiles, K_ // 512))


def gemv(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0) -> None:
    """out = a . w^T for up to 16 rows of a (bfloat16, float32 accumulation).  ``epilogue=1``:
    w holds gate|up rows interleaved in groups of 8 and out = silu(gate)*up with N/2 columns.
    ``epilogue=3`` / ``4`` / ``5`` (the streamed kernel, bfloat16 out): the gelu in its erf / tanh form, the square of relu.
    ``out`` of shape [P, M, N] float32 receives P partial products over P ranges of K."""
    _dev(a, w, out)
    M, K_ = a.shape
    N = w.shape[0]
    splits, part_stride = 1, 0
    if out.dim() == 3:
        assert epilogue == 0 and out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape[1:]) == (M, N)
        splits, part_stride = out.shape[0], M * N
    else:
        assert w.shape[1] == K_ and out.shape == (M, N // 2 if epilogue == 1 else N)
    assert epilogue in (0, 1) or gemv_takes_activation(K_)
    fn = lib().aien_gemv_stream_bf16 if (GEMV_IMPL == "stream" and K_ % 64 == 0) else lib().aien_gemv_bf16
    _check(fn(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), dt(out), out.stride(-2), M, N, K_,
              epilogue, splits, part_stride, _stream()), "gemv_bf16")


def gemv_takes_activation(K_: int) -> bool:
    """Whether the decode product over K_ columns has the gelu epilogues (the streamed kernel has, the direct one has not)."""
    return GEMV_IMPL == "stream" and K_ % 64 == 0


def gemv_stream_error() -> int:
    """Error code left by a bounded wait inside the streamed decode product (0: none); clears it."""
    return int(lib().aien_gemv_stream_error())


def gemm_tc_supports(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    K_ = a.shape[1]
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K_ % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0) -> None:
    """out = a . w^T on the tcgen05 tensor cores (bfloat16 operands, float32 accumulation in
    tensor memory).  ``epilogue=1``: w holds gate|up rows interleaved in runs of 8 and
    out = silu(gate)*up with N/2 columns.  ``epilogue=2`` / ``3`` / ``4`` (bfloat16 out): the gelu in its erf / tanh
    form, the square of relu."""
    _dev(a, w, out)
    M, K_ = a.shape
    N = w.shape[0]
    splits, part_stride = 1, 0
    if out.dim() == 3:                      # float32 partial products over ranges of K, for the consumer to add
        assert epilogue == 0 and out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape[1:]) == (M, N)
        assert out.shape[0] == gemm_tc_ranges(K_, out.shape[0])
        splits, part_stride = out.shape[0], M * N
    else:
        assert w.shape[1] == K_ and out.shape == (M, N // 2 if epilogue == 1 else N)
    _check(lib().aien_gemm_tc(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), dt(out), out.stride(-2), M, N, K_,
                              epilogue, splits, part_stride, _stream()), "gemm_tc")


# Upper bound of the float32 partial products one deferred product may leave in the workspace:
# ranges x M x N <= (296 / tiles) x (tiles x 128 x 128) elements within one wave of units; ranges over
# several waves (gemm_tc_splits) are taken only while they fit.
PARTIALS_MAX_BYTES = 40 * 1024 * 1024 + (1 << 16)


def gemm_tc_ranges(K_: int, splits: int) -> int:
    """How many ranges of K the tensor-core kernel makes when asked for ``splits``."""
    return int(lib().aien_gemm_tc_ranges(int(K_), int(splits)))


def gemm_tc_takes_256_rows(M: int, N: int, K_: int, splits: int = 1) -> bool:
    """Whether gemm_tc runs this product on the persistent kernel with tiles of 256 x 256."""
    return bool(lib().aien_gemm_tc_m256_supports(int(M), int(N), int(K_), int(splits)))


def gemm_tc_splits(M: int, N: int, K_: int) -> int:
    """Ranges of K for a product with few rows: enough CTAs to occupy the GPU (148 SMs, two CTAs
    each) when the tile grid alone is small.  Depends on the shapes only."""
    if M > 64 and N >= 256:
        # the persistent kernel with 128 x 256 tiles: as many ranges (eight at most) as still give every range
        # 8 k-blocks and every SM at most one unit (128 rows x 4,096 x 12,288: 16 tiles, 4 -> 8 ranges, 29.9 -> 25.9 us)
        tiles = ((M + 127) // 128) * ((N + 255) // 256)
        if tiles >= 148:
            return 1
        one_wave = gemm_tc_ranges(K_, max(1, min(8, 148 // tiles, K_ // 512)))
        # Three sevenths of the SMs or more idle over a long K: ranges over two or three waves of units can still be
        # faster, the float32 partial products they write and their consumer reads counted in (536 rows x 4,096
        # x 12,288: 80 tiles; one range 80.1 us, three 60.0 us + 3.5 us for the consumer; x 14,336: 89.9 -> 68.4 us).
        # Costs in cycles: a k-block of a tile 768, a tile's fixed part 1,500, a partly filled GPU clocks higher,
        # partial products at 3,800 bytes a cycle both ways.  Taken when a tenth faster by this count.
        kb = (K_ + 63) // 64

        def cost(r: int) -> float:
            units = tiles * r
            waves = (units + 147) // 148
            c = waves * (-(-kb // r) * 768 + 1500)
            if units < 148:
                c *= 0.75 + 0.25 * units / 148
            return c + ((r * M * N * 8) / 3800 + 2000 if r > 1 else 0)

        best, best_cost = one_wave, cost(one_wave)
        if tiles * 7 > 148 * 4:         # with more than four sevenths of the SMs busy it measured no faster (724 rows: 96 tiles)
            return best
        for r in range(one_wave + 1, 9):
            if K_ // 512 < r or r * M * N * 4 > PARTIALS_MAX_BYTES - (1 << 16) or gemm_tc_ranges(K_, r) != r:
                continue
            if cost(r) < 0.9 * best_cost:
                best, best_cost = r, cost(r)
        return best
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    if tiles >= 148:
        return 1
    return gemm_tc_ranges(K_, max(1, min(8, 296 // tiles, K_ // 512)))


def small_step_products_fuse(dtype: torch.dtype, num_tokens: int) -> bool:
    """Whether the products of this step are the streamed decode kernel, whose epilogues can do a
    norm's work (residual add and preparation before it, the row factor after it).  The one place
    that knows the routing; norms of any kind ask here."""
    return dtype == torch.bfloat16 and num_tokens <= GEMV_ROUTE_ROWS and GEMV_IMPL == "stream"


def FUSED_NORM_SCRATCH_BYTES(hidden: int) -> int:
    """What a product that ends a residual branch takes for the next norm: bfloat16 rows and partial sums, with slack."""
    return GEMV_MAX_ROWS * hidden * 2 + 1024 * 16 * 4 + 1024


def gemv_stream_fusable(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the streamed decode product, and so its fusions with the norm around it, takes a . w^T."""
    return (GEMV_IMPL == "stream" and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2
            and a.shape[0] <= GEMV_MAX_ROWS and a.shape[1] % 64 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemv_stream_grid(n_rows: int) -> int:
    """Number of CTAs (and so of partial sums of squares) of a streamed product over ``n_rows`` rows of W."""
    return int(lib().aien_gemv_stream_grid(int(n_rows)))


def gemv_scaled(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ssq: torch.Tensor, parts: int, eps: float, epilogue: int = 0) -> None:
    """out = (a . w^T) with row t multiplied by 1/sqrt(sum_p ssq[p, t] / K + eps) first; epilogue 1
    then applies silu(gate)*up over rows of w interleaved in runs of 8."""
    _dev(a, w, out, ssq)
    M, Kd = a.shape
    N = w.shape[0]
    assert gemv_stream_fusable(a, w) and ssq.dtype == torch.float32 and ssq.is_contiguous() and ssq.numel() >= parts * 16
    assert out.shape == (M, N // 2 if epilogue else N) and out.stride(1) == 1
    _check(lib().aien_gemv_stream_scaled(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), dt(out), out.stride(0), M, N, Kd,
                                         int(epilogue), _p(ssq), int(parts), float(eps), _stream()), "gemv_stream_scaled")


def gemv_residual(a: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, norm_w: torch.Tensor, xw: torch.Tensor, ssq_out: torch.Tensor) -> int:
    """resid += a . w^T in place (float32); xw = bfloat16(resid * norm_w); ssq_out[p, t] = partial
    sums of resid[t]^2.  Returns the number of parts written."""
    _dev(a, w, resid, norm_w, xw, ssq_out)
    M, Kd = a.shape
    N = w.shape[0]
    parts = gemv_stream_grid(N)
    assert gemv_stream_fusable(a, w) and resid.dtype == torch.float32 and resid.shape == (M, N) and resid.stride(1) == 1
    assert xw.dtype == torch.bfloat16 and xw.shape == (M, N) and xw.stride(1) == 1 and norm_w.numel() == N and norm_w.is_contiguous()
    assert ssq_out.dtype == torch.float32 and ssq_out.is_contiguous() and ssq_out.numel() >= parts * 16
    _check(lib().aien_gemv_stream_residual(_p(a), a.stride(0), _p(w), w.stride(0), _p(resid), resid.stride(0), _p(norm_w), dt(norm_w),
                                           _p(xw), xw.stride(0), _p(ssq_out), M, N, Kd, _stream()), "gemv_stream_residual")
    return parts


def feed_token_ids(token_ids: torch.Tensor, src: torch.Tensor, prev: torch.Tensor) -> None:
    """token_ids[i] = prev[src[i]] where src[i] >= 0 (int32 device tensors)."""
    _dev(token_ids, src, prev)
    assert token_ids.dtype == torch.int32 and src.dtype == torch.int32 and prev.dtype == torch.int32 and src.numel() >= token_ids.numel()
    _check(lib().aien_feed_token_ids(_p(token_ids), _p(src), _p(prev), token_ids.numel(), _stream()), "feed_token_ids")


def copy_rows(storage: torch.Tensor, src: int, dst: int, count: int = 1) -> None:
    """storage[:, dst:dst+count] = storage[:, src:src+count] for a contiguous [runs, rows, ...] tensor: the copy
    of a cache page (count = tokens a page) or of a state slot in every run of a cache group."""
    _dev(storage)
    assert storage.is_contiguous() and storage.dim() >= 2
    row = storage[0, 0].numel() * storage.element_size()
    _check(lib().aien_copy_spans(_p(storage), storage.shape[1] * row, storage.shape[0], src * row, dst * row, count * row, _stream()),
           "copy_spans")


def zero_fill(t: torch.Tensor) -> torch.Tensor:
    """Zeroes a contiguous device tensor in place (the cache pools at start: the paged kernels load whole pages)."""
    _dev(t)
    assert t.is_contiguous()
    _check(lib().aien_zero_fill(_p(t), t.numel() * t.element_size(), _stream()), "zero_fill")
    return t


def scale_rows_ssq(xw: torch.Tensor, ssq: torch.Tensor, parts: int, eps: float, out: torch.Tensor) -> None:
    """out[t] = bfloat16(xw[t] / sqrt(sum_p ssq[p, t] / H + eps)): the rest of a norm whose weight is inside xw."""
    _dev(xw, ssq, out)
    T, H = xw.shape
    assert xw.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape == (T, H) and xw.stride(1) == 1 and out.stride(1) == 1
    _check(lib().aien_scale_rows_ssq(_p(xw), xw.stride(0), _p(ssq), int(parts), float(eps), _p(out), out.stride(0), T, H, _stream()),
           "scale_rows_ssq")


def gemm_tc_error() -> int:
    """Error code left by a bounded wait inside the tensor-core kernel (0: none); clears it."""
    return int(lib().aien_gemm_tc_error())


# ---------------------------------------------------------------------------- attention choice
DECODE_CHUNK = 128
PREFILL_TILE = 128         # query tokens per CTA of the prefill attention kernel


def attention_workspace_bytes(lim, num_heads: int, head_dim: int) -> int:
    """Scratch of the split-key decode kernel for the largest decode-only step."""
    splits = (lim.max_context + DECODE_CHUNK - 1) // DECODE_CHUNK
    return lim.max_seqs * num_heads * splits * (head_dim + 2) * 4 + 1024 \
        + prefill_split_scratch_bytes(PREFILL_SPLIT_MAX_TILES, num_heads, head_dim, lim.max_context) + 256


_ticket_counters: Optional[torch.Tensor] = None


_DECODE_ATTN_IMPL = __import__("os").environ.get("AIEN_B200_DECODE_ATTENTION", "stream").strip().lower()     # "stream" | "direct"


def decode_stream_supports(num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, max_splits: int) -> bool:
    """Whether the streamed decode attention kernel takes this case (head size 64 or 128, pages that divide 128)."""
    return bool(lib().aien_paged_attention_decode_stream_supports(num_q_heads, num_kv_heads, head_dim, page_size, max_splits))


def paged_attention_decode(q, k_cache, v_cache, block_table, max_blocks, seq_of_token, positions, out,
                           part_out, part_ml, num_q_heads, num_kv_heads, head_dim, page_size, window, scale,
                           max_splits, token_list=None, num_tokens=None, impl: Optional[str] = None, chunk: int = 0,
                           sinks: Optional[torch.Tensor] = None, head_scale: Optional[torch.Tensor] = None,
                           slopes: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Split-key decode attention; the CTA that finishes last merges the chunks.  The ticket
    counters are one small device buffer that every launch finds zero and leaves zero.
    ``impl``: "stream" (TMA ring, persistent CTAs; where the sizes allow) or "direct" (one CTA per
    chunk); both give the same bits.  Default from ``AIEN_B200_DECODE_ATTENTION``, else "stream".
    ``chunk`` > 0 (a token sees only the keys of its own chunk of that many positions; ``max_splits`` then counts
    the 128-key blocks a chunk can touch, see decode_splits) and ``sinks`` (float32 [heads]) are the direct kernel's,
    and so are the terms per head ``head_scale``, ``slopes`` and ``gate`` and the cap ``softcap`` on the scaled score (see
    :func:`paged_attention_generic`)."""
    global _ticket_counters
    _dev(q, k_cache, v_cache, block_table, seq_of_token, positions, out, part_out, part_ml, sinks, head_scale, slopes, gate)
    # seq_of_token None: token t belongs to row t of the block table.  token_list: serve only these tokens.
    T = q.shape[0] if token_list is None else int(num_tokens)
    if _ticket_counters is None:
        _ticket_counters = torch.zeros(1 << 16, dtype=torch.int32, device=q.device)
    assert T * num_kv_heads <= _ticket_counters.numel()
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert part_out.dtype == torch.float32 and part_out.numel() >= T * num_q_heads * max_splits * head_dim
    assert part_ml.dtype == torch.float32 and part_ml.numel() >= T * num_q_heads * max_splits * 2
    impl = impl or _DECODE_ATTN_IMPL
    if head_scale is not None or slopes is not None or gate is not None or softcap:
        assert not chunk and sinks is None
        _check_head_terms(num_q_heads, head_scale, slopes, gate)
        _check(lib().aien_paged_attention_decode_terms(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), max_blocks, _p(seq_of_token), _p(positions),
            _p(token_list), _p(out), out.stride(0), _p(part_out), _p(part_ml), _p(_ticket_counters), num_q_heads, num_kv_heads, head_dim,
            page_size, window, float(scale), max_splits, T, _p(head_scale), _p(slopes), _p(gate),
            gate.stride(0) if gate is not None else 0, float(softcap or 0.0), _stream()), "paged_attention_decode_terms")
        return
    if chunk or sinks is not None:
        assert sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == num_q_heads)
        _check(lib().aien_paged_attention_decode_masked(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), max_blocks, _p(seq_of_token), _p(positions),
            _p(token_list), _p(out), out.stride(0), _p(part_out), _p(part_ml), _p(_ticket_counters), num_q_heads, num_kv_heads, head_dim,
            page_size, window, float(scale), max_splits, T, int(chunk), _p(sinks), _stream()), "paged_attention_decode_masked")
        return
    if impl == "stream" and decode_stream_supports(num_q_heads, num_kv_heads, head_dim, page_size, max_splits):
        _check(lib().aien_paged_attention_decode_stream(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), k_cache.shape[0], _p(block_table), max_blocks, _p(seq_of_token),
            _p(positions), _p(token_list), _p(out), out.stride(0), _p(part_out), _p(part_ml), _p(_ticket_counters), num_q_heads,
            num_kv_heads, head_dim, page_size, window, float(scale), max_splits, T, _stream()), "paged_attention_decode_stream")
        return
    _check(lib().aien_paged_attention_decode(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), max_blocks, _p(seq_of_token), _p(positions),
        _p(token_list), _p(out), out.stride(0), _p(part_out), _p(part_ml), _p(_ticket_counters), num_q_heads, num_kv_heads, head_dim,
        page_size, window, float(scale), max_splits, T, _stream()), "paged_attention_decode")


def _check_head_terms(num_q_heads: int, head_scale, slopes, gate) -> None:
    for v in (head_scale, slopes):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == num_q_heads)
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[1] >= num_q_heads)


def attention_decode_stream_error() -> int:
    """Code left by a wait that ran out in the streamed decode attention kernel (0: none)."""
    return int(lib().aien_attention_decode_stream_error())


def paged_attention_decode_fused(ctx, q, k, v, q_norm_w, k_norm_w, eps, cos, sin, rotary_dim, group, k_cache, v_cache, out,
                                 num_q_heads, num_kv_heads, head_dim, window, scale) -> None:
    """Decode-only steps: per-head q/k norm, rotation, the write of k and v into the cache and the
    split-key attention in one launch.  q, k, v are the raw projections [T, heads*head_dim]."""
    global _ticket_counters
    _dev(q, k, v, q_norm_w, k_norm_w, cos, sin, k_cache, v_cache, out)
    T = q.shape[0]
    if _ticket_counters is None:
        _ticket_counters = torch.zeros(1 << 16, dtype=torch.int32, device=q.device)
    assert T * num_kv_heads <= _ticket_counters.numel()
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and out.stride(1) == 1
    wdt = F32
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            assert w.numel() == head_dim and w.is_contiguous()
            wdt = dt(w)
    if cos is not None:
        assert cos.shape == (T, rotary_dim // 2) and cos.is_contiguous() and sin.is_contiguous()
    splits = max(1, (ctx.max_ctx_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
    part_out = ctx.workspace.take((T * num_q_heads * splits * head_dim,), torch.float32)
    part_ml = ctx.workspace.take((T * num_q_heads * splits * 2,), torch.float32)
    k2 = k_cache.view(-1, num_kv_heads, head_dim)
    v2 = v_cache.view(-1, num_kv_heads, head_dim)
    _check(lib().aien_paged_attention_decode_fused(
        _p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(q_norm_w), _p(k_norm_w), wdt, float(eps),
        _p(cos), _p(sin), rotary_dim if cos is not None else 0, _p(group.slot_map), _p(k2), _p(v2), _p(group.block_table),
        group.max_blocks, _p(ctx.positions), _p(out), out.stride(0), _p(part_out), _p(part_ml), _p(_ticket_counters),
        num_q_heads, num_kv_heads, head_dim, group.page_size, window, float(scale), splits, T, _stream()),
        "paged_attention_decode_fused")


def decode_attention_supports(q: torch.Tensor, k_cache: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return (q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
            and num_q_heads // num_kv_heads <= 16 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


_FORCE_ATTN = __import__("os").environ.get("AIEN_B200_ATTENTION", "").strip().lower()


def paged_attention(ctx, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, group, out: torch.Tensor,
                    num_q_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float) -> None:
    """Attention of the step's tokens over one cache group; picks the kernel for the step:
    the split-key kernel when every request brings one token (bfloat16), else the generic one.
    ``AIEN_B200_ATTENTION=generic`` pins the generic kernel for debugging; ``fused`` folds the q/k
    kernel into the decode attention launch (see parts/attention.py)."""
    k2 = k_cache.view(-1, num_kv_heads, head_dim)
    v2 = v_cache.view(-1, num_kv_heads, head_dim)
    if (ctx.decode_only and _FORCE_ATTN != "generic"
            and decode_attention_supports(q, k2, num_q_heads, num_kv_heads, head_dim)):
        T = q.shape[0]
        splits = max(1, (ctx.max_ctx_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
        part_out = ctx.workspace.take((T * num_q_heads * splits * head_dim,), torch.float32)
        part_ml = ctx.workspace.take((T * num_q_heads * splits * 2,), torch.float32)
        paged_attention_decode(q, k2, v2, group.block_table, group.max_blocks, None, ctx.positions, out,
                               part_out, part_ml, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale, splits)
        return
    if (not ctx.decode_only and _FORCE_ATTN != "generic" and ctx.prefill_tiles is not None
            and prefill_attention_supports(q, k2, out, head_dim)
            and decode_attention_supports(q, k2, num_q_heads, num_kv_heads, head_dim)):
        # a mixed step: portions go through the tiled kernel, single tokens through the split-key kernel
        tile_seq, tile_q0, n = ctx.prefill_tiles
        if n > 0:
            room = prefill_split_scratch_bytes(n, num_q_heads, head_dim, ctx.max_ctx_len)
            scratch = ctx.workspace.take((room // 4,), torch.float32) if room else None
            paged_attention_prefill(q, k2, v2, group.block_table, group.max_blocks, ctx.q_start, ctx.ctx_len, tile_seq, tile_q0, n,
                                    out, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                                    scratch=scratch, max_ctx=ctx.max_ctx_len)
        tokens, nd = ctx.single_tokens if ctx.single_tokens is not None else (None, 0)
        if nd > 0:
            splits = max(1, (ctx.max_ctx_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
            part_out = ctx.workspace.take((nd * num_q_heads * splits * head_dim,), torch.float32)
            part_ml = ctx.workspace.take((nd * num_q_heads * splits * 2,), torch.float32)
            paged_attention_decode(q, k2, v2, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, out,
                                   part_out, part_ml, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                                   splits, token_list=tokens, num_tokens=nd)
        return
    paged_attention_generic(q, k2, v2, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, out,
                            num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale)


def decode_splits(max_ctx: int, chunk: int) -> int:
    """Key blocks of 128 that the split-key decode kernel runs per token: those of the longest context, or,
    under a chunk mask, those a chunk can touch."""
    splits = max(1, (max_ctx + DECODE_CHUNK - 1) // DECODE_CHUNK)
    return min(splits, (chunk + DECODE_CHUNK - 1) // DECODE_CHUNK + 1) if chunk > 0 else splits


def decode_masked_takes(num_q_heads: int, num_kv_heads: int, head_dim: int, splits: int) -> bool:
    """Whether the split-key kernel's shared memory (a block of keys and values, scores, and the merge's
    scratch, which grows with the number of blocks) stays within what a CTA can have; else the plain kernel runs."""
    G = num_q_heads // num_kv_heads
    nh = 8 * ((G + 7) // 8)
    loop = (DECODE_CHUNK * nh + 2 * nh) * 4 + nh * DECODE_CHUNK * 2
    r4 = lambda n: (n + 3) & ~3
    merge = (r4(G) + r4(splits * G) + max(r4(splits * G), 8 * head_dim)) * 4
    kv = DECODE_CHUNK * (head_dim * 2 + 16) * 2
    return ((max(loop, merge) + 127) & ~127) + kv <= 200 * 1024 - 1024


def chunk_attention_workspace_bytes(lim, num_heads: int, value_dim: int, chunk: int) -> int:
    """Scratch of attention under a chunk mask for the largest step: the partial results of the split-key kernel."""
    return lim.max_seqs * num_heads * decode_splits(lim.max_context, chunk) * (value_dim + 2) * 4 + 4096


def chunk_sink_attention(ctx, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, group, out: torch.Tensor,
                         num_q_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, window: int, chunk: int,
                         sinks: Optional[torch.Tensor], scale: float) -> None:
    """Attention of the step's tokens over one cache group under a chunk mask (``chunk`` > 0: a token
    sees the keys of its own chunk of that many positions), an optional window, and an optional
    per-head softmax sink; values of size ``value_dim``.  Picks the kernel for the step."""
    k2 = k_cache.view(-1, num_kv_heads, head_dim)
    v2 = v_cache.view(-1, num_kv_heads, value_dim)
    split_key = (_FORCE_ATTN != "generic" and value_dim == head_dim
                 and decode_attention_supports(q, k2, num_q_heads, num_kv_heads, head_dim) and out.dtype == torch.bfloat16)

    def single_tokens(tokens, n):
        """The tokens that come alone: the split-key kernel over the 128-key blocks their chunk touches."""
        splits = decode_splits(ctx.max_ctx_len, chunk)
        part_out = ctx.workspace.take((n * num_q_heads * splits * head_dim,), torch.float32)
        part_ml = ctx.workspace.take((n * num_q_heads * splits * 2,), torch.float32)
        paged_attention_decode(q, k2, v2, group.block_table, group.max_blocks, None if tokens is None else ctx.seq_of_token,
                               ctx.positions, out, part_out, part_ml, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                               splits, token_list=tokens, num_tokens=n, impl="direct", chunk=chunk, sinks=sinks)

    if ctx.decode_only and split_key and decode_masked_takes(num_q_heads, num_kv_heads, head_dim, decode_splits(ctx.max_ctx_len, chunk)):
        single_tokens(None, q.shape[0])
        return
    if (not ctx.decode_only and _FORCE_ATTN != "generic" and ctx.prefill_tiles is not None and value_dim == head_dim
            and prefill_attention_supports(q, k2, out, head_dim)):
        # portions go through the tiled tensor-core kernels (tcgen05 for heads of 64 or 128, else mma.sync), which
        # visit only the key blocks that a tile's chunks reach; the single tokens beside them through the plain kernel
        tile_seq, tile_q0, n = ctx.prefill_tiles
        if n > 0:
            paged_attention_prefill(q, k2, v2, group.block_table, group.max_blocks, ctx.q_start, ctx.ctx_len, tile_seq, tile_q0, n,
                                    out, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                                    chunk=chunk, sinks=sinks)
        tokens, nd = ctx.single_tokens if ctx.single_tokens is not None else (None, 0)
        if nd > 0 and split_key and decode_masked_takes(num_q_heads, num_kv_heads, head_dim, decode_splits(ctx.max_ctx_len, chunk)):
            single_tokens(tokens, nd)
        elif nd > 0:
            paged_attention_generic(q, k2, v2, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, out,
                                    num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                                    chunk=chunk, sinks=sinks, value_dim=value_dim, token_list=tokens, num_tokens=nd)
        return
    paged_attention_generic(q, k2, v2, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, out,
                            num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                            chunk=chunk, sinks=sinks, value_dim=value_dim)


def prefill_attention_supports(q: torch.Tensor, k_cache: torch.Tensor, out: torch.Tensor, head_dim: int) -> bool:
    return (q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 128
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0)


_PREFILL_IMPL = __import__("os").environ.get("AIEN_B200_PREFILL", "tc").strip().lower()     # "tc" | "mma"


def prefill_tc_supports(q, out, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill kernel takes this case (head size 64 or 128, pages that divide 128)."""
    return (bool(lib().aien_paged_attention_prefill_tc_supports(head_dim, page_size)) and q.stride(0) % 8 == 0
            and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


PREFILL_SPLIT_MAX_TILES = 8          # steps with more tiles fill the GPU without cutting the keys


def prefill_split_scratch_bytes(num_tiles: int, num_q_heads: int, head_dim: int, max_ctx: int) -> int:
    """Room the tcgen05 prefill kernel can use to cut the keys of `num_tiles` tiles into ranges
    (float32 partial results); 0 where it would not cut."""
    if num_tiles <= 0 or num_tiles > PREFILL_SPLIT_MAX_TILES or max_ctx < 8 * PREFILL_TILE:
        return 0
    return num_tiles * PREFILL_TILE * num_q_heads * 8 * (head_dim + 2) * 4


def paged_attention_prefill(q, k_cache, v_cache, block_table, max_blocks, q_start, ctx_len, tile_seq, tile_q0, num_tiles,
                            out, num_q_heads, num_kv_heads, head_dim, page_size, window, scale, impl: Optional[str] = None,
                            scratch: Optional[torch.Tensor] = None, max_ctx: int = 0, splits: int = 0, chunk: int = 0,
                            sinks: Optional[torch.Tensor] = None, head_scale: Optional[torch.Tensor] = None,
                            slopes: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Causal attention of portions of prompts over their requests' pages (bfloat16, tensor
    cores).  ``tile_seq``/``tile_q0``: for every 128-token query tile, the index of its request in
    the step and the tile's offset inside that request's portion.  ``impl``: "tc" (tcgen05, where
    the sizes allow) or "mma" (mma.sync); default from ``AIEN_B200_PREFILL``, else "tc".
    ``scratch`` (float32, optional) with ``max_ctx`` (an upper bound of the contexts) lets the
    tcgen05 kernel cut the keys of a step with few tiles into ranges that run on separate SMs;
    ``splits`` > 0 asks for that many ranges (tests).  ``chunk`` > 0 (a query sees only the keys of
    its own chunk of that many positions) and ``sinks`` (float32 [heads], one more term exp(sink) in
    the softmax denominator): both kernels take them; the tcgen05 kernel then keeps every tile's keys in one range.
    ``head_scale``, ``slopes``, ``gate`` (see :func:`paged_attention_generic`): the tcgen05 kernel's alone; it keeps
    every tile's keys in one range with these too.  ``softcap`` c > 0 (the scaled score s becomes c * tanh(s / c)): the
    tcgen05 kernel's alone; it leaves the key ranges as they are."""
    _dev(q, k_cache, v_cache, block_table, q_start, ctx_len, tile_seq, tile_q0, out, sinks, head_scale, slopes, gate)
    terms = head_scale is not None or slopes is not None or gate is not None or bool(softcap)
    _check_head_terms(num_q_heads, head_scale, slopes, gate)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == num_q_heads)
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    for t in (block_table, q_start, ctx_len, tile_seq, tile_q0):
        assert t.dtype == torch.int32
    impl = impl or _PREFILL_IMPL
    if impl == "tc" and prefill_tc_supports(q, out, head_dim, page_size):
        if scratch is not None:
            _dev(scratch)
            assert scratch.dtype == torch.float32 and scratch.is_contiguous()
        _check(lib().aien_paged_attention_prefill_tc_terms(
            _p(q), q.stride(0), q.shape[0], _p(k_cache), _p(v_cache), k_cache.shape[0], _p(block_table), max_blocks, _p(q_start),
            _p(ctx_len), _p(tile_seq), _p(tile_q0), num_tiles, _p(out), out.stride(0), num_q_heads, num_kv_heads, head_dim,
            page_size, window, float(scale), _p(scratch) if scratch is not None else None,
            scratch.numel() * 4 if scratch is not None else 0, int(max_ctx), int(splits), int(chunk), _p(sinks),
            _p(head_scale), _p(slopes), _p(gate), gate.stride(0) if gate is not None else 0, float(softcap or 0.0), _stream()),
            "paged_attention_prefill_tc")
        return
    if terms:
        raise KernelError("paged_attention_prefill: only the tcgen05 kernel takes terms per head")
    _check(lib().aien_paged_attention_prefill(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), max_blocks, _p(q_start), _p(ctx_len), _p(tile_seq),
        _p(tile_q0), num_tiles, _p(out), out.stride(0), num_q_heads, num_kv_heads, head_dim, page_size, window,
        float(scale), int(chunk), _p(sinks), _stream()), "paged_attention_prefill")


def attention_prefill_tc_error() -> int:
    """Code left by a wait that ran out in the tcgen05 prefill attention kernel (0: none)."""
    return int(lib().aien_attention_prefill_tc_error())


# ---------------------------------------------------------------------------- bounded waits
# The kernels whose mbarrier waits are bounded, in the order of the words collect_wait_errors writes.
WAIT_KERNELS = ("gemm_tc", "gemv_stream", "attention_prefill_tc", "attention_decode_stream")


def collect_wait_errors(out: torch.Tensor) -> None:
    """out[0:4] (int32, device) = the error words of WAIT_KERNELS, read in the stream behind
    whatever was launched before.  The words stay set until read_wait_errors() clears them."""
    _dev(out)
    assert out.dtype == torch.int32 and out.numel() >= 4 and out.is_contiguous()
    _check(lib().aien_collect_wait_errors(_p(out), _stream()), "collect_wait_errors")


def read_wait_errors() -> tuple:
    """The four error words, read with synchronous copies (the device is idle afterwards) and
    cleared.  All zero: every bounded wait so far was met."""
    return (gemm_tc_error(), gemv_stream_error(), attention_prefill_tc_error(), attention_decode_stream_error())


def wait_error_message(words) -> str:
    """'' when all words are zero, else which kernels gave up and with which code."""
    bad = [f"{name} (code {int(w)})" for name, w in zip(WAIT_KERNELS, words) if int(w) != 0]
    if not bad:
        return ""
    return ("a bounded wait ran out inside " + ", ".join(bad) +
            ": the results of the step are not valid (a broken TMA / tensor-core pipeline, not a property of the inputs)")


# ---------------------------------------------------------------------------- norms around a sublayer, scaled ends
def embed_gather_scaled(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor, scale: float) -> None:
    """x[t] = table[ids[t]] * scale as float32."""
    _dev(table, ids, x)
    T, H = x.shape
    assert table.is_contiguous() and x.is_contiguous() and ids.dtype == torch.int32 and x.dtype == torch.float32
    assert table.shape[1] == H and ids.numel() >= T
    _check(lib().aien_embed_gather_scaled(_p(table), dt(table), _p(ids), _p(x), T, H, table.shape[0], float(scale), _stream()),
           "embed_gather_scaled")


def post_norm_add(x: torch.Tensor, a: torch.Tensor, weight: torch.Tensor, eps: float, mult: float = 1.0,
                  next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0, h: Optional[torch.Tensor] = None) -> None:
    """x += mult * y / sqrt(mean(y^2) + eps) * weight with y = a ([T,H], or float32 parts [P,T,H] added in order), in
    float32; then ``h`` (optional, [T,H]) = x / sqrt(mean(x^2) + next_eps) * next_weight, or the plain copy of the new
    x when ``next_weight`` is None."""
    _dev(x, a, weight, next_weight, h)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and weight.numel() == H and weight.is_contiguous()
    assert next_weight is None or (next_weight.numel() == H and next_weight.is_contiguous() and h is not None)
    assert h is None or (h.is_contiguous() and tuple(h.shape) == (T, H))
    pa, da, na, sa = _source(a, x.shape)
    _check(lib().aien_post_norm_add(_p(x), pa, da, na, sa, _p(weight), dt(weight), float(eps), float(mult), _p(next_weight),
                                    dt(next_weight) if next_weight is not None else F32, float(next_eps), _p(h),
                                    dt(h) if h is not None else F32, T, H, _stream()), "post_norm_add")


def gelu_times_table(z: torch.Tensor, table: torch.Tensor, col0: int, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col0 + j] for the n columns of out."""
    _dev(z, table, ids, out)
    T, n = out.shape
    assert z.shape == (T, n) and z.stride(1) == 1 and out.stride(1) == 1 and table.is_contiguous() and table.dim() == 2
    assert 0 <= col0 and col0 + n <= table.shape[1] and ids.dtype == torch.int32 and ids.numel() >= T
    _check(lib().aien_gelu_times_table(_p(z), dt(z), z.stride(0), _p(table), dt(table), table.shape[1], int(col0), _p(ids),
                                       table.shape[0], _p(out), dt(out), out.stride(0), T, n, _stream()), "gelu_times_table")


def softcap(v: torch.Tensor, cap: float) -> None:
    """v = cap * tanh(v / cap) in place (float32)."""
    _dev(v)
    assert v.dtype == torch.float32 and v.is_contiguous()
    _check(lib().aien_softcap(_p(v), v.numel(), float(cap), _stream()), "softcap")


# ---------------------------------------------------------------------------- mixers with a state of fixed size
def decay_linear_attention(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: torch.Tensor, state: torch.Tensor,
                           slot_map: torch.Tensor, q_start: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                           num_seqs: int, heads: int, dim: int, vdim: int, scratch: Optional[torch.Tensor] = None,
                           single_tokens: bool = False) -> None:
    """Per head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v = silu of the columns of ``proj`` [T, *]
    at q_off (heads*dim), k_off (heads*dim), v_off (heads*vdim).  ``state`` float32 [slots, heads, dim, vdim]: request s
    of the step (tokens q_start[s]..q_start[s+1]) continues from slot slot_map[s], from zero when its first token has
    position 0, and leaves its state there.  ``out`` float32 [T, heads*vdim].  With ``scratch`` (float32,
    ``decay_linear_attention_scratch(T, num_seqs, ...)`` numbers) the chunks of a portion run side by side in three
    launches (for portions of prompts); without it one CTA walks a portion's chunks in order.  ``single_tokens``: every
    request brings exactly one token, and the state streams through a kernel made for that."""
    _dev(proj, decay, state, slot_map, q_start, positions, out)
    assert proj.stride(1) == 1 and out.dtype == torch.float32 and out.stride(1) == 1 and out.shape[1] == heads * vdim
    assert decay.dtype == torch.float32 and decay.numel() == heads and decay.is_contiguous()
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim)
    for t in (slot_map, q_start, positions):
        assert t.dtype == torch.int32
    assert max(q_off, k_off) + heads * dim <= proj.shape[1] and v_off + heads * vdim <= proj.shape[1]
    if scratch is not None:
        T = proj.shape[0]
        assert scratch.dtype == torch.float32 and scratch.is_contiguous() and out.shape[0] == T
        assert scratch.numel() >= decay_linear_attention_scratch(T, num_seqs, heads, dim, vdim)
        _check(lib().aien_decay_linear_attention_chunked(_p(proj), dt(proj), proj.stride(0), int(q_off), int(k_off), int(v_off), _p(decay),
                                                         _p(state), _p(slot_map), _p(q_start), _p(positions), _p(out), out.stride(0),
                                                         _p(scratch), T, int(num_seqs), int(heads), int(dim), int(vdim), _stream()),
               "decay_linear_attention_chunked")
        return
    _check(lib().aien_decay_linear_attention(_p(proj), dt(proj), proj.stride(0), int(q_off), int(k_off), int(v_off), _p(decay),
                                             _p(state), _p(slot_map), _p(q_start), _p(positions), _p(out), out.stride(0),
                                             int(num_seqs), int(heads), int(dim), int(vdim), 1 if single_tokens else 0, _stream()),
           "decay_linear_attention")


def decay_linear_attention_scratch(num_tokens: int, num_seqs: int, heads: int, dim: int, vdim: int) -> int:
    """float32 numbers the chunked form needs: one state-sized block per chunk of 64 tokens, at most T / 64 + S chunks."""
    return (num_tokens // 64 + num_seqs) * heads * dim * vdim


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[t] = o[t] / sqrt(mean(o[t]^2) + eps) * weight * sigmoid(gate[t]); o float32 [T,N], gate [T,N] (row stride free)."""
    _dev(o, gate, weight, out)
    T, N = o.shape
    assert o.dtype == torch.float32 and o.stride(1) == 1 and gate.stride(1) == 1 and out.stride(1) == 1
    assert tuple(gate.shape) == (T, N) and tuple(out.shape) == (T, N) and weight.numel() == N and weight.is_contiguous()
    _check(lib().aien_gated_rmsnorm(_p(o), o.stride(0), _p(gate), dt(gate), gate.stride(0), _p(weight), dt(weight), float(eps),
                                    _p(out), dt(out), out.stride(0), T, N, _stream()), "gated_rmsnorm")


def gated_recurrence(proj: torch.Tensor, z_off: int, x_off: int, g_off: int, bz: Optional[torch.Tensor], bx: Optional[torch.Tensor],
                     state: torch.Tensor, slot_map: torch.Tensor, q_start: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                     num_seqs: int, width: int, segments: bool = False) -> None:
    """Per channel S_t = (1 - z) S_(t-1) + z c with z = sigmoid(proj[z] + bz), u = proj[x] + bx, c = u + 1/2 (u >= 0) or
    sigmoid(u) (u < 0); out_t = S_t * silu(proj[g]).  ``state`` float32 [slots, width], slots as in decay_linear_attention.
    ``segments``: every portion is cut into 32 segments that run side by side (for portions of prompts)."""
    _dev(proj, bz, bx, state, slot_map, q_start, positions, out)
    assert proj.stride(1) == 1 and out.stride(1) == 1 and out.shape[1] == width
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == width
    assert max(z_off, x_off, g_off) + width <= proj.shape[1]
    bdt = F32
    for b in (bz, bx):
        if b is not None:
            assert b.numel() == width and b.is_contiguous()
            bdt = dt(b)
    assert bz is None or bx is None or bz.dtype == bx.dtype
    for t in (slot_map, q_start, positions):
        assert t.dtype == torch.int32
    _check(lib().aien_gated_recurrence(_p(proj), dt(proj), proj.stride(0), int(z_off), int(x_off), int(g_off), _p(bz), _p(bx), bdt,
                                       _p(state), _p(slot_map), _p(q_start), _p(positions), _p(out), dt(out), out.stride(0),
                                       int(num_seqs), int(width), 1 if segments else 0, _stream()), "gated_recurrence")


# ---------------------------------------------------------------------------- attention over a cached latent
_LATENT_IMPL = __import__("os").environ.get("AIEN_B200_LATENT_ATTENTION", "tc").strip().lower()     # "tc" | "plain": pins the plain kernels


def latent_prepare(d: torch.Tensor, q_rank: int, wq: Optional[torch.Tensor], eps: float, cq: Optional[torch.Tensor],
                   kv_off: int = 0, kv_rank: int = 0, rot_dim: int = 0, rot_dims: int = 0, wkv: Optional[torch.Tensor] = None,
                   cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                   slot_map: Optional[torch.Tensor] = None, cache: Optional[torch.Tensor] = None) -> None:
    """From the down projections d [T, *] (float32): cq = RMS norm of the first ``q_rank`` columns times ``wq``; and, with
    ``cache`` [slots, kv_rank + rot_dim], the token's cache row = RMS norm of the ``kv_rank`` columns at ``kv_off`` times
    ``wkv``, then the next ``rot_dim`` columns with their first ``rot_dims`` rotated in neighbouring pairs."""
    _dev(d, wq, cq, wkv, cos, sin, slot_map, cache)
    T = d.shape[0]
    assert d.stride(1) == 1 and (q_rank == 0 or (cq is not None and cq.stride(1) == 1 and wq is not None and wq.numel() == q_rank))
    wdt = F32
    for w in (wq, wkv):
        if w is not None:
            assert w.is_contiguous()
            wdt = dt(w)
    assert wq is None or wkv is None or wq.dtype == wkv.dtype
    if cache is not None:
        assert cache.is_contiguous() and cache.shape[-1] == kv_rank + rot_dim and wkv is not None and wkv.numel() == kv_rank
        assert slot_map is not None and slot_map.dtype == torch.int32 and slot_map.numel() >= T
        assert kv_off + kv_rank + rot_dim <= d.shape[1]
        if rot_dims:
            assert cos is not None and tuple(cos.shape) == (T, rot_dims // 2) and cos.is_contiguous() and sin.is_contiguous()
    _check(lib().aien_latent_prepare(_p(d), dt(d), d.stride(0), int(q_rank), _p(wq), _p(wkv), wdt, float(eps), _p(cq),
                                     dt(cq) if cq is not None else F32, cq.stride(0) if cq is not None else 0, int(kv_off),
                                     int(kv_rank), int(rot_dim), int(rot_dims), _p(cos), _p(sin), _p(slot_map), _p(cache),
                                     dt(cache) if cache is not None else F32, T, _stream()), "latent_prepare")


def rotate_pairs_rows(q: torch.Tensor, q_head: int, col0: int, out: torch.Tensor, o_head: int, ocol0: int, heads: int, rot_dim: int,
                      rot_dims: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor]) -> None:
    """out[t, h*o_head + ocol0 + i] = q[t, h*q_head + col0 + i], i < rot_dim, the first ``rot_dims`` of them rotated in
    neighbouring pairs by the token's angle (the rotation itself in float32)."""
    _dev(q, out, cos, sin)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1
    if rot_dims:
        assert cos is not None and tuple(cos.shape) == (T, rot_dims // 2) and cos.is_contiguous() and sin.is_contiguous()
    qv, ov = q[:, col0:], out[:, ocol0:]
    _check(lib().aien_rotate_pairs_rows(_p(qv), dt(q), q.stride(0), int(q_head), _p(ov), dt(out), out.stride(0), int(o_head), T, int(heads),
                                        int(rot_dim), int(rot_dims), _p(cos), _p(sin), _stream()), "rotate_pairs_rows")


def head_project(a: torch.Tensor, a_head: int, a_col0: int, w: torch.Tensor, out: torch.Tensor, o_head: int, o_col0: int) -> None:
    """out[t, h*o_head + o_col0 + n] = sum_k a[t, h*a_head + a_col0 + k] * w[h, n, k]: one product per head, w [heads, N, K].
    bfloat16 operands whose rows are whole aligned 16-byte pieces run on the tensor cores, everything else on the CUDA cores;
    both sum in float32."""
    _dev(a, w, out)
    heads, N, K_ = w.shape
    M = a.shape[0]
    assert a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous() and out.shape[0] == M
    assert (heads - 1) * a_head + a_col0 + K_ <= a.shape[1] and (heads - 1) * o_head + o_col0 + N <= out.shape[1]
    av, ov = a[:, a_col0:], out[:, o_col0:]
    if (_LATENT_IMPL != "plain" and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K_ % 8 == 0 and a.stride(0) % 8 == 0
            and a_head % 8 == 0 and av.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        _check(lib().aien_head_project_tc(_p(av), a.stride(0), int(a_head), _p(w), _p(ov), dt(out), out.stride(0), int(o_head), M, N, K_,
                                          heads, _stream()), "head_project_tc")
        return
    _check(lib().aien_head_project(_p(av), dt(a), a.stride(0), int(a_head), _p(w), dt(w), K_, N * K_, _p(ov), dt(out), out.stride(0),
                                   int(o_head), M, N, K_, heads, _stream()), "head_project")


def latent_attention(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, max_blocks: int, seq_of_token: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, heads: int, kv_rank: int, rot_dim: int, page_size: int,
                     window: int, scale: float, sinks: Optional[torch.Tensor]) -> None:
    """Attention of the step's tokens over cached latent rows [slots, kv_rank + rot_dim] shared by all heads: q float32
    [T, heads*(kv_rank + rot_dim)], out [T, heads*kv_rank] = the softmax-weighted sums of the rows' first kv_rank numbers.
    ``window`` > 0: a token sees itself and the window - 1 tokens before it.  ``sinks`` float32 [heads] or None."""
    _dev(q, cache, block_table, seq_of_token, positions, out, sinks)
    T = q.shape[0]
    D = kv_rank + rot_dim
    assert q.dtype == torch.float32 and q.stride(1) == 1 and q.shape[1] == heads * D and out.stride(1) == 1
    assert out.shape == (T, heads * kv_rank) and cache.is_contiguous() and cache.shape[-1] == D
    assert block_table.dtype == torch.int32 and seq_of_token.dtype == torch.int32 and positions.dtype == torch.int32
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == heads)
    _check(lib().aien_latent_attention(_p(q), q.stride(0), _p(cache), dt(cache), _p(block_table), int(max_blocks), _p(seq_of_token),
                                       _p(positions), None, _p(out), dt(out), out.stride(0), T, int(heads), int(kv_rank),
                                       int(rot_dim), int(page_size), int(window), float(scale), _p(sinks), _stream()),
           "latent_attention")



def latent_attention_tc_supports(dtype: torch.dtype, kv_rank: int, rot_dim: int) -> bool:
    """Whether the tensor-core kernel takes this case: bfloat16, a latent of 64 / 128 / 256 / 512, a rotated part that is a multiple of 16."""
    return _LATENT_IMPL != "plain" and dtype == torch.bfloat16 and bool(lib().aien_latent_attention_tc_supports(int(kv_rank), int(rot_dim)))


def latent_attention_tc(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, max_blocks: int, q_start: torch.Tensor,
                        positions: torch.Tensor, out: torch.Tensor, num_seqs: int, heads: int, kv_rank: int, rot_dim: int,
                        page_size: int, window: int, scale: float, sinks: Optional[torch.Tensor], ksplit: int = 1,
                        scratch: Optional[torch.Tensor] = None, small_tiles: bool = False) -> None:
    """latent_attention on the tensor cores.  q bfloat16 [T, heads*(kv_rank + rot_dim)] and out bfloat16 [T, heads*kv_rank],
    both contiguous; the T tokens are the portions q_start[s]..q_start[s+1] of ``num_seqs`` requests (row s of the block
    table), each portion's positions counting up from positions[q_start[s]].  ``ksplit`` > 1 deals the key blocks of every
    tile out to that many CTAs and merges their results in a second launch (steps with few tiles); ``scratch`` is then
    float32 with ``latent_attention_tc_scratch(T, heads, kv_rank, ksplit)`` numbers.  ``small_tiles``: tiles of 16 rows
    instead of 64, for steps in which every request brings one token (latents of 128 and more)."""
    _dev(q, cache, block_table, q_start, positions, out, sinks)
    T, D = q.shape[0], kv_rank + rot_dim
    assert q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and cache.shape[-1] == D
    assert q.shape[1] == heads * D and tuple(out.shape) == (T, heads * kv_rank)
    assert block_table.dtype == torch.int32 and q_start.dtype == torch.int32 and positions.dtype == torch.int32
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == heads)
    part_o = part_ml = None
    if ksplit > 1:
        _dev(scratch)
        n_o = T * heads * ksplit * kv_rank
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
        assert scratch.numel() >= latent_attention_tc_scratch(T, heads, kv_rank, ksplit)
        part_o, part_ml = scratch[:n_o], scratch[n_o:]
    _check(lib().aien_latent_attention_tc(_p(q), _p(cache), _p(block_table), int(max_blocks), _p(q_start), _p(positions), _p(out), T,
                                          int(num_seqs), int(heads), int(kv_rank), int(rot_dim), int(page_size), int(window),
                                          float(scale), _p(sinks), int(ksplit), _p(part_o), _p(part_ml), 1 if small_tiles else 0, _stream()),
           "latent_attention_tc")


LATENT_TC_TILE = 64          # (token, head) rows and keys per tile of the tensor-core kernel


def latent_attention_tc_scratch(num_tokens: int, heads: int, kv_rank: int, ksplit: int) -> int:
    return num_tokens * heads * ksplit * (kv_rank + 2) if ksplit > 1 else 0


def latent_attention_tc_small_tiles(decode_only: bool, kv_rank: int) -> bool:
    """Whether a step takes the tiles of 16 rows: every request brings one token, and the latent is wide enough."""
    return bool(decode_only) and kv_rank >= 128


def latent_attention_tc_ksplit(num_tokens: int, num_seqs: int, heads: int, max_ctx: int, window: int, small_tiles: bool = False) -> int:
    """Into how many CTAs the key blocks of a tile are dealt: enough to occupy the GPU (148 SMs, two rounds of CTAs)
    when the step has few tiles, never more than a tile has blocks.  Depends on the step's sizes only."""
    tiles = (num_tokens * heads) // (16 if small_tiles else LATENT_TC_TILE) + num_seqs
    span = min(window, max_ctx) if window > 0 else max_ctx
    blocks = max(1, (span + LATENT_TC_TILE - 1) // LATENT_TC_TILE + 1)
    return max(1, min(blocks, 296 // tiles)) if tiles <= 148 else 1


# ---------------------------------------------------------------------------- several residual streams, token shift
def replicate_streams(x: torch.Tensor) -> None:
    """x float32 [n, T, H]: copies x[0] into x[1:]."""
    _dev(x)
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 3
    _check(lib().aien_replicate_streams(_p(x), x.shape[1] * x.shape[2], x.shape[0], _stream()), "replicate_streams")


def _pending(y: Optional[torch.Tensor], T: int, H: int) -> tuple:
    if y is None:
        return 0, F32, 1, 0
    assert y.is_contiguous()
    if y.dim() == 3:
        assert y.dtype == torch.float32 and tuple(y.shape[1:]) == (T, H)
        return _p(y), F32, y.shape[0], T * H
    assert tuple(y.shape) == (T, H)
    return _p(y), dt(y), 1, 0


def hc_norm(x: torch.Tensor, y: Optional[torch.Tensor], prev: Optional[torch.Tensor], cur: torch.Tensor, weight: torch.Tensor,
            eps: float, h: torch.Tensor, shift_w: Optional[torch.Tensor] = None, shift_state: Optional[torch.Tensor] = None,
            slot_map: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None) -> None:
    """Streams x float32 [n, T, H] with sublayer packs [in(n) | out(n) | mix(n*n)] (float32; mix indexed [from, to]):
    first, when ``y`` is given (a branch output [T, H], or float32 partial products [P, T, H]), the write that ``prev``
    describes, in place: x_t <- sum_s mix[s, t] x_s + out[t] y; then u = sum_s in[s] x_s with ``cur``'s in, and
    h = u / sqrt(mean u^2 + eps) * weight.  With ``shift_w`` (a step of single tokens): h <- h + (h' - h) * shift_w,
    h' the row that request's slot ``shift_state[slot_map[t]]`` held (zeros at position 0); the slot then holds h
    as it was before the shift."""
    _dev(x, y, prev, cur, weight, h, shift_w, shift_state, slot_map, positions)
    n, T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and h.is_contiguous() and tuple(h.shape) == (T, H)
    assert cur.dtype == torch.float32 and cur.numel() == 2 * n + n * n and (prev is None or (prev.dtype == torch.float32 and prev.numel() == cur.numel()))
    assert weight.numel() == H and weight.is_contiguous()
    if shift_w is not None:
        assert shift_w.numel() == H and shift_state.dtype == torch.float32 and shift_state.is_contiguous() and shift_state.shape[-1] == H
        assert slot_map.dtype == torch.int32 and positions.dtype == torch.int32
    yp, ydt, parts, stride = _pending(y, T, H)
    _check(lib().aien_hc_norm(_p(x), n, yp, ydt, parts, stride, _p(prev), _p(cur), _p(weight), dt(weight), float(eps), _p(h), dt(h), T, H,
                              _p(shift_w), dt(shift_w) if shift_w is not None else F32, _p(shift_state), _p(slot_map), _p(positions),
                              _stream()), "hc_norm")


def token_shift(hn: torch.Tensor, shift_w: torch.Tensor, state: torch.Tensor, slot_map: torch.Tensor, seq_of_token: torch.Tensor,
                q_start: torch.Tensor, positions: torch.Tensor, h: torch.Tensor) -> None:
    """h[t] = hn[t] + (hn[t-1] - hn[t]) * shift_w within a request; the row before a portion's first token comes from
    the request's slot of ``state`` (float32 [slots, H]; zeros at position 0), which then takes the portion's last row."""
    _dev(hn, shift_w, state, slot_map, seq_of_token, q_start, positions, h)
    T, H = hn.shape
    assert hn.dtype == torch.float32 and hn.is_contiguous() and h.is_contiguous() and tuple(h.shape) == (T, H)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[-1] == H and shift_w.numel() == H
    _check(lib().aien_token_shift(_p(hn), _p(shift_w), dt(shift_w), _p(state), _p(slot_map), _p(seq_of_token), _p(q_start), _p(positions),
                                  _p(h), dt(h), T, H, _stream()), "token_shift")


def hc_sum_rows(x: torch.Tensor, y: Optional[torch.Tensor], prev: Optional[torch.Tensor], rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = sum over the streams of x[:, rows[r]], after the pending write (``y`` with the pack ``prev``) if given."""
    _dev(x, y, prev, rows, out)
    n, T, H = x.shape
    R = out.shape[0]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.dtype == torch.float32 and out.is_contiguous() and out.shape[1] == H
    assert rows.dtype == torch.int32 and rows.numel() >= R
    yp, ydt, parts, stride = _pending(y, T, H)
    _check(lib().aien_hc_sum_rows(_p(x), n, T, yp, ydt, parts, stride, _p(prev), _p(rows), _p(out), R, H, _stream()), "hc_sum_rows")


def embed_gather_sinusoid(table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, x: torch.Tensor,
                          scale: float) -> None:
    """x[t] = table[ids[t]] * scale + s(positions[t]); s(p)[2i] = sin(p f_i), s(p)[2i+1] = cos(p f_i), f = inv_freq (float64)."""
    _dev(table, ids, positions, inv_freq, x)
    T, H = x.shape
    assert table.is_contiguous() and x.is_contiguous() and x.dtype == torch.float32 and table.shape[1] == H
    assert ids.dtype == torch.int32 and positions.dtype == torch.int32 and inv_freq.dtype == torch.float64 and inv_freq.numel() >= (H + 1) // 2
    _check(lib().aien_embed_gather_sinusoid(_p(table), dt(table), _p(ids), _p(positions), _p(inv_freq), _p(x), T, H, table.shape[0],
                                            float(scale), _stream()), "embed_gather_sinusoid")


# ---------------------------------------------------------------------------- short convolutions, the delta rule
def attn_conv_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, Cq: int, Ck: int, Cv: int, wq: torch.Tensor,
                      wk: Optional[torch.Tensor], wv: Optional[torch.Tensor], taps: int, q_norm: torch.Tensor, k_norm: Optional[torch.Tensor],
                      eps: float, kv_heads: int, value_dim: int, value_norm: bool, state: Optional[torch.Tensor], state_slots: torch.Tensor,
                      seq_of_token: torch.Tensor, q_start: torch.Tensor, positions: torch.Tensor, kv_slots: Optional[torch.Tensor],
                      k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], q_out: torch.Tensor) -> None:
    """Causal convolution over time (``taps`` taps, weights [C, taps]) of the q block (and, with Ck > 0, the k and v
    blocks) of ``proj`` float32 [T, *]; RMS norm of the whole q row and of the whole k row with the plain weights
    ``q_norm`` / ``k_norm``; with ``value_norm`` every value head divided by its root mean square.  q goes to ``q_out``
    [T, Cq]; k and v to the token's slot ``kv_slots[t]`` of the caches.  ``state`` float32 [slots, (taps-1) * (Cq+Ck+Cv)]
    keeps every request's last taps-1 projected rows between steps."""
    _dev(proj, wq, wk, wv, q_norm, k_norm, state, state_slots, seq_of_token, q_start, positions, kv_slots, k_cache, v_cache, q_out)
    T = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.stride(1) == 1 and q_out.shape == (T, Cq)
    ws = [w for w in (wq, wk, wv) if w is not None]
    assert all(w.is_contiguous() and w.dtype == wq.dtype and w.shape[1] == taps for w in ws)
    assert q_norm.is_contiguous() and q_norm.numel() == Cq and (k_norm is None or (k_norm.dtype == q_norm.dtype and k_norm.numel() == Ck))
    if taps > 1:
        assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == (taps - 1) * (Cq + Ck + Cv)
    if Ck > 0:
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == v_cache.dtype and kv_slots.dtype == torch.int32
    _check(lib().aien_attn_conv_prepare(
        _p(proj), proj.stride(0), int(q_off), int(k_off), int(v_off), int(Cq), int(Ck), int(Cv), _p(wq), _p(wk), _p(wv), dt(wq), int(taps),
        _p(q_norm), _p(k_norm), dt(q_norm), float(eps), int(kv_heads), int(value_dim), 1 if value_norm else 0, _p(state), _p(state_slots),
        _p(seq_of_token), _p(q_start), _p(positions), _p(kv_slots), _p(k_cache), _p(v_cache), dt(k_cache) if k_cache is not None else dt(q_out),
        _p(q_out), dt(q_out), q_out.stride(0), T, _stream()), "attn_conv_prepare")


def delta_conv_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, b_off: int, a_off: int, qk_heads: int, dim: int, heads: int,
                       vdim: int, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, taps: int, a_log: torch.Tensor, dt_bias: torch.Tensor,
                       state: torch.Tensor, state_slots: torch.Tensor, seq_of_token: torch.Tensor, q_start: torch.Tensor,
                       positions: torch.Tensor, out: torch.Tensor, gb: torch.Tensor) -> None:
    """The inputs of the gated delta rule from ``proj`` float32 [T, *]: convolution over time and silu of q, k (qk_heads x
    dim each) and v (heads x vdim); q and k made unit vectors per head, q times dim^-1/2 -> ``out`` float32 [T, q | k | v];
    per head the decay exp(-exp(a_log) * softplus(a + dt_bias)) and beta = sigmoid(b) -> ``gb`` float32 [T, 2 * heads].
    ``state`` float32 [slots, n]: the first (taps-1) * channels numbers of a slot are the convolution's."""
    _dev(proj, wq, wk, wv, a_log, dt_bias, state, state_slots, seq_of_token, q_start, positions, out, gb)
    T = proj.shape[0]
    C = 2 * qk_heads * dim + heads * vdim
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and out.dtype == torch.float32 and out.shape == (T, C) and out.stride(1) == 1
    assert gb.dtype == torch.float32 and gb.shape == (T, 2 * heads) and gb.stride(1) == 1
    assert all(w.is_contiguous() and w.dtype == wq.dtype and w.shape[1] == taps for w in (wq, wk, wv))
    assert a_log.dtype == dt_bias.dtype and a_log.numel() == heads and dt_bias.numel() == heads and a_log.is_contiguous() and dt_bias.is_contiguous()
    assert state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2 and state.shape[1] >= (taps - 1) * C
    _check(lib().aien_delta_conv_prepare(
        _p(proj), proj.stride(0), int(q_off), int(k_off), int(v_off), int(b_off), int(a_off), int(qk_heads), int(dim), int(heads), int(vdim),
        _p(wq), _p(wk), _p(wv), dt(wq), int(taps), _p(a_log), _p(dt_bias), dt(a_log), _p(state), state.shape[1], _p(state_slots),
        _p(seq_of_token), _p(q_start), _p(positions), _p(out), out.stride(0), _p(gb), gb.stride(0), T, _stream()), "delta_conv_prepare")


def delta_rule(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, gb: torch.Tensor, state: torch.Tensor, s_off: int,
               slot_map: torch.Tensor, q_start: torch.Tensor, positions: torch.Tensor, o: torch.Tensor, num_seqs: int, heads: int,
               qk_heads: int, dim: int, vdim: int) -> None:
    """Per value head, token by token: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, all float32.  ``qkv``
    float32 [T, *] holds the prepared q, k (qk_heads x dim) and v (heads x vdim), ``gb`` [T, 2 * heads] the decay g and
    beta.  S [heads, dim, vdim] of request s lies ``s_off`` numbers into slot slot_map[s] of ``state`` (float32 [slots, n])."""
    _dev(qkv, gb, state, slot_map, q_start, positions, o)
    assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and gb.dtype == torch.float32 and gb.stride(1) == 1
    assert o.dtype == torch.float32 and o.stride(1) == 1 and o.shape[1] == heads * vdim
    assert state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2 and state.shape[1] >= s_off + heads * dim * vdim
    _check(lib().aien_delta_rule(_p(qkv), qkv.stride(0), int(q_off), int(k_off), int(v_off), _p(gb), gb.stride(0), _p(state), state.shape[1],
                                 int(s_off), _p(slot_map), _p(q_start), _p(positions), _p(o), o.stride(0), int(num_seqs), int(heads),
                                 int(qk_heads), int(dim), int(vdim), _stream()), "delta_rule")


GATE_ACTS = {"sigmoid": 0, "silu": 1}


def grouped_gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, group: int,
                          gate_act: str = "sigmoid") -> None:
    """out = o / sqrt(mean over each group of ``group`` neighbouring columns of o^2 + eps) * weight[column mod group] *
    act(gate); o float32 [T, N], gate [T, N] (row stride free), weight [group] shared by the groups."""
    _dev(o, gate, weight, out)
    T, N = o.shape
    assert o.dtype == torch.float32 and o.stride(1) == 1 and gate.stride(1) == 1 and out.stride(1) == 1 and N % group == 0
    assert tuple(gate.shape) == (T, N) and tuple(out.shape) == (T, N) and weight.numel() == group and weight.is_contiguous()
    _check(lib().aien_grouped_gated_rmsnorm(_p(o), o.stride(0), _p(gate), dt(gate), gate.stride(0), _p(weight), dt(weight), float(eps),
                                            _p(out), dt(out), out.stride(0), T, N // group, int(group), GATE_ACTS[gate_act], _stream()),
           "grouped_gated_rmsnorm")


# ---------------------------------------------------------------------------- attention with a distance bias
def biased_attention_workspace_bytes(lim, num_heads: int, value_dim: int, window: int) -> int:
    """Scratch of :func:`biased_attention` for the largest step: the partial results of the split-key kernel."""
    splits = (lim.max_context + DECODE_CHUNK - 1) // DECODE_CHUNK
    return lim.max_seqs * num_heads * splits * (value_dim + 2) * 4 + 4096


def biased_attention(ctx, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, group, out: torch.Tensor, num_q_heads: int,
                     num_kv_heads: int, head_dim: int, value_dim: int, window: int, scale: float, head_scale: Optional[torch.Tensor],
                     slopes: Optional[torch.Tensor], gate: Optional[torch.Tensor]) -> None:
    """Attention of the step's tokens over one cache group with, per head, a factor on the scaled score, a bias
    -slope * (query position - key position) and a sigmoid gate on the output; an optional window; values of size
    ``value_dim``.  Picks the kernel for the step: in bfloat16 with values as large as keys, portions of prompts go
    through the tcgen05 kernel and tokens that come alone through the split-key kernel; all else through the plain one."""
    k2 = k_cache.view(-1, num_kv_heads, head_dim)
    v2 = v_cache.view(-1, num_kv_heads, value_dim)
    terms = dict(head_scale=head_scale, slopes=slopes, gate=gate)
    fast = (_FORCE_ATTN != "generic" and value_dim == head_dim and out.dtype == torch.bfloat16
            and decode_attention_supports(q, k2, num_q_heads, num_kv_heads, head_dim))

    def single_tokens(tokens, n):
        splits = max(1, (ctx.max_ctx_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
        part_out = ctx.workspace.take((n * num_q_heads * splits * head_dim,), torch.float32)
        part_ml = ctx.workspace.take((n * num_q_heads * splits * 2,), torch.float32)
        paged_attention_decode(q, k2, v2, group.block_table, group.max_blocks, None if tokens is None else ctx.seq_of_token,
                               ctx.positions, out, part_out, part_ml, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                               splits, token_list=tokens, num_tokens=n, impl="direct", **terms)

    splits_ok = fast and decode_masked_takes(num_q_heads, num_kv_heads, head_dim, max(1, (ctx.max_ctx_len + DECODE_CHUNK - 1) // DECODE_CHUNK))
    if ctx.decode_only and splits_ok:
        single_tokens(None, q.shape[0])
        return
    if (not ctx.decode_only and fast and ctx.prefill_tiles is not None and _PREFILL_IMPL == "tc"
            and prefill_tc_supports(q, out, head_dim, group.page_size)):
        tile_seq, tile_q0, n = ctx.prefill_tiles
        if n > 0:
            paged_attention_prefill(q, k2, v2, group.block_table, group.max_blocks, ctx.q_start, ctx.ctx_len, tile_seq, tile_q0, n,
                                    out, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale, impl="tc", **terms)
        tokens, nd = ctx.single_tokens if ctx.single_tokens is not None else (None, 0)
        if nd > 0 and splits_ok:
            single_tokens(tokens, nd)
        elif nd > 0:
            paged_attention_generic(q, k2, v2, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, out,
                                    num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale, value_dim=value_dim,
                                    token_list=tokens, num_tokens=nd, **terms)
        return
    paged_attention_generic(q, k2, v2, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, out,
                            num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale, value_dim=value_dim, **terms)


# ---------------------------------------------------------------------------- state-space recurrences
def conv_act(proj: torch.Tensor, off: int, channels: int, w: torch.Tensor, bias: Optional[torch.Tensor], taps: int, act: str,
             state: Optional[torch.Tensor], slot_map: torch.Tensor, seq_of_token: torch.Tensor, q_start: torch.Tensor,
             positions: torch.Tensor, out: torch.Tensor, out16: Optional[torch.Tensor] = None) -> None:
    """out[t, c] = f(sum_j w[c, j] * u[t - taps + 1 + j, c] + bias[c]) for the ``channels`` columns of the float32 rows
    ``proj`` [T, *] from column ``off`` on; f the identity ("none") or silu.  Rows before a portion come from the
    request's state row (its first (taps - 1) * channels numbers, the newest row last; zeros at a sequence's start),
    which is rewritten with the portion's last rows.  out float32 [T, >= channels]; ``out16`` (bfloat16 [T, >= channels]): the
    same rows once more, rounded, for a product that follows."""
    _dev(proj, w, bias, state, slot_map, seq_of_token, q_start, positions, out, out16)
    assert out16 is None or (out16.dtype == torch.bfloat16 and out16.stride(1) == 1 and out16.shape[0] == proj.shape[0])
    T = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and out.dtype == torch.float32 and out.stride(1) == 1
    assert w.is_contiguous() and tuple(w.shape) == (channels, taps) and (bias is None or (bias.is_contiguous() and bias.numel() == channels))
    assert taps == 1 or (state is not None and state.dtype == torch.float32 and state.stride(-1) == 1 and state.shape[-1] >= (taps - 1) * channels)
    _check(lib().aien_conv_act(_p(proj), proj.stride(0), int(off), int(channels), _p(w), dt(w), _p(bias), dt(bias) if bias is not None else F32,
                               int(taps), {"none": 0, "silu": 1}[act], _p(state), state.stride(0) if state is not None else 0, _p(slot_map),
                               _p(seq_of_token), _p(q_start), _p(positions), _p(out), out.stride(0), _p(out16),
                               out16.stride(0) if out16 is not None else 0, T, _stream()), "conv_act")


SCAN_SEGMENT_MIN_TOKENS = 128        # steps with fewer tokens walk every portion in one piece
# with this many lanes at work a portion is walked whole; with fewer it is cut until there are about as many
# (AIEN_B200_SCAN_LANES pins another number for measurements)
SCAN_TARGET_LANES = int(__import__("os").environ.get("AIEN_B200_SCAN_LANES", "65536"))
SCAN_MIN_SEGMENT = 32                # tokens: shorter segments cost more in their second pass than they win


def scan_segments(num_tokens: int, decode_only: bool, parallel: int = 0) -> tuple:
    """(segment length, most segments a portion has) for the portion-parallel recurrences of a step; (0, 1): one piece.
    ``parallel``: the lanes the recurrence has without cutting (requests x state columns x lanes a column).  A walk over a
    portion costs its length in dependent steps, so a step with few lanes is cut into segments that run side by side (two
    passes, each a segment long) until about SCAN_TARGET_LANES lanes are at work; measured at 65,536 lanes, four segments
    were slower than the whole walk (the second pass repeats every instruction).  It depends on the step's token and
    request counts alone, so that steps of equal shape launch alike."""
    if decode_only or num_tokens < SCAN_SEGMENT_MIN_TOKENS:
        return 0, 1
    want = -(-SCAN_TARGET_LANES // max(int(parallel), 1))
    want = min(want, num_tokens // SCAN_MIN_SEGMENT)
    if want <= 2:                                   # two passes over halves win nothing
        return 0, 1
    seg = -(-num_tokens // want)
    return seg, -(-num_tokens // seg)


def scan_scratch_floats(max_tokens: int, max_seqs: int, lanes: int, parallel: int = 1) -> int:
    """Upper bound of the float32 scratch the portion-parallel recurrences take for ``lanes`` state values a request
    whose recurrence has ``parallel`` lanes a request without cutting."""
    want = min(-(-SCAN_TARGET_LANES // max(int(parallel), 1)), max(max_tokens // SCAN_MIN_SEGMENT, 1))
    return 2 * (want + 1 + max_seqs) * lanes


def selective_scan(x: torch.Tensor, dtz: torch.Tensor, bc: torch.Tensor, b_off: int, c_off: int, z: torch.Tensor, A: torch.Tensor,
                   dt_bias: torch.Tensor, D: torch.Tensor, state: torch.Tensor, s_off: int, slot_map: torch.Tensor, q_start: torch.Tensor,
                   positions: torch.Tensor, out: torch.Tensor, num_seqs: int, N: int, seg_len: int = 0, nseg: int = 1,
                   scratch: Optional[torch.Tensor] = None) -> None:
    """The selective scan over every request's portion: per channel c and state n, token by token,
    dt = softplus(dtz[c] + dt_bias[c]); S[c, n] = exp(dt * A[c, n]) * S[c, n] + dt * x[c] * B[n]; y[c] = sum_n S[c, n] * C[n]
    + D[c] * x[c]; out[c] = y[c] * silu(z[c]).  x, dtz, z float32 [T, inner] (row strides free; dtz is overwritten with the
    step sizes); B and C are the N numbers
    from columns ``b_off`` / ``c_off`` of the float32 rows ``bc``; A float32 [inner, N]; S lives in the request's state row
    from ``s_off`` on ([inner, N]) and starts from zeros where a portion's first token has position 0."""
    _dev(x, dtz, bc, z, A, dt_bias, D, state, slot_map, q_start, positions, out, scratch)
    T, inner = x.shape
    for t in (x, dtz, bc, z):
        assert t.dtype == torch.float32 and t.stride(1) == 1
    assert A.dtype == torch.float32 and A.is_contiguous() and tuple(A.shape) == (inner, N) and dt_bias.dtype == D.dtype
    assert dt_bias.is_contiguous() and D.is_contiguous() and state.dtype == torch.float32 and state.stride(-1) == 1 and out.stride(1) == 1
    if seg_len and nseg > 1:
        assert scratch is not None and scratch.numel() >= 2 * (T // seg_len + num_seqs) * inner * N
    _check(lib().aien_selective_scan(_p(x), x.stride(0), _p(dtz), dtz.stride(0), _p(bc), bc.stride(0), int(b_off), int(c_off), _p(z), z.stride(0),
                                     _p(A), _p(dt_bias), _p(D), dt(D), _p(state), state.stride(0), int(s_off), _p(slot_map), _p(q_start),
                                     _p(positions), _p(out), dt(out), out.stride(0), T, int(num_seqs), inner, int(N), int(seg_len), int(nseg),
                                     _p(scratch), _stream()), "selective_scan")
    add_launches(3 if (seg_len and nseg > 1) else 1)


def ssd_scan(xbc: torch.Tensor, x_off: int, b_off: int, c_off: int, dtr: torch.Tensor, A: torch.Tensor, dt_bias: torch.Tensor, D: torch.Tensor,
             state: torch.Tensor, s_off: int, slot_map: torch.Tensor, q_start: torch.Tensor, positions: torch.Tensor, y: torch.Tensor,
             num_seqs: int, heads: int, V: int, G: int, N: int, seg_len: int = 0, nseg: int = 1, scratch: Optional[torch.Tensor] = None,
             steps: Optional[torch.Tensor] = None) -> None:
    """The state-space-duality recurrence over every request's portion: per head h (group g = h // (heads // G)), token by
    token, dt = softplus(dtr[h] + dt_bias[h]); S = exp(-A[h] * dt) * S + dt * B[g] x[h]^T (S is N x V); y[h] = S^T C[g] +
    D[h] * x[h].  x, B, C are column blocks of the float32 rows ``xbc``; dtr float32 [T, heads] (row stride free); A float32
    [heads]; S lives in the request's state row from ``s_off`` on (as [heads, V, N]); y float32 [T, heads * V].  ``steps``:
    float32 scratch of T * 2 * heads numbers (made here when not given)."""
    _dev(xbc, dtr, A, dt_bias, D, state, slot_map, q_start, positions, y, scratch, steps)
    T = xbc.shape[0]
    if steps is None:
        steps = torch.empty(T * 2 * heads, dtype=torch.float32, device=xbc.device)
    assert steps.dtype == torch.float32 and steps.is_contiguous() and steps.numel() >= T * 2 * heads
    assert xbc.dtype == torch.float32 and xbc.stride(1) == 1 and dtr.dtype == torch.float32 and dtr.stride(1) == 1
    assert A.dtype == torch.float32 and A.numel() == heads and dt_bias.dtype == D.dtype and dt_bias.is_contiguous() and D.is_contiguous()
    assert state.dtype == torch.float32 and state.stride(-1) == 1 and y.dtype == torch.float32 and y.stride(1) == 1
    if seg_len and nseg > 1:
        assert scratch is not None and scratch.numel() >= 2 * (T // seg_len + num_seqs) * heads * N * V
    _check(lib().aien_ssd_scan(_p(xbc), xbc.stride(0), int(x_off), int(b_off), int(c_off), _p(dtr), dtr.stride(0), _p(A), _p(dt_bias), _p(D),
                               dt(D), _p(state), state.stride(0), int(s_off), _p(slot_map), _p(q_start), _p(positions), _p(y), y.stride(0),
                               T, int(num_seqs), int(heads), int(V), int(G), int(N), int(seg_len), int(nseg), _p(scratch), _p(steps), _stream()), "ssd_scan")
    add_launches(3 if (seg_len and nseg > 1) else 1)


def gate_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, mult: float, out: torch.Tensor, groups: int) -> None:
    """out = (y * silu(z)) / rms(its part) * weight * mult, the row cut into ``groups`` equal parts with a root mean square
    each.  y, z float32 [T, width] (row strides free), out [T, width] in its own dtype (row stride free)."""
    _dev(y, z, weight, out)
    T, width = y.shape
    assert y.dtype == torch.float32 and z.dtype == torch.float32 and y.stride(1) == 1 and z.stride(1) == 1 and out.stride(1) == 1
    assert weight.is_contiguous() and weight.numel() == width and tuple(out.shape) == (T, width)
    _check(lib().aien_gate_group_norm(_p(y), y.stride(0), _p(z), z.stride(0), _p(weight), dt(weight), float(eps), float(mult), _p(out), dt(out),
                                      out.stride(0), T, width, int(groups), _stream()), "gate_group_norm")


# ---------------------------------------------------------------------------- layers with a scale per channel on each branch
def scaled_add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], vec: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                       weight: Optional[torch.Tensor], eps: float, out: Optional[torch.Tensor]) -> None:
    """x += vec * (delta + bias) in float32 (delta [T,H] or partial products [P,T,H]; vec, bias float32 [H] or None), then
    out = rmsnorm(x) * weight when ``out`` is given."""
    _dev(x, delta, vec, bias, weight, out)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    for v in (vec, bias):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == H)
    assert out is None or (out.is_contiguous() and out.shape == x.shape and weight is not None and weight.is_contiguous() and weight.numel() == H)
    nparts, stride = _parts_of(delta, x.shape)
    _check(lib().aien_scaled_add_rmsnorm(_p(x), _p(delta), dt(delta) if delta is not None else F32, nparts, stride, _p(vec), _p(bias),
                                         _p(weight), dt(weight) if weight is not None else F32, float(eps), _p(out),
                                         dt(out) if out is not None else F32, T, H, _stream()), "scaled_add_rmsnorm")


def pass_input(x: torch.Tensor, again: Optional[torch.Tensor], row: torch.Tensor) -> None:
    """x += again (float32 [T,H], when given), then x += row ([H]) for every token."""
    _dev(x, again, row)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and row.is_contiguous() and row.numel() == H
    assert again is None or (again.dtype == torch.float32 and again.is_contiguous() and again.shape == x.shape)
    _check(lib().aien_pass_input(_p(x), _p(again), _p(row), dt(row), T, H, _stream()), "pass_input")


def clamped_glu(a: torch.Tensor, gate_off: int, up_off: int, F_: int, bias_gate: Optional[torch.Tensor], bias_up: Optional[torch.Tensor],
                limit: float, alpha: float, out: torch.Tensor) -> None:
    """g = min(a[:, gate_off:][:F] + bias_gate, limit); u = clamp(a[:, up_off:][:F] + bias_up, -limit, limit);
    out = g * sigmoid(alpha * g) * (u + 1)."""
    _dev(a, bias_gate, bias_up, out)
    T = a.shape[0]
    assert a.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (T, F_)
    bdt = F32
    for b in (bias_gate, bias_up):
        if b is not None:
            assert b.is_contiguous() and b.numel() == F_
            bdt = dt(b)
    assert bias_gate is None or bias_up is None or bias_gate.dtype == bias_up.dtype
    _check(lib().aien_clamped_glu(_p(a), dt(a), a.stride(0), int(gate_off), int(up_off), _p(bias_gate), _p(bias_up), bdt, float(limit),
                                  float(alpha), _p(out), dt(out), out.stride(0), T, int(F_), _stream()), "clamped_glu")


def sigmoid_gate(o: torch.Tensor, g: Optional[torch.Tensor], mult: float, out: torch.Tensor) -> None:
    """out = o * sigmoid(g) * mult element by element; o [T, C], g float32 [T, C] or None (no gate), out [T, C]; row strides free."""
    _dev(o, g, out)
    T, C = o.shape
    assert o.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (T, C)
    assert g is None or (g.dtype == torch.float32 and g.stride(1) == 1 and tuple(g.shape) == (T, C))
    _check(lib().aien_sigmoid_gate(_p(o), dt(o), o.stride(0), _p(g), g.stride(0) if g is not None else 0, float(mult), _p(out), dt(out),
                                   out.stride(0), T, C, _stream()), "sigmoid_gate")


def scale_rows(o: torch.Tensor, mult: float, out: torch.Tensor) -> None:
    """out = o * mult (row strides free)."""
    sigmoid_gate(o, None, mult, out)


# ---------------------------------------------------------------------------- attention with a capped score
def capped_attention_workspace_bytes(lim, num_heads: int, value_dim: int) -> int:
    """Scratch of :func:`capped_attention` for the largest step: the partial results of the split-key kernel and of the
    key ranges of the tcgen05 kernel."""
    return biased_attention_workspace_bytes(lim, num_heads, value_dim, 0) + attention_workspace_bytes(lim, num_heads, value_dim)


def capped_attention(ctx, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, group, out: torch.Tensor, num_q_heads: int,
                     num_kv_heads: int, head_dim: int, value_dim: int, window: int, scale: float, softcap: float) -> None:
    """Causal attention of the step's tokens over one cache group with the scaled score s turned into softcap * tanh(s /
    softcap) (softcap 0: left as it is), an optional window, values of size ``value_dim``.  Picks the kernel for the step:
    in bfloat16 with values as large as keys, portions of prompts go through the tcgen05 kernel and tokens that come alone
    through the split-key kernel; all else through the plain one."""
    k2 = k_cache.view(-1, num_kv_heads, head_dim)
    v2 = v_cache.view(-1, num_kv_heads, value_dim)
    fast = (_FORCE_ATTN != "generic" and value_dim == head_dim and out.dtype == torch.bfloat16
            and decode_attention_supports(q, k2, num_q_heads, num_kv_heads, head_dim))
    splits = max(1, (ctx.max_ctx_len + DECODE_CHUNK - 1) // DECODE_CHUNK)

    def single_tokens(tokens, n):
        part_out = ctx.workspace.take((n * num_q_heads * splits * head_dim,), torch.float32)
        part_ml = ctx.workspace.take((n * num_q_heads * splits * 2,), torch.float32)
        paged_attention_decode(q, k2, v2, group.block_table, group.max_blocks, None if tokens is None else ctx.seq_of_token,
                               ctx.positions, out, part_out, part_ml, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                               splits, token_list=tokens, num_tokens=n, impl="direct", softcap=softcap)

    def plain(tokens=None, n=None):
        paged_attention_generic(q, k2, v2, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, out, num_q_heads,
                                num_kv_heads, head_dim, group.page_size, window, scale, value_dim=value_dim, softcap=softcap,
                                token_list=tokens, num_tokens=n)

    splits_ok = fast and decode_masked_takes(num_q_heads, num_kv_heads, head_dim, splits)
    if ctx.decode_only and splits_ok:
        single_tokens(None, q.shape[0])
        return
    if (not ctx.decode_only and fast and ctx.prefill_tiles is not None and _PREFILL_IMPL == "tc"
            and prefill_tc_supports(q, out, head_dim, group.page_size)):
        tile_seq, tile_q0, n = ctx.prefill_tiles
        if n > 0:
            scratch = None
            if n <= PREFILL_SPLIT_MAX_TILES:
                nbytes = prefill_split_scratch_bytes(n, num_q_heads, head_dim, ctx.max_ctx_len)
                scratch = ctx.workspace.take((nbytes // 4,), torch.float32) if nbytes else None
            paged_attention_prefill(q, k2, v2, group.block_table, group.max_blocks, ctx.q_start, ctx.ctx_len, tile_seq, tile_q0, n,
                                    out, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale, impl="tc",
                                    scratch=scratch, max_ctx=ctx.max_ctx_len, softcap=softcap)
        tokens, nd = ctx.single_tokens if ctx.single_tokens is not None else (None, 0)
        if nd > 0 and splits_ok:
            single_tokens(tokens, nd)
        elif nd > 0:
            plain(tokens, nd)
        return
    plain()



def routed_combine(parts: torch.Tensor, h: Optional[torch.Tensor], w_same: Optional[torch.Tensor], shared: Optional[torch.Tensor],
                   zs: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = sum_p parts[p] + w_same[t] * h[t] + sigmoid(zs[t]) * shared[t] (float32 [T,H]).  parts [P,T,H]; ``h`` with
    ``w_same`` float32 [T] or neither; ``shared`` [T,H] or partial products [Q,T,H], or None; ``zs`` float32 [T] (stride free)
    or None (the shared term then counts whole)."""
    _dev(parts, h, w_same, shared, zs, out)
    P_, T, H = parts.shape
    assert parts.is_contiguous() and out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (T, H)
    assert (h is None) == (w_same is None)
    if h is not None:
        assert h.stride(1) == 1 and w_same.dtype == torch.float32 and w_same.is_contiguous() and w_same.numel() >= T
    sparts, sstride = _parts_of(shared, (T, H))
    assert zs is None or zs.dtype == torch.float32
    _check(lib().aien_routed_combine(_p(parts), dt(parts), P_, T * H, _p(h), dt(h) if h is not None else F32, h.stride(0) if h is not None else 0,
                                     _p(w_same), _p(shared), dt(shared) if shared is not None else F32, sparts, sstride, _p(zs),
                                     zs.stride(0) if zs is not None else 0, _p(out), T, H, _stream()), "routed_combine")


def moe_route_biased(z: torch.Tensor, num_experts: int, real: int, top: int, renorm: bool, renorm_eps: float,
                     correction: Optional[torch.Tensor], ids: torch.Tensor, wts: torch.Tensor, w_same: Optional[torch.Tensor],
                     expert_count: Optional[torch.Tensor] = None) -> None:
    """Router with a correction on the choice: s = softmax(z[:, :num_experts]) (float32); the ``top`` largest s + correction
    are chosen; weights s (``renorm``: divided by their sum + renorm_eps).  Experts from ``real`` on return their input:
    their weights are summed into ``w_same`` [T] and their choices handed on as expert 0 with weight zero."""
    _dev(z, correction, ids, wts, w_same, expert_count)
    T = z.shape[0]
    assert z.dtype == torch.float32 and z.stride(1) == 1 and z.shape[1] >= num_experts and ids.dtype == torch.int32 and wts.dtype == torch.float32
    assert ids.is_contiguous() and wts.is_contiguous() and ids.numel() >= T * top and wts.numel() >= T * top
    assert correction is None or (correction.is_contiguous() and correction.numel() == num_experts)
    assert w_same is None or (w_same.dtype == torch.float32 and w_same.is_contiguous() and w_same.numel() >= T)
    _check(lib().aien_moe_route_biased(_p(z), z.stride(0), T, int(num_experts), int(real), int(top), 1 if renorm else 0, float(renorm_eps),
                                       _p(correction), dt(correction) if correction is not None else F32, _p(ids), _p(wts), _p(w_same),
                                       _p(expert_count), _stream()), "moe_route_biased")


def rope_halves_value_write(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, nq: int, nkv: int, hd: int, hdv: int,
                            cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot: int, slot_map: torch.Tensor,
                            q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    """q, k (heads of ``hd``) and v (heads of ``hdv``) are column blocks of the float32 rows ``proj``; the first ``rot``
    dimensions of every q and k head turn (i with i + rot/2) by cos/sin float32 [T, rot/2]; q goes to ``q_out`` [T, nq*hd],
    k and v to the token's cache slot (k_cache [slots, nkv, hd], v_cache [slots, nkv, hdv])."""
    _dev(proj, cos, sin, slot_map, q_out, k_cache, v_cache)
    T = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.dtype == v_cache.dtype and slot_map.dtype == torch.int32
    if rot:
        assert cos is not None and tuple(cos.shape) == (T, rot // 2) and cos.is_contiguous() and sin.is_contiguous()
    _check(lib().aien_rope_halves_value_write(_p(proj), proj.stride(0), int(q_off), int(k_off), int(v_off), int(nq), int(nkv), int(hd), int(hdv),
                                              _p(cos), _p(sin), int(rot), _p(slot_map), _p(q_out), dt(q_out), q_out.stride(0), _p(k_cache),
                                              _p(v_cache), dt(k_cache), T, _stream()), "rope_halves_value_write")
