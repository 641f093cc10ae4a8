// A short causal convolution over time on every channel of a projection, carried across steps, with what two kinds
// of mixer do to the result in the same kernel.
//
//   y_t[c] = sum_j w[c][j] * u_(t - taps + 1 + j)[c],   j = 0 .. taps-1,  zeros before the sequence's start.
//
// u are rows of a float32 projection [T, ld] (several convolved blocks of channels side by side).  The last taps-1
// rows of u of every request live in a float32 state slot [taps-1][C] (C = all convolved channels of the mixer; row
// taps-2 is the newest; rows that would lie before position 0 hold zeros).  One CTA serves one token, except at the
// start of a portion: the CTA of a portion's first token also serves the next taps-2 tokens (the only ones that read
// the slot) and then writes the slot's new contents, so no other CTA reads a slot while it is rewritten.  The sum runs
// over j in rising order whatever the cut of the prompt, so a token's value does not depend on the cut.
//
// attn_conv_prepare: q | k | v blocks; then an RMS norm over the whole q row and the whole k row (plain weights), each
// value head divided by its root mean square; q leaves in the compute dtype, k and v go to the token's cache slot.
// delta_conv_prepare: q | k | v blocks; silu; q and k made unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q times
// dim^-1/2; besides, per value head, beta = sigmoid(b) and the decay g = exp(-exp(A_log) * softplus(a + dt_bias)).
// All of it is float32.
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int SC_MAX_TAPS = 8;
constexpr int SC_THREADS = 256;
constexpr int SC_THREADS_WIDE = 1024;       // for a step of few tokens: its CTAs are too few to hide a row's loads behind one another

inline int conv_threads(int T, int C) { return (T <= 2 * 148 && C >= 2048) ? SC_THREADS_WIDE : SC_THREADS; }

struct ConvRow {
    int t, first, last, slot;
    bool fresh;
};

// The same for a number of taps known when the kernel is compiled: the addresses are one pointer a source and a stride,
// a token with all its taps inside the step (every token but a portion's first ones) reads without a test, and four
// bfloat16 weights are one load.  What the kernel spends is instructions, not bytes: with the taps a run-time number
// it issued several hundred a channel.
template <int TAPS>
__device__ __forceinline__ float conv_fixed(const float* __restrict__ proj, long ld, int off, int cc, const void* __restrict__ w, int wdt,
                                            const float* __restrict__ st, int C, int c0, const ConvRow& r) {
    const int t_first = r.t - (TAPS - 1);
    float u[TAPS], wv[TAPS];
    if (t_first >= r.first) {
        const float* p = proj + (long)t_first * ld + off + cc;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) u[j] = __ldcg(p + (long)j * ld);
    } else {
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            const int tt = t_first + j;
            if (tt >= r.first) u[j] = __ldcg(proj + (long)tt * ld + off + cc);
            else u[j] = r.fresh ? 0.f : st[(long)((TAPS - 1) + (tt - r.first)) * C + c0 + cc];
        }
    }
    if (wdt == AIEN_DT_F32) {
        const float* wf = reinterpret_cast<const float*>(w) + (size_t)cc * TAPS;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wv[j] = wf[j];
    } else if (TAPS == 4 && (reinterpret_cast<uintptr_t>(w) & 7) == 0) {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(w) + (size_t)cc * 4);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        wv[0] = lo.x; wv[1] = lo.y; wv[2 % TAPS] = hi.x; wv[3 % TAPS] = hi.y;
    } else {
        const __nv_bfloat16* wh = reinterpret_cast<const __nv_bfloat16*>(w) + (size_t)cc * TAPS;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wv[j] = __bfloat162float(wh[j]);
    }
    float y = 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) y = fmaf(wv[j], u[j], y);
    return y;
}

// channel cc of the convolved block that starts at column `off` of proj and at channel `c0` of the state
__device__ __forceinline__ float conv_value(const float* __restrict__ proj, long ld, int off, int cc, const void* __restrict__ w, int wdt,
                                            int taps, const float* __restrict__ st, int C, int c0, const ConvRow& r) {
    switch (taps) {
        case 2: return conv_fixed<2>(proj, ld, off, cc, w, wdt, st, C, c0, r);
        case 3: return conv_fixed<3>(proj, ld, off, cc, w, wdt, st, C, c0, r);
        case 4: return conv_fixed<4>(proj, ld, off, cc, w, wdt, st, C, c0, r);
        default: break;
    }
    float y = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int tt = r.t - (taps - 1) + j;
        float u;
        if (tt >= r.first) u = ld_act(proj + (size_t)tt * ld + off + cc);
        else if (r.fresh) u = 0.f;
        else u = st[(size_t)((taps - 1) + (tt - r.first)) * C + c0 + cc];
        y = fmaf(load_dyn(w, wdt, (size_t)cc * taps + j), u, y);
    }
    return y;
}

// the slot's new rows for one block of channels, by the thread that owns the channel
__device__ __forceinline__ void conv_state_update(const float* __restrict__ proj, long ld, int off, int n, int taps,
                                                  float* __restrict__ st, int C, int c0, const ConvRow& r) {
    for (int cc = threadIdx.x; cc < n; cc += blockDim.x) {
        float keep[SC_MAX_TAPS];
        for (int k = 0; k < taps - 1; ++k) {
            const int tt = r.last - (taps - 1) + k;
            if (tt >= r.first) keep[k] = ld_act(proj + (size_t)tt * ld + off + cc);
            else keep[k] = r.fresh ? 0.f : st[(size_t)((taps - 1) + (tt - r.first)) * C + c0 + cc];
        }
        for (int k = 0; k < taps - 1; ++k) st[(size_t)k * C + c0 + cc] = keep[k];
    }
}

// which rows this CTA serves: returns the count (0: another CTA serves this token)
__device__ __forceinline__ int conv_rows(int t, int taps, const int* seq_of_token, const int* q_start, const int* positions,
                                         const int* slot_map, ConvRow& r) {
    const int s = seq_of_token[t];
    r.first = q_start[s];
    r.last = q_start[s + 1];
    r.slot = slot_map[s];
    r.fresh = positions[r.first] == 0;
    r.t = t;
    const int k = t - r.first;
    if (k > 0 && k < taps - 1) return 0;
    if (k > 0) return 1;
    const int n = r.last - r.first;
    return taps - 1 < 1 ? 1 : (n < taps - 1 ? n : taps - 1);
}

template <typename TQ, typename TKV>
__global__ void __launch_bounds__(SC_THREADS_WIDE)
attn_conv_prepare_kernel(const float* __restrict__ proj, long ld, int q_off, int k_off, int v_off, int Cq, int Ck, int Cv,
                         const void* __restrict__ wq, const void* __restrict__ wk, const void* __restrict__ wv, int wdt, int taps,
                         const void* __restrict__ qn, const void* __restrict__ kn, int ndt, float eps, int G, int V, int value_norm,
                         float* __restrict__ state, const int* __restrict__ state_slots, const int* __restrict__ seq_of_token,
                         const int* __restrict__ q_start, const int* __restrict__ positions, const int* __restrict__ kv_slots,
                         TKV* __restrict__ k_cache, TKV* __restrict__ v_cache, TQ* __restrict__ q_out, long ldq) {
    extern __shared__ float vals[];               // q | k | v of the row at hand
    __shared__ float red[32];
    ConvRow r;
    const int rows = conv_rows(blockIdx.x, taps, seq_of_token, q_start, positions, state_slots, r);
    if (rows == 0) return;
    const bool own_kv = Ck > 0;
    const int C = Cq + Ck + Cv;
    float* st = state + (size_t)r.slot * (size_t)(taps - 1) * C;
    const int t0 = r.t;
    for (int i = 0; i < rows; ++i) {
        r.t = t0 + i;
        float sq = 0.f, sk = 0.f;
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            float y;
            if (c < Cq) { y = conv_value(proj, ld, q_off, c, wq, wdt, taps, st, C, 0, r); sq = fmaf(y, y, sq); }
            else if (c < Cq + Ck) { y = conv_value(proj, ld, k_off, c - Cq, wk, wdt, taps, st, C, Cq, r); sk = fmaf(y, y, sk); }
            else y = conv_value(proj, ld, v_off, c - Cq - Ck, wv, wdt, taps, st, C, Cq + Ck, r);
            vals[c] = y;
        }
        const float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)Cq + eps);
        for (int c = threadIdx.x; c < Cq; c += blockDim.x)
            q_out[(size_t)r.t * ldq + c] = from_f<TQ>(vals[c] * rq * load_dyn(qn, ndt, c));
        if (own_kv) {
            const float rk = 1.0f / sqrtf(block_sum(sk, red) / (float)Ck + eps);
            const int slot = kv_slots[r.t];
            if (slot >= 0) {
                for (int c = threadIdx.x; c < Ck; c += blockDim.x)
                    k_cache[(size_t)slot * Ck + c] = from_f<TKV>(vals[Cq + c] * rk * load_dyn(kn, ndt, c));
                const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
                for (int g = warp; g < G; g += nwarps) {
                    const float* v = vals + Cq + Ck + (size_t)g * V;
                    float rv = 1.f;
                    if (value_norm) {
                        float sv = 0.f;
                        for (int d = lane; d < V; d += 32) sv = fmaf(v[d], v[d], sv);
                        rv = 1.0f / sqrtf(warp_sum(sv) / (float)V + eps);
                    }
                    for (int d = lane; d < V; d += 32) v_cache[(size_t)slot * Cv + (size_t)g * V + d] = from_f<TKV>(v[d] * rv);
                }
            }
        }
        __syncthreads();
    }
    if (t0 == r.first && taps > 1) {
        conv_state_update(proj, ld, q_off, Cq, taps, st, C, 0, r);
        if (own_kv) {
            conv_state_update(proj, ld, k_off, Ck, taps, st, C, Cq, r);
            conv_state_update(proj, ld, v_off, Cv, taps, st, C, Cq + Ck, r);
        }
    }
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// out float32 [T, Cq+Ck+Cv] (q | k | v prepared), gb float32 [T, 2*heads] (decay g | beta)
__global__ void __launch_bounds__(SC_THREADS_WIDE)
delta_conv_prepare_kernel(const float* __restrict__ proj, long ld, int q_off, int k_off, int v_off, int b_off, int a_off,
                          int G, int D, int heads, int V,
                          const void* __restrict__ wq, const void* __restrict__ wk, const void* __restrict__ wv, int wdt, int taps,
                          const void* __restrict__ a_log, const void* __restrict__ dt_bias, int pdt,
                          float* __restrict__ state, size_t state_stride, const int* __restrict__ state_slots,
                          const int* __restrict__ seq_of_token, const int* __restrict__ q_start, const int* __restrict__ positions,
                          float* __restrict__ out, long ldo, float* __restrict__ gb, long ldgb) {
    extern __shared__ float vals[];
    ConvRow r;
    const int rows = conv_rows(blockIdx.x, taps, seq_of_token, q_start, positions, state_slots, r);
    if (rows == 0) return;
    const int Cq = G * D, Ck = G * D, Cv = heads * V, C = Cq + Ck + Cv;
    float* st = state + (size_t)r.slot * state_stride;
    const int t0 = r.t;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const float qmul = 1.0f / sqrtf((float)D);
    for (int i = 0; i < rows; ++i) {
        r.t = t0 + i;
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            float y;
            if (c < Cq) y = conv_value(proj, ld, q_off, c, wq, wdt, taps, st, C, 0, r);
            else if (c < Cq + Ck) y = conv_value(proj, ld, k_off, c - Cq, wk, wdt, taps, st, C, Cq, r);
            else y = conv_value(proj, ld, v_off, c - Cq - Ck, wv, wdt, taps, st, C, Cq + Ck, r);
            y = silu_f(y);
            if (c >= Cq + Ck) out[(size_t)r.t * ldo + c] = y;
            else vals[c] = y;
        }
        for (int h = threadIdx.x; h < heads; h += blockDim.x) {
            const float a = ld_act(proj + (size_t)r.t * ld + a_off + h) + load_dyn(dt_bias, pdt, h);
            const float sp = a > 20.f ? a : log1pf(expf(a));
            gb[(size_t)r.t * ldgb + h] = expf(-expf(load_dyn(a_log, pdt, h)) * sp);
            gb[(size_t)r.t * ldgb + heads + h] = 1.0f / (1.0f + expf(-ld_act(proj + (size_t)r.t * ld + b_off + h)));
        }
        __syncthreads();
        for (int g = warp; g < 2 * G; g += nwarps) {            // q heads then k heads, each a unit vector
            const float* v = vals + (size_t)g * D;
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) ss = fmaf(v[d], v[d], ss);
            const float m = (g < G ? qmul : 1.0f) / sqrtf(warp_sum(ss) + 1e-6f);
            for (int d = lane; d < D; d += 32) out[(size_t)r.t * ldo + (size_t)g * D + d] = v[d] * m;
        }
        __syncthreads();
    }
    if (t0 == r.first && taps > 1) {
        conv_state_update(proj, ld, q_off, Cq, taps, st, C, 0, r);
        conv_state_update(proj, ld, k_off, Ck, taps, st, C, Cq, r);
        conv_state_update(proj, ld, v_off, Cv, taps, st, C, Cq + Ck, r);
    }
}

// One block of C convolved channels with a bias and an activation of its own:
// out[t][c] = f(conv(c) + bias[c]), f the identity (act 0) or silu (act 1); float32 out, and on request the same rows
// once more in bfloat16 (the operand of a product that follows).
__global__ void __launch_bounds__(SC_THREADS_WIDE)
conv_act_kernel(const float* __restrict__ proj, long ld, int off, int C, const void* __restrict__ w, int wdt,
                const void* __restrict__ bias, int bdt, int taps, int act, float* __restrict__ state, size_t state_stride,
                const int* __restrict__ state_slots, const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                const int* __restrict__ positions, float* __restrict__ out, long ldo, __nv_bfloat16* __restrict__ out16, long ldo16) {
    ConvRow r;
    const int rows = conv_rows(blockIdx.x, taps, seq_of_token, q_start, positions, state_slots, r);
    if (rows == 0) return;
    float* st = state + (size_t)r.slot * state_stride;
    const int t0 = r.t;
    for (int i = 0; i < rows; ++i) {
        r.t = t0 + i;
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            float y = conv_value(proj, ld, off, c, w, wdt, taps, st, C, 0, r);
            if (bias != nullptr) y += load_dyn(bias, bdt, c);
            y = act == 1 ? silu_f(y) : y;
            out[(size_t)r.t * ldo + c] = y;
            if (out16 != nullptr) out16[(size_t)r.t * ldo16 + c] = __float2bfloat16_rn(y);
        }
    }
    __syncthreads();
    if (t0 == r.first && taps > 1) conv_state_update(proj, ld, off, C, taps, st, C, 0, r);
}

}  // namespace aien

using namespace aien;

template <typename TQ, typename TKV>
static int launch_attn_conv_prepare(size_t smem, cudaStream_t stream, int T, const float* proj, long ld, int q_off, int k_off, int v_off,
                                    int Cq, int Ck, int Cv, const void* wq, const void* wk, const void* wv, int wdt, int taps,
                                    const void* qn, const void* kn, int ndt, float eps, int G, int V, int value_norm, float* state,
                                    const int* state_slots, const int* seq_of_token, const int* q_start, const int* positions,
                                    const int* kv_slots, TKV* k_cache, TKV* v_cache, TQ* q_out, long ldq) {
    auto kern = attn_conv_prepare_kernel<TQ, TKV>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AIEN_E_STATE;
    kern<<<T, conv_threads(T, Cq + Ck + Cv), smem, stream>>>(proj, ld, q_off, k_off, v_off, Cq, Ck, Cv, wq, wk, wv, wdt, taps, qn, kn, ndt, eps, G, V,
                                          value_norm, state, state_slots, seq_of_token, q_start, positions, kv_slots, k_cache, v_cache,
                                          q_out, ldq);
    return 0;
}

// proj float32 [T, ld] with the q block at q_off (Cq channels) and, when the run keeps its own keys and values
// (Ck > 0), k at k_off (Ck = G * head size) and v at v_off (Cv = G * V).  Convolution weights [C, taps] in w_dt, norm
// weights in n_dt.  state float32 [slots][taps-1][Cq+Ck+Cv]; kv_slots[t]: cache slot of token t (-1: write nothing).
AIEN_API int aien_attn_conv_prepare(const float* proj, long ld, int q_off, int k_off, int v_off, int Cq, int Ck, int Cv,
                                    const void* wq, const void* wk, const void* wv, int w_dt, int taps,
                                    const void* qn, const void* kn, int n_dt, float eps, int G, int V, int value_norm,
                                    float* state, const int* state_slots, const int* seq_of_token, const int* q_start,
                                    const int* positions, const int* kv_slots, void* k_cache, void* v_cache, int kv_dt,
                                    void* q_out, int q_dt, long ldq, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (taps < 1 || taps > SC_MAX_TAPS || Cq <= 0 || Ck < 0 || Cv < 0 || (Ck > 0 && (G <= 0 || Cv != G * V))) return AIEN_E_SHAPE;
    if (taps > 1 && state == nullptr) return AIEN_E_SHAPE;
    const size_t smem = (size_t)(Cq + Ck + Cv) * sizeof(float);
    if (smem > 200 * 1024) return AIEN_E_SHAPE;
    int rc = 0;
    AIEN_DISPATCH_DTYPE(q_dt, TQ, AIEN_DISPATCH_DTYPE(kv_dt, TKV,
        (rc = launch_attn_conv_prepare<TQ, TKV>(smem, stream, T, proj, ld, q_off, k_off, v_off, Cq, Ck, Cv, wq, wk, wv, w_dt, taps, qn, kn,
                                                n_dt, eps, G, V, value_norm, state, state_slots, seq_of_token, q_start, positions,
                                                kv_slots, (TKV*)k_cache, (TKV*)v_cache, (TQ*)q_out, ldq))));
    if (rc != 0) return rc;
    return launch_status();
}

// proj float32 [T, ld]: q (G*D) at q_off, k (G*D) at k_off, v (heads*V) at v_off, beta's input (heads) at b_off, the
// decay's input (heads) at a_off.  state float32 rows of state_stride numbers whose first (taps-1)*(2*G*D + heads*V)
// are the convolution's.  out float32 [T, ldo] = q | k | v prepared; gb float32 [T, ldgb] = decay | beta.
AIEN_API int aien_delta_conv_prepare(const float* proj, long ld, int q_off, int k_off, int v_off, int b_off, int a_off,
                                     int G, int D, int heads, int V, const void* wq, const void* wk, const void* wv, int w_dt, int taps,
                                     const void* a_log, const void* dt_bias, int p_dt, float* state, size_t state_stride,
                                     const int* state_slots, const int* seq_of_token, const int* q_start, const int* positions,
                                     float* out, long ldo, float* gb, long ldgb, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (taps < 1 || taps > SC_MAX_TAPS || G <= 0 || D <= 0 || heads <= 0 || V <= 0 || heads % G) return AIEN_E_SHAPE;
    const size_t smem = (size_t)(2 * G * D) * sizeof(float);
    if (smem > 200 * 1024) return AIEN_E_SHAPE;
    auto kern = delta_conv_prepare_kernel;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AIEN_E_STATE;
    kern<<<T, conv_threads(T, 2 * G * D + heads * V), smem, stream>>>(proj, ld, q_off, k_off, v_off, b_off, a_off, G, D, heads, V, wq, wk, wv, w_dt, taps, a_log, dt_bias,
                                          p_dt, state, state_stride, state_slots, seq_of_token, q_start, positions, out, ldo, gb, ldgb);
    return launch_status();
}

// proj float32 [T, ld] with the C convolved channels from column `off` on; weights [C, taps] in w_dt, bias [C] in b_dt (or
// null); state float32 rows of state_stride numbers whose first (taps-1)*C are the convolution's; out float32 [T, ldo];
// out16 (or null) bfloat16 [T, ldo16]: the same rows rounded.
AIEN_API int aien_conv_act(const float* proj, long ld, int off, int C, const void* w, int w_dt, const void* bias, int b_dt, int taps,
                           int act, float* state, size_t state_stride, const int* state_slots, const int* seq_of_token,
                           const int* q_start, const int* positions, float* out, long ldo, void* out16, long ldo16, int T,
                           cudaStream_t stream) {
    if (T <= 0) return 0;
    if (taps < 1 || taps > SC_MAX_TAPS || C <= 0 || (act != 0 && act != 1)) return AIEN_E_SHAPE;
    if (taps > 1 && state == nullptr) return AIEN_E_SHAPE;
    conv_act_kernel<<<T, conv_threads(T, C), 0, stream>>>(proj, ld, off, C, w, w_dt, bias, b_dt, taps, act, state, state_stride, state_slots,
                                                          seq_of_token, q_start, positions, out, ldo, (__nv_bfloat16*)out16, ldo16);
    return launch_status();
}
