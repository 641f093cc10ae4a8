// Several residual streams per token ("hyper-connections"), the token shift of a sublayer's input, and an
// embedding with sinusoidal positions.
//
// The stream tensor x is float32 [n][T][H] (n <= 8 copies of the residual stream, all equal after the
// embedding).  A sublayer q with parameters in[n], out[n], mix[n][n] (indexed [from][to]) works as
//     u = sum_s in[s] x_s ;  y = sublayer(norm(u)) ;  x_t <- sum_s mix[s][t] x_s + out[t] y   (all t at once).
// The write of one sublayer and the read of the next meet in one kernel: hc_norm first applies the write that is
// still pending (y of the sublayer before, with that sublayer's mix and out), in place, then forms u with its own
// in[], and the RMS norm of u with the norm's weight.  Everything is float32; only the normed row leaves in the
// compute dtype.  The parameters of a sublayer are one float32 pack [in(n) | out(n) | mix(n*n)].
//
// Token shift: what the mixer reads is h + (h' - h) * shift, h' being the normed row of the token before (zeros for
// the first token of a sequence), kept in a float32 state slot [H] per request between steps.  In a step of single
// tokens hc_norm does the shift itself (every row's predecessor is its request's slot); a step with portions writes
// the normed rows in float32 and token_shift follows, where the CTA of a portion's first token both reads the slot
// and leaves the portion's last row in it (the same thread reads and writes a channel, so no other row races it).
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int HC_MAX = 8;

struct HcPack {
    float in[HC_MAX], out[HC_MAX], mix[HC_MAX * HC_MAX];
};

__device__ __forceinline__ void hc_load(const float* __restrict__ p, int n, float* in, float* out, float* mix) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) { in[i] = p[i]; out[i] = p[n + i]; }
    for (int i = threadIdx.x; i < n * n; i += blockDim.x) mix[i] = p[2 * n + i];
}

template <typename TA>
__device__ __forceinline__ float hc_pending(const TA* __restrict__ y, int parts, size_t pstride, size_t idx) {
    float v = 0.f;
    for (int p = 0; p < parts; ++p) v += ld_act(y + (size_t)p * pstride + idx);
    return v;
}

__global__ void replicate_streams_kernel(float* __restrict__ x, size_t per, int n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        for (int s = 1; s < n; ++s) x[(size_t)s * per + i] = v;
    }
}

// One CTA per token.  y (or null): the pending branch output [T,H] in TA, or `parts` float32 partial products
// pstride apart; prev: the pack whose mix/out apply to it.  cur: the pack whose in[] forms u.  h: the normed row.
// shift_w (or null): the fused token shift of a step of single tokens, with the float32 slots `shift_state`
// [slots][H], slot_map[t] and positions[t].
// NT threads: 256, or 1024 for a step of few tokens, whose CTAs are too few to hide a row's loads behind one another.
template <typename TA, typename TH, int NT>
__global__ void __launch_bounds__(NT)
hc_norm_kernel(float* __restrict__ x, size_t sstride, int n, const TA* __restrict__ y, int parts, size_t pstride,
               const float* __restrict__ prev, const float* __restrict__ cur, const void* __restrict__ w, int wdt, float eps,
               TH* __restrict__ h, int H, const void* __restrict__ shift_w, int sdt, float* __restrict__ shift_state,
               const int* __restrict__ slot_map, const int* __restrict__ positions) {
    extern __shared__ float u_s[];
    __shared__ float red[32];
    __shared__ float p_in[HC_MAX], p_out[HC_MAX], p_mix[HC_MAX * HC_MAX], c_in[HC_MAX], c_out[HC_MAX], c_mix[HC_MAX * HC_MAX];
    const size_t t = blockIdx.x;
    hc_load(cur, n, c_in, c_out, c_mix);
    if (y != nullptr) hc_load(prev, n, p_in, p_out, p_mix);
    __syncthreads();
    float ss = 0.f;
    // four neighbouring columns a thread and pass (16-byte loads and stores of every stream) where the row allows it
    const bool vec4 = NT == 256 && (H & 3) == 0 && (pstride & 3) == 0;   // the wide CTA of a short step has a thread for every column or two
    const int step = vec4 ? 4 : 1;
    for (int c = threadIdx.x * step; c < H; c += blockDim.x * step) {
        const size_t idx = t * H + c;
        float xs[HC_MAX][4];
#pragma unroll
        for (int s = 0; s < HC_MAX; ++s) {
            if (s < n && vec4) {
                const float4 v = *reinterpret_cast<const float4*>(x + (size_t)s * sstride + idx);
                xs[s][0] = v.x; xs[s][1] = v.y; xs[s][2] = v.z; xs[s][3] = v.w;
            } else {
                xs[s][0] = s < n ? x[(size_t)s * sstride + idx] : 0.f;
                xs[s][1] = xs[s][2] = xs[s][3] = 0.f;
            }
        }
        if (y != nullptr) {
            float yv[4] = {0.f, 0.f, 0.f, 0.f};
            if (vec4) {
                for (int p = 0; p < parts; ++p) {
                    const float4 v = ld_act4(y + (size_t)p * pstride + idx);
                    yv[0] += v.x; yv[1] += v.y; yv[2] += v.z; yv[3] += v.w;
                }
            } else {
                yv[0] = hc_pending(y, parts, pstride, idx);
            }
            float nx[HC_MAX][4];
#pragma unroll
            for (int r = 0; r < HC_MAX; ++r) {
                if (r < n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float acc = p_out[r] * yv[e];
#pragma unroll
                        for (int s = 0; s < HC_MAX; ++s)
                            if (s < n) acc = fmaf(p_mix[s * n + r], xs[s][e], acc);
                        nx[r][e] = acc;
                    }
                    if (vec4) *reinterpret_cast<float4*>(x + (size_t)r * sstride + idx) = make_float4(nx[r][0], nx[r][1], nx[r][2], nx[r][3]);
                    else x[(size_t)r * sstride + idx] = nx[r][0];
                }
            }
#pragma unroll
            for (int r = 0; r < HC_MAX; ++r)
#pragma unroll
                for (int e = 0; e < 4; ++e) xs[r][e] = r < n ? nx[r][e] : 0.f;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (e >= step) break;
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX; ++s)
                if (s < n) u = fmaf(c_in[s], xs[s][e], u);
            u_s[c + e] = u;
            ss = fmaf(u, u, ss);
        }
    }
    const float scale = 1.0f / sqrtf(block_sum(ss, red) / (float)H + eps);
    if (shift_w == nullptr) {
        for (int c = threadIdx.x; c < H; c += blockDim.x) h[t * H + c] = from_f<TH>(u_s[c] * scale * load_dyn(w, wdt, c));
        return;
    }
    float* st = shift_state + (size_t)slot_map[t] * H;
    const bool fresh = positions[t] == 0;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = u_s[c] * scale * load_dyn(w, wdt, c);
        const float before = fresh ? 0.f : st[c];
        st[c] = v;
        h[t * H + c] = from_f<TH>(v + (before - v) * load_dyn(shift_w, sdt, c));
    }
}

// hn float32 [T,H] -> h = hn + (hn of the token before - hn) * shift, per request across steps (see the head of the file).
template <typename TH>
__global__ void __launch_bounds__(256)
token_shift_kernel(const float* __restrict__ hn, const void* __restrict__ shift_w, int sdt, float* __restrict__ state,
                   const int* __restrict__ slot_map, const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                   const int* __restrict__ positions, TH* __restrict__ h, int H) {
    const int t = blockIdx.x;
    const int s = seq_of_token[t];
    const int first = q_start[s];
    const float* row = hn + (size_t)t * H;
    if (t != first) {
        const float* before = row - H;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float v = row[c];
            h[(size_t)t * H + c] = from_f<TH>(v + (before[c] - v) * load_dyn(shift_w, sdt, c));
        }
        return;
    }
    float* st = state + (size_t)slot_map[s] * H;
    const float* last = hn + (size_t)(q_start[s + 1] - 1) * H;
    const bool fresh = positions[t] == 0;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = row[c];
        const float before = fresh ? 0.f : st[c];
        st[c] = last[c];
        h[(size_t)t * H + c] = from_f<TH>(v + (before - v) * load_dyn(shift_w, sdt, c));
    }
}

// out[r] = sum over the streams of row rows[r], with the pending write (if any) applied on the way:
// sum_t x_t' = sum_s (sum_t mix[s][t]) x_s + (sum_t out[t]) y, the sums taken in index order.
template <typename TA>
__global__ void __launch_bounds__(256)
hc_sum_rows_kernel(const float* __restrict__ x, size_t sstride, int n, const TA* __restrict__ y, int parts, size_t pstride,
                   const float* __restrict__ prev, const int* __restrict__ rows, float* __restrict__ out, int H) {
    __shared__ float p_in[HC_MAX], p_out[HC_MAX], p_mix[HC_MAX * HC_MAX];
    const size_t t = rows[blockIdx.x];
    if (y != nullptr) hc_load(prev, n, p_in, p_out, p_mix);
    __syncthreads();
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const size_t idx = t * H + c;
        float xs[HC_MAX];
#pragma unroll
        for (int s = 0; s < HC_MAX; ++s) xs[s] = s < n ? x[(size_t)s * sstride + idx] : 0.f;
        float total = 0.f;
        if (y != nullptr) {
            const float yv = hc_pending(y, parts, pstride, idx);
            for (int r = 0; r < n; ++r) {
                float acc = p_out[r] * yv;
                for (int s = 0; s < n; ++s) acc = fmaf(p_mix[s * n + r], xs[s], acc);
                total += acc;
            }
        } else {
            for (int s = 0; s < n; ++s) total += xs[s];
        }
        out[(size_t)blockIdx.x * H + c] = total;
    }
}

// x[t] = table[ids[t]] * scale + the sinusoidal vector of positions[t]: entry 2i is sin(p f_i), entry 2i+1 cos(p f_i)
// with f_i = inv_freq[i] (float64, made on the host); the angle is taken in float64.
template <typename TW>
__global__ void embed_gather_sinusoid_kernel(const TW* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ positions,
                                             const double* __restrict__ inv_freq, float* __restrict__ x, int H, int V, float scale) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const double p = (double)positions[t];
    float* row = x + (size_t)t * H;
    const bool ok = id >= 0 && id < V;                  // refused on the host; never read out of range
    const TW* src = table + (size_t)(ok ? id : 0) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const double a = p * inv_freq[i >> 1];
        const float pe = (i & 1) ? (float)cos(a) : (float)sin(a);
        row[i] = (ok ? to_f(src[i]) * scale : 0.f) + pe;
    }
}

}  // namespace aien

using namespace aien;

template <typename TA, typename TH>
static int launch_hc_norm(size_t smem, cudaStream_t stream, float* x, size_t sstride, int n, const TA* y, int parts, size_t pstride,
                          const float* prev, const float* cur, const void* w, int wdt, float eps, TH* h, int T, int H,
                          const void* shift_w, int sdt, float* shift_state, const int* slot_map, const int* positions) {
    const bool wide = T <= 2 * 148 && H >= 1024;
    auto kern = wide ? hc_norm_kernel<TA, TH, 1024> : hc_norm_kernel<TA, TH, 256>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AIEN_E_STATE;
    kern<<<T, wide ? 1024 : 256, smem, stream>>>(x, sstride, n, y, parts, pstride, prev, cur, w, wdt, eps, h, H, shift_w, sdt, shift_state, slot_map, positions);
    return 0;
}

AIEN_API int aien_replicate_streams(float* x, size_t per, int n, cudaStream_t stream) {
    if (per == 0 || n <= 1) return 0;
    const int blocks = (int)((per + 255) / 256 < 148 * 8 ? (per + 255) / 256 : 148 * 8);
    replicate_streams_kernel<<<blocks, 256, 0, stream>>>(x, per, n);
    return launch_status();
}

// x float32 [n][T][H]; y: pending branch output ([T,H] in y_dt, or y_parts float32 partial products y_pstride apart) or
// null; prev / cur: parameter packs [in | out | mix] of the sublayer that produced y / of the one that reads now.
AIEN_API int aien_hc_norm(float* x, int n, const void* y, int y_dt, int y_parts, size_t y_pstride, const float* prev, const float* cur,
                          const void* w, int w_dt, float eps, void* h, int h_dt, int T, int H,
                          const void* shift_w, int s_dt, float* shift_state, const int* slot_map, const int* positions,
                          cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || n < 1 || n > HC_MAX || cur == nullptr || (y != nullptr && prev == nullptr) || (size_t)H * 4 > 160 * 1024) return AIEN_E_SHAPE;
    if (shift_w != nullptr && (shift_state == nullptr || slot_map == nullptr || positions == nullptr)) return AIEN_E_SHAPE;
    const size_t smem = (size_t)H * sizeof(float);
    const size_t sstride = (size_t)T * H;
    int rc = 0;
    AIEN_DISPATCH_DTYPE(y_dt, TA, AIEN_DISPATCH_DTYPE(h_dt, TH,
        (rc = launch_hc_norm<TA, TH>(smem, stream, x, sstride, n, (const TA*)y, y_parts, y_pstride, prev, cur, w, w_dt, eps, (TH*)h, T, H,
                                     shift_w, s_dt, shift_state, slot_map, positions))));
    if (rc != 0) return rc;
    return launch_status();
}

AIEN_API int aien_token_shift(const float* hn, const void* shift_w, int s_dt, float* state, const int* slot_map, const int* seq_of_token,
                              const int* q_start, const int* positions, void* h, int h_dt, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(h_dt, TH, (token_shift_kernel<TH><<<T, 256, 0, stream>>>(hn, shift_w, s_dt, state, slot_map, seq_of_token, q_start,
                                                                                positions, (TH*)h, H)));
    return launch_status();
}

AIEN_API int aien_hc_sum_rows(const float* x, int n, int T, const void* y, int y_dt, int y_parts, size_t y_pstride, const float* prev,
                              const int* rows, float* out, int R, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (H <= 0 || n < 1 || n > HC_MAX || (y != nullptr && prev == nullptr)) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(y_dt, TA, (hc_sum_rows_kernel<TA><<<R, 256, 0, stream>>>(x, (size_t)T * H, n, (const TA*)y, y_parts, y_pstride, prev,
                                                                                rows, out, H)));
    return launch_status();
}

AIEN_API int aien_embed_gather_sinusoid(const void* table, int table_dt, const int* ids, const int* positions, const double* inv_freq,
                                        float* x, int T, int H, int V, float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    AIEN_DISPATCH_DTYPE(table_dt, TW, (embed_gather_sinusoid_kernel<TW><<<T, 256, 0, stream>>>((const TW*)table, ids, positions, inv_freq,
                                                                                              x, H, V, scale)));
    return launch_status();
}
