// State-space recurrences with a float32 state per request: the selective scan (a state per channel) and the
// state-space-duality form (a state matrix per head), and the gate and grouped norm that follows the latter.
//
//   selective scan   per channel c and state n, token by token:
//                      dt = softplus(dtz[c] + dt_bias[c]) (made once per token and channel by a kernel ahead of the scan);
//                      S[c][n] = exp(dt * A[c][n]) * S[c][n] + dt * x[c] * B[n];
//                      y[c] = sum_n S[c][n] * C[n] + D[c] * x[c];  out[c] = y[c] * silu(z[c])
//   duality form     per head h (group g = h / (heads / groups)) with S [N][V], token by token:
//                      dt = softplus(dtr[h] + dt_bias[h]) and exp(-A[h] * dt) (made once per token and head, likewise);
//                      S = exp(-A[h] * dt) * S + dt * B[g] x[h]^T;  y[h] = S^T C[g] + D[h] * x[h]
//   gate and norm    v = y * silu(z); every one of `groups` equal parts of the row divided by its own root mean
//                    square (eps inside the root), times the weight, times a constant
//
// The state of request s lives in row slot_map[s] of `state` (rows of state_stride floats, the recurrence's part from
// s_off on); a portion whose first token has position 0 starts from zeros.  A few neighbouring lanes own a channel (or a
// column of a head's state), keep its N state values in registers between them and walk the portion's tokens in order, so
// a token's result depends only on the tokens before it, never on what else is in the batch.
// Everything here is float32 in both engine precisions; only the result leaves in the compute dtype.
//
// The portion-parallel forms cut a portion into segments that run side by side: every segment first runs from a zero
// state and records the product of its decays and its end state; the segments' starting states then follow one from
// another; a second pass repeats the segment from its true starting state and writes the results.
#include "common.cuh"
#include <math.h>

namespace aien {

__device__ __forceinline__ float ssm_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float ssm_softplus(float a) { return a > 20.f ? a : log1pf(expf(a)); }

constexpr int SSM_THREADS = 128;

// mode 0: the whole portion from the slot's state, results and new state written (the plain form).
// mode 1: segment `blockIdx.z` of the portion from zeros; writes its decay product and end state to scratch.
// mode 2: segment from the state the combine step left for it; writes results (the combine step wrote the slot).
struct Segments {
    int mode;
    int seg_len;
    float* decay;       // [segments][lanes]   product of the decays over the segment
    float* end;         // [segments][lanes]   mode 1: end state from zeros; after the combine: the state at the segment's end
    int nseg;           // the most segments one portion has (grid z); request s's segments start at q_start[s] / seg_len + s
};

// dtz[t][c] <- softplus(dtz[t][c] + bias[c]): the step sizes, once per token and channel, ahead of the scan.
__global__ void __launch_bounds__(256)
step_sizes_kernel(float* __restrict__ dtz, long lddt, const void* __restrict__ bias, int pdt, int T, int inner) {
    const int t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c < inner) dtz[(size_t)t * lddt + c] = ssm_softplus(dtz[(size_t)t * lddt + c] + load_dyn(bias, pdt, c));
}

// LANES neighbouring lanes share one channel: lane ln keeps the CH state values n = ln * CH .. ln * CH + CH - 1 in
// registers (N <= LANES * CH) and the partial sums of y meet by shuffles.  U tokens are fetched ahead of their arithmetic.
// The rows U tokens bring to one lane of the selective scan.
template <int U, int CH>
struct ScanRows {
    float dt[U], x[U], z[U], b[U][CH], c[U][CH];
    __device__ __forceinline__ void fetch(const float* __restrict__ xs, long ldx, const float* __restrict__ dtv, long lddt,
                                          const float* __restrict__ zs, long ldz, const float* __restrict__ bc, long ldbc, int b_off,
                                          int c_off, int ch, int n0, int N, int t, int t1, bool wants_z) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int tt = t + u < t1 ? t + u : t1 - 1;            // beyond the portion's end the last token's rows are read again
            dt[u] = dtv[(size_t)tt * lddt + ch];
            x[u] = xs[(size_t)tt * ldx + ch];
            z[u] = wants_z ? zs[(size_t)tt * ldz + ch] : 0.f;
            const float* br = bc + (size_t)tt * ldbc + b_off + n0;
            const float* cr = bc + (size_t)tt * ldbc + c_off + n0;
#pragma unroll
            for (int i = 0; i < CH; ++i) { const bool in = n0 + i < N; b[u][i] = in ? br[i] : 0.f; c[u][i] = in ? cr[i] : 0.f; }
        }
    }
};

// exp for the decays: full precision where the result leaves in float32; through the special-function unit (relative
// error near 2^-21) where it leaves in bfloat16, whose own rounding is a hundred times coarser.
template <typename TO> __device__ __forceinline__ float decay_exp(float v);
template <> __device__ __forceinline__ float decay_exp<float>(float v) { return expf(v); }
template <> __device__ __forceinline__ float decay_exp<__nv_bfloat16>(float v) { return __expf(v); }

template <int LANES, int CH, int U, typename TO>
__global__ void __launch_bounds__(SSM_THREADS)
selective_scan_kernel(const float* __restrict__ x, long ldx, const float* __restrict__ dtv, long lddt,
                      const float* __restrict__ bc, long ldbc, int b_off, int c_off, const float* __restrict__ z, long ldz,
                      const float* __restrict__ A, const void* __restrict__ D, int pdt,
                      float* __restrict__ state, size_t state_stride, size_t s_off, const int* __restrict__ slots,
                      const int* __restrict__ q_start, const int* __restrict__ positions,
                      TO* __restrict__ out, long ldo, int inner, int N, Segments sg) {
    const int s = blockIdx.y, gid = blockIdx.x * SSM_THREADS + threadIdx.x;
    const bool live = gid / LANES < inner;
    const int c = live ? gid / LANES : inner - 1, ln = gid % LANES, n0 = ln * CH;   // lanes beyond the last channel repeat it and write nothing
    int t0 = q_start[s];
    int t1 = q_start[s + 1];
    const bool fresh = positions[t0] == 0;
    const int seg = sg.mode == 0 ? 0 : blockIdx.z;
    const size_t seg0 = sg.mode == 0 ? 0 : (size_t)(t0 / sg.seg_len + s);          // the request's first segment in the scratch
    if (sg.mode != 0) {
        t0 += seg * sg.seg_len;
        if (t0 + sg.seg_len < t1) t1 = t0 + sg.seg_len;                            // a segment beyond the portion's end walks no token
    }
    const bool mine = t0 < t1 || sg.mode == 0;
    float* st = state + (size_t)slots[s] * state_stride + s_off + (size_t)c * N + n0;
    const size_t lanes = (size_t)inner * N;
    const size_t so = (seg0 + seg) * lanes + (size_t)c * N + n0;
    const float* init = sg.mode == 2 ? (seg > 0 ? sg.end + so - lanes : sg.decay + so) : st;      // see segment_combine_kernel
    const bool zero = !mine || sg.mode == 1 || (sg.mode == 0 && fresh);
    float S[CH], a[CH], P[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const bool in = n0 + i < N;
        a[i] = in ? A[(size_t)c * N + n0 + i] : 0.f;
        P[i] = 1.f;
        S[i] = (in && !zero) ? init[i] : 0.f;
    }
    const float dskip = load_dyn(D, pdt, c);
    const bool wants_z = ln == 0 && sg.mode != 1;
    // The rows of U tokens are fetched while the U tokens before them are worked on (two sets of registers): at the few
    // warps a scheduler has here, a fetch that started only after the arithmetic would be waited for in full.
    ScanRows<U, CH> cur, nxt;
    if (t0 < t1) cur.fetch(x, ldx, dtv, lddt, z, ldz, bc, ldbc, b_off, c_off, c, n0, N, t0, t1, wants_z);
    for (int t = t0; t < t1; t += U) {
        if (t + U < t1) nxt.fetch(x, ldx, dtv, lddt, z, ldz, bc, ldbc, b_off, c_off, c, n0, N, t + U, t1, wants_z);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (t + u < t1) {
                const float dt = cur.dt[u], dx = dt * cur.x[u];
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const float e = decay_exp<TO>(dt * a[i]);
                    S[i] = fmaf(e, S[i], dx * cur.b[u][i]);
                    if (sg.mode == 1) P[i] *= e;
                    y = fmaf(S[i], cur.c[u][i], y);
                }
                if (sg.mode != 1) {
#pragma unroll
                    for (int o = 1; o < LANES; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                    if (ln == 0 && live) out[(size_t)(t + u) * ldo + c] = from_f<TO>(fmaf(dskip, cur.x[u], y) * ssm_silu(cur.z[u]));
                }
            }
        }
        cur = nxt;
    }
    if (!live || !mine) return;
    if (sg.mode == 1) {
#pragma unroll
        for (int i = 0; i < CH; ++i) if (n0 + i < N) { sg.decay[so + i] = P[i]; sg.end[so + i] = S[i]; }
    } else if (sg.mode == 0) {
#pragma unroll
        for (int i = 0; i < CH; ++i) if (n0 + i < N) st[i] = S[i];
    }
}

// Between the two passes: end[k] becomes the state at the end of segment k with the true start, one after another;
// the state the portion started from moves into decay[0] (the second pass reads no slot) and the state after the
// portion's last token into the slot.  lanes = values per request (inner * N, or heads * N * V).
__global__ void __launch_bounds__(256)
segment_combine_kernel(float* __restrict__ state, size_t state_stride, size_t s_off, const int* __restrict__ slots,
                       const int* __restrict__ q_start, const int* __restrict__ positions, Segments sg, size_t lanes) {
    const int s = blockIdx.y;
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= lanes) return;
    const int t0 = q_start[s], n_tok = q_start[s + 1] - t0;
    const int used = (n_tok + sg.seg_len - 1) / sg.seg_len;
    const size_t seg0 = (size_t)(t0 / sg.seg_len + s);
    float* slot = state + (size_t)slots[s] * state_stride + s_off + i;
    const float init = positions[t0] == 0 ? 0.f : *slot;
    float cur = init;
    for (int k = 0; k < used; ++k) {
        const size_t o = (seg0 + k) * lanes + i;
        cur = fmaf(sg.decay[o], cur, sg.end[o]);
        sg.end[o] = cur;
    }
    sg.decay[seg0 * lanes + i] = init;
    *slot = cur;
}

// steps[t][h] = softplus(dtr[t][h] + bias[h]) and steps[t][heads + h] = exp(-A[h] * that): once per token and head.
__global__ void __launch_bounds__(256)
ssd_steps_kernel(const float* __restrict__ dtr, long lddt, const float* __restrict__ A, const void* __restrict__ bias, int pdt,
                 float* __restrict__ steps, int T, int heads) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= T * heads) return;
    const int t = i / heads, h = i - t * heads;
    const float dt = ssm_softplus(dtr[(size_t)t * lddt + h] + load_dyn(bias, pdt, h));
    steps[(size_t)t * 2 * heads + h] = dt;
    steps[(size_t)t * 2 * heads + heads + h] = expf(-A[h] * dt);
}

// LANES neighbouring lanes share one (head, value column): lane ln keeps the CH state values n = ln * CH .. ln * CH + CH - 1
// of S[:, v] in registers (N <= LANES * CH) and the partial sums of y meet by shuffles.  The slot holds S as
// [heads][value column][N], so the lanes read one contiguous row.  VEC: B, C and the state move as float4.  U tokens are
// fetched ahead of their arithmetic.
constexpr int SSD_THREADS = 256;

template <int LANES, int CH, int U, bool VEC>
__global__ void __launch_bounds__(SSD_THREADS)
ssd_scan_kernel(const float* __restrict__ xbc, long ld, int x_off, int b_off, int c_off,
                const float* __restrict__ steps, const void* __restrict__ D, int pdt, float* __restrict__ state, size_t state_stride, size_t s_off,
                const int* __restrict__ slots, const int* __restrict__ q_start, const int* __restrict__ positions,
                float* __restrict__ y_out, long ldy, int heads, int V, int G, int N, Segments sg) {
    const int s = blockIdx.y, gid = blockIdx.x * SSD_THREADS + threadIdx.x;
    const int cols = heads * V;
    const bool live = gid / LANES < cols;
    const int col = live ? gid / LANES : cols - 1, ln = gid % LANES;       // lanes beyond the last column repeat it and write nothing
    const int h = col / V, g = h / (heads / G), n0 = ln * CH;
    int t0 = q_start[s];
    int t1 = q_start[s + 1];
    const bool fresh = positions[t0] == 0;
    const int seg = sg.mode == 0 ? 0 : blockIdx.z;
    const size_t seg0 = sg.mode == 0 ? 0 : (size_t)(t0 / sg.seg_len + s);
    if (sg.mode != 0) {
        t0 += seg * sg.seg_len;
        if (t0 + sg.seg_len < t1) t1 = t0 + sg.seg_len;              // a segment beyond the portion's end walks no token
    }
    float* st = state + (size_t)slots[s] * state_stride + s_off + (size_t)col * N + n0;
    const size_t lanes = (size_t)cols * N;
    const size_t so = (seg0 + seg) * lanes + (size_t)col * N + n0;
    const bool mine = t0 < t1 || sg.mode == 0;
    float S[CH];
    float P = 1.f;
    const float* init = sg.mode == 2 ? (seg > 0 ? sg.end + so - lanes : sg.decay + so) : st;
    const bool zero = !mine || sg.mode == 1 || (sg.mode == 0 && fresh);
    if (VEC) {
#pragma unroll
        for (int i = 0; i < CH; i += 4) {
            float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (!zero && n0 + i < N) v4 = *reinterpret_cast<const float4*>(init + i);
            S[i] = v4.x;
            if (i + 1 < CH) S[i + 1] = v4.y;
            if (i + 2 < CH) S[i + 2] = v4.z;
            if (i + 3 < CH) S[i + 3] = v4.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < CH; ++i) S[i] = (!zero && n0 + i < N) ? init[i] : 0.f;
    }
    const float dskip = load_dyn(D, pdt, h);
    for (int t = t0; t < t1; t += U) {
        float dtu[U], eu[U], xu[U], bv[U][CH], cv[U][CH];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int tt = t + u < t1 ? t + u : t1 - 1;
            dtu[u] = steps[(size_t)tt * 2 * heads + h];
            eu[u] = steps[(size_t)tt * 2 * heads + heads + h];
            xu[u] = xbc[(size_t)tt * ld + x_off + col];
            const float* br = xbc + (size_t)tt * ld + b_off + (size_t)g * N + n0;
            const float* cr = xbc + (size_t)tt * ld + c_off + (size_t)g * N + n0;
            if (VEC) {
#pragma unroll
                for (int i = 0; i < CH; i += 4) {
                    float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), c4 = b4;
                    if (n0 + i < N) { b4 = *reinterpret_cast<const float4*>(br + i); c4 = *reinterpret_cast<const float4*>(cr + i); }
                    bv[u][i] = b4.x; cv[u][i] = c4.x;
                    if (i + 1 < CH) { bv[u][i + 1] = b4.y; cv[u][i + 1] = c4.y; }
                    if (i + 2 < CH) { bv[u][i + 2] = b4.z; cv[u][i + 2] = c4.z; }
                    if (i + 3 < CH) { bv[u][i + 3] = b4.w; cv[u][i + 3] = c4.w; }
                }
            } else {
#pragma unroll
                for (int i = 0; i < CH; ++i) { const bool in = n0 + i < N; bv[u][i] = in ? br[i] : 0.f; cv[u][i] = in ? cr[i] : 0.f; }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (t + u < t1) {
                const float e = eu[u], dx = dtu[u] * xu[u];
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    S[i] = fmaf(e, S[i], dx * bv[u][i]);
                    y = fmaf(S[i], cv[u][i], y);
                }
                if (sg.mode == 1) {
                    P *= e;
                } else {
#pragma unroll
                    for (int o = 1; o < LANES; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                    if (ln == 0 && live) y_out[(size_t)(t + u) * ldy + col] = fmaf(dskip, xu[u], y);
                }
            }
        }
    }
    if (!live || !mine) return;
    if (sg.mode == 1) {
#pragma unroll
        for (int i = 0; i < CH; ++i) if (n0 + i < N) { sg.decay[so + i] = P; sg.end[so + i] = S[i]; }
    } else if (sg.mode == 0) {
#pragma unroll
        for (int i = 0; i < CH; ++i) if (n0 + i < N) st[i] = S[i];
    }
}

// out[t][o_off + c] = (y * silu(z))[c] / rms(part of c) * w[c] * mult; one CTA per (token, part)
template <typename TO>
__global__ void __launch_bounds__(256)
gate_group_norm_kernel(const float* __restrict__ y, long ldy, const float* __restrict__ z, long ldz, const void* __restrict__ w, int wdt,
                       float eps, float mult, TO* __restrict__ out, long ldo, int part) {
    __shared__ float red[32];
    const int t = blockIdx.x, c0 = blockIdx.y * part;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += 256) {
        const float v = y[(size_t)t * ldy + c0 + i] * ssm_silu(z[(size_t)t * ldz + c0 + i]);
        ss = fmaf(v, v, ss);
    }
    const float r = mult / sqrtf(block_sum(ss, red) / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += 256) {
        const float v = y[(size_t)t * ldy + c0 + i] * ssm_silu(z[(size_t)t * ldz + c0 + i]);
        out[(size_t)t * ldo + c0 + i] = from_f<TO>(v * r * load_dyn(w, wdt, c0 + i));
    }
}

}  // namespace aien

using namespace aien;

// Floats of scratch that the portion-parallel forms need: T tokens of S requests in segments of seg_len tokens.
AIEN_API long aien_ssm_segments_scratch(int T, int S, int seg_len, long lanes) { return 2L * (T / seg_len + S) * lanes; }

struct ScanArgs {
    const float* x; long ldx; float* dtz; long lddt; const float* bc; long ldbc; int b_off, c_off; const float* z; long ldz;
    const float* A; const void* dt_bias; const void* D; int p_dt; float* state; size_t state_stride, s_off; const int* slots;
    const int* q_start; const int* positions; void* out; long ldo; int T, S, inner, N; Segments sg; cudaStream_t stream;
};

template <int LANES, int CH, int U, typename TO>
static void launch_selective_scan(const ScanArgs& a) {
    auto kern = selective_scan_kernel<LANES, CH, U, TO>;
    const unsigned gx = (unsigned)(((long)a.inner * LANES + SSM_THREADS - 1) / SSM_THREADS);
    Segments sg = a.sg;
    const dim3 grid(gx, a.S, sg.mode == 0 ? 1 : sg.nseg);
    step_sizes_kernel<<<dim3((a.inner + 255) / 256, a.T), 256, 0, a.stream>>>(a.dtz, a.lddt, a.dt_bias, a.p_dt, a.T, a.inner);
    kern<<<grid, SSM_THREADS, 0, a.stream>>>(a.x, a.ldx, a.dtz, a.lddt, a.bc, a.ldbc, a.b_off, a.c_off, a.z, a.ldz, a.A, a.D, a.p_dt,
                                             a.state, a.state_stride, a.s_off, a.slots, a.q_start, a.positions, (TO*)a.out, a.ldo, a.inner, a.N, sg);
    if (sg.mode == 0) return;
    const size_t lanes = (size_t)a.inner * a.N;
    segment_combine_kernel<<<dim3((unsigned)((lanes + 255) / 256), a.S), 256, 0, a.stream>>>(a.state, a.state_stride, a.s_off, a.slots, a.q_start,
                                                                                             a.positions, sg, lanes);
    sg.mode = 2;
    kern<<<grid, SSM_THREADS, 0, a.stream>>>(a.x, a.ldx, a.dtz, a.lddt, a.bc, a.ldbc, a.b_off, a.c_off, a.z, a.ldz, a.A, a.D, a.p_dt,
                                             a.state, a.state_stride, a.s_off, a.slots, a.q_start, a.positions, (TO*)a.out, a.ldo, a.inner, a.N, sg);
}

template <typename TO>
static int dispatch_selective_scan(const ScanArgs& a) {
    const int N = a.N;
    if (N > 128) return AIEN_E_SHAPE;
    if (a.T == a.S) {
        // single tokens: a CTA lives for one token, so what counts is how many are resident and how much each moves:
        // four lanes a channel, no rows fetched ahead (fewer registers)
        if (N <= 4) launch_selective_scan<4, 1, 1, TO>(a);
        else if (N <= 8) launch_selective_scan<4, 2, 1, TO>(a);
        else if (N <= 16) launch_selective_scan<4, 4, 1, TO>(a);
        else if (N <= 32) launch_selective_scan<4, 8, 1, TO>(a);
        else if (N <= 64) launch_selective_scan<16, 4, 1, TO>(a);
        else launch_selective_scan<16, 8, 1, TO>(a);
        return 0;
    }
    if (N <= 2) launch_selective_scan<1, 2, 4, TO>(a);
    else if (N <= 8) launch_selective_scan<4, 2, 4, TO>(a);
    else if (N <= 16) launch_selective_scan<16, 1, 4, TO>(a);
    else if (N <= 32) launch_selective_scan<16, 2, 4, TO>(a);
    else if (N <= 64) launch_selective_scan<16, 4, 4, TO>(a);
    else launch_selective_scan<16, 8, 2, TO>(a);
    return 0;
}

// x [T, ldx] (after convolution and silu), dtz [T, lddt] = W_dt dt before its bias (overwritten with the step sizes
// softplus(dtz + dt_bias)), bc [T, ldbc] with B at b_off and C at c_off (N numbers each, N <= 128), z [T, ldz] the gate's
// input, A float32 [inner, N] (negative rates), dt_bias and D [inner] in p_dt.  seg_len > 0: portions are cut into nseg
// segments of seg_len tokens that run side by side (scratch float32, aien_ssm_segments_scratch(T, S, seg_len, inner * N)
// numbers); nseg * seg_len must cover the longest portion; T is the number of tokens in the step.
AIEN_API int aien_selective_scan(const float* x, long ldx, float* dtz, long lddt, const float* bc, long ldbc, int b_off, int c_off,
                                 const float* z, long ldz, const float* A, const void* dt_bias, const void* D, int p_dt,
                                 float* state, size_t state_stride, size_t s_off, const int* slots, const int* q_start,
                                 const int* positions, void* out, int o_dt, long ldo, int T, int S, int inner, int N,
                                 int seg_len, int nseg, float* scratch, cudaStream_t stream) {
    if (S <= 0 || T <= 0) return 0;
    if (inner <= 0 || N <= 0 || S > 65535 || T > 65535 || nseg > 65535) return AIEN_E_SHAPE;
    Segments sg{0, 0, nullptr, nullptr, 1};
    if (seg_len > 0 && nseg > 1) {
        if (scratch == nullptr) return AIEN_E_SHAPE;
        sg = Segments{1, seg_len, scratch, scratch + (size_t)(T / seg_len + S) * (size_t)inner * N, nseg};
    }
    const ScanArgs a{x, ldx, dtz, lddt, bc, ldbc, b_off, c_off, z, ldz, A, dt_bias, D, p_dt, state, state_stride, s_off, slots, q_start,
                     positions, out, ldo, T, S, inner, N, sg, stream};
    int rc = 0;
    AIEN_DISPATCH_DTYPE(o_dt, TO, (rc = dispatch_selective_scan<TO>(a)));
    if (rc != 0) return rc;
    return launch_status();
}

struct SsdArgs {
    const float* xbc; long ld; int x_off, b_off, c_off; const float* dtr; long lddt; const float* A; const void* dt_bias; const void* D;
    int p_dt; float* state; size_t state_stride, s_off; const int* slots; const int* q_start; const int* positions; float* y; long ldy;
    int T, S, heads, V, G, N; Segments sg; float* steps; cudaStream_t stream;
};

template <int LANES, int CH, int U, bool VEC>
static void launch_ssd_scan(const SsdArgs& a) {
    auto kern = ssd_scan_kernel<LANES, CH, U, VEC>;
    const long threads = (long)a.heads * a.V * LANES;
    const unsigned gx = (unsigned)((threads + SSD_THREADS - 1) / SSD_THREADS);
    Segments sg = a.sg;
    const dim3 grid(gx, a.S, sg.mode == 0 ? 1 : sg.nseg);
    ssd_steps_kernel<<<(unsigned)(((long)a.T * a.heads + 255) / 256), 256, 0, a.stream>>>(a.dtr, a.lddt, a.A, a.dt_bias, a.p_dt, a.steps, a.T, a.heads);
    kern<<<grid, SSD_THREADS, 0, a.stream>>>(a.xbc, a.ld, a.x_off, a.b_off, a.c_off, a.steps, a.D, a.p_dt, a.state,
                                             a.state_stride, a.s_off, a.slots, a.q_start, a.positions, a.y, a.ldy, a.heads, a.V, a.G, a.N, sg);
    if (sg.mode == 0) return;
    const size_t lanes = (size_t)a.heads * a.N * a.V;
    segment_combine_kernel<<<dim3((unsigned)((lanes + 255) / 256), a.S), 256, 0, a.stream>>>(a.state, a.state_stride, a.s_off, a.slots, a.q_start,
                                                                                             a.positions, sg, lanes);
    sg.mode = 2;
    kern<<<grid, SSD_THREADS, 0, a.stream>>>(a.xbc, a.ld, a.x_off, a.b_off, a.c_off, a.steps, a.D, a.p_dt, a.state,
                                             a.state_stride, a.s_off, a.slots, a.q_start, a.positions, a.y, a.ldy, a.heads, a.V, a.G, a.N, sg);
}

// xbc [T, ld] (after convolution and silu): x (heads * V) at x_off, B (G * N) at b_off, C (G * N) at c_off; dtr [T, lddt]
// the raw step sizes, one per head; A float32 [heads] (positive rates exp(A_log)); dt_bias and D [heads] in p_dt;
// y float32 [T, ldy]; N <= 256; steps: float32 scratch of T * 2 * heads numbers (the step sizes and decays of the step's
// tokens).  The slot holds S as [heads][V][N].  Segments as for aien_selective_scan, with heads * N * V state values per
// request.
AIEN_API int aien_ssd_scan(const float* xbc, long ld, int x_off, int b_off, int c_off, const float* dtr, long lddt, const float* A,
                           const void* dt_bias, const void* D, int p_dt, float* state, size_t state_stride, size_t s_off,
                           const int* slots, const int* q_start, const int* positions, float* y, long ldy, int T, int S, int heads, int V,
                           int G, int N, int seg_len, int nseg, float* scratch, float* steps, cudaStream_t stream) {
    if (S <= 0 || T <= 0) return 0;
    if (heads <= 0 || V <= 0 || G <= 0 || heads % G || N <= 0 || N > 256 || S > 65535 || nseg > 65535 || steps == nullptr) return AIEN_E_SHAPE;
    Segments sg{0, 0, nullptr, nullptr, 1};
    if (seg_len > 0 && nseg > 1) {
        if (scratch == nullptr) return AIEN_E_SHAPE;
        sg = Segments{1, seg_len, scratch, scratch + (size_t)(T / seg_len + S) * (size_t)heads * N * V, nseg};
    }
    const SsdArgs a{xbc, ld, x_off, b_off, c_off, dtr, lddt, A, dt_bias, D, p_dt, state, state_stride, s_off, slots, q_start, positions,
                    y, ldy, T, S, heads, V, G, N, sg, steps, stream};
    // float4 moves: every lane's first state value, B and C value on a 16-byte boundary, whole groups of four inside N
    const bool vec = N >= 128 && N % 4 == 0 && ld % 4 == 0 && b_off % 4 == 0 && c_off % 4 == 0 && state_stride % 4 == 0 && s_off % 4 == 0 &&
                     ((uintptr_t)xbc & 15) == 0 && ((uintptr_t)state & 15) == 0 && (scratch == nullptr || ((uintptr_t)scratch & 15) == 0);
    if (T == S) {                                     // single tokens: no rows fetched ahead (fewer registers, more CTAs resident)
        if (N <= 8) launch_ssd_scan<8, 1, 1, false>(a);
        else if (N <= 16) launch_ssd_scan<8, 2, 1, false>(a);
        else if (N <= 32) launch_ssd_scan<32, 1, 1, false>(a);
        else if (N <= 64) launch_ssd_scan<32, 2, 1, false>(a);
        else if (N <= 128) { if (vec) launch_ssd_scan<32, 4, 1, true>(a); else launch_ssd_scan<32, 4, 1, false>(a); }
        else { if (vec && N % 8 == 0) launch_ssd_scan<32, 8, 1, true>(a); else launch_ssd_scan<32, 8, 1, false>(a); }
        return launch_status();
    }
    if (N <= 8) launch_ssd_scan<8, 1, 4, false>(a);
    else if (N <= 16) launch_ssd_scan<8, 2, 4, false>(a);
    else if (N <= 32) launch_ssd_scan<32, 1, 4, false>(a);
    else if (N <= 64) launch_ssd_scan<32, 2, 4, false>(a);
    else if (N <= 128) { if (vec) launch_ssd_scan<32, 4, 4, true>(a); else launch_ssd_scan<32, 4, 4, false>(a); }
    else { if (vec && N % 8 == 0) launch_ssd_scan<32, 8, 2, true>(a); else launch_ssd_scan<32, 8, 2, false>(a); }
    return launch_status();
}

// y float32 [T, ldy], z float32 [T, ldz] (the gate's input), w [width] in w_dt; the row is `groups` equal parts.
// out [T, ldo] in o_dt = (y * silu(z)) / rms(its part) * w * mult.
AIEN_API int aien_gate_group_norm(const float* y, long ldy, const float* z, long ldz, const void* w, int w_dt, float eps, float mult,
                                  void* out, int o_dt, long ldo, int T, int width, int groups, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (groups <= 0 || width <= 0 || width % groups || groups > 65535) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(o_dt, TO,
        (gate_group_norm_kernel<TO><<<dim3(T, groups), 256, 0, stream>>>(y, ldy, z, ldz, w, w_dt, eps, mult, (TO*)out, ldo, width / groups)));
    return launch_status();
}
