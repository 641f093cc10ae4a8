// State-space recurrences with a float32 state per request: the selective scan (a state per channel) and the
// state-space-duality form (a state matrix per head), and the gate and grouped norm that follows the latter.
//
//   selective scan   per channel c and state n, token by token:
//                      dt = softplus(dtz[c] + dt_bias[c]);  S[c][n] = exp(dt * A[c][n]) * S[c][n] + dt * x[c] * B[n];
//                      y[c] = sum_n S[c][n] * C[n] + D[c] * x[c];  out[c] = y[c] * silu(z[c])
//   duality form     per head h (group g = h / (heads / groups)) with S [N][V], token by token:
//                      dt = softplus(dtr[h] + dt_bias[h]);  S = exp(-A[h] * dt) * S + dt * B[g] x[h]^T;
//                      y[h] = S^T C[g] + D[h] * x[h]
//   gate and norm    v = y * silu(z); every one of `groups` equal parts of the row divided by its own root mean
//                    square (eps inside the root), times the weight, times a constant
//
// The state of request s lives in row slot_map[s] of `state` (rows of state_stride floats, the recurrence's part from
// s_off on); a portion whose first token has position 0 starts from zeros.  One thread owns a channel (or a column of
// a head's state), keeps its N state values in registers and walks the portion's tokens in order, so a token's result
// depends only on the tokens before it, never on how the request was cut into steps or on what else is in the batch.
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

constexpr int SSM_THREADS = 64;

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

template <int NMAX, typename TO>
__global__ void __launch_bounds__(SSM_THREADS)
selective_scan_kernel(const float* __restrict__ x, long ldx, const float* __restrict__ dtz, long lddt,
                      const float* __restrict__ bc, long ldbc, int b_off, int c_off, const float* __restrict__ z, long ldz,
                      const float* __restrict__ A, const void* __restrict__ dt_bias, const void* __restrict__ D, int pdt,
                      float* __restrict__ state, size_t state_stride, size_t s_off, const int* __restrict__ slots,
                      const int* __restrict__ q_start, const int* __restrict__ positions,
                      TO* __restrict__ out, long ldo, int inner, int N, Segments sg) {
    const int s = blockIdx.y, c = blockIdx.x * SSM_THREADS + threadIdx.x;
    if (c >= inner) return;
    int t0 = q_start[s];
    int t1 = q_start[s + 1];
    const bool fresh = positions[t0] == 0;
    const int seg = sg.mode == 0 ? 0 : blockIdx.z;
    const int p0 = t0;
    if (sg.mode != 0) {
        t0 = p0 + seg * sg.seg_len;
        if (t0 >= t1) return;
        if (t0 + sg.seg_len < t1) t1 = t0 + sg.seg_len;
    }
    float* st = state + (size_t)slots[s] * state_stride + s_off + (size_t)c * N;
    float S[NMAX], a[NMAX], P[NMAX];
    const size_t seg0 = sg.mode == 0 ? 0 : (size_t)(p0 / sg.seg_len + s);          // the request's first segment in the scratch
    const size_t so = ((seg0 + seg) * inner + c) * (size_t)N;
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
        a[n] = n < N ? A[(size_t)c * N + n] : 0.f;
        P[n] = 1.f;
        if (n >= N || sg.mode == 1) S[n] = 0.f;
        else if (sg.mode == 2) S[n] = seg > 0 ? sg.end[so - (size_t)inner * N + n] : sg.decay[so + n];      // see segment_combine_kernel
        else S[n] = fresh ? 0.f : st[n];
    }
    const float bias = load_dyn(dt_bias, pdt, c), dskip = load_dyn(D, pdt, c);
    for (int t = t0; t < t1; ++t) {
        const float dt = ssm_softplus(dtz[(size_t)t * lddt + c] + bias);
        const float xv = x[(size_t)t * ldx + c];
        const float dx = dt * xv;
        const float* br = bc + (size_t)t * ldbc + b_off;
        const float* cr = bc + (size_t)t * ldbc + c_off;
        float y = 0.f;
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
            if (n < N) {
                const float e = expf(dt * a[n]);
                S[n] = fmaf(e, S[n], dx * br[n]);
                if (sg.mode == 1) P[n] *= e;
                y = fmaf(S[n], cr[n], y);
            }
        }
        if (sg.mode != 1) {
            y = fmaf(dskip, xv, y);
            out[(size_t)t * ldo + c] = from_f<TO>(y * ssm_silu(z[(size_t)t * ldz + c]));
        }
    }
    if (sg.mode == 1) {
#pragma unroll
        for (int n = 0; n < NMAX; ++n) if (n < N) { sg.decay[so + n] = P[n]; sg.end[so + n] = S[n]; }
    } else if (sg.mode == 0) {
#pragma unroll
        for (int n = 0; n < NMAX; ++n) if (n < N) st[n] = S[n];
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

// One thread per (head, value column): its N state values S[:, v] stay in registers.
template <int NMAX>
__global__ void __launch_bounds__(SSM_THREADS)
ssd_scan_kernel(const float* __restrict__ xbc, long ld, int x_off, int b_off, int c_off,
                const float* __restrict__ dtr, long lddt, const float* __restrict__ A, const void* __restrict__ dt_bias,
                const void* __restrict__ D, int pdt, float* __restrict__ state, size_t state_stride, size_t s_off,
                const int* __restrict__ slots, const int* __restrict__ q_start, const int* __restrict__ positions,
                float* __restrict__ y_out, long ldy, int heads, int V, int G, int N, Segments sg) {
    const int s = blockIdx.y, idx = blockIdx.x * SSM_THREADS + threadIdx.x;
    if (idx >= heads * V) return;
    const int h = idx / V, v = idx - h * V, g = h / (heads / G);
    int t0 = q_start[s];
    int t1 = q_start[s + 1];
    const bool fresh = positions[t0] == 0;
    const int seg = sg.mode == 0 ? 0 : blockIdx.z;
    const size_t seg0 = sg.mode == 0 ? 0 : (size_t)(t0 / sg.seg_len + s);
    if (sg.mode != 0) {
        t0 += seg * sg.seg_len;
        if (t0 >= t1) return;
        if (t0 + sg.seg_len < t1) t1 = t0 + sg.seg_len;
    }
    float* st = state + (size_t)slots[s] * state_stride + s_off + (size_t)h * N * V + v;       // S[n][v] at st[n * V]
    const size_t lanes = (size_t)heads * N * V;
    const size_t so = (seg0 + seg) * lanes + (size_t)h * N * V + v;
    float S[NMAX];
    float P = 1.f;
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
        if (n >= N || sg.mode == 1) S[n] = 0.f;
        else if (sg.mode == 2) S[n] = seg > 0 ? sg.end[so - lanes + (size_t)n * V] : sg.decay[so + (size_t)n * V];
        else S[n] = fresh ? 0.f : st[(size_t)n * V];
    }
    const float rate = A[h], bias = load_dyn(dt_bias, pdt, h), dskip = load_dyn(D, pdt, h);
    for (int t = t0; t < t1; ++t) {
        const float dt = ssm_softplus(dtr[(size_t)t * lddt + h] + bias);
        const float e = expf(-rate * dt);
        const float xv = xbc[(size_t)t * ld + x_off + idx];
        const float dx = dt * xv;
        const float* br = xbc + (size_t)t * ld + b_off + (size_t)g * N;
        const float* cr = xbc + (size_t)t * ld + c_off + (size_t)g * N;
        float y = 0.f;
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
            if (n < N) {
                S[n] = fmaf(e, S[n], dx * br[n]);
                y = fmaf(S[n], cr[n], y);
            }
        }
        if (sg.mode == 1) P *= e;
        else y_out[(size_t)t * ldy + idx] = fmaf(dskip, xv, y);
    }
    if (sg.mode == 1) {
#pragma unroll
        for (int n = 0; n < NMAX; ++n) if (n < N) { sg.decay[so + (size_t)n * V] = P; sg.end[so + (size_t)n * V] = S[n]; }
    } else if (sg.mode == 0) {
#pragma unroll
        for (int n = 0; n < NMAX; ++n) if (n < N) st[(size_t)n * V] = S[n];
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

static int pick_nmax(int N) { return N <= 16 ? 16 : N <= 32 ? 32 : N <= 64 ? 64 : N <= 128 ? 128 : N <= 256 ? 256 : 0; }

// Floats of scratch that the portion-parallel forms need: T tokens of S requests in segments of seg_len tokens.
AIEN_API long aien_ssm_segments_scratch(int T, int S, int seg_len, long lanes) { return 2L * (T / seg_len + S) * lanes; }

struct ScanArgs {
    const float* x; long ldx; const float* dtz; long lddt; const float* bc; long ldbc; int b_off, c_off; const float* z; long ldz;
    const float* A; const void* dt_bias; const void* D; int p_dt; float* state; size_t state_stride, s_off; const int* slots;
    const int* q_start; const int* positions; void* out; long ldo; int S, inner, N; Segments sg; cudaStream_t stream;
};

template <int NMAX, typename TO>
static void launch_selective_scan(const ScanArgs& a) {
    auto kern = selective_scan_kernel<NMAX, TO>;
    const unsigned gx = (unsigned)((a.inner + SSM_THREADS - 1) / SSM_THREADS);
    Segments sg = a.sg;
    const dim3 grid(gx, a.S, sg.mode == 0 ? 1 : sg.nseg);
    kern<<<grid, SSM_THREADS, 0, a.stream>>>(a.x, a.ldx, a.dtz, a.lddt, a.bc, a.ldbc, a.b_off, a.c_off, a.z, a.ldz, a.A, a.dt_bias, a.D, a.p_dt,
                                             a.state, a.state_stride, a.s_off, a.slots, a.q_start, a.positions, (TO*)a.out, a.ldo, a.inner, a.N, sg);
    if (sg.mode == 0) return;
    const size_t lanes = (size_t)a.inner * a.N;
    segment_combine_kernel<<<dim3((unsigned)((lanes + 255) / 256), a.S), 256, 0, a.stream>>>(a.state, a.state_stride, a.s_off, a.slots, a.q_start,
                                                                                             a.positions, sg, lanes);
    sg.mode = 2;
    kern<<<grid, SSM_THREADS, 0, a.stream>>>(a.x, a.ldx, a.dtz, a.lddt, a.bc, a.ldbc, a.b_off, a.c_off, a.z, a.ldz, a.A, a.dt_bias, a.D, a.p_dt,
                                             a.state, a.state_stride, a.s_off, a.slots, a.q_start, a.positions, (TO*)a.out, a.ldo, a.inner, a.N, sg);
}

template <typename TO>
static int dispatch_selective_scan(const ScanArgs& a) {
    switch (pick_nmax(a.N)) {
        case 16: launch_selective_scan<16, TO>(a); break;
        case 32: launch_selective_scan<32, TO>(a); break;
        case 64: launch_selective_scan<64, TO>(a); break;
        case 128: launch_selective_scan<128, TO>(a); break;
        default: return AIEN_E_SHAPE;
    }
    return 0;
}

// x [T, ldx] (after convolution and silu), dtz [T, lddt] = W_dt dt before its bias, bc [T, ldbc] with B at b_off and C
// at c_off (N numbers each, N <= 128), z [T, ldz] the gate's input, A float32 [inner, N] (negative rates), dt_bias and D
// [inner] in p_dt.  seg_len > 0: portions are cut into nseg segments of seg_len tokens that run side by side (scratch
// float32, aien_ssm_segments_scratch(T, S, seg_len, inner * N) numbers); nseg * seg_len must cover the longest portion;
// T is the number of tokens in the step.
AIEN_API int aien_selective_scan(const float* x, long ldx, const float* dtz, long lddt, const float* bc, long ldbc, int b_off, int c_off,
                                 const float* z, long ldz, const float* A, const void* dt_bias, const void* D, int p_dt,
                                 float* state, size_t state_stride, size_t s_off, const int* slots, const int* q_start,
                                 const int* positions, void* out, int o_dt, long ldo, int T, int S, int inner, int N,
                                 int seg_len, int nseg, float* scratch, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (inner <= 0 || N <= 0 || S > 65535 || nseg > 65535) return AIEN_E_SHAPE;
    Segments sg{0, 0, nullptr, nullptr, 1};
    if (seg_len > 0 && nseg > 1) {
        if (scratch == nullptr) return AIEN_E_SHAPE;
        sg = Segments{1, seg_len, scratch, scratch + (size_t)(T / seg_len + S) * (size_t)inner * N, nseg};
    }
    const ScanArgs a{x, ldx, dtz, lddt, bc, ldbc, b_off, c_off, z, ldz, A, dt_bias, D, p_dt, state, state_stride, s_off, slots, q_start,
                     positions, out, ldo, S, inner, N, sg, stream};
    int rc = 0;
    AIEN_DISPATCH_DTYPE(o_dt, TO, (rc = dispatch_selective_scan<TO>(a)));
    if (rc != 0) return rc;
    return launch_status();
}

struct SsdArgs {
    const float* xbc; long ld; int x_off, b_off, c_off; const float* dtr; long lddt; const float* A; const void* dt_bias; const void* D;
    int p_dt; float* state; size_t state_stride, s_off; const int* slots; const int* q_start; const int* positions; float* y; long ldy;
    int S, heads, V, G, N; Segments sg; cudaStream_t stream;
};

template <int NMAX>
static void launch_ssd_scan(const SsdArgs& a) {
    auto kern = ssd_scan_kernel<NMAX>;
    const unsigned gx = (unsigned)((a.heads * a.V + SSM_THREADS - 1) / SSM_THREADS);
    Segments sg = a.sg;
    const dim3 grid(gx, a.S, sg.mode == 0 ? 1 : sg.nseg);
    kern<<<grid, SSM_THREADS, 0, a.stream>>>(a.xbc, a.ld, a.x_off, a.b_off, a.c_off, a.dtr, a.lddt, a.A, a.dt_bias, a.D, a.p_dt, a.state,
                                             a.state_stride, a.s_off, a.slots, a.q_start, a.positions, a.y, a.ldy, a.heads, a.V, a.G, a.N, sg);
    if (sg.mode == 0) return;
    const size_t lanes = (size_t)a.heads * a.N * a.V;
    segment_combine_kernel<<<dim3((unsigned)((lanes + 255) / 256), a.S), 256, 0, a.stream>>>(a.state, a.state_stride, a.s_off, a.slots, a.q_start,
                                                                                             a.positions, sg, lanes);
    sg.mode = 2;
    kern<<<grid, SSM_THREADS, 0, a.stream>>>(a.xbc, a.ld, a.x_off, a.b_off, a.c_off, a.dtr, a.lddt, a.A, a.dt_bias, a.D, a.p_dt, a.state,
                                             a.state_stride, a.s_off, a.slots, a.q_start, a.positions, a.y, a.ldy, a.heads, a.V, a.G, a.N, sg);
}

// xbc [T, ld] (after convolution and silu): x (heads * V) at x_off, B (G * N) at b_off, C (G * N) at c_off; dtr [T, lddt]
// the raw step sizes, one per head; A float32 [heads] (positive rates exp(A_log)); dt_bias and D [heads] in p_dt;
// y float32 [T, ldy]; N <= 256.  Segments as for aien_selective_scan, with heads * N * V state values per request.
AIEN_API int aien_ssd_scan(const float* xbc, long ld, int x_off, int b_off, int c_off, const float* dtr, long lddt, const float* A,
                           const void* dt_bias, const void* D, int p_dt, float* state, size_t state_stride, size_t s_off,
                           const int* slots, const int* q_start, const int* positions, float* y, long ldy, int T, int S, int heads, int V,
                           int G, int N, int seg_len, int nseg, float* scratch, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (heads <= 0 || V <= 0 || G <= 0 || heads % G || N <= 0 || S > 65535 || nseg > 65535) return AIEN_E_SHAPE;
    Segments sg{0, 0, nullptr, nullptr, 1};
    if (seg_len > 0 && nseg > 1) {
        if (scratch == nullptr) return AIEN_E_SHAPE;
        sg = Segments{1, seg_len, scratch, scratch + (size_t)(T / seg_len + S) * (size_t)heads * N * V, nseg};
    }
    const SsdArgs a{xbc, ld, x_off, b_off, c_off, dtr, lddt, A, dt_bias, D, p_dt, state, state_stride, s_off, slots, q_start, positions,
                    y, ldy, S, heads, V, G, N, sg, stream};
    switch (pick_nmax(N)) {
        case 16: launch_ssd_scan<16>(a); break;
        case 32: launch_ssd_scan<32>(a); break;
        case 64: launch_ssd_scan<64>(a); break;
        case 128: launch_ssd_scan<128>(a); break;
        case 256: launch_ssd_scan<256>(a); break;
        default: return AIEN_E_SHAPE;
    }
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
