// The gated delta rule: per value head a float32 state S [D][V] that every token first decays, then corrects along
// its key, then reads with its query:
//     S <- g S ;   u = beta (v - S^T k) ;   S <- S + k u^T ;   o = S^T q
// (g a decay in (0, 1], beta in (0, 1), k a unit vector; heads/G value heads share one q/k head).  Column j of S
// never meets another column: S^T k, u, the update and S^T q are all per column.  So a thread owns part of one column
// in registers and a portion is walked token by token with no barrier inside a chunk of tokens: a warp holds 8
// columns x 4 row ranges (the four partial dot products meet through two shuffles), a CTA 32 columns of one head of
// one request.  q, k, v, g and beta of the next chunk of tokens arrive through cp.async while the current one is
// walked.  Every operation is float32 and runs in the order written above, so a token's output depends on the
// tokens before it only through S, whatever the cut of the prompt or the batch.
//
// The state lives in the request's slot between steps (a portion whose first token has position 0 starts from zero).
//
// grouped_gated_rmsnorm: out = o / sqrt(mean_group(o^2) + eps) * w[c mod group] * act(gate), the norm taken over
// every group of `group` neighbouring columns (one head) with one weight vector shared by the groups.
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int DR_THREADS = 128;
constexpr int DR_COLS = 32;         // columns of S per CTA

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int DPT>
struct DeltaCfg {
    static constexpr int DP = 4 * DPT;                         // rows of S, padded
    static constexpr int TC = DPT <= 32 ? 16 : 8;              // tokens per chunk
    static constexpr int ROW = 2 * DP + DR_COLS + 4;           // floats per token: k | q | v | g, beta, -, -
};

template <int DPT>
__device__ __forceinline__ void delta_fetch(float* __restrict__ buf, const float* __restrict__ qkv, long ld, int q_col, int k_col,
                                            int v_col, const float* __restrict__ gb, long ldgb, int h, int heads, int t, int t1,
                                            int D, int V, int col0) {
    using C = DeltaCfg<DPT>;
    for (int idx = threadIdx.x; idx < C::TC * C::ROW; idx += DR_THREADS) {
        const int tok = idx / C::ROW, e = idx - tok * C::ROW;
        const int tt = t + tok;
        float* dst = buf + idx;
        const float* src = nullptr;
        if (tt < t1) {
            if (e < C::DP) { if (e < D) src = qkv + (size_t)tt * ld + k_col + e; }
            else if (e < 2 * C::DP) { if (e - C::DP < D) src = qkv + (size_t)tt * ld + q_col + (e - C::DP); }
            else if (e < 2 * C::DP + DR_COLS) { if (col0 + (e - 2 * C::DP) < V) src = qkv + (size_t)tt * ld + v_col + col0 + (e - 2 * C::DP); }
            else if (e == 2 * C::DP + DR_COLS) src = gb + (size_t)tt * ldgb + h;
            else if (e == 2 * C::DP + DR_COLS + 1) src = gb + (size_t)tt * ldgb + heads + h;
        }
        if (src != nullptr) cp_async4(dst, src);
        else *dst = 0.f;
    }
    cp_async_commit();
}

template <int DPT>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ qkv, long ld, int q_off, int k_off, int v_off, const float* __restrict__ gb, long ldgb,
                  float* __restrict__ state, size_t state_stride, size_t s_off, const int* __restrict__ slot_map,
                  const int* __restrict__ q_start, const int* __restrict__ positions, float* __restrict__ o, long ldo,
                  int heads, int G, int D, int V) {
    using C = DeltaCfg<DPT>;
    __shared__ __align__(16) float bufs[2][C::TC * C::ROW];
    const int s = blockIdx.z, h = blockIdx.y, kvh = h / (heads / G);
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (t1 <= t0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rs = lane >> 3, cw = lane & 7;
    const int col0 = blockIdx.x * DR_COLS, cl = warp * 8 + cw, col = col0 + cl;
    const bool col_ok = col < V;
    const int i0 = rs * DPT;
    float* S = state + (size_t)slot_map[s] * state_stride + s_off + (size_t)h * D * V;
    const int q_col = q_off + kvh * D, k_col = k_off + kvh * D, v_col = v_off + h * V;

    delta_fetch<DPT>(bufs[0], qkv, ld, q_col, k_col, v_col, gb, ldgb, h, heads, t0, t1, D, V, col0);
    float Sr[DPT];
    const bool fresh = positions[t0] == 0;
#pragma unroll
    for (int i = 0; i < DPT; ++i) Sr[i] = (!fresh && col_ok && i0 + i < D) ? S[(size_t)(i0 + i) * V + col] : 0.f;

    int b = 0;
    for (int t = t0; t < t1; t += C::TC, b ^= 1) {
        cp_async_wait_all();
        __syncthreads();                                        // chunk b has arrived; everyone is done with chunk b^1
        if (t + C::TC < t1) delta_fetch<DPT>(bufs[b ^ 1], qkv, ld, q_col, k_col, v_col, gb, ldgb, h, heads, t + C::TC, t1, D, V, col0);
        const int n = t1 - t < C::TC ? t1 - t : C::TC;
        for (int tt = 0; tt < n; ++tt) {
            const float* row = bufs[b] + tt * C::ROW;
            const float4* kk = reinterpret_cast<const float4*>(row + i0);
            const float4* qq = reinterpret_cast<const float4*>(row + C::DP + i0);
            const float vj = row[2 * C::DP + cl];
            const float g = row[2 * C::DP + DR_COLS], beta = row[2 * C::DP + DR_COLS + 1];
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                const float4 k4 = kk[i];
                Sr[4 * i + 0] *= g; a0 = fmaf(Sr[4 * i + 0], k4.x, a0);
                Sr[4 * i + 1] *= g; a1 = fmaf(Sr[4 * i + 1], k4.y, a1);
                Sr[4 * i + 2] *= g; a2 = fmaf(Sr[4 * i + 2], k4.z, a2);
                Sr[4 * i + 3] *= g; a3 = fmaf(Sr[4 * i + 3], k4.w, a3);
            }
            float sk = (a0 + a1) + (a2 + a3);
            sk += __shfl_xor_sync(0xffffffffu, sk, 8);
            sk += __shfl_xor_sync(0xffffffffu, sk, 16);
            const float u = beta * (vj - sk);
            a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                const float4 k4 = kk[i], q4 = qq[i];
                Sr[4 * i + 0] = fmaf(k4.x, u, Sr[4 * i + 0]); a0 = fmaf(Sr[4 * i + 0], q4.x, a0);
                Sr[4 * i + 1] = fmaf(k4.y, u, Sr[4 * i + 1]); a1 = fmaf(Sr[4 * i + 1], q4.y, a1);
                Sr[4 * i + 2] = fmaf(k4.z, u, Sr[4 * i + 2]); a2 = fmaf(Sr[4 * i + 2], q4.z, a2);
                Sr[4 * i + 3] = fmaf(k4.w, u, Sr[4 * i + 3]); a3 = fmaf(Sr[4 * i + 3], q4.w, a3);
            }
            float oj = (a0 + a1) + (a2 + a3);
            oj += __shfl_xor_sync(0xffffffffu, oj, 8);
            oj += __shfl_xor_sync(0xffffffffu, oj, 16);
            if (rs == 0 && col_ok) o[(size_t)(t + tt) * ldo + (size_t)h * V + col] = oj;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < DPT; ++i)
            if (i0 + i < D) S[(size_t)(i0 + i) * V + col] = Sr[i];
    }
}

__device__ __forceinline__ float gate_act(float z, int kind) {
    const float sg = 1.0f / (1.0f + expf(-z));
    return kind == 1 ? z * sg : sg;
}

// one warp per (token, group)
template <typename TP, typename TO>
__global__ void __launch_bounds__(256)
grouped_gated_rmsnorm_kernel(const float* __restrict__ o, long ldo, const TP* __restrict__ gate, long ldg, const void* __restrict__ w,
                             int wdt, float eps, TO* __restrict__ out, long ldout, int T, int groups, int group, int act) {
    const size_t unit = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (size_t)T * groups) return;
    const int lane = threadIdx.x & 31;
    const size_t t = unit / groups;
    const int g = (int)(unit - t * groups);
    const float* row = o + t * ldo + (size_t)g * group;
    float ss = 0.f;
    for (int d = lane; d < group; d += 32) { const float v = ld_act(row + d); ss = fmaf(v, v, ss); }
    const float scale = 1.0f / sqrtf(warp_sum(ss) / (float)group + eps);
    for (int d = lane; d < group; d += 32) {
        const float z = ld_act(gate + t * ldg + (size_t)g * group + d);
        out[t * ldout + (size_t)g * group + d] = from_f<TO>(ld_act(row + d) * scale * load_dyn(w, wdt, d) * gate_act(z, act));
    }
}

}  // namespace aien

using namespace aien;

template <int DPT>
static void launch_delta_rule(dim3 grid, cudaStream_t stream, const float* qkv, long ld, int q_off, int k_off, int v_off, const float* gb,
                              long ldgb, float* state, size_t state_stride, size_t s_off, const int* slot_map, const int* q_start,
                              const int* positions, float* o, long ldo, int heads, int G, int D, int V) {
    delta_rule_kernel<DPT><<<grid, DR_THREADS, 0, stream>>>(qkv, ld, q_off, k_off, v_off, gb, ldgb, state, state_stride, s_off, slot_map,
                                                            q_start, positions, o, ldo, heads, G, D, V);
}

// qkv float32 [T, ld]: prepared q (G*D) at q_off, k (G*D) at k_off, v (heads*V) at v_off; gb float32 [T, ldgb]: decay
// of head h at column h, beta at heads + h.  state: float32 rows of state_stride numbers per slot, S [heads][D][V] at
// s_off.  Request s of the step (tokens q_start[s] .. q_start[s+1]) continues from slot slot_map[s].  o float32 [T, ldo].
AIEN_API int aien_delta_rule(const float* qkv, long ld, int q_off, int k_off, int v_off, const float* gb, long ldgb, float* state,
                             size_t state_stride, size_t s_off, const int* slot_map, const int* q_start, const int* positions,
                             float* o, long ldo, int S, int heads, int G, int D, int V, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (heads <= 0 || G <= 0 || heads % G || D <= 0 || D > 256 || V <= 0 || S > 65535 || heads > 65535) return AIEN_E_SHAPE;
    dim3 grid((V + DR_COLS - 1) / DR_COLS, heads, S);
    const int dpt = (D + 3) / 4;
#define DR_CASE(N) launch_delta_rule<N>(grid, stream, qkv, ld, q_off, k_off, v_off, gb, ldgb, state, state_stride, s_off, slot_map, q_start, positions, o, ldo, heads, G, D, V)
    if (dpt <= 4) DR_CASE(4);
    else if (dpt <= 8) DR_CASE(8);
    else if (dpt <= 16) DR_CASE(16);
    else if (dpt <= 24) DR_CASE(24);
    else if (dpt <= 32) DR_CASE(32);
    else if (dpt <= 48) DR_CASE(48);
    else DR_CASE(64);
#undef DR_CASE
    return launch_status();
}

// o float32 [T, groups*group]; gate [T, *] in g_dt; w [group]; act 0: sigmoid(gate), 1: silu(gate).
AIEN_API int aien_grouped_gated_rmsnorm(const float* o, long ldo, const void* gate, int g_dt, long ldg, const void* w, int w_dt, float eps,
                                        void* out, int o_dt, long ldout, int T, int groups, int group, int act, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (groups <= 0 || group <= 0) return AIEN_E_SHAPE;
    const size_t units = (size_t)T * groups;
    const unsigned blocks = (unsigned)((units + 7) / 8);
    AIEN_DISPATCH_DTYPE(g_dt, TP, AIEN_DISPATCH_DTYPE(o_dt, TO,
        (grouped_gated_rmsnorm_kernel<TP, TO><<<blocks, 256, 0, stream>>>(o, ldo, (const TP*)gate, ldg, w, w_dt, eps, (TO*)out, ldout, T,
                                                                         groups, group, act))));
    return launch_status();
}
