// The gated delta rule: per value head a float32 state S [D][V] that every token first decays, then corrects along
// its key, then reads with its query:
//     S <- g S ;   u = beta (v - S^T k) ;   S <- S + k u^T ;   o = S^T q
// (g a decay in (0, 1], beta in (0, 1), k a unit vector; heads/G value heads share one q/k head).  Column j of S
// never meets another column: S^T k, u, the update and S^T q are all per column.  So a thread owns part of one column
// in registers and a portion is walked token by token with no barrier inside a chunk of tokens.  Both products are
// taken from the state as the token finds it, in one pass over the registers:
//     a = S^T k ,  b = S^T q ,  c = k . q ;   u = beta (v - g a) ;   o = g b + c u ;   S <- g S + k u^T
// which is the same arithmetic with the decay drawn out of the sums.  A warp holds 32/RS columns x RS row ranges (the
// partial sums meet through log2(RS) shuffles), a CTA four warps' columns of one head of one request.  What the
// walk is bound by is the reading of k and q from shared memory, once per token and thread: the row ranges lie
// DPT + 4 floats apart there, so that the 16-byte reads of a warp fall into different banks.  q, k, v, g and beta of
// the next chunk of tokens arrive through cp.async while the current one is walked, and the next token's are taken
// into registers while the current one's sums are on their way.  Every operation is float32 and a token's are the
// same whatever the cut of the prompt or the batch, so its output depends on the tokens before it only through S.
//
// The state lives in the request's slot between steps (a portion whose first token has position 0 starts from zero).
//
// grouped_gated_rmsnorm: out = o / sqrt(mean_group(o^2) + eps) * w[c mod group] * act(gate), the norm taken over
// every group of `group` neighbouring columns (one head) with one weight vector shared by the groups.
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int DR_THREADS = 128;

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int DPT, int RS>
struct DeltaCfg {
    static constexpr int DP = RS * DPT;                        // rows of S, padded
    static constexpr int PS = DPT == 4 ? 4 : DPT + 4;          // floats between two row ranges of k (or q) in shared memory
    static constexpr int CW = 32 / RS;                         // columns per warp
    static constexpr int COLS = (DR_THREADS / 32) * CW;        // columns of S per CTA
    static constexpr int KQ = RS * PS;                         // floats of k (or q) per token, padded
    static constexpr int ROW = 2 * KQ + COLS + 4;              // floats per token: k | q | v | g, beta, -, -
    static constexpr int TC = 2 * 16 * ROW * 4 <= 48 * 1024 ? 16 : 8;   // tokens per chunk: two chunks within 48 KB
};

// What one thread copies for every token of a chunk: up to NE pieces, found once per kernel (where in the token's
// row of the source, where in its row of shared memory, 16 bytes or 4), so that a chunk's copies are an address
// and a cp.async each.  The walk shares its warps with the copies, so their instructions count.
template <int DPT, int RS>
struct DeltaPieces {
    using C = DeltaCfg<DPT, RS>;
    static constexpr int NE = (2 * C::DP + C::COLS + 2 + DR_THREADS - 1) / DR_THREADS;
    const float* src[NE];
    long stride[NE];
    int dst[NE];
    int kind[NE];                                              // 0: none, 1: 4 bytes, 2: 16 bytes; +4: always zero

    __device__ __forceinline__ void find(bool vec, const float* qkv, long ld, int q_col, int k_col, int v_col, const float* gb,
                                         long ldgb, int h, int heads, int D, int V, int col0) {
        const int unit = vec ? 4 : 1;
        const int n_kq = C::DP / unit, n_v = C::COLS / unit;
#pragma unroll
        for (int i = 0; i < NE; ++i) {
            const int e = threadIdx.x + i * DR_THREADS;
            src[i] = qkv; stride[i] = ld; dst[i] = 0; kind[i] = 0;
            if (e < 2 * n_kq) {
                const int which = e >= n_kq, r = (e - which * n_kq) * unit;        // 0: k, 1: q; row r
                dst[i] = which * C::KQ + (r / DPT) * C::PS + (r % DPT);
                src[i] = qkv + (which ? q_col : k_col) + r;
                kind[i] = (vec ? 2 : 1) + (r < D ? 0 : 4);
            } else if (e < 2 * n_kq + n_v) {
                const int c = (e - 2 * n_kq) * unit;
                dst[i] = 2 * C::KQ + c;
                src[i] = qkv + v_col + col0 + c;
                kind[i] = (vec ? 2 : 1) + (col0 + c < V ? 0 : 4);
            } else if (e < 2 * n_kq + n_v + 2) {
                const int w = e - 2 * n_kq - n_v;                                   // 0: decay, 1: beta
                dst[i] = 2 * C::KQ + C::COLS + w;
                src[i] = gb + w * heads + h;
                stride[i] = ldgb;
                kind[i] = 1;
            }
        }
    }

    __device__ __forceinline__ void fetch(float* __restrict__ buf, int t, int t1) const {
#pragma unroll 4
        for (int tok = 0; tok < C::TC; ++tok) {
            const int tt = t + tok;
#pragma unroll
            for (int i = 0; i < NE; ++i) {
                if (kind[i] == 0) continue;
                float* d = buf + tok * C::ROW + dst[i];
                const bool wide = (kind[i] & 2) != 0;
                if (tt < t1 && kind[i] < 4) {
                    const float* sp = src[i] + (size_t)tt * stride[i];
                    if (wide) cp_async16(d, sp);
                    else cp_async4(d, sp);
                } else if (wide) {
                    *reinterpret_cast<float4*>(d) = make_float4(0.f, 0.f, 0.f, 0.f);
                } else {
                    *d = 0.f;
                }
            }
        }
        cp_async_commit();
    }
};

template <int DPT, int RS>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ qkv, long ld, int q_off, int k_off, int v_off, const float* __restrict__ gb, long ldgb,
                  float* __restrict__ state, size_t state_stride, size_t s_off, const int* __restrict__ slot_map,
                  const int* __restrict__ q_start, const int* __restrict__ positions, float* __restrict__ o, long ldo,
                  int heads, int G, int D, int V) {
    using C = DeltaCfg<DPT, RS>;
    constexpr int N4 = DPT / 4;
    __shared__ __align__(16) float bufs[2][C::TC * C::ROW];
    const int s = blockIdx.z, h = blockIdx.y, kvh = h / (heads / G);
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (t1 <= t0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rs = lane / C::CW, cw = lane % C::CW;
    const int col0 = blockIdx.x * C::COLS, cl = warp * C::CW + cw, col = col0 + cl;
    const bool col_ok = col < V;
    const int i0 = rs * DPT;
    float* S = state + (size_t)slot_map[s] * state_stride + s_off + (size_t)h * D * V;
    const int q_col = q_off + kvh * D, k_col = k_off + kvh * D, v_col = v_off + h * V;

    // 16-byte copies where every piece of four neighbours starts on a 16-byte boundary and lies inside or outside whole
    const bool vec = ((reinterpret_cast<uintptr_t>(qkv) & 15) == 0) && ((ld | q_col | k_col | v_col | D | V) & 3) == 0;
    DeltaPieces<DPT, RS> pieces;
    pieces.find(vec, qkv, ld, q_col, k_col, v_col, gb, ldgb, h, heads, D, V, col0);
    pieces.fetch(bufs[0], t0, t1);
    // the thread's rows of its column, two to a register pair: the sums and the update run on packed pairs
    // (fma.rn.f32x2, each half rounded as the single operation is), which halves the instructions of the walk
    float2 Sr[2 * N4];
    const bool fresh = positions[t0] == 0;
#pragma unroll
    for (int i = 0; i < 2 * N4; ++i) {
        Sr[i].x = (!fresh && col_ok && i0 + 2 * i < D) ? S[(size_t)(i0 + 2 * i) * V + col] : 0.f;
        Sr[i].y = (!fresh && col_ok && i0 + 2 * i + 1 < D) ? S[(size_t)(i0 + 2 * i + 1) * V + col] : 0.f;
    }

    float4 kc[N4], qc[N4];
    float vj, g, beta;
    auto take = [&](const float* row) {                        // one token's numbers into registers
        const float4* kk = reinterpret_cast<const float4*>(row + rs * C::PS);
        const float4* qq = reinterpret_cast<const float4*>(row + C::KQ + rs * C::PS);
#pragma unroll
        for (int i = 0; i < N4; ++i) { kc[i] = kk[i]; qc[i] = qq[i]; }
        vj = row[2 * C::KQ + cl];
        g = row[2 * C::KQ + C::COLS];
        beta = row[2 * C::KQ + C::COLS + 1];
    };

    int b = 0;
    for (int t = t0; t < t1; t += C::TC, b ^= 1) {
        cp_async_wait_all();
        __syncthreads();                                        // chunk b has arrived; everyone is done with chunk b^1
        if (t + C::TC < t1) pieces.fetch(bufs[b ^ 1], t + C::TC, t1);
        const int n = t1 - t < C::TC ? t1 - t : C::TC;
        take(bufs[b]);
        for (int tt = 0; tt < n; ++tt) {
            float2 a0 = make_float2(0.f, 0.f), a1 = a0, b0 = a0, b1 = a0, c0 = a0, c1 = a0;
#pragma unroll
            for (int i = 0; i < N4; ++i) {
                const float2 k0 = make_float2(kc[i].x, kc[i].y), k1 = make_float2(kc[i].z, kc[i].w);
                const float2 q0 = make_float2(qc[i].x, qc[i].y), q1 = make_float2(qc[i].z, qc[i].w);
                a0 = __ffma2_rn(Sr[2 * i], k0, a0); a1 = __ffma2_rn(Sr[2 * i + 1], k1, a1);
                b0 = __ffma2_rn(Sr[2 * i], q0, b0); b1 = __ffma2_rn(Sr[2 * i + 1], q1, b1);
                c0 = __ffma2_rn(k0, q0, c0); c1 = __ffma2_rn(k1, q1, c1);
            }
            float sa = (a0.x + a0.y) + (a1.x + a1.y), sb = (b0.x + b0.y) + (b1.x + b1.y), sc = (c0.x + c0.y) + (c1.x + c1.y);
#pragma unroll
            for (int off = C::CW; off < 32; off <<= 1) {
                sa += __shfl_xor_sync(0xffffffffu, sa, off);
                sb += __shfl_xor_sync(0xffffffffu, sb, off);
                sc += __shfl_xor_sync(0xffffffffu, sc, off);
            }
            const float gg = g;
            const float u = beta * (vj - gg * sa);
            const float oj = fmaf(sc, u, gg * sb);
            const float2 g2 = make_float2(gg, gg), u2 = make_float2(u, u);
#pragma unroll
            for (int i = 0; i < N4; ++i) {
                Sr[2 * i] = __ffma2_rn(make_float2(kc[i].x, kc[i].y), u2, __fmul2_rn(g2, Sr[2 * i]));
                Sr[2 * i + 1] = __ffma2_rn(make_float2(kc[i].z, kc[i].w), u2, __fmul2_rn(g2, Sr[2 * i + 1]));
            }
            if (tt + 1 < n) take(bufs[b] + (tt + 1) * C::ROW);  // the next token's, while this one's output leaves
            if (rs == 0 && col_ok) o[(size_t)(t + tt) * ldo + (size_t)h * V + col] = oj;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < 2 * N4; ++i) {
            if (i0 + 2 * i < D) S[(size_t)(i0 + 2 * i) * V + col] = Sr[i].x;
            if (i0 + 2 * i + 1 < D) S[(size_t)(i0 + 2 * i + 1) * V + col] = Sr[i].y;
        }
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

template <int DPT, int RS>
static void launch_delta_rule(cudaStream_t stream, const float* qkv, long ld, int q_off, int k_off, int v_off, const float* gb,
                              long ldgb, float* state, size_t state_stride, size_t s_off, const int* slot_map, const int* q_start,
                              const int* positions, float* o, long ldo, int S, int heads, int G, int D, int V) {
    constexpr int COLS = DeltaCfg<DPT, RS>::COLS;
    dim3 grid((V + COLS - 1) / COLS, heads, S);
    delta_rule_kernel<DPT, RS><<<grid, DR_THREADS, 0, stream>>>(qkv, ld, q_off, k_off, v_off, gb, ldgb, state, state_stride, s_off,
                                                                slot_map, q_start, positions, o, ldo, heads, G, D, V);
}

// qkv float32 [T, ld]: prepared q (G*D) at q_off, k (G*D) at k_off, v (heads*V) at v_off; gb float32 [T, ldgb]: decay
// of head h at column h, beta at heads + h.  state: float32 rows of state_stride numbers per slot, S [heads][D][V] at
// s_off.  Request s of the step (tokens q_start[s] .. q_start[s+1]) continues from slot slot_map[s].  o float32 [T, ldo].
AIEN_API int aien_delta_rule(const float* qkv, long ld, int q_off, int k_off, int v_off, const float* gb, long ldgb, float* state,
                             size_t state_stride, size_t s_off, const int* slot_map, const int* q_start, const int* positions,
                             float* o, long ldo, int S, int heads, int G, int D, int V, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (heads <= 0 || G <= 0 || heads % G || D <= 0 || D > 256 || V <= 0 || S > 65535 || heads > 65535) return AIEN_E_SHAPE;
#define DR_CASE(N, R) launch_delta_rule<N, R>(stream, qkv, ld, q_off, k_off, v_off, gb, ldgb, state, state_stride, s_off, slot_map, q_start, positions, o, ldo, S, heads, G, D, V)
    if (D <= 16) DR_CASE(4, 4);
    else if (D <= 32) DR_CASE(8, 4);
    else if (D <= 64) DR_CASE(8, 8);
    else if (D <= 96) DR_CASE(12, 8);
    else if (D <= 128) DR_CASE(16, 8);
    else if (D <= 192) DR_CASE(24, 8);
    else DR_CASE(32, 8);
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
