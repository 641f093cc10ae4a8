// Routed feed-forward: the router's choice, the rows sorted by expert for the grouped tensor-core
// products (gemm_tc.cu), the experts' products of a few tokens, and the plain expert products.
//
//   route        scores s = softmax(z) over all E experts (float32); experts lie in `groups` equal
//                groups of neighbours, a group scores its best expert, only the `keep` best groups
//                stay eligible; the `top` best eligible experts are taken, weight = their score
//                (divided by the sum of the taken scores when `renorm` is set).  Ties go to the lower
//                index.  One warp per token.  On request it also counts the choices per expert.
//   plan_rows, place_rows   every expert's (token, choice) pairs in a run of rows of their own (see below)
//   expert_rows_bf16        up and down products of a few tokens, bfloat16, a warp per four output rows
//   expert_up    act[t, c, :] = f(W_up[e(t,c)] h[t])             c < top, f = gelu (erf or tanh form)
//   expert_down  part[c][t, :] = weight(t,c) * W_down[e(t,c)] act[t, c, :]   float32 parts, one per choice,
//                which the consumer (the norm that takes the branch) adds in index order
//   act_rows     f applied in place to [T, F] rows (the shared expert's hidden layer)
//
// expert_up / expert_down are one warp per output value with the reduction in a fixed lane order, so a
// token's result depends on its own row alone; they serve the 32-bit engine and sizes the others do not
// take, and are what the faster products are held to.
#include "common.cuh"
#include <math.h>

namespace aien {

// kind 0: gelu (erf form), 1: gelu (tanh form), 2: the square of relu
__device__ __forceinline__ float act_apply(float z, int kind) {
    if (kind == 2) { const float r = fmaxf(z, 0.f); return r * r; }
    if (kind == 1) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
}

// ---------------------------------------------------------------- router
constexpr int ROUTE_MAX_EXPERTS = 1024;

__global__ void __launch_bounds__(32)
moe_route_kernel(const float* __restrict__ z, int E, int groups, int keep, int top, int renorm,
                 int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ expert_count) {
    __shared__ float s[ROUTE_MAX_EXPERTS];
    __shared__ float gs[ROUTE_MAX_EXPERTS];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* zr = z + (size_t)t * E;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) { const float v = __ldcg(zr + e); s[e] = v; m = fmaxf(m, v); }
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = expf(s[e] - m); s[e] = v; sum += v; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) s[e] *= inv;
    __syncwarp();
    const int per = E / groups;
    if (groups > 1 && keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int j = 0; j < per; ++j) best = fmaxf(best, s[g * per + j]);
            gs[g] = best;
        }
        __syncwarp();
        // every group starts ineligible (score negated below zero); the `keep` best are restored
        for (int r = 0; r < keep; ++r) {
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) if (gs[g] > bv) { bv = gs[g]; bi = g; }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) gs[bi] = -1.0f;                 // marks a kept group (scores are >= 0)
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) if (gs[e / per] != -1.0f) s[e] = -1.0f;      // not eligible
        __syncwarp();
    }
    float wsum = 0.f;
    for (int r = 0; r < top; ++r) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) if (s[e] > bv) { bv = s[e]; bi = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            ids[(size_t)t * top + r] = bi;
            wts[(size_t)t * top + r] = bv;
            s[bi] = -2.0f;                                 // taken
            if (expert_count != nullptr) atomicAdd(expert_count + bi, 1);     // for the plan of the grouped products
        }
        wsum += bv;
        __syncwarp();
    }
    if (renorm && lane == 0) {
        for (int r = 0; r < top; ++r) wts[(size_t)t * top + r] /= wsum;
    }
}

// The router with a correction on the choice and experts that return their input.  s = softmax(z[t][0..E)) (rows ldz
// apart); the `top` experts with the largest s + correction are chosen (ties to the lower index); a choice weighs s,
// divided by the sum of the chosen s plus renorm_eps when `renorm` is set.  Experts from `real` on have no tensors:
// their output is their input, so their weights are summed into w_same[t] and the choice is handed on as expert 0
// with weight zero (the expert products need no case for it).  One warp per token.
__global__ void __launch_bounds__(32)
moe_route_biased_kernel(const float* __restrict__ z, long ldz, int E, int real, int top, int renorm, float renorm_eps,
                        const void* __restrict__ correction, int cdt, int* __restrict__ ids, float* __restrict__ wts,
                        float* __restrict__ w_same, int* __restrict__ expert_count) {
    __shared__ float s[ROUTE_MAX_EXPERTS];
    __shared__ float ch[ROUTE_MAX_EXPERTS];
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* zr = z + (size_t)t * ldz;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) { const float v = zr[e]; s[e] = v; m = fmaxf(m, v); }
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = expf(s[e] - m); s[e] = v; sum += v; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) {
        s[e] *= inv;
        ch[e] = correction != nullptr ? s[e] + load_dyn(correction, cdt, e) : s[e];
    }
    __syncwarp();
    float wsum = 0.f;
    for (int r = 0; r < top; ++r) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) if (ch[e] > bv) { bv = ch[e]; bi = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        const float w = s[bi];
        wsum += w;
        __syncwarp();
        if (lane == 0) {
            ids[(size_t)t * top + r] = bi;
            wts[(size_t)t * top + r] = w;
            ch[bi] = -INFINITY;                            // taken
        }
        __syncwarp();
    }
    if (lane == 0) {
        const float div = renorm ? wsum + renorm_eps : 1.0f;
        float same = 0.f;
        for (int r = 0; r < top; ++r) {
            const size_t at = (size_t)t * top + r;
            const float w = wts[at] / div;
            int e = ids[at];
            if (e >= real) { same += w; e = 0; wts[at] = 0.f; } else wts[at] = w;
            ids[at] = e;
            if (expert_count != nullptr) atomicAdd(expert_count + e, 1);
        }
        if (w_same != nullptr) w_same[t] = same;
    }
}

// ---------------------------------------------------------------- plain expert products
// One warp per output value; 8 warps a CTA take 8 consecutive output rows of one (token, choice).
template <typename TH, typename TW, typename TO>
__global__ void __launch_bounds__(256)
moe_expert_up_kernel(const TH* __restrict__ h, long h_stride, const TW* __restrict__ w_up, const int* __restrict__ ids,
                     TO* __restrict__ act, int top, int D, int F, int act_kind) {
    griddep_launch();
    griddep_wait();
    const int pair = blockIdx.x;                       // t * top + c
    const int t = pair / top;
    const int f = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (f >= F) return;
    const int e = __ldcg(ids + pair);
    const TW* wr = w_up + ((size_t)e * F + f) * D;
    const TH* hr = h + (size_t)t * h_stride;
    float acc = 0.f;
    for (int i = lane; i < D; i += 32) acc = fmaf(to_f(wr[i]), ld_act(hr + i), acc);
    acc = warp_sum(acc);
    if (lane == 0) act[(size_t)pair * F + f] = from_f<TO>(act_apply(acc, act_kind));
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
moe_expert_down_kernel(const TA* __restrict__ act, const TW* __restrict__ w_down, const int* __restrict__ ids,
                       const float* __restrict__ wts, float* __restrict__ parts, int T, int top, int D, int F) {
    griddep_launch();
    griddep_wait();
    const int pair = blockIdx.x;
    const int t = pair / top, c = pair - t * top;
    const int n = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= D) return;
    const int e = __ldcg(ids + pair);
    const TW* wr = w_down + ((size_t)e * D + n) * F;
    const TA* ar = act + (size_t)pair * F;
    float acc = 0.f;
    for (int i = lane; i < F; i += 32) acc = fmaf(to_f(wr[i]), ld_act(ar + i), acc);
    acc = warp_sum(acc);
    if (lane == 0) parts[((size_t)c * T + t) * D + n] = acc * __ldcg(wts + pair);
}

// ---------------------------------------------------------------- rows sorted by expert, for the grouped product
// Pair p = t * top + c chose expert ids[p].  Every expert's pairs get a run of rows that starts at a multiple of 128
// (the row tile of the grouped tensor-core product); the runs follow one another in expert order.
//   tile_group[i] = expert of row tile i (-1 beyond the last run, whose rows are not written at all);
//   row_dest[r] = c * T + t, the row of the [top, T, D] parts that the pair in row r belongs to (-1: padding);
//   row_scale[r] = the pair's weight;  a_sorted[r, :] = the pair's token's row of h.
// Which row of its run a pair gets depends on the order the threads arrive in; no result depends on it, since a row
// of a product depends on that row alone.
constexpr int SORT_THREADS = 1024;

// Two launches.  The router's choice has counted the pairs of every expert (expert_count).  moe_plan_rows (one CTA): the first row of every expert's run, a cursor
// into it, the experts of the row tiles, -1 as the destination of the padding rows; the counts are zeroed for the
// next step.  moe_place_rows (64 threads a pair): the pair takes the next row of its expert's run and its token's
// row of h is copied there, with the pair's destination and weight.  Padding rows of a_sorted are left as they are:
// a row of a product depends on that row alone, and their results are never stored.
__global__ void __launch_bounds__(SORT_THREADS)
moe_plan_rows_kernel(int* __restrict__ expert_count, int E, int max_tiles, int* __restrict__ cursor, int* __restrict__ tile_group,
                     int* __restrict__ row_dest) {
    __shared__ int count[ROUTE_MAX_EXPERTS];
    __shared__ int start[ROUTE_MAX_EXPERTS];
    __shared__ int used_rows;
    griddep_launch();
    griddep_wait();
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += SORT_THREADS) { count[e] = __ldcg(expert_count + e); expert_count[e] = 0; }
    __syncthreads();
    if (tid == 0) {
        int row = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = row;
            row += (count[e] + 127) & ~127;
        }
        used_rows = row;
    }
    __syncthreads();
    for (int e = tid; e < E; e += SORT_THREADS) cursor[e] = start[e];
    for (int i = (used_rows >> 7) + tid; i < max_tiles; i += SORT_THREADS) tile_group[i] = -1;
    for (int e = tid; e < E; e += SORT_THREADS) {
        const int first = start[e] >> 7, n = (count[e] + 127) >> 7;
        for (int i = 0; i < n; ++i) tile_group[first + i] = e;
    }
    for (int e = tid >> 7; e < E; e += SORT_THREADS >> 7) {
        const int r = start[e] + count[e] + (tid & 127);
        if (r < start[e] + ((count[e] + 127) & ~127)) row_dest[r] = -1;
    }
}

__global__ void __launch_bounds__(256)
moe_place_rows_kernel(const __nv_bfloat16* __restrict__ h, long h_stride, const int* __restrict__ ids, const float* __restrict__ wts,
                      int* __restrict__ cursor, int P, int T, int top, __nv_bfloat16* __restrict__ a_sorted, int D,
                      int* __restrict__ row_dest, float* __restrict__ row_scale) {
    __shared__ int rows[4];
    griddep_launch();
    griddep_wait();
    const int sub = threadIdx.x >> 6, lane = threadIdx.x & 63;
    const int p = blockIdx.x * 4 + sub;
    if (p < P && lane == 0) {
        const int r = atomicAdd(cursor + __ldcg(ids + p), 1);
        const int t = p / top, c = p - t * top;
        row_dest[r] = c * T + t;
        row_scale[r] = __ldcg(wts + p);
        rows[sub] = r;
    }
    __syncthreads();
    if (p >= P) return;
    const int r = rows[sub];
    const int vec = D >> 3;
    const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(p / top) * h_stride);
    uint4* dst = reinterpret_cast<uint4*>(a_sorted + (size_t)r * D);
    for (int v0 = lane; v0 < vec; v0 += 256) {
        uint4 val[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int v = v0 + 64 * j;
            val[j] = v < vec ? __ldcg(src + v) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int v = v0 + 64 * j;
            if (v < vec) dst[v] = val[j];
        }
    }
}

// ---------------------------------------------------------------- expert products of a few tokens (bfloat16)
// A step that decodes brings few (token, choice) pairs, each with a whole expert's matrices to read:
// the products are bound by that stream.  One warp per output value, 16-byte loads, ROWS output rows
// of one pair per warp so that as many loads are in flight; K % 256 == 0 keeps every lane on whole vectors.
__device__ __forceinline__ float dot8(const uint4 w, const uint4 a) {
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&w);
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 wf = __bfloat1622float2(wp[j]), af = __bfloat1622float2(ap[j]);
        acc = fmaf(wf.x, af.x, acc);
        acc = fmaf(wf.y, af.y, acc);
    }
    return acc;
}

constexpr int SV_ROWS = 4;        // output rows per warp

// MODE 0: act[pair, f] = f(w[e, f, :] . x[pair / top, :])   (x = the tokens' rows, K = D)
// MODE 1: parts[c, t, n] = wts[pair] * (w[e, n, :] . x[pair, :])  (x = the pairs' hidden rows, K = F)
template <int MODE>
__global__ void __launch_bounds__(256)
moe_expert_rows_bf16_kernel(const __nv_bfloat16* __restrict__ x, long x_stride, const __nv_bfloat16* __restrict__ w,
                            const int* __restrict__ ids, const float* __restrict__ wts, void* __restrict__ out,
                            int T, int top, int N, int K, int act_kind) {
    griddep_launch();
    const int pair = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int n0 = (blockIdx.y * 8 + (threadIdx.x >> 5)) * SV_ROWS;
    griddep_wait();
    if (n0 >= N) return;
    const int e = __ldcg(ids + pair);
    const int t = pair / top;
    const __nv_bfloat16* xr = x + (size_t)(MODE == 0 ? t : pair) * x_stride;
    const __nv_bfloat16* wr = w + ((size_t)e * N + n0) * K;
    float acc[SV_ROWS];
#pragma unroll
    for (int j = 0; j < SV_ROWS; ++j) acc[j] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 a = __ldcg(reinterpret_cast<const uint4*>(xr + k));
        uint4 wv[SV_ROWS];
#pragma unroll
        for (int j = 0; j < SV_ROWS; ++j)
            wv[j] = (n0 + j < N) ? __ldg(reinterpret_cast<const uint4*>(wr + (size_t)j * K + k)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int j = 0; j < SV_ROWS; ++j) acc[j] += dot8(wv[j], a);
    }
#pragma unroll
    for (int j = 0; j < SV_ROWS; ++j) acc[j] = warp_sum(acc[j]);
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < SV_ROWS; ++j) {
            if (n0 + j >= N) break;
            if (MODE == 0) {
                reinterpret_cast<__nv_bfloat16*>(out)[(size_t)pair * N + n0 + j] = __float2bfloat16_rn(act_apply(acc[j], act_kind));
            } else {
                const int c = pair - t * top;
                reinterpret_cast<float*>(out)[((size_t)c * T + t) * N + n0 + j] = acc[j] * __ldcg(wts + pair);
            }
        }
    }
}

template <typename T>
__global__ void act_rows_kernel(T* __restrict__ a, size_t n, int act_kind) {
    griddep_launch();
    griddep_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        a[i] = from_f<T>(act_apply(ld_act(a + i), act_kind));
}

}  // namespace aien

using namespace aien;

// expert_count (may be null): E ints that hold zero on entry; every choice adds one to its expert's
// (aien_moe_plan_rows reads them and leaves zeros behind).
AIEN_API int aien_moe_route(const float* z, int T, int E, int groups, int keep, int top, int renorm, int* ids, float* wts,
                            int* expert_count, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E > ROUTE_MAX_EXPERTS || groups <= 0 || E % groups != 0 || keep <= 0 || keep > groups || top <= 0 ||
        top > keep * (E / groups)) return AIEN_E_SHAPE;
    launch_chain(moe_route_kernel, dim3(T), dim3(32), 0, stream, z, E, groups, keep, top, renorm, ids, wts, expert_count);
    return launch_status();
}

// z float32 [T, ldz]: the first E numbers of a row are the router's; correction [E] in c_dt (or null); experts from
// `real` on return their input (w_same float32 [T], needed when real < E).
AIEN_API int aien_moe_route_biased(const float* z, long ldz, int T, int E, int real, int top, int renorm, float renorm_eps,
                                   const void* correction, int c_dt, int* ids, float* wts, float* w_same, int* expert_count,
                                   cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E > ROUTE_MAX_EXPERTS || real <= 0 || real > E || top <= 0 || top > E || (real < E && w_same == nullptr)) return AIEN_E_SHAPE;
    moe_route_biased_kernel<<<T, 32, 0, stream>>>(z, ldz, E, real, top, renorm, renorm_eps, correction, c_dt, ids, wts, w_same, expert_count);
    return launch_status();
}

// h [T, D] (row stride h_stride), w_up [E, F, D], act [T * top, F]; act_kind 0: erf gelu, 1: tanh gelu.
AIEN_API int aien_moe_expert_up(const void* h, int h_dt, long h_stride, const void* w_up, int w_dt, const int* ids,
                                void* act, int act_dt, int T, int top, int D, int F, int act_kind, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (T * (long)top > 2147483647L || D <= 0 || F <= 0 || (F + 7) / 8 > 65535) return AIEN_E_SHAPE;
    dim3 grid(T * top, (F + 7) / 8);
    AIEN_DISPATCH_DTYPE(h_dt, TH, AIEN_DISPATCH_DTYPE(w_dt, TW, AIEN_DISPATCH_DTYPE(act_dt, TO,
        (launch_chain(moe_expert_up_kernel<TH, TW, TO>, grid, dim3(256), 0, stream,
                      (const TH*)h, h_stride, (const TW*)w_up, ids, (TO*)act, top, D, F, act_kind)))));
    return launch_status();
}

// act [T * top, F], w_down [E, D, F], parts float32 [top, T, D].
AIEN_API int aien_moe_expert_down(const void* act, int act_dt, const void* w_down, int w_dt, const int* ids, const float* wts,
                                  float* parts, int T, int top, int D, int F, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (T * (long)top > 2147483647L || D <= 0 || F <= 0 || (D + 7) / 8 > 65535) return AIEN_E_SHAPE;
    dim3 grid(T * top, (D + 7) / 8);
    AIEN_DISPATCH_DTYPE(act_dt, TA, AIEN_DISPATCH_DTYPE(w_dt, TW,
        (launch_chain(moe_expert_down_kernel<TA, TW>, grid, dim3(256), 0, stream,
                      (const TA*)act, (const TW*)w_down, ids, wts, parts, T, top, D, F))));
    return launch_status();
}

// expert_count: what aien_moe_route counted (left zero); cursor: E ints of scratch; tile_group: max_tiles; row_dest: max_tiles * 128.
AIEN_API int aien_moe_plan_rows(int* expert_count, int E, int max_tiles, int* cursor, int* tile_group, int* row_dest, cudaStream_t stream) {
    if (E <= 0 || E > ROUTE_MAX_EXPERTS || max_tiles <= 0) return AIEN_E_SHAPE;
    launch_chain(moe_plan_rows_kernel, dim3(1), dim3(SORT_THREADS), 0, stream, expert_count, E, max_tiles, cursor, tile_group, row_dest);
    return launch_status();
}

AIEN_API int aien_moe_place_rows(const void* h, long h_stride, const int* ids, const float* wts, int* cursor, int T, int top,
                                 void* a_sorted, int D, int* row_dest, float* row_scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long P = (long)T * top;
    if (top <= 0 || P > 2147483647L / 2) return AIEN_E_SHAPE;
    if (D <= 0 || (D & 7) || (h_stride & 7) || ((uintptr_t)h & 15) || ((uintptr_t)a_sorted & 15)) return AIEN_E_ALIGN;
    launch_chain(moe_place_rows_kernel, dim3((unsigned)((P + 3) / 4)), dim3(256), 0, stream, (const __nv_bfloat16*)h, h_stride, ids, wts,
                 cursor, (int)P, T, top, (__nv_bfloat16*)a_sorted, D, row_dest, row_scale);
    return launch_status();
}

// The expert products of a few tokens, bfloat16: mode 0 = up with activation (out bfloat16 [T*top, N], K = D),
// mode 1 = down, weighted, into float32 parts [top, T, N] (K = F).  K % 256 == 0, 16-byte aligned rows.
AIEN_API int aien_moe_expert_rows_bf16(int mode, const void* x, long x_stride, const void* w, const int* ids, const float* wts,
                                       void* out, int T, int top, int N, int K, int act_kind, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (N <= 0 || K <= 0 || (K & 255) || (x_stride & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return AIEN_E_ALIGN;
    const int tiles = (N + 8 * SV_ROWS - 1) / (8 * SV_ROWS);
    if (tiles > 65535 || (long)T * top > 2147483647L) return AIEN_E_SHAPE;
    dim3 grid(T * top, tiles);
    if (mode == 0)
        launch_chain(moe_expert_rows_bf16_kernel<0>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)x, x_stride,
                     (const __nv_bfloat16*)w, ids, wts, out, T, top, N, K, act_kind);
    else
        launch_chain(moe_expert_rows_bf16_kernel<1>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)x, x_stride,
                     (const __nv_bfloat16*)w, ids, wts, out, T, top, N, K, act_kind);
    return launch_status();
}

AIEN_API int aien_act_rows(void* a, int dt, size_t n, int act_kind, cudaStream_t stream) {
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    AIEN_DISPATCH_DTYPE(dt, TT, (launch_chain(act_rows_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (TT*)a, n, act_kind)));
    return launch_status();
}
