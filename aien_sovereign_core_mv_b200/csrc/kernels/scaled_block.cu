// What a pre-norm layer with a scale per channel on every branch needs around its sublayers, and the small kernels
// of the feed-forwards that such layers carry.
//
//   scaled_add_rmsnorm   x += vec * (sum of the branch's parts + bias)   (float32, in place; vec and bias may be null);
//                        then, when asked, out = x / sqrt(mean(x^2) + eps) * w in the compute dtype
//   pass_input           x += again (when given), then x += row (one vector for every token): what a repeated run of
//                        layers adds to the stream before each pass
//   clamped_glu          g = min(a_gate + b_gate, limit), u = clamp(a_up + b_up, -limit, limit);
//                        out = g * sigmoid(alpha * g) * (u + 1)
//   sigmoid_gate         out = o * sigmoid(g) * mult, element by element (g null: out = o * mult)
//   routed_combine       out = sum of the routed parts + w_same[t] * h[t] + sigmoid(zs[t]) * shared[t]
//
// Sums, norms and gates are float32 in both engine precisions.
#include "common.cuh"
#include <math.h>

namespace aien {

template <typename TD, typename TO>
__global__ void __launch_bounds__(1024)
scaled_add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int nparts, size_t part_stride,
                          const float* __restrict__ vec, const float* __restrict__ bias, const void* __restrict__ w, int wdt,
                          float eps, TO* __restrict__ out, int H) {
    __shared__ float red[32];
    const size_t row = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[row + i];
        if (delta != nullptr) {
            float d = 0.f;
            for (int p = 0; p < nparts; ++p) d += to_f(delta[(size_t)p * part_stride + row + i]);
            if (bias != nullptr) d += bias[i];
            v = vec != nullptr ? fmaf(vec[i], d, v) : v + d;
            x[row + i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    if (out == nullptr) return;
    const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[row + i] = from_f<TO>(x[row + i] * r * load_dyn(w, wdt, i));
}

__global__ void __launch_bounds__(256)
pass_input_kernel(float* __restrict__ x, const float* __restrict__ again, const void* __restrict__ row, int rdt, size_t n, int H) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    if (again != nullptr) v += again[i];
    x[i] = v + load_dyn(row, rdt, i % H);
}

template <typename TA, typename TO>
__global__ void __launch_bounds__(256)
clamped_glu_kernel(const TA* __restrict__ a, long lda, int gate_off, int up_off, const void* __restrict__ bg, const void* __restrict__ bu,
                   int bdt, float limit, float alpha, TO* __restrict__ out, long ldo, int F) {
    const int t = blockIdx.y, f = blockIdx.x * 256 + threadIdx.x;
    if (f >= F) return;
    float g = to_f(a[(size_t)t * lda + gate_off + f]);
    float u = to_f(a[(size_t)t * lda + up_off + f]);
    if (bg != nullptr) g += load_dyn(bg, bdt, f);
    if (bu != nullptr) u += load_dyn(bu, bdt, f);
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    out[(size_t)t * ldo + f] = from_f<TO>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(const TI* __restrict__ o, long ldi, const float* __restrict__ g, long ldg, float mult, TO* __restrict__ out, long ldo, int C) {
    const int t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c >= C) return;
    float v = to_f(o[(size_t)t * ldi + c]) * mult;
    if (g != nullptr) v /= 1.0f + expf(-g[(size_t)t * ldg + c]);
    out[(size_t)t * ldo + c] = from_f<TO>(v);
}

template <typename TP, typename TH, typename TS>
__global__ void __launch_bounds__(256)
routed_combine_kernel(const TP* __restrict__ parts, int nparts, size_t part_stride, const TH* __restrict__ h, long ldh,
                      const float* __restrict__ w_same, const TS* __restrict__ shared, int sparts, size_t sstride,
                      const float* __restrict__ zs, long ldzs, float* __restrict__ out, int H) {
    const int t = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x;
    if (i >= H) return;
    const size_t at = (size_t)t * H + i;
    float v = 0.f;
    for (int p = 0; p < nparts; ++p) v += to_f(parts[(size_t)p * part_stride + at]);
    if (w_same != nullptr) v = fmaf(w_same[t], to_f(h[(size_t)t * ldh + i]), v);
    if (shared != nullptr) {
        float sv = 0.f;
        for (int p = 0; p < sparts; ++p) sv += to_f(shared[(size_t)p * sstride + at]);
        v = zs != nullptr ? fmaf(1.0f / (1.0f + expf(-zs[(size_t)t * ldzs])), sv, v) : v + sv;
    }
    out[at] = v;
}

}  // namespace aien

using namespace aien;

// x float32 [T, H]; delta [nparts][T, H] in d_dt (null: nothing to add); vec and bias float32 [H] or null; out [T, H] in
// o_dt or null (only the sum is made); w [H] in w_dt.
AIEN_API int aien_scaled_add_rmsnorm(float* x, const void* delta, int d_dt, int nparts, size_t part_stride, const float* vec,
                                     const float* bias, const void* w, int w_dt, float eps, void* out, int o_dt, int T, int H,
                                     cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || (delta != nullptr && nparts <= 0)) return AIEN_E_SHAPE;
    // a step of few tokens has too few CTAs to hide a row's loads behind one another: wide CTAs then
    const int threads = (T <= 2 * 148 && H >= 1024) ? 1024 : 256;
    AIEN_DISPATCH_DTYPE(d_dt, TD, AIEN_DISPATCH_DTYPE(o_dt, TO,
        (scaled_add_rmsnorm_kernel<TD, TO><<<T, threads, 0, stream>>>(x, (const TD*)delta, nparts, part_stride, vec, bias, w, w_dt, eps, (TO*)out, H))));
    return launch_status();
}

// x float32 [T, H] += again (float32 [T, H] or null), then += row ([H] in r_dt) for every token.
AIEN_API int aien_pass_input(float* x, const float* again, const void* row, int r_dt, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    const size_t n = (size_t)T * H;
    pass_input_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, again, row, r_dt, n, H);
    return launch_status();
}

// a [T, lda] in a_dt with the gate's F numbers from gate_off and the other half's from up_off; biases [F] in b_dt or null.
AIEN_API int aien_clamped_glu(const void* a, int a_dt, long lda, int gate_off, int up_off, const void* bg, const void* bu, int b_dt,
                              float limit, float alpha, void* out, int o_dt, long ldo, int T, int F, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (F <= 0 || T > 65535) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(a_dt, TA, AIEN_DISPATCH_DTYPE(o_dt, TO,
        (clamped_glu_kernel<TA, TO><<<dim3((F + 255) / 256, T), 256, 0, stream>>>((const TA*)a, lda, gate_off, up_off, bg, bu, b_dt, limit,
                                                                                   alpha, (TO*)out, ldo, F))));
    return launch_status();
}

// out[t][c] = o[t][c] * sigmoid(g[t][c]) * mult; o [T, ldi] in i_dt, g float32 [T, ldg] (null: no gate), out [T, ldo] in o_dt.
AIEN_API int aien_sigmoid_gate(const void* o, int i_dt, long ldi, const float* g, long ldg, float mult, void* out, int o_dt, long ldo,
                               int T, int C, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (C <= 0 || T > 65535) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(i_dt, TI, AIEN_DISPATCH_DTYPE(o_dt, TO,
        (sigmoid_gate_kernel<TI, TO><<<dim3((C + 255) / 256, T), 256, 0, stream>>>((const TI*)o, ldi, g, ldg, mult, (TO*)out, ldo, C))));
    return launch_status();
}

// parts [nparts][T, H] in p_dt; h [T, ldh] in h_dt with w_same float32 [T] (or null: no such term); shared [sparts][T, H] in
// s_dt (or null) times sigmoid(zs[t * ldzs]) (zs null: times one); out float32 [T, H].
AIEN_API int aien_routed_combine(const void* parts, int p_dt, int nparts, size_t part_stride, const void* h, int h_dt, long ldh,
                                 const float* w_same, const void* shared, int s_dt, int sparts, size_t sstride, const float* zs, long ldzs,
                                 float* out, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || T > 65535) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(p_dt, TP, AIEN_DISPATCH_DTYPE(h_dt, TH, AIEN_DISPATCH_DTYPE(s_dt, TS,
        (routed_combine_kernel<TP, TH, TS><<<dim3((H + 255) / 256, T), 256, 0, stream>>>(
            (const TP*)parts, nparts, part_stride, (const TH*)h, ldh, w_same, (const TS*)shared, sparts, sstride, zs, ldzs, out, H)))));
    return launch_status();
}
