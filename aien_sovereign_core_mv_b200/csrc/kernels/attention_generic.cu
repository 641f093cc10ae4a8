// Paged causal grouped-query attention, one block per (query token, query head), any head size
// up to 256, any number of heads and groups, any page size, optional window, optional chunk
// mask (a token sees only keys of its own chunk of `chunk` positions, counted from position 0),
// optional per-head sink (one more term exp(sink[h]) in the softmax denominator, with no key and
// no value), values of their own size `hdv` <= head size, optionally only the tokens that
// `token_list` names (T of them).  Optional per head: a factor on the scaled score (`head_scale`), a distance bias
// (`slopes`: slope[h] * (query position - key position) is taken off the score) and an output gate (`gate` float32
// [T, ldg]: the head's output is multiplied by sigmoid(gate[t][h])).  `softcap` c > 0: the scaled score s becomes
// c * tanh(s / c) before the other terms.
//
// It serves the true-32-bit engine for every kind of step (whole prompts, portions with an
// offset, single decoded tokens) and is the plain kernel the faster attention kernels are
// checked against.  A token at position p of request s sees the keys at positions
// max(0, p-window+1) .. p of that request, read through the request's block table; keys are
// visited in position order in chunks of 128 with an online softmax, so the result depends
// only on the token's own position and cache contents, never on how the step was cut or
// batched.  Scores, softmax and the weighted sum are float32
// (formulas: crates/aien-inference-abi/src/backend.rs:311-379, scale 1/sqrt(head_dim)).
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int AG_THREADS = 128;

template <typename TQ, typename TKV, typename TO>
__global__ void __launch_bounds__(AG_THREADS)
paged_attention_generic_kernel(const TQ* __restrict__ q, long q_stride,
                               const TKV* __restrict__ k_cache, const TKV* __restrict__ v_cache,
                               const int* __restrict__ block_table, int max_blocks,
                               const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                               TO* __restrict__ out, long out_stride,
                               int nq, int nkv, int hd, int page_size, int window, float scale,
                               int chunk, const float* __restrict__ sinks, int hdv, const int* __restrict__ token_list,
                               const float* __restrict__ head_scale, const float* __restrict__ slopes,
                               const float* __restrict__ gate, long ldg, float softcap) {
    __shared__ float qs[256];
    __shared__ float p[AG_THREADS];
    __shared__ int slots[AG_THREADS];
    __shared__ float red[32];
    const int h = blockIdx.x, t = token_list ? token_list[blockIdx.y] : blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    const int* bt = block_table + (size_t)seq_of_token[t] * max_blocks;
    const int kvh = h / (nq / nkv);
    int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (chunk > 0 && (pos / chunk) * chunk > start) start = (pos / chunk) * chunk;

    for (int d = tid; d < hd; d += AG_THREADS) qs[d] = to_f(q[(size_t)t * q_stride + (size_t)h * hd + d]);
    __syncthreads();
    const float hscale = head_scale ? head_scale[h] : 1.0f;
    const float slope = slopes ? slopes[h] : 0.0f;

    float m = -INFINITY, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;                      // dims tid and tid + 128
    for (int base = start; base <= pos; base += AG_THREADS) {
        const int j = base + tid;
        float score = -INFINITY;
        int slot = -1;
        if (j <= pos) {
            const int page = bt[j / page_size];
            if (page >= 0) {
                slot = page * page_size + (j % page_size);
                const TKV* kp = k_cache + ((size_t)slot * nkv + kvh) * hd;
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;       // four chains: a quarter of the rounding error's growth
                int d = 0;
                for (; d + 3 < hd; d += 4) {
                    d0 = fmaf(qs[d], to_f(kp[d]), d0);
                    d1 = fmaf(qs[d + 1], to_f(kp[d + 1]), d1);
                    d2 = fmaf(qs[d + 2], to_f(kp[d + 2]), d2);
                    d3 = fmaf(qs[d + 3], to_f(kp[d + 3]), d3);
                }
                for (; d < hd; ++d) d0 = fmaf(qs[d], to_f(kp[d]), d0);
                const float dot = (d0 + d1) + (d2 + d3);
                score = dot * scale;
                if (softcap > 0.f) score = softcap * tanhf(score / softcap);
                if (head_scale) score *= hscale;
                if (slopes) score -= slope * (float)(pos - j);
            }
        }
        slots[tid] = slot;
        const float cmax = block_max(score, red);
        const float m_new = fmaxf(m, cmax);
        if (m_new == -INFINITY) continue;              // nothing visible yet (whole chunk masked)
        const float e = (slot >= 0) ? expf(score - m_new) : 0.f;
        p[tid] = e;
        const float csum = block_sum(e, red);           // also orders the writes to p/slots
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + csum;
        const int n = (pos - base + 1 < AG_THREADS) ? pos - base + 1 : AG_THREADS;
        float part0 = 0.f, part1 = 0.f;                   // the chunk's own sum, added to the running one at its end
        for (int jj = 0; jj < n; ++jj) {
            const int sl = slots[jj];
            if (sl < 0) continue;
            const float pj = p[jj];
            const TKV* vp = v_cache + ((size_t)sl * nkv + kvh) * hdv;
            if (tid < hdv) part0 = fmaf(pj, to_f(vp[tid]), part0);
            if (tid + AG_THREADS < hdv) part1 = fmaf(pj, to_f(vp[tid + AG_THREADS]), part1);
        }
        acc0 = fmaf(acc0, corr, part0);
        acc1 = fmaf(acc1, corr, part1);
        m = m_new;
        __syncthreads();
    }
    if (sinks != nullptr) {                            // the sink joins the denominator once, unscaled
        const float sk = sinks[h];
        const float m_new = fmaxf(m, sk);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + expf(sk - m_new);
        acc0 *= corr;
        acc1 *= corr;
    }
    float inv = l > 0.f ? 1.0f / l : 0.f;              // empty context gives zeros (backend.rs:320)
    if (gate) inv *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));
    TO* o = out + (size_t)t * out_stride + (size_t)h * hdv;
    if (tid < hdv) o[tid] = from_f<TO>(acc0 * inv);
    if (tid + AG_THREADS < hdv) o[tid + AG_THREADS] = from_f<TO>(acc1 * inv);
}

}  // namespace aien

using namespace aien;

AIEN_API int aien_paged_attention_generic(
    const void* q, long q_stride, const void* k_cache, const void* v_cache,
    const int* block_table, int max_blocks, const int* seq_of_token, const int* positions,
    void* out, long out_stride, int nq, int nkv, int hd, int page_size, int window, float scale,
    int act_dt, int kv_dt, int T, int chunk, const float* sinks, int hdv, const int* token_list,
    const float* head_scale, const float* slopes, const float* gate, long ldg, float softcap, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hdv <= 0) hdv = hd;
    if (hd <= 0 || hd > 256 || hdv > 256 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || chunk < 0) return AIEN_E_SHAPE;
    if (T > 65535) return AIEN_E_SHAPE;
    dim3 grid(nq, T);
    AIEN_DISPATCH_DTYPE(act_dt, TQ, AIEN_DISPATCH_DTYPE(kv_dt, TKV,
        (paged_attention_generic_kernel<TQ, TKV, TQ><<<grid, AG_THREADS, 0, stream>>>(
            (const TQ*)q, q_stride, (const TKV*)k_cache, (const TKV*)v_cache, block_table, max_blocks,
            seq_of_token, positions, (TQ*)out, out_stride, nq, nkv, hd, page_size, window, scale, chunk, sinks, hdv, token_list,
            head_scale, slopes, gate, ldg, softcap))));
    return launch_status();
}
