// Rotation of q and k and the cache write for attention whose values have a size of their own.
//
// q (nq heads of hd numbers), k (nkv heads of hd) and v (nkv heads of hdv) are column blocks of one float32 projection
// [T, ld].  The first `rot` dimensions of every q and k head turn by the token's angles, dimension i with dimension
// i + rot/2 (cos and sin float32 [T, rot/2]); the rest pass unchanged.  q leaves in the compute dtype, k and v go to the
// token's cache slot (slot < 0: nothing is written).  One warp per (token, head); all of it float32.
#include "common.cuh"

namespace aien {

template <typename TQ, typename TKV>
__global__ void __launch_bounds__(128)
rope_halves_value_write_kernel(const float* __restrict__ proj, long ld, int q_off, int k_off, int v_off, int nq, int nkv, int hd, int hdv,
                               const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                               const int* __restrict__ slot_map, TQ* __restrict__ q_out, long ldq,
                               TKV* __restrict__ k_cache, TKV* __restrict__ v_cache) {
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int head = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (head >= nq + 2 * nkv) return;
    const float* row = proj + (size_t)t * ld;
    const int half = rot >> 1;
    if (head >= nq + nkv) {                                    // a value head: a copy
        const long slot = slot_map[t];
        if (slot < 0) return;
        const int g = head - nq - nkv;
        for (int i = lane; i < hdv; i += 32)
            v_cache[((size_t)slot * nkv + g) * hdv + i] = from_f<TKV>(row[v_off + (size_t)g * hdv + i]);
        return;
    }
    const bool is_q = head < nq;
    const int hh = is_q ? head : head - nq;
    const long slot = is_q ? 0 : (long)slot_map[t];
    if (slot < 0) return;
    const float* src = row + (is_q ? q_off : k_off) + (size_t)hh * hd;
    for (int i = lane; i < hd; i += 32) {
        float v = src[i];
        if (i < rot) {
            const int j = i < half ? i : i - half;
            const float c = cos_t[(size_t)t * half + j], s = sin_t[(size_t)t * half + j];
            v = i < half ? v * c - src[i + half] * s : v * c + src[i - half] * s;
        }
        if (is_q) q_out[(size_t)t * ldq + (size_t)hh * hd + i] = from_f<TQ>(v);
        else k_cache[((size_t)slot * nkv + hh) * hd + i] = from_f<TKV>(v);
    }
}

}  // namespace aien

using namespace aien;

AIEN_API int aien_rope_halves_value_write(const float* proj, long ld, int q_off, int k_off, int v_off, int nq, int nkv, int hd, int hdv,
                                          const float* cos_t, const float* sin_t, int rot, const int* slot_map, void* q_out, int q_dt,
                                          long ldq, void* k_cache, void* v_cache, int kv_dt, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || hd <= 0 || hdv <= 0 || rot < 0 || rot > hd || (rot & 1) || (rot > 0 && (cos_t == nullptr || sin_t == nullptr)))
        return AIEN_E_SHAPE;
    const dim3 grid(T, (nq + 2 * nkv + 3) / 4);
    AIEN_DISPATCH_DTYPE(q_dt, TQ, AIEN_DISPATCH_DTYPE(kv_dt, TKV,
        (rope_halves_value_write_kernel<TQ, TKV><<<grid, 128, 0, stream>>>(proj, ld, q_off, k_off, v_off, nq, nkv, hd, hdv, cos_t, sin_t, rot,
                                                                           slot_map, (TQ*)q_out, ldq, (TKV*)k_cache, (TKV*)v_cache))));
    return launch_status();
}
