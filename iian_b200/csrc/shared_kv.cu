// What an attention mixer whose values are its keys does between its input product and the attention itself.
//
// Per token, from one row of the stacked product [.. q (heads x hd) .. k (kv_heads x hd) ..]:
//   * RMS norm of q over the WHOLE projection (all heads at once), weight per column; the same for k;
//   * rotation of the first `rot` entries of every head of q and k by the token's position (pairs (2i, 2i+1) or
//     (i, i + rot/2)), angle p * f_i formed as a float64 product, cos and sin once per token and pair;
//   * q goes to the attention's query rows; the normalised, rotated k into the key cache cell of the token; the k
//     AS PROJECTED (before norm and rotation) into the value cache cell: the values are the keys.
// Sums, norm factors, angles and the rotation are float32 or better; one CTA per token, so a token's result depends on
// that token only.
#include "common.cuh"

namespace iian {

template <typename A>
__global__ void projection_norm_rope_store_kernel(
    const A * __restrict__ proj, long long ld, int q_off, int k_off, A * __restrict__ q_out, A * __restrict__ k_cache,
    A * __restrict__ v_cache, const float * __restrict__ q_weight, const float * __restrict__ k_weight,
    const double * __restrict__ inv_freq, const int * __restrict__ positions, const int * __restrict__ slots, int nh,
    int nkv, int hd, int rot, int style, float eps, int page_size, int num_pages, int normed) {
    pdl_wait();
    extern __shared__ float cs[];                  // cos [rot / 2], sin [rot / 2]
    __shared__ float scratch[32];
    const size_t t = blockIdx.x;
    const A * qr = proj + t * ld + q_off;
    const A * kr = proj + t * ld + k_off;
    const int nq = nh * hd, nk = nkv * hd;
    const int half = rot / 2;
    const int p = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double s, c;
        sincos((double) p * inv_freq[i], &s, &c);
        cs[i] = (float) c;
        cs[half + i] = (float) s;
    }
    float inv_q = 1.0f, inv_k = 1.0f;
    if (normed) {
        float sq = 0.0f, sk = 0.0f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = to_f32(qr[i]); sq += v * v; }
        for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = to_f32(kr[i]); sk += v * v; }
        sq = block_sum(sq, scratch);
        sk = block_sum(sk, scratch);
        inv_q = rsqrtf(sq / (float) nq + eps);
        inv_k = rsqrtf(sk / (float) nk + eps);
    }
    __syncthreads();
    const int slot = (slots != nullptr && k_cache != nullptr) ? slots[t] : -1;
    const int page = slot >= 0 ? slot / page_size : -1, cell = slot >= 0 ? slot % page_size : 0;
    const bool store = page >= 0 && page < num_pages;
    // one item per (head, pair or single entry): entries below `rot` in pairs, the rest alone
    const int per_head = half + (hd - rot);
    for (int it = threadIdx.x; it < (nh + nkv) * per_head; it += blockDim.x) {
        const int h = it / per_head, j = it - h * per_head;
        const bool is_q = h < nh;
        const int hh = is_q ? h : h - nh;
        const A * src = (is_q ? qr : kr) + hh * hd;
        const float * w = normed ? (is_q ? q_weight : k_weight) + hh * hd : nullptr;
        const float inv = is_q ? inv_q : inv_k;
        A * dst = is_q ? q_out + (t * nh + hh) * hd : (store ? k_cache + (((size_t) page * nkv + hh) * page_size + cell) * hd : nullptr);
        A * vdst = (!is_q && store) ? v_cache + (((size_t) page * nkv + hh) * page_size + cell) * hd : nullptr;
        if (j < half) {
            const int i0 = style == 1 ? 2 * j : j, i1 = style == 1 ? 2 * j + 1 : j + half;
            const float r0 = to_f32(src[i0]), r1 = to_f32(src[i1]);
            const float x0 = normed ? r0 * inv * w[i0] : r0, x1 = normed ? r1 * inv * w[i1] : r1;
            const float c = cs[j], s = cs[half + j];
            if (dst != nullptr) {
                dst[i0] = from_f32<A>(rot_lo(x0, x1, c, s));
                dst[i1] = from_f32<A>(rot_hi(x0, x1, c, s));
            }
            if (vdst != nullptr) { vdst[i0] = src[i0]; vdst[i1] = src[i1]; }
        } else {
            const int i0 = rot + (j - half);
            const float r0 = to_f32(src[i0]);
            if (dst != nullptr) dst[i0] = from_f32<A>(normed ? r0 * inv * w[i0] : r0);
            if (vdst != nullptr) vdst[i0] = src[i0];
        }
    }
}

}  // namespace iian

using namespace iian;

// proj: A rows with stride ld; q_out: A [N, nh, hd]; caches: A [num_pages, nkv, page_size, hd] (null: store nothing);
// q_weight [nh * hd], k_weight [nkv * hd] f32 (both null: no norm); inv_freq f64 [rot / 2] (null when rot == 0);
// style 0: pairs (i, i + rot / 2), 1: pairs (2i, 2i + 1); slots: cache cell of each token (-1: store nothing)
IIAN_API int iian_projection_norm_rope_store(const void * proj, long long ld, int q_off, int k_off, void * q_out, void * k_cache,
                                             void * v_cache, const float * q_weight, const float * k_weight,
                                             const double * inv_freq, const int * positions, const int * slots, int act_dtype,
                                             int N, int nh, int nkv, int hd, int rot, int style, float eps, int page_size,
                                             int num_pages, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (nh <= 0 || nkv < 0 || hd <= 0 || rot < 0 || rot > hd || rot % 2 || (rot > 0 && inv_freq == nullptr) || page_size <= 0 ||
        (q_weight == nullptr) != (k_weight == nullptr))
        return IIAN_ERR_SHAPE;
    const int normed = q_weight != nullptr ? 1 : 0;
    const int threads = 256;
    const size_t smem = (size_t) rot * sizeof(float);
    if (act_dtype == IIAN_F32)
        return iian_launch(projection_norm_rope_store_kernel<float>, dim3(N), dim3(threads), smem, stream, (const float *) proj, ld,
                           q_off, k_off, (float *) q_out, (float *) k_cache, (float *) v_cache, q_weight, k_weight, inv_freq,
                           positions, slots, nh, nkv, hd, rot, style, eps, page_size, num_pages, normed);
    if (act_dtype == IIAN_BF16)
        return iian_launch(projection_norm_rope_store_kernel<__nv_bfloat16>, dim3(N), dim3(threads), smem, stream,
                           (const __nv_bfloat16 *) proj, ld, q_off, k_off, (__nv_bfloat16 *) q_out, (__nv_bfloat16 *) k_cache,
                           (__nv_bfloat16 *) v_cache, q_weight, k_weight, inv_freq, positions, slots, nh, nkv, hd, rot, style, eps,
                           page_size, num_pages, normed);
    return IIAN_ERR_DTYPE;
}
