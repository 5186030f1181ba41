// Row-wise kernels of post-norm layers: the gated residual sum with its LayerNorm, a weighted sum of several
// streams (depth mix), and the gated activation of a feed-forward with a choice of activation.
//
// The stream is float32; `A` is the activation type (float in the 32-bit path, bfloat16 in the serving path).
// Every row is reduced in an order fixed by the row length alone, so a row's result does not depend on the batch.
//
//   gated_add_layer_norm:  s = alpha * x + sub * sigmoid(g + gb);   y = (s - mean(s)) / sqrt(var(s) + eps) * w + b
//                          with var the mean of the squared deviations (two passes over the row, held in shared memory)
//   depth_mix:             y[r] = sum_j c[j] * X_j[row_j(r)]   in the order j = 0, 1, 2, ...
//   gated_act:             y = act(gate) * up,  act = silu (z / (1 + exp(-z))) or the tanh form of gelu
//                          (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))))
#include "common.cuh"

namespace iian {

constexpr int kMaxMixTerms = 128;
struct MixTerms {
    const float * x[kMaxMixTerms];
};

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename A, typename G>
__global__ void gated_add_layer_norm_kernel(const float * __restrict__ x, const A * __restrict__ sub, long long ld_sub,
                                            const G * __restrict__ glogit, long long ld_g, const float * __restrict__ gbias,
                                            const float * __restrict__ w, const float * __restrict__ b,
                                            float * __restrict__ out, A * __restrict__ out_act,
                                            int H, float alpha, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const size_t n = blockIdx.x;
    const float * xr = x + n * H;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = alpha * xr[i];
        if (sub != nullptr) {
            float s = to_f32(sub[n * ld_sub + i]);
            if (glogit != nullptr) s *= sigmoid_f(to_f32(glogit[n * ld_g + i]) + (gbias != nullptr ? gbias[i] : 0.0f));
            v += s;
        }
        row[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float) H;
    float dev = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = row[i] - mean;
        dev += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(dev, scratch) / (float) H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float y = (row[i] - mean) * inv * w[i] + (b != nullptr ? b[i] : 0.0f);
        if (out != nullptr) out[n * H + i] = y;
        if (out_act != nullptr) out_act[n * H + i] = from_f32<A>(y);
    }
}

// four consecutive elements as float4: 16-byte (float) or 8-byte (bfloat16) accesses
template <typename T> struct V4;
template <> struct V4<float> {
    static __device__ __forceinline__ float4 load(const float * p) { return *reinterpret_cast<const float4 *>(p); }
    static __device__ __forceinline__ void store(float * p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
};
template <> struct V4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16 * p) {
        const uint2 raw = *reinterpret_cast<const uint2 *>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 * p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned *>(&a);
        raw.y = *reinterpret_cast<unsigned *>(&b);
        *reinterpret_cast<uint2 *>(p) = raw;
    }
};

// The same for H % 4 == 0, H <= 16 * blockDim and aligned operands: the row stays in registers (thread t owns the
// groups of four t, t + blockDim, ...: fixed by H alone), one pass over memory, wide accesses.  The sums run over the
// same values as in the general form; their order differs, so a model uses one form or the other for a given H.
template <typename A, typename G, int VPT>
__global__ void gated_add_layer_norm_vec_kernel(const float * __restrict__ x, const A * __restrict__ sub, long long ld_sub,
                                                const G * __restrict__ glogit, long long ld_g, const float * __restrict__ gbias,
                                                const float * __restrict__ w, const float * __restrict__ b,
                                                float * __restrict__ out, A * __restrict__ out_act,
                                                int H, float alpha, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t n = blockIdx.x;
    const int groups = H >> 2;
    float4 v[VPT];
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int gi = threadIdx.x + k * blockDim.x;
        if (gi < groups) {
            float4 t = V4<float>::load(x + n * H + 4 * gi);
            t.x *= alpha; t.y *= alpha; t.z *= alpha; t.w *= alpha;
            if (sub != nullptr) {
                float4 s4 = V4<A>::load(sub + n * ld_sub + 4 * gi);
                if (glogit != nullptr) {
                    float4 g4 = V4<G>::load(glogit + n * ld_g + 4 * gi);
                    if (gbias != nullptr) {
                        const float4 b4 = V4<float>::load(gbias + 4 * gi);
                        g4.x += b4.x; g4.y += b4.y; g4.z += b4.z; g4.w += b4.w;
                    }
                    s4.x *= sigmoid_f(g4.x); s4.y *= sigmoid_f(g4.y); s4.z *= sigmoid_f(g4.z); s4.w *= sigmoid_f(g4.w);
                }
                t.x += s4.x; t.y += s4.y; t.z += s4.z; t.w += s4.w;
            }
            v[k] = t;
            sum += (t.x + t.y) + (t.z + t.w);
        }
    }
    const float mean = block_sum(sum, scratch) / (float) H;
    float dev = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int gi = threadIdx.x + k * blockDim.x;
        if (gi < groups) {
            const float dx = v[k].x - mean, dy = v[k].y - mean, dz = v[k].z - mean, dw = v[k].w - mean;
            dev += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(dev, scratch) / (float) H + eps);
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int gi = threadIdx.x + k * blockDim.x;
        if (gi < groups) {
            const float4 w4 = V4<float>::load(w + 4 * gi);
            float4 y = make_float4((v[k].x - mean) * inv * w4.x, (v[k].y - mean) * inv * w4.y, (v[k].z - mean) * inv * w4.z,
                                   (v[k].w - mean) * inv * w4.w);
            if (b != nullptr) {
                const float4 b4 = V4<float>::load(b + 4 * gi);
                y.x += b4.x; y.y += b4.y; y.z += b4.z; y.w += b4.w;
            }
            if (out != nullptr) V4<float>::store(out + n * H + 4 * gi, y);
            if (out_act != nullptr) V4<A>::store(out_act + n * H + 4 * gi, y);
        }
    }
}

// depth mix, four columns a thread (H % 4 == 0, aligned streams)
template <typename A>
__global__ void depth_mix_vec_kernel(MixTerms terms, int n_terms, const float * __restrict__ coef, const int * __restrict__ rows,
                                     int n_src, int last_is_selected, float * __restrict__ out, A * __restrict__ out_act, int H) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t r = blockIdx.x;
    long long src = (long long) r;
    if (rows != nullptr) src = rows[r];
    const bool src_ok = src >= 0 && src < n_src;
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int j = 0; j < n_terms; j++) {
            const bool own = rows == nullptr || (last_is_selected && j == n_terms - 1);
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (own) v = V4<float>::load(terms.x[j] + r * H + i);
            else if (src_ok) v = V4<float>::load(terms.x[j] + (size_t) src * H + i);
            const float c = coef[j];
            acc.x = fmaf(c, v.x, acc.x); acc.y = fmaf(c, v.y, acc.y); acc.z = fmaf(c, v.z, acc.z); acc.w = fmaf(c, v.w, acc.w);
        }
        if (out != nullptr) V4<float>::store(out + r * H + i, acc);
        if (out_act != nullptr) V4<A>::store(out_act + r * H + i, acc);
    }
}

template <typename A>
__global__ void depth_mix_kernel(MixTerms terms, int n_terms, const float * __restrict__ coef, const int * __restrict__ rows,
                                 int n_src, int last_is_selected, float * __restrict__ out, A * __restrict__ out_act, int H) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t r = blockIdx.x;
    long long src = (long long) r;
    if (rows != nullptr) src = rows[r];
    const bool src_ok = src >= 0 && src < n_src;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < n_terms; j++) {
            const bool own = rows == nullptr || (last_is_selected && j == n_terms - 1);
            float v = 0.0f;
            if (own) v = terms.x[j][r * H + i];
            else if (src_ok) v = terms.x[j][(size_t) src * H + i];
            acc = fmaf(coef[j], v, acc);
        }
        if (out != nullptr) out[r * H + i] = acc;
        if (out_act != nullptr) out_act[r * H + i] = from_f32<A>(acc);
    }
}

__device__ __forceinline__ float act_apply(float z, int act) {
    if (act == 0) return z / (1.0f + expf(-z));
    const float t = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(t));
}

// in rows: [gate (F) | up (F)] (interleave 0) or groups of 16 columns holding 8 gate values and then the 8 up
// values of the same features (interleave 8); row stride ld_in elements
template <typename A>
__global__ void gated_act_kernel(const A * __restrict__ in, long long ld_in, A * __restrict__ out, int F, size_t total,
                                 int interleave, int act, float limit) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t idx = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t r = idx / F;
    const int col = (int) (idx - r * F);
    const size_t gi = r * ld_in + (interleave ? (size_t) (col / 8) * 16 + col % 8 : (size_t) col);
    const size_t ui = interleave ? gi + 8 : gi + F;
    float g = to_f32(in[gi]), u = to_f32(in[ui]);
    if (act == 2) {     // clamped: g' = min(g, limit), u' = clamp(u, -limit, limit); g' sigmoid(1.702 g') (u' + 1)
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        out[idx] = from_f32<A>(g / (1.0f + expf(-1.702f * g)) * (u + 1.0f));
        return;
    }
    out[idx] = from_f32<A>(act_apply(g, act) * u);
}

}  // namespace iian

using namespace iian;

static int norm_threads(int H) { return H >= 2048 ? 512 : H >= 512 ? 256 : 128; }

// x f32 [N, H]; sub (act dtype, row stride ld_sub) or null; glogit (gate dtype, row stride ld_g) or null; gbias f32 [H] or
// null; w f32 [H]; b f32 [H] or null; out f32 [N, H] or null; out_act (act dtype) [N, H] or null
IIAN_API int iian_gated_add_layer_norm(const float * x, const void * sub, long long ld_sub, const void * glogit, long long ld_g,
                                       int gate_dtype, const float * gbias, const float * w, const float * b, float * out,
                                       void * out_act, int act_dtype, int N, int H, float alpha, float eps, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (H <= 0 || (size_t) H * 4 > 200 * 1024) return IIAN_ERR_LIMIT;
    const size_t smem = (size_t) H * 4;
    int threads = norm_threads(H);
    typedef __nv_bfloat16 bf;
    // the register form: a function of H and of the operands' alignment alone, never of the batch
    const size_t a_al = act_dtype == IIAN_BF16 ? 7 : 15, g_al = gate_dtype == IIAN_BF16 ? 7 : 15;
    const size_t a_ld = 4, g_ld = 4;
    const bool vec = H % 4 == 0 && H <= 16 * 1024 && ((uintptr_t) x & 15) == 0 && ((uintptr_t) w & 15) == 0 && ((uintptr_t) b & 15) == 0 &&
                     ((uintptr_t) gbias & 15) == 0 && ((uintptr_t) out & 15) == 0 && ((uintptr_t) out_act & a_al) == 0 &&
                     ((uintptr_t) sub & a_al) == 0 && ld_sub % (long long) a_ld == 0 && ((uintptr_t) glogit & g_al) == 0 &&
                     ld_g % (long long) g_ld == 0;
    if (vec) {
        const int groups = H / 4;
        threads = 128;                                       // a group of four a thread up to 1024 threads, then up to four
        while (threads < 1024 && threads < groups) threads *= 2;
    }
#define IIAN_GLN(AT, GT)                                                                                                     \
    do {                                                                                                                     \
        if (vec)                                                                                                             \
            return iian_launch(gated_add_layer_norm_vec_kernel<AT, GT, 4>, dim3(N), dim3(threads), 0, stream, x, (const AT *) sub, \
                               ld_sub, (const GT *) glogit, ld_g, gbias, w, b, out, (AT *) out_act, H, alpha, eps);          \
        if (smem > 48 * 1024) cudaFuncSetAttribute(gated_add_layer_norm_kernel<AT, GT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem); \
        return iian_launch(gated_add_layer_norm_kernel<AT, GT>, dim3(N), dim3(threads), smem, stream, x, (const AT *) sub, ld_sub, \
                           (const GT *) glogit, ld_g, gbias, w, b, out, (AT *) out_act, H, alpha, eps);                      \
    } while (0)
    if (act_dtype == IIAN_F32 && gate_dtype == IIAN_F32) IIAN_GLN(float, float);
    if (act_dtype == IIAN_BF16 && gate_dtype == IIAN_BF16) IIAN_GLN(bf, bf);
    if (act_dtype == IIAN_BF16 && gate_dtype == IIAN_F32) IIAN_GLN(bf, float);
#undef IIAN_GLN
    return IIAN_ERR_DTYPE;
}

// terms: n_terms pointers to f32 [*, H]; coef f32 [n_terms]; rows (i32 [R]) or null: term j < n_terms - 1 (all terms
// unless last_is_selected) is read at row rows[r], the last one at row r
IIAN_API int iian_depth_mix(const float * const * terms, int n_terms, const float * coef, const int * rows, int n_src,
                            int last_is_selected, float * out, void * out_act, int act_dtype, int R, int H, cudaStream_t stream) {
    if (R <= 0) return IIAN_OK;
    if (n_terms <= 0 || n_terms > kMaxMixTerms) return IIAN_ERR_LIMIT;
    MixTerms t;
    for (int j = 0; j < kMaxMixTerms; j++) t.x[j] = j < n_terms ? terms[j] : nullptr;
    const int threads = norm_threads(H);
    bool vec = H % 4 == 0 && ((uintptr_t) out & 15) == 0 && ((uintptr_t) out_act & (act_dtype == IIAN_BF16 ? 7 : 15)) == 0;
    for (int j = 0; j < n_terms; j++) vec = vec && ((uintptr_t) terms[j] & 15) == 0;
    if (vec) {
        const int vt = H >= 2048 ? 256 : 128;
        if (act_dtype == IIAN_F32) return iian_launch(depth_mix_vec_kernel<float>, dim3(R), dim3(vt), 0, stream, t, n_terms, coef, rows, n_src, last_is_selected, out, (float *) out_act, H);
        if (act_dtype == IIAN_BF16) return iian_launch(depth_mix_vec_kernel<__nv_bfloat16>, dim3(R), dim3(vt), 0, stream, t, n_terms, coef, rows, n_src, last_is_selected, out, (__nv_bfloat16 *) out_act, H);
        return IIAN_ERR_DTYPE;
    }
    if (act_dtype == IIAN_F32) return iian_launch(depth_mix_kernel<float>, dim3(R), dim3(threads), 0, stream, t, n_terms, coef, rows, n_src, last_is_selected, out, (float *) out_act, H);
    if (act_dtype == IIAN_BF16) return iian_launch(depth_mix_kernel<__nv_bfloat16>, dim3(R), dim3(threads), 0, stream, t, n_terms, coef, rows, n_src, last_is_selected, out, (__nv_bfloat16 *) out_act, H);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_gated_act_limit(const void * in, long long ld_in, void * out, int act_dtype, int N, int F, int interleave, int act,
                                  float limit, cudaStream_t stream);

// act: 0 silu, 1 gelu (tanh form)
IIAN_API int iian_gated_act(const void * in, long long ld_in, void * out, int act_dtype, int N, int F, int interleave, int act,
                            cudaStream_t stream) {
    if (act != 0 && act != 1) return IIAN_ERR_SHAPE;
    return iian_gated_act_limit(in, ld_in, out, act_dtype, N, F, interleave, act, 0.0f, stream);
}

// act: 0 silu, 1 gelu (tanh form), 2 clamped (takes `limit`)
IIAN_API int iian_gated_act_limit(const void * in, long long ld_in, void * out, int act_dtype, int N, int F, int interleave, int act,
                                  float limit, cudaStream_t stream) {
    if (interleave != 0 && (interleave != 8 || F % 8 != 0)) return IIAN_ERR_SHAPE;
    if (act < 0 || act > 2) return IIAN_ERR_SHAPE;
    const size_t total = (size_t) N * F;
    if (total == 0) return IIAN_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned) ((total + threads - 1) / threads);
    if (act_dtype == IIAN_F32) return iian_launch(gated_act_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float *) in, ld_in, (float *) out, F, total, interleave, act, limit);
    if (act_dtype == IIAN_BF16) return iian_launch(gated_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16 *) in, ld_in, (__nv_bfloat16 *) out, F, total, interleave, act, limit);
    return IIAN_ERR_DTYPE;
}
