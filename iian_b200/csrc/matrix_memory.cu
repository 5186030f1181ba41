// The matrix-memory recurrence (mLSTM): a step's tokens of every sequence walked in order, from the state the steps
// before left in the sequence's slot and back into it.
//
// Per head a memory C [d, dv], a normaliser n [d] and a running maximum m that starts at zero.  With the log input
// gate a_t = cap tanh((z_i + b_i) / cap) and the log forget gate b_t = logsigmoid(cap tanh((z_f + b_f) / cap)):
//
//     m_t = max(b_t + m_{t-1}, a_t)
//     C_t = exp(b_t + m_{t-1} - m_t) C_{t-1} + exp(a_t - m_t) k_t v_t^T          n_t alike with k_t alone
//     o_t = C_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// The columns of C are independent of one another, so a CTA owns `cb` of them for one (sequence, head): a group of R
// lanes per column holds that column (and a copy of n) in registers, element e on lane e % R.  A step needs no
// shared memory and no barrier: two sums over the R lanes by shuffles.  Every CTA of a (sequence, head) keeps its own
// copy of n and m in the state (a column block is `cb * d` floats of C column by column, then d floats of n, then m,
// padded to a multiple of 4), so no CTA reads what another writes.  Gates, decays, state and sums are float32 whatever
// the activation type; the order of every sum is fixed by (d, R) alone, so a sequence's results do not depend on how
// it was cut into steps or on what else is in the batch.
#include "common.cuh"

namespace iian {

__device__ __forceinline__ float log_sigmoid_f32(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

// proj: rows [.. q (heads x d) .. k (heads x d) .. v (heads x dv) ..] at column offsets q_off, k_off, v_off, row stride ld
// gates: f32 [N, 2 heads]: z_i of every head, then z_f; gate_bias alike
// state: f32 [slots, heads, nblk, block_floats]; out: f32 [N, heads * dv]
template <typename A, int MAXE, int R>
__global__ void __launch_bounds__(256) matrix_memory_scan_kernel(
    const A * __restrict__ proj, long long ld, int q_off, int k_off, int v_off, const float * __restrict__ gates,
    const float * __restrict__ gate_bias, float * __restrict__ state, const int * __restrict__ cu_q,
    const int * __restrict__ state_slots, float * __restrict__ out, int heads, int d, int dv, int cb, int block_floats,
    float cap, float q_scale) {
    pdl_wait();
    const int blk = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int nblk = gridDim.x;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    const int slot = state_slots[seq];
    const int r = threadIdx.x % R;
    int c = threadIdx.x / R;
    const bool owner = c < cb && r == 0;
    if (c >= cb) c = cb - 1;          // lanes beyond the block's columns repeat its last one and store nothing
    const int col = blk * cb + c;
    if (slot < 0) {                   // a padding sequence: no state, zeros out
        if (owner)
            for (int t = t0; t < t1; t++) out[(size_t) t * heads * dv + head * dv + col] = 0.0f;
        return;
    }
    float * sb = state + (((size_t) slot * heads + head) * nblk + blk) * block_floats;
    float C[MAXE], n[MAXE];
#pragma unroll
    for (int i = 0; i < MAXE; i++) {
        const int e = i * R + r;
        C[i] = e < d ? sb[(size_t) c * d + e] : 0.0f;
        n[i] = e < d ? sb[(size_t) cb * d + e] : 0.0f;
    }
    float m = sb[(size_t) (cb + 1) * d];
    __syncthreads();                  // every warp has read n and m before the first one writes them back
    const float bias_i = gate_bias[head], bias_f = gate_bias[heads + head];

    for (int t = t0; t < t1; t++) {
        const A * row = proj + (size_t) t * ld;
        const float zi = gates[(size_t) t * 2 * heads + head] + bias_i;
        const float zf = gates[(size_t) t * 2 * heads + heads + head] + bias_f;
        const float vj = to_f32(row[v_off + head * dv + col]);
        float qv[MAXE], kv[MAXE];
#pragma unroll
        for (int i = 0; i < MAXE; i++) {
            const int e = i * R + r;
            qv[i] = e < d ? to_f32(row[q_off + head * d + e]) * q_scale : 0.0f;
            kv[i] = e < d ? to_f32(row[k_off + head * d + e]) : 0.0f;
        }
        const float a = cap * tanhf(zi / cap);
        const float b = log_sigmoid_f32(cap * tanhf(zf / cap));
        const float m_new = fmaxf(b + m, a);
        const float keep = expf(b + m - m_new);
        const float take = expf(a - m_new);
        const float tv = take * vj;
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int i = 0; i < MAXE; i++) {
            C[i] = fmaf(keep, C[i], tv * kv[i]);
            n[i] = fmaf(keep, n[i], take * kv[i]);
            num = fmaf(C[i], qv[i], num);
            den = fmaf(n[i], qv[i], den);
        }
#pragma unroll
        for (int o = R / 2; o > 0; o >>= 1) {
            num += __shfl_xor_sync(0xffffffffu, num, o);
            den += __shfl_xor_sync(0xffffffffu, den, o);
        }
        m = m_new;
        if (owner) out[(size_t) t * heads * dv + head * dv + col] = num / (fmaxf(fabsf(den), expf(-m)) + 1e-6f);
    }
    if (t1 > t0 && threadIdx.x / R < cb) {
#pragma unroll
        for (int i = 0; i < MAXE; i++) {
            const int e = i * R + r;
            if (e < d) {
                sb[(size_t) c * d + e] = C[i];
                if (c == 0) sb[(size_t) cb * d + e] = n[i];
            }
        }
        if (threadIdx.x == 0) sb[(size_t) (cb + 1) * d] = m;
    }
}

}  // namespace iian

using namespace iian;

// floats of one column block of the state for memories of d rows cut into blocks of cb columns
IIAN_API int iian_matrix_memory_block_floats(int d, int cb) { return ((cb + 1) * d + 1 + 3) / 4 * 4; }

// lanes that share a column: 8 up to d = 128, 16 up to 256, 32 beyond; a CTA has at most 256 threads, so cb * lanes <= 256
IIAN_API int iian_matrix_memory_lanes(int d) { return d <= 128 ? 8 : d <= 256 ? 16 : 32; }

IIAN_API int iian_matrix_memory_scan(const void * proj, long long ld, int q_off, int k_off, int v_off, const float * gates,
                                     const float * gate_bias, float * state, const int * cu_q, const int * state_slots,
                                     float * out, int act_dtype, int num_seqs, int heads, int d, int dv, int cb, float cap,
                                     float q_scale, cudaStream_t stream) {
    if (num_seqs <= 0) return IIAN_OK;
    if (heads <= 0 || d <= 0 || dv <= 0 || cb <= 0 || dv % cb != 0 || d > 512 || heads > 65535 || num_seqs > 65535) return IIAN_ERR_SHAPE;
    const int bf = iian_matrix_memory_block_floats(d, cb);
    dim3 grid(dv / cb, heads, num_seqs);
    typedef __nv_bfloat16 bf16;
#define IIAN_MM(AT, MAXE, R)                                                                                                     \
    do {                                                                                                                         \
        const int threads = (cb * R + 31) / 32 * 32;                                                                             \
        if (threads > 256) return IIAN_ERR_SHAPE;                                                                                \
        return iian_launch(matrix_memory_scan_kernel<AT, MAXE, R>, grid, dim3(threads), 0, stream, (const AT *) proj, ld, q_off, \
                           k_off, v_off, gates, gate_bias, state, cu_q, state_slots, out, heads, d, dv, cb, bf, cap, q_scale);    \
    } while (0)
#define IIAN_MM_SIZES(AT)                       \
    do {                                        \
        if (d <= 32) IIAN_MM(AT, 4, 8);         \
        if (d <= 64) IIAN_MM(AT, 8, 8);         \
        if (d <= 128) IIAN_MM(AT, 16, 8);       \
        if (d <= 256) IIAN_MM(AT, 16, 16);      \
        IIAN_MM(AT, 16, 32);                    \
    } while (0)
    if (act_dtype == IIAN_F32) IIAN_MM_SIZES(float);
    if (act_dtype == IIAN_BF16) IIAN_MM_SIZES(bf16);
#undef IIAN_MM_SIZES
#undef IIAN_MM
    return IIAN_ERR_DTYPE;
}
