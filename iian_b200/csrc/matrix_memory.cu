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
// lanes per column holds that column (and a copy of n) in registers.  The gates do not depend on C, so one more warp (the
// gate warp) runs their chain (m, the two decays, exp(-m)) a chunk of tokens ahead of the others and leaves them in
// shared memory; loader threads fetch the next chunk's q, k and v rows and put them there while the column holders work
// on the current chunk out of shared memory: a step's loads never lie on the chain from token to token.  A step then costs d / R fused multiply-adds times four per lane and two sums over R lanes by shuffles.
// Every CTA of a (sequence, head) keeps its own copy of n and m in the state (a column block is `cb * d` floats of C
// column by column, then d floats of n, then m, padded to a multiple of 4), so no CTA reads what another writes.
// Gates, decays, state and sums are float32 whatever the activation type; the order of every sum is fixed by (d, R)
// alone and the chain of m is the same whatever the chunks are, so a sequence's results do not depend on how it was cut
// into steps or on what else is in the batch.
#include "common.cuh"

namespace iian {

__device__ __forceinline__ float log_sigmoid_f32(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

constexpr int kMemPrefetch = 40;        // elements of the next chunk a thread holds in registers at most (long form)
constexpr int kMemPrefetchShort = 4;    // the same in the form for steps of single tokens (chunks of one token)
constexpr unsigned kMemTokShift = 27, kMemIsQ = 1u << 26, kMemSkip = 0xffffffffu;

// proj: rows [.. q (heads x d) .. k (heads x d) .. v (heads x dv) ..] at column offsets q_off, k_off, v_off, row stride ld
// gates: f32 [N, 2 heads]: z_i of every head, then z_f; gate_bias alike
// state: f32 [slots, heads, nblk, block_floats]; out: f32 [N, heads * dv]
// V: elements a lane holds side by side (4 when d is a multiple of 4: 16-byte accesses to the state and to shared memory)
// PF: registers for the next chunk's rows; U: tokens whose read-outs (two sums over the lanes, a division, a store) are
// issued together -- only the update of C and n is a chain from token to token, one multiply-add deep, and the
// read-outs of U tokens overlap each other and the next tokens' updates.  (PF, U) = (40, 4) for portions of prompts,
// (4, 1) with chunks of one token for steps of single tokens: fewer registers, more CTAs on an SM.
template <typename A, int MAXE, int R, int V, int PF, int U, bool LOADERS>
__global__ void __launch_bounds__(288) matrix_memory_scan_kernel(
    const A * __restrict__ proj, long long ld, int q_off, int k_off, int v_off, const float * __restrict__ gates,
    const float * __restrict__ gate_bias, float * __restrict__ state, const int * __restrict__ cu_q,
    const int * __restrict__ state_slots, float * __restrict__ out, int heads, int d, int dv, int cb, int block_floats,
    float cap, float q_scale, int chunk) {
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    const int blk = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int nblk = gridDim.x;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    const int slot = state_slots[seq];
    const int tid = threadIdx.x;
    // Roles: the threads that hold columns; one gate warp; and, with LOADERS (portions, up to 128 column holders), as many
    // loader threads as column holders, which fetch and put down the next chunk so that the column holders do nothing but
    // the recurrence.  Without them the column holders fetch their own rows (the form for single tokens: fewer threads,
    // more CTAs on an SM; and CTAs of 256 column holders).
    const int n_cons = LOADERS ? (blockDim.x - 32) / 2 : blockDim.x - 32;
    const bool gate_warp = tid >= n_cons && tid < n_cons + 32;
    const bool loader = LOADERS ? tid >= n_cons + 32 : tid < n_cons;     // who fetches
    const int ltid = LOADERS ? tid - n_cons - 32 : tid;                  // its index among those who fetch
    const int r = tid % R;
    int c = tid / R;
    const bool owner = tid < n_cons && c < cb && r == 0;
    const bool holds = tid < n_cons && c < cb;
    if (c >= cb) c = cb - 1;          // lanes beyond the block's columns repeat its last one and store nothing
    const int col = blk * cb + c;
    if (slot < 0) {                   // a padding sequence: no state, zeros out
        if (owner)
            for (int t = t0; t < t1; t++) out[(size_t) t * heads * dv + head * dv + col] = 0.0f;
        return;
    }
    if (t1 <= t0) return;
    const int rowp = (2 * d + cb + 3) / 4 * 4;           // floats of a token in shared memory: q, k, the block's v
    const int total = chunk * rowp;
    unsigned * tab = reinterpret_cast<unsigned *>(sm);   // [total]: where each of them comes from
    float * buf0 = sm + total;                            // two buffers of [chunk][rowp] rows (q, k, v as projected) and [chunk][4] gate values
    const int buf_floats = total + chunk * 4;
    for (int idx = tid; idx < total; idx += blockDim.x) {
        const int tt = chunk == 1 ? 0 : idx / rowp, cc = idx - tt * rowp;
        unsigned e = kMemSkip;
        if (cc < d) e = ((unsigned) tt << kMemTokShift) | kMemIsQ | (unsigned) (q_off + head * d + cc);
        else if (cc < 2 * d) e = ((unsigned) tt << kMemTokShift) | (unsigned) (k_off + head * d + cc - d);
        else if (cc < 2 * d + cb) e = ((unsigned) tt << kMemTokShift) | (unsigned) (v_off + head * dv + blk * cb + cc - 2 * d);
        tab[idx] = e;
    }
    float * sb = state + (((size_t) slot * heads + head) * nblk + blk) * block_floats;
    float C[MAXE], n[MAXE];
    float m = 0.0f;
    if (tid < n_cons) {
#pragma unroll
        for (int g = 0; g < MAXE / V; g++) {
            const int e0 = (g * R + r) * V;
            if (V == 4) {
                const bool in = e0 < d;                  // loads from a valid address either way: all of them in flight at once
                float4 cv = *reinterpret_cast<const float4 *>(sb + (size_t) c * d + (in ? e0 : 0));
                float4 nv = *reinterpret_cast<const float4 *>(sb + (size_t) cb * d + (in ? e0 : 0));
                if (!in) cv = nv = make_float4(0.f, 0.f, 0.f, 0.f);
                C[g * V] = cv.x; C[g * V + 1 % V] = cv.y; C[g * V + 2 % V] = cv.z; C[g * V + 3 % V] = cv.w;
                n[g * V] = nv.x; n[g * V + 1 % V] = nv.y; n[g * V + 2 % V] = nv.z; n[g * V + 3 % V] = nv.w;
            } else {
                const float cv = sb[(size_t) c * d + (e0 < d ? e0 : 0)], nv = sb[(size_t) cb * d + (e0 < d ? e0 : 0)];
                C[g] = e0 < d ? cv : 0.0f;
                n[g] = e0 < d ? nv : 0.0f;
            }
        }
    } else if (gate_warp) {
        m = sb[(size_t) (cb + 1) * d];
    }
    const float bias_i = gate_bias[head], bias_f = gate_bias[heads + head];
    __syncthreads();                  // the table is whole; every warp has read its part of the state

    float pf[PF];
    unsigned long long pf_ok = 0ull;
    // What the threads that hold columns do for the chunk that begins at token tc: fetch into registers ...  Every load is
    // issued whether its value is wanted or not (from a valid address, chosen without a branch), so that all of them are
    // in flight together; what was not wanted becomes zero when the values are put into shared memory.
    auto fetch = [&](int tc) {
        const int ntok = min(chunk, t1 - tc);
        const size_t safe = (size_t) tc * ld + (size_t) (q_off + head * d);
        pf_ok = 0ull;
#pragma unroll
        for (int k = 0; k < PF; k++) {
            const int want = ltid + k * n_cons;
            const unsigned e = tab[min(want, total - 1)];
            const int tt = (int) (e >> kMemTokShift);
            const bool ok = want < total && e != kMemSkip && tt < ntok;
            const size_t off = ok ? (size_t) (tc + tt) * ld + (e & (kMemIsQ - 1)) : safe;
            pf[k] = to_f32(proj[off]);
            pf_ok |= ok ? (1ull << k) : 0ull;
        }
    };
    // ... and put them into a buffer
    auto stash = [&](float * buf) {
#pragma unroll
        for (int k = 0; k < PF; k++) {
            const int idx = ltid + k * n_cons;
            if (idx < total) buf[idx] = ((pf_ok >> k) & 1ull) ? pf[k] : 0.0f;
        }
    };
    // what the gate warp does for that chunk: the gates of its tokens side by side, then the chain of m token by token
    auto gate_chain = [&](int tc, float * buf) {
        const int lane = tid - n_cons;
        const int ntok = min(chunk, t1 - tc);
        float a = 0.0f, b = 0.0f;
        if (lane < ntok) {
            const size_t t = (size_t) (tc + lane);
            a = cap * tanhf((gates[t * 2 * heads + head] + bias_i) / cap);
            b = log_sigmoid_f32(cap * tanhf((gates[t * 2 * heads + heads + head] + bias_f) / cap));
        }
        for (int tt = 0; tt < ntok; tt++) {
            const float at = __shfl_sync(0xffffffffu, a, tt), bt = __shfl_sync(0xffffffffu, b, tt);
            const float m_new = fmaxf(bt + m, at);
            const float keep = expf(bt + m - m_new), take = expf(at - m_new);
            m = m_new;
            if (lane == 0) *reinterpret_cast<float4 *>(buf + total + tt * 4) = make_float4(keep, take, expf(-m), 0.0f);
        }
    };

    if (gate_warp) gate_chain(t0, buf0);
    else if (loader) { fetch(t0); stash(buf0); }
    __syncthreads();
    int which = 0;
    for (int tc = t0; tc < t1; tc += chunk, which ^= 1) {
        float * cur = buf0 + which * buf_floats;
        float * nxt = buf0 + (which ^ 1) * buf_floats;
        const bool more = tc + chunk < t1;
        if (gate_warp) {
            if (more) gate_chain(tc + chunk, nxt);
        } else if (LOADERS && loader) {
            if (more) { fetch(tc + chunk); stash(nxt); }
        } else {
            if (!LOADERS && more) fetch(tc + chunk);
            const int ntok = min(chunk, t1 - tc);
            for (int tt0 = 0; tt0 < ntok; tt0 += U) {
                float num[U], den[U], floor_[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int tt = tt0 + u;
                    const bool live = tt < ntok;                 // a token beyond the chunk: keep 1, take 0 change nothing
                    const float * row = cur + (live ? tt : 0) * rowp;
                    const float4 gk = live ? *reinterpret_cast<const float4 *>(cur + total + tt * 4) : make_float4(1.0f, 0.0f, 1.0f, 0.0f);
                    const float keep = gk.x, take = gk.y;
                    floor_[u] = gk.z;
                    const float tv = take * row[2 * d + c];
                    float ps[4] = {0.0f, 0.0f, 0.0f, 0.0f}, pd[4] = {0.0f, 0.0f, 0.0f, 0.0f};     // sums in four parts, in a fixed order
#pragma unroll
                    for (int g = 0; g < MAXE / V; g++) {
                        const int e0 = (g * R + r) * V;
                        float qv[V], kv[V];
                        if (V == 4) {
                            const bool in = e0 < d;
                            const float4 q4 = in ? *reinterpret_cast<const float4 *>(row + e0) : make_float4(0.f, 0.f, 0.f, 0.f);
                            const float4 k4 = in ? *reinterpret_cast<const float4 *>(row + d + e0) : make_float4(0.f, 0.f, 0.f, 0.f);
                            qv[0] = q4.x; qv[1 % V] = q4.y; qv[2 % V] = q4.z; qv[3 % V] = q4.w;
                            kv[0] = k4.x; kv[1 % V] = k4.y; kv[2 % V] = k4.z; kv[3 % V] = k4.w;
                        } else {
                            qv[0] = e0 < d ? row[e0] : 0.0f;
                            kv[0] = e0 < d ? row[d + e0] : 0.0f;
                        }
#pragma unroll
                        for (int j = 0; j < V; j++) {
                            const int i = g * V + j;
                            C[i] = fmaf(keep, C[i], tv * kv[j]);
                            n[i] = fmaf(keep, n[i], take * kv[j]);
                            ps[i & 3] = fmaf(C[i], qv[j], ps[i & 3]);
                            pd[i & 3] = fmaf(n[i], qv[j], pd[i & 3]);
                        }
                    }
                    num[u] = ((ps[0] + ps[1]) + (ps[2] + ps[3])) * q_scale;      // q enters both sums once: its scale is applied here
                    den[u] = ((pd[0] + pd[1]) + (pd[2] + pd[3])) * q_scale;
                }
#pragma unroll
                for (int o = R / 2; o > 0; o >>= 1) {
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        num[u] += __shfl_xor_sync(0xffffffffu, num[u], o);
                        den[u] += __shfl_xor_sync(0xffffffffu, den[u], o);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; u++)
                    if (owner && tt0 + u < ntok)
                        out[(size_t) (tc + tt0 + u) * heads * dv + head * dv + col] = num[u] / (fmaxf(fabsf(den[u]), floor_[u]) + 1e-6f);
            }
            if (!LOADERS && more) stash(nxt);
        }
        __syncthreads();
    }
    if (holds) {
#pragma unroll
        for (int g = 0; g < MAXE / V; g++) {
            const int e0 = (g * R + r) * V;
            if (e0 >= d) continue;
            if (V == 4) {
                *reinterpret_cast<float4 *>(sb + (size_t) c * d + e0) = make_float4(C[g * V], C[g * V + 1 % V], C[g * V + 2 % V], C[g * V + 3 % V]);
                if (c == 0)
                    *reinterpret_cast<float4 *>(sb + (size_t) cb * d + e0) = make_float4(n[g * V], n[g * V + 1 % V], n[g * V + 2 % V], n[g * V + 3 % V]);
            } else {
                sb[(size_t) c * d + e0] = C[g];
                if (c == 0) sb[(size_t) cb * d + e0] = n[g];
            }
        }
    }
    if (tid == n_cons) sb[(size_t) (cb + 1) * d] = m;
}

}  // namespace iian

using namespace iian;

// floats of one column block of the state for memories of d rows cut into blocks of cb columns
IIAN_API int iian_matrix_memory_block_floats(int d, int cb) { return ((cb + 1) * d + 1 + 3) / 4 * 4; }

// lanes that share a column: 8 up to d = 128, 16 up to 256, 32 beyond (16 lanes at d = 128 -- eight working warps with half
// the elements each -- measured slower: 0.94 against 0.87 ms for 2,048 tokens); at most 256 threads of a CTA hold columns,
// so cb * lanes <= 256
IIAN_API int iian_matrix_memory_lanes(int d) { return d <= 128 ? 8 : d <= 256 ? 16 : 32; }

// Which form portions of prompts take: 1 with loader warps, 2 without, 0 (default) chosen by the launch: with loader warps a
// CTA has 288 threads of 168 registers and an SM holds one; without, 160 threads and an SM holds two.  Loader warps win
// while there is at most one CTA per SM to run (0.58 against 0.87 ms for 128 CTAs); beyond that two CTAs per SM do.
static int g_mm_form = 0;
IIAN_API int iian_matrix_memory_form(int form) {
    if (form < 0 || form > 2) return IIAN_ERR_SHAPE;
    g_mm_form = form;
    return IIAN_OK;
}

static int mm_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    return sms;
}

IIAN_API int iian_matrix_memory_scan(const void * proj, long long ld, int q_off, int k_off, int v_off, const float * gates,
                                     const float * gate_bias, float * state, const int * cu_q, const int * state_slots,
                                     float * out, int act_dtype, int num_seqs, int heads, int d, int dv, int cb, float cap,
                                     float q_scale, int max_q_len, cudaStream_t stream) {
    // max_q_len: the most tokens a sequence brings, a hint (1: the form for single tokens; any form is right for any step)
    if (num_seqs <= 0) return IIAN_OK;
    if (heads <= 0 || d <= 0 || dv <= 0 || cb <= 0 || dv % cb != 0 || d > 512 || heads > 65535 || num_seqs > 65535) return IIAN_ERR_SHAPE;
    if (ld <= 0 || ld >= (1LL << 26)) return IIAN_ERR_LIMIT;          // column offsets are kept in 26 bits
    const int bf = iian_matrix_memory_block_floats(d, cb);
    const int lanes = iian_matrix_memory_lanes(d);
    const int n_cons = (cb * lanes + 31) / 32 * 32;
    if (n_cons > 256) return IIAN_ERR_SHAPE;
    const int rowp = (2 * d + cb + 3) / 4 * 4;
    const bool short_form = max_q_len == 1 && (rowp + n_cons - 1) / n_cons <= kMemPrefetchShort;
    int chunk = short_form ? 1 : 16;      // tokens a chunk holds: as many as the threads can keep in flight in registers
    while (chunk > 1 && (chunk * rowp + n_cons - 1) / n_cons > kMemPrefetch) chunk /= 2;
    if ((chunk * rowp + n_cons - 1) / n_cons > kMemPrefetch) return IIAN_ERR_SHAPE;
    const size_t smem = ((size_t) chunk * rowp + 2 * ((size_t) chunk * rowp + chunk * 4)) * sizeof(float);
    dim3 grid(dv / cb, heads, num_seqs);
    const long long ctas = (long long) (dv / cb) * heads * num_seqs;
    const bool with_loaders = n_cons <= 128 && (g_mm_form == 1 || (g_mm_form == 0 && ctas <= mm_sm_count()));
    typedef __nv_bfloat16 bf16;
#define IIAN_MM(AT, MAXE, R, V)                                                                                                   \
    do {                                                                                                                          \
        if (short_form) IIAN_MM_FORM(AT, MAXE, R, V, kMemPrefetchShort, 1, false);                                                \
        if (with_loaders) IIAN_MM_FORM(AT, MAXE, R, V, kMemPrefetch, 4, true);                                                    \
        IIAN_MM_FORM(AT, MAXE, R, V, kMemPrefetch, 4, false);                                                                     \
    } while (0)
#define IIAN_MM_FORM(AT, MAXE, R, V, PF, U, LD)                                                                                   \
    do {                                                                                                                          \
        auto kernel = matrix_memory_scan_kernel<AT, MAXE, R, V, PF, U, LD>;                                                       \
        static size_t configured = 48 * 1024;                                                                                     \
        if (smem > configured) {                                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);                \
            if (e != cudaSuccess) return 1000 + (int) e;                                                                          \
            configured = smem;                                                                                                    \
        }                                                                                                                         \
        return iian_launch(kernel, grid, dim3((LD ? 2 * n_cons : n_cons) + 32), smem, stream, (const AT *) proj, ld, q_off, k_off, v_off, gates,      \
                           gate_bias, state, cu_q, state_slots, out, heads, d, dv, cb, bf, cap, q_scale, chunk);                  \
    } while (0)
#define IIAN_MM_SIZES(AT)                                       \
    do {                                                        \
        if (d % 4 == 0) {                                       \
            if (d <= 32) IIAN_MM(AT, 4, 8, 4);                  \
            if (d <= 64) IIAN_MM(AT, 8, 8, 4);                  \
            if (d <= 128) IIAN_MM(AT, 16, 8, 4);                \
            if (d <= 256) IIAN_MM(AT, 16, 16, 4);               \
            IIAN_MM(AT, 16, 32, 4);                             \
        }                                                       \
        if (d <= 32) IIAN_MM(AT, 4, 8, 1);                      \
        if (d <= 64) IIAN_MM(AT, 8, 8, 1);                      \
        if (d <= 128) IIAN_MM(AT, 16, 8, 1);                    \
        if (d <= 256) IIAN_MM(AT, 16, 16, 1);                   \
        IIAN_MM(AT, 16, 32, 1);                                 \
    } while (0)
    if (act_dtype == IIAN_F32) IIAN_MM_SIZES(float);
    if (act_dtype == IIAN_BF16) IIAN_MM_SIZES(bf16);
#undef IIAN_MM_SIZES
#undef IIAN_MM
#undef IIAN_MM_FORM
    return IIAN_ERR_DTYPE;
}
