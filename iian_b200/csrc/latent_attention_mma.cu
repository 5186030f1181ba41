// Attention over a cached low-rank latent on the tensor cores (bfloat16, mma.sync m16n8k16), for prompts' portions and
// for decoded tokens alike.
//
// All heads of a token score the SAME cached rows (see latent_attention.cu), so the rows of one product are
// (token, head) pairs: a CTA takes up to 32 of them from one sequence (16 in the form for decoded tokens) -- with 16 heads that is two
// tokens, in a decode step all heads of the one token -- and walks the keys they can see in tiles of 64 (32) that start
// at multiples of the tile size of the ABSOLUTE key position (the order of every sum depends on the row's own position only).  Per tile:
//   1. the tile's cache rows come by 16-byte cp.async through the block table into one of two shared-memory stages
//      (rows past the newest key, or in a page that was given back, are zero-filled);
//   2. S = Q K^T: each of the four warps takes 16 of the 64 keys for all rows (Q stays in shared memory; a cache row
//      as stored is the B operand), masks by window and causality per row, and leaves float32 scores in shared memory;
//   3. every warp reads all scores, keeps the running maximum and sum of every row (the sink opens them: maximum
//      sink, sum 1) and forms P = exp(S - max) as its A operand;
//   4. O += P V: each warp owns a quarter of the latent's columns (V is the front of the same cache rows, read
//      transposed by ldmatrix), so the wide output (rank 512: 128 accumulators a thread for 32 rows) fits registers.
// The keys may be cut into parts (gridDim.z, up to 32) for steps with few rows; a part leaves unnormalised sums with
// its maximum and denominator in scratch memory and a second kernel merges them.
#include "common.cuh"

namespace iian {

constexpr int kWarps = 4;
// Two forms.  MT = 2, KEYS = 64: 32 rows a CTA and tiles of 64 keys, for prompts' portions (at the widths of real models one
// CTA holds most of an SM's shared memory).  MT = 1, KEYS = 32: 16 rows and tiles of 32 keys, for decoded tokens: the
// CTA needs under half the shared memory and half the registers, so two or more share an SM and one's waits on
// shared and global memory are covered by the other's products.

__device__ __forceinline__ void cp_async16(void * smem, const void * gmem, bool pred) {
    const unsigned s = (unsigned) __cvta_generic_to_shared(smem);
    const int n = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void * smem) {
    const unsigned s = (unsigned) __cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], const void * smem) {
    const unsigned s = (unsigned) __cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned (&r)[2], const void * smem) {
    const unsigned s = (unsigned) __cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned *>(&v);
}

// NT: n8 tiles of the output a warp owns (rank = 32 * NT); MT: m16 tiles of rows; KEYS: keys per tile (32 or 64).
// q: [N, H, width]; cache: [num_pages * page_size, width]; out: [N, H, rank].
// With gridDim.z > 1: part_o [N * H, parts, rank] f32 (unnormalised), part_ml [N * H, parts, 2] (maximum, denominator).
template <int NT, int MT, int KEYS, int STAGES>
__global__ void __launch_bounds__(kWarps * 32) latent_attention_mma_kernel(
    const __nv_bfloat16 * __restrict__ q, const __nv_bfloat16 * __restrict__ cache, __nv_bfloat16 * __restrict__ out,
    float * __restrict__ part_o, float * __restrict__ part_ml, const float * __restrict__ sink,
    const int * __restrict__ cu_q, const int * __restrict__ ctx_len, const int * __restrict__ block_table, int max_blocks,
    int H, int width, int page_size, int num_pages, float scale, int window) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int rank = 32 * NT;
    constexpr int kRows = 16 * MT, kKeys = KEYS;
    constexpr int NS = KEYS / 32;                         // n8 tiles of the scores a warp computes
    constexpr int KB = KEYS / 16;                         // 16-key blocks of a tile
    const int s = blockIdx.y;
    const int q0 = cu_q[s], q_len = cu_q[s + 1] - q0;
    const int rows_total = q_len * H;
    const int row0 = blockIdx.x * kRows;
    if (row0 >= rows_total) return;
    const int n_rows = min(kRows, rows_total - row0);
    const int ctx = ctx_len[s];
    const int pos0 = ctx - q_len;                         // position of the sequence's first token in this step
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tq = lane & 3;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int ldb = width * 2 + 16;                        // bytes per padded row: rows 4 banks apart
    unsigned char * q_s = smem_raw;                        // [kRows][ldb]
    unsigned char * k_s = q_s + kRows * ldb;               // [STAGES][kKeys][ldb]
    float * s_s = reinterpret_cast<float *>(k_s + STAGES * kKeys * ldb);      // [kRows][kKeys + 4]
    constexpr int lds = kKeys + 4;
    const int chunks = width / 8;                          // 16-byte chunks per row

    // the rows' positions: row r is token (row0 + r) / H of the step, head (row0 + r) % H
    const int t_first = row0 / H, t_last = (row0 + n_rows - 1) / H;
    const int p_first = pos0 + t_first, p_last = pos0 + t_last;
    int lo_all = window > 0 ? max(0, p_first - window + 1) : 0;
    int hi_all = min(p_last, ctx - 1);
    // this CTA's part of the key tiles
    int tile_lo = lo_all / kKeys, tile_hi = hi_all / kKeys;                  // inclusive
    const int parts = gridDim.z;
    if (parts > 1) {
        const int n_tiles = tile_hi - tile_lo + 1;
        const int per = (n_tiles + parts - 1) / parts;
        tile_lo = tile_lo + (int) blockIdx.z * per;
        tile_hi = min(tile_hi, tile_lo + per - 1);
    }

    // Q rows into shared memory (rows past n_rows are zero): a few threads a row, 16-byte chunks interleaved among them
    {
        constexpr int per = kWarps * 32 / kRows;
        const int r = tid / per;
        const bool ok = r < n_rows;
        const int R = row0 + (ok ? r : 0);
        const __nv_bfloat16 * src = q + ((size_t) (q0 + R / H) * H + R % H) * width;
        for (int c = tid % per; c < chunks; c += per) cp_async16(q_s + r * ldb + c * 16, src + c * 8, ok);
    }
    const int * bt = block_table + (size_t) s * max_blocks;
    // a tile's cache rows: a few threads a row (one look-up in the block table each), chunks interleaved among them
    auto load_tile = [&](int tile, int stage) {
        constexpr int per = kWarps * 32 / kKeys;
        unsigned char * dst = k_s + (size_t) stage * kKeys * ldb;
        const int r = tid / per;
        const int j = tile * kKeys + r;
        bool ok = j <= hi_all && j >= 0;
        size_t cell = 0;
        if (ok) {
            const int page = bt[j / page_size];
            ok = page >= 0 && page < num_pages;
            if (ok) cell = (size_t) page * page_size + (j % page_size);
        }
        const __nv_bfloat16 * src = cache + cell * width;
        unsigned char * drow = dst + r * ldb;
        for (int c = tid % per; c < chunks; c += per) cp_async16(drow + c * 16, src + c * 8, ok);
    };
    if (tile_lo <= tile_hi) load_tile(tile_lo, 0);
    cp_async_commit();

    // running softmax state of the rows this thread sees in its fragments: m-tile mt, rows g and g + 8
    float m_run[MT][2], l_run[MT][2];
    int p_row[MT][2], lo_row[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
            const int r = mt * 16 + g + hh * 8;
            const int R = row0 + min(r, n_rows - 1);
            const int p = pos0 + R / H;
            p_row[mt][hh] = r < n_rows ? p : -1;           // a row beyond the end sees nothing
            lo_row[mt][hh] = window > 0 ? max(0, p - window + 1) : 0;
            const bool opens = sink != nullptr && (parts == 1 || blockIdx.z == 0);      // the sink counts once
            m_run[mt][hh] = opens ? sink[R % H] : -INFINITY;
            l_run[mt][hh] = opens ? 1.0f : 0.0f;
        }
    float o_acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) o_acc[mt][nt][e] = 0.0f;

    const int ksteps = width / 16;
    for (int tile = tile_lo; tile <= tile_hi; tile++) {
        const int stage = STAGES == 2 ? (tile - tile_lo) & 1 : 0;
        if (STAGES == 1 && tile > tile_lo) {               // one stage: the next tile may come only when all are done with this one
            __syncthreads();
            load_tile(tile, 0);
            cp_async_commit();
        }
        cp_async_wait<0>();
        __syncthreads();                                   // this tile (and Q) are in shared memory for all; everyone is done with the last tile
        if (STAGES == 2) {
            if (tile + 1 <= tile_hi) load_tile(tile + 1, stage ^ 1);      // arrives while this tile is worked on
            cp_async_commit();
        }
        const unsigned char * kt = k_s + (size_t) stage * kKeys * ldb;
        // ---- S[:, this warp's quarter of the tile's keys] ----
        float sc[MT][NS][4];
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < NS; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) sc[mt][nt][e] = 0.0f;
#pragma unroll 4
        for (int ks = 0; ks < ksteps; ks++) {
            unsigned a[MT][4], b[NS][2];
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
                ldmatrix_x4(a[mt], q_s + (mt * 16 + (lane & 15)) * ldb + (ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int nt = 0; nt < NS; nt++)
                ldmatrix_x2(b[nt], kt + (warp * (8 * NS) + nt * 8 + (lane & 7)) * ldb + (ks * 16 + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int nt = 0; nt < NS; nt++) mma_bf16(sc[mt][nt], a[mt], b[nt]);
        }
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < NS; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int hh = e >> 1;
                    const int col = warp * (8 * NS) + nt * 8 + tq * 2 + (e & 1);
                    const int j = tile * kKeys + col;
                    const bool vis = j <= p_row[mt][hh] && j >= lo_row[mt][hh] && j < ctx;
                    s_s[(mt * 16 + g + hh * 8) * lds + col] = vis ? sc[mt][nt][e] * scale : -INFINITY;
                }
        __syncthreads();
        // ---- softmax over the keys of the tile, per row (every warp does all rows) ----
        unsigned pa[MT][KB][4];                            // P as A fragments: [m-tile][16-key block][4]
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            float v[2][4 * KB];
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const float * srow = s_s + (mt * 16 + g + hh * 8) * lds;
#pragma unroll
                for (int kb = 0; kb < KB; kb++) {
                    const float2 x0 = *reinterpret_cast<const float2 *>(srow + kb * 16 + tq * 2);
                    const float2 x1 = *reinterpret_cast<const float2 *>(srow + kb * 16 + 8 + tq * 2);
                    v[hh][kb * 4 + 0] = x0.x; v[hh][kb * 4 + 1] = x0.y; v[hh][kb * 4 + 2] = x1.x; v[hh][kb * 4 + 3] = x1.y;
                    tmax[hh] = fmaxf(tmax[hh], fmaxf(fmaxf(x0.x, x0.y), fmaxf(x1.x, x1.y)));
                }
                tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 1));
                tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 2));
            }
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const float m_new = fmaxf(m_run[mt][hh], tmax[hh]);
                const float corr = m_run[mt][hh] == -INFINITY ? 0.0f : __expf(m_run[mt][hh] - m_new);
                float psum = 0.0f;
#pragma unroll
                for (int i = 0; i < 4 * KB; i++) {
                    const float p = m_new == -INFINITY ? 0.0f : __expf(v[hh][i] - m_new);
                    v[hh][i] = p;
                    psum += p;
                }
                psum += __shfl_xor_sync(0xffffffffu, psum, 1);
                psum += __shfl_xor_sync(0xffffffffu, psum, 2);
                l_run[mt][hh] = l_run[mt][hh] * corr + psum;
                m_run[mt][hh] = m_new;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    o_acc[mt][nt][hh * 2] *= corr;
                    o_acc[mt][nt][hh * 2 + 1] *= corr;
                }
            }
#pragma unroll
            for (int kb = 0; kb < KB; kb++) {
                pa[mt][kb][0] = pack_bf16(v[0][kb * 4 + 0], v[0][kb * 4 + 1]);     // row g,     keys 2 tq, 2 tq + 1
                pa[mt][kb][1] = pack_bf16(v[1][kb * 4 + 0], v[1][kb * 4 + 1]);     // row g + 8
                pa[mt][kb][2] = pack_bf16(v[0][kb * 4 + 2], v[0][kb * 4 + 3]);     // row g,     keys 8 + 2 tq, ...
                pa[mt][kb][3] = pack_bf16(v[1][kb * 4 + 2], v[1][kb * 4 + 3]);
            }
        }
        // ---- O[:, warp's columns] += P V ----
#pragma unroll
        for (int kb = 0; kb < KB; kb++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                unsigned b[2];
                ldmatrix_x2_trans(b, kt + (kb * 16 + (lane & 15)) * ldb + (warp * (rank / 4) + nt * 8) * 2);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) mma_bf16(o_acc[mt][nt], pa[mt][kb], b);
            }
    }
    cp_async_wait<0>();

    // ---- write ----
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
            const int r = mt * 16 + g + hh * 8;
            if (r >= n_rows) continue;
            const int R = row0 + r;
            const size_t grow = (size_t) (q0 + R / H) * H + R % H;
            if (parts == 1) {
                const float inv = l_run[mt][hh] > 0.0f ? 1.0f / l_run[mt][hh] : 0.0f;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int col = warp * (rank / 4) + nt * 8 + tq * 2;
                    *reinterpret_cast<unsigned *>(out + grow * rank + col) =
                        pack_bf16(o_acc[mt][nt][hh * 2] * inv, o_acc[mt][nt][hh * 2 + 1] * inv);
                }
            } else {
                float * po = part_o + (grow * parts + blockIdx.z) * rank;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int col = warp * (rank / 4) + nt * 8 + tq * 2;
                    *reinterpret_cast<float2 *>(po + col) = make_float2(o_acc[mt][nt][hh * 2], o_acc[mt][nt][hh * 2 + 1]);
                }
                if (warp == 0 && tq == 0) {
                    part_ml[(grow * parts + blockIdx.z) * 2] = m_run[mt][hh];
                    part_ml[(grow * parts + blockIdx.z) * 2 + 1] = l_run[mt][hh];
                }
            }
        }
}

// out[row] = sum_z o_z exp(m_z - m) / sum_z l_z exp(m_z - m),  z ascending
__global__ void latent_merge_kernel(const float * __restrict__ part_o, const float * __restrict__ part_ml,
                                    __nv_bfloat16 * __restrict__ out, const int * __restrict__ seq_of_token, int H, int parts,
                                    int rank) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float wz[64];                  // the weight of every part: exp(m_z - m) / l
    const size_t row = blockIdx.x;
    if (seq_of_token[row / H] < 0) {
        for (int c = threadIdx.x; c < rank; c += blockDim.x) out[row * rank + c] = __float2bfloat16_rn(0.0f);
        return;
    }
    if (threadIdx.x < 32) {
        const int z = threadIdx.x;
        const float mz = z < parts ? part_ml[(row * parts + z) * 2] : -INFINITY;
        const float lz = z < parts ? part_ml[(row * parts + z) * 2 + 1] : 0.0f;
        const float m = warp_max(mz);
        const float e = mz == -INFINITY ? 0.0f : __expf(mz - m);
        float l = lz * e;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {     // in the order of the parts: a prefix-style sum keeps z ascending pairs together
            l += __shfl_xor_sync(0xffffffffu, l, o);
        }
        wz[z] = l > 0.0f ? e / l : 0.0f;
    }
    __syncthreads();
    const float * po = part_o + row * parts * rank;
    for (int c = threadIdx.x * 2; c < rank; c += blockDim.x * 2) {
        float a0 = 0.0f, a1 = 0.0f;
        for (int z = 0; z < parts; z++) {
            const float2 v = *reinterpret_cast<const float2 *>(po + (size_t) z * rank + c);
            a0 = fmaf(v.x, wz[z], a0);
            a1 = fmaf(v.y, wz[z], a1);
        }
        *reinterpret_cast<unsigned *>(out + row * rank + c) = pack_bf16(a0, a1);
    }
}

}  // namespace iian

using namespace iian;

static size_t latent_mma_smem(int width, int rows, int keys, int stages = 2) {
    const size_t ldb = (size_t) width * 2 + 16;
    return rows * ldb + stages * keys * ldb + (size_t) rows * (keys + 4) * sizeof(float);
}

// the form for prompts' portions: 0 = 32 rows, tiles of 64 keys in two stages (one CTA an SM at width 576);
// 1 = 32 rows, tiles of 32 keys in one stage (two CTAs an SM, each covers the other's loads)
static int g_large_form = 1;
IIAN_API int iian_latent_attention_large_form(int form) {
    if (form != 0 && form != 1) return IIAN_ERR_SHAPE;
    g_large_form = form;
    return IIAN_OK;
}
// the form for decoded tokens (16 rows, tiles of 32 keys): 0 = two stages (two CTAs an SM at width 576), 1 = one stage (three)
static int g_small_form = 0;
IIAN_API int iian_latent_attention_small_form(int form) {
    if (form != 0 && form != 1) return IIAN_ERR_SHAPE;
    g_small_form = form;
    return IIAN_OK;
}

// 0 if the sizes are ones this kernel takes
IIAN_API int iian_latent_attention_mma_ok(int rank, int width, int H) {
    if (rank != 64 && rank != 128 && rank != 256 && rank != 512) return IIAN_ERR_SHAPE;
    if (width < rank || width % 16 != 0 || H <= 0) return IIAN_ERR_SHAPE;
    if (latent_mma_smem(width, 32, 64) > 220 * 1024) return IIAN_ERR_LIMIT;
    return IIAN_OK;
}

template <int NT, int MT, int KEYS, int STAGES>
static int launch_latent_mma(const void * q, const void * cache, void * out, float * part_o, float * part_ml, const float * sink,
                             const int * cu_q, const int * ctx_len, const int * block_table, int max_blocks, int S, int max_q_len,
                             int H, int width, int page_size, int num_pages, float scale, int window, int parts, cudaStream_t stream) {
    const size_t smem = latent_mma_smem(width, 16 * MT, KEYS, STAGES);
    static size_t attr_done = 0;
    if (smem > attr_done) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<NT, MT, KEYS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return 1000 + (int) e;
        attr_done = smem;
    }
    const long long tiles = ((long long) max_q_len * H + 16 * MT - 1) / (16 * MT);
    if (tiles > 2147483647LL || S > 65535 || parts > 32) return IIAN_ERR_LIMIT;
    return iian_launch(latent_attention_mma_kernel<NT, MT, KEYS, STAGES>, dim3((unsigned) tiles, S, parts), dim3(kWarps * 32), smem, stream,
                       (const __nv_bfloat16 *) q, (const __nv_bfloat16 *) cache, (__nv_bfloat16 *) out, part_o, part_ml, sink, cu_q,
                       ctx_len, block_table, max_blocks, H, width, page_size, num_pages, scale, window);
}

// q: [N, H, width] bf16; cache: [num_pages * page_size, width] bf16; out: [N, H, rank] bf16; sink f32 [H] or null.
// parts > 1: part_o f32 [N * H * parts * rank], part_ml f32 [N * H * parts * 2] and seq_of_token are needed.
IIAN_API int iian_latent_attention_mma(const void * q, const void * cache, void * out, float * part_o, float * part_ml,
                                       const float * sink, const int * cu_q, const int * ctx_len, const int * seq_of_token,
                                       const int * block_table, int max_blocks, int N, int S, int max_q_len, int H, int rank,
                                       int width, int page_size, int num_pages, float scale, int window, int parts,
                                       cudaStream_t stream) {
    if (N <= 0 || S <= 0) return IIAN_OK;
    int code = iian_latent_attention_mma_ok(rank, width, H);
    if (code != IIAN_OK) return code;
    if (parts < 1 || (parts > 1 && (part_o == nullptr || part_ml == nullptr || seq_of_token == nullptr))) return IIAN_ERR_SHAPE;
    if (((uintptr_t) q & 15) || ((uintptr_t) cache & 15) || ((uintptr_t) out & 3)) return IIAN_ERR_ALIGN;
    // decoded tokens (and any step whose sequences bring at most 16 rows): the form of which several CTAs share an SM
    const bool small = (long long) max_q_len * H <= 16 || max_q_len == 1;
#define IIAN_LAT(NTV)                                                                                                        \
    code = small ? (g_small_form == 1                                                                                           \
                    ? launch_latent_mma<NTV, 1, 32, 1>(q, cache, out, part_o, part_ml, sink, cu_q, ctx_len, block_table, max_blocks, S, \
                                                       max_q_len, H, width, page_size, num_pages, scale, window, parts, stream) \
                    : launch_latent_mma<NTV, 1, 32, 2>(q, cache, out, part_o, part_ml, sink, cu_q, ctx_len, block_table, max_blocks, S, \
                                                       max_q_len, H, width, page_size, num_pages, scale, window, parts, stream)) \
         : g_large_form == 1 ? launch_latent_mma<NTV, 2, 32, 1>(q, cache, out, part_o, part_ml, sink, cu_q, ctx_len, block_table, max_blocks, S, \
                                                    max_q_len, H, width, page_size, num_pages, scale, window, parts, stream) \
                 : launch_latent_mma<NTV, 2, 64, 2>(q, cache, out, part_o, part_ml, sink, cu_q, ctx_len, block_table, max_blocks, S, \
                                                    max_q_len, H, width, page_size, num_pages, scale, window, parts, stream)
    if (rank == 64) IIAN_LAT(2);
    else if (rank == 128) IIAN_LAT(4);
    else if (rank == 256) IIAN_LAT(8);
    else IIAN_LAT(16);
#undef IIAN_LAT
    if (code != IIAN_OK || parts == 1) return code;
    return iian_launch(latent_merge_kernel, dim3((unsigned) ((size_t) N * H)), dim3(rank >= 256 ? 128 : 64), 0, stream,
                       (const float *) part_o, (const float *) part_ml, (__nv_bfloat16 *) out, seq_of_token, H, parts, rank);
}
