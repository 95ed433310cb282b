// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16),
// compiled for one head size (MLS_HEAD_DIM, a multiple of 16).
//
// Reference math (train/model.py:55-70): S = (q . k) * scale, key j hidden from
// the query at absolute position p iff j > p (or j <= p - window); softmax and
// P . V with float32 scores, maxima, sums and accumulators; P is rounded to
// bfloat16 for the second product, as in the reference's prefill kernel
// (kernels/attention_fwd.py:106).  Pages are walked through the block table as
// in its decode kernel (kernels/paged_attention.py:60-66).
//
// Rows of a tile are (token, head-in-group) pairs of ONE kv head, so the keys and
// values of a kv head are loaded once for all G query heads that share it.
//
//  attention_tile_kernel   64 rows per CTA, 16 per warp: prompts and portions.
//  attention_split_kernel  up to 16 rows per CTA (single decoded tokens, portions
//                          of a few tokens), the keys of a tile split over the 4
//                          warps, the context split over gridDim.z CTAs; partial
//                          results go to scratch memory and are merged by
//  attention_merge_kernel.
#include "common.cuh"
#include "tma.cuh"
#include <map>
#include <mutex>
#include <tuple>

#ifndef MLS_HEAD_DIM
#error "compile with -DMLS_HEAD_DIM=<head size>"
#endif

namespace {
constexpr int HD = MLS_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head sizes 16..256 in steps of 16");
constexpr int BN = 64;                   // keys per tile
constexpr int NT = 128;                  // threads per CTA
constexpr int ROWB = HD * 2 + 16;        // bytes of a padded row in shared memory: the
                                         // 16 extra bytes spread 8 rows over all banks
constexpr int KCH = HD / 8;              // 16-byte chunks per row
constexpr int TILE_BYTES = BN * ROWB;
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
    const __nv_bfloat16* qkv;            // [T, (H + 2 Hkv) * HD]
    __nv_bfloat16* out;                  // [T, H * HD]
    const __nv_bfloat16* k_pool;         // [Hkv, pages, block, HD]
    const __nv_bfloat16* v_pool;
    const int* block_table;              // [R, max_blocks], -1 = no page
    const int* cu_q;                     // [R + 1]
    const int* ctx_len;                  // [R]
    float* part_o;                       // [splits, T * H, HD]   (split kernel, splits > 1)
    float* part_lse;                     // [splits, T * H]       (log2 domain)
    int max_blocks, n_req, n_tokens, n_heads, n_kv, group, block_size, window, n_split;
    int small_only;                      // tile kernel: 1 = skip requests the split kernel takes
    int cluster_merge;                   // split TMA kernel: the splits of a request and kv head are
                                         // one cluster and merge through shared memory
    float scale_log2;                    // scale * log2(e)
    int* status;                         // device status word (a bounded wait that ran out)
    long long n_pages;                   // pages of the pool: [Hkv, pages, block, HD]
};

// What the split kernel needs to take the rotation and the cache write upon itself in a
// step of single decoded tokens (parts == nullptr: it does not).  The q/k/v projection is
// then read as the float32 K-parts of its matrix product ([n_parts][T][(H + 2 Hkv) * HD]);
// every CTA adds up, rounds and rotates the queries of its kv head's group, and the CTA whose
// stretch of the context holds the new token does the same for the new key and value,
// writes them to their slot of the cache and into its own tile of keys and values in shared
// memory (the copy of that page from memory may have been made before the write).
struct Fused {
    const float* parts;
    int n_parts;
    long long part_stride;
    const int* positions;                // [T]
    const float* cos_t;                  // [max_pos, HD / 2]
    const float* sin_t;
    const int* slot_map;                 // [T]
    __nv_bfloat16* k_out;                // the pools, writable
    __nv_bfloat16* v_out;
    int max_pos, writes;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;       // size 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special function unit (relative error about 2^-22; 2^-inf = 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A request goes to the split kernel when all its (token, head) rows of one kv
// head fit one 16-row tile.
__device__ __forceinline__ bool is_small(int q_len, int group) { return q_len * group <= 16; }

// Key tiles a context split holds: the most tiles a small request of this step can have,
// shared out over the splits.  Every request is cut at the same multiples, so a shorter one
// fills only its first splits (the others find no tile; the merge knows) and no CTA walks more
// tiles than the longest request's.  The step's longest context lies one past the requests'
// in ctx_len (the batch builder puts it there): all threads of the grid, and the merge
// kernel, work the same number out from it, also when a captured step is replayed with
// longer contexts.  With a window a small request (at most 16 new tokens) sees at most
// window + 15 keys, which begin anywhere in a tile.
__device__ __forceinline__ int tiles_per_split(const int* ctx_len, int n_req, int window, int bn,
                                               int n_split) {
    int most = (ctx_len[n_req] + bn - 1) / bn;
    if (window > 0) most = min(most, (window + 15 + bn - 2) / bn + 1);
    return (max(most, 1) + n_split - 1) / n_split;
}

// Keys kbase .. kbase+63 of one kv head into shared memory; rows outside [lo, hi]
// or on a released page are zero-filled, so nothing that is not a key of this
// request can reach the products.
__device__ __forceinline__ void load_kv_tile(uint8_t* ks, uint8_t* vs, const Params& P,
                                             const int* table, int kvh, int kbase, int lo, int hi) {
    const uint32_t ka = smem_u32(ks), va = smem_u32(vs);
    for (int idx = threadIdx.x; idx < BN * KCH; idx += NT) {
        const int row = idx / KCH, ch = idx - row * KCH;
        const int j = kbase + row;
        bool ok = j >= lo && j <= hi;
        size_t off = 0;
        if (ok) {
            const int page = table[j / P.block_size];
            ok = page >= 0;
            if (ok)
                off = (((size_t)kvh * P.n_pages + page) * P.block_size + (j % P.block_size)) * HD +
                      ch * 8;
        }
        cp_async16(ka + row * ROWB + ch * 16, P.k_pool + off, ok);
        cp_async16(va + row * ROWB + ch * 16, P.v_pool + off, ok);
    }
}

// Rows row0 .. row0+n_rows-1 of the request's (token, head) rows into shared memory.
__device__ __forceinline__ void load_q_rows(uint8_t* qs, const Params& P, int tok0, int kvh,
                                            int row0, int n_rows, int rows_total) {
    const uint32_t qa = smem_u32(qs);
    const int row_w = (P.n_heads + 2 * P.n_kv) * HD;
    for (int idx = threadIdx.x; idx < n_rows * KCH; idx += NT) {
        const int rr = idx / KCH, ch = idx - rr * KCH;
        const int row = row0 + rr;
        const bool ok = row < rows_total;
        size_t off = 0;
        if (ok) {
            const int i = row / P.group, g = row - i * P.group;
            off = (size_t)(tok0 + i) * row_w + (size_t)(kvh * P.group + g) * HD + ch * 8;
        }
        cp_async16(qa + rr * ROWB + ch * 16, P.qkv + off, ok);
    }
}

// ----------------------------------------------------------------------------------------
// 64 rows per CTA, 16 per warp
// ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NT) attention_tile_kernel(const Params P) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* qs = smem;                               // [64][ROWB]
    uint8_t* kbuf = smem + TILE_BYTES;                // 2 x [64][ROWB]
    uint8_t* vbuf = smem + 3 * TILE_BYTES;            // 2 x [64][ROWB]

    // which request and which 64-row tile of it
    int r = 0, tile = blockIdx.x, q_len = 0, rows = 0;
    for (; r < P.n_req; ++r) {
        q_len = P.cu_q[r + 1] - P.cu_q[r];
        rows = q_len * P.group;
        int tiles = (P.small_only && is_small(q_len, P.group)) ? 0 : (rows + 63) / 64;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (r >= P.n_req) return;
    const int kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok0 = P.cu_q[r], ctx = P.ctx_len[r];
    const int row0 = tile * 64;
    const int pos0 = ctx - q_len;                     // position of the portion's first token
    const int i_first = row0 / P.group;
    const int i_last = (min(rows, row0 + 64) - 1) / P.group;
    const int hi = pos0 + i_last;
    const int lo = P.window > 0 ? max(0, pos0 + i_first - P.window + 1) : 0;
    const int* table = P.block_table + (size_t)r * P.max_blocks;
    const int kbase0 = (lo / BN) * BN;
    const int n_tiles = (hi - kbase0) / BN + 1;

    load_q_rows(qs, P, tok0, kvh, row0, 64, rows);
    load_kv_tile(kbuf, vbuf, P, table, kvh, kbase0, lo, hi);
    cp_async_commit();

    // positions of this thread's two rows (-1: the row does not exist)
    const int rA = row0 + warp * 16 + (lane >> 2), rB = rA + 8;
    const int pA = rA < rows ? pos0 + rA / P.group : -1;
    const int pB = rB < rows ? pos0 + rB / P.group : -1;
    const int loA = P.window > 0 ? pA - P.window + 1 : 0;
    const int loB = P.window > 0 ? pB - P.window + 1 : 0;

    uint32_t qf[HD / 16][4];
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;

    for (int t = 0; t < n_tiles; ++t) {
        cp_async_wait<0>();
        __syncthreads();
        if (t == 0) {
            const uint32_t qa = smem_u32(qs) + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROWB +
                                (lane >> 4) * 16;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) ldsm_x4(qf[ks], qa + ks * 32);
        }
        const int kbase = kbase0 + t * BN;
        if (t + 1 < n_tiles) {
            load_kv_tile(kbuf + ((t + 1) & 1) * TILE_BYTES, vbuf + ((t + 1) & 1) * TILE_BYTES, P,
                         table, kvh, kbase + BN, lo, hi);
            cp_async_commit();
        }
        const uint32_t ka = smem_u32(kbuf + (t & 1) * TILE_BYTES);
        const uint32_t va = smem_u32(vbuf + (t & 1) * TILE_BYTES);

        // S = Q K^T for 16 rows x 64 keys
        float s[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const uint32_t kaddr = ka + ((lane & 7) + (lane >> 4) * 8) * ROWB + ((lane >> 3) & 1) * 16;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
                uint32_t b[4];
                ldsm_x4(b, kaddr + np * 16 * ROWB + ks * 32);
                mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
        // scale, mask, running maximum
        float tmA = -INFINITY, tmB = -INFINITY;
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
            const int j = kbase + n * 8 + (lane & 3) * 2;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int jj = j + e;
                const float a = (jj <= pA && jj >= loA) ? s[n][e] * P.scale_log2 : -INFINITY;
                const float b = (jj <= pB && jj >= loB) ? s[n][2 + e] * P.scale_log2 : -INFINITY;
                s[n][e] = a;
                s[n][2 + e] = b;
                tmA = fmaxf(tmA, a);
                tmB = fmaxf(tmB, b);
            }
        }
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1));
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
        const float nmA = fmaxf(mA, tmA), nmB = fmaxf(mB, tmB);
        const float baseA = nmA == -INFINITY ? 0.f : nmA, baseB = nmB == -INFINITY ? 0.f : nmB;
        const float cA = fast_exp2(mA - baseA), cB = fast_exp2(mB - baseB);   // exp2(-inf) = 0
        mA = nmA;
        mB = nmB;
        float sumA = 0.f, sumB = 0.f;
        uint32_t pf[BN / 16][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
            const float p0 = fast_exp2(s[n][0] - baseA), p1 = fast_exp2(s[n][1] - baseA);
            const float p2 = fast_exp2(s[n][2] - baseB), p3 = fast_exp2(s[n][3] - baseB);
            sumA += p0 + p1;
            sumB += p2 + p3;
            pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        lA = lA * cA + sumA;
        lB = lB * cB + sumB;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= cA;
            o[i][1] *= cA;
            o[i][2] *= cB;
            o[i][3] *= cB;
        }
        // O += P V
        const uint32_t vaddr = va + ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (lane >> 4) * 16;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                uint32_t b[4];
                ldsm_x4_trans(b, vaddr + kk * 16 * ROWB + dp * 32);
                mma_bf16(o[2 * dp], pf[kk], b[0], b[1]);
                mma_bf16(o[2 * dp + 1], pf[kk], b[2], b[3]);
            }
        }
    }
    // the row sums live in four threads each
    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    const float invA = lA > 0.f ? 1.f / lA : 0.f, invB = lB > 0.f ? 1.f / lB : 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half ? rB : rA;
        if (row >= rows) continue;
        const int i = row / P.group, g = row - i * P.group;
        __nv_bfloat16* dst = P.out + (size_t)(tok0 + i) * P.n_heads * HD +
                             (size_t)(kvh * P.group + g) * HD + (lane & 3) * 2;
        const float inv = half ? invB : invA;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            *reinterpret_cast<uint32_t*>(dst + n * 8) =
                pack_bf16(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
        }
    }
}

// ----------------------------------------------------------------------------------------
// up to 16 rows per CTA, the keys of a tile split over the warps, the context over CTAs
// ----------------------------------------------------------------------------------------
constexpr int STAGES = 3;

__global__ void __launch_bounds__(NT) attention_split_kernel(const Params P) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* qs = smem;                               // [16][ROWB]
    uint8_t* kbuf = smem + 16 * ROWB;                 // STAGES x [64][ROWB]
    uint8_t* vbuf = kbuf + STAGES * TILE_BYTES;

    const int r = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int q_len = P.cu_q[r + 1] - P.cu_q[r];
    if (!is_small(q_len, P.group)) return;            // the tile kernel's
    const int rows = q_len * P.group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok0 = P.cu_q[r], ctx = P.ctx_len[r];
    const int pos0 = ctx - q_len;
    const int hi = ctx - 1;
    const int lo = P.window > 0 ? max(0, pos0 - P.window + 1) : 0;
    const int* table = P.block_table + (size_t)r * P.max_blocks;
    const int kbase0 = (lo / BN) * BN;
    const int tiles_all = (hi - kbase0) / BN + 1;
    const int per = P.n_split == 1 ? tiles_all
        : tiles_per_split(P.ctx_len, P.n_req, P.window, BN, P.n_split);
    const int t_begin = split * per, t_end = min(tiles_all, t_begin + per);
    const int n_tiles = max(0, t_end - t_begin);
    if (n_tiles == 0) return;                         // a stretch past the request's end: the merge knows

    const int rA = lane >> 2, rB = rA + 8;
    const int pA = rA < rows ? pos0 + rA / P.group : -1;
    const int pB = rB < rows ? pos0 + rB / P.group : -1;
    const int loA = P.window > 0 ? pA - P.window + 1 : 0;
    const int loB = P.window > 0 ? pB - P.window + 1 : 0;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
    uint32_t qf[HD / 16][4];

    if (n_tiles > 0) {
        load_q_rows(qs, P, tok0, kvh, 0, 16, rows);
#pragma unroll
        for (int st = 0; st < STAGES - 1; ++st) {
            if (st < n_tiles)
                load_kv_tile(kbuf + st * TILE_BYTES, vbuf + st * TILE_BYTES, P, table, kvh,
                             kbase0 + (t_begin + st) * BN, lo, hi);
            cp_async_commit();
        }
    }
    for (int t = 0; t < n_tiles; ++t) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (t == 0) {
            const uint32_t qa = smem_u32(qs) + ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB +
                                (lane >> 4) * 16;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) ldsm_x4(qf[ks], qa + ks * 32);
        }
        {
            const int nt = t + STAGES - 1;
            if (nt < n_tiles)
                load_kv_tile(kbuf + (nt % STAGES) * TILE_BYTES, vbuf + (nt % STAGES) * TILE_BYTES,
                             P, table, kvh, kbase0 + (t_begin + nt) * BN, lo, hi);
            cp_async_commit();
        }
        const int kbase = kbase0 + (t_begin + t) * BN + warp * 16;     // this warp's 16 keys
        const uint32_t ka = smem_u32(kbuf + (t % STAGES) * TILE_BYTES) + warp * 16 * ROWB;
        const uint32_t va = smem_u32(vbuf + (t % STAGES) * TILE_BYTES) + warp * 16 * ROWB;

        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        const uint32_t kaddr = ka + ((lane & 7) + (lane >> 4) * 8) * ROWB + ((lane >> 3) & 1) * 16;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t b[4];
            ldsm_x4(b, kaddr + ks * 32);
            mma_bf16(s[0], qf[ks], b[0], b[1]);
            mma_bf16(s[1], qf[ks], b[2], b[3]);
        }
        float tmA = -INFINITY, tmB = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const int j = kbase + n * 8 + (lane & 3) * 2;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int jj = j + e;
                const float a = (jj <= pA && jj >= loA) ? s[n][e] * P.scale_log2 : -INFINITY;
                const float b = (jj <= pB && jj >= loB) ? s[n][2 + e] * P.scale_log2 : -INFINITY;
                s[n][e] = a;
                s[n][2 + e] = b;
                tmA = fmaxf(tmA, a);
                tmB = fmaxf(tmB, b);
            }
        }
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1));
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
        const float nmA = fmaxf(mA, tmA), nmB = fmaxf(mB, tmB);
        const float baseA = nmA == -INFINITY ? 0.f : nmA, baseB = nmB == -INFINITY ? 0.f : nmB;
        const float cA = fast_exp2(mA - baseA), cB = fast_exp2(mB - baseB);
        mA = nmA;
        mB = nmB;
        uint32_t pf[4];
        float sumA = 0.f, sumB = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const float p0 = fast_exp2(s[n][0] - baseA), p1 = fast_exp2(s[n][1] - baseA);
            const float p2 = fast_exp2(s[n][2] - baseB), p3 = fast_exp2(s[n][3] - baseB);
            sumA += p0 + p1;
            sumB += p2 + p3;
            pf[n * 2] = pack_bf16(p0, p1);
            pf[n * 2 + 1] = pack_bf16(p2, p3);
        }
        lA = lA * cA + sumA;
        lB = lB * cB + sumB;
        const uint32_t vaddr = va + ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (lane >> 4) * 16;
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
            uint32_t b[4];
            ldsm_x4_trans(b, vaddr + dp * 32);
            o[2 * dp][0] *= cA;
            o[2 * dp][1] *= cA;
            o[2 * dp][2] *= cB;
            o[2 * dp][3] *= cB;
            o[2 * dp + 1][0] *= cA;
            o[2 * dp + 1][1] *= cA;
            o[2 * dp + 1][2] *= cB;
            o[2 * dp + 1][3] *= cB;
            mma_bf16(o[2 * dp], pf, b[0], b[1]);
            mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                  // the tiles are no longer read

    // merge the four warps' partial results through shared memory
    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    float* m_s = reinterpret_cast<float*>(smem);      // [4][16]
    float* l_s = m_s + 64;                            // [4][16]
    float* o_s = l_s + 64;                            // [4][16][HD]
    if ((lane & 3) == 0) {
        m_s[warp * 16 + rA] = mA;
        m_s[warp * 16 + rB] = mB;
        l_s[warp * 16 + rA] = lA;
        l_s[warp * 16 + rB] = lB;
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        float* a = o_s + ((size_t)warp * 16 + rA) * HD + n * 8 + (lane & 3) * 2;
        float* b = o_s + ((size_t)warp * 16 + rB) * HD + n * 8 + (lane & 3) * 2;
        a[0] = o[n][0];
        a[1] = o[n][1];
        b[0] = o[n][2];
        b[1] = o[n][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows * HD; idx += NT) {
        const int row = idx / HD, d = idx - row * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, m_s[w * 16 + row]);
        float l = 0.f, acc = 0.f;
        if (m != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float c = fast_exp2(m_s[w * 16 + row] - m);
                l += l_s[w * 16 + row] * c;
                acc += o_s[((size_t)w * 16 + row) * HD + d] * c;
            }
        }
        const float val = l > 0.f ? acc / l : 0.f;
        const int i = row / P.group, g = row - i * P.group;
        const size_t unit = (size_t)(tok0 + i) * P.n_heads + (kvh * P.group + g);
        if (P.n_split == 1) {
            P.out[unit * HD + d] = __float2bfloat16_rn(val);
        } else {
            const size_t units = (size_t)P.n_tokens * P.n_heads;
            P.part_o[((size_t)split * units + unit) * HD + d] = val;
            if (d == 0)
                P.part_lse[(size_t)split * units + unit] = l > 0.f ? m + log2f(l) : -INFINITY;
        }
    }
}

// out[unit] = sum_s w_s part_o[s, unit] with w_s = 2^(lse_s - max lse) normalised.
// One block per (token, head), one thread per element of the head.
constexpr int MAX_SPLITS = 256;
__global__ void attention_merge_kernel(const Params P) {
    chain_release();
    __shared__ float weight[MAX_SPLITS];
    __shared__ float total;
    const int t = blockIdx.x, h = blockIdx.y;
    // only the requests the split kernel took have partial results (the step's index
    // arrays were copied before its first kernel began)
    int r = 0;
    while (r + 1 < P.n_req && P.cu_q[r + 1] <= t) ++r;
    const int q_len = P.cu_q[r + 1] - P.cu_q[r];
    const bool mine = is_small(q_len, P.group);
    __shared__ int parts_here;
    if (threadIdx.x < 32) {
        // the stretches of this request that hold tiles: the others wrote nothing
        const int per = tiles_per_split(P.ctx_len, P.n_req, P.window, BN, P.n_split);
        const int ctx = P.ctx_len[r];
        const int lo = P.window > 0 ? max(0, ctx - q_len - P.window + 1) : 0;
        const int tiles_all = (ctx - 1 - (lo / BN) * BN) / BN + 1;
        if (threadIdx.x == 0) parts_here = min(P.n_split, (tiles_all + per - 1) / per);
    }
    __syncthreads();
    const int n_parts = parts_here;
    chain_wait();
    if (!mine) return;
    const size_t units = (size_t)P.n_tokens * P.n_heads;
    const size_t unit = (size_t)t * P.n_heads + h;
    // the parts' weights 2^(lse - max), by the first warp: all loads under way together
    if (threadIdx.x < 32) {
        float lse[MAX_SPLITS / 32];
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < MAX_SPLITS / 32; ++i) {
            const int s = threadIdx.x + 32 * i;
            lse[i] = s < n_parts ? P.part_lse[s * units + unit] : -INFINITY;
            m = fmaxf(m, lse[i]);
        }
        m = warp_max(m);
        float wsum = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_SPLITS / 32; ++i) {
            const int s = threadIdx.x + 32 * i;
            const float w = (m == -INFINITY || s >= n_parts) ? 0.f : fast_exp2(lse[i] - m);
            if (s < n_parts) weight[s] = w;
            wsum += w;
        }
        wsum = warp_sum(wsum);
        if (threadIdx.x == 0) total = wsum;
    }
    __syncthreads();
    const float wsum = total;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.f;
        for (int s0 = 0; s0 < n_parts; s0 += 8) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < n_parts) o[j] = P.part_o[((s0 + j) * units + unit) * HD + d];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < n_parts) acc += weight[s0 + j] * o[j];
        }
        P.out[unit * HD + d] = __float2bfloat16_rn(wsum > 0.f ? acc / wsum : 0.f);
    }
}


#if MLS_HEAD_DIM % 64 == 0
// ----------------------------------------------------------------------------------------
// The split kernel with the keys and values brought in by TMA: one bulk tensor copy
// per page and 64-wide half of the head, issued by a producer warp, 128-byte swizzle
// so that ldmatrix reads without bank conflicts.  Page sizes 8, 16, 32, 64.
// ----------------------------------------------------------------------------------------
using namespace mls_tma;
constexpr int HALVES = HD / 64;
constexpr int HALF_BYTES = BN * 128;                    // 64 keys x 128 bytes
constexpr int KV_STAGE = 2 * HALVES * HALF_BYTES;       // keys, then values
constexpr int TSTAGES = HD <= 128 ? 3 : 2;
constexpr int TMA_THREADS = 160;                        // 4 consumer warps + 1 producer warp
constexpr int MAX_CLUSTER = 8;                          // most context splits merged inside a cluster

// address of the 16-byte chunk `chunk` (of the whole head) of key row `row`
__device__ __forceinline__ uint32_t swz(uint32_t tile, int row, int chunk) {
    return tile + (chunk >> 3) * HALF_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// The producer warp: for every 64-key tile, wait until its stage is free, then
// bring in the keys and values of the tile's pages with one bulk tensor copy per
// page and 64-wide half, for tiles t_from .. t_to - 1.  Stage `late_slot` (if any)
// is lent to the consumers at the start and is first free after they have released
// it once.
__device__ __forceinline__ void produce_tiles(const Params& P, const CUtensorMap* kmap,
                                              const CUtensorMap* vmap, const CUtensorMap* kmap_wide,
                                              const CUtensorMap* vmap_wide, const int* table, int kvh,
                                              int kb_first, int t_from, int t_to, int lo, int hi,
                                              uint32_t base, uint32_t bar0, int late_slot) {
    const int lane = threadIdx.x & 31;
    const int bs = P.block_size, ppt = BN / bs;
    const uint32_t page_bytes = bs * 128;
    for (int t = t_from; t < t_to; ++t) {
        const int slot = t % TSTAGES, round = t / TSTAGES;
        const uint32_t full = bar0 + 8u * slot, empty = bar0 + 8u * (TSTAGES + slot);
        const uint32_t parity = slot == late_slot ? (round & 1) : ((round & 1) ^ 1);
        if (!mbar_wait(empty, parity)) {
            if (lane == 0 && P.status) atomicOr(P.status, MLS_STATUS_TIMEOUT);
            return;
        }
        const int kb = kb_first + t * BN;
        const uint32_t stage = base + slot * KV_STAGE;
        bool valid = false;
        int page = -1;
        if (lane < ppt) {
            const int j0 = kb + lane * bs;
            if (j0 <= hi && j0 + bs > lo) {
                page = table[j0 / bs];
                valid = page >= 0;
            }
        }
        const unsigned mask = __ballot_sync(0xffffffffu, valid);
        const unsigned all = ppt >= 32 ? 0xffffffffu : ((1u << ppt) - 1u);
        // pages that follow one another in the pool are one contiguous run of rows:
        // a single wide copy per 64-wide half and tensor instead of one per page
        const int first = __shfl_sync(0xffffffffu, page, 0);
        if (mask == all && __all_sync(0xffffffffu, lane >= ppt || page == first + lane)) {
            if (lane == 0) mbar_arrive_expect_tx(full, BN * 128 * 2 * HALVES);
            __syncwarp();
            if (lane < 2 * HALVES) {
                const int h = lane % HALVES, is_v = lane / HALVES;
                tma_load_2d(stage + lane * HALF_BYTES, is_v ? vmap_wide : kmap_wide, h * 64,
                            (int)((kvh * P.n_pages + first) * bs), full);
            }
            continue;
        }
        if (mask != all) {
            // pages that are not keys of this request read as zeros
            for (int pi = 0; pi < ppt; ++pi) {
                if ((mask >> pi) & 1u) continue;
                for (int part = 0; part < 2 * HALVES; ++part) {
                    const uint32_t dst = stage + part * HALF_BYTES + pi * page_bytes;
                    for (uint32_t o = lane * 16; o < page_bytes; o += 512)
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(dst + o),
                                     "r"(0u) : "memory");
                }
            }
            fence_proxy_async();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_expect_tx(full, __popc(mask) * page_bytes * 2 * HALVES);
        __syncwarp();
        if (valid) {
            const int y = (int)((kvh * P.n_pages + page) * bs);
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
                tma_load_2d(stage + h * HALF_BYTES + lane * page_bytes, kmap, h * 64, y, full);
                tma_load_2d(stage + (HALVES + h) * HALF_BYTES + lane * page_bytes, vmap, h * 64, y,
                            full);
            }
        }
    }
}

__global__ void __launch_bounds__(TMA_THREADS)
attention_split_tma_kernel(const Params P, const Fused F,
                           const __grid_constant__ CUtensorMap kmap,
                           const __grid_constant__ CUtensorMap vmap,
                           const __grid_constant__ CUtensorMap kmap_wide,
                           const __grid_constant__ CUtensorMap vmap_wide) {
    // The step's index arrays were copied before the step's first kernel began, so
    // they may be read at once; what earlier kernels of this step write (the new
    // tokens' queries, keys and values) is read after chain_wait.
    chain_release();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;       // the swizzle needs 1024-byte tiles
    uint8_t* gbase = smem_raw + (base - raw);
    const uint32_t q_addr = base + TSTAGES * KV_STAGE;
    const uint32_t bar0 = q_addr + 16 * ROWB;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (TSTAGES + s); };

    const int r = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int q_len = P.cu_q[r + 1] - P.cu_q[r];
    if (!is_small(q_len, P.group)) {
        chain_wait();
        return;
    }
    const int rows = q_len * P.group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok0 = P.cu_q[r], ctx = P.ctx_len[r];
    const int pos0 = ctx - q_len;
    const int hi = ctx - 1;
    const int lo = P.window > 0 ? max(0, pos0 - P.window + 1) : 0;
    const int* table = P.block_table + (size_t)r * P.max_blocks;
    const int kbase0 = (lo / BN) * BN;
    const int tiles_all = (hi - kbase0) / BN + 1;
    const int per = P.n_split == 1 ? tiles_all
        : tiles_per_split(P.ctx_len, P.n_req, P.window, BN, P.n_split);
    const int t_begin = split * per, t_end = min(tiles_all, t_begin + per);
    const int n_tiles = max(0, t_end - t_begin);
    if (n_tiles == 0 && !P.cluster_merge) {           // a stretch past the request's end: the merge
        chain_wait();                                 // kernel knows; inside a cluster it takes part
        return;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < TSTAGES; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 4);
        }
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == 4) {
        // Tiles that end before this request's first new token hold keys of earlier
        // steps only: the first ring of them is asked for while the kernels that
        // write the new token may still run.
        const int kb_first = kbase0 + t_begin * BN;
        const int old_tiles = max(0, (pos0 - kb_first) / BN);
        const int ahead = min(min(n_tiles, TSTAGES), old_tiles);
        produce_tiles(P, &kmap, &vmap, &kmap_wide, &vmap_wide, table, kvh, kb_first, 0, ahead, lo,
                      hi, base, bar0, /*late_slot=*/-1);
        chain_wait();
        produce_tiles(P, &kmap, &vmap, &kmap_wide, &vmap_wide, table, kvh, kb_first, ahead,
                      n_tiles, lo, hi, base, bar0, /*late_slot=*/-1);
        if (P.cluster_merge) {           // every thread of the cluster meets at its two barriers
            cluster_sync_all();
            cluster_sync_all();
        }
        return;
    }
    // fused rotation (single decoded tokens): the position, its rows of the angle tables and
    // the new token's slot are the step's own input and are read while the projection before
    // this kernel may still run
    const bool fused = F.parts != nullptr;
    constexpr int ROT_HALF = HD / 2, ROT_QPH = ROT_HALF / 4, ROT_ITERS = (16 * ROT_QPH + 127) / 128;
    float4 rot_cos[ROT_ITERS], rot_sin[ROT_ITERS];
    int rot_slot = -1;
    if (fused && n_tiles > 0) {
        int pos = F.positions[tok0];
        if (pos < 0 || pos >= F.max_pos || q_len != 1) {
            if (threadIdx.x == 0 && P.status) atomicOr(P.status, MLS_STATUS_BAD_POSITION);
            pos = pos < 0 ? 0 : (pos >= F.max_pos ? F.max_pos - 1 : pos);
        }
        const float* cr = F.cos_t + (size_t)pos * ROT_HALF;
        const float* sr = F.sin_t + (size_t)pos * ROT_HALF;
#pragma unroll
        for (int k = 0; k < ROT_ITERS; ++k) {
            const int u = threadIdx.x + k * 128;
            if (u < 16 * ROT_QPH) {
                const int c = u % ROT_QPH;
                rot_cos[k] = *reinterpret_cast<const float4*>(cr + c * 4);
                rot_sin[k] = *reinterpret_cast<const float4*>(sr + c * 4);
            }
        }
        if (F.writes && t_end == tiles_all) rot_slot = F.slot_map[tok0];
    }
    chain_wait();

    // --------------------------------------------------------------------- consumers
    const int rA = lane >> 2, rB = rA + 8;
    const int pA = rA < rows ? pos0 + rA / P.group : -1;
    const int pB = rB < rows ? pos0 + rB / P.group : -1;
    const int loA = P.window > 0 ? pA - P.window + 1 : 0;
    const int loB = P.window > 0 ? pB - P.window + 1 : 0;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
    uint32_t qf[HD / 16][4];

    // this CTA's queries from the projection's parts, and, in the CTA whose tiles end at the
    // new token, the new key and value
    const bool owns_new = fused && F.writes && n_tiles > 0 && t_end == tiles_all;
    uint2 new_kv[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};     // this thread's share of them
    if (fused && n_tiles > 0) {
        constexpr int half = ROT_HALF, qph = ROT_QPH;
        const size_t width = (size_t)(P.n_heads + 2 * P.n_kv) * HD;
        const size_t row_at = (size_t)tok0 * width;
#pragma unroll
        for (int k = 0; k < ROT_ITERS; ++k) {
            const int u = threadIdx.x + k * 128;
            if (u >= 16 * qph) break;
            const int g = u / qph, c = u - g * qph;
            uint2 w1 = make_uint2(0u, 0u), w2 = w1;
            if (g < rows) {
                const size_t col = (size_t)(kvh * P.group + g) * HD + c * 4;
                const size_t at[2] = {row_at + col, row_at + col + half};
                float4 x[2], o1, o2;
                sum_parts4_of<2, 8>(F.parts, at, F.n_parts, (size_t)F.part_stride, x);
                rotate_half4(round_bf16(x[0]), round_bf16(x[1]), rot_cos[k], rot_sin[k], o1, o2);
                w1 = pack_bf16x4(o1);
                w2 = pack_bf16x4(o2);
            }
            const uint32_t dst = q_addr + g * ROWB + c * 8;
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};\n" ::"r"(dst), "r"(w1.x), "r"(w1.y) : "memory");
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};\n" ::"r"(dst + half * 2), "r"(w2.x), "r"(w2.y)
                         : "memory");
        }
        if (owns_new) {
            // threads 0 .. qph-1: four rotated pairs of the key each; the next HD / 4: four
            // values of the value each.  Into the cache now, into the tile when it has landed.
            const int slot = rot_slot;
            const long long pool_slots = P.n_pages * P.block_size;
            const bool slot_ok = slot >= 0 && slot < pool_slots;
            if (!slot_ok && threadIdx.x == 0 && P.status) atomicOr(P.status, MLS_STATUS_BAD_SLOT);
            const int page = slot_ok ? slot / P.block_size : 0;
            const int off = slot_ok ? slot - page * P.block_size : 0;
            const size_t cache_at = (((size_t)kvh * P.n_pages + page) * P.block_size + off) * HD;
            const int u = threadIdx.x;
            if (u < qph) {
                const size_t col = (size_t)(P.n_heads + kvh) * HD + u * 4;
                const size_t at[2] = {row_at + col, row_at + col + half};
                float4 x[2], o1, o2;
                sum_parts4_of<2, 8>(F.parts, at, F.n_parts, (size_t)F.part_stride, x);
                // thread u < qph took chunk u of the angles in its first round above
                rotate_half4(round_bf16(x[0]), round_bf16(x[1]), rot_cos[0], rot_sin[0], o1, o2);
                new_kv[0] = pack_bf16x4(o1);
                new_kv[1] = pack_bf16x4(o2);
                if (slot_ok) {
                    *reinterpret_cast<uint2*>(F.k_out + cache_at + u * 4) = new_kv[0];
                    *reinterpret_cast<uint2*>(F.k_out + cache_at + half + u * 4) = new_kv[1];
                }
            } else if (u < qph + HD / 4) {
                const int c = u - qph;
                const size_t at[1] = {row_at + (size_t)(P.n_heads + P.n_kv + kvh) * HD + c * 4};
                float4 x[1];
                sum_parts4_of<1, 8>(F.parts, at, F.n_parts, (size_t)F.part_stride, x);
                new_kv[0] = pack_bf16x4(x[0]);
                if (slot_ok) *reinterpret_cast<uint2*>(F.v_out + cache_at + c * 4) = new_kv[0];
            }
            // a page that this token enters: what its previous owner left in the other slots
            // must not reach a later step as 0 * NaN
            if (slot_ok && off == 0 && P.block_size > 1) {
                const int chunks = (P.block_size - 1) * (HD / 8);
                for (int i = threadIdx.x; i < 2 * chunks; i += 128) {
                    __nv_bfloat16* pool = i < chunks ? F.k_out : F.v_out;
                    reinterpret_cast<uint4*>(pool + cache_at + HD)[i < chunks ? i : i - chunks] =
                        make_uint4(0u, 0u, 0u, 0u);
                }
            }
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        const uint32_t qa = q_addr + ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (lane >> 4) * 16;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) ldsm_x4(qf[ks], qa + ks * 32);
    } else if (n_tiles > 0) {
        // the queries: plain asynchronous copies into a padded tile, then registers
        const int row_w = (P.n_heads + 2 * P.n_kv) * HD;
        for (int idx = threadIdx.x; idx < 16 * KCH; idx += 128) {
            const int rr = idx / KCH, ch = idx - rr * KCH;
            const bool ok = rr < rows;
            size_t off = 0;
            if (ok) {
                const int i = rr / P.group, g = rr - i * P.group;
                off = (size_t)(tok0 + i) * row_w + (size_t)(kvh * P.group + g) * HD + ch * 8;
            }
            cp_async16(q_addr + rr * ROWB + ch * 16, P.qkv + off, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        const uint32_t qa = q_addr + ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (lane >> 4) * 16;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) ldsm_x4(qf[ks], qa + ks * 32);
    }
    const int krow = warp * 16 + (lane & 7) + (lane >> 4) * 8, kch = (lane >> 3) & 1;
    const int vrow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, vch = lane >> 4;
    bool timed_out = false;
    for (int t = 0; t < n_tiles; ++t) {
        const int slot = t % TSTAGES, ph = (t / TSTAGES) & 1;
        if (!mbar_wait(full(slot), ph)) {
            timed_out = true;
            break;
        }
        const uint32_t ktile = base + slot * KV_STAGE;
        const uint32_t vtile = ktile + HALVES * HALF_BYTES;
        const int kbase = kbase0 + (t_begin + t) * BN + warp * 16;
        if (owns_new && t == n_tiles - 1) {
            // the new token's key and value over whatever the page held when it was copied
            constexpr int half = HD / 2, qph = half / 4;
            const int row = pos0 - (kbase0 + (t_begin + t) * BN);
            const int u = threadIdx.x;
            if (u < qph) {
                const uint32_t a = swz(ktile, row, (u * 4) >> 3) + ((u * 4) & 7) * 2;
                const uint32_t b = swz(ktile, row, (half + u * 4) >> 3) + ((half + u * 4) & 7) * 2;
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};\n" ::"r"(a), "r"(new_kv[0].x),
                             "r"(new_kv[0].y) : "memory");
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};\n" ::"r"(b), "r"(new_kv[1].x),
                             "r"(new_kv[1].y) : "memory");
            } else if (u < qph + HD / 4) {
                const int c = u - qph;
                const uint32_t a = swz(vtile, row, (c * 4) >> 3) + ((c * 4) & 7) * 2;
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};\n" ::"r"(a), "r"(new_kv[0].x),
                             "r"(new_kv[0].y) : "memory");
            }
            // the rows after it are no keys yet: whatever the page held when it was copied
            // (this CTA clears a page it enters in memory, but the copy may have come first)
            // must not meet a probability of zero as NaN
            for (int i = threadIdx.x; i < (BN - 1 - row) * KCH * 2; i += 128) {
                const int which = i / ((BN - 1 - row) * KCH), w = i - which * (BN - 1 - row) * KCH;
                const int rr = row + 1 + w / KCH, ch = w - (w / KCH) * KCH;
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n"
                             ::"r"(swz(which ? vtile : ktile, rr, ch)), "r"(0u) : "memory");
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
        }

        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t b[4];
            ldsm_x4(b, swz(ktile, krow, ks * 2 + kch));
            mma_bf16(s[0], qf[ks], b[0], b[1]);
            mma_bf16(s[1], qf[ks], b[2], b[3]);
        }
        float tmA = -INFINITY, tmB = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const int j = kbase + n * 8 + (lane & 3) * 2;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int jj = j + e;
                const float a = (jj <= pA && jj >= loA) ? s[n][e] * P.scale_log2 : -INFINITY;
                const float b = (jj <= pB && jj >= loB) ? s[n][2 + e] * P.scale_log2 : -INFINITY;
                s[n][e] = a;
                s[n][2 + e] = b;
                tmA = fmaxf(tmA, a);
                tmB = fmaxf(tmB, b);
            }
        }
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1));
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
        const float nmA = fmaxf(mA, tmA), nmB = fmaxf(mB, tmB);
        const float baseA = nmA == -INFINITY ? 0.f : nmA, baseB = nmB == -INFINITY ? 0.f : nmB;
        const float cA = fast_exp2(mA - baseA), cB = fast_exp2(mB - baseB);
        mA = nmA;
        mB = nmB;
        uint32_t pf[4];
        float sumA = 0.f, sumB = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const float p0 = fast_exp2(s[n][0] - baseA), p1 = fast_exp2(s[n][1] - baseA);
            const float p2 = fast_exp2(s[n][2] - baseB), p3 = fast_exp2(s[n][3] - baseB);
            sumA += p0 + p1;
            sumB += p2 + p3;
            pf[n * 2] = pack_bf16(p0, p1);
            pf[n * 2 + 1] = pack_bf16(p2, p3);
        }
        lA = lA * cA + sumA;
        lB = lB * cB + sumB;
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
            uint32_t b[4];
            ldsm_x4_trans(b, swz(vtile, vrow, dp * 2 + vch));
            o[2 * dp][0] *= cA;
            o[2 * dp][1] *= cA;
            o[2 * dp][2] *= cB;
            o[2 * dp][3] *= cB;
            o[2 * dp + 1][0] *= cA;
            o[2 * dp + 1][1] *= cA;
            o[2 * dp + 1][2] *= cB;
            o[2 * dp + 1][3] *= cB;
            mma_bf16(o[2 * dp], pf, b[0], b[1]);
            mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty(slot));
    }
    // a wait that ran out is recorded; the warp still joins the barriers below so
    // that no other warp waits for it (the host raises on the status word)
    if (timed_out && lane == 0 && P.status) atomicOr(P.status, MLS_STATUS_TIMEOUT);
    asm volatile("bar.sync 1, 128;\n" ::: "memory");     // every tile has been read

    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    float* m_s = reinterpret_cast<float*>(gbase);     // [4][16]
    float* l_s = m_s + 64;                            // [4][16]
    float* o_s = l_s + 64;                            // [4][16][HD]
    if ((lane & 3) == 0) {
        m_s[warp * 16 + rA] = mA;
        m_s[warp * 16 + rB] = mB;
        l_s[warp * 16 + rA] = lA;
        l_s[warp * 16 + rB] = lB;
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        float* a = o_s + ((size_t)warp * 16 + rA) * HD + n * 8 + (lane & 3) * 2;
        float* b = o_s + ((size_t)warp * 16 + rB) * HD + n * 8 + (lane & 3) * 2;
        a[0] = o[n][0];
        a[1] = o[n][1];
        b[0] = o[n][2];
        b[1] = o[n][3];
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    for (int idx = threadIdx.x; idx < rows * HD; idx += 128) {
        const int row = idx / HD, d = idx - row * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, m_s[w * 16 + row]);
        float l = 0.f, acc = 0.f;
        if (m != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float c = fast_exp2(m_s[w * 16 + row] - m);
                l += l_s[w * 16 + row] * c;
                acc += o_s[((size_t)w * 16 + row) * HD + d] * c;
            }
        }
        const float val = l > 0.f ? acc / l : 0.f;
        const int i = row / P.group, g = row - i * P.group;
        const size_t unit = (size_t)(tok0 + i) * P.n_heads + (kvh * P.group + g);
        if (P.n_split == 1) {
            P.out[unit * HD + d] = __float2bfloat16_rn(val);
        } else if (P.cluster_merge) {
            // this CTA's result stays in its shared memory for the merge inside the cluster
            o_s[(size_t)4 * 16 * HD + idx] = val;
            if (d == 0) o_s[(size_t)5 * 16 * HD + row] = l > 0.f ? m + log2f(l) : -INFINITY;
        } else {
            const size_t units = (size_t)P.n_tokens * P.n_heads;
            P.part_o[((size_t)split * units + unit) * HD + d] = val;
            if (d == 0)
                P.part_lse[(size_t)split * units + unit] = l > 0.f ? m + log2f(l) : -INFINITY;
        }
    }
    if (P.cluster_merge) {
        // The CTAs of this request and kv head (one per stretch of the context) are one
        // cluster: each merges a share of the (row, element) pairs, reading every CTA's
        // result and log-sum from its shared memory; weights 2^(lse - max lse), normalised,
        // added in the order of the stretches.
        cluster_sync_all();
        const uint32_t cta_o = smem_u32(o_s + (size_t)4 * 16 * HD);
        const uint32_t cta_lse = smem_u32(o_s + (size_t)5 * 16 * HD);
        auto peer = [](uint32_t addr, int rank) {
            uint32_t ra;
            float v;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(ra) : "r"(addr), "r"(rank));
            asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(ra) : "memory");
            return v;
        };
        for (int idx = split * 128 + threadIdx.x; idx < rows * HD; idx += P.n_split * 128) {
            const int row = idx / HD, d = idx - row * HD;
            float lse[MAX_CLUSTER], m = -INFINITY;
#pragma unroll
            for (int sidx = 0; sidx < MAX_CLUSTER; ++sidx) {
                lse[sidx] = sidx < P.n_split ? peer(cta_lse + row * 4, sidx) : -INFINITY;
                m = fmaxf(m, lse[sidx]);
            }
            float wsum = 0.f, acc = 0.f;
            if (m != -INFINITY) {
#pragma unroll
                for (int sidx = 0; sidx < MAX_CLUSTER; ++sidx) {
                    if (sidx < P.n_split) {
                        const float w = fast_exp2(lse[sidx] - m);
                        wsum += w;
                        acc += w * peer(cta_o + idx * 4, sidx);
                    }
                }
            }
            const int i = row / P.group, g = row - i * P.group;
            const size_t unit = (size_t)(tok0 + i) * P.n_heads + (kvh * P.group + g);
            P.out[unit * HD + d] = __float2bfloat16_rn(wsum > 0.f ? acc / wsum : 0.f);
        }
        cluster_sync_all();              // nobody's shared memory goes away while it is read
    }
}

// ----------------------------------------------------------------------------------------
// The tile kernel (64 rows per CTA, 16 per warp) with the same TMA producer.  The
// queries borrow the last stage until they are in registers.  Tiles are handed out
// from the end of each request backwards: the last rows see the most keys, and the
// longest work should start first.
// ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(TMA_THREADS)
attention_tile_tma_kernel(const Params P, const __grid_constant__ CUtensorMap kmap,
                          const __grid_constant__ CUtensorMap vmap,
                          const __grid_constant__ CUtensorMap kmap_wide,
                          const __grid_constant__ CUtensorMap vmap_wide) {
    chain_release();
    chain_wait();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t bar0 = base + TSTAGES * KV_STAGE;
    const uint32_t q_addr = base + (TSTAGES - 1) * KV_STAGE;     // lent by the last stage
    static_assert(64 * ROWB <= KV_STAGE, "the queries must fit one stage");

    int r = 0, tile = blockIdx.x, q_len = 0, rows = 0;
    for (; r < P.n_req; ++r) {
        q_len = P.cu_q[r + 1] - P.cu_q[r];
        rows = q_len * P.group;
        int tiles = (P.small_only && is_small(q_len, P.group)) ? 0 : (rows + 63) / 64;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (r >= P.n_req) return;
    tile = (rows + 63) / 64 - 1 - tile;                           // heavy tiles first
    const int kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok0 = P.cu_q[r], ctx = P.ctx_len[r];
    const int row0 = tile * 64;
    const int pos0 = ctx - q_len;
    const int i_first = row0 / P.group;
    const int i_last = (min(rows, row0 + 64) - 1) / P.group;
    const int hi = pos0 + i_last;
    const int lo = P.window > 0 ? max(0, pos0 + i_first - P.window + 1) : 0;
    const int* table = P.block_table + (size_t)r * P.max_blocks;
    const int kbase0 = (lo / BN) * BN;
    const int n_tiles = (hi - kbase0) / BN + 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TSTAGES; ++s) {
            mbar_init(bar0 + 8u * s, 1);
            mbar_init(bar0 + 8u * (TSTAGES + s), 4);
        }
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == 4) {
        produce_tiles(P, &kmap, &vmap, &kmap_wide, &vmap_wide, table, kvh, kbase0, 0, n_tiles, lo,
                      hi, base, bar0, /*late_slot=*/TSTAGES - 1);
        return;
    }

    // queries: asynchronous copies into a padded tile, then registers, then the stage is free
    {
        const int row_w = (P.n_heads + 2 * P.n_kv) * HD;
        for (int idx = threadIdx.x; idx < 64 * KCH; idx += 128) {
            const int rr = idx / KCH, ch = idx - rr * KCH;
            const int row = row0 + rr;
            const bool ok = row < rows;
            size_t off = 0;
            if (ok) {
                const int i = row / P.group, g = row - i * P.group;
                off = (size_t)(tok0 + i) * row_w + (size_t)(kvh * P.group + g) * HD + ch * 8;
            }
            cp_async16(q_addr + rr * ROWB + ch * 16, P.qkv + off, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
    }
    uint32_t qf[HD / 16][4];
    {
        const uint32_t qa = q_addr + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROWB +
                            (lane >> 4) * 16;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) ldsm_x4(qf[ks], qa + ks * 32);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar0 + 8u * (TSTAGES + TSTAGES - 1));   // hand the stage back

    const int rA = row0 + warp * 16 + (lane >> 2), rB = rA + 8;
    const int pA = rA < rows ? pos0 + rA / P.group : -1;
    const int pB = rB < rows ? pos0 + rB / P.group : -1;
    const int loA = P.window > 0 ? pA - P.window + 1 : 0;
    const int loB = P.window > 0 ? pB - P.window + 1 : 0;
    // keys up to this position are seen by all 16 rows of the warp: no mask needed
    const int first_row = row0 + warp * 16;
    const int p_first = first_row < rows ? pos0 + first_row / P.group : -1;
    const int last_row = min(rows, first_row + 16) - 1;
    const int lo_last = P.window > 0 ? pos0 + last_row / P.group - P.window + 1 : 0;
    const bool full_warp = first_row + 16 <= rows;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;

    const int krow = (lane & 7) + (lane >> 4) * 8, kch = (lane >> 3) & 1;
    const int vrow = (lane & 7) + ((lane >> 3) & 1) * 8, vch = lane >> 4;
    bool timed_out = false;
    for (int t = 0; t < n_tiles; ++t) {
        const int slot = t % TSTAGES, ph = (t / TSTAGES) & 1;
        if (!mbar_wait(bar0 + 8u * slot, ph)) {
            timed_out = true;
            break;
        }
        const uint32_t ktile = base + slot * KV_STAGE;
        const uint32_t vtile = ktile + HALVES * HALF_BYTES;
        const int kbase = kbase0 + t * BN;

        float s[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
                uint32_t b[4];
                ldsm_x4(b, swz(ktile, np * 16 + krow, ks * 2 + kch));
                mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
        float tmA = -INFINITY, tmB = -INFINITY;
        const bool need_mask = !full_warp || kbase + BN - 1 > p_first || kbase < lo_last;
        if (need_mask) {
#pragma unroll
            for (int n = 0; n < BN / 8; ++n) {
                const int j = kbase + n * 8 + (lane & 3) * 2;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int jj = j + e;
                    const float a = (jj <= pA && jj >= loA) ? s[n][e] * P.scale_log2 : -INFINITY;
                    const float b = (jj <= pB && jj >= loB) ? s[n][2 + e] * P.scale_log2 : -INFINITY;
                    s[n][e] = a;
                    s[n][2 + e] = b;
                    tmA = fmaxf(tmA, a);
                    tmB = fmaxf(tmB, b);
                }
            }
        } else {
#pragma unroll
            for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    s[n][e] *= P.scale_log2;
                    s[n][2 + e] *= P.scale_log2;
                    tmA = fmaxf(tmA, s[n][e]);
                    tmB = fmaxf(tmB, s[n][2 + e]);
                }
            }
        }
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1));
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
        const float nmA = fmaxf(mA, tmA), nmB = fmaxf(mB, tmB);
        const float baseA = nmA == -INFINITY ? 0.f : nmA, baseB = nmB == -INFINITY ? 0.f : nmB;
        const float cA = fast_exp2(mA - baseA), cB = fast_exp2(mB - baseB);
        mA = nmA;
        mB = nmB;
        float sumA = 0.f, sumB = 0.f;
        uint32_t pf[BN / 16][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
            const float p0 = fast_exp2(s[n][0] - baseA), p1 = fast_exp2(s[n][1] - baseA);
            const float p2 = fast_exp2(s[n][2] - baseB), p3 = fast_exp2(s[n][3] - baseB);
            sumA += p0 + p1;
            sumB += p2 + p3;
            pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        lA = lA * cA + sumA;
        lB = lB * cB + sumB;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= cA;
            o[i][1] *= cA;
            o[i][2] *= cB;
            o[i][3] *= cB;
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                uint32_t b[4];
                ldsm_x4_trans(b, swz(vtile, kk * 16 + vrow, dp * 2 + vch));
                mma_bf16(o[2 * dp], pf[kk], b[0], b[1]);
                mma_bf16(o[2 * dp + 1], pf[kk], b[2], b[3]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar0 + 8u * (TSTAGES + slot));
    }
    if (timed_out && lane == 0 && P.status) atomicOr(P.status, MLS_STATUS_TIMEOUT);

    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    const float invA = lA > 0.f ? 1.f / lA : 0.f, invB = lB > 0.f ? 1.f / lB : 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half ? rB : rA;
        if (row >= rows) continue;
        const int i = row / P.group, g = row - i * P.group;
        __nv_bfloat16* dst = P.out + (size_t)(tok0 + i) * P.n_heads * HD +
                             (size_t)(kvh * P.group + g) * HD + (lane & 3) * 2;
        const float inv = half ? invB : invA;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            *reinterpret_cast<uint32_t*>(dst + n * 8) =
                pack_bf16(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
        }
    }
}

constexpr int TILE_TMA_SMEM = TSTAGES * KV_STAGE + 16 * TSTAGES + 1024;

constexpr int TMA_SMEM_PIPE = TSTAGES * KV_STAGE + 16 * ROWB + 16 * TSTAGES + 1024;
constexpr int TMA_SMEM_MERGE = (128 + 6 * 16 * HD) * 4 + 1024;   // + this CTA's result and log-sums
constexpr int TMA_SMEM = TMA_SMEM_PIPE > TMA_SMEM_MERGE ? TMA_SMEM_PIPE : TMA_SMEM_MERGE;

// Tensor maps of the pools, made once per (pool, size) and kept.
struct MapKey {
    const void* ptr;
    long long rows;
    int block;
    bool operator<(const MapKey& o) const {
        return std::tie(ptr, rows, block) < std::tie(o.ptr, o.rows, o.block);
    }
};
static std::map<MapKey, CUtensorMap> g_maps;
static std::mutex g_maps_lock;

static bool pool_map(const void* pool, long long pool_rows, int block, CUtensorMap* out) {
    std::lock_guard<std::mutex> guard(g_maps_lock);
    MapKey key{pool, pool_rows, block};
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
        CUtensorMap m;
        if (!make_map_bf16_2d(&m, pool, HD, (uint64_t)pool_rows, (uint64_t)HD * 2, 64, block))
            return false;
        it = g_maps.emplace(key, m).first;
    }
    *out = it->second;
    return true;
}

// The split kernel and what merges its context splits: two to eight splits are launched as
// clusters (one per request and kv head) that merge through their shared memory, if all CTAs
// are resident at once (with several rounds of CTAs, having to place whole clusters costs
// more than the merge kernel: 2.5 % of a step at batch 64; and sixteen splits in clusters of
// sixteen lost 2 % at batch 1 against twenty-two splits and the merge kernel); otherwise the
// splits leave their results in scratch memory for attention_merge_kernel.
// MLS_B200_CLUSTER_MERGE=0 keeps the merge kernel for every count.
static int launch_split_tma(Params P, const Fused& F, const CUtensorMap& kmap,
                            const CUtensorMap& vmap, const CUtensorMap& kmap_wide,
                            const CUtensorMap& vmap_wide, int merge_tokens, cudaStream_t stream) {
    static const bool allowed = [] {
        const char* v = getenv("MLS_B200_CLUSTER_MERGE");
        return !(v && v[0] == '0');
    }();
    const dim3 grid(P.n_req, P.n_kv, P.n_split);
    P.cluster_merge = (allowed && P.n_split >= 2 && P.n_split <= MAX_CLUSTER &&
                       (long long)P.n_req * P.n_kv * P.n_split <= 2LL * sm_count()) ? 1 : 0;
    if (P.cluster_merge) {
        const int rc = launch_chained_cluster(attention_split_tma_kernel, grid, dim3(TMA_THREADS),
                                              TMA_SMEM, stream, dim3(1, 1, P.n_split), P, F, kmap,
                                              vmap, kmap_wide, vmap_wide);
        return rc ? rc : launch_status();
    }
    MLS_LAUNCH((attention_split_tma_kernel), grid, dim3(TMA_THREADS), TMA_SMEM, stream, P, F, kmap,
               vmap, kmap_wide, vmap_wide);
    if (P.n_split > 1)
        MLS_LAUNCH((attention_merge_kernel), dim3(merge_tokens, P.n_heads),
                   dim3(HD < 32 ? 32 : (HD < 128 ? HD : 128)), 0, stream, P);
    return launch_status();
}
#endif  // MLS_HEAD_DIM % 64 == 0

constexpr int TILE_SMEM = 5 * TILE_BYTES;
constexpr int SPLIT_SMEM_PIPE = 16 * ROWB + 2 * STAGES * TILE_BYTES;
constexpr int SPLIT_SMEM_MERGE = (128 + 4 * 16 * HD) * 4;
constexpr int SPLIT_SMEM = SPLIT_SMEM_PIPE > SPLIT_SMEM_MERGE ? SPLIT_SMEM_PIPE : SPLIT_SMEM_MERGE;
}  // namespace

// n_tiles: 64-row tiles the tile kernel has to run (0: none); n_small: 1 if any
// request goes to the split kernel.  part_o / part_lse are scratch memory of
// n_split * T * H * (HD + 1) floats, needed when n_split > 1.
MLS_API int mls_attention_mma(const void* qkv, void* out, const void* k_pool, const void* v_pool,
                              const int* block_table, int max_blocks, const int* cu_q,
                              const int* ctx_len, int n_req, int n_tokens, int n_heads, int n_kv,
                              int block_size, float scale, int window, int n_tiles, int n_small,
                              int n_split, float* part_o, float* part_lse, long long pool_pages,
                              int* status, int use_tma, cudaStream_t stream) {
    if (n_tokens <= 0 || n_req <= 0) return 0;
    if (n_heads % n_kv || n_split < 1 || n_split > MAX_SPLITS ||
        (n_split > 1 && (!part_o || !part_lse)))
        return MLS_ERR_UNSUPPORTED;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tile_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, TILE_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attention_split_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, SPLIT_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    Params P;
    P.qkv = (const __nv_bfloat16*)qkv;
    P.out = (__nv_bfloat16*)out;
    P.k_pool = (const __nv_bfloat16*)k_pool;
    P.v_pool = (const __nv_bfloat16*)v_pool;
    P.block_table = block_table;
    P.cu_q = cu_q;
    P.ctx_len = ctx_len;
    P.part_o = part_o;
    P.part_lse = part_lse;
    P.max_blocks = max_blocks;
    P.n_req = n_req;
    P.n_tokens = n_tokens;
    P.n_heads = n_heads;
    P.n_kv = n_kv;
    P.group = n_heads / n_kv;
    P.block_size = block_size;
    P.window = window;
    P.n_split = n_split;
    P.small_only = n_small ? 1 : 0;
    P.cluster_merge = 0;
    P.scale_log2 = scale * LOG2E;
    P.status = status;
    P.n_pages = pool_pages;
    const bool tma_ok = use_tma && (block_size == 8 || block_size == 16 || block_size == 32 ||
                                    block_size == 64) && (HD % 64 == 0);
    (void)tma_ok;
#if MLS_HEAD_DIM % 64 == 0
    CUtensorMap kmap, vmap, kmap_wide, vmap_wide;
    if (tma_ok) {
        static bool tma_configured = false;
        if (!tma_configured) {
            cudaError_t e = cudaFuncSetAttribute(attention_split_tma_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 TMA_SMEM);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(attention_tile_tma_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TILE_TMA_SMEM);
            if (e != cudaSuccess) return (int)e;
            tma_configured = true;
        }
        const long long rows = pool_pages * n_kv * block_size;
        if (!pool_map(k_pool, rows, block_size, &kmap) || !pool_map(v_pool, rows, block_size, &vmap) ||
            !pool_map(k_pool, rows, BN, &kmap_wide) || !pool_map(v_pool, rows, BN, &vmap_wide))
            return MLS_ERR_TENSOR_MAP;
    }
#endif
    if (n_tiles > 0) {
#if MLS_HEAD_DIM % 64 == 0
        if (tma_ok)
            MLS_LAUNCH((attention_tile_tma_kernel), dim3(n_tiles, n_kv), dim3(TMA_THREADS),
                       TILE_TMA_SMEM, stream, P, kmap, vmap, kmap_wide, vmap_wide);
        else
#endif
            MLS_LAUNCH((attention_tile_kernel), dim3(n_tiles, n_kv), dim3(NT), TILE_SMEM, stream,
                       P);
        int rc = launch_status();
        if (rc) return rc;
    }
    if (n_small) {
#if MLS_HEAD_DIM % 64 == 0
        if (tma_ok)
            return launch_split_tma(P, Fused{}, kmap, vmap, kmap_wide, vmap_wide, n_tokens, stream);
#endif
        MLS_LAUNCH((attention_split_kernel), dim3(n_req, n_kv, n_split), dim3(NT), SPLIT_SMEM,
                   stream, P);
        int rc = launch_status();
        if (rc) return rc;
        if (n_split > 1) {
            MLS_LAUNCH((attention_merge_kernel), dim3(n_tokens, n_heads),
                       dim3(HD < 32 ? 32 : (HD < 128 ? HD : 128)),
                       0, stream, P);
            rc = launch_status();
            if (rc) return rc;
        }
    }
    return 0;
}

// A step of single decoded tokens (one token a request) with the rotation and the cache
// write inside the attention kernel: q, k and v are read as the n_parts float32 K-parts of
// their projection ([n_parts][n_req][(H + 2 Hkv) * HD], part_stride elements apart), rotated
// by the rows of cos / sin at positions[t]; with `writes` the rotated key and the value go to
// slot_map[t] of the pools.  Otherwise as mls_attention_mma with every request small.
// Head sizes that are multiples of 64 and pages of 8, 16, 32 or 64 only (else
// MLS_ERR_UNSUPPORTED and nothing is launched).
MLS_API int mls_attention_decode_fused(const float* parts, int n_parts, long long part_stride,
                                       const int* positions, const float* cos_t,
                                       const float* sin_t, int max_pos, const int* slot_map,
                                       int writes, void* out, void* k_pool, void* v_pool,
                                       const int* block_table, int max_blocks, const int* cu_q,
                                       const int* ctx_len, int n_req, int n_heads, int n_kv,
                                       int block_size, float scale, int window, int n_split,
                                       float* part_o, float* part_lse, long long pool_pages,
                                       int* status, cudaStream_t stream) {
#if MLS_HEAD_DIM % 64 == 0
    if (n_req <= 0) return 0;
    if (n_heads % n_kv || n_heads / n_kv > 16 || n_split < 1 || n_split > MAX_SPLITS ||
        (n_split > 1 && (!part_o || !part_lse)) || !parts || n_parts < 1 || part_stride % 4 != 0)
        return MLS_ERR_UNSUPPORTED;
    if (!(block_size == 8 || block_size == 16 || block_size == 32 || block_size == 64))
        return MLS_ERR_UNSUPPORTED;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_split_tma_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, TMA_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    CUtensorMap kmap, vmap, kmap_wide, vmap_wide;
    const long long rows = pool_pages * n_kv * block_size;
    if (!pool_map(k_pool, rows, block_size, &kmap) || !pool_map(v_pool, rows, block_size, &vmap) ||
        !pool_map(k_pool, rows, BN, &kmap_wide) || !pool_map(v_pool, rows, BN, &vmap_wide))
        return MLS_ERR_TENSOR_MAP;
    Params P;
    P.qkv = nullptr;
    P.out = (__nv_bfloat16*)out;
    P.k_pool = (const __nv_bfloat16*)k_pool;
    P.v_pool = (const __nv_bfloat16*)v_pool;
    P.block_table = block_table;
    P.cu_q = cu_q;
    P.ctx_len = ctx_len;
    P.part_o = part_o;
    P.part_lse = part_lse;
    P.max_blocks = max_blocks;
    P.n_req = n_req;
    P.n_tokens = n_req;
    P.n_heads = n_heads;
    P.n_kv = n_kv;
    P.group = n_heads / n_kv;
    P.block_size = block_size;
    P.window = window;
    P.n_split = n_split;
    P.small_only = 1;
    P.cluster_merge = 0;
    P.scale_log2 = scale * LOG2E;
    P.status = status;
    P.n_pages = pool_pages;
    Fused F;
    F.parts = parts;
    F.n_parts = n_parts;
    F.part_stride = part_stride;
    F.positions = positions;
    F.cos_t = cos_t;
    F.sin_t = sin_t;
    F.slot_map = slot_map;
    F.k_out = (__nv_bfloat16*)k_pool;
    F.v_out = (__nv_bfloat16*)v_pool;
    F.max_pos = max_pos;
    F.writes = writes ? 1 : 0;
    return launch_split_tma(P, F, kmap, vmap, kmap_wide, vmap_wide, n_req, stream);
#else
    return MLS_ERR_UNSUPPORTED;
#endif
}

MLS_API int mls_attention_head_dim() { return HD; }

// CTAs of the context-split kernel that one SM holds at a time (registers and shared memory
// decide: two at head size 128, more at smaller heads); use_tma as in mls_attention_mma.
// 0 if the driver cannot say.
MLS_API int mls_attention_split_ctas_per_sm(int use_tma) {
    int n = 0;
#if MLS_HEAD_DIM % 64 == 0
    if (use_tma) {
        if (cudaFuncSetAttribute(attention_split_tma_kernel,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, TMA_SMEM) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_split_tma_kernel, TMA_THREADS,
                                                          TMA_SMEM) != cudaSuccess)
            return 0;
        return n;
    }
#endif
    if (cudaFuncSetAttribute(attention_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SPLIT_SMEM) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_split_kernel, NT, SPLIT_SMEM) !=
            cudaSuccess)
        return 0;
    return n;
}
