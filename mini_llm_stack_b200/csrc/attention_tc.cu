// Causal grouped-query attention for prompts and portions on the 5th-generation
// tensor cores (tcgen05), compiled for one head size (64 or 128).
//
// Reference math (train/model.py:55-70): S = (q . k) * scale, key j hidden from the
// query at position p iff j > p (or j <= p - window); softmax and P . V with float32
// scores, maxima, sums and accumulators; P rounded to bfloat16 for the second
// product (kernels/attention_fwd.py:106).
//
// A CTA runs two chains in turn.  A chain is 128 rows, (token, head-in-group) pairs of
// one kv head, that walk key tiles of 128: S = Q K^T into tensor memory, softmax by one
// thread a row, P written over its scores in tensor memory as bfloat16, O += P V with P
// read from there.  While one chain's softmax runs, the tensor cores work for the other:
//   warp 0      brings keys and values in with TMA, one copy per page and 64-wide half
//               (one per half for a run of consecutive pages), into a ring of key tiles
//               and a ring of value tiles;
//   warp 1      issues the products (tcgen05.mma), accumulators in tensor memory;
//   warps 2..5  softmax of chain 0, warps 6..9 of chain 1: read S, mask, exponentiate,
//               write P, rescale O when the running maximum has grown by more than 2^8,
//               and store O at the end.
// Two ways to be two chains:
//   two row tiles   the CTA owns 256 rows; each chain walks all key tiles of its 128 rows,
//                   and a key tile brought in once serves both (steps with many rows);
//   two key halves  the CTA owns 128 rows; chain 0 walks the even key tiles, chain 1 the
//                   odd ones, and their (maximum, sum, O) are merged at the end (steps
//                   with too few rows to fill the SMs otherwise).
// Every wait is bounded and reports MLS_STATUS_TIMEOUT.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"
#include <map>
#include <mutex>
#include <tuple>

#ifndef MLS_HEAD_DIM
#error "compile with -DMLS_HEAD_DIM=<head size>"
#endif

#if MLS_HEAD_DIM == 64 || MLS_HEAD_DIM == 128
namespace {
using namespace mls_tma;
using namespace mls_tc;

constexpr int HD = MLS_HEAD_DIM;
constexpr int CHAIN_ROWS = 128;                  // rows of a chain
constexpr int BN = 128;                          // keys of a tile
constexpr int HALVES = HD / 64;
constexpr int BLOCK = 128 * 128;                 // bytes of [128 rows][64 elements]: 16 KB
constexpr int KBLOCK = BN * 128;                 // bytes of [128 keys][64 elements]: 16 KB
constexpr int Q_BYTES = HALVES * BLOCK;          // per chain
constexpr int K_STAGE = HALVES * KBLOCK, V_STAGE = HALVES * KBLOCK;
constexpr int K_STAGES = HD == 128 ? 3 : 4, V_STAGES = HD == 128 ? 2 : 4;
constexpr int SOFTMAX_THREADS = 256;             // one thread a row, two chains
constexpr int THREADS = 64 + SOFTMAX_THREADS;
constexpr int TMEM_COLS = 512;                   // S0 | S1 | O0 | O1, 128 columns each
constexpr int COL_S = 0, COL_O = 2 * BN;
static_assert(COL_O + BN + HD <= TMEM_COLS, "tensor memory columns");
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;             // log2: P stays below 2^8

// barrier slots
constexpr int B_K_FULL = 0, B_K_EMPTY = K_STAGES, B_V_FULL = 2 * K_STAGES,
              B_V_EMPTY = B_V_FULL + V_STAGES, B_S_FULL = B_V_EMPTY + V_STAGES,   // [chain]
              B_P_FULL = B_S_FULL + 2, B_O_REST = B_P_FULL + 2, B_Q_FULL = B_O_REST + 2,
              N_BARS = B_Q_FULL + 1;
constexpr int SMEM_BYTES = 2 * Q_BYTES + K_STAGES * K_STAGE + V_STAGES * V_STAGE + 8 * N_BARS + 16;

struct Params {
    const __nv_bfloat16* qkv;
    __nv_bfloat16* out;
    const int* block_table;
    const int* cu_q;
    const int* ctx_len;
    int max_blocks, n_req, n_heads, n_kv, group, block_size, window, small_only;
    int two_tiles;                       // 1: a CTA owns two row tiles; 0: one, its keys in halves
    float scale_log2;
    int* status;
    long long n_pages;                   // pages of the pool: [Hkv, pages, block, HD]
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ bool is_small(int q_len, int group) { return q_len * group <= 16; }

// address of the 16-byte chunk `chunk` of row `row` in a [..][128 rows][64] block set
__device__ __forceinline__ uint32_t swz(uint32_t tile, int row, int chunk) {
    return tile + (chunk >> 3) * BLOCK + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}
#define MLS_STATUS_BAD_SMEM 16       // dynamic shared memory is not 1024-byte aligned

__global__ void __launch_bounds__(THREADS)
attention_tc_kernel(const Params P, const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap vmap,
                    const __grid_constant__ CUtensorMap kmap_wide,
                    const __grid_constant__ CUtensorMap vmap_wide) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ float2 chain_state[2][CHAIN_ROWS];    // (maximum, sum) of a row, per chain
    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {                          // the swizzled tiles need this alignment
        if (threadIdx.x == 0 && P.status) atomicOr(P.status, MLS_STATUS_BAD_SMEM);
        return;
    }
    uint8_t* gbase = smem_raw;
    const uint32_t q_smem = base, k_smem = base + 2 * Q_BYTES, v_smem = k_smem + K_STAGES * K_STAGE;
    const uint32_t bars = v_smem + V_STAGES * V_STAGE;
    auto bar = [&](int i) { return bars + 8u * i; };
    volatile uint32_t* tmem_slot =
        reinterpret_cast<volatile uint32_t*>(gbase + (bars - base) + 8 * N_BARS);

    // which request and which tile of rows of it; the last rows see the most keys and
    // go first, for all kv heads (blockIdx.x) before the next tile
    const int tile_rows = P.two_tiles ? 2 * CHAIN_ROWS : CHAIN_ROWS;
    int r = 0, tile = blockIdx.y, q_len = 0, rows = 0;
    for (; r < P.n_req; ++r) {
        q_len = P.cu_q[r + 1] - P.cu_q[r];
        rows = q_len * P.group;
        int tiles = (P.small_only && is_small(q_len, P.group)) ? 0 : (rows + tile_rows - 1) / tile_rows;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (r >= P.n_req) return;
    tile = (rows + tile_rows - 1) / tile_rows - 1 - tile;
    const int kvh = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok0 = P.cu_q[r], ctx = P.ctx_len[r];
    const int row0 = tile * tile_rows;
    const int pos0 = ctx - q_len;
    const int i_first = row0 / P.group;
    const int i_last = (min(rows, row0 + tile_rows) - 1) / P.group;
    const int hi = pos0 + i_last;
    const int lo = P.window > 0 ? max(0, pos0 + i_first - P.window + 1) : 0;
    const int* table = P.block_table + (size_t)r * P.max_blocks;
    const int kbase0 = (lo / BN) * BN;
    const int n_tiles = (hi - kbase0) / BN + 1;
    // steps of each chain, and the key tile of chain c's step i
    int n_steps[2];
    if (P.two_tiles) {
        // chain 0's rows end earlier: it may need a key tile less; chain 1 may have no rows
        const int last0 = (min(rows, row0 + CHAIN_ROWS) - 1) / P.group;
        n_steps[0] = (pos0 + last0 - kbase0) / BN + 1;
        n_steps[1] = row0 + CHAIN_ROWS < rows ? n_tiles : 0;
    } else {
        n_steps[0] = (n_tiles + 1) / 2;
        n_steps[1] = n_tiles / 2;
    }
    const int chains = n_steps[1] > 0 ? 2 : 1;
    auto key_tile = [&](int c, int i) { return P.two_tiles ? i : 2 * i + c; };

    // a softmax thread's row of Q (its half of the row when both chains share the rows) is
    // asked for before the set-up below, so that the two latencies overlap
    const int chain = warp >= 2 ? (warp - 2) >> 2 : 0;          // of a softmax warp
    const int quarter = warp & 3;                                // its lanes of tensor memory
    const int row_in = quarter * 32 + lane;                      // row of the chain = TMEM lane
    constexpr int Q_CHUNKS = HD / 8;                             // 16-byte chunks of a row
    const int q_chunks = P.two_tiles ? Q_CHUNKS : Q_CHUNKS / 2;  // this thread's
    const int q_chunk0 = P.two_tiles ? 0 : chain * (Q_CHUNKS / 2);
    const int row = row0 + (P.two_tiles ? chain * CHAIN_ROWS : 0) + row_in;
    const bool live = warp >= 2 && row < rows;
    const int ti = live ? row / P.group : 0, g = live ? row - ti * P.group : 0;
    uint4 q_regs[Q_CHUNKS];
    if (warp >= 2) {
        const int row_w = (P.n_heads + 2 * P.n_kv) * HD;
        const __nv_bfloat16* src =
            P.qkv + (size_t)(tok0 + ti) * row_w + (size_t)(kvh * P.group + g) * HD;
#pragma unroll
        for (int i = 0; i < Q_CHUNKS; ++i) {
            q_regs[i] = make_uint4(0u, 0u, 0u, 0u);
            if (live && i < q_chunks)
                q_regs[i] = *reinterpret_cast<const uint4*>(src + (q_chunk0 + i) * 8);
        }
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < K_STAGES; ++s) {
            mbar_init(bar(B_K_FULL + s), 1);
            mbar_init(bar(B_K_EMPTY + s), 1);
        }
        for (int s = 0; s < V_STAGES; ++s) {
            mbar_init(bar(B_V_FULL + s), 1);
            mbar_init(bar(B_V_EMPTY + s), 1);
        }
        for (int c = 0; c < 2; ++c) {
            mbar_init(bar(B_S_FULL + c), 1);
            mbar_init(bar(B_P_FULL + c), CHAIN_ROWS);
            mbar_init(bar(B_O_REST + c), 1);
        }
        mbar_init(bar(B_Q_FULL), SOFTMAX_THREADS);
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool timed_out = false;

    if (warp == 0) {
        // -------------------------------------------------------------- TMA producer
        const int bs = P.block_size, ppt = BN / bs;
        const uint32_t page_bytes = bs * 128;
        // one ring for keys, one for values; `which` 0 = keys, 1 = values
        auto load = [&](int t, int which) -> bool {
            const int stages = which ? V_STAGES : K_STAGES;
            const int slot = t % stages;
            const uint32_t full = bar((which ? B_V_FULL : B_K_FULL) + slot);
            const uint32_t empty = bar((which ? B_V_EMPTY : B_K_EMPTY) + slot);
            if (!mbar_wait(empty, ((t / stages) & 1) ^ 1)) return false;
            const int kb = kbase0 + t * BN;
            const uint32_t stage = which ? v_smem + slot * V_STAGE : k_smem + slot * K_STAGE;
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
            // pages that follow one another in the pool are one contiguous run of
            // rows: a single wide copy per 64-wide half instead of one per page
            const int first = __shfl_sync(0xffffffffu, page, 0);
            if (mask == all && __all_sync(0xffffffffu, lane >= ppt || page == first + lane)) {
                if (lane == 0) mbar_arrive_expect_tx(full, BN * 128 * HALVES);
                __syncwarp();
                if (lane < HALVES)
                    tma_load_2d(stage + lane * KBLOCK, which ? &vmap_wide : &kmap_wide, lane * 64,
                                (int)((kvh * P.n_pages + first) * bs), full);
                return true;
            }
            if (mask != all) {
                // pages that are not keys of this request read as zeros
                for (int pi = 0; pi < ppt; ++pi) {
                    if ((mask >> pi) & 1u) continue;
                    for (int part = 0; part < HALVES; ++part) {
                        const uint32_t dst = stage + part * KBLOCK + pi * page_bytes;
                        for (uint32_t o = lane * 16; o < page_bytes; o += 512)
                            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(dst + o),
                                         "r"(0u) : "memory");
                    }
                }
                fence_proxy_async();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_expect_tx(full, __popc(mask) * page_bytes * HALVES);
            __syncwarp();
            if (valid) {
                const int y = (int)((kvh * P.n_pages + page) * bs);
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                    tma_load_2d(stage + h * KBLOCK + lane * page_bytes, which ? &vmap : &kmap,
                                h * 64, y, full);
            }
            return true;
        };
        for (int t = 0; t < n_tiles; ++t) {
            if (!load(t, 0) || !load(t, 1)) {
                timed_out = true;
                break;
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(BN, 0);
            constexpr uint32_t idesc_o = umma_idesc(HD, 1);
            // S_c = Q_c K^T for chain c's step i, over whatever the chain's score columns hold
            // (the product of its step before has read its P from there: the tensor cores
            // run the instructions in the order they were issued)
            auto issue_s = [&](int c, int i) -> bool {
                const int t = key_tile(c, i), slot = t % K_STAGES;
                if (!mbar_wait(bar(B_K_FULL + slot), (t / K_STAGES) & 1)) return false;
                tc_fence_after();
                const uint32_t k_src = k_smem + slot * K_STAGE;
                const uint32_t q_src = q_smem + (P.two_tiles ? c * Q_BYTES : 0);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * BLOCK + (kk & 3) * 32;
                    umma(tmem + COL_S + c * BN, umma_desc(q_src + off), umma_desc(k_src + off),
                         idesc_s, kk ? 1u : 0u);
                }
                umma_commit(bar(B_S_FULL + c));
                // the keys are done with after the last chain that reads them
                if (!P.two_tiles || c == chains - 1) umma_commit(bar(B_K_EMPTY + slot));
                return true;
            };
            // O_c += P_c V for chain c's step i, P read from tensor memory
            auto issue_pv = [&](int c, int i) -> bool {
                const int t = key_tile(c, i), slot = t % V_STAGES;
                if (!mbar_wait(bar(B_P_FULL + c), i & 1)) return false;
                if (!mbar_wait(bar(B_V_FULL + slot), (t / V_STAGES) & 1)) return false;
                tc_fence_after();
                const uint32_t v_src = v_smem + slot * V_STAGE;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk)
                    umma_ts(tmem + COL_O + c * BN, tmem + COL_S + c * BN + kk * 8,
                            umma_desc_mn(v_src + kk * 16 * 128, KBLOCK), idesc_o, (i | kk) ? 1u : 0u);
                umma_commit(bar(B_O_REST + c));            // O_c holds step i
                if (!P.two_tiles || c == chains - 1) umma_commit(bar(B_V_EMPTY + slot));
                return true;
            };
            if (!mbar_wait(bar(B_Q_FULL), 0)) timed_out = true;
            for (int c = 0; c < chains && !timed_out; ++c)
                if (n_steps[c] > 0 && !issue_s(c, 0)) timed_out = true;
            const int most = max(n_steps[0], n_steps[1]);
            for (int i = 0; i < most && !timed_out; ++i) {
                for (int c = 0; c < chains; ++c) {
                    if (i >= n_steps[c]) continue;
                    if (!issue_pv(c, i) || (i + 1 < n_steps[c] && !issue_s(c, i + 1))) {
                        timed_out = true;
                        break;
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------- softmax, correction, epilogue
        // One thread a row: warps 2..5 are chain 0, warps 6..9 chain 1; a warp reaches the
        // lanes of tensor memory of its quarter (warp index modulo four).
        const int c = chain;
        const int pos = live ? pos0 + ti : -1;
        const int lo_row = P.window > 0 ? pos - P.window + 1 : 0;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t s_addr = tmem + lane_base + COL_S + c * BN;
        const uint32_t o_addr = tmem + lane_base + COL_O + c * BN;

        // this thread's part of Q into shared memory, in the operand layout
        {
            const uint32_t q_dst = q_smem + (P.two_tiles ? c * Q_BYTES : 0);
#pragma unroll
            for (int i = 0; i < Q_CHUNKS; ++i) {
                if (i < q_chunks) {
                    const uint4 v = q_regs[i];
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n"
                                 ::"r"(swz(q_dst, row_in, q_chunk0 + i)),
                                   "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                }
            }
            fence_proxy_async();
            mbar_arrive(bar(B_Q_FULL));
        }

        float m_used = -INFINITY, l = 0.f;
        const int steps = n_steps[c];
        for (int i = 0; i < steps && !timed_out; ++i) {
            const int kbase = kbase0 + key_tile(c, i) * BN;
            if (!mbar_wait(bar(B_S_FULL + c), i & 1)) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            // the row of raw scores into registers (the scale to the log2 domain is folded
            // into the exponent's multiply-add); a key needs a mask only on the diagonal
            // tiles and at a window's edge
            float sc[BN];
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t a[16];
                tmem_ld16(s_addr + c0, a);
#pragma unroll
                for (int e = 0; e < 16; ++e) sc[c0 + e] = __uint_as_float(a[e]);
            }
            tmem_ld_wait();
            const bool masked = kbase + BN - 1 > pos || kbase < lo_row;
            if (__any_sync(0xffffffffu, masked)) {
#pragma unroll
                for (int e = 0; e < BN; ++e) {
                    const int jj = kbase + e;
                    if (jj > pos || jj < lo_row) sc[e] = -INFINITY;
                }
            }
            // eight running maxima, then their maximum: no chain of dependent steps
            float mx[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) mx[e] = sc[e];
#pragma unroll
            for (int e = 8; e < BN; ++e) mx[e & 7] = fmaxf(mx[e & 7], sc[e]);
            const float m_tile = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                                       fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]))) *
                                 P.scale_log2;    // the scale is positive
            const bool grow = m_tile > m_used + RESCALE_STEP || (m_used == -INFINITY && m_tile > m_used);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? m_tile : m_used;
                const float cf = (grow && m_used != -INFINITY) ? fast_exp2(m_used - m_new) : 1.0f;
                if (i > 0) {
                    // O must be at rest: the product of the step before has to be done
                    if (!mbar_wait(bar(B_O_REST + c), (i - 1) & 1)) {
                        timed_out = true;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        uint32_t v[16], w[16];
                        tmem_ld16(o_addr + c0, v);
                        tmem_ld16(o_addr + c0 + 16, w);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            v[e] = __float_as_uint(__uint_as_float(v[e]) * cf);
                            w[e] = __float_as_uint(__uint_as_float(w[e]) * cf);
                        }
                        tmem_st16(o_addr + c0, v);
                        tmem_st16(o_addr + c0 + 16, w);
                    }
                }
                l *= cf;
                m_used = m_new;
            }
            // probabilities, their sum, and P over the scores as the next product's operand:
            // keys 2j, 2j + 1 share column j
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
            float part[4] = {0.f, 0.f, 0.f, 0.f};             // four running sums
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t pk[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const float p0 = fast_exp2(fmaf(sc[c0 + 2 * u], P.scale_log2, neg_m));
                    const float p1 = fast_exp2(fmaf(sc[c0 + 2 * u + 1], P.scale_log2, neg_m));
                    part[u & 3] += p0 + p1;
                    __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    pk[u] = *reinterpret_cast<uint32_t*>(&h);
                }
                tmem_st16(s_addr + c0 / 2, pk);
            }
            l += (part[0] + part[1]) + (part[2] + part[3]);
            tmem_st_wait();                    // P and a rescaled O are in place
            tc_fence_before();
            mbar_arrive(bar(B_P_FULL + c));
        }
        // the chain's last product (the products end in the order they were issued)
        if (!timed_out && steps > 0 && !mbar_wait(bar(B_O_REST + c), (steps - 1) & 1))
            timed_out = true;
        tc_fence_after();
        if (P.two_tiles) {
            // the chain's rows are its own: O / l
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16* dst = P.out + (size_t)(tok0 + ti) * P.n_heads * HD +
                                 (size_t)(kvh * P.group + g) * HD;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t v[16], w[16];
                tmem_ld16(o_addr + c0, v);
                tmem_ld16(o_addr + c0 + 16, w);
                tmem_ld_wait();
                if (live) {
                    uint32_t o[16];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * e]) * inv,
                                                                 __uint_as_float(v[2 * e + 1]) * inv);
                        o[e] = *reinterpret_cast<uint32_t*>(&h);
                        h = __floats2bfloat162_rn(__uint_as_float(w[2 * e]) * inv,
                                                  __uint_as_float(w[2 * e + 1]) * inv);
                        o[8 + e] = *reinterpret_cast<uint32_t*>(&h);
                    }
#pragma unroll
                    for (int e = 0; e < 16; e += 4)
                        *reinterpret_cast<uint4*>(dst + c0 + 2 * e) = make_uint4(o[e], o[e + 1], o[e + 2], o[e + 3]);
                }
            }
        } else {
            // both chains hold the same rows over different keys: each thread merges its half
            // of the columns from the two accumulators (chain 0's first)
            chain_state[c][row_in] = make_float2(m_used, l);
            tc_fence_before();
            asm volatile("bar.sync 1, %0;\n" ::"n"(SOFTMAX_THREADS) : "memory");
            tc_fence_after();
            const float2 s0 = chain_state[0][row_in], s1 = chain_state[1][row_in];
            const float m = fmaxf(s0.x, s1.x);
            const float f0 = s0.x == -INFINITY ? 0.f : fast_exp2(s0.x - m);
            const float f1 = s1.x == -INFINITY ? 0.f : fast_exp2(s1.x - m);
            const float l_row = s0.y * f0 + s1.y * f1;
            const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
            const float w0 = f0 * inv, w1 = f1 * inv;
            const bool second = n_steps[1] > 0;            // else its accumulator was never written
            constexpr int HO = HD / 2;
            const uint32_t o0 = tmem + lane_base + COL_O + c * HO, o1 = o0 + BN;
            __nv_bfloat16* dst = P.out + (size_t)(tok0 + ti) * P.n_heads * HD +
                                 (size_t)(kvh * P.group + g) * HD + c * HO;
#pragma unroll
            for (int c0 = 0; c0 < HO; c0 += 16) {
                uint32_t v[16], w[16];
                tmem_ld16(o0 + c0, v);
                if (second) tmem_ld16(o1 + c0, w);
                tmem_ld_wait();
                if (live) {
                    uint32_t o[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float a = __uint_as_float(v[2 * e]) * w0, b = __uint_as_float(v[2 * e + 1]) * w0;
                        if (second) {
                            a = fmaf(__uint_as_float(w[2 * e]), w1, a);
                            b = fmaf(__uint_as_float(w[2 * e + 1]), w1, b);
                        }
                        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                        o[e] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(dst + c0) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(dst + c0 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                }
            }
        }
    }
    if (timed_out && (threadIdx.x & 31) == 0 && P.status) atomicOr(P.status, MLS_STATUS_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

struct MapKey {
    const void* ptr;
    long long rows;
    int block;
    bool operator<(const MapKey& o) const {
        return std::tie(ptr, rows, block) < std::tie(o.ptr, o.rows, o.block);
    }
};
std::map<MapKey, CUtensorMap> g_maps;
std::mutex g_lock;

bool pool_map(const void* pool, long long pool_rows, int block, CUtensorMap* out) {
    std::lock_guard<std::mutex> guard(g_lock);
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

// MLS_B200_ATTENTION_ROWS = 128 | 256 fixes the rows of a CTA (for measurements and tests);
// mls_attention_tc_set_rows does the same at run time (0: choose by the step).
int g_forced_rows = [] {
    const char* v = getenv("MLS_B200_ATTENTION_ROWS");
    return v ? atoi(v) : 0;
}();
}  // namespace
#endif

MLS_API void mls_attention_tc_set_rows(int rows) {
#if MLS_HEAD_DIM == 64 || MLS_HEAD_DIM == 128
    g_forced_rows = rows;
#endif
}

// Rows of one tile of mls_attention_tc (0: this head size has no such kernel).
MLS_API int mls_attention_tc_rows() {
#if MLS_HEAD_DIM == 64 || MLS_HEAD_DIM == 128
    return CHAIN_ROWS;
#else
    return 0;
#endif
}

// Prompts and portions of a step: n_tiles = number of tiles of mls_attention_tc_rows() rows
// over the requests, n_tiles_wide = of twice as many rows (requests that the split kernel
// takes are left out of both when skip_small is set).  A CTA takes a wide tile when those
// give every SM one, else a tile whose keys it walks in two halves.  Returns
// MLS_ERR_UNSUPPORTED (and launches nothing) for head or page sizes it does not take.
MLS_API int mls_attention_tc(const void* qkv, void* out, const void* k_pool, const void* v_pool,
                             const int* block_table, int max_blocks, const int* cu_q,
                             const int* ctx_len, int n_req, int n_heads, int n_kv, int block_size,
                             float scale, int window, int n_tiles, int n_tiles_wide,
                             int skip_small, long long pool_pages, int* status,
                             cudaStream_t stream) {
#if MLS_HEAD_DIM == 64 || MLS_HEAD_DIM == 128
    if (n_tiles <= 0 || n_req <= 0) return 0;
    if (n_heads % n_kv) return MLS_ERR_UNSUPPORTED;
    if (!(block_size == 8 || block_size == 16 || block_size == 32 || block_size == 64))
        return MLS_ERR_UNSUPPORTED;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    CUtensorMap kmap, vmap, kmap_wide, vmap_wide;
    const long long rows = pool_pages * n_kv * block_size;
    if (!pool_map(k_pool, rows, block_size, &kmap) || !pool_map(v_pool, rows, block_size, &vmap) ||
        !pool_map(k_pool, rows, BN, &kmap_wide) || !pool_map(v_pool, rows, BN, &vmap_wide))
        return MLS_ERR_TENSOR_MAP;
    Params P;
    P.qkv = (const __nv_bfloat16*)qkv;
    P.out = (__nv_bfloat16*)out;
    P.block_table = block_table;
    P.cu_q = cu_q;
    P.ctx_len = ctx_len;
    P.max_blocks = max_blocks;
    P.n_req = n_req;
    P.n_heads = n_heads;
    P.n_kv = n_kv;
    P.group = n_heads / n_kv;
    P.block_size = block_size;
    P.window = window;
    P.small_only = skip_small ? 1 : 0;
    P.two_tiles = (n_tiles_wide > 0 && (long long)n_tiles_wide * n_kv >= sm_count()) ? 1 : 0;
    if (g_forced_rows == CHAIN_ROWS) P.two_tiles = 0;
    if (g_forced_rows == 2 * CHAIN_ROWS && n_tiles_wide > 0) P.two_tiles = 1;
    P.scale_log2 = scale * LOG2E;
    P.status = status;
    P.n_pages = pool_pages;
    MLS_LAUNCH((attention_tc_kernel), dim3(n_kv, P.two_tiles ? n_tiles_wide : n_tiles),
               dim3(THREADS), SMEM_BYTES, stream, P, kmap, vmap, kmap_wide, vmap_wide);
    return launch_status();
#else
    return MLS_ERR_UNSUPPORTED;
#endif
}
