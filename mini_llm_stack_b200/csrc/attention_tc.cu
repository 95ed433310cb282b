// Causal grouped-query attention for prompts and portions on the 5th-generation
// tensor cores (tcgen05), compiled for one head size (64 or 128).
//
// Reference math (train/model.py:55-70): S = (q . k) * scale, key j hidden from the
// query at position p iff j > p (or j <= p - window); softmax and P . V with float32
// scores, maxima, sums and accumulators; P rounded to bfloat16 for the second
// product (kernels/attention_fwd.py:106).
//
// One CTA owns 128 rows, (token, head-in-group) pairs of one kv head, and walks the
// keys 128 at a time (a tcgen05.mma costs about the same whatever its width, so
// wide tiles pay):
//   warp 0      brings keys and values in with TMA, one copy per page and 64-wide half,
//               into a ring of two key tiles and a ring of two value tiles;
//   warp 1      issues S = Q K^T and O += P V (tcgen05.mma), accumulators in TMEM;
//   warps 2..9  two threads per row, each half of the tile's keys: read S from TMEM, mask,
//               exponentiate, write P to shared memory as the next product's operand,
//               rescale O when the running maximum has grown by more than 2^8, and
//               store O at the end.
// S is double-buffered in TMEM and P in shared memory, so the next tile's Q K^T and
// this tile's P V run during the next tile's softmax.
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
constexpr int CHAINS = 1;                        // row blocks of 128 a CTA owns
constexpr int ROWS = 128 * CHAINS;               // rows of a tile
constexpr int BN = 128;                          // keys of a tile: the wider a tcgen05.mma, the better
constexpr int HALVES = HD / 64;
constexpr int BLOCK = 128 * 128;                 // bytes of [128 rows][64 elements]: 16 KB
constexpr int KBLOCK = BN * 128;                 // bytes of [128 keys][64 elements]: 16 KB
constexpr int Q_BYTES = HALVES * BLOCK;          // per chain
constexpr int P_BYTES = (BN / 64) * BLOCK;       // per chain and buffer: [128 rows][128 keys]
constexpr int P_BUFS = 2;                        // the softmax writes P(j+1) while P(j) V runs
constexpr int K_STAGE = HALVES * KBLOCK, V_STAGE = HALVES * KBLOCK;
constexpr int K_STAGES = 2, V_STAGES = 2;
constexpr int SOFTMAX_THREADS = 256 * CHAINS;      // two warps share 32 rows, half the keys each
constexpr int THREADS = 64 + SOFTMAX_THREADS;
constexpr int TMEM_COLS = 512;                   // per chain S0 | S1, then per chain O
constexpr int COL_S = 0, COL_O = CHAINS * 2 * BN;
static_assert(COL_O + CHAINS * HD <= TMEM_COLS, "tensor memory columns");
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;             // log2: P stays below 2^8

// barrier slots
constexpr int B_K_FULL = 0, B_K_EMPTY = K_STAGES, B_V_FULL = 2 * K_STAGES,
              B_V_EMPTY = B_V_FULL + V_STAGES, B_S_FULL = B_V_EMPTY + V_STAGES,       // [chain][2]
              B_S_EMPTY = B_S_FULL + 2 * CHAINS, B_P_FULL = B_S_EMPTY + 2 * CHAINS,   // [chain][buf]
              B_P_EMPTY = B_P_FULL + P_BUFS * CHAINS, B_Q_FULL = B_P_EMPTY + P_BUFS * CHAINS,
              N_BARS = B_Q_FULL + 1;
// no alignment slack: two CTAs must fit one SM; the kernel checks the alignment
constexpr int SMEM_BYTES = CHAINS * (Q_BYTES + P_BUFS * P_BYTES) + K_STAGES * K_STAGE +
                           V_STAGES * V_STAGE +
                           8 * N_BARS + 16;

struct Params {
    const __nv_bfloat16* qkv;
    __nv_bfloat16* out;
    const int* block_table;
    const int* cu_q;
    const int* ctx_len;
    int max_blocks, n_req, n_heads, n_kv, group, block_size, window, small_only;
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
    __shared__ float row_max[2][2][128];         // [tile parity][half of the keys][row]
    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {                          // the swizzled tiles need this alignment
        if (threadIdx.x == 0 && P.status) atomicOr(P.status, MLS_STATUS_BAD_SMEM);
        return;
    }
    uint8_t* gbase = smem_raw;
    const uint32_t q_smem = base, p_smem = base + CHAINS * Q_BYTES,
                   k_smem = p_smem + CHAINS * P_BUFS * P_BYTES, v_smem = k_smem + K_STAGES * K_STAGE;
    const uint32_t bars = v_smem + V_STAGES * V_STAGE;
    auto bar = [&](int i) { return bars + 8u * i; };
    volatile uint32_t* tmem_slot =
        reinterpret_cast<volatile uint32_t*>(gbase + (bars - base) + 8 * N_BARS);

    // which request and which 128-row tile of it; the last rows see the most keys and
    // go first, for all kv heads (blockIdx.x) before the next tile
    int r = 0, tile = blockIdx.y, q_len = 0, rows = 0;
    for (; r < P.n_req; ++r) {
        q_len = P.cu_q[r + 1] - P.cu_q[r];
        rows = q_len * P.group;
        int tiles = (P.small_only && is_small(q_len, P.group)) ? 0 : (rows + ROWS - 1) / ROWS;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (r >= P.n_req) return;
    tile = (rows + ROWS - 1) / ROWS - 1 - tile;
    const int kvh = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok0 = P.cu_q[r], ctx = P.ctx_len[r];
    const int row0 = tile * ROWS;
    const int pos0 = ctx - q_len;
    const int i_first = row0 / P.group;
    const int i_last = (min(rows, row0 + ROWS) - 1) / P.group;
    const int hi = pos0 + i_last;
    const int lo = P.window > 0 ? max(0, pos0 + i_first - P.window + 1) : 0;
    const int* table = P.block_table + (size_t)r * P.max_blocks;
    const int kbase0 = (lo / BN) * BN;
    const int n_tiles = (hi - kbase0) / BN + 1;

    // a softmax thread's half of its row of Q is asked for before the set-up below, so
    // that the two latencies overlap
    uint4 q_regs[HD / 16];
    if (warp >= 2) {
        const int q = warp & 3, half = (warp - 2) >> 2;
        const int row = row0 + q * 32 + lane;
        const bool live = row < rows;
        const int ti = live ? row / P.group : 0, g = live ? row - ti * P.group : 0;
        const int row_w = (P.n_heads + 2 * P.n_kv) * HD;
        const __nv_bfloat16* src =
            P.qkv + (size_t)(tok0 + ti) * row_w + (size_t)(kvh * P.group + g) * HD;
#pragma unroll
        for (int i = 0; i < HD / 16; ++i) {
            q_regs[i] = make_uint4(0u, 0u, 0u, 0u);
            if (live) q_regs[i] = *reinterpret_cast<const uint4*>(src + (half * (HD / 16) + i) * 8);
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
        for (int s = 0; s < 2 * CHAINS; ++s) {
            mbar_init(bar(B_S_FULL + s), 1);
            mbar_init(bar(B_S_EMPTY + s), SOFTMAX_THREADS);
        }
        for (int c = 0; c < P_BUFS * CHAINS; ++c) {
            mbar_init(bar(B_P_FULL + c), SOFTMAX_THREADS);
            mbar_init(bar(B_P_EMPTY + c), 1);
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
            // S(c, j) = Q_c K_j^T into chain c's score buffer j & 1
            auto issue_qk = [&](int c, int j) -> bool {
                const int slot = j % K_STAGES, sb = j & 1;
                if (!mbar_wait(bar(B_K_FULL + slot), (j / K_STAGES) & 1)) return false;
                if (!mbar_wait(bar(B_S_EMPTY + 2 * c + sb), ((j >> 1) & 1) ^ 1)) return false;
                tc_fence_after();
                const uint32_t k_src = k_smem + slot * K_STAGE;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t q_off = c * Q_BYTES + (kk >> 2) * BLOCK + (kk & 3) * 32;
                    const uint32_t k_off = (kk >> 2) * KBLOCK + (kk & 3) * 32;
                    umma(tmem + COL_S + (2 * c + sb) * BN, umma_desc(q_smem + q_off),
                         umma_desc(k_src + k_off), idesc_s, kk ? 1u : 0u);
                }
                umma_commit(bar(B_S_FULL + 2 * c + sb));
                if (c == CHAINS - 1) umma_commit(bar(B_K_EMPTY + slot));   // the keys are done with
                return true;
            };
            if (!mbar_wait(bar(B_Q_FULL), 0)) timed_out = true;
            for (int c = 0; c < CHAINS && !timed_out && n_tiles > 0; ++c)
                if (!issue_qk(c, 0)) timed_out = true;
            for (int j = 0; j < n_tiles && !timed_out; ++j) {
                for (int c = 0; c < CHAINS && !timed_out; ++c) {
                    if (j + 1 < n_tiles && !issue_qk(c, j + 1)) {
                        timed_out = true;
                        break;
                    }
                    const int pb = j % P_BUFS;
                    if (!mbar_wait(bar(B_P_FULL + P_BUFS * c + pb), (j / P_BUFS) & 1)) {
                        timed_out = true;
                        break;
                    }
                    if (c == 0 && !mbar_wait(bar(B_V_FULL + j % V_STAGES), (j / V_STAGES) & 1)) {
                        timed_out = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t v_src = v_smem + (j % V_STAGES) * V_STAGE;
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk)
                        umma(tmem + COL_O + c * HD,
                             umma_desc(p_smem + (P_BUFS * c + pb) * P_BYTES + (kk >> 2) * BLOCK +
                                       (kk & 3) * 32),
                             umma_desc_mn(v_src + kk * 16 * 128, KBLOCK), idesc_o,
                             (j | kk) ? 1u : 0u);
                    umma_commit(bar(B_P_EMPTY + P_BUFS * c + pb));   // this P is free, O holds tile j
                }
                umma_commit(bar(B_V_EMPTY + (j % V_STAGES)));  // the values of tile j are done with
            }
        }
    } else {
        // ------------------------------------------------- softmax, correction, epilogue
        // Warps w and w + 4 own the same 32 rows (TMEM lanes of quarter w % 4); the first
        // takes keys 0..63 of a tile, the second keys 64..127, and of O and of Q each
        // half of the columns.  A scheduler thus has two warps to issue from.  The pair
        // meets once a tile (named barrier) to agree on the row maximum.
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;                      // which half of the keys
        const int row_in = q * 32 + lane;                      // row of the tile = TMEM lane
        const int row = row0 + row_in;
        constexpr int HB = BN / 2;                             // keys of a half
        constexpr int HO = HD / 2;                             // columns of O of a half
        const bool live = row < rows;
        const int ti = live ? row / P.group : 0, g = live ? row - ti * P.group : 0;
        const int pos = live ? pos0 + ti : -1;
        const int lo_row = P.window > 0 ? pos - P.window + 1 : 0;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;\n" ::"r"(1 + q) : "memory"); };

        // this thread's half of its row of Q into shared memory, in the operand layout
        {
#pragma unroll
            for (int i = 0; i < HD / 16; ++i) {
                const uint4 v = q_regs[i];
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n"
                             ::"r"(swz(q_smem, row_in, half * (HD / 16) + i)),
                               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
            }
            fence_proxy_async();
            mbar_arrive(bar(B_Q_FULL));
        }

        float m_used = -INFINITY, l = 0.f;                     // l: the sum over this half's keys
        for (int j = 0; j < n_tiles && !timed_out; ++j) {
            const int sb = j & 1;
            const int kbase = kbase0 + j * BN + half * HB;     // first key of this half
            if (!mbar_wait(bar(B_S_FULL + sb), (j >> 1) & 1)) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            const uint32_t s_addr = tmem + lane_base + COL_S + sb * BN + half * HB;
            // this half of the row of raw scores into registers (the scale to the log2
            // domain is folded into the exponent's multiply-add); a key needs a mask only
            // on the diagonal tiles and at a window's edge
            float sc[HB];
#pragma unroll
            for (int c0 = 0; c0 < HB; c0 += 32) {
                uint32_t a[16], b[16];
                tmem_ld16(s_addr + c0, a);
                tmem_ld16(s_addr + c0 + 16, b);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    sc[c0 + e] = __uint_as_float(a[e]);
                    sc[c0 + 16 + e] = __uint_as_float(b[e]);
                }
            }
            // the scores are in registers: the tile after next may overwrite them
            tc_fence_before();
            mbar_arrive(bar(B_S_EMPTY + sb));
            const bool masked = kbase + HB - 1 > pos || kbase < lo_row;
            if (__any_sync(0xffffffffu, masked)) {
#pragma unroll
                for (int e = 0; e < HB; ++e) {
                    const int jj = kbase + e;
                    if (jj > pos || jj < lo_row) sc[e] = -INFINITY;
                }
            }
            // eight running maxima, then their maximum: no chain of dependent steps
            float mx[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) mx[e] = sc[e];
#pragma unroll
            for (int e = 8; e < HB; ++e) mx[e & 7] = fmaxf(mx[e & 7], sc[e]);
            const float m_half = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                                       fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]))) *
                                 P.scale_log2;    // the scale is positive
            // both halves' maxima: the row's maximum over the tile (slots alternate
            // with the tile, so one meeting a tile is enough)
            row_max[sb][half][row_in] = m_half;
            pair_sync();
            const float m_tile = fmaxf(row_max[sb][0][row_in], row_max[sb][1][row_in]);
            const bool grow = m_tile > m_used + RESCALE_STEP || (m_used == -INFINITY && m_tile > m_used);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? m_tile : m_used;
                const float cf = (grow && m_used != -INFINITY) ? fast_exp2(m_used - m_new) : 1.0f;
                if (j > 0) {
                    // O must be at rest: the product of the tile before has to be done
                    if (!mbar_wait(bar(B_P_EMPTY + (j - 1) % P_BUFS), ((j - 1) / P_BUFS) & 1)) {
                        timed_out = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t o_addr = tmem + lane_base + COL_O + half * HO;
#pragma unroll
                    for (int c0 = 0; c0 < HO; c0 += 32) {
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
                    tmem_st_wait();
                }
                l *= cf;
                m_used = m_new;
            }
            // this tile's P buffer was last read by the product of the tile two before
            const int pb = j % P_BUFS;
            if (j >= P_BUFS && !mbar_wait(bar(B_P_EMPTY + pb), ((j / P_BUFS) & 1) ^ 1)) {
                timed_out = true;
                break;
            }
            // probabilities, their sum, and P as the next product's operand
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
            float part[4] = {0.f, 0.f, 0.f, 0.f};             // four running sums
#pragma unroll
            for (int ch = 0; ch < HB / 8; ++ch) {
                uint32_t pk[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float p0 = fast_exp2(fmaf(sc[ch * 8 + 2 * u], P.scale_log2, neg_m));
                    const float p1 = fast_exp2(fmaf(sc[ch * 8 + 2 * u + 1], P.scale_log2, neg_m));
                    part[u] += p0 + p1;
                    __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    pk[u] = *reinterpret_cast<uint32_t*>(&h);
                }
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n"
                             ::"r"(swz(p_smem + pb * P_BYTES, row_in, half * (HB / 8) + ch)),
                               "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
            }
            l += (part[0] + part[1]) + (part[2] + part[3]);
            tc_fence_before();                 // a rescaled O is in place before the product adds to it
            fence_proxy_async();
            mbar_arrive(bar(B_P_FULL + pb));
        }
        // the row's sum is the two halves' sums (first half first); they meet in the
        // slots the last tile did not use
        float (*row_sum)[128] = row_max[n_tiles & 1];
        row_sum[half][row_in] = l;
        pair_sync();
        const float l_row = row_sum[0][row_in] + row_sum[1][row_in];
        const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
        // the last P V (the products end in the order they were issued), then the row's output
        if (!timed_out && n_tiles > 0 &&
            !mbar_wait(bar(B_P_EMPTY + (n_tiles - 1) % P_BUFS), ((n_tiles - 1) / P_BUFS) & 1))
            timed_out = true;
        tc_fence_after();
        __nv_bfloat16* dst = P.out + (size_t)(tok0 + ti) * P.n_heads * HD +
                             (size_t)(kvh * P.group + g) * HD + half * HO;
        uint32_t ov[HO / 16][16];                  // all loads under way, one wait
#pragma unroll
        for (int c0 = 0; c0 < HO; c0 += 16)
            tmem_ld16(tmem + lane_base + COL_O + half * HO + c0, ov[c0 / 16]);
        tmem_ld_wait();
        if (live) {
#pragma unroll
            for (int c0 = 0; c0 < HO; c0 += 16) {
                uint32_t w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    __nv_bfloat162 h =
                        __floats2bfloat162_rn(__uint_as_float(ov[c0 / 16][2 * e]) * inv,
                                              __uint_as_float(ov[c0 / 16][2 * e + 1]) * inv);
                    w[e] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(dst + c0) = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(dst + c0 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
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
}  // namespace
#endif

// Rows of one tile of mls_attention_tc (0: this head size has no such kernel).
MLS_API int mls_attention_tc_rows() {
#if MLS_HEAD_DIM == 64 || MLS_HEAD_DIM == 128
    return ROWS;
#else
    return 0;
#endif
}

// Prompts and portions of a step: n_tiles = number of tiles of mls_attention_tc_rows() rows (requests that
// the split kernel takes are left out when skip_small is set).  Returns
// MLS_ERR_UNSUPPORTED (and launches nothing) for head or page sizes it does not take.
MLS_API int mls_attention_tc(const void* qkv, void* out, const void* k_pool, const void* v_pool,
                             const int* block_table, int max_blocks, const int* cu_q,
                             const int* ctx_len, int n_req, int n_heads, int n_kv, int block_size,
                             float scale, int window, int n_tiles, int skip_small,
                             long long pool_pages, int* status, cudaStream_t stream) {
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
    P.scale_log2 = scale * LOG2E;
    P.status = status;
    P.n_pages = pool_pages;
    MLS_LAUNCH((attention_tc_kernel), dim3(n_kv, n_tiles), dim3(THREADS), SMEM_BYTES, stream, P,
               kmap, vmap, kmap_wide, vmap_wide);
    return launch_status();
#else
    return MLS_ERR_UNSUPPORTED;
#endif
}
