// bfloat16 matrix product on the 5th-generation tensor cores:
//
//     D[MM, NN] = A[MM, K] * B[NN, K]^T        (both operands K-contiguous)
//
// A tile of 128 rows of A and BN rows of B is accumulated in tensor memory (TMEM)
// by tcgen05.mma instructions that one thread issues; the operands reach shared
// memory by TMA (64 K-elements = 128 bytes wide boxes, 128-byte swizzle) through a
// ring of stages guarded by mbarriers; four warps read the accumulator back with
// tcgen05.ld and store it.  The reference multiplies with nn.Linear
// (train/model.py:79-82,130-132,227); float32 accumulation as there.
//
// Two uses, same kernel:
//   prompts:  A = activations [tokens, K], B = weights [out, K]; D stored as is.
//   decoding: A = weights [out, K] (they fill the 128-row side of the instruction),
//             B = activations [tokens <= 64, K]; D is stored transposed, and K may be
//             cut over gridDim.z CTAs whose partial sums go to float32 scratch.
//
// Warp roles: 0 = TMA producer, 1 = TMEM allocation and MMA issue, 2..5 = epilogue.
// Every wait is bounded; a wait that runs out sets MLS_STATUS_TIMEOUT and the
// kernel still frees its tensor memory and returns.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"
#include <map>
#include <mutex>
#include <tuple>

namespace {
using namespace mls_tma;
using namespace mls_tc;

constexpr int BM = mls_tc::UMMA_M;       // rows of A per tile
constexpr int BK = 64;                   // K elements per stage = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;

struct GemmParams {
    void* out;                           // bf16 or f32, [MM, NN] or transposed [NN, MM]
    float* partial;                      // [splits, ...] float32 when splits > 1
    int mm, nn, k;                       // problem size
    int ld_out;                          // leading dimension of out (elements)
    int out_f32;                         // 1: out is float32
    int transposed;                      // 1: store D^T (out[n][m])
    int splits;                          // parts along K
    int epilogue;                        // 0: store D; 1: SwiGLU over interleaved gate / up blocks of 16
    int* status;
    // pairs of CTAs only: the tiles from tail_full on are cut along K into tail_parts parts of
    // tail_per k-blocks, whose raw sums go to `partial` (tail_parts <= 1: no tile is cut)
    int tail_full = 0, tail_parts = 0, tail_per = 0;
};

// The tiles of a product on pairs of CTAs are dealt out in rounds of one tile a pair.  The
// tiles that would make a last, incomplete round (those from tail_full on) are cut along K so
// that every pair gets a piece, and the pieces come first: their sums are stored while the
// first whole tiles are multiplied.  Unit u < cut is part u % tail_parts of tile
// tail_full + u / tail_parts; the later units are the whole tiles 0 .. tail_full - 1.
struct PairUnit {
    int tile, kb0, kb1, part;            // part < 0: a whole tile
};
__device__ __forceinline__ PairUnit pair_unit(const GemmParams& p, int u, int cut, int kblocks) {
    if (u >= cut) return {u - cut, 0, kblocks, -1};
    const int t = u / p.tail_parts, part = u - t * p.tail_parts;
    const int kb0 = part * p.tail_per;
    return {p.tail_full + t, kb0, min(kblocks, kb0 + p.tail_per), part};
}

template <int BN, int STAGES>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;              // 16 KB
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
    static constexpr int BARS = STAGES * STAGE;              // full[S], empty[S], acc_full[2], acc_empty[2]
    static constexpr int TMEM_SLOT = BARS + 8 * (2 * STAGES + 4);
    static constexpr int TOTAL = TMEM_SLOT + 16 + 1024;      // + alignment slack
};

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

// Store 16 consecutive columns (col0 ..) of D's row `row`.  With the SwiGLU
// epilogue `v` holds 16 gate columns and `u` the 16 matching up columns.
__device__ __forceinline__ void store_normal(const GemmParams& p, int row, int col0,
                                             const float (&v)[16], const float (&u)[16]) {
    if (row >= p.mm) return;
    float r[16];
    int col = col0, width = p.nn;
    if (p.epilogue == 1) {
#pragma unroll
        for (int e = 0; e < 16; ++e) r[e] = silu_mul(v[e], u[e]);
        col = col0 >> 1;
        width = p.nn >> 1;
    } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) r[e] = v[e];
    }
    const size_t at = (size_t)row * p.ld_out + col;
    const bool whole = col + 16 <= width && (p.ld_out % 8) == 0;
    if (p.out_f32) {
        float* dst = (float*)p.out + at;
        if (whole) {
#pragma unroll
            for (int e = 0; e < 16; e += 4)
                *reinterpret_cast<float4*>(dst + e) = make_float4(r[e], r[e + 1], r[e + 2], r[e + 3]);
        } else {
            _Pragma("unroll") for (int e = 0; e < 16; ++e) if (col + e < width) dst[e] = r[e];
        }
    } else {
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + at;
        if (whole) {
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * e], r[2 * e + 1]);
                w[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
            _Pragma("unroll") for (int e = 0; e < 16; ++e) if (col + e < width) dst[e] = __float2bfloat16_rn(r[e]);
        }
    }
}

// The same for the weight-major orientation: D's rows are output features, its
// columns tokens; out[token][feature].  With the SwiGLU epilogue lanes 0..15 of a
// warp hold gate features and lanes 16..31 the matching up features.
__device__ __forceinline__ void store_transposed(const GemmParams& p, int row, int col0,
                                                 const float (&v)[16], int lane) {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int col = col0 + e;                     // token
        float val = v[e];
        int feature = row, width = p.mm;
        bool mine = true;
        if (p.epilogue == 1) {
            const float other = __shfl_xor_sync(0xffffffffu, val, 16);
            val = silu_mul(val, other);               // meaningful in lanes 0..15
            feature = ((row - lane) >> 1) + lane;
            width = p.mm >> 1;
            mine = lane < 16;
        }
        if (col < p.nn && mine && feature < width && row < p.mm) {
            const size_t at = (size_t)col * p.ld_out + feature;
            if (p.out_f32) ((float*)p.out)[at] = val;
            else ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(val);
        }
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const GemmParams p, const __grid_constant__ CUtensorMap amap,
                    const __grid_constant__ CUtensorMap bmap) {
    using L = Smem<BN, STAGES>;
    constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;     // two accumulators
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && BN % 16 == 0 && TMEM_COLS <= 512,
                  "tile width");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - raw);
    auto full = [&](int s) { return base + L::BARS + 8u * s; };
    auto empty = [&](int s) { return base + L::BARS + 8u * (STAGES + s); };
    auto acc_full = [&](int a) { return base + L::BARS + 8u * (2 * STAGES + a); };
    auto acc_empty = [&](int a) { return base + L::BARS + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + L::TMEM_SLOT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (p.mm + BM - 1) / BM, n_tiles = (p.nn + BN - 1) / BN;
    const int tile_count = m_tiles * n_tiles * p.splits;
    const int kblocks = (p.k + BK - 1) / BK;
    const int per = (kblocks + p.splits - 1) / p.splits;

    chain_release();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full(a), 1);
            mbar_init(acc_empty(a), 4);
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool timed_out = false;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            // The weights are nobody's output: the first ring of them is asked for
            // while the kernel before this one may still run.  The activations, and
            // all that follows from them, come after chain_wait.
            const bool w_is_a = p.transposed != 0;
            int ahead = 0;
            if ((int)blockIdx.x < tile_count) {
                const int tile = blockIdx.x;
                const int mi = tile % m_tiles, rest = tile / m_tiles;
                const int ni = rest % n_tiles, z = rest / n_tiles;
                const int kb0 = z * per, n_kb = max(0, min(kblocks, kb0 + per) - kb0);
                ahead = min(n_kb, STAGES);
                for (int i = 0; i < ahead; ++i) {
                    const uint32_t a_dst = base + i * L::STAGE, b_dst = a_dst + L::A_BYTES;
                    mbar_arrive_expect_tx(full(i), L::A_BYTES + L::B_BYTES);
                    if (w_is_a) tma_load_2d(a_dst, &amap, (kb0 + i) * BK, mi * BM, full(i));
                    else tma_load_2d(b_dst, &bmap, (kb0 + i) * BK, ni * BN, full(i));
                }
            }
            chain_wait();
            int g = 0;                                       // k-blocks issued so far
            for (int tile = blockIdx.x; tile < tile_count && !timed_out; tile += gridDim.x) {
                const int mi = tile % m_tiles, rest = tile / m_tiles;
                const int ni = rest % n_tiles, z = rest / n_tiles;
                const int kb0 = z * per, n_kb = max(0, min(kblocks, kb0 + per) - kb0);
                for (int i = 0; i < n_kb; ++i, ++g) {
                    const int slot = g % STAGES;
                    const uint32_t a_dst = base + slot * L::STAGE, b_dst = a_dst + L::A_BYTES;
                    const bool begun = g < ahead;            // its weights are on their way
                    if (!begun) {
                        if (!mbar_wait(empty(slot), ((g / STAGES) & 1) ^ 1)) {
                            timed_out = true;
                            break;
                        }
                        mbar_arrive_expect_tx(full(slot), L::A_BYTES + L::B_BYTES);
                    }
                    if (!begun || !w_is_a)
                        tma_load_2d(a_dst, &amap, (kb0 + i) * BK, mi * BM, full(slot));
                    if (!begun || w_is_a)
                        tma_load_2d(b_dst, &bmap, (kb0 + i) * BK, ni * BN, full(slot));
                }
            }
        }
        chain_wait();
    } else if (warp == 1) {
        chain_wait();
        // --------------------------------------------------------------- MMA issue
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BN);
            int g = 0, it = 0;
            for (int tile = blockIdx.x; tile < tile_count && !timed_out; tile += gridDim.x, ++it) {
                const int z = tile / (m_tiles * n_tiles);
                const int kb0 = z * per, n_kb = max(0, min(kblocks, kb0 + per) - kb0);
                const int acc = it & 1;
                if (!mbar_wait(acc_empty(acc), ((it >> 1) & 1) ^ 1)) {
                    timed_out = true;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int i = 0; i < n_kb; ++i, ++g) {
                    const int slot = g % STAGES;
                    if (!mbar_wait(full(slot), (g / STAGES) & 1)) {
                        timed_out = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_src = base + slot * L::STAGE, b_src = a_src + L::A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk)
                        umma(tmem_d, umma_desc(a_src + kk * UMMA_K * 2),
                             umma_desc(b_src + kk * UMMA_K * 2), idesc, (i | kk) ? 1u : 0u);
                    umma_commit(empty(slot));       // the stage is free when these are done
                }
                umma_commit(acc_full(acc));         // the accumulator is complete
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        chain_wait();
        const int q = warp & 3;                     // this warp's quarter of the 128 lanes
        int it = 0;
        for (int tile = blockIdx.x; tile < tile_count; tile += gridDim.x, ++it) {
            const int mi = tile % m_tiles, rest = tile / m_tiles;
            const int ni = rest % n_tiles, z = rest / n_tiles;
            const int acc = it & 1;
            const int row = mi * BM + q * 32 + lane;
            if (!mbar_wait(acc_full(acc), (it >> 1) & 1)) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
            const bool to_partial = p.splits > 1;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t ra[16], rb[16];
                tmem_ld16(tmem_d + c0, ra);
                if (BN > 16) tmem_ld16(tmem_d + c0 + 16, rb);
                tmem_ld_wait();
                float va[16], vb[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    va[e] = __uint_as_float(ra[e]);
                    vb[e] = BN > 16 ? __uint_as_float(rb[e]) : 0.f;
                }
                const int col = ni * BN + c0;
                if (to_partial) {
                    if (row < p.mm) {
                        if (p.transposed) {
                            // [part][token][feature]: a warp writes 32 consecutive features
                            float* dst = p.partial + ((size_t)z * p.nn + col) * p.mm + row;
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                if (col + e < p.nn) dst[(size_t)e * p.mm] = va[e];
                                if (BN > 16 && col + 16 + e < p.nn) dst[(size_t)(16 + e) * p.mm] = vb[e];
                            }
                        } else {
                            float* dst = p.partial + ((size_t)z * p.mm + row) * p.nn + col;
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                if (col + e < p.nn) dst[e] = va[e];
                                if (BN > 16 && col + 16 + e < p.nn) dst[16 + e] = vb[e];
                            }
                        }
                    }
                } else if (p.transposed) {
                    store_transposed(p, row, col, va, lane);
                    if (BN > 16) store_transposed(p, row, col + 16, vb, lane);
                } else if (p.epilogue == 1) {
                    store_normal(p, row, col, va, vb);
                } else {
                    store_normal(p, row, col, va, va);
                    if (BN > 16) store_normal(p, row, col + 16, vb, vb);
                }
            }
            // the accumulator has been read: the MMA warp may fill it again
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(acc));

        }
    }
    if (timed_out && p.status) atomicOr(p.status, MLS_STATUS_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------
// The same product with pairs of CTAs (tcgen05 cta_group::2) for prompts: a cluster of two
// CTAs on neighbouring SMs owns a tile of 256 rows of A by 256 rows of B.  Each CTA brings
// in its 128 rows of A and its half (128 rows) of the B tile, so an SM reads 32 KB of
// shared memory a k-block where a lone CTA with the same 128 x 256 share of the output
// reads 48 KB; the instruction, issued by one thread of the pair's first CTA, multiplies
// both CTAs' A rows with both halves of B and leaves each CTA its 128 rows of the result
// in its own tensor memory.
//
// Hand-overs inside the pair:
//   full[s]       (first CTA) both CTAs' TMA copies of stage s have landed: the second CTA's
//                 copies complete on the first CTA's barrier (the cta_group::2 form of the
//                 load; forwarding the second CTA's own barrier by an arrival across the
//                 cluster cost 0.03 us a k-block, a releasing arrival 0.5 us);
//   empty[s]      the instructions reading stage s are done: tcgen05.commit arrives on
//                 both CTAs' barriers at once;
//   acc_full[a]   accumulator a is complete: commit to both CTAs;
//   acc_empty[a]  (first CTA) both CTAs' epilogue warps have read accumulator a: four local
//                 arrivals and four from the second CTA.
// Every load lands in the loading CTA's own shared memory only (no multicast).
//
// The epilogue (bfloat16 output whose rows are whole 16-byte chunks): the four epilogue
// warps round 64 output columns of their 128 rows into a swizzled staging tile in shared
// memory, and one thread hands the tile to TMA, which writes whole 128-byte row pieces and
// clips at the matrix's edge; two staging tiles alternate.  (Storing from registers, each
// thread 32 bytes of its own row, cost 7-10 % of the K = 4,096 products.)  Other outputs
// are stored from registers.
template <int STAGES>
struct PairSmem {
    static constexpr int A_BYTES = BM * BK * 2;              // this CTA's 128 rows of A
    static constexpr int B_BYTES = BM * BK * 2;              // its half of the tile's 256 rows of B
    static constexpr int STAGE = A_BYTES + B_BYTES;
    static constexpr int OUT_TILE = BM * 128;                // 128 rows of 64 bfloat16
    static constexpr int OUT = STAGES * STAGE;               // two staging tiles
    static constexpr int BARS = OUT + 2 * OUT_TILE;          // full, empty [S]; acc_full, acc_empty [2]
    static constexpr int TMEM_SLOT = BARS + 8 * (2 * STAGES + 4);
    static constexpr int TOTAL = TMEM_SLOT + 16 + 1024;
};
constexpr int PAIR_BN = 256;

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS)
gemm_tcgen05_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap amap,
                         const __grid_constant__ CUtensorMap bmap,
                         const __grid_constant__ CUtensorMap omap,
                         const __grid_constant__ CUtensorMap pmap, int staged_stores) {
    using L = PairSmem<STAGES>;
    constexpr int BN = PAIR_BN;
    constexpr int TMEM_COLS = 2 * BN;                        // two accumulators of 256 columns
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - raw);
    auto full = [&](int s) { return base + L::BARS + 8u * s; };
    auto empty = [&](int s) { return base + L::BARS + 8u * (STAGES + s); };
    auto acc_full = [&](int a) { return base + L::BARS + 8u * (2 * STAGES + a); };
    auto acc_empty = [&](int a) { return base + L::BARS + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + L::TMEM_SLOT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                    // 0: issues the instructions
    const int m_pairs = (p.mm + 2 * BM - 1) / (2 * BM), n_tiles = (p.nn + BN - 1) / BN;
    const int tile_count = m_pairs * n_tiles;
    const int kblocks = (p.k + BK - 1) / BK;
    const int cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    const int cut = p.tail_parts > 1 ? (tile_count - p.tail_full) * p.tail_parts : 0;
    const int unit_count = cut ? cut + p.tail_full : tile_count;

    chain_release();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full(a), 1);
            mbar_init(acc_empty(a), 8);
        }
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tc_fence_before();
    cluster_sync_all();                  // both CTAs' barriers and tensor memory are ready
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool timed_out = false;
    chain_wait();

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int g = 0;
            for (int unit = cluster; unit < unit_count && !timed_out; unit += clusters) {
                const PairUnit w = pair_unit(p, unit, cut, kblocks);
                const int mi = w.tile % m_pairs, ni = w.tile / m_pairs;
                const int a_row = mi * 2 * BM + (int)rank * BM, b_row = ni * BN + (int)rank * BM;
                for (int i = w.kb0; i < w.kb1; ++i, ++g) {
                    const int slot = g % STAGES;
                    if (!mbar_wait(empty(slot), ((g / STAGES) & 1) ^ 1)) {
                        timed_out = true;
                        break;
                    }
                    const uint32_t a_dst = base + slot * L::STAGE, b_dst = a_dst + L::A_BYTES;
                    if (rank == 0) {
                        // both CTAs' copies of the stage complete on this barrier
                        mbar_arrive_expect_tx(full(slot), 2 * L::STAGE);
                        tma_load_2d(a_dst, &amap, i * BK, a_row, full(slot));
                        tma_load_2d(b_dst, &bmap, i * BK, b_row, full(slot));
                    } else {
                        tma_load_2d_pair(a_dst, &amap, i * BK, a_row, full(slot));
                        tma_load_2d_pair(b_dst, &bmap, i * BK, b_row, full(slot));
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ----------------------------------------------- MMA issue for the pair
            constexpr uint32_t idesc = umma_idesc_pair(BN);
            int g = 0, it = 0;
            for (int unit = cluster; unit < unit_count && !timed_out; unit += clusters, ++it) {
                const PairUnit w = pair_unit(p, unit, cut, kblocks);
                const int acc = it & 1;
                if (!mbar_wait_cluster(acc_empty(acc), ((it >> 1) & 1) ^ 1)) {
                    timed_out = true;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int i = w.kb0; i < w.kb1; ++i, ++g) {
                    const int slot = g % STAGES;
                    if (!mbar_wait_cluster(full(slot), (g / STAGES) & 1)) {
                        timed_out = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_src = base + slot * L::STAGE, b_src = a_src + L::A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk)
                        umma_pair(tmem_d, umma_desc(a_src + kk * UMMA_K * 2),
                                  umma_desc(b_src + kk * UMMA_K * 2), idesc,
                                  (i > w.kb0 || kk) ? 1u : 0u);
                    umma_commit_pair(empty(slot), 3);        // both CTAs' stage is free
                }
                umma_commit_pair(acc_full(acc), 3);          // both CTAs' accumulator is complete
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;
        const int row_in = q * 32 + lane;
        const bool issuer = q == 0 && lane == 0;
        const int acc_cols = p.epilogue == 1 ? 128 : 64;     // accumulator columns behind 64 outputs
        int it = 0, fills = 0;
        for (int unit = cluster; unit < unit_count; unit += clusters, ++it) {
            const PairUnit w = pair_unit(p, unit, cut, kblocks);
            const int mi = w.tile % m_pairs, ni = w.tile / m_pairs;
            const int acc = it & 1;
            const int row0 = mi * 2 * BM + (int)rank * BM;
            const int row = row0 + row_in;
            if (!mbar_wait(acc_full(acc), (it >> 1) & 1)) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
            if (w.part >= 0) {
                // a part of a cut tile: the raw sums, [tile of the tail][part][256 rows][256],
                // 32 columns at a time through the staging tiles (128 bytes a row)
                const int part_row0 =
                    ((w.tile - p.tail_full) * p.tail_parts + w.part) * (2 * BM) + (int)rank * BM;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32, ++fills) {
                    const uint32_t stage = base + L::OUT + (fills & 1) * L::OUT_TILE;
                    if (issuer) tma_store_wait_read<1>();
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");
                    uint32_t ra[16], rb[16];
                    tmem_ld16(tmem_d + c0, ra);
                    tmem_ld16(tmem_d + c0 + 16, rb);
                    tmem_ld_wait();
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n"
                                     ::"r"(stage + row_in * 128 + ((ch ^ (row_in & 7)) << 4)),
                                       "r"(ra[4 * ch]), "r"(ra[4 * ch + 1]), "r"(ra[4 * ch + 2]),
                                       "r"(ra[4 * ch + 3]) : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n"
                                     ::"r"(stage + row_in * 128 + (((ch + 4) ^ (row_in & 7)) << 4)),
                                       "r"(rb[4 * ch]), "r"(rb[4 * ch + 1]), "r"(rb[4 * ch + 2]),
                                       "r"(rb[4 * ch + 3]) : "memory");
                    }
                    if (c0 + 32 >= BN) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (rank == 0) mbar_arrive(acc_empty(acc));
                            else mbar_arrive_remote(acc_empty(acc), 0);
                        }
                    }
                    fence_proxy_async();
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");
                    // the map sees the float32 scratch as rows of 512 two-byte elements
                    if (issuer) tma_store_2d(&pmap, c0 * 2, part_row0, stage);
                }
                continue;
            }
            if (staged_stores) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += acc_cols, ++fills) {
                    const uint32_t stage = base + L::OUT + (fills & 1) * L::OUT_TILE;
                    // the store that last read this staging tile has read it
                    if (issuer) tma_store_wait_read<1>();
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");
#pragma unroll
                    for (int part = 0; part < 2; ++part) {   // 32 outputs each
                        float r[32];
                        if (p.epilogue == 1) {
#pragma unroll
                            for (int b = 0; b < 2; ++b) {    // 16 gate columns, then the 16 up columns
                                uint32_t g[16], u[16];
                                tmem_ld16(tmem_d + c0 + part * 64 + b * 32, g);
                                tmem_ld16(tmem_d + c0 + part * 64 + b * 32 + 16, u);
                                tmem_ld_wait();
#pragma unroll
                                for (int e = 0; e < 16; ++e)
                                    r[b * 16 + e] = silu_mul(__uint_as_float(g[e]), __uint_as_float(u[e]));
                            }
                        } else {
                            uint32_t a[16], b[16];
                            tmem_ld16(tmem_d + c0 + part * 32, a);
                            tmem_ld16(tmem_d + c0 + part * 32 + 16, b);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                r[e] = __uint_as_float(a[e]);
                                r[16 + e] = __uint_as_float(b[e]);
                            }
                        }
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {     // 16-byte chunks of the row's 128 bytes
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(r[ch * 8 + 2 * e], r[ch * 8 + 2 * e + 1]);
                                w[e] = *reinterpret_cast<uint32_t*>(&h);
                            }
                            const int chunk = part * 4 + ch;
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n"
                                         ::"r"(stage + row_in * 128 + (((chunk ^ (row_in & 7))) << 4)),
                                           "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                        }
                    }
                    if (c0 + acc_cols >= BN) {
                        // the accumulator has been read: the MMA thread may fill it again
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (rank == 0) mbar_arrive(acc_empty(acc));
                            else mbar_arrive_remote(acc_empty(acc), 0);
                        }
                    }
                    fence_proxy_async();
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");
                    if (issuer) {
                        // a box that lies wholly outside the matrix is not handed over at all
                        const int out_col = (ni * BN + c0) / (p.epilogue == 1 ? 2 : 1);
                        const int width = p.epilogue == 1 ? p.nn / 2 : p.nn;
                        if (row0 < p.mm && out_col < width) tma_store_2d(&omap, out_col, row0, stage);
                    }
                }
                continue;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t ra[16], rb[16];
                tmem_ld16(tmem_d + c0, ra);
                tmem_ld16(tmem_d + c0 + 16, rb);
                tmem_ld_wait();
                float va[16], vb[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    va[e] = __uint_as_float(ra[e]);
                    vb[e] = __uint_as_float(rb[e]);
                }
                const int col = ni * BN + c0;
                if (p.epilogue == 1) {
                    store_normal(p, row, col, va, vb);
                } else {
                    store_normal(p, row, col, va, va);
                    store_normal(p, row, col + 16, vb, vb);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(acc_empty(acc));
                else mbar_arrive_remote(acc_empty(acc), 0);
            }
        }
        if (issuer) tma_store_wait_all();
    }
    if (timed_out && p.status) atomicOr(p.status, MLS_STATUS_TIMEOUT);
    __syncwarp();
    tc_fence_before();
    cluster_sync_all();                  // nobody of the pair touches tensor memory any more
    if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// Sum of the split-K parts, then the epilogue.  Parts are [part][row][col] in the
// order the output has ([token][feature] in both orientations).
__global__ void splitk_sum_kernel(const float* __restrict__ partial, void* __restrict__ out,
                                  int out_f32, int rows, int cols, int splits, int epilogue) {
    chain_release();
    chain_wait();
    const size_t n = (size_t)rows * cols;
    const int out_cols = epilogue == 1 ? cols / 2 : cols;
    const size_t total = (size_t)rows * out_cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        float r;
        if (epilogue == 1) {
            const size_t row = i / out_cols;
            const int f = (int)(i - row * out_cols);
            const size_t g = row * cols + (size_t)(f / 16) * 32 + (f % 16);
            float gs = 0.f, us = 0.f;
            for (int k = 0; k < splits; ++k) {
                gs += partial[(size_t)k * n + g];
                us += partial[(size_t)k * n + g + 16];
            }
            r = silu_mul(gs, us);
        } else {
            r = 0.f;
            for (int k = 0; k < splits; ++k) r += partial[(size_t)k * n + i];
        }
        if (out_f32) ((float*)out)[i] = r;
        else ((__nv_bfloat16*)out)[i] = __float2bfloat16_rn(r);
    }
}

// The cut tiles of a product on pairs of CTAs: their parts added up in the order of the
// parts, then the epilogue.  One thread an output; the loads of eight parts are under way
// at a time.
__global__ void pair_tail_sum_kernel(const GemmParams p, int m_pairs, int tail_tiles) {
    chain_release();
    chain_wait();
    constexpr int TILE = 2 * BM, BN = 256;
    const int shift = p.epilogue == 1 ? 7 : 8, outs = 1 << shift;   // outputs of a tile's row
    const int width = p.epilogue == 1 ? p.nn / 2 : p.nn;
    const unsigned total = (unsigned)tail_tiles * TILE * outs;
    const size_t part_stride = (size_t)TILE * BN;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int o = (int)(i & (outs - 1)), r = (int)((i >> shift) & (TILE - 1)),
                  t = (int)(i >> (shift + 8));
        const int tile = p.tail_full + t, mi = tile % m_pairs, ni = tile / m_pairs;
        const int row = mi * TILE + r, col = ni * outs + o;
        if (row >= p.mm || col >= width) continue;
        const float* src = p.partial + ((size_t)t * p.tail_parts * TILE + r) * BN;
        float v;
        if (p.epilogue == 1) {
            const int g = (o / 16) * 32 + (o % 16);
            float gs = 0.f, us = 0.f;
#pragma unroll 8
            for (int k = 0; k < p.tail_parts; ++k) {
                gs += src[k * part_stride + g];
                us += src[k * part_stride + g + 16];
            }
            v = silu_mul(gs, us);
        } else {
            v = 0.f;
#pragma unroll 8
            for (int k = 0; k < p.tail_parts; ++k) v += src[k * part_stride + o];
        }
        const size_t at = (size_t)row * p.ld_out + col;
        if (p.out_f32) ((float*)p.out)[at] = v;
        else ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(v);
    }
}

struct MapKey {
    const void* ptr;
    long long rows, k;
    int box_rows;
    bool operator<(const MapKey& o) const {
        return std::tie(ptr, rows, k, box_rows) < std::tie(o.ptr, o.rows, o.k, o.box_rows);
    }
};
std::map<MapKey, CUtensorMap> g_maps;
std::mutex g_lock;

bool operand_map(const void* ptr, long long rows, long long k, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> guard(g_lock);
    MapKey key{ptr, rows, k, box_rows};
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
        if (g_maps.size() > 4096) g_maps.clear();           // activations come and go
        CUtensorMap m;
        if (!make_map_bf16_2d(&m, ptr, (uint64_t)k, (uint64_t)rows, (uint64_t)k * 2, BK, box_rows))
            return false;
        it = g_maps.emplace(key, m).first;
    }
    *out = it->second;
    return true;
}

// A map for storing [rows, cols] bfloat16 (rows ld elements apart) in boxes of 128 rows x 64.
bool output_map(const void* ptr, long long rows, long long cols, long long ld, CUtensorMap* out) {
    std::lock_guard<std::mutex> guard(g_lock);
    MapKey key{ptr, rows, cols + (ld << 24), -BM};
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
        if (g_maps.size() > 4096) g_maps.clear();
        CUtensorMap m;
        if (!make_map_bf16_2d(&m, ptr, (uint64_t)cols, (uint64_t)rows, (uint64_t)ld * 2, 64, BM))
            return false;
        it = g_maps.emplace(key, m).first;
    }
    *out = it->second;
    return true;
}

template <int BN, int STAGES>
int launch(const GemmParams& p, const void* a, const void* b, int ctas_per_sm,
           cudaStream_t stream) {
    using L = Smem<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    CUtensorMap amap, bmap;
    if (!operand_map(a, p.mm, p.k, BM, &amap) || !operand_map(b, p.nn, p.k, BN, &bmap))
        return MLS_ERR_TENSOR_MAP;
    const long long tiles = (long long)((p.mm + BM - 1) / BM) * ((p.nn + BN - 1) / BN) * p.splits;
    const long long most = (long long)sm_count() * ctas_per_sm;
    const int grid = (int)(tiles < most ? tiles : most);
    MLS_LAUNCH((gemm_tcgen05_kernel<BN, STAGES>), dim3(grid), dim3(THREADS), L::TOTAL, stream, p,
               amap, bmap);
    return launch_status();
}

// How a product on pairs of CTAs cuts the tiles of its last round (see pair_unit): so many
// parts that every pair gets one, at least four k-blocks each.  parts <= 1: nothing is cut.
//
// When it pays (measured, Llama-3-8B products): at full occupancy the pairs are bound by what
// all SMs together draw from L2, not by rounds, so a last round of a few tiles runs faster
// than a whole one and cutting it only moves work; the parts cost a float32 round trip
// through L2 and a second kernel.  512 x 28,672 x 4,096 with SwiGLU (three rounds and two
// tiles): 99.5 us cut, 106.8 whole; 2,048 rows of the same (twelve rounds and eight tiles):
// 326.6 against 322.7; 512 x 4,096 x 14,336 (32 tiles in all): 59 against 81; 512 x 4,096 x
// 4,096: 30.4 against 29.1.  So: cut a last round of at most a sixteenth of the pairs, or a
// single incomplete round whose K is long (128 k-blocks or more).
// MLS_B200_GEMM_TAIL = 0 never cuts, "always" cuts whenever every piece gets four k-blocks.
int g_cut_tail = [] {
    const char* v = getenv("MLS_B200_GEMM_TAIL");
    if (v && v[0] == '0') return 0;
    return (v && v[0] == 'a') ? 2 : 1;
}();

struct TailPlan {
    int full, parts, per;
    long long floats;                    // float32 scratch for the parts
};
TailPlan tail_plan(int m, int n, int k) {
    TailPlan t{0, 0, 0, 0};
    const long long tiles = (long long)((m + 2 * BM - 1) / (2 * BM)) * ((n + PAIR_BN - 1) / PAIR_BN);
    const int most = sm_count() / 2, kblocks = (k + BK - 1) / BK;
    if (!g_cut_tail || most <= 0) return t;
    const int tail = (int)(tiles % most);
    if (tail == 0) return t;
    const bool pays = tail * 16 <= most || (tiles < most && kblocks >= 128);
    if (g_cut_tail == 1 && !pays) return t;
    int parts = most / tail;
    if (parts > kblocks / 4) parts = kblocks / 4;
    if (parts < 2) return t;
    t.per = (kblocks + parts - 1) / parts;
    t.parts = (kblocks + t.per - 1) / t.per;
    t.full = (int)(tiles - tail);
    t.floats = (long long)tail * t.parts * (2 * BM) * PAIR_BN;
    return t;
}

template <int STAGES>
int launch_pair(const GemmParams& p, const void* a, const void* b, cudaStream_t stream) {
    using L = PairSmem<STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    CUtensorMap amap, bmap, omap;
    if (!operand_map(a, p.mm, p.k, BM, &amap) || !operand_map(b, p.nn, p.k, BM, &bmap))
        return MLS_ERR_TENSOR_MAP;
    // bfloat16 output with rows of whole 16-byte chunks goes out through shared memory and TMA
    const int out_cols = p.epilogue == 1 ? p.nn / 2 : p.nn;
    const int staged = (!p.out_f32 && p.ld_out % 8 == 0 &&
                        (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) ? 1 : 0;
    if (staged) {
        if (!output_map(p.out, p.mm, out_cols, p.ld_out, &omap)) return MLS_ERR_TENSOR_MAP;
    } else {
        omap = amap;                                         // unused
    }
    GemmParams q = p;
    CUtensorMap pmap = amap;                                 // unused unless tiles are cut
    const TailPlan plan = tail_plan(p.mm, p.nn, p.k);
    const int m_pairs = (p.mm + 2 * BM - 1) / (2 * BM);
    const long long tiles = (long long)m_pairs * ((p.nn + PAIR_BN - 1) / PAIR_BN);
    long long units = tiles;
    if (plan.parts > 1 && p.partial != nullptr && (reinterpret_cast<uintptr_t>(p.partial) & 15) == 0) {
        // the scratch as [pieces x 256 rows] of 256 float32 = 512 two-byte elements, in boxes of
        // 128 rows x 128 bytes
        const long long rows = (tiles - plan.full) * plan.parts * 2 * BM;
        if (!output_map(p.partial, rows, 2 * PAIR_BN, 2 * PAIR_BN, &pmap)) return MLS_ERR_TENSOR_MAP;
        q.tail_full = plan.full;
        q.tail_parts = plan.parts;
        q.tail_per = plan.per;
        units = plan.full + (tiles - plan.full) * plan.parts;
    }
    const long long most = sm_count() / 2;                   // one pair on two SMs
    const int grid = 2 * (int)(units < most ? units : most);
    MLS_LAUNCH((gemm_tcgen05_pair_kernel<STAGES>), dim3(grid), dim3(THREADS), L::TOTAL, stream, q,
               amap, bmap, omap, pmap, staged);
    int rc = launch_status();
    if (rc || q.tail_parts <= 1) return rc;
    const int tail_tiles = (int)(tiles - plan.full);
    const long long work = (long long)tail_tiles * 2 * BM * (p.epilogue == 1 ? 128 : 256);
    long long blocks = (work + 255) / 256;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    MLS_LAUNCH((pair_tail_sum_kernel), dim3((int)blocks), dim3(256), 0, stream, q, m_pairs,
               tail_tiles);
    return launch_status();
}

// Which kernel takes prompts of more than 128 rows: MLS_B200_GEMM_KERNEL = pair (default: two
// CTAs a tile of 256 x 256) or tiles (one CTA a tile of 128 x 256).  Measured at 2,048 rows of
// the Llama-3-8B products the pairs run at 1.33-1.39 PFLOP/s against 1.26-1.30 (with the
// SwiGLU epilogue 1.45 against 1.43; at 512 rows 1.12 against 1.07).
int g_prompt_kernel = [] {
    const char* v = getenv("MLS_B200_GEMM_KERNEL");
    return (v && v[0] == 't') ? 0 : 1;
}();

}  // namespace

// 0: prompts of more than 128 rows take one CTA a tile; 1: pairs of CTAs.
MLS_API void mls_gemm_set_prompt_kernel(int which) { g_prompt_kernel = which ? 1 : 0; }

// The last round's tiles of a product on pairs: 0 = never cut, 1 = cut where it pays,
// 2 = cut whenever every piece gets four k-blocks.
MLS_API void mls_gemm_set_tail_cut(int mode) { g_cut_tail = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }

// float32 scratch (`partial`) that a prompt's product of this size wants for the tiles of its
// last round; 0: none.  Without the scratch the product runs all tiles whole.
MLS_API long long mls_gemm_prompt_scratch_floats(int m, int n, int k) {
    if (m <= BM || g_prompt_kernel != 1) return 0;
    return tail_plan(m, n, k).floats;
}

// out[M, N] = act[M, K] * w[N, K]^T, bfloat16 operands, out bfloat16 or float32.
// swap: 1 = the weights take the 128-row side (decoding, M <= 64).  splits > 1 cuts K
// (weight-major orientation only) and needs `partial`, float32 scratch of
// splits * M * N, which a second kernel adds up (with out == nullptr the parts are left
// to the caller, [part][M][N]).  With swap = 0 `partial` is optional scratch of
// mls_gemm_prompt_scratch_floats(m, n, k) floats.  epilogue 1: the weight rows alternate
// between 16 gate rows and the 16 matching up rows, and out[M, N / 2] = silu(gate) * up.
MLS_API int mls_gemm_bf16(const void* act, const void* w, void* out, int out_f32, int m, int n,
                          int k, int swap, int splits, int epilogue, float* partial, int* status,
                          cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k % 8 != 0 || k <= 0) return MLS_ERR_UNSUPPORTED;      // rows must be 16-byte multiples
    if (out == nullptr && (splits < 2 || !swap || epilogue != 0)) return MLS_ERR_UNSUPPORTED;
    if (splits < 1 || (splits > 1 && partial == nullptr))
        return MLS_ERR_UNSUPPORTED;
    if (epilogue == 1 && n % 32 != 0) return MLS_ERR_UNSUPPORTED;
    GemmParams p;
    p.out = out;
    p.partial = partial;
    p.k = k;
    p.ld_out = epilogue == 1 ? n / 2 : n;
    p.out_f32 = out_f32;
    p.splits = splits;
    p.epilogue = epilogue;
    p.status = status;
    if (swap) {
        if (m > 64) return MLS_ERR_UNSUPPORTED;
        p.mm = n;                       // rows of the weights
        p.nn = m;                       // tokens
        p.transposed = 1;
        // two CTAs fit an SM, so up to 296 tiles stream at the same time
        int rc;
        if (m <= 16) rc = launch<16, 6>(p, w, act, 2, stream);
        else if (m <= 32) rc = launch<32, 5>(p, w, act, 2, stream);
        else rc = launch<64, 4>(p, w, act, 2, stream);
        if (rc || splits == 1 || out == nullptr) return rc;
        const size_t total = (size_t)m * p.ld_out;
        int blocks = (int)((total + 255) / 256);
        if (blocks > sm_count() * 8) blocks = sm_count() * 8;
        MLS_LAUNCH((splitk_sum_kernel), dim3(blocks), dim3(256), 0, stream, partial, out, out_f32,
                   m, n, splits, epilogue);
        return launch_status();
    }
    if (splits != 1) return MLS_ERR_UNSUPPORTED;               // prompts cut K by themselves
    p.mm = m;
    p.nn = n;
    p.transposed = 0;
    if (g_prompt_kernel == 1 && m > BM) return launch_pair<6>(p, act, w, stream);
    return launch<256, 4>(p, act, w, 1, stream);
}
