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
#include <map>
#include <mutex>
#include <tuple>

namespace {
using namespace mls_tma;

constexpr int BM = 128;                  // rows of A per tile = UMMA M
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
    int splits;                          // CTAs along K
    int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// Shared-memory matrix descriptor for a K-major tile with 128-byte rows and the
// 128-byte swizzle: 8-row groups are 1024 bytes apart; version 1 (Blackwell).
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);                  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                  // leading byte offset (unused here)
    d |= (uint64_t)(1024 >> 4) << 32;                        // stride byte offset
    d |= (uint64_t)1 << 46;                                  // descriptor version
    d |= (uint64_t)2 << 61;                                  // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                     uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
          "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

template <int BN, int STAGES>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;              // 16 KB
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
    static constexpr int BARS = STAGES * STAGE;              // full[S], empty[S], tmem_full
    static constexpr int TMEM_SLOT = BARS + 8 * (2 * STAGES + 1);
    static constexpr int TOTAL = TMEM_SLOT + 16 + 1024;      // + alignment slack
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const GemmParams p, const __grid_constant__ CUtensorMap amap,
                    const __grid_constant__ CUtensorMap bmap) {
    using L = Smem<BN, STAGES>;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;             // a power of two >= 32
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && BN % 16 == 0 && BN <= 256, "tile width");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - raw);
    auto full = [&](int s) { return base + L::BARS + 8u * s; };
    auto empty = [&](int s) { return base + L::BARS + 8u * (STAGES + s); };
    const uint32_t tmem_full = base + L::BARS + 8u * (2 * STAGES);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + L::TMEM_SLOT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int kblocks = (p.k + BK - 1) / BK;
    const int per = (kblocks + p.splits - 1) / p.splits;
    const int kb0 = blockIdx.z * per, kb1 = min(kblocks, kb0 + per);
    const int n_kb = max(0, kb1 - kb0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        mbar_init(tmem_full, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(const_cast<uint32_t*>(tmem_slot))), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;
    bool timed_out = false;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            for (int i = 0; i < n_kb; ++i) {
                const int slot = i % STAGES;
                if (!mbar_wait(empty(slot), ((i / STAGES) & 1) ^ 1)) {
                    timed_out = true;
                    break;
                }
                const uint32_t a_dst = base + slot * L::STAGE, b_dst = a_dst + L::A_BYTES;
                mbar_arrive_expect_tx(full(slot), L::A_BYTES + L::B_BYTES);
                tma_load_2d(a_dst, &amap, (kb0 + i) * BK, m0, full(slot));
                tma_load_2d(b_dst, &bmap, (kb0 + i) * BK, n0, full(slot));
            }
        }
    } else if (warp == 1) {
        // --------------------------------------------------------------- MMA issue
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BN);
            for (int i = 0; i < n_kb; ++i) {
                const int slot = i % STAGES;
                if (!mbar_wait(full(slot), (i / STAGES) & 1)) {
                    timed_out = true;
                    break;
                }
                tc_fence_after();
                const uint32_t a_src = base + slot * L::STAGE, b_src = a_src + L::A_BYTES;
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk)
                    umma(tmem_d, umma_desc(a_src + kk * UMMA_K * 2),
                         umma_desc(b_src + kk * UMMA_K * 2), idesc, (i | kk) ? 1u : 0u);
                umma_commit(empty(slot));           // the stage is free when these are done
            }
            umma_commit(tmem_full);                 // the accumulator is complete
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        if (n_kb > 0 && !mbar_wait(tmem_full, 0)) timed_out = true;
        tc_fence_after();
        const int q = warp & 3;                     // this warp's quarter of the 128 lanes
        const int row = m0 + q * 32 + lane;         // row of A (and of D)
        const bool to_partial = p.splits > 1;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t v[16];
            if (n_kb > 0) {
                tmem_ld16(tmem_d + ((uint32_t)(q * 32) << 16) + c0, v);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = 0u;
            }
            if (row >= p.mm) continue;
            if (p.transposed) {
                // out[col][row]: the 32 lanes of a warp write 32 consecutive rows
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int col = n0 + c0 + e;
                    if (col >= p.nn) break;
                    const size_t at = (size_t)col * p.ld_out + row;
                    const float f = __uint_as_float(v[e]);
                    if (to_partial)
                        p.partial[(size_t)blockIdx.z * p.nn * p.ld_out + at] = f;
                    else if (p.out_f32)
                        ((float*)p.out)[at] = f;
                    else
                        ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(f);
                }
            } else {
                const int col = n0 + c0;
                const size_t at = (size_t)row * p.ld_out + col;
                const bool whole = col + 16 <= p.nn && (p.ld_out % 8) == 0;
                if (to_partial) {
                    float* dst = p.partial + (size_t)blockIdx.z * p.mm * p.ld_out + at;
                    for (int e = 0; e < 16 && col + e < p.nn; ++e) dst[e] = __uint_as_float(v[e]);
                } else if (p.out_f32) {
                    float* dst = (float*)p.out + at;
                    if (whole) {
#pragma unroll
                        for (int e = 0; e < 16; e += 4)
                            *reinterpret_cast<uint4*>(dst + e) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
                    } else {
                        for (int e = 0; e < 16 && col + e < p.nn; ++e) dst[e] = __uint_as_float(v[e]);
                    }
                } else {
                    __nv_bfloat16* dst = (__nv_bfloat16*)p.out + at;
                    if (whole) {
                        uint32_t w[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * e]),
                                                                     __uint_as_float(v[2 * e + 1]));
                            w[e] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                        *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                    } else {
                        for (int e = 0; e < 16 && col + e < p.nn; ++e)
                            dst[e] = __float2bfloat16_rn(__uint_as_float(v[e]));
                    }
                }
            }
        }
    }
    if (timed_out && p.status) atomicOr(p.status, MLS_STATUS_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n"
                     ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
    }
}

// sum of split-K partial results: out[i] = sum_s partial[s][i]
__global__ void splitk_sum_kernel(const float* __restrict__ partial, void* __restrict__ out,
                                  int out_f32, size_t n, int splits) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += partial[(size_t)k * n + i];
        if (out_f32) ((float*)out)[i] = s;
        else ((__nv_bfloat16*)out)[i] = __float2bfloat16_rn(s);
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

template <int BN, int STAGES>
int launch(const GemmParams& p, const void* a, const void* b, cudaStream_t stream) {
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
    dim3 grid((p.mm + BM - 1) / BM, (p.nn + BN - 1) / BN, p.splits);
    gemm_tcgen05_kernel<BN, STAGES><<<grid, THREADS, L::TOTAL, stream>>>(p, amap, bmap);
    return launch_status();
}
}  // namespace

// out[M, N] = act[M, K] * w[N, K]^T, bfloat16 operands, out bfloat16 or float32.
// swap: 1 = the weights take the 128-row side (decoding, M <= 64); splits > 1 cuts K
// and needs `partial`, float32 scratch of splits * M * N.
MLS_API int mls_gemm_bf16(const void* act, const void* w, void* out, int out_f32, int m, int n,
                          int k, int swap, int splits, float* partial, int* status,
                          cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k % 8 != 0 || k <= 0) return MLS_ERR_UNSUPPORTED;      // rows must be 16-byte multiples
    if (splits < 1 || (splits > 1 && partial == nullptr)) return MLS_ERR_UNSUPPORTED;
    GemmParams p;
    p.out = out;
    p.partial = partial;
    p.k = k;
    p.ld_out = n;
    p.out_f32 = out_f32;
    p.splits = splits;
    p.status = status;
    int rc;
    if (swap) {
        if (m > 64) return MLS_ERR_UNSUPPORTED;
        p.mm = n;                       // rows of the weights
        p.nn = m;                       // tokens
        p.transposed = 1;
        // two CTAs fit an SM, so up to 296 tiles stream at the same time
        if (m <= 16) rc = launch<16, 6>(p, w, act, stream);
        else if (m <= 32) rc = launch<32, 5>(p, w, act, stream);
        else rc = launch<64, 4>(p, w, act, stream);
    } else {
        p.mm = m;
        p.nn = n;
        p.transposed = 0;
        rc = launch<256, 4>(p, act, w, stream);
    }
    if (rc) return rc;
    if (splits > 1) {
        const size_t total = (size_t)m * n;
        int blocks = (int)((total + 255) / 256);
        if (blocks > 148 * 8) blocks = 148 * 8;
        splitk_sum_kernel<<<blocks, 256, 0, stream>>>(partial, out, out_f32, total, splits);
        return launch_status();
    }
    return 0;
}
