// Shared helpers for the sm_100a kernels: element types, conversions, reductions.
//
// Every launcher is `extern "C"`, takes raw device pointers, sizes and a stream,
// and returns the cudaError_t of its launch as an int (0 = ok).  Element types
// are passed as codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#define MLS_F32 0
#define MLS_BF16 1

#define MLS_API extern "C" __attribute__((visibility("default")))

// Error codes a launcher may return besides a cudaError_t.
#define MLS_ERR_UNSUPPORTED 100001   // a size this kernel refuses

// Bits of the device status word (set by kernels, read by the host).
#define MLS_STATUS_BAD_TOKEN 1       // token id outside the vocabulary
#define MLS_STATUS_BAD_POSITION 2    // position outside the rotary table
#define MLS_STATUS_BAD_SLOT 4        // a slot or page index outside the pool

template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) {
        return __bfloat162float(*p);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) {
        *p = __float2bfloat16_rn(v);
    }
};

static __device__ __forceinline__ float load_as_float(const void* base, size_t i, int dtype) {
    return dtype == MLS_BF16 ? __bfloat162float(((const __nv_bfloat16*)base)[i])
                             : ((const float*)base)[i];
}
static __device__ __forceinline__ void store_from_float(void* base, size_t i, int dtype, float v) {
    if (dtype == MLS_BF16) ((__nv_bfloat16*)base)[i] = __float2bfloat16_rn(v);
    else ((float*)base)[i] = v;
}

static __device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
static __device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of the additions depends only on blockDim, never on the data or on what
// else runs, so a row's result does not depend on the batch it is in.
static __device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Four consecutive float32 values at `at`, summed over the n_parts slices of a
// matrix product that was cut along K (slices `stride` elements apart), in the
// order of the slices.  The loads of up to AT_ONCE slices are under way together.
template <int AT_ONCE = 8>
static __device__ __forceinline__ float4 sum_parts4(const float* __restrict__ base, size_t at,
                                                    int n_parts, size_t stride) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < n_parts; k0 += AT_ONCE) {
        float4 b[AT_ONCE];
#pragma unroll
        for (int j = 0; j < AT_ONCE; ++j)
            if (k0 + j < n_parts)
                b[j] = *reinterpret_cast<const float4*>(base + at + (size_t)(k0 + j) * stride);
#pragma unroll
        for (int j = 0; j < AT_ONCE; ++j)
            if (k0 + j < n_parts) {
                s.x += b[j].x;
                s.y += b[j].y;
                s.z += b[j].z;
                s.w += b[j].w;
            }
    }
    return s;
}

// The same at M places at once: all their loads are under way together.
template <int M, int AT_ONCE>
static __device__ __forceinline__ void sum_parts4_of(const float* __restrict__ base,
                                                     const size_t (&at)[M], int n_parts,
                                                     size_t stride, float4 (&out)[M]) {
#pragma unroll
    for (int m = 0; m < M; ++m) out[m] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < n_parts; k0 += AT_ONCE) {
        float4 b[M][AT_ONCE];
#pragma unroll
        for (int j = 0; j < AT_ONCE; ++j)
            if (k0 + j < n_parts) {
#pragma unroll
                for (int m = 0; m < M; ++m)
                    b[m][j] = *reinterpret_cast<const float4*>(base + at[m] +
                                                               (size_t)(k0 + j) * stride);
            }
#pragma unroll
        for (int j = 0; j < AT_ONCE; ++j)
            if (k0 + j < n_parts) {
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    out[m].x += b[m][j].x;
                    out[m].y += b[m][j].y;
                    out[m].z += b[m][j].z;
                    out[m].w += b[m][j].w;
                }
            }
    }
}

// Four values rounded to bfloat16, as floats again / as the eight bytes to store.
static __device__ __forceinline__ float4 round_bf16(float4 v) {
    return make_float4(__bfloat162float(__float2bfloat16_rn(v.x)),
                       __bfloat162float(__float2bfloat16_rn(v.y)),
                       __bfloat162float(__float2bfloat16_rn(v.z)),
                       __bfloat162float(__float2bfloat16_rn(v.w)));
}
static __device__ __forceinline__ uint2 pack_bf16x4(float4 v) {
    uint2 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
    h[0] = __floats2bfloat162_rn(v.x, v.y);
    h[1] = __floats2bfloat162_rn(v.z, v.w);
    return raw;
}
// Rotate-half of four pairs (x1 from the first half of a head, x2 from the second), as the
// reference's expression: o1 = x1*c - x2*s, o2 = x2*c + x1*s, products and sums separate
// float32 operations (train/model.py:47-52).
static __device__ __forceinline__ void rotate_half4(float4 x1, float4 x2, float4 cs, float4 sn,
                                                    float4& o1, float4& o2) {
    o1.x = __fsub_rn(__fmul_rn(x1.x, cs.x), __fmul_rn(x2.x, sn.x));
    o1.y = __fsub_rn(__fmul_rn(x1.y, cs.y), __fmul_rn(x2.y, sn.y));
    o1.z = __fsub_rn(__fmul_rn(x1.z, cs.z), __fmul_rn(x2.z, sn.z));
    o1.w = __fsub_rn(__fmul_rn(x1.w, cs.w), __fmul_rn(x2.w, sn.w));
    o2.x = __fadd_rn(__fmul_rn(x2.x, cs.x), __fmul_rn(x1.x, sn.x));
    o2.y = __fadd_rn(__fmul_rn(x2.y, cs.y), __fmul_rn(x1.y, sn.y));
    o2.z = __fadd_rn(__fmul_rn(x2.z, cs.z), __fmul_rn(x1.z, sn.z));
    o2.w = __fadd_rn(__fmul_rn(x2.w, cs.w), __fmul_rn(x1.w, sn.w));
}

// Streaming multiprocessors of the current device (148 on a B200), asked once.
static inline int sm_count() {
    static const int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
            v = 148;
        return v;
    }();
    return n;
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch.  A kernel started with `launch_chained` may
// begin while the kernel before it on the stream still runs, as soon as every
// block of that kernel has called `chain_release` (or has ended).  What it reads
// of that kernel's results, and everything it writes, comes after `chain_wait`,
// which returns once all earlier kernels have finished and their writes are
// visible.  Between the two a kernel may only touch memory that no kernel writes
// (weights).  Both are no-ops in a kernel that was launched the plain way.
static __device__ __forceinline__ void chain_release() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
static __device__ __forceinline__ void chain_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Whether launches are chained: off for good with MLS_B200_CHAINED=0 in the
// environment, else as the host last said through mls_set_chained (one switch per
// shared library).  A chained kernel that waits keeps its warps resident beside the
// kernel before it; under long kernels (a prompt's matrix products) that costs more
// than the early start gains, so the host chains the steps of few tokens only.
inline int g_chained = 1;
static inline bool chained_launches() {
    static const bool allowed = [] {
        const char* v = getenv("MLS_B200_CHAINED");
        return !(v && v[0] == '0');
    }();
    return allowed && g_chained != 0;
}
extern "C" __attribute__((visibility("default"), used)) inline void mls_set_chained(int on) {
    g_chained = on;
}

template <typename... Params, typename... Args>
static inline int launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = chained_launches() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// The same for a kernel whose CTAs form clusters of (cx, cy, cz) (the grid must be a multiple
// of the cluster in every dimension).
template <typename... Params, typename... Args>
static inline int launch_chained_cluster(void (*kernel)(Params...), dim3 grid, dim3 block,
                                         size_t smem, cudaStream_t stream, dim3 cluster,
                                         Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = chained_launches() ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// Launch inside a launcher that returns an int: leaves with the error if there is one.
#define MLS_LAUNCH(kernel, grid, block, smem, stream, ...)                              \
    do {                                                                                \
        const int rc_ = launch_chained(kernel, grid, block, smem, stream, __VA_ARGS__); \
        if (rc_) return rc_;                                                            \
    } while (0)
