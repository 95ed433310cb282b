// RMS norm fused with the pending residual addition.
//
// Reference formula (train/model.py:29-33): xf = float(x);
// y = xf * rsqrt(mean(xf^2) + eps); out = (y * float(w)) cast to the activation
// type.  eps is added to the mean inside the root; the weight multiplies after
// the normalisation.  Everything is float32 with one rounding at the store.
//
// rows == nullptr: for every row t: x[t] += delta[t] (if delta), h[t] = norm(x[t]).
// rows != nullptr: for i < n_rows: v = x[rows[i]] + delta[rows[i]], h[i] = norm(v);
//                  x is not modified.
//
// delta_parts > 1: delta is that many float32 slices, part_stride elements apart (the
// parts of a matrix product cut along K); their sum, taken in the order of the
// slices, is the delta.
//
// The sum of squares is taken in an order that depends on the row's width only,
// so a row's result does not depend on the batch it is in.
#include "common.cuh"
#include "tma.cuh"

namespace {
__device__ __forceinline__ uint32_t shared_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ float4 load4(const void* base, size_t i, int dtype) {
    if (dtype == MLS_BF16) {
        const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)base + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return *reinterpret_cast<const float4*>((const float*)base + i);
}
__device__ __forceinline__ void store4(void* base, size_t i, int dtype, float4 v) {
    if (dtype == MLS_BF16) {
        uint2 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
        h[0] = __floats2bfloat162_rn(v.x, v.y);
        h[1] = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>((__nv_bfloat16*)base + i) = raw;
    } else {
        *reinterpret_cast<float4*>((float*)base + i) = v;
    }
}

__device__ __forceinline__ float4 load_delta4(const void* delta, size_t i, int dtype, int parts,
                                              size_t stride) {
    if (parts > 1) return sum_parts4<4>((const float*)delta, i, parts, stride);
    return load4(delta, i, dtype);
}
__device__ __forceinline__ float load_delta(const void* delta, size_t i, int dtype, int parts,
                                            size_t stride) {
    float s = load_as_float(delta, i, dtype);
    for (int k = 1; k < parts; ++k) s += load_as_float(delta, i + k * stride, dtype);
    return s;
}

// 16 bytes as they come from memory: four float32, or four bfloat16 in the first half.
struct Raw16 {
    uint4 bits;
};
__device__ __forceinline__ Raw16 load_raw4(const void* base, size_t i, int dtype) {
    Raw16 r;
    if (dtype == MLS_BF16) {
        const uint2 two = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)base + i);
        r.bits = make_uint4(two.x, two.y, 0u, 0u);
    } else {
        r.bits = *reinterpret_cast<const uint4*>((const float*)base + i);
    }
    return r;
}
__device__ __forceinline__ float4 as_float4(const Raw16& r, int dtype) {
    if (dtype == MLS_BF16) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r.bits);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return make_float4(__uint_as_float(r.bits.x), __uint_as_float(r.bits.y),
                       __uint_as_float(r.bits.z), __uint_as_float(r.bits.w));
}

// d a multiple of 4 and d / 4 <= blockDim.x * VEC: a row lives in registers.  A block
// takes rows blockIdx.x, blockIdx.x + gridDim.x, ...; with VEC == 1 (rows up to 4096
// wide) the loads of its next row are under way while it reduces and stores the
// present one; wider rows have no registers to spare for that.  Which thread holds
// which values, and the order of the sum of squares, depend on d alone.
template <int VEC>
__global__ void __launch_bounds__(1024)
add_rmsnorm_vec_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype,
                       const void* __restrict__ w, int w_dtype, float eps, void* __restrict__ h,
                       int h_dtype, int n_rows, int d, const int* __restrict__ rows,
                       int delta_parts, size_t part_stride) {
    chain_release();
    __shared__ float scratch[33];
    const int n4 = d >> 2;
    constexpr bool AHEAD = VEC == 1;
    float4 ww[VEC];                       // the weight is nobody's output: read before the wait
    if constexpr (AHEAD) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < n4) ww[k] = load4(w, 4 * c, w_dtype);
        }
    }
    chain_wait();
    const bool in_place = rows == nullptr;
    const bool summed = delta != nullptr && delta_parts > 1;    // few rows: nothing to run ahead of
    Raw16 nx[VEC], nd[VEC];
    auto ask = [&](int out_row) {         // start the loads of a row
        const size_t xoff = (size_t)(rows ? rows[out_row] : out_row) * d;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < n4) {
                nx[k] = load_raw4(x, xoff + 4 * c, MLS_F32);
                if (delta && !summed) nd[k] = load_raw4(delta, xoff + 4 * c, delta_dtype);
            }
        }
    };
    int out_row = blockIdx.x;
    if (AHEAD && out_row < n_rows) ask(out_row);
    for (; out_row < n_rows; out_row += gridDim.x) {
        const size_t xoff = (size_t)(rows ? rows[out_row] : out_row) * d;
        float4 v[VEC];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < n4) {
                float4 a, b;
                if constexpr (AHEAD) {
                    a = as_float4(nx[k], MLS_F32);
                    if (delta)
                        b = summed ? sum_parts4<4>((const float*)delta, xoff + 4 * c, delta_parts,
                                                   part_stride)
                                   : as_float4(nd[k], delta_dtype);
                } else {
                    a = *reinterpret_cast<const float4*>(x + xoff + 4 * c);
                    if (delta)
                        b = load_delta4(delta, xoff + 4 * c, delta_dtype, delta_parts, part_stride);
                }
                if (delta) {
                    a.x += b.x;
                    a.y += b.y;
                    a.z += b.z;
                    a.w += b.w;
                    if (in_place) *reinterpret_cast<float4*>(x + xoff + 4 * c) = a;
                }
                v[k] = a;
                ss += a.x * a.x;
                ss += a.y * a.y;
                ss += a.z * a.z;
                ss += a.w * a.w;
            }
        }
        if (AHEAD && out_row + (int)gridDim.x < n_rows) ask(out_row + gridDim.x);
        const float total = block_sum(ss, scratch);
        const float r = 1.0f / sqrtf(total / (float)d + eps);
        const size_t hoff = (size_t)out_row * d;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < n4) {
                float4 g;
                if constexpr (AHEAD) g = ww[k];
                else g = load4(w, 4 * c, w_dtype);
                float4 y;
                y.x = (v[k].x * r) * g.x;
                y.y = (v[k].y * r) * g.y;
                y.z = (v[k].z * r) * g.z;
                y.w = (v[k].w * r) * g.w;
                store4(h, hoff + 4 * c, h_dtype, y);
            }
        }
    }
}

// block_sum for R values at once: the same additions in the same order for each.
template <int R>
__device__ __forceinline__ void block_sum_each(float (&v)[R], float (*scratch)[33]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int r = 0; r < R; ++r) v[r] = warp_sum(v[r]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) scratch[r][warp] = v[r];
    }
    __syncthreads();
    if (warp < R) {                       // warp r sums row r's per-warp values
        float t = lane < nwarps ? scratch[warp][lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[warp][32] = t;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) v[r] = scratch[r][32];
}

// Many rows (a prompt): block b of one an SM takes a run of consecutive rows, in
// groups of STREAM_ROWS; a group of x and of delta comes into one of two halves of
// shared memory by two bulk copies while the group before it is worked on, so that
// the memory system always has this SM's next rows to fetch.  Thread c holds chunk
// c of each row of the group and the sums of squares run as in
// add_rmsnorm_vec_kernel<1> with the same block size: the results are the same bits.
// In place only (rows == nullptr), one part, d a multiple of 8 and at most 4096.
constexpr int STREAM_ROWS = 4;
__global__ void __launch_bounds__(1024)
add_rmsnorm_stream_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype,
                          const void* __restrict__ w, int w_dtype, float eps,
                          void* __restrict__ h, int h_dtype, int n_rows, int d, int* status) {
    using namespace mls_tma;
    constexpr int R = STREAM_ROWS;
    chain_release();
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ float scratch[R][33];
    __shared__ int arrived;
    __shared__ __align__(8) uint64_t full_bars[2];
    const int n4 = d >> 2;
    const int c = threadIdx.x;
    const uint32_t xrow = (uint32_t)d * 4u;
    const uint32_t drow = delta ? (uint32_t)d * (delta_dtype == MLS_BF16 ? 2u : 4u) : 0u;
    const uint32_t half_bytes = (R * (xrow + drow) + 127u) & ~127u;
    const uint32_t ring0 = shared_addr(ring);
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < n4) g = load4(w, 4 * c, w_dtype);
    if (threadIdx.x == 0) {
        mbar_init(shared_addr(&full_bars[0]), 1);
        mbar_init(shared_addr(&full_bars[1]), 1);
        fence_barrier_init();
    }
    __syncthreads();
    chain_wait();
    const int per = (n_rows + (int)gridDim.x - 1) / (int)gridDim.x;
    const int row0 = (int)blockIdx.x * per, row1 = min(n_rows, row0 + per);
    const int n_groups = row1 > row0 ? (row1 - row0 + R - 1) / R : 0;
    auto ask = [&](int i) {               // one thread: start the copies of my i-th group
        const int s = i & 1;
        const size_t first = (size_t)row0 + (size_t)i * R;
        const uint32_t rows_here = (uint32_t)min(R, row1 - (int)first);
        const uint32_t bar = shared_addr(&full_bars[s]), dst = ring0 + s * half_bytes;
        mbar_arrive_expect_tx(bar, rows_here * (xrow + drow));
        bulk_load_1d(dst, x + first * d, rows_here * xrow, bar);
        if (drow)
            bulk_load_1d(dst + R * xrow, (const uint8_t*)delta + first * drow, rows_here * drow,
                         bar);
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < min(2, n_groups); ++i) ask(i);
    for (int i = 0; i < n_groups; ++i) {
        const int s = i & 1;
        if (threadIdx.x == 0) arrived = mbar_wait(shared_addr(&full_bars[s]), (i >> 1) & 1) ? 1 : 0;
        __syncthreads();
        if (!arrived) {                   // every thread leaves at the same place
            if (threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_TIMEOUT);
            return;
        }
        const size_t first = (size_t)row0 + (size_t)i * R;
        const int rows_here = min(R, row1 - (int)first);
        const uint8_t* xs = ring + (size_t)s * half_bytes;
        const uint8_t* ds = xs + (size_t)R * xrow;
        float4 a[R];
        float ss[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            a[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            ss[r] = 0.f;
            if (c < n4 && r < rows_here) {
                a[r] = *reinterpret_cast<const float4*>(xs + (size_t)r * xrow + 16 * c);
                if (drow) {
                    const float4 b = load4(ds + (size_t)r * drow, 4 * c, delta_dtype);
                    a[r].x += b.x;
                    a[r].y += b.y;
                    a[r].z += b.z;
                    a[r].w += b.w;
                    *reinterpret_cast<float4*>(x + (first + r) * d + 4 * c) = a[r];
                }
                ss[r] += a[r].x * a[r].x;
                ss[r] += a[r].y * a[r].y;
                ss[r] += a[r].z * a[r].z;
                ss[r] += a[r].w * a[r].w;
            }
        }
        // the barriers in there come after every thread has read its part of the half
        block_sum_each<R>(ss, scratch);
        if (threadIdx.x == 0 && i + 2 < n_groups) ask(i + 2);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (c < n4 && r < rows_here) {
                const float rs = 1.0f / sqrtf(ss[r] / (float)d + eps);
                float4 y;
                y.x = (a[r].x * rs) * g.x;
                y.y = (a[r].y * rs) * g.y;
                y.z = (a[r].z * rs) * g.z;
                y.w = (a[r].w * rs) * g.w;
                store4(h, (first + r) * d + 4 * c, h_dtype, y);
            }
        }
    }
}

__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ delta,
                                   int delta_dtype, const void* __restrict__ w, int w_dtype,
                                   float eps, void* __restrict__ h, int h_dtype, int d,
                                   const int* __restrict__ rows, int delta_parts,
                                   size_t part_stride) {
    chain_release();
    chain_wait();
    __shared__ float scratch[33];
    const int out_row = blockIdx.x;
    const int src_row = rows ? rows[out_row] : out_row;
    float* xr = x + (size_t)src_row * d;
    const size_t doff = (size_t)src_row * d;
    const bool in_place = rows == nullptr;

    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (delta) v += load_delta(delta, doff + i, delta_dtype, delta_parts, part_stride);
        if (in_place && delta) xr[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(total / (float)d + eps);
    const size_t hoff = (size_t)out_row * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (!in_place && delta)
            v += load_delta(delta, doff + i, delta_dtype, delta_parts, part_stride);
        float y = (v * r) * load_as_float(w, i, w_dtype);
        store_from_float(h, hoff + i, h_dtype, y);
    }
}
}  // namespace

MLS_API int mls_add_rmsnorm(float* x, const void* delta, int delta_dtype, const void* w,
                            int w_dtype, float eps, void* h, int h_dtype, int n_rows, int d,
                            const int* rows, int delta_parts, long long part_stride, int* status,
                            cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (delta_parts < 1 || (delta_parts > 1 && (delta_dtype != MLS_F32 || part_stride % 4 != 0)))
        return MLS_ERR_UNSUPPORTED;
    const size_t stride = (size_t)part_stride;
    if (d % 4 == 0 && d / 4 <= 1024 * 4) {
        const int n4 = d / 4;
        int threads = 32;
        while (threads < 1024 && threads < n4) threads <<= 1;
        const int vec = (n4 + threads - 1) / threads;      // chunks of four per thread: 1..4
        const int esize = delta ? (delta_dtype == MLS_BF16 ? 2 : 4) : 0;
        const int half_bytes = (STREAM_ROWS * d * (4 + esize) + 127) / 128 * 128;
        if (vec == 1 && threads >= 32 * STREAM_ROWS && d % 8 == 0 && rows == nullptr &&
            delta_parts == 1 && n_rows >= 2 * sm_count() && 2 * half_bytes <= 200 * 1024) {
            static bool configured = false;
            if (!configured) {
                cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_stream_kernel,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     200 * 1024);
                if (e != cudaSuccess) return (int)e;
                configured = true;
            }
            MLS_LAUNCH((add_rmsnorm_stream_kernel), dim3(sm_count()), dim3(threads),
                       (size_t)2 * half_bytes, stream, x, delta, delta_dtype, w, w_dtype, eps, h,
                       h_dtype, n_rows, d, status);
            return launch_status();
        }
        // as many blocks as run at the same time; each takes its rows in turn
        const int vv = vec <= 1 ? 1 : (vec <= 2 ? 2 : 4);
        int resident = sm_count() * (1024 / threads < 16 ? 1024 / threads : 16);
        const int blocks = n_rows < resident ? n_rows : resident;
        if (vv == 1)
            MLS_LAUNCH((add_rmsnorm_vec_kernel<1>), dim3(blocks), dim3(threads), 0, stream, x,
                       delta, delta_dtype, w, w_dtype, eps, h, h_dtype, n_rows, d, rows,
                       delta_parts, stride);
        else if (vv == 2)
            MLS_LAUNCH((add_rmsnorm_vec_kernel<2>), dim3(blocks), dim3(threads), 0, stream, x,
                       delta, delta_dtype, w, w_dtype, eps, h, h_dtype, n_rows, d, rows,
                       delta_parts, stride);
        else
            MLS_LAUNCH((add_rmsnorm_vec_kernel<4>), dim3(blocks), dim3(threads), 0, stream, x,
                       delta, delta_dtype, w, w_dtype, eps, h, h_dtype, n_rows, d, rows,
                       delta_parts, stride);
        return launch_status();
    }
    int threads = 32;
    while (threads < 1024 && threads * 4 < d) threads <<= 1;
    MLS_LAUNCH((add_rmsnorm_kernel), dim3(n_rows), dim3(threads), 0, stream, x, delta, delta_dtype,
               w, w_dtype, eps, h, h_dtype, d, rows, delta_parts, stride);
    return launch_status();
}
