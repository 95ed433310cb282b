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

namespace {
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

// d a multiple of 4 and d / 4 <= blockDim.x * VEC: a row lives in registers.
template <int VEC>
__global__ void __launch_bounds__(1024) add_rmsnorm_vec_kernel(float* __restrict__ x, const void* __restrict__ delta,
                                       int delta_dtype, const void* __restrict__ w, int w_dtype,
                                       float eps, void* __restrict__ h, int h_dtype, int d,
                                       const int* __restrict__ rows, int delta_parts,
                                       size_t part_stride) {
    chain_release();
    __shared__ float scratch[33];
    const int n4 = d >> 2;
    float4 ww[VEC];                       // the weight is nobody's output: read before the wait
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < n4) ww[k] = load4(w, 4 * c, w_dtype);
    }
    chain_wait();
    const int out_row = blockIdx.x;
    const int src_row = rows ? rows[out_row] : out_row;
    const size_t xoff = (size_t)src_row * d;
    const bool in_place = rows == nullptr;
    float4 v[VEC];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < n4) {
            float4 a = *reinterpret_cast<const float4*>(x + xoff + 4 * c);
            if (delta) {
                const float4 b = load_delta4(delta, xoff + 4 * c, delta_dtype, delta_parts,
                                             part_stride);
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
    const float total = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(total / (float)d + eps);
    const size_t hoff = (size_t)out_row * d;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < n4) {
            float4 y;
            y.x = (v[k].x * r) * ww[k].x;
            y.y = (v[k].y * r) * ww[k].y;
            y.z = (v[k].z * r) * ww[k].z;
            y.w = (v[k].w * r) * ww[k].w;
            store4(h, hoff + 4 * c, h_dtype, y);
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
                            const int* rows, int delta_parts, long long part_stride,
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
        if (vec <= 1)
            MLS_LAUNCH((add_rmsnorm_vec_kernel<1>), dim3(n_rows), dim3(threads), 0, stream, x,
                       delta, delta_dtype, w, w_dtype, eps, h, h_dtype, d, rows, delta_parts,
                       stride);
        else if (vec <= 2)
            MLS_LAUNCH((add_rmsnorm_vec_kernel<2>), dim3(n_rows), dim3(threads), 0, stream, x,
                       delta, delta_dtype, w, w_dtype, eps, h, h_dtype, d, rows, delta_parts,
                       stride);
        else
            MLS_LAUNCH((add_rmsnorm_vec_kernel<4>), dim3(n_rows), dim3(threads), 0, stream, x,
                       delta, delta_dtype, w, w_dtype, eps, h, h_dtype, d, rows, delta_parts,
                       stride);
        return launch_status();
    }
    int threads = 32;
    while (threads < 1024 && threads * 4 < d) threads <<= 1;
    MLS_LAUNCH((add_rmsnorm_kernel), dim3(n_rows), dim3(threads), 0, stream, x, delta, delta_dtype,
               w, w_dtype, eps, h, h_dtype, d, rows, delta_parts, stride);
    return launch_status();
}
