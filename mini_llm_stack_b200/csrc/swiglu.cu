// SwiGLU activation: out[t, i] = silu(gate[t, i]) * up[t, i] with
// silu(z) = z * sigmoid(z) (reference: train/model.py:135), computed in float32.
// gu: [T, 2*I], a row holds [gate | up].
#include "common.cuh"

namespace {
__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

// 16 bytes per thread and operand: I must be a multiple of 8 (bfloat16) or 4 (float32).
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu,
                                     __nv_bfloat16* __restrict__ out, int inter) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;       // chunk of 8
    if (c * 8 >= inter) return;
    const __nv_bfloat16* row = gu + t * 2 * (size_t)inter;
    const uint4 g4 = *reinterpret_cast<const uint4*>(row + c * 8);
    const uint4 u4 = *reinterpret_cast<const uint4*>(row + inter + c * 8);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
        o2[e] = __floats2bfloat162_rn(silu_mul(g.x, u.x), silu_mul(g.y, u.y));
    }
    *reinterpret_cast<uint4*>(out + t * (size_t)inter + c * 8) = o4;
}

__global__ void swiglu_f32x4_kernel(const float* __restrict__ gu, float* __restrict__ out,
                                    int inter) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;       // chunk of 4
    if (c * 4 >= inter) return;
    const float* row = gu + t * 2 * (size_t)inter;
    const float4 g = *reinterpret_cast<const float4*>(row + c * 4);
    const float4 u = *reinterpret_cast<const float4*>(row + inter + c * 4);
    float4 o;
    o.x = silu_mul(g.x, u.x);
    o.y = silu_mul(g.y, u.y);
    o.z = silu_mul(g.z, u.z);
    o.w = silu_mul(g.w, u.w);
    *reinterpret_cast<float4*>(out + t * (size_t)inter + c * 4) = o;
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const T* row = gu + t * 2 * (size_t)inter;
    Elem<T>::store(out + t * (size_t)inter + i,
                   silu_mul(Elem<T>::load(row + i), Elem<T>::load(row + inter + i)));
}
}  // namespace

MLS_API int mls_swiglu(const void* gu, void* out, int dtype, int n_tokens, int inter,
                       cudaStream_t stream) {
    if (n_tokens <= 0 || inter <= 0) return 0;
    const int threads = 256;
    if (dtype == MLS_BF16 && inter % 8 == 0) {
        dim3 grid((inter / 8 + threads - 1) / threads, n_tokens);
        MLS_LAUNCH((swiglu_bf16x8_kernel), dim3(grid), dim3(threads), 0, stream,
                   (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter);
    } else if (dtype == MLS_F32 && inter % 4 == 0) {
        dim3 grid((inter / 4 + threads - 1) / threads, n_tokens);
        MLS_LAUNCH((swiglu_f32x4_kernel), dim3(grid), dim3(threads), 0, stream, (const float*)gu,
                   (float*)out, inter);
    } else {
        dim3 grid((inter + threads - 1) / threads, n_tokens);
        if (dtype == MLS_BF16)
            MLS_LAUNCH((swiglu_kernel<__nv_bfloat16>), dim3(grid), dim3(threads), 0, stream,
                       (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter);
        else
            MLS_LAUNCH((swiglu_kernel<float>), dim3(grid), dim3(threads), 0, stream,
                       (const float*)gu, (float*)out, inter);
    }
    return launch_status();
}
