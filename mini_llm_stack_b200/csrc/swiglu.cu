// SwiGLU activation: out[t, i] = silu(gate[t, i]) * up[t, i] with
// silu(z) = z * sigmoid(z) (reference: train/model.py:135), computed in float32.
// gu: [T, 2*I], a row holds [gate | up].
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter,
                              size_t total) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / inter;
        const int i = (int)(e - t * inter);
        const T* row = gu + t * 2 * (size_t)inter;
        const float g = Elem<T>::load(row + i), u = Elem<T>::load(row + inter + i);
        const float s = g / (1.0f + expf(-g));
        Elem<T>::store(out + e, s * u);
    }
}

MLS_API int mls_swiglu(const void* gu, void* out, int dtype, int n_tokens, int inter,
                       cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * inter;
    if (total == 0) return 0;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == MLS_BF16)
        swiglu_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
            (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total);
    else
        swiglu_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gu, (float*)out,
                                                                 inter, total);
    return launch_status();
}
