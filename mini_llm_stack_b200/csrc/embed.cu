// Token embedding: x[t, :] = E[token[t], :], widened to the float32 residual
// stream.  No scaling and no position term (reference: train/model.py:224,239).
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ x, int d, int vocab, int* status) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    bool bad = id < 0 || id >= vocab;
    if (bad) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_TOKEN);
    }
    const T* row = table + (size_t)(bad ? 0 : id) * d;
    float* out = x + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        out[i] = bad ? 0.f : Elem<T>::load(row + i);
}

MLS_API int mls_embed(const int* ids, const void* table, int table_dtype, float* x,
                      int n_tokens, int d, int vocab, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    int threads = d >= 1024 ? 256 : (d >= 256 ? 128 : 64);
    if (table_dtype == MLS_BF16)
        MLS_LAUNCH((embed_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(threads), 0, stream, ids,
                   (const __nv_bfloat16*)table, x, d, vocab, status);
    else
        MLS_LAUNCH((embed_kernel<float>), dim3(n_tokens), dim3(threads), 0, stream, ids,
                   (const float*)table, x, d, vocab, status);
    return launch_status();
}
