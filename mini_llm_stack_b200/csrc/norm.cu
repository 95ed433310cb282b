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
#include "common.cuh"

__global__ void add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ delta,
                                   int delta_dtype, const void* __restrict__ w, int w_dtype,
                                   float eps, void* __restrict__ h, int h_dtype, int d,
                                   const int* __restrict__ rows) {
    __shared__ float scratch[33];
    const int out_row = blockIdx.x;
    const int src_row = rows ? rows[out_row] : out_row;
    float* xr = x + (size_t)src_row * d;
    const size_t doff = (size_t)src_row * d;
    const bool in_place = rows == nullptr;

    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (delta) v += load_as_float(delta, doff + i, delta_dtype);
        if (in_place && delta) xr[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(total / (float)d + eps);
    const size_t hoff = (size_t)out_row * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (!in_place && delta) v += load_as_float(delta, doff + i, delta_dtype);
        float y = (v * r) * load_as_float(w, i, w_dtype);
        store_from_float(h, hoff + i, h_dtype, y);
    }
}

MLS_API int mls_add_rmsnorm(float* x, const void* delta, int delta_dtype, const void* w,
                            int w_dtype, float eps, void* h, int h_dtype, int n_rows, int d,
                            const int* rows, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    int threads = 32;
    while (threads < 1024 && threads * 4 < d) threads <<= 1;
    add_rmsnorm_kernel<<<n_rows, threads, 0, stream>>>(x, delta, delta_dtype, w, w_dtype, eps,
                                                       h, h_dtype, d, rows);
    return launch_status();
}
