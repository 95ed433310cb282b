// True 32-bit matrix product for the float32 path: out[M, N] = A[M, K] * W[N, K]^T.
//
// Plain FFMA on CUDA cores: no tensor cores, no TF32, no reduced-precision mode.
// Each output element is accumulated over k = 0 .. K-1 in that order, whatever M
// and N are, so a token's result does not depend on the batch it is computed in.
// Both operands are K-contiguous (the reference's nn.Linear layout [out, in],
// train/model.py:79-82,130-132).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ out,
                int M, int N, int K, int ldo) {
    chain_release();
    chain_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of each tile: row = tid / 4 (0..63), k = (tid % 4) * 4 ..
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + e][lrow] = (am < M && k < K) ? A[(size_t)am * K + k] : 0.f;
            Ws[lk + e][lrow] = (wn < N && k < K) ? W[(size_t)wn * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) out[(size_t)m * ldo + n] = acc[i][j];
        }
    }
}
}  // namespace

MLS_API int mls_gemm_f32(const float* A, const float* W, float* out, int M, int N, int K,
                         cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    MLS_LAUNCH((gemm_f32_kernel), dim3(grid), dim3(256), 0, stream, A, W, out, M, N, K, N);
    return launch_status();
}
