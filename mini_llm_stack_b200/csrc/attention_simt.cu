// Causal grouped-query attention over the paged cache on CUDA cores, for any
// mix of prompt portions and single decoded tokens.  It serves the float32 path
// (everything in 32-bit) and checks the tensor-core kernels of the bfloat16 path.
//
// Reference math (train/model.py:55-70): S = (q . k) * scale in float32; key j is
// hidden from the query at absolute position p iff j > p (the bottom-right
// aligned causal mask with p = i + Sk - Sq); P = softmax(S); O = P . V in
// float32, rounded once.  q head h reads kv head h / G.  With a window w, keys
// j <= p - w are hidden too.  The paged walk follows the reference's decode
// kernel (kernels/paged_attention.py:34-88): page = table[r, j / block],
// offset = j % block, online softmax over chunks of keys.
//
// One warp per (token, q head).  Keys are taken 32 at a time from an absolute
// multiple of 32, so the order of every sum depends only on the token's own
// position and window: the result is bit-for-bit the same however the tokens
// were cut into steps and whatever else is in the batch.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

// q . k over one key row, accumulated in the order i = 0 .. hd-1.
__device__ __forceinline__ float dot_row(const float* q, const float* k, int hd) {
    float dot = 0.f;
    if ((hd & 3) == 0) {
        for (int i = 0; i < hd; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(k + i);
            dot = fmaf(q[i], v.x, dot);
            dot = fmaf(q[i + 1], v.y, dot);
            dot = fmaf(q[i + 2], v.z, dot);
            dot = fmaf(q[i + 3], v.w, dot);
        }
    } else {
        for (int i = 0; i < hd; ++i) dot = fmaf(q[i], k[i], dot);
    }
    return dot;
}
__device__ __forceinline__ float dot_row(const float* q, const __nv_bfloat16* k, int hd) {
    float dot = 0.f;
    if ((hd & 7) == 0) {
        for (int i = 0; i < hd; i += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h2[e]);
                dot = fmaf(q[i + 2 * e], f.x, dot);
                dot = fmaf(q[i + 2 * e + 1], f.y, dot);
            }
        }
    } else {
        for (int i = 0; i < hd; ++i) dot = fmaf(q[i], __bfloat162float(k[i]), dot);
    }
    return dot;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* __restrict__ qkv, T* __restrict__ out,
                      const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                      const int* __restrict__ block_table, int max_blocks,
                      const int* __restrict__ positions, const int* __restrict__ req_of_token,
                      int n_tokens, int n_heads, int n_kv, int hd, int block_size, float scale,
                      int window, long long n_pages) {
    chain_release();
    chain_wait();
    __shared__ float q_s[WARPS][MAX_HD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * WARPS + warp;   // (token, head)
    if (unit >= (long long)n_tokens * n_heads) return;
    const int t = (int)(unit / n_heads), h = (int)(unit % n_heads);
    const int kvh = h / (n_heads / n_kv);
    const int r = req_of_token[t];
    const int p = positions[t];
    const int row_w = (n_heads + 2 * n_kv) * hd;

    const T* qp = qkv + (size_t)t * row_w + (size_t)h * hd;
    for (int i = lane; i < hd; i += 32) q_s[warp][i] = Elem<T>::load(qp + i);
    __syncwarp();

    const int j_lo = window > 0 ? max(0, p - window + 1) : 0;
    const int* table = block_table + (size_t)r * max_blocks;
    const int nd = (hd + 31) / 32;

    float m = -INFINITY, l = 0.f;
    float acc[MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;

    for (int j0 = (j_lo / 32) * 32; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j >= j_lo && j <= p;
        float s = -INFINITY;
        if (valid) {
            const int page = table[j / block_size];
            const T* kr = k_pool + (((size_t)kvh * n_pages + page) * block_size + j % block_size) * hd;
            s = dot_row(q_s[warp], kr, hd) * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float pj = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);       // m = -inf on the first chunk: exp(-inf) = 0
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const int key = j0 + jj;
            if (key < j_lo || key > p) continue;        // uniform across the warp
            const float pk = __shfl_sync(0xffffffffu, pj, jj);
            const int page = table[key / block_size];
            const T* vr = v_pool + (((size_t)kvh * n_pages + page) * block_size + key % block_size) * hd;
#pragma unroll
            for (int i = 0; i < MAX_HD / 32; ++i) {
                const int dd = lane + 32 * i;
                if (i < nd && dd < hd) acc[i] = fmaf(pk, Elem<T>::load(vr + dd), acc[i]);
            }
        }
        m = m_new;
    }
    T* op = out + (size_t)t * n_heads * hd + (size_t)h * hd;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) {
        const int dd = lane + 32 * i;
        if (i < nd && dd < hd) Elem<T>::store(op + dd, acc[i] * inv);
    }
}
}  // namespace

MLS_API int mls_attention_simt(const void* qkv, void* out, int dtype, const void* k_pool,
                               const void* v_pool, const int* block_table, int max_blocks,
                               const int* positions, const int* req_of_token, int n_tokens,
                               int n_heads, int n_kv, int hd, int block_size, float scale,
                               int window, long long n_pages, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd > MAX_HD || hd <= 0 || n_heads % n_kv) return MLS_ERR_UNSUPPORTED;
    const long long units = (long long)n_tokens * n_heads;
    const int blocks = (int)((units + WARPS - 1) / WARPS);
    if (dtype == MLS_BF16)
        MLS_LAUNCH((attention_simt_kernel<__nv_bfloat16>), dim3(blocks), dim3(WARPS * 32), 0,
                   stream, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_table,
                   max_blocks, positions, req_of_token, n_tokens, n_heads, n_kv, hd, block_size,
                   scale, window, n_pages);
    else
        MLS_LAUNCH((attention_simt_kernel<float>), dim3(blocks), dim3(WARPS * 32), 0, stream,
                   (const float*)qkv, (float*)out, (const float*)k_pool, (const float*)v_pool,
                   block_table, max_blocks, positions, req_of_token, n_tokens, n_heads, n_kv, hd,
                   block_size, scale, window, n_pages);
    return launch_status();
}
