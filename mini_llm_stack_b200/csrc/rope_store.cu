// Rotary position encoding of q and k, and the write of k and v into the pages.
//
// Reference: tables cos/sin [max_pos, hd/2] in float32 (train/model.py:41-45);
// x1, x2 = halves of a head; out = cat(x1*cos - x2*sin, x2*cos + x1*sin)
// (train/model.py:47-52, serve/engine.py:53-58), applied to q and k only; the
// rotated k and the raw v of the step's tokens are stored before attention
// (serve/engine.py:99-100,137-139).  The products and sums are separate float32
// operations (no fused multiply-add), as in the reference's expression.
//
// qkv: [T, (H + 2*Hkv) * hd], rows [q heads | k heads | v heads]; q is rotated in
// place.  Pools: [pages, Hkv, block, hd]; slot = page * block + offset.
#include "common.cuh"

template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const int* __restrict__ slot_map, T* __restrict__ k_pool,
                                  T* __restrict__ v_pool, int n_heads, int n_kv, int hd,
                                  int block_size, int max_pos, long long pool_slots, int writes,
                                  int* status) {
    const int t = blockIdx.x;
    const int half = hd >> 1;
    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_POSITION);
        pos = pos < 0 ? 0 : max_pos - 1;
    }
    const float* cr = cos_t + (size_t)pos * half;
    const float* sr = sin_t + (size_t)pos * half;
    T* row = qkv + (size_t)t * (n_heads + 2 * n_kv) * hd;

    long long slot = writes ? (long long)slot_map[t] : 0;
    bool slot_ok = slot >= 0 && slot < pool_slots;
    if (writes && !slot_ok) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_SLOT);
    }
    const long long page = slot / block_size, off = slot % block_size;

    const int rot_heads = n_heads + (writes ? n_kv : 0);
    for (int u = threadIdx.x; u < rot_heads * half; u += blockDim.x) {
        const int head = u / half, i = u - head * half;
        T* hp = row + (size_t)head * hd;
        const float x1 = Elem<T>::load(hp + i), x2 = Elem<T>::load(hp + i + half);
        const float c = cr[i], s = sr[i];
        const float o1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
        const float o2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
        if (head < n_heads) {
            Elem<T>::store(hp + i, o1);
            Elem<T>::store(hp + i + half, o2);
        } else if (slot_ok) {
            const int kvh = head - n_heads;
            T* dst = k_pool + (((size_t)page * n_kv + kvh) * block_size + off) * hd;
            Elem<T>::store(dst + i, o1);
            Elem<T>::store(dst + i + half, o2);
        }
    }
    if (writes && slot_ok) {
        const T* vsrc = row + (size_t)(n_heads + n_kv) * hd;
        for (int u = threadIdx.x; u < n_kv * hd; u += blockDim.x) {
            const int kvh = u / hd, i = u - kvh * hd;
            v_pool[(((size_t)page * n_kv + kvh) * block_size + off) * hd + i] = vsrc[u];
        }
    }
}

MLS_API int mls_rope_store(void* qkv, int dtype, const int* positions, const float* cos_t,
                           const float* sin_t, const int* slot_map, void* k_pool, void* v_pool,
                           int n_tokens, int n_heads, int n_kv, int hd, int block_size,
                           int max_pos, long long pool_slots, int writes, int* status,
                           cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd % 2) return MLS_ERR_UNSUPPORTED;
    const int work = (n_heads + n_kv) * hd / 2;
    int threads = 64;
    while (threads < 512 && threads < work) threads <<= 1;
    if (dtype == MLS_BF16)
        rope_store_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            (__nv_bfloat16*)qkv, positions, cos_t, sin_t, slot_map, (__nv_bfloat16*)k_pool,
            (__nv_bfloat16*)v_pool, n_heads, n_kv, hd, block_size, max_pos, pool_slots, writes,
            status);
    else
        rope_store_kernel<float><<<n_tokens, threads, 0, stream>>>(
            (float*)qkv, positions, cos_t, sin_t, slot_map, (float*)k_pool, (float*)v_pool,
            n_heads, n_kv, hd, block_size, max_pos, pool_slots, writes, status);
    return launch_status();
}
