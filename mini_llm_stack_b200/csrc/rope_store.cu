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
// place.  Pools: [Hkv, pages, block, hd] (the pages of one kv head lie side by side);
// slot = page * block + offset.
#include "common.cuh"

template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const int* __restrict__ slot_map, T* __restrict__ k_pool,
                                  T* __restrict__ v_pool, int n_heads, int n_kv, int hd,
                                  int block_size, int max_pos, long long pool_slots, int writes,
                                  int* status) {
    chain_release();
    chain_wait();
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
    const long long n_pages = pool_slots / block_size;

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
            T* dst = k_pool + (((size_t)kvh * n_pages + page) * block_size + off) * hd;
            Elem<T>::store(dst + i, o1);
            Elem<T>::store(dst + i + half, o2);
        }
    }
    if (writes && slot_ok) {
        const T* vsrc = row + (size_t)(n_heads + n_kv) * hd;
        for (int u = threadIdx.x; u < n_kv * hd; u += blockDim.x) {
            const int kvh = u / hd, i = u - kvh * hd;
            v_pool[(((size_t)kvh * n_pages + page) * block_size + off) * hd + i] = vsrc[u];
        }
    }
}

// 16 bytes at a time: VEC = 8 bfloat16 or 4 float32 elements.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            v[2 * e] = f.x;
            v[2 * e + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

// The same work as rope_store_kernel for head sizes whose halves are whole 16-byte
// chunks; one thread rotates one chunk pair of one head, or copies one chunk of v.
template <typename T>
__global__ void rope_store_vec_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                      const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t,
                                      const int* __restrict__ slot_map, T* __restrict__ k_pool,
                                      T* __restrict__ v_pool, int n_heads, int n_kv, int hd,
                                      int block_size, int max_pos, long long pool_slots, int writes,
                                      int* status) {
    chain_release();
    chain_wait();
    constexpr int N = Vec16<T>::N;
    const int t = blockIdx.x;
    const int half = hd >> 1, cph = half / N;            // chunks per half head
    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_POSITION);
        pos = pos < 0 ? 0 : max_pos - 1;
    }
    const float* cr = cos_t + (size_t)pos * half;
    const float* sr = sin_t + (size_t)pos * half;
    T* row = qkv + (size_t)t * (n_heads + 2 * n_kv) * hd;
    long long slot = writes ? (long long)slot_map[t] : 0;
    const bool slot_ok = slot >= 0 && slot < pool_slots;
    if (writes && !slot_ok && threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_SLOT);
    const long long page = slot / block_size, off = slot % block_size;
    const long long n_pages = pool_slots / block_size;

    const int rot_units = (n_heads + (writes ? n_kv : 0)) * cph;
    const int v_units = writes ? n_kv * (hd / N) : 0;
    for (int u = threadIdx.x; u < rot_units + v_units; u += blockDim.x) {
        if (u < rot_units) {
            const int head = u / cph, c = u - head * cph;
            T* hp = row + (size_t)head * hd + c * N;
            float x1[N], x2[N], o1[N], o2[N];
            Vec16<T>::load(hp, x1);
            Vec16<T>::load(hp + half, x2);
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const float cs = cr[c * N + e], sn = sr[c * N + e];
                o1[e] = __fsub_rn(__fmul_rn(x1[e], cs), __fmul_rn(x2[e], sn));
                o2[e] = __fadd_rn(__fmul_rn(x2[e], cs), __fmul_rn(x1[e], sn));
            }
            if (head < n_heads) {
                Vec16<T>::store(hp, o1);
                Vec16<T>::store(hp + half, o2);
            } else if (slot_ok) {
                const int kvh = head - n_heads;
                T* dst = k_pool + (((size_t)kvh * n_pages + page) * block_size + off) * hd + c * N;
                Vec16<T>::store(dst, o1);
                Vec16<T>::store(dst + half, o2);
            }
        } else if (slot_ok) {
            const int w = u - rot_units;
            const int per = hd / N;
            const int kvh = w / per, c = w - kvh * per;
            const uint4 raw = *reinterpret_cast<const uint4*>(
                row + (size_t)(n_heads + n_kv + kvh) * hd + c * N);
            *reinterpret_cast<uint4*>(
                v_pool + (((size_t)kvh * n_pages + page) * block_size + off) * hd + c * N) = raw;
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
    const int vec_n = dtype == MLS_BF16 ? 8 : 4;
    if ((hd / 2) % vec_n == 0) {
        const int units = ((n_heads + n_kv) * (hd / 2) + n_kv * hd) / vec_n;
        int vthreads = 32;
        while (vthreads < 512 && vthreads < units) vthreads <<= 1;
        if (dtype == MLS_BF16)
            MLS_LAUNCH((rope_store_vec_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(vthreads), 0,
                       stream, (__nv_bfloat16*)qkv, positions, cos_t, sin_t, slot_map,
                       (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_heads, n_kv, hd,
                       block_size, max_pos, pool_slots, writes, status);
        else
            MLS_LAUNCH((rope_store_vec_kernel<float>), dim3(n_tokens), dim3(vthreads), 0, stream,
                       (float*)qkv, positions, cos_t, sin_t, slot_map, (float*)k_pool,
                       (float*)v_pool, n_heads, n_kv, hd, block_size, max_pos, pool_slots, writes,
                       status);
        return launch_status();
    }
    const int work = (n_heads + n_kv) * hd / 2;
    int threads = 64;
    while (threads < 512 && threads < work) threads <<= 1;
    if (dtype == MLS_BF16)
        MLS_LAUNCH((rope_store_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(threads), 0, stream,
                   (__nv_bfloat16*)qkv, positions, cos_t, sin_t, slot_map, (__nv_bfloat16*)k_pool,
                   (__nv_bfloat16*)v_pool, n_heads, n_kv, hd, block_size, max_pos, pool_slots,
                   writes, status);
    else
        MLS_LAUNCH((rope_store_kernel<float>), dim3(n_tokens), dim3(threads), 0, stream,
                   (float*)qkv, positions, cos_t, sin_t, slot_map, (float*)k_pool, (float*)v_pool,
                   n_heads, n_kv, hd, block_size, max_pos, pool_slots, writes, status);
    return launch_status();
}
