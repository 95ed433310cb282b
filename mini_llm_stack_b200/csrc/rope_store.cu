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

// What lies in a page past its owner's last token is whatever the page's previous owner
// left there.  The attention kernels never count those slots, but the tensor-core ones
// mask the scores, not the values: a probability of 0 times a leftover NaN or Inf would
// still be NaN.  So the slots are cleared when a request enters a page: the token that
// is the last of its request in this step zeroes the rest of its page (keys and values
// of every kv head) if the page's first slot was written in this step too.  Pages are
// owned by one request, so "the next token has the next slot" means "same request", and
// "the token `off` places back has this page's first slot" means the page was entered
// in this step.  Cleared by all threads of one block per token, after chain_wait().
// How many slots after `slot` are to be cleared by token t's block (0: none).  Reads only
// the step's slot map, which no kernel of the step writes: callers ask before chain_wait,
// so that the two loads do not add to what follows the wait.
__device__ __forceinline__ int page_tail_to_clear(const int* __restrict__ slot_map, int t,
                                                  int n_tokens, int slot, int block_size) {
    const int off = slot % block_size;
    const int rest = block_size - 1 - off;
    if (rest <= 0 || slot < 0) return 0;
    const int next = t + 1 < n_tokens ? slot_map[t + 1] : -1;
    const int first = (off > 0 && t - off >= 0) ? slot_map[t - off] : -1;
    if (next == slot + 1) return 0;                                     // not the last one
    if (off > 0 && first != slot - off) return 0;                       // an older page
    return rest;
}
template <typename T>
__device__ __forceinline__ void clear_page_tail(int rest, int slot, int block_size, int n_pages,
                                                int n_kv, int hd, T* __restrict__ k_pool,
                                                T* __restrict__ v_pool) {
    if (rest <= 0) return;
    const int page = slot / block_size, off = slot - page * block_size;
    const size_t row_bytes = (size_t)hd * sizeof(T);
    if (row_bytes % 16 == 0) {
        const int chunks = (int)(row_bytes / 16) * rest;                 // per kv head and pool
        for (int u = threadIdx.x; u < 2 * n_kv * chunks; u += blockDim.x) {
            const int which = u / (n_kv * chunks), w = u - which * n_kv * chunks;
            const int kvh = w / chunks, c = w - kvh * chunks;
            T* base = (which ? v_pool : k_pool) +
                      (((size_t)kvh * n_pages + page) * block_size + off + 1) * hd;
            reinterpret_cast<uint4*>(base)[c] = make_uint4(0u, 0u, 0u, 0u);
        }
    } else {
        const int elems = hd * rest;
        for (int u = threadIdx.x; u < 2 * n_kv * elems; u += blockDim.x) {
            const int which = u / (n_kv * elems), w = u - which * n_kv * elems;
            const int kvh = w / elems, c = w - kvh * elems;
            T* base = (which ? v_pool : k_pool) +
                      (((size_t)kvh * n_pages + page) * block_size + off + 1) * hd;
            Elem<T>::store(base + c, 0.f);
        }
    }
}

template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const int* __restrict__ slot_map, T* __restrict__ k_pool,
                                  T* __restrict__ v_pool, int n_heads, int n_kv, int hd,
                                  int block_size, int max_pos, int pool_slots, int writes,
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

    const int slot = writes ? slot_map[t] : 0;      // 32-bit: the divisions below are per thread
    bool slot_ok = slot >= 0 && slot < pool_slots;
    if (writes && !slot_ok) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_SLOT);
    }
    const int page = slot / block_size, off = slot - page * block_size;
    const int n_pages = pool_slots / block_size;

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
        clear_page_tail<T>(page_tail_to_clear(slot_map, t, gridDim.x, slot, block_size), slot,
                           block_size, n_pages, n_kv, hd, k_pool, v_pool);
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
__global__ void __launch_bounds__(512, 3)
rope_store_vec_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                      const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t,
                                      const int* __restrict__ slot_map, T* __restrict__ k_pool,
                                      T* __restrict__ v_pool, int n_heads, int n_kv, int hd,
                                      int block_size, int max_pos, int pool_slots, int writes,
                                      int* status) {
    chain_release();
    constexpr int N = Vec16<T>::N;
    const int t = blockIdx.x;
    const int half = hd >> 1, cph = half / N;            // chunks per half head
    // positions and slots were copied before the step's first kernel began
    int pos = positions[t];
    const bool bad_pos = pos < 0 || pos >= max_pos;
    if (bad_pos) pos = pos < 0 ? 0 : max_pos - 1;
    const float* cr = cos_t + (size_t)pos * half;
    const float* sr = sin_t + (size_t)pos * half;
    T* row = qkv + (size_t)t * (n_heads + 2 * n_kv) * hd;
    const int slot = writes ? slot_map[t] : 0;      // 32-bit: the divisions below are per thread
    const bool slot_ok = slot >= 0 && slot < pool_slots;
    const int page = slot / block_size, off = slot - page * block_size;
    const int n_pages = pool_slots / block_size;
    const int tail = (writes && slot_ok)
                         ? page_tail_to_clear(slot_map, t, gridDim.x, slot, block_size) : 0;
    chain_wait();
    if (threadIdx.x == 0 && status) {
        if (bad_pos) atomicOr(status, MLS_STATUS_BAD_POSITION);
        if (writes && !slot_ok) atomicOr(status, MLS_STATUS_BAD_SLOT);
    }

    const int rot_units = (n_heads + (writes ? n_kv : 0)) * cph;
    const int v_units = writes ? n_kv * (hd / N) : 0;
    for (int u = threadIdx.x; u < rot_units + v_units; u += blockDim.x) {
        if (u < rot_units) {
            const int head = u / cph, c = u - head * cph;
            T* hp = row + (size_t)head * hd + c * N;
            float x1[N], x2[N], o1[N], o2[N], cs[N], sn[N];
            Vec16<T>::load(hp, x1);
            Vec16<T>::load(hp + half, x2);
#pragma unroll
            for (int e = 0; e < N; e += 4) {          // half is a multiple of N: whole float4s
                const float4 c4 = *reinterpret_cast<const float4*>(cr + c * N + e);
                const float4 s4 = *reinterpret_cast<const float4*>(sr + c * N + e);
                cs[e] = c4.x, cs[e + 1] = c4.y, cs[e + 2] = c4.z, cs[e + 3] = c4.w;
                sn[e] = s4.x, sn[e + 1] = s4.y, sn[e + 2] = s4.z, sn[e + 3] = s4.w;
            }
#pragma unroll
            for (int e = 0; e < N; ++e) {
                o1[e] = __fsub_rn(__fmul_rn(x1[e], cs[e]), __fmul_rn(x2[e], sn[e]));
                o2[e] = __fadd_rn(__fmul_rn(x2[e], cs[e]), __fmul_rn(x1[e], sn[e]));
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
    clear_page_tail<T>(tail, slot, block_size, n_pages, n_kv, hd, k_pool, v_pool);
}

// The rows are still in the parts a matrix product was cut into along K (float32
// [n_parts][tokens][row width]): a thread adds up four values of each half of a head
// in the order of the parts, rounds them to bfloat16 as the finished product would
// have been, and goes on as above.  Rotated queries go to qkv; the keys and values
// only to the pages.  gridDim.y blocks share a token, so that with few tokens more
// than a handful of SMs pull the parts in.
constexpr int PARTS_THREADS = 64;
__global__ void __launch_bounds__(PARTS_THREADS)
rope_store_parts_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                        const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                        const int* __restrict__ slot_map, __nv_bfloat16* __restrict__ k_pool,
                        __nv_bfloat16* __restrict__ v_pool, int n_heads, int n_kv, int hd,
                        int block_size, int max_pos, int pool_slots, int writes,
                        const float* __restrict__ parts, int n_parts, size_t part_stride,
                        int* status) {
    chain_release();
    const int t = blockIdx.x;
    const int half = hd >> 1, qph = half / 4;            // groups of four per half head
    int pos = positions[t];
    const bool bad_pos = pos < 0 || pos >= max_pos;
    if (bad_pos) pos = pos < 0 ? 0 : max_pos - 1;
    const float* cr = cos_t + (size_t)pos * half;
    const float* sr = sin_t + (size_t)pos * half;
    const size_t width = (size_t)(n_heads + 2 * n_kv) * hd;
    const int slot = writes ? slot_map[t] : 0;      // 32-bit: the divisions below are per thread
    const bool slot_ok = slot >= 0 && slot < pool_slots;
    const int page = slot / block_size, off = slot - page * block_size;
    const int n_pages = pool_slots / block_size;
    const int rot_units = (n_heads + (writes ? n_kv : 0)) * qph;
    const int v_units = writes ? n_kv * (hd / 4) : 0;
    const int per_block = (rot_units + v_units + gridDim.y - 1) / gridDim.y;
    const int u_end = min(rot_units + v_units, (int)(blockIdx.y + 1) * per_block);
    const int tail = (writes && slot_ok && blockIdx.y == gridDim.y - 1)
                         ? page_tail_to_clear(slot_map, t, gridDim.x, slot, block_size) : 0;
    chain_wait();
    if (threadIdx.x == 0 && blockIdx.y == 0 && status) {
        if (bad_pos) atomicOr(status, MLS_STATUS_BAD_POSITION);
        if (writes && !slot_ok) atomicOr(status, MLS_STATUS_BAD_SLOT);
    }
    for (int u = blockIdx.y * per_block + threadIdx.x; u < u_end; u += blockDim.x) {
        if (u < rot_units) {
            const int head = u / qph, c = u - head * qph;
            const size_t col = (size_t)head * hd + c * 4;
            const size_t at[2] = {(size_t)t * width + col, (size_t)t * width + col + half};
            float4 x[2];
            sum_parts4_of<2, 8>(parts, at, n_parts, part_stride, x);
            const float4 x1 = round_bf16(x[0]), x2 = round_bf16(x[1]);
            const float4 cs = *reinterpret_cast<const float4*>(cr + c * 4);
            const float4 sn = *reinterpret_cast<const float4*>(sr + c * 4);
            float4 o1, o2;
            o1.x = __fsub_rn(__fmul_rn(x1.x, cs.x), __fmul_rn(x2.x, sn.x));
            o1.y = __fsub_rn(__fmul_rn(x1.y, cs.y), __fmul_rn(x2.y, sn.y));
            o1.z = __fsub_rn(__fmul_rn(x1.z, cs.z), __fmul_rn(x2.z, sn.z));
            o1.w = __fsub_rn(__fmul_rn(x1.w, cs.w), __fmul_rn(x2.w, sn.w));
            o2.x = __fadd_rn(__fmul_rn(x2.x, cs.x), __fmul_rn(x1.x, sn.x));
            o2.y = __fadd_rn(__fmul_rn(x2.y, cs.y), __fmul_rn(x1.y, sn.y));
            o2.z = __fadd_rn(__fmul_rn(x2.z, cs.z), __fmul_rn(x1.z, sn.z));
            o2.w = __fadd_rn(__fmul_rn(x2.w, cs.w), __fmul_rn(x1.w, sn.w));
            __nv_bfloat16* dst = nullptr;
            if (head < n_heads) {
                dst = qkv + (size_t)t * width + col;
            } else if (slot_ok) {
                const int kvh = head - n_heads;
                dst = k_pool + (((size_t)kvh * n_pages + page) * block_size + off) * hd + c * 4;
            }
            if (dst) {
                *reinterpret_cast<uint2*>(dst) = pack_bf16x4(o1);
                *reinterpret_cast<uint2*>(dst + half) = pack_bf16x4(o2);
            }
        } else if (slot_ok) {
            const int w = u - rot_units;
            const int per = hd / 4;
            const int kvh = w / per, c = w - kvh * per;
            const size_t at[1] = {(size_t)t * width + (size_t)(n_heads + n_kv + kvh) * hd + c * 4};
            float4 x[1];
            sum_parts4_of<1, 8>(parts, at, n_parts, part_stride, x);
            *reinterpret_cast<uint2*>(
                v_pool + (((size_t)kvh * n_pages + page) * block_size + off) * hd + c * 4) =
                pack_bf16x4(x[0]);
        }
    }
    clear_page_tail<__nv_bfloat16>(tail, slot, block_size, n_pages, n_kv, hd, k_pool, v_pool);
}

MLS_API int mls_rope_store(void* qkv, int dtype, const int* positions, const float* cos_t,
                           const float* sin_t, const int* slot_map, void* k_pool, void* v_pool,
                           int n_tokens, int n_heads, int n_kv, int hd, int block_size,
                           int max_pos, long long pool_slots, int writes, const float* parts,
                           int n_parts, long long part_stride, int* status,
                           cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd % 2) return MLS_ERR_UNSUPPORTED;
    // slots are int32
    if (pool_slots > 0x7fffffffLL || block_size <= 0) return MLS_ERR_UNSUPPORTED;
    const int vec_n = dtype == MLS_BF16 ? 8 : 4;
    if (parts) {
        // rows still in parts: bfloat16 activations, whole float4s in every part
        if (dtype != MLS_BF16 || (hd / 2) % 4 != 0 || n_parts < 1 || part_stride % 4 != 0)
            return MLS_ERR_UNSUPPORTED;
        const int units = ((n_heads + n_kv) * (hd / 2) + n_kv * hd) / 4;
        int per_token = (units + PARTS_THREADS - 1) / PARTS_THREADS;
        if (n_tokens * per_token > 592) per_token = (592 + n_tokens - 1) / n_tokens;
        MLS_LAUNCH((rope_store_parts_kernel), dim3(n_tokens, per_token), dim3(PARTS_THREADS), 0,
                   stream, (__nv_bfloat16*)qkv, positions, cos_t, sin_t, slot_map,
                   (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_heads, n_kv, hd, block_size,
                   max_pos, (int)pool_slots, writes, parts, n_parts, (size_t)part_stride, status);
        return launch_status();
    }
    if ((hd / 2) % vec_n == 0) {
        const int units = ((n_heads + n_kv) * (hd / 2) + n_kv * hd) / vec_n;
        int vthreads = 32;
        while (vthreads < 512 && vthreads < units) vthreads <<= 1;
        if (dtype == MLS_BF16)
            MLS_LAUNCH((rope_store_vec_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(vthreads), 0,
                       stream, (__nv_bfloat16*)qkv, positions, cos_t, sin_t, slot_map,
                       (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_heads, n_kv, hd,
                       block_size, max_pos, (int)pool_slots, writes, status);
        else
            MLS_LAUNCH((rope_store_vec_kernel<float>), dim3(n_tokens), dim3(vthreads), 0, stream,
                       (float*)qkv, positions, cos_t, sin_t, slot_map, (float*)k_pool,
                       (float*)v_pool, n_heads, n_kv, hd, block_size, max_pos, (int)pool_slots,
                       writes, status);
        return launch_status();
    }
    const int work = (n_heads + n_kv) * hd / 2;
    int threads = 64;
    while (threads < 512 && threads < work) threads <<= 1;
    if (dtype == MLS_BF16)
        MLS_LAUNCH((rope_store_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(threads), 0, stream,
                   (__nv_bfloat16*)qkv, positions, cos_t, sin_t, slot_map, (__nv_bfloat16*)k_pool,
                   (__nv_bfloat16*)v_pool, n_heads, n_kv, hd, block_size, max_pos, (int)pool_slots,
                   writes, status);
    else
        MLS_LAUNCH((rope_store_kernel<float>), dim3(n_tokens), dim3(threads), 0, stream,
                   (float*)qkv, positions, cos_t, sin_t, slot_map, (float*)k_pool, (float*)v_pool,
                   n_heads, n_kv, hd, block_size, max_pos, (int)pool_slots, writes, status);
    return launch_status();
}
