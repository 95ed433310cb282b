// Greedy token choice with its scratch memory inside the library image; see
// argmax_static.h for the contract.  The kernels are the two-step arg max of
// sampling.cu (one block per 4096 logits, then one warp per row), reading and
// writing a file-scope device array instead of memory the caller allocated.
#include "argmax_static.h"
#include "common.cuh"

namespace {
constexpr int THREADS = 256;
constexpr int NONE = 0x7fffffff;
constexpr int MAX_DEVICES = 64;

struct Pair {
    float value;
    int index;
};

// The scratch memory: lives in the library's image on every device that loads it.
static __device__ __align__(256) Pair g_pairs[MLS_ARGMAX_STATIC_MAX_PAIRS];

__global__ void __launch_bounds__(THREADS)
static_chunks_kernel(const float* __restrict__ logits, Pair* __restrict__ pairs, int vocab,
                     int n_chunks) {
    __shared__ float vs[THREADS];
    __shared__ int is[THREADS];
    const int begin = blockIdx.y * MLS_ARGMAX_STATIC_CHUNK;
    const int len = min(MLS_ARGMAX_STATIC_CHUNK, vocab - begin);
    const float* row = logits + (size_t)blockIdx.x * vocab + begin;
    float best = -INFINITY;
    int idx = NONE;
    for (int i = threadIdx.x; i < len; i += THREADS) {
        const float v = row[i];
        if (v > best || (idx == NONE && v == best)) { best = v; idx = i; }
    }
    vs[threadIdx.x] = best;
    is[threadIdx.x] = idx;
    __syncthreads();
    for (int s = THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float v2 = vs[threadIdx.x + s];
            const int i2 = is[threadIdx.x + s];
            if (v2 > vs[threadIdx.x] || (v2 == vs[threadIdx.x] && i2 < is[threadIdx.x])) {
                vs[threadIdx.x] = v2;
                is[threadIdx.x] = i2;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const int local = is[0] == NONE ? 0 : is[0];
        Pair p;
        p.value = row[local];
        p.index = begin + local;
        pairs[blockIdx.x * n_chunks + blockIdx.y] = p;
    }
}

__global__ void static_pick_kernel(const Pair* __restrict__ pairs, int* __restrict__ out,
                                   int n_chunks) {
    const Pair* mine = pairs + (size_t)blockIdx.x * n_chunks;
    float best = -INFINITY;
    int idx = NONE;
    for (int c = threadIdx.x; c < n_chunks; c += 32) {
        const Pair p = mine[c];
        if (p.value > best || (idx == NONE && p.value == best)) { best = p.value; idx = p.index; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        if (b2 > best || (b2 == best && i2 < idx)) { best = b2; idx = i2; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = idx == NONE ? 0 : idx;
}

// In host code `g_pairs` is only a handle for the runtime, not an address the GPU
// can use: the address a kernel may be given comes from cudaGetSymbolAddress, asked
// once per device while that device is current.
Pair* g_pairs_on_device[MAX_DEVICES] = {nullptr};

int scratch_address(Pair** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    if (g_pairs_on_device[dev] == nullptr) {
        Pair* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_pairs);
        if (e != cudaSuccess) return (int)e;
        g_pairs_on_device[dev] = p;
    }
    *out = g_pairs_on_device[dev];
    return 0;
}
}  // namespace

extern "C" __attribute__((visibility("default")))
int mls_argmax_static(const float* logits, int* out, int n_rows, int vocab, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return (int)cudaErrorInvalidValue;
    const long long n_chunks =
        ((long long)vocab + MLS_ARGMAX_STATIC_CHUNK - 1) / MLS_ARGMAX_STATIC_CHUNK;
    if ((long long)n_rows * n_chunks > MLS_ARGMAX_STATIC_MAX_PAIRS)
        return MLS_ARGMAX_STATIC_TOO_LARGE;
    Pair* pairs = nullptr;
    const int rc = scratch_address(&pairs);
    if (rc != 0) return rc;
    static_chunks_kernel<<<dim3(n_rows, (unsigned)n_chunks), THREADS, 0, stream>>>(
        logits, pairs, vocab, (int)n_chunks);
    static_pick_kernel<<<n_rows, 32, 0, stream>>>(pairs, out, (int)n_chunks);
    return (int)cudaGetLastError();
}
