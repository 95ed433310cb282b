// Sampling over float32 logits [n, V].
//
// Greedy: the reference takes logits.argmax(-1) (serve/engine.py:187-188); ties go
// to the lowest index.  Temperature: the reference draws from
// softmax(logits / temperature) (train/model.py:262-264).  Here the draw is an
// inverse-CDF lookup with a uniform number u given by the host: the token is
// the first index whose cumulative probability exceeds u, in vocabulary order,
// so the same (logits, temperature, u) always gives the same token.  A row whose
// temperature is <= 0 is taken greedily.
#include "common.cuh"

namespace {
constexpr int THREADS = 256;
constexpr int NONE = 0x7fffffff;

__device__ __forceinline__ int block_argmax(const float* row, int vocab, float scale,
                                            float* vs, int* is) {
    float best = -INFINITY;
    int idx = NONE;
    for (int i = threadIdx.x; i < vocab; i += THREADS) {
        const float v = row[i] * scale;
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
    return is[0] == NONE ? 0 : is[0];
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int* __restrict__ out, int vocab) {
    chain_release();
    chain_wait();
    __shared__ float vs[THREADS];
    __shared__ int is[THREADS];
    __shared__ float scratch[33];
    __shared__ int cand;
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const float temp = temperature ? temperature[blockIdx.x] : 0.f;
    if (!(temp > 0.f)) {
        const int tok = block_argmax(row, vocab, 1.0f, vs, is);
        if (threadIdx.x == 0) out[blockIdx.x] = tok;
        return;
    }
    const float inv_t = 1.0f / temp;
    const int top = block_argmax(row, vocab, inv_t, vs, is);
    const float mx = row[top] * inv_t;

    float part = 0.f;
    for (int i = threadIdx.x; i < vocab; i += THREADS) part += expf(row[i] * inv_t - mx);
    const float total = block_sum(part, scratch);
    const float target = uniform[blockIdx.x] * total;

    float running = 0.f;
    int found = -1;
    for (int base = 0; base < vocab && found < 0; base += THREADS) {
        const int i = base + threadIdx.x;
        if (threadIdx.x == 0) cand = NONE;
        vs[threadIdx.x] = i < vocab ? expf(row[i] * inv_t - mx) : 0.f;
        __syncthreads();
        for (int off = 1; off < THREADS; off <<= 1) {       // inclusive scan of the chunk
            const float add = threadIdx.x >= off ? vs[threadIdx.x - off] : 0.f;
            __syncthreads();
            vs[threadIdx.x] += add;
            __syncthreads();
        }
        if (i < vocab && running + vs[threadIdx.x] > target) atomicMin(&cand, i);
        __syncthreads();
        if (cand != NONE) found = cand;
        running += vs[THREADS - 1];
        __syncthreads();
    }
    // u * total may round past the last cumulative sum: the last token then
    if (threadIdx.x == 0) out[blockIdx.x] = found < 0 ? vocab - 1 : found;
}
// Greedy rows only, in two steps so that a few rows still use many SMs: every
// block finds the maximum of CHUNK logits, then one block a row picks among the
// chunks (the lower index on ties, as before).
constexpr int CHUNK = 4096;

__global__ void __launch_bounds__(THREADS)
argmax_chunks_kernel(const float* __restrict__ logits, float* __restrict__ part_val,
                     int* __restrict__ part_idx, int vocab, int n_chunks) {
    chain_release();
    chain_wait();
    __shared__ float vs[THREADS];
    __shared__ int is[THREADS];
    const int begin = blockIdx.y * CHUNK;
    const int len = min(CHUNK, vocab - begin);
    const float* row = logits + (size_t)blockIdx.x * vocab + begin;
    const int local = block_argmax(row, len, 1.0f, vs, is);
    if (threadIdx.x == 0) {
        part_val[blockIdx.x * n_chunks + blockIdx.y] = row[local];
        part_idx[blockIdx.x * n_chunks + blockIdx.y] = begin + local;
    }
}

__global__ void argmax_pick_kernel(const float* __restrict__ part_val,
                                   const int* __restrict__ part_idx, int* __restrict__ out,
                                   int n_chunks) {
    chain_release();
    chain_wait();
    // one warp a row; chunks are in index order, so the first maximum wins
    const float* v = part_val + (size_t)blockIdx.x * n_chunks;
    const int* ix = part_idx + (size_t)blockIdx.x * n_chunks;
    float best = -INFINITY;
    int idx = NONE;
    for (int c = threadIdx.x; c < n_chunks; c += 32) {
        const float x = v[c];
        if (x > best || (idx == NONE && x == best)) { best = x; idx = ix[c]; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        if (b2 > best || (b2 == best && i2 < idx)) { best = b2; idx = i2; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = idx == NONE ? 0 : idx;
}
}  // namespace

// scratch: n_rows * ceil(vocab / 4096) * 2 words, used by the all-greedy path
// (temperature == nullptr); pass nullptr to take the one-block-a-row kernel.
MLS_API int mls_sample(const float* logits, const float* temperature, const float* uniform,
                       int* out, int n_rows, int vocab, float* scratch, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (temperature == nullptr && scratch != nullptr && vocab > CHUNK) {
        const int n_chunks = (vocab + CHUNK - 1) / CHUNK;
        float* part_val = scratch;
        int* part_idx = reinterpret_cast<int*>(scratch + (size_t)n_rows * n_chunks);
        MLS_LAUNCH((argmax_chunks_kernel), dim3(n_rows, n_chunks), dim3(THREADS), 0, stream, logits,
                   part_val, part_idx, vocab, n_chunks);
        MLS_LAUNCH((argmax_pick_kernel), dim3(n_rows), dim3(32), 0, stream, part_val, part_idx, out,
                   n_chunks);
        return launch_status();
    }
    MLS_LAUNCH((sample_kernel), dim3(n_rows), dim3(THREADS), 0, stream, logits, temperature,
               uniform, out, vocab);
    return launch_status();
}
