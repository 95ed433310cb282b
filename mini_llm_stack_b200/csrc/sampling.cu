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

// Rows with temperatures, over a large vocabulary, in two steps like the greedy rows, so
// that the vocabulary is read by many SMs instead of one block a row:
//   1. every block takes CHUNK logits of a row: their maximum z_c = max(x / T) (and where
//      it lies, for rows that turn out greedy), and s_c = sum exp(x / T - z_c);
//   2. one block a row: Z = max z_c; the chunks' weights s_c * exp(z_c - Z) in vocabulary
//      order give the total and, with u, the chunk the draw falls into; inside that
//      chunk the cumulative sum of exp(x / T - z_c) is walked in vocabulary order (every
//      thread sums 16 consecutive tokens, the threads' sums are scanned, one thread
//      walks its tokens).
// The token is still the first whose cumulative probability exceeds u; where the chunk's
// recomputed sum rounds below the stored one, the chunk's last token is taken.
constexpr int PER_THREAD = CHUNK / THREADS;

__global__ void __launch_bounds__(THREADS)
sample_chunks_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                     float* __restrict__ part_val, int* __restrict__ part_idx,
                     float* __restrict__ part_sum, int vocab, int n_chunks) {
    chain_release();
    chain_wait();
    __shared__ float vs[THREADS];
    __shared__ int is[THREADS];
    __shared__ float scratch[33];
    const int begin = blockIdx.y * CHUNK;
    const int len = min(CHUNK, vocab - begin);
    const float* row = logits + (size_t)blockIdx.x * vocab + begin;
    const float temp = temperature[blockIdx.x];
    const float inv_t = temp > 0.f ? 1.0f / temp : 1.0f;
    const int local = block_argmax(row, len, inv_t, vs, is);
    const float mx = row[local] * inv_t;
    float part = 0.f;
    if (temp > 0.f)
        for (int i = threadIdx.x; i < len; i += THREADS) part += expf(row[i] * inv_t - mx);
    const float sum = block_sum(part, scratch);
    if (threadIdx.x == 0) {
        const size_t at = (size_t)blockIdx.x * n_chunks + blockIdx.y;
        part_val[at] = mx;
        part_idx[at] = begin + local;
        part_sum[at] = sum;
    }
}

__global__ void __launch_bounds__(THREADS)
sample_pick_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                   const float* __restrict__ uniform, const float* __restrict__ part_val,
                   const int* __restrict__ part_idx, const float* __restrict__ part_sum,
                   int* __restrict__ out, int vocab, int n_chunks) {
    chain_release();
    chain_wait();
    __shared__ float warp_tot[THREADS / 32];
    __shared__ int s_chunk, s_thread;
    __shared__ float s_before, s_top;
    const float* v = part_val + (size_t)blockIdx.x * n_chunks;
    const int* ix = part_idx + (size_t)blockIdx.x * n_chunks;
    const float* sm = part_sum + (size_t)blockIdx.x * n_chunks;
    const float temp = temperature[blockIdx.x];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp == 0) {
        // the largest chunk maximum, the first chunk on ties (chunks are in index order)
        float best = -INFINITY;
        int idx = NONE, chunk = 0;
        for (int c = lane; c < n_chunks; c += 32) {
            const float x = v[c];
            if (x > best || (idx == NONE && x == best)) { best = x; idx = ix[c]; chunk = c; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
            const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
            const int c2 = __shfl_xor_sync(0xffffffffu, chunk, o);
            if (b2 > best || (b2 == best && i2 < idx)) { best = b2; idx = i2; chunk = c2; }
        }
        if (!(temp > 0.f)) {
            if (lane == 0) out[blockIdx.x] = idx == NONE ? 0 : idx;
        } else if (lane == 0) {
            // the chunks' weights in order: the total, then the chunk the draw falls into
            float total = 0.f;
            for (int c = 0; c < n_chunks; ++c) total += sm[c] * expf(v[c] - best);
            const float target = uniform[blockIdx.x] * total;
            float run = 0.f;
            int pick = -1;
            for (int c = 0; c < n_chunks && pick < 0; ++c) {
                const float w = sm[c] * expf(v[c] - best);
                if (run + w > target) pick = c; else run += w;
            }
            if (pick < 0) {                       // u * total rounded past the last sum
                pick = n_chunks - 1;
                run -= sm[pick] * expf(v[pick] - best);
            }
            s_chunk = pick;
            s_top = best;
            // what is left of the target inside the chunk, in the chunk's own scale
            s_before = (target - run) * expf(best - v[pick]);
        }
    }
    if (!(temp > 0.f)) return;
    if (threadIdx.x == 0) s_thread = NONE;
    __syncthreads();
    const int chunk = s_chunk;
    const float target = s_before;
    const float inv_t = 1.0f / temp, mx = v[chunk];
    const int begin = chunk * CHUNK, len = min(CHUNK, vocab - begin);
    const float* row = logits + (size_t)blockIdx.x * vocab + begin;
    float e[PER_THREAD];
    float mine = 0.f;
    const int first = threadIdx.x * PER_THREAD;
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        e[j] = first + j < len ? expf(row[first + j] * inv_t - mx) : 0.f;
        mine += e[j];
    }
    // exclusive scan of the threads' sums: inside a warp, then over the warps
    float incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    float base = 0.f;
    for (int w = 0; w < warp; ++w) base += warp_tot[w];
    const float before = base + incl - mine;
    if (before + mine > target) atomicMin(&s_thread, (int)threadIdx.x);
    __syncthreads();
    const int who = s_thread == NONE ? (len - 1) / PER_THREAD : s_thread;
    if ((int)threadIdx.x == who) {
        float cum = before;
        int tok = min(len, first + PER_THREAD) - 1;         // where rounding hides the crossing
        for (int j = 0; j < PER_THREAD && first + j < len; ++j) {
            cum += e[j];
            if (cum > target) { tok = first + j; break; }
        }
        out[blockIdx.x] = begin + tok;
    }
}
}  // namespace

// scratch: n_rows * ceil(vocab / 4096) * 3 words, used when the vocabulary is larger
// than 4096 (all rows greedy, temperature == nullptr: two of the three words a chunk);
// pass nullptr to take the one-block-a-row kernel.
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
    if (temperature != nullptr && scratch != nullptr && vocab > CHUNK) {
        const int n_chunks = (vocab + CHUNK - 1) / CHUNK;
        float* part_val = scratch;
        int* part_idx = reinterpret_cast<int*>(scratch + (size_t)n_rows * n_chunks);
        float* part_sum = scratch + 2 * (size_t)n_rows * n_chunks;
        MLS_LAUNCH((sample_chunks_kernel), dim3(n_rows, n_chunks), dim3(THREADS), 0, stream, logits,
                   temperature, part_val, part_idx, part_sum, vocab, n_chunks);
        MLS_LAUNCH((sample_pick_kernel), dim3(n_rows), dim3(THREADS), 0, stream, logits,
                   temperature, uniform, part_val, part_idx, part_sum, out, vocab, n_chunks);
        return launch_status();
    }
    MLS_LAUNCH((sample_kernel), dim3(n_rows), dim3(THREADS), 0, stream, logits, temperature,
               uniform, out, vocab);
    return launch_status();
}
