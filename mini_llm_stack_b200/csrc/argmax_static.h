/* Greedy token choice without any allocation.
 *
 * This entry point has no counterpart in grenver/mini-llm-stack; it exists for
 * callers of this library that are not allowed to allocate device memory at the
 * moment they need a token: code that runs inside a memory budget fixed at start-up
 * (an embedded or multi-tenant host that forbids cudaMalloc after initialisation),
 * code that must not take the allocator's lock or trigger its implicit
 * synchronisation in a latency-critical loop, and hosts that are not PyTorch and so
 * cannot hand the library a scratch tensor from PyTorch's allocator, which is how
 * mls_sample gets its scratch memory.
 *
 *   int mls_argmax_static(const float* logits, int* out, int n_rows, int vocab,
 *                         cudaStream_t stream);
 *
 * logits: device pointer, [n_rows, vocab] float32, row-major.  out: device pointer,
 * n_rows int32; out[i] becomes the index of the largest logit of row i, the lowest
 * index on ties: the same rule and the same result as mls_sample with no
 * temperatures.  Returns 0, a cudaError_t, or MLS_ARGMAX_STATIC_TOO_LARGE.
 *
 * The two-step search keeps one (value, index) pair per 4096 logits in a fixed
 * array in device memory that is part of this library's image:
 * MLS_ARGMAX_STATIC_MAX_PAIRS pairs, 128 KiB, held on every GPU that loads the
 * library until the process exits.  A call needs n_rows * ceil(vocab / 4096) pairs
 * and is refused with MLS_ARGMAX_STATIC_TOO_LARGE (nothing is launched) if that is
 * more; e.g. up to 512 rows of a 131072-token vocabulary.
 *
 * The call allocates nothing and frees nothing.  The first call on a device looks up
 * the array's device address (cudaGetSymbolAddress) and remembers it for that
 * device; make that first call outside any stream capture, with the device current
 * on which `stream` lives.  Later calls only launch two kernels on `stream`.
 *
 * All calls on a device share the array, and it keeps the pairs of the last call.
 * Nothing in it has to start at zero: every pair a call reads it has written itself
 * first.  Two calls that may overlap on the GPU (different streams, no event between
 * them) would overwrite each other's pairs: order them.
 */
#pragma once
#include <cuda_runtime.h>

#define MLS_ARGMAX_STATIC_CHUNK 4096
#define MLS_ARGMAX_STATIC_MAX_PAIRS 16384
#define MLS_ARGMAX_STATIC_TOO_LARGE 100003

#ifdef __cplusplus
extern "C" {
#endif
int mls_argmax_static(const float* logits, int* out, int n_rows, int vocab, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
