// Allocation-free entry point of the kernel library.
//
// This declaration has no counterpart in NKKdev/TFFinfer: the reference allocates every
// node's output from its own memory manager and has no split-key attention at all.
//
// Who needs it.  The split-key decode attention of this library needs scratch memory
// for the partial results of the splits, and its ordinary entry point
// (tff_attention_bf16) expects the caller to bring that scratch.  Some callers cannot:
//   * a host program that handed all device memory to a pool of its own at start-up,
//     so that a later cudaMalloc would simply fail;
//   * a latency-critical serving loop, where cudaMalloc / cudaFree synchronise the whole
//     device and stall every stream;
//   * a plain C or C++ host that loads this library without PyTorch and therefore has no
//     caching allocator to ask.
// For them tff_attention_bf16_noalloc keeps the scratch inside the library, in a
// file-scope __device__ array of fixed size, and allocates nothing: no cudaMalloc, no
// cudaFree, no allocating library routine.  The caller still passes inputs and outputs.
//
// Limits and rules.
//   * The array holds TFF_ATTENTION_NOALLOC_SCRATCH_BYTES bytes on every GPU that loads
//     the library, from load until the process exits.
//   * A call needs  tokens * nq * num_splits * (d + 2) * 4  bytes when num_splits > 1
//     (nothing when num_splits == 1); a call that needs more is refused with
//     TFF_ERR_SCRATCH_TOO_SMALL and launches nothing.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and remembers it; make that first
//     call before any stream capture begins on that device.
//   * All calls share the one array, and it keeps what the last call left in it.  Nothing
//     has to be cleared: a call writes every word that it reads back.  Two calls that
//     overlap on the GPU (different streams, no dependency) race on the array; order them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TFF_ATTENTION_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)
#define TFF_ERR_SCRATCH_TOO_SMALL (-6)

// Same arguments and results as tff_attention_bf16 without the workspace pointer:
//   q [tokens, nq*d] bf16 (normalised, rotated), out [tokens, nq*d] bf16, paged cache
//   [pages, cache_layers, 2, nkv, page_size, d] bf16, block_table int32 [requests, table_width],
//   q_start int32 [requests+1], pos_start int32 [requests].
// A cache stored with the layers outermost ([cache_layers, pages, 2, nkv, page_size, d], as the engine
// allocates it) is passed as the block of the layer wanted: cache = that layer's [pages, 2, ...] block,
// cache_layers = 1, layer = 0.
// Returns 0 when the kernels were launched, TFF_ERR_SCRATCH_TOO_SMALL when the call needs
// more scratch than the library holds, or the error codes of tff_attention_bf16.
__attribute__((visibility("default")))
int tff_attention_bf16_noalloc(
    const void* q, const int* q_start, const int* pos_start, const int* block_table, int table_width,
    const void* cache, int cache_layers, int layer, int page_size,
    void* out, int num_tokens, int num_requests, int max_q_len, int num_splits,
    int nq, int nkv, int d, float scale, int window, cudaStream_t stream);

// How many bytes of the array a call with these counts uses (0 when num_splits == 1), computed in 64 bits;
// -1 when a count is not positive or the product is beyond 62 bits.  The entry point above refuses a call
// whose answer is -1 or more than TFF_ATTENTION_NOALLOC_SCRATCH_BYTES.  Launches nothing.
__attribute__((visibility("default")))
long long tff_attention_bf16_noalloc_bytes(long long num_tokens, long long nq, long long num_splits, long long d);

#ifdef __cplusplus
}
#endif
