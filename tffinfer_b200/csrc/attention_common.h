// Internal interfaces shared by the attention translation units.
#pragma once
#include <cuda_runtime.h>

// Decode kernel (attention_decode.cu): at most 16 packed query rows per (request, kv head),
// keys streamed by TMA.  Writes ``out`` when num_splits == 1, else the partial results.
int tff_attention_decode_launch(
    const void* q, const int* q_start, const int* pos_start, const int* req_ids, const int* block_table, int table_width,
    const void* cache, long long cache_pages, int cache_layers, int layer, int page_size,
    void* out, float* part_o, float* part_ml, int num_requests, int max_q_len, int num_splits,
    int nq, int nkv, int d, float scale, int window, cudaStream_t stream);

// Prompt-portion kernel (attention_prefill.cu): 128 packed rows per CTA on tcgen05, keys by TMA.
int tff_attention_prefill_launch(
    const void* q, const int* q_start, const int* pos_start, const int* req_ids, const int* block_table, int table_width,
    const void* cache, long long cache_pages, int cache_layers, int layer, int page_size,
    void* out, int num_requests, int max_q_len, int nq, int nkv, int d, float scale, int window, cudaStream_t stream);
