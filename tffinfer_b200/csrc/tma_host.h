// Host-side helpers shared by the kernels that use TMA: tensor-map construction (through the
// driver entry point, so that the library does not link against libcuda), the device word in
// which a kernel reports that one of its bounded waits ran out, and the SM count.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

// Tensor map of a row-major matrix [rows, cols] of 2-byte (bfloat16) or 4-byte (float32)
// elements: boxes of box_cols x box_rows, 128-byte swizzle (box_cols * elt must be 128), zero fill
// outside the matrix.  Maps are cached by their arguments.  False if the driver refuses.
bool tff_tensor_map_2d(const void* ptr, long long rows, long long cols, int box_rows, int box_cols, int elt,
                       CUtensorMap* out);

// Tensor map over a paged cache [pages, layers, 2 (K,V), kv_heads, page_size, head_dim] of bfloat16 whose
// box is one (page, layer, kv head): 64 columns x (head_dim / 64) halves x page_size rows x {K, V}, with
// 128-byte swizzle.  Coordinates are (0, 0, first K row, 0), rows counted over the whole tensor viewed as
// [rows, head_dim].  False if the driver refuses.
bool tff_tensor_map_kv_page(const void* cache, long long total_rows, int head_dim, int page_size, int kv_heads,
                            CUtensorMap* out);

// Device pointer to the error word (allocated and cleared at first use; nullptr on failure).
int* tff_device_error_flag();

// Number of SMs of the current device (0 on failure).
int tff_num_sms();

// CTAs of a decode-sized product (16 token columns) over ``units`` (tile, K block) units: about a twelfth of the
// SMs' three-a-piece CTA slots stay free, so that a CTA of the product after next can become resident early.
long long tff_decode_gemm_ctas(long long units);
