// Launcher of the tcgen05 product that runs on pairs of SMs (gemm_tc_pair.cu), called by the entry
// points in gemm_tc.cu.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

// out[M, N] (+)= A[M, K] * W[N, K]^T on 256 x 256 tiles, one tile a cluster of two CTAs.
//   tm_a        A as [M, K], box 64 x 128
//   tm_w_half   W as [N, K], box 64 x 128 (each CTA of a pair loads half of the tile's 256 rows)
//   tm_out      out, boxes of 128 bytes x 32 rows
//   epilogue    0 store, 1 add to what out (float32) holds, 2 SwiGLU of interleaved gate/up columns (bfloat16 out)
//   stream_k    0, or S >= 1: the tiles of the last wave in S slices of their K range (float32 out that holds
//               the initial value)
// Returns a TFF_* status.
int tff_gemm_tc_pair_launch(const CUtensorMap& tm_a, const CUtensorMap& tm_w_half, const CUtensorMap& tm_out, int epilogue,
                            int out_is_bf16, int M, int N, int K, int stream_k, cudaStream_t stream);
