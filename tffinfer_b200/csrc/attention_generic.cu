// Causal grouped-query attention over the paged cache for flat token rows: one warp
// per (token, query head), any head size, any numbers of heads and groups, optional
// sliding window.  It is the attention of the true 32-bit path and takes every size
// the faster bfloat16 kernels refuse.
//
// For the token at position p of request b and query head h (kv head h / (nq/nkv),
// src/kernel/cuda/paged_flash_attention.cu:891-892):
//   s[n] = (q . k[n]) * scale for lo <= n <= p, lo = window ? max(0, p-window+1) : 0
//   out  = sum_n softmax(s)[n] * v[n]
// with the running-maximum ("online") softmax of the reference
// (paged_flash_attention.cu:696-792) in float32, over key blocks of 32 aligned to
// absolute positions.  The block boundaries depend on p and the window only, so a
// token's result does not depend on how the batch was cut or what else is in it.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q_in, int row_stride,
                         const int* __restrict__ positions, const int* __restrict__ tok_req,
                         const int* __restrict__ block_table, int table_width,
                         const T* __restrict__ cache, KvLayout L, int layer,
                         T* __restrict__ out, int num_tokens, int nq, int nkv, int d,
                         float scale, int window) {
    extern __shared__ float smem[];            // WARPS * d floats: the warp's query row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)num_tokens * nq) return;
    const int t = (int)(item / nq), h = (int)(item % nq);
    const int kvh = h / (nq / nkv);
    const int p = positions[t];
    const int b = tok_req[t];
    const int* table = block_table + (size_t)b * table_width;
    float* q = smem + warp * d;
    const T* qrow = q_in + (size_t)t * row_stride + (size_t)h * d;
    for (int i = lane; i < d; i += 32) q[i] = to_f32<T>(qrow[i]);
    __syncwarp();

    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int nd = (d + 31) / 32;              // output dims per lane (<= 16 for d <= 512)
    float o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int k0 = (lo / 32) * 32; k0 <= p; k0 += 32) {
        const int n = k0 + lane;
        const bool valid = n >= lo && n <= p;
        float s = -INFINITY;
        const T* vbase = nullptr;
        if (valid) {
            const int page = table[n / L.page_size];
            const T* kbase = cache + (size_t)page * L.page_stride + (size_t)layer * L.layer_stride +
                             (size_t)kvh * L.head_stride + (size_t)(n % L.page_size) * d;
            vbase = kbase + L.kv_stride;
            float acc = 0.f;
            for (int i = 0; i < d; ++i) acc = fmaf(q[i], to_f32<T>(kbase[i]), acc);
            s = acc * scale;
        }
        const float bm = warp_max(s);          // at least lane with n == max(k0, lo) .. is valid
        const float m_new = fmaxf(m, bm);
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pr = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pr);
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j] *= alpha;
        for (int kk = 0; kk < 32; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, pr, kk);
            const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)vbase, kk);
            if (vp == 0ull) continue;          // uniform across the warp
            const T* v = (const T*)vp;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (j < nd) {
                    const int i = j * 32 + lane;
                    if (i < d) o[j] = fmaf(pk, to_f32<T>(v[i]), o[j]);
                }
            }
        }
        m = m_new;
    }
    const float inv = 1.f / l;
    T* orow = out + (size_t)t * nq * d + (size_t)h * d;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (j < nd) {
            const int i = j * 32 + lane;
            if (i < d) orow[i] = from_f32<T>(o[j] * inv);
        }
    }
}

}  // namespace

TFF_API int tff_attention_generic(
    const void* qkv, int is_bf16, int row_stride,
    const int* positions, const int* tok_req, const int* block_table, int table_width,
    const void* cache, int cache_layers, int layer, int page_size,
    void* out, int num_tokens, int nq, int nkv, int d, float scale, int window, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || d <= 0 || page_size <= 0) return TFF_ERR_BAD_ARGUMENT;
    if (d > 512) return TFF_ERR_UNSUPPORTED;
    const KvLayout L = make_kv_layout(cache_layers, nkv, page_size, d);
    const long long items = (long long)num_tokens * nq;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * d * sizeof(float);
    if (is_bf16)
        attention_generic_kernel<bf16><<<blocks, WARPS * 32, smem, stream>>>(
            (const bf16*)qkv, row_stride, positions, tok_req, block_table, table_width,
            (const bf16*)cache, L, layer, (bf16*)out, num_tokens, nq, nkv, d, scale, window);
    else
        attention_generic_kernel<float><<<blocks, WARPS * 32, smem, stream>>>(
            (const float*)qkv, row_stride, positions, tok_req, block_table, table_width,
            (const float*)cache, L, layer, (float*)out, num_tokens, nq, nkv, d, scale, window);
    return tff_launch_status();
}
