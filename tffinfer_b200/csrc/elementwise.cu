// Memory-bound kernels of the step: embedding gather, RMSNorm, SwiGLU, the rotary
// table, and the fused per-head q/k RMSNorm + RoPE + paged K/V write.
// Every reduction and every rotation is done in float32 whatever the storage type.
#include "common.cuh"
#include "tma_host.h"

// grids of the grid-stride kernels: a few CTAs for every SM of the device the call runs on
static inline long long sm_count() { const int n = tff_num_sms(); return n > 0 ? n : 1; }

// ---------------------------------------------------------------- embedding
// x[t, :] = float(E[token[t], :]).  Stands where the reference gathers (and
// de-quantises) embedding rows on the CPU: src/kernel/cpu/embedding.cpp:35-49.
// ``scale`` multiplies every element (1 for this architecture, whose embedding is not scaled: the product
// with 1.0f is exact; architectures that scale by sqrt(hidden) or another constant say so in their description).
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ out, int hidden, int vocab, float scale) {
    pdl_launch_dependents();          // the next kernel may become resident (it waits before it reads or writes)
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* o = out + (size_t)t * hidden;
    if (tok < 0 || tok >= vocab) {             // never a wrong row: poison instead
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = __int_as_float(0x7fc00000);
        return;
    }
    const TW* row = table + (size_t)tok * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = to_f32<TW>(row[h]) * scale;
}

TFF_API int tff_embed(const int* tokens, const void* table, int table_is_bf16, float* out,
                      int num_tokens, int hidden, int vocab, float scale, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (hidden <= 0 || vocab <= 0) return TFF_ERR_BAD_ARGUMENT;
    const int nt = hidden >= 1024 ? 256 : 128;
    if (table_is_bf16) return tff_launch_pdl(embed_kernel<bf16>, num_tokens, nt, 0, stream, tokens, (const bf16*)table, out, hidden, vocab, scale);
    return tff_launch_pdl(embed_kernel<float>, num_tokens, nt, 0, stream, tokens, (const float*)table, out, hidden, vocab, scale);
}

// four consecutive outputs in one store
template <typename T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

// ------------------------------------------------------------------ RMSNorm
// out[r, :] = (x[row, :] * rsqrt(mean(x[row]^2) + eps)) * w, row = row_index ? row_index[r] : r.
// Formula and multiplication order of src/kernel/cuda/norm.cu:31-48.
template <typename TO, int NT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               const int* __restrict__ row_index, TO* __restrict__ out,
                               int dim, float eps) {
    __shared__ float red[32];
    pdl_launch_dependents();          // the next kernel may become resident (it waits before it reads or writes)
    // the row index and the weights are older than the kernel ahead: fetched before waiting for it
    const int r = blockIdx.x;
    const int row = row_index ? row_index[r] : r;
    const float* xr = x + (size_t)row * dim;
    TO* o = out + (size_t)r * dim;
    float ss = 0.f;
    // four elements a thread at a time when the row allows 16-byte accesses (the order of the additions
    // still depends on the row's width alone)
    const bool vec = (dim & 3) == 0 && (((uintptr_t)xr | (uintptr_t)w) & 15) == 0 && ((uintptr_t)o & 7) == 0 &&
                     (sizeof(TO) == 2 || ((uintptr_t)o & 15) == 0);
    if (vec) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        const float4* w4 = reinterpret_cast<const float4*>(w);
        const int n4 = dim >> 2;
        // a thread's first KEEP pieces stay in registers between the two passes (rows up to 16 * KEEP * NT / 4
        // elements are read from memory once); the loads of a pass are issued together
        constexpr int KEEP = 4;
        float4 keep[KEEP], wk[KEEP];
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int i = threadIdx.x + k * NT;
            wk[k] = i < n4 ? w4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        pdl_wait();
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int i = threadIdx.x + k * NT;
            keep[k] = i < n4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            ss = fmaf(keep[k].x, keep[k].x, ss); ss = fmaf(keep[k].y, keep[k].y, ss);
            ss = fmaf(keep[k].z, keep[k].z, ss); ss = fmaf(keep[k].w, keep[k].w, ss);
        }
        for (int i = threadIdx.x + KEEP * NT; i < n4; i += NT) {
            const float4 v = x4[i];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum<NT>(ss, red);
        const float rs = rsqrtf(ss / (float)dim + eps);
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int i = threadIdx.x + k * NT;
            if (i < n4) {
                const float4 v = keep[k], g = wk[k];
                store4<TO>(o + 4 * i, (v.x * rs) * g.x, (v.y * rs) * g.y, (v.z * rs) * g.z, (v.w * rs) * g.w);
            }
        }
        for (int i = threadIdx.x + KEEP * NT; i < n4; i += NT) {
            const float4 v = x4[i], g = w4[i];
            store4<TO>(o + 4 * i, (v.x * rs) * g.x, (v.y * rs) * g.y, (v.z * rs) * g.z, (v.w * rs) * g.w);
        }
        return;
    }
    pdl_wait();
    for (int i = threadIdx.x; i < dim; i += NT) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum<NT>(ss, red);
    const float rs = rsqrtf(ss / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += NT) o[i] = from_f32<TO>((xr[i] * rs) * w[i]);
}

TFF_API int tff_rmsnorm(const float* x, const float* w, const int* row_index, void* out, int out_is_bf16,
                        int rows, int dim, float eps, cudaStream_t stream) {
    if (rows <= 0) return TFF_OK;
    if (dim <= 0) return TFF_ERR_BAD_ARGUMENT;
    if (dim >= 1024) {
        if (out_is_bf16) return tff_launch_pdl(rmsnorm_kernel<bf16, 256>, rows, 256, 0, stream, x, w, row_index, (bf16*)out, dim, eps);
        return tff_launch_pdl(rmsnorm_kernel<float, 256>, rows, 256, 0, stream, x, w, row_index, (float*)out, dim, eps);
    }
    if (out_is_bf16) return tff_launch_pdl(rmsnorm_kernel<bf16, 64>, rows, 64, 0, stream, x, w, row_index, (bf16*)out, dim, eps);
    return tff_launch_pdl(rmsnorm_kernel<float, 64>, rows, 64, 0, stream, x, w, row_index, (float*)out, dim, eps);
}

// ------------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(g) = g / (1 + exp(-g))
// (src/kernel/cuda/unary.cu:10-27: x1 = gate, x2 = up).
// ``block`` = 0: gu[t] = [gate (I) | up (I)]; ``block`` = b > 0: gate and up alternate in blocks of b
// columns, gate feature i at column (i / b) * 2b + i % b and its up feature b columns further.
// ``clear`` != 0: the input is set to zero once it has been read (it is an accumulator buffer the
// next split product adds into).
template <typename TIN, typename T>
__global__ void swiglu_kernel(TIN* __restrict__ gu, T* __restrict__ out, long long total, int inter, int block, int clear) {
    pdl_launch_dependents();          // the next kernel may become resident (it waits before it reads or writes)
    pdl_wait();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / inter;
        const int i = (int)(idx - t * inter);
        const int gc = block > 0 ? (i / block) * 2 * block + i % block : i;
        const int uc = block > 0 ? gc + block : inter + i;
        const float g = to_f32<TIN>(gu[t * 2 * inter + gc]);
        const float u = to_f32<TIN>(gu[t * 2 * inter + uc]);
        out[idx] = from_f32<T>((g / (1.0f + expf(-g))) * u);
        if (clear) { gu[t * 2 * inter + gc] = from_f32<TIN>(0.f); gu[t * 2 * inter + uc] = from_f32<TIN>(0.f); }
    }
}

// dtype codes: 0 = float32, 1 = bfloat16; the input may be float32 with a bfloat16 output.
TFF_API int tff_swiglu(void* gu, int in_dt, void* out, int out_dt, int rows, int inter, int block, int clear,
                       cudaStream_t stream) {
    if (rows <= 0) return TFF_OK;
    if (inter <= 0 || block < 0 || (block > 0 && inter % block != 0)) return TFF_ERR_BAD_ARGUMENT;
    const long long total = (long long)rows * inter;
    const int nt = 256;
    const long long most = sm_count() * 16;
    const int blocks = (int)((total + nt - 1) / nt < most ? (total + nt - 1) / nt : most);
    if (in_dt == 1 && out_dt == 1) return tff_launch_pdl(swiglu_kernel<bf16, bf16>, blocks, nt, 0, stream, (bf16*)gu, (bf16*)out, total, inter, block, clear);
    if (in_dt == 0 && out_dt == 1) return tff_launch_pdl(swiglu_kernel<float, bf16>, blocks, nt, 0, stream, (float*)gu, (bf16*)out, total, inter, block, clear);
    if (in_dt == 0 && out_dt == 0) return tff_launch_pdl(swiglu_kernel<float, float>, blocks, nt, 0, stream, (float*)gu, (float*)out, total, inter, block, clear);
    return TFF_ERR_BAD_ARGUMENT;
}

// ------------------------------------------------------------- rotary table
// table[p][i] = (cos, sin)(float(p) * inv_freq[i]), i < rot_dim/2; the angle is one
// float32 product.  Same table as src/kernel/cuda/rope_table.cu:10-40, whose
// frequencies are exp(-(2i/d) * ln(base)); here they arrive as an array.
__global__ void rope_table_kernel(float2* __restrict__ table, const float* __restrict__ inv_freq,
                                  int max_pos, int half) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)max_pos * half) return;
    const int p = (int)(idx / half), i = (int)(idx % half);
    const float angle = (float)p * inv_freq[i];
    float s, c;
    sincosf(angle, &s, &c);
    table[idx] = make_float2(c, s);
}

TFF_API int tff_rope_table(float* table, const float* inv_freq, int max_pos, int rot_dim, cudaStream_t stream) {
    if (max_pos <= 0 || rot_dim <= 0 || (rot_dim & 1)) return TFF_ERR_BAD_ARGUMENT;
    const int half = rot_dim / 2;
    const long long total = (long long)max_pos * half;
    rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>((float2*)table, inv_freq, max_pos, half);
    return tff_launch_status();
}

// ------------------------------- q/k RMSNorm + RoPE + paged K/V write (fused)
// One warp per (token, head of [q heads | k heads | v heads]) of the projection row
// qkv[t] = [q (nq*d) | k (nkv*d) | v (nkv*d)], which may be float32 (the projection's
// accumulators, unrounded) or the activation type.
//   q head: normalise over d with q_w (if given), rotate, write to q_out[t, head];
//   k head: normalise with k_w (if given), rotate, write to the K page of the token;
//   v head: copy to the V page.
// Per-head norm before RoPE: src/core/model/qwen3/QWen3Creator.cpp:93-101; rotate-half
// pairing (i, i + rot/2): src/kernel/cuda/paged_flash_attention.cu:300-384; cache write:
// src/kernel/cuda/set_row.cu:72-123.  Unlike the reference, keys are stored rotated.
template <typename TIN, typename T>
__global__ void qk_norm_rope_kv_write_kernel(
    TIN* __restrict__ qkv, int clear_input, T* __restrict__ q_out,
    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const float2* __restrict__ table, int rot_dim,
    const int* __restrict__ positions, const int* __restrict__ tok_req,
    const int* __restrict__ block_table, int table_width,
    T* __restrict__ cache, KvLayout L, int layer, int write_cache,
    int nq, int nkv, int d, int max_pos) {
    pdl_launch_dependents();          // the next kernel may become resident (it waits before it reads or writes)
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    const int head = blockIdx.x * (blockDim.x >> 5) + warp;
    const int heads = nq + 2 * nkv;
    if (head >= heads) return;
    const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
    TIN* src = qkv + (size_t)t * heads * d + (size_t)head * d;
    if (!is_q && !write_cache) {
        if (clear_input) for (int i = lane; i < d; i += 32) src[i] = from_f32<TIN>(0.f);
        return;
    }
    const int pos = positions[t];

    T* dst;
    if (is_q) {
        dst = q_out + (size_t)t * nq * d + (size_t)head * d;
    } else {
        const int kvh = is_k ? head - nq : head - nq - nkv;
        const int b = tok_req[t];
        const int page = block_table[(size_t)b * table_width + pos / L.page_size];
        if (page < 0) {                       // no page: the host never schedules this; write nothing
            if (clear_input) for (int i = lane; i < d; i += 32) src[i] = from_f32<TIN>(0.f);
            return;
        }
        dst = cache + (size_t)page * L.page_stride + (size_t)layer * L.layer_stride +
              (is_k ? 0 : L.kv_stride) + (size_t)kvh * L.head_stride + (size_t)(pos % L.page_size) * d;
    }
    if (!is_q && !is_k) {                     // V: plain copy
        for (int i = lane; i < d; i += 32) {
            dst[i] = from_f32<T>(to_f32<TIN>(src[i]));
            if (clear_input) src[i] = from_f32<TIN>(0.f);
        }
        return;
    }
    const float* w = is_q ? q_w : k_w;
    float rs = 1.f;
    if (w) {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) { const float v = to_f32<TIN>(src[i]); ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        rs = rsqrtf(ss / (float)d + eps);
    }
    const int half = rot_dim >> 1;
    const bool rotate = table != nullptr && half > 0 && pos >= 0 && pos < max_pos;
    // pairs (i, i + half), i < half; then the unrotated tail [rot_dim, d)
    for (int i = lane; i < half; i += 32) {
        float a = to_f32<TIN>(src[i]), b2 = to_f32<TIN>(src[i + half]);
        if (w) { a = (a * rs) * w[i]; b2 = (b2 * rs) * w[i + half]; }
        float ra = a, rb = b2;
        if (rotate) {
            const float2 cs = table[(size_t)pos * half + i];
            ra = a * cs.x - b2 * cs.y;
            rb = a * cs.y + b2 * cs.x;
        }
        dst[i] = from_f32<T>(ra);
        dst[i + half] = from_f32<T>(rb);
    }
    for (int i = 2 * half + lane; i < d; i += 32) {
        float a = to_f32<TIN>(src[i]);
        if (w) a = (a * rs) * w[i];
        dst[i] = from_f32<T>(a);
    }
    if (clear_input) {
        // every lane has read what it needs of the row (the stores above follow the loads in program
        // order, and a lane only ever reads the elements it clears or their rotation partners, which it
        // has already consumed): the accumulator row goes back to zero for the next split product
        __syncwarp();
        for (int i = lane; i < d; i += 32) src[i] = from_f32<TIN>(0.f);
    }
}

// in_is_f32: the projection row is float32 (else it has the activation type given by is_bf16).
// The same for head size 128 with the whole head rotated (the common case): a lane owns four
// consecutive elements (one 16-byte load of float32 accumulators), its rotation partner is lane ^ 16.
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_rope_kv_write_d128_kernel(
    float* __restrict__ qkv, int clear_input, T* __restrict__ q_out,
    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const float2* __restrict__ table,
    const int* __restrict__ positions, const int* __restrict__ tok_req,
    const int* __restrict__ block_table, int table_width,
    T* __restrict__ cache, KvLayout L, int layer, int write_cache, int nq, int nkv, int max_pos) {
    pdl_launch_dependents();
    // Everything but the projection row is older than the kernel ahead (the step's batch arrays, the block
    // table, the norm weights, the rotation table): it is fetched first, the wait comes just before the row.
    constexpr int d = 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    const int head = blockIdx.x * 8 + warp;
    const int heads = nq + 2 * nkv;
    if (head >= heads) return;
    const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
    float* src = qkv + (size_t)t * heads * d + (size_t)head * d + lane * 4;
    const bool wanted = is_q || write_cache;
    const int pos = wanted ? positions[t] : 0;
    T* dst = nullptr;
    if (is_q) {
        dst = q_out + (size_t)t * nq * d + (size_t)head * d + lane * 4;
    } else if (wanted) {
        const int kvh = is_k ? head - nq : head - nq - nkv;
        const int page = block_table[(size_t)tok_req[t] * table_width + pos / L.page_size];
        if (page >= 0)
            dst = cache + (size_t)page * L.page_stride + (size_t)layer * L.layer_stride +
                  (is_k ? 0 : L.kv_stride) + (size_t)kvh * L.head_stride + (size_t)(pos % L.page_size) * d + lane * 4;
    }
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    float4 wv = make_float4(1.f, 1.f, 1.f, 1.f);
    if (w) wv = *reinterpret_cast<const float4*>(w + lane * 4);
    const bool rotate = (is_q || is_k) && table != nullptr && pos >= 0 && pos < max_pos;
    float4 c01 = make_float4(1.f, 0.f, 1.f, 0.f), c23 = c01;
    if (rotate) {
        const float4* cs = reinterpret_cast<const float4*>(table + (size_t)pos * 64 + (lane & 15) * 4);
        c01 = cs[0]; c23 = cs[1];                               // (cos0, sin0, cos1, sin1), (cos2, sin2, cos3, sin3)
    }
    pdl_wait();
    const float4 x = *reinterpret_cast<const float4*>(src);
    if (clear_input) *reinterpret_cast<float4*>(src) = make_float4(0.f, 0.f, 0.f, 0.f);   // this lane alone reads these four
    if (dst == nullptr) return;
    if (!is_q && !is_k) { store4<T>(dst, x.x, x.y, x.z, x.w); return; }
    float n0 = x.x, n1 = x.y, n2 = x.z, n3 = x.w;
    if (w) {
        float ss = fmaf(x.x, x.x, fmaf(x.y, x.y, fmaf(x.z, x.z, x.w * x.w)));
        ss = warp_sum(ss);
        const float rs = rsqrtf(ss / (float)d + eps);
        n0 = (x.x * rs) * wv.x; n1 = (x.y * rs) * wv.y; n2 = (x.z * rs) * wv.z; n3 = (x.w * rs) * wv.w;
    }
    if (rotate) {
        const float p0 = __shfl_xor_sync(0xffffffffu, n0, 16), p1 = __shfl_xor_sync(0xffffffffu, n1, 16);
        const float p2 = __shfl_xor_sync(0xffffffffu, n2, 16), p3 = __shfl_xor_sync(0xffffffffu, n3, 16);
        if (lane < 16) {                                        // first half: a cos - b sin, b = partner
            n0 = n0 * c01.x - p0 * c01.y; n1 = n1 * c01.z - p1 * c01.w;
            n2 = n2 * c23.x - p2 * c23.y; n3 = n3 * c23.z - p3 * c23.w;
        } else {                                                // second half: a sin + b cos, a = partner
            n0 = p0 * c01.y + n0 * c01.x; n1 = p1 * c01.w + n1 * c01.z;
            n2 = p2 * c23.y + n2 * c23.x; n3 = p3 * c23.w + n3 * c23.z;
        }
    }
    store4<T>(dst, n0, n1, n2, n3);
}

// clear_input != 0: the projection row is set to zero once it has been read.
TFF_API int tff_qk_norm_rope_kv_write(
    void* qkv, int in_is_f32, int clear_input, void* q_out, int is_bf16, const float* q_w, const float* k_w, float eps,
    const float* table, int rot_dim, int max_pos,
    const int* positions, const int* tok_req, const int* block_table, int table_width,
    void* cache, int cache_layers, int layer, int page_size, int write_cache,
    int num_tokens, int nq, int nkv, int d, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || rot_dim < 0 || rot_dim > d || (rot_dim & 1)) return TFF_ERR_BAD_ARGUMENT;
    if (write_cache && (cache == nullptr || block_table == nullptr || page_size <= 0)) return TFF_ERR_BAD_ARGUMENT;
    const KvLayout L = make_kv_layout(cache_layers, nkv, page_size > 0 ? page_size : 1, d);
    const int heads = nq + 2 * nkv;
    if (d == 128 && in_is_f32 && (table == nullptr || rot_dim == 128) && ((uintptr_t)qkv & 15) == 0 &&
        ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)cache & 15) == 0) {
        dim3 grid8((heads + 7) / 8, num_tokens);
        if (is_bf16)
            return tff_launch_pdl(qk_norm_rope_kv_write_d128_kernel<bf16>, grid8, dim3(256), 0, stream, (float*)qkv,
                                  clear_input, (bf16*)q_out, q_w, k_w, eps, (const float2*)table, positions, tok_req,
                                  block_table, table_width, (bf16*)cache, L, layer, write_cache, nq, nkv, max_pos);
        return tff_launch_pdl(qk_norm_rope_kv_write_d128_kernel<float>, grid8, dim3(256), 0, stream, (float*)qkv,
                              clear_input, (float*)q_out, q_w, k_w, eps, (const float2*)table, positions, tok_req,
                              block_table, table_width, (float*)cache, L, layer, write_cache, nq, nkv, max_pos);
    }
    const int warps = 4;
    dim3 grid((heads + warps - 1) / warps, num_tokens);
#define TFF_QK_LAUNCH(TIN, T)                                                                                  \
    tff_launch_pdl(qk_norm_rope_kv_write_kernel<TIN, T>, grid, warps * 32, 0, stream,                          \
        (TIN*)qkv, clear_input, (T*)q_out, q_w, k_w, eps, (const float2*)table, rot_dim, positions, tok_req,          \
        block_table, table_width, (T*)cache, L, layer, write_cache, nq, nkv, d, max_pos)
    if (is_bf16) {
        if (in_is_f32) return TFF_QK_LAUNCH(float, bf16);
        return TFF_QK_LAUNCH(bf16, bf16);
    }
    return TFF_QK_LAUNCH(float, float);
#undef TFF_QK_LAUNCH
}

// --------------------------------------------------------------------- zero fill
// Clears a float32 buffer that a following product adds its partial sums to.  A kernel of
// this library rather than a memset, so that the dependent-launch chain is not broken.
__global__ void zero_f32_kernel(float4* __restrict__ p4, float* __restrict__ tail, long long n4, int ntail) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x)
        p4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (blockIdx.x == 0 && (int)threadIdx.x < ntail) tail[threadIdx.x] = 0.f;
}

TFF_API int tff_zero_f32(float* p, long long n, cudaStream_t stream) {
    if (n <= 0) return TFF_OK;
    if ((uintptr_t)p & 15) return TFF_ERR_BAD_ARGUMENT;
    const long long n4 = n / 4;
    const int ntail = (int)(n - n4 * 4);
    long long blocks = (n4 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    return tff_launch_pdl(zero_f32_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (float4*)p, p + n4 * 4, n4, ntail);
}

// ------------------------------------------------------------ token hand-over
// token_ids[i] = drawn[src[i]] where src[i] >= 0: the tokens a step drew go into the next step's
// batch on the device, without a round trip through the host.
__global__ void gather_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ drawn,
                                     const int* __restrict__ src, int n, int num_drawn) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int s = src[i];
    if (s >= 0 && s < num_drawn) token_ids[i] = drawn[s];
}

TFF_API int tff_gather_tokens(int* token_ids, const int* drawn, const int* src, int n, int num_drawn, cudaStream_t stream) {
    if (n <= 0) return TFF_OK;
    return tff_launch_pdl(gather_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, token_ids, drawn, src, n, num_drawn);
}

// ------------------------------------------------------------ state slots
// Fixed-size per-request state starts from zero: every request of the step whose first token of this
// step is at position 0 (a new request, or one that is recomputed after it gave way) has its slot
// cleared before the layers run.  On the device and part of the step, so that it happens wherever a
// step is launched from (and inside a replayed CUDA graph), not at some host-side admission call.
// state: [slots, slot_bytes] bytes; one CTA row per request.
__global__ void reset_state_slots_kernel(unsigned char* __restrict__ state, long long slot_bytes, int num_slots,
                                         const int* __restrict__ slots, const int* __restrict__ pos_start) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    if (pos_start[b] != 0) return;
    const int slot = slots[b];
    if (slot < 0 || slot >= num_slots) return;
    unsigned char* p = state + (long long)slot * slot_bytes;
    const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x, step = (long long)gridDim.x * blockDim.x;
    if (((uintptr_t)p & 15) == 0 && (slot_bytes & 15) == 0) {
        uint4* p4 = reinterpret_cast<uint4*>(p);
        for (long long i = i0; i < (slot_bytes >> 4); i += step) p4[i] = make_uint4(0u, 0u, 0u, 0u);
    } else {
        for (long long i = i0; i < slot_bytes; i += step) p[i] = 0;
    }
}

TFF_API int tff_reset_state_slots(void* state, long long slot_bytes, int num_slots, const int* slots,
                                  const int* pos_start, int num_requests, cudaStream_t stream) {
    if (num_requests <= 0 || slot_bytes <= 0) return TFF_OK;
    if (!state || !slots || !pos_start || num_slots <= 0 || num_requests > 65535) return TFF_ERR_BAD_ARGUMENT;
    long long chunks = (slot_bytes / 16 + 255) / 256;
    if (chunks < 1) chunks = 1;
    if (chunks > 64) chunks = 64;
    return tff_launch_pdl(reset_state_slots_kernel, dim3((unsigned)chunks, (unsigned)num_requests), dim3(256), 0, stream,
                          (unsigned char*)state, slot_bytes, num_slots, slots, pos_start);
}

// ------------------------------------------------------------ logit transform
// logits = softcap > 0 ? softcap * tanh(logits * scale / softcap) : logits * scale, in place, float32.
// Not launched for this architecture (scale 1, no cap); a description that sets either gets it after the
// output projection.
__global__ void logit_transform_kernel(float* __restrict__ logits, long long n, float scale, float softcap) {
    pdl_launch_dependents();
    pdl_wait();
    const float inv = softcap > 0.f ? 1.f / softcap : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = logits[i] * scale;
        if (softcap > 0.f) v = softcap * tanhf(v * inv);
        logits[i] = v;
    }
}

TFF_API int tff_logit_transform(float* logits, long long n, float scale, float softcap, cudaStream_t stream) {
    if (n <= 0) return TFF_OK;
    if (!logits || softcap < 0.f) return TFF_ERR_BAD_ARGUMENT;
    long long blocks = (n + 255) / 256;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    return tff_launch_pdl(logit_transform_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, logits, n, scale, softcap);
}
