// The epilogue of a 128 x BN accumulator tile in the normal orientation (activation rows on the TMEM
// lanes) through shared memory and TMA, shared by the tcgen05 product kernels.
#pragma once
#include "tcgen05.cuh"

namespace tc5 {

// write the product | add it to what ``out`` holds | write silu(gate) * up of a product whose columns
// alternate between 64 gate and 64 up features (normal orientation, bfloat16 out, through TMA)
// EPI_QKV: the product is a q/k/v projection with heads of 128: per-head RMSNorm of q and k, rotation, q to its
// own tensor and k, v to the token's slot of the paged cache (epilogue_quarter_qkv below)
enum Epilogue : int { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2, EPI_QKV = 3 };

// One warp's quarter (32 rows) of the tile: TMEM -> registers -> two alternating 4 KB boxes of swizzled
// shared memory (``my_stage``) -> TMA stores, or float32 add-reductions when the product is added to what
// ``out`` holds or the tile is a share of its K range (``partial``).  ``t_addr``: TMEM address of the warp's
// lane quarter and the tile's first column; ``chunk_no`` counts the warp's boxes over the whole kernel.
template <int BN, int EPI, typename TC>
__device__ __forceinline__ void epilogue_quarter_tma(uint32_t t_addr, uint32_t my_stage, uint32_t& chunk_no, int lane, int q,
                                                     int lane_row0, int col_row0, bool partial, const CUtensorMap* tm_out) {
    // 128-byte-wide column chunks: 32 float32 or 64 bfloat16 per row
    constexpr int CW = 128 / (int)sizeof(TC);      // output columns per chunk
    constexpr int AW = EPI == EPI_SWIGLU ? 128 : CW;   // accumulator columns per chunk
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += AW, ++chunk_no) {
        const uint32_t buf = my_stage + (chunk_no & 1) * 4096u;
        if (chunk_no >= 2) {                       // the store that last used this buffer has read it
            if (lane == 0) bulk_wait_read<1>();
            __syncwarp();
        }
        uint32_t packed[32];                       // this thread's row: 128 bytes
        if constexpr (EPI == EPI_SWIGLU) {
            // columns [c0, c0+64) are the gate, [c0+64, c0+128) the up projection of the
            // same 64 features: silu(g) * u, silu(g) = g / (1 + exp(-g)).  The division is the fast one (the result
            // is rounded to bfloat16): the exact one takes its slow path for a numerator of zero, which is what every
            // row beyond the last token holds, and a tile with such rows took half as long again.
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                uint32_t g[16], u[16];
                tmem_ld16(t_addr + (uint32_t)(c0 + h * 16), g);
                tmem_ld16(t_addr + (uint32_t)(c0 + 64 + h * 16), u);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
                    const float a0 = __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(u[2 * j]);
                    const float a1 = __fdividef(g1, 1.0f + __expf(-g1)) * __uint_as_float(u[2 * j + 1]);
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(a0, a1);
                    packed[h * 8 + j] = *reinterpret_cast<uint32_t*>(&b2);
                }
            }
        } else {
#pragma unroll
            for (int h = 0; h < CW / 16; ++h) {
                uint32_t v[16];
                tmem_ld16(t_addr + (uint32_t)(c0 + h * 16), v);
                tmem_ld_wait();
                if constexpr (sizeof(TC) == 4) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) packed[h * 16 + j] = v[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                        packed[h * 8 + j] = *reinterpret_cast<uint32_t*>(&b2);
                    }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {              // 16-byte chunk c of row ``lane`` at chunk c ^ (lane % 8)
            const uint32_t dst = buf + (uint32_t)lane * 128u + (uint32_t)((c ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[4 * c]),
                         "r"(packed[4 * c + 1]), "r"(packed[4 * c + 2]), "r"(packed[4 * c + 3]) : "memory");
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            if (EPI == EPI_SWIGLU) tma_store_2d(tm_out, buf, (col_row0 + c0) / 2, lane_row0 + q * 32);
            else if (EPI == EPI_ADD || partial) tma_reduce_add_2d(tm_out, buf, col_row0 + c0, lane_row0 + q * 32);
            else tma_store_2d(tm_out, buf, col_row0 + c0, lane_row0 + q * 32);
            bulk_commit();
        }
    }
}


// What the q/k/v epilogue needs beside the accumulators.  Columns of the product are
// [q heads | k heads | v heads] of 128 each, rows are tokens.
struct QkvEpilogue {
    bf16* q_out;                 // [T, nq * 128]
    bf16* cache;                 // paged cache (may be null when write_cache == 0)
    const float* q_w;            // norm weights of q and k heads [128] (null: no norm)
    const float* k_w;
    const float2* table;         // (cos, sin)[max_pos][64] (null: no rotation)
    const int* positions;        // [T]
    const int* tok_req;          // [T] row of the block table
    const int* block_table;
    KvLayout L;
    float eps;
    int table_width, layer, write_cache, nq, nkv, T, max_pos;
};

__device__ __forceinline__ void store16_bf16(bf16* dst, const float* v) {
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&b2);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
}

// One warp's quarter (32 token rows) of a 128 x 256 accumulator tile = two heads of a q/k/v projection.
// A thread owns a token's row, so the sum of squares of a head and the rotation partners (i, i + 64) are
// its own: no exchange between threads.  Same arithmetic as qk_norm_rope_kv_write in elementwise.cu,
// on the unrounded float32 accumulators.  TMEM loads are executed by the whole warp, stores by the
// threads whose token exists (and whose page exists).
__device__ __forceinline__ void epilogue_quarter_qkv(uint32_t t_addr, int lane, int q, int lane_row0, int col_row0,
                                                     const QkvEpilogue& e) {
    const int t = lane_row0 + q * 32 + lane;
    const bool valid = t < e.T;
    int pos = 0, req = 0;
    if (valid) { pos = e.positions[t]; req = e.tok_req[t]; }
    const bool rotate = e.table != nullptr && pos >= 0 && pos < e.max_pos;
    const int heads = e.nq + 2 * e.nkv;
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
        const int head = col_row0 / 128 + hh;
        if (head >= heads) break;
        const bool is_q = head < e.nq, is_k = !is_q && head < e.nq + e.nkv;
        if (!is_q && !e.write_cache) continue;
        bf16* dst = nullptr;
        if (valid) {
            if (is_q) {
                dst = e.q_out + (size_t)t * e.nq * 128 + (size_t)head * 128;
            } else {
                const int kvh = is_k ? head - e.nq : head - e.nq - e.nkv;
                const int page = e.block_table[(size_t)req * e.table_width + pos / e.L.page_size];
                if (page >= 0)
                    dst = e.cache + (size_t)page * e.L.page_stride + (size_t)e.layer * e.L.layer_stride +
                          (is_k ? 0 : e.L.kv_stride) + (size_t)kvh * e.L.head_stride + (size_t)(pos % e.L.page_size) * 128;
            }
        }
        const uint32_t th = t_addr + (uint32_t)(hh * 128);
        if (!is_q && !is_k) {                          // a v head: as it is
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(th + (uint32_t)c0, v);
                tmem_ld_wait();
                float f[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(v[j]);
                if (dst) store16_bf16(dst + c0, f);
            }
            continue;
        }
        const float* w = is_q ? e.q_w : e.k_w;
        float rs = 1.f;
        if (w != nullptr) {
            float ss = 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(th + (uint32_t)c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) ss = fmaf(__uint_as_float(v[j]), __uint_as_float(v[j]), ss);
            }
            rs = rsqrtf(ss / 128.f + e.eps);
        }
#pragma unroll 1
        for (int i0 = 0; i0 < 64; i0 += 16) {
            uint32_t lo[16], hi[16];
            tmem_ld16(th + (uint32_t)i0, lo);
            tmem_ld16(th + (uint32_t)(64 + i0), hi);
            tmem_ld_wait();
            float a[16], b[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) { a[j] = __uint_as_float(lo[j]); b[j] = __uint_as_float(hi[j]); }
            if (w != nullptr) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const float4 wa = *reinterpret_cast<const float4*>(w + i0 + j);
                    const float4 wb = *reinterpret_cast<const float4*>(w + 64 + i0 + j);
                    a[j] = (a[j] * rs) * wa.x; a[j + 1] = (a[j + 1] * rs) * wa.y; a[j + 2] = (a[j + 2] * rs) * wa.z; a[j + 3] = (a[j + 3] * rs) * wa.w;
                    b[j] = (b[j] * rs) * wb.x; b[j + 1] = (b[j + 1] * rs) * wb.y; b[j + 2] = (b[j + 2] * rs) * wb.z; b[j + 3] = (b[j + 3] * rs) * wb.w;
                }
            }
            if (rotate) {
                const float4* cs = reinterpret_cast<const float4*>(e.table + (size_t)pos * 64 + i0);
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const float4 c2 = cs[j >> 1];          // (cos, sin) of elements j and j + 1
                    const float a0 = a[j], b0 = b[j], a1 = a[j + 1], b1 = b[j + 1];
                    a[j] = a0 * c2.x - b0 * c2.y;  b[j] = a0 * c2.y + b0 * c2.x;
                    a[j + 1] = a1 * c2.z - b1 * c2.w;  b[j + 1] = a1 * c2.w + b1 * c2.z;
                }
            }
            if (dst) { store16_bf16(dst + i0, a); store16_bf16(dst + 64 + i0, b); }
        }
    }
}

}  // namespace tc5
