// The epilogue of a 128 x BN accumulator tile in the normal orientation (activation rows on the TMEM
// lanes) through shared memory and TMA, shared by the tcgen05 product kernels.
#pragma once
#include "tcgen05.cuh"

namespace tc5 {

// write the product | add it to what ``out`` holds | write silu(gate) * up of a product whose columns
// alternate between 64 gate and 64 up features (normal orientation, bfloat16 out, through TMA)
enum Epilogue : int { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2 };

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
            // same 64 features: silu(g) * u, silu(g) = g / (1 + exp(-g))
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                uint32_t g[16], u[16];
                tmem_ld16(t_addr + (uint32_t)(c0 + h * 16), g);
                tmem_ld16(t_addr + (uint32_t)(c0 + 64 + h * 16), u);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
                    const float a0 = (g0 / (1.0f + __expf(-g0))) * __uint_as_float(u[2 * j]);
                    const float a1 = (g1 / (1.0f + __expf(-g1))) * __uint_as_float(u[2 * j + 1]);
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

}  // namespace tc5
