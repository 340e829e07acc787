// bfloat16 matrix product on the 5th-generation tensor cores:
//   out[M, N] = A[M, K] * W[N, K]^T  (+ residual), float32 accumulation in tensor memory.
//
// A persistent kernel: each CTA walks a list of segments, a segment being a range of
// 64-element K blocks of one 128 x BN accumulator tile.  Both operands are K-major
// ([rows, K] row-major) and come to shared memory by TMA in 128-byte-swizzled tiles;
// tcgen05.mma (M = 128, N = BN, K = 16), issued by one thread, accumulates in TMEM; two
// accumulator buffers alternate, so the epilogue of one segment overlaps the mainloop of
// the next.
//   warp 0      TMA producer       (one lane)
//   warp 1      TMEM allocation, MMA issue (one lane), TMEM release
//   warps 2-5   epilogue: TMEM -> registers -> (shared memory -> TMA store | global memory)
// Two orientations share the kernel:
//   normal   the 128-row operand is the activations (M on TMEM lanes), the BN-row operand
//            the weights; for prompt portions.  Tiles go round-robin over the CTAs, rows of
//            tiles fastest, so that CTAs running together share a weight tile in L2.  The
//            epilogue stages 32-row slabs in swizzled shared memory and writes them with
//            TMA stores (TMA float32 add-reductions when the product is added to ``out``).
//   swapped  the 128-row operand is the weights (N on TMEM lanes), the BN-row operand the
//            activations, BN = M rounded up to 16; for decode-sized M, where the product is
//            one pass of the weights through the SMs.  With few tiles the (tile, K block)
//            units are dealt to the CTAs in equal contiguous shares ("stream-K"), every CTA
//            streaming the same number of bytes; partial tiles meet in float32 atomics.
// It replaces the reference's int8 dp4a product (src/kernel/cuda/quant/quant_q_8_0_mat_mul.cu:338-447)
// and its unfinished dense product (src/kernel/cuda/mat_mul.cu:151-660) on the serving path.
//
// Every wait on an mbarrier is bounded; when one runs out the CTA raises a flag in global
// memory, stops issuing work, lets its copies in flight land, frees its tensor memory and
// returns.
#include <type_traits>
#include "gemm_epilogue.cuh"
#include "gemm_tc_pair.h"

namespace {

using namespace tc5;

template <int BN, bool TMA_OUT, bool SWAP = false> struct TileCfg {
    static constexpr int kStageBytes = BM * BK * 2 + BN * BK * 2;
    // Small column tiles stream weights: several CTAs on an SM keep more loads in flight than one CTA with a
    // deep ring (measured: one CTA of 8 stages reads 4.5 TB/s at 64 tokens, two of 3 stages 4.8).  Stages are
    // as many as let kCtasPerSm CTAs fit into the SM's 227 KB with their staging (2 x 5 stages of BN = 32
    // did not: only one CTA was resident and the 296-CTA grid ran as two waves).
    static constexpr int kStages = BN >= 256 ? 4 : BN >= 128 ? 5 : (BN >= 64 ? 3 : 4);
    static constexpr int kCtasPerSm = BN >= 128 ? 1 : (BN >= 32 ? 2 : 3);
    static constexpr int kAccCols = BN < 32 ? 32 : BN;              // columns of one accumulator buffer
    static constexpr int kTmemCols = 2 * kAccCols;                  // 64 .. 512, a power of two
    // epilogue staging: 4 warps x (32 rows x 128 B); two buffers a warp in the normal orientation, one when swapped
    static constexpr int kStagingBytes = TMA_OUT ? (SWAP ? 4 * 4096 : 4 * 2 * 4096) : 0;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
    // an SM has 228 KB of shared memory, of which each resident CTA reserves 1 KB; checked for the
    // configurations that the decode steps launch (swapped; through TMA from BN = 32 on)
    static_assert(!SWAP || TMA_OUT != (BN >= 32) || kCtasPerSm * (kSmemBytes + 1024) <= 228 * 1024,
                  "the CTAs meant to share an SM do not fit");
};

// out element (m, n): normal -> lane operand row = m, column operand row = n; swapped -> the reverse.
// TMA_OUT: the epilogue goes through shared memory and TMA (stores, or float32 add-reductions).
template <int BN, bool SWAP, int EPI, typename TC, bool TMA_OUT>
__global__ void __launch_bounds__(NUM_THREADS, TileCfg<BN, TMA_OUT, SWAP>::kCtasPerSm)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_lane,   // operand whose rows land on TMEM lanes (box 64 x 128)
               const __grid_constant__ CUtensorMap tm_col,    // operand whose rows land on TMEM columns (box 64 x BN)
               const __grid_constant__ CUtensorMap tm_out,    // output, boxes of 128 bytes x 32 rows (TMA_OUT only)
               TC* __restrict__ out, int rows_lane, int rows_col, int K, int ldo, int stream_k, int* error_flag) {
    using Cfg = TileCfg<BN, TMA_OUT, SWAP>;
    using SegIter = typename std::conditional<SWAP, SegIterShares, SegIterSlices>::type;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t staging = base + STAGES * Cfg::kStageBytes;          // 1024-aligned (stage sizes are multiples of 1024)
    const uint32_t bars = staging + Cfg::kStagingBytes;
    // barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then the TMEM address word and the abort flag
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot =
        (volatile uint32_t*)(gen_base + STAGES * Cfg::kStageBytes + Cfg::kStagingBytes + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kbt = (K + BK - 1) / BK;
    const int n_lane_tiles = (rows_lane + BM - 1) / BM;
    const int n_col_tiles = (rows_col + BN - 1) / BN;
    const int n_tiles = n_lane_tiles * n_col_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_lane) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_col) : "memory");
        if (TMA_OUT) asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_out) : "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------------ TMA producer
            // The weights do not depend on the kernel before this one: the weight tiles of
            // the first ring of stages are requested before waiting for it, the activations
            // after.
            const CUtensorMap* tm_w = SWAP ? &tm_lane : &tm_col;
            const CUtensorMap* tm_x = SWAP ? &tm_col : &tm_lane;
            const uint32_t w_off = SWAP ? 0u : (uint32_t)(BM * BK * 2);
            const uint32_t x_off = SWAP ? (uint32_t)(BM * BK * 2) : 0u;
            int pre_k[STAGES], pre_wrow[STAGES], pre_xrow[STAGES];
            int pre = 0;
            {
                SegIter it(n_tiles, kbt, stream_k, blockIdx.x, gridDim.x);
                while (pre < STAGES && it.next()) {
                    const int lrow = (it.tile % n_lane_tiles) * BM, crow = (it.tile / n_lane_tiles) * BN;
                    for (int kb = it.kb0; kb < it.kb1 && pre < STAGES; ++kb, ++pre) {
                        pre_k[pre] = kb * BK;
                        pre_wrow[pre] = SWAP ? lrow : crow;
                        pre_xrow[pre] = SWAP ? crow : lrow;
                    }
                }
            }
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(full_bar(i), Cfg::kStageBytes);
                tma_load_2d(base + i * Cfg::kStageBytes + w_off, tm_w, full_bar(i), pre_k[i], pre_wrow[i]);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i)
                tma_load_2d(base + i * Cfg::kStageBytes + x_off, tm_x, full_bar(i), pre_k[i], pre_xrow[i]);
            SegIter it(n_tiles, kbt, stream_k, blockIdx.x, gridDim.x);
            uint32_t n = 0;
            bool ok = true;
            while (ok && it.next()) {
                const int lrow = (it.tile % n_lane_tiles) * BM, crow = (it.tile / n_lane_tiles) * BN;
                for (int kb = it.kb0; kb < it.kb1; ++kb, ++n) {
                    if (n < (uint32_t)pre) continue;                 // already requested above
                    const int s = n % STAGES;
                    const uint32_t round = n / STAGES;
                    if (!mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag)) { ok = false; break; }
                    const uint32_t a_dst = base + s * Cfg::kStageBytes;
                    mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
                    tma_load_2d(a_dst, &tm_lane, full_bar(s), kb * BK, lrow);
                    tma_load_2d(a_dst + BM * BK * 2, &tm_col, full_bar(s), kb * BK, crow);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // -------------------------------------------------------- MMA issuer
            constexpr uint32_t idesc = make_idesc(BM, BN);
            SegIter it(n_tiles, kbt, stream_k, blockIdx.x, gridDim.x);
            uint32_t n = 0, seg = 0;
            bool ok = true;
            while (ok && it.next()) {
                const uint32_t acc = seg & 1, use = seg >> 1;
                if (use > 0 && !mbar_wait(tempty_bar(acc), (use - 1) & 1, abort_flag)) break;   // epilogue has drained it
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * Cfg::kAccCols;
                for (int kb = it.kb0; kb < it.kb1; ++kb, ++n) {
                    const int s = n % STAGES;
                    const uint32_t round = n / STAGES;
                    if (!mbar_wait(full_bar(s), round & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = base + s * Cfg::kStageBytes;
                    const uint64_t adesc = make_smem_desc(a_addr);
                    const uint64_t bdesc = make_smem_desc(a_addr + BM * BK * 2);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // 16 K-elements = 32 bytes = 2 descriptor units further along the swizzled row
                        umma_bf16(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                                  (kb > it.kb0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));          // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(tfull_bar(acc));    // this segment's accumulators are complete
                ++seg;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                     // TMEM lane quarter this warp may read
        pdl_wait();                                 // nothing is written before the kernel ahead has finished
        SegIter it(n_tiles, kbt, stream_k, blockIdx.x, gridDim.x);
        uint32_t seg = 0, chunk_no = 0;
        while (it.next()) {
            const uint32_t acc = seg & 1, use = seg >> 1;
            if (!mbar_wait(tfull_bar(acc), use & 1, abort_flag)) break;
            tc_fence_after();
            const int lane_row0 = (it.tile % n_lane_tiles) * BM, col_row0 = (it.tile / n_lane_tiles) * BN;
            const uint32_t t_addr = tmem_base + acc * Cfg::kAccCols + ((uint32_t)(q * 32) << 16);
            const bool partial = stream_k && (it.kb1 - it.kb0) < kbt;   // a share of the tile's K range: add
            if constexpr (TMA_OUT && SWAP) {
                // Swapped orientation, float32 out: the thread holds feature n = its TMEM lane for 16 tokens at a
                // time.  A warp stages a box of 32 tokens x 32 features (one 128-byte row per token, written by the
                // 32 lanes side by side, 16-byte chunks XOR-swizzled by token % 8) and one lane hands it to TMA:
                // a store, or an add-reduction done in L2 when the product is added to ``out``.
                const uint32_t buf = staging + (uint32_t)(warp - 2) * 4096u;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (lane == 0) bulk_wait_read<0>();        // the box staged before this one has been read
                    __syncwarp();
#pragma unroll
                    for (int h = 0; h < (BN >= 32 ? 2 : 1); ++h) {
                        uint32_t v[16];
                        tmem_ld16(t_addr + (uint32_t)(c0 + h * 16), v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int m = h * 16 + j;              // token row of the box
                            const uint32_t dst = buf + (uint32_t)m * 128u + (uint32_t)((((lane >> 2) ^ (m & 7)) << 4) + ((lane & 3) << 2));
                            asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst), "r"(v[j]) : "memory");
                        }
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        // rows of the box beyond M are clipped by TMA (with BN = 16 the box's upper half is never written)
                        if (EPI == EPI_ADD || partial) tma_reduce_add_2d(&tm_out, buf, lane_row0 + q * 32, col_row0 + c0);
                        else tma_store_2d(&tm_out, buf, lane_row0 + q * 32, col_row0 + c0);
                        bulk_commit();
                    }
                }
            } else if constexpr (TMA_OUT) {
                epilogue_quarter_tma<BN, EPI, TC>(t_addr, staging + (uint32_t)((warp - 2) * 2) * 4096u, chunk_no, lane, q,
                                                  lane_row0, col_row0, partial, &tm_out);
            } else {
                const int lr = lane_row0 + q * 32 + lane;          // row of the lane operand
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(t_addr + (uint32_t)c0, v);
                    tmem_ld_wait();
                    if (lr >= rows_lane) continue;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int cr = col_row0 + c0 + j;
                        if (cr < rows_col) {
                            const float x = __uint_as_float(v[j]);
                            // normal: out[lr, cr]; swapped: out[cr, lr] (a warp then writes 32 consecutive n)
                            const size_t idx = SWAP ? (size_t)cr * ldo + lr : (size_t)lr * ldo + cr;
                            if constexpr (sizeof(TC) == 4) {
                                if (EPI == EPI_ADD || partial) atomicAdd(reinterpret_cast<float*>(&out[idx]), x);
                                else out[idx] = from_f32<TC>(x);
                            } else {
                                out[idx] = from_f32<TC>(x);
                            }
                        }
                    }
                }
            }
            // the accumulator buffer may be overwritten
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            ++seg;
        }
        if (TMA_OUT && lane == 0) bulk_wait_read<0>();       // staged rows must have been read before the CTA leaves
    }
    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give copies still in flight time to land in this CTA's shared memory before it is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ------------------------------------------------------------------- host side
template <int BN, bool SWAP, int EPI, typename TC, bool TMA_OUT>
int launch_tc(const CUtensorMap& tl, const CUtensorMap& tc, const CUtensorMap& to, void* out,
              int rows_lane, int rows_col, int K, int ldo, int stream_k, cudaStream_t stream) {
    using Cfg = TileCfg<BN, TMA_OUT, SWAP>;
    auto kern = gemm_tc_kernel<BN, SWAP, EPI, TC, TMA_OUT>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
            return TFF_ERR_LAUNCH;
        configured = true;
    }
    const long long n_tiles = (long long)((rows_lane + BM - 1) / BM) * ((rows_col + BN - 1) / BN);
    const long long units = stream_k ? n_tiles * ((K + BK - 1) / BK) : n_tiles;
    long long ctas = (long long)tff_num_sms() * Cfg::kCtasPerSm;
    // Products of a decode layer follow one another with a small kernel in between, and a CTA of the product
    // after next can only become resident -- and ask for its first ring of weight tiles before it waits for its
    // predecessor -- where an SM has room.  A grid that fills every CTA slot leaves none: the next product then
    // starts from empty rings when this one has drained.  The 16-column configuration therefore leaves about a
    // twelfth of its slots free (measured at the Qwen3-8B shape, 8 requests: 3.66 ms a step with 2.75 CTAs an SM,
    // 3.72 with 2.6, 3.85 with all 3).  The output projection alone is one long kernel and takes every slot.
    // (Asking the L2 for the successor's first weight tiles from this product's producers, once they have asked
    // for their own last tile, was measured too: 0.17 ms a step slower -- the prefetches delay the tail they
    // were meant to use.)
    if (SWAP && BN == 16 && rows_lane < 65536) ctas = tff_decode_gemm_ctas(units);
    if (ctas <= 0) return TFF_ERR_LAUNCH;
    if (ctas > units) ctas = units;
    return tff_launch_pdl(kern, dim3((unsigned)ctas), dim3(NUM_THREADS), (size_t)Cfg::kSmemBytes, stream, tl, tc, to,
                          (TC*)out, rows_lane, rows_col, K, ldo, stream_k, tff_device_error_flag());
}

template <int BN, bool SWAP, bool TMA_OUT>
int dispatch_epi(const CUtensorMap& tl, const CUtensorMap& tc, const CUtensorMap& to, void* out, int out_is_bf16,
                 int add, int rows_lane, int rows_col, int K, int ldo, int stream_k, cudaStream_t s) {
    if (out_is_bf16) {
        if (add || stream_k) return TFF_ERR_BAD_ARGUMENT;
        return launch_tc<BN, SWAP, EPI_STORE, bf16, TMA_OUT>(tl, tc, to, out, rows_lane, rows_col, K, ldo, 0, s);
    }
    if (add) return launch_tc<BN, SWAP, EPI_ADD, float, TMA_OUT>(tl, tc, to, out, rows_lane, rows_col, K, ldo, stream_k, s);
    return launch_tc<BN, SWAP, EPI_STORE, float, TMA_OUT>(tl, tc, to, out, rows_lane, rows_col, K, ldo, stream_k, s);
}

}  // namespace

// out[M, N] (+)= A[M, K] * W[N, K]^T; A, W bfloat16.
//   swap      0: A rows on TMEM lanes (tiles 128 x bn over M x N); 1: W rows on lanes (tiles 128 x bn over N x M)
//   bn        16, 32, 64, 128 or 256; 512 (normal orientation): 256 x 256 tiles on pairs of SMs
//   add       1: the product is added to what ``out`` (float32) holds -- a residual stream in place
//   stream_k  1: (tile, K block) units are dealt in equal shares; S >= 2: the tiles of the last, partial wave
//             are cut into S slices of their K range; tiles that are split between CTAs
//             are accumulated with float32 adds, so ``out`` (float32) must hold the initial value
//             (zero, or the residual with add = 1) before the call
TFF_API int tff_gemm_tc(const void* A, const void* W, void* out, int out_is_bf16, int add,
                        int M, int N, int K, int swap, int bn, int stream_k, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return TFF_OK;
    if (K <= 0 || ((add || stream_k) && out_is_bf16)) return TFF_ERR_BAD_ARGUMENT;
    if (K % 8 != 0) return TFF_ERR_UNSUPPORTED;                         // TMA row pitch must be a multiple of 16 bytes
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return TFF_ERR_UNSUPPORTED;
    if (tff_device_error_flag() == nullptr) return TFF_ERR_LAUNCH;
    if (bn == 512) {
        // pairs of SMs: the output must suit TMA (row pitch a multiple of 16 bytes, aligned base); else single CTAs
        const int elt = out_is_bf16 ? 2 : 4;
        if (!swap && ((long long)N * elt) % 16 == 0 && ((uintptr_t)out & 15) == 0) {
            CUtensorMap ta, tw, to2;
            if (!tff_tensor_map_2d(A, M, K, BM, BK, 2, &ta)) return TFF_ERR_DRIVER;
            if (!tff_tensor_map_2d(W, N, K, 128, BK, 2, &tw)) return TFF_ERR_DRIVER;
            if (!tff_tensor_map_2d(out, M, N, 32, 128 / elt, elt, &to2)) return TFF_ERR_DRIVER;
            return tff_gemm_tc_pair_launch(ta, tw, to2, add ? EPI_ADD : EPI_STORE, out_is_bf16, M, N, K, stream_k, stream);
        }
        bn = 256;
    }
    const void* lane_ptr = swap ? W : A;
    const void* col_ptr = swap ? A : W;
    const int rows_lane = swap ? N : M, rows_col = swap ? M : N;
    CUtensorMap tl, tc, to;
    if (!tff_tensor_map_2d(lane_ptr, rows_lane, K, BM, BK, 2, &tl)) return TFF_ERR_DRIVER;
    if (!tff_tensor_map_2d(col_ptr, rows_col, K, bn, BK, 2, &tc)) return TFF_ERR_DRIVER;
    // TMA output: row pitch a multiple of 16 bytes, 16-byte aligned base
    const int elt = out_is_bf16 ? 2 : 4;
    // (swapped: float32 only, boxes of 32 tokens x 32 features)
    const bool tma_out = ((long long)N * elt) % 16 == 0 && ((uintptr_t)out & 15) == 0 &&
                         (swap ? (!out_is_bf16 && bn >= 32) : bn >= 128 / elt);
    to = tl;
    if (tma_out && !tff_tensor_map_2d(out, M, N, 32, 128 / elt, elt, &to)) return TFF_ERR_DRIVER;
#define TFF_CASE(BN_)                                                                                              \
    case BN_:                                                                                                      \
        if (swap && tma_out) return dispatch_epi<BN_, true, true>(tl, tc, to, out, out_is_bf16, add, rows_lane, rows_col, K, N, stream_k, stream); \
        if (swap) return dispatch_epi<BN_, true, false>(tl, tc, to, out, out_is_bf16, add, rows_lane, rows_col, K, N, stream_k, stream); \
        if (tma_out) return dispatch_epi<BN_, false, true>(tl, tc, to, out, out_is_bf16, add, rows_lane, rows_col, K, N, stream_k, stream); \
        return dispatch_epi<BN_, false, false>(tl, tc, to, out, out_is_bf16, add, rows_lane, rows_col, K, N, stream_k, stream);
    switch (bn) {
        TFF_CASE(16)
        TFF_CASE(32)
        TFF_CASE(64)
        TFF_CASE(128)
        TFF_CASE(256)
    }
#undef TFF_CASE
    return TFF_ERR_BAD_ARGUMENT;
}

// out[M, I] = silu(A Wg^T) * (A Wu^T), with W [2I, K] holding the gate and up rows alternating in
// blocks of 64: rows [128 b, 128 b + 64) = gate features [64 b, 64 b + 64), rows [128 b + 64, 128 b + 128)
// = the same up features.  Normal orientation only (prompt-sized M); I must be a multiple of 64.
// TFF_ERR_UNSUPPORTED for shapes it does not take.
TFF_API int tff_gemm_tc_swiglu(const void* A, const void* W, void* out, int M, int I, int K, int bn, cudaStream_t stream) {
    if (M <= 0 || I <= 0) return TFF_OK;
    if (K <= 0) return TFF_ERR_BAD_ARGUMENT;
    if (K % 8 != 0 || I % 64 != 0 || (bn != 128 && bn != 256 && bn != 512)) return TFF_ERR_UNSUPPORTED;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)out & 15)) return TFF_ERR_UNSUPPORTED;
    if (tff_device_error_flag() == nullptr) return TFF_ERR_LAUNCH;
    CUtensorMap tl, tc, to;
    if (!tff_tensor_map_2d(A, M, K, BM, BK, 2, &tl)) return TFF_ERR_DRIVER;
    if (bn == 512) {                                  // 256 x 256 tiles on pairs of SMs
        if (!tff_tensor_map_2d(W, 2ll * I, K, 128, BK, 2, &tc)) return TFF_ERR_DRIVER;
        if (!tff_tensor_map_2d(out, M, I, 32, 64, 2, &to)) return TFF_ERR_DRIVER;
        return tff_gemm_tc_pair_launch(tl, tc, to, EPI_SWIGLU, 1, M, 2 * I, K, 0, stream);
    }
    if (!tff_tensor_map_2d(W, 2ll * I, K, bn, BK, 2, &tc)) return TFF_ERR_DRIVER;
    if (!tff_tensor_map_2d(out, M, I, 32, 64, 2, &to)) return TFF_ERR_DRIVER;
    if (bn == 256) return launch_tc<256, false, EPI_SWIGLU, bf16, true>(tl, tc, to, out, M, 2 * I, K, I, 0, stream);
    return launch_tc<128, false, EPI_SWIGLU, bf16, true>(tl, tc, to, out, M, 2 * I, K, I, 0, stream);
}
