// bfloat16 matrix product on the 5th-generation tensor cores:
//   out[M, N] = A[M, K] * W[N, K]^T  (+ residual), float32 accumulation in tensor memory.
//
// One CTA computes one 128 x BN tile of accumulators.  Both operands are K-major
// ([rows, K] row-major), brought to shared memory by TMA in 128-byte-swizzled tiles
// of 64 K-elements, multiplied by tcgen05.mma (M = 128, N = BN, K = 16) issued by one
// thread, accumulated in TMEM and read back with tcgen05.ld by four epilogue warps.
//   warp 0      TMA producer       (one lane)
//   warp 1      TMEM allocation, MMA issue (one lane), TMEM release
//   warps 2-5   epilogue: TMEM -> registers -> global memory
// Two orientations share the kernel:
//   normal   the 128-row operand is the activations (M on TMEM lanes), the BN-row
//            operand the weights; used when M is large (prompt portions);
//   swapped  the 128-row operand is the weights (N on TMEM lanes), the BN-row operand
//            the activations, BN = M rounded up to 16; used for decode-sized M, where
//            the product is a stream of the weights through the SMs.  The K range may
//            be split over blockIdx.z, the partial sums then meet in float32 atomics.
// It replaces the reference's int8 dp4a product (src/kernel/cuda/quant/quant_q_8_0_mat_mul.cu:338-447)
// and its unfinished dense product (src/kernel/cuda/mat_mul.cu:151-660) on the serving path.
//
// Every wait on an mbarrier is bounded; when one runs out the CTA raises a flag in
// global memory, stops issuing work, lets its copies in flight land, frees its
// tensor memory and returns.
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace {

constexpr int BM = 128;           // rows of the lane operand per tile
constexpr int BK = 64;            // K elements per stage: 128 bytes of bf16 = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

enum Epilogue : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_ATOMIC = 2 };

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait.  Returns false when it gave up or when another role already had.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i >= 64) {
            __nanosleep(32);
            if (*abort_flag) return false;
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128
// bytes, groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1,
// layout type 2 (SWIZZLE_128B).  Addresses and offsets are in units of 16 bytes.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                           // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                           // version, bits [46,48)
    d |= (uint64_t)2 << 61;                           // layout type, bits [61,64)
    return d;
}
// Instruction descriptor of kind::f16: D = float32, A = B = bfloat16, both K-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4)                                  // c_format = F32
         | (1u << 7)                                  // a_format = BF16
         | (1u << 10)                                 // b_format = BF16
         | ((uint32_t)(n >> 3) << 17)                 // n_dim
         | ((uint32_t)(m >> 4) << 24);                // m_dim
}

template <int BN> struct TileCfg {
    static constexpr int kStageBytes = BM * BK * 2 + BN * BK * 2;
    static constexpr int kStages = BN >= 256 ? 4 : BN >= 128 ? 6 : (BN >= 64 ? 4 : 5);
    static constexpr int kCtasPerSm = BN >= 128 ? 1 : 2;
    static constexpr int kTmemCols = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// out element (m, n): normal -> lane operand row = m, column operand row = n; swapped -> the reverse.
template <int BN, bool SWAP, int EPI, typename TC>
__global__ void __launch_bounds__(NUM_THREADS, TileCfg<BN>::kCtasPerSm)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_lane,   // operand whose rows land on TMEM lanes (box 64 x 128)
               const __grid_constant__ CUtensorMap tm_col,    // operand whose rows land on TMEM columns (box 64 x BN)
               TC* __restrict__ out, const float* residual,
               int rows_lane, int rows_col, int K, int ldo, int kblocks_per_split, int* error_flag) {
    using Cfg = TileCfg<BN>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + STAGES * Cfg::kStageBytes;           // 8-byte aligned
    // barrier layout: full[STAGES], empty[STAGES], tmem_full, then the TMEM address word and the abort flag
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t tmem_full_bar = bars + 8u * (2 * STAGES);
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + STAGES * Cfg::kStageBytes + 8 * (2 * STAGES + 1));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lane_row0 = blockIdx.x * BM;
    const int col_row0 = blockIdx.y * BN;
    const int total_kb = (K + BK - 1) / BK;
    const int kb_begin = blockIdx.z * kblocks_per_split;
    const int kb_end = min(total_kb, kb_begin + kblocks_per_split);
    const int num_kb = kb_end - kb_begin;                   // >= 1 by construction of the grid

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(tmem_full_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_lane) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_col) : "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------------ TMA producer
            // The weights do not depend on the kernel before this one: the first stages'
            // weight tiles are requested before waiting for it, the activations after.
            const CUtensorMap* tm_w = SWAP ? &tm_lane : &tm_col;
            const CUtensorMap* tm_x = SWAP ? &tm_col : &tm_lane;
            const int pre = num_kb < STAGES ? num_kb : STAGES;
            for (int i = 0; i < pre; ++i) {
                const uint32_t a_dst = base + i * Cfg::kStageBytes;
                mbar_expect_tx(full_bar(i), Cfg::kStageBytes);
                tma_load_2d(SWAP ? a_dst : a_dst + BM * BK * 2, tm_w, full_bar(i), (kb_begin + i) * BK,
                            SWAP ? lane_row0 : col_row0);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                const uint32_t a_dst = base + i * Cfg::kStageBytes;
                tma_load_2d(SWAP ? a_dst + BM * BK * 2 : a_dst, tm_x, full_bar(i), (kb_begin + i) * BK,
                            SWAP ? col_row0 : lane_row0);
            }
            for (int i = pre; i < num_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t round = i / STAGES;
                if (round > 0 && !mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag)) break;
                const uint32_t a_dst = base + s * Cfg::kStageBytes;
                const uint32_t b_dst = a_dst + BM * BK * 2;
                mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
                const int k = (kb_begin + i) * BK;
                tma_load_2d(a_dst, &tm_lane, full_bar(s), k, lane_row0);
                tma_load_2d(b_dst, &tm_col, full_bar(s), k, col_row0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // -------------------------------------------------------- MMA issuer
            constexpr uint32_t idesc = make_idesc(BM, BN);
            bool ok = true;
            for (int i = 0; i < num_kb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t round = i / STAGES;
                ok = mbar_wait(full_bar(s), round & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = base + s * Cfg::kStageBytes;
                const uint64_t adesc = make_smem_desc(a_addr);
                const uint64_t bdesc = make_smem_desc(a_addr + BM * BK * 2);
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                    // 16 K-elements = 32 bytes = 2 descriptor units further along the swizzled row
                    umma_bf16(tmem_acc, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                              (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar(s));          // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(tmem_full_bar);     // accumulators complete
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                     // TMEM lane quarter this warp may read
        pdl_wait();                                 // nothing is written before the kernel ahead has finished
        const bool ok = mbar_wait(tmem_full_bar, 0, abort_flag);
        tc_fence_after();
        if (ok) {
            const int lr = lane_row0 + q * 32 + lane;          // row of the lane operand
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                tmem_ld_wait();
                if (lr >= rows_lane) continue;
                if constexpr (!SWAP) {
                    // thread owns out[lr, col_row0 + c0 .. +16)
                    const int n0 = col_row0 + c0;
                    TC* o = out + (size_t)lr * ldo + n0;
                    const float* r = (EPI == EPI_RESIDUAL) ? residual + (size_t)lr * ldo + n0 : nullptr;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (n0 + j < rows_col) {
                            float x = __uint_as_float(v[j]);
                            if constexpr (EPI == EPI_RESIDUAL) x = r[j] + x;
                            if constexpr (EPI == EPI_ATOMIC) atomicAdd((float*)&o[j], x);
                            else o[j] = from_f32<TC>(x);
                        }
                    }
                } else {
                    // thread owns out[col_row0 + c0 .. +16, lr]: a warp writes 32 consecutive n
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = col_row0 + c0 + j;
                        if (m < rows_col) {
                            float x = __uint_as_float(v[j]);
                            const size_t idx = (size_t)m * ldo + lr;
                            if constexpr (EPI == EPI_RESIDUAL) x = residual[idx] + x;
                            if constexpr (EPI == EPI_ATOMIC) atomicAdd((float*)&out[idx], x);
                            else out[idx] = from_f32<TC>(x);
                        }
                    }
                }
            }
        }
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
        tc_fence_after();
        tmem_dealloc(tmem_acc, Cfg::kTmemCols);
    }
}

// ------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

struct MapKey {
    const void* ptr; int rows; int K; int box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && K == o.K && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h ^= (size_t)k.rows * 0x9E3779B97F4A7C15ull; h ^= (size_t)k.K * 0xC2B2AE3D27D4EB4Full; h ^= (size_t)k.box_rows << 48;
        return h;
    }
};

// Tensor map of a row-major bf16 matrix [rows, K]: boxes of 64 K-elements x box_rows rows,
// 128-byte swizzle, zero fill outside the matrix.
bool get_tensor_map(const void* ptr, int rows, int K, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    const MapKey key{ptr, rows, K, box_rows};
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return true; }
    }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    {
        std::lock_guard<std::mutex> g(mu);
        if (cache.size() > 4096) cache.clear();
        cache[key] = m;
    }
    *out = m;
    return true;
}

int* g_error_flag = nullptr;

template <int BN, bool SWAP, int EPI, typename TC>
int launch_tc(const CUtensorMap& tl, const CUtensorMap& tc, void* out, const float* residual,
              int rows_lane, int rows_col, int K, int ldo, int splits, cudaStream_t stream) {
    using Cfg = TileCfg<BN>;
    auto kern = gemm_tc_kernel<BN, SWAP, EPI, TC>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
            return TFF_ERR_LAUNCH;
        configured = true;
    }
    const int total_kb = (K + BK - 1) / BK;
    const int per = (total_kb + splits - 1) / splits;
    const int real_splits = (total_kb + per - 1) / per;        // no empty split
    dim3 grid((rows_lane + BM - 1) / BM, (rows_col + BN - 1) / BN, real_splits);
    return tff_launch_pdl(kern, grid, NUM_THREADS, Cfg::kSmemBytes, stream, tl, tc, (TC*)out, residual, rows_lane,
                          rows_col, K, ldo, per, g_error_flag);
}

template <int BN, bool SWAP>
int dispatch_epi(const CUtensorMap& tl, const CUtensorMap& tc, void* out, int out_is_bf16, const float* residual,
                 int atomic, int rows_lane, int rows_col, int K, int ldo, int splits, cudaStream_t s) {
    if (atomic) {
        if (out_is_bf16) return TFF_ERR_BAD_ARGUMENT;
        return launch_tc<BN, SWAP, EPI_ATOMIC, float>(tl, tc, out, nullptr, rows_lane, rows_col, K, ldo, splits, s);
    }
    if (residual) {
        if (out_is_bf16) return TFF_ERR_BAD_ARGUMENT;
        return launch_tc<BN, SWAP, EPI_RESIDUAL, float>(tl, tc, out, residual, rows_lane, rows_col, K, ldo, 1, s);
    }
    if (out_is_bf16) return launch_tc<BN, SWAP, EPI_STORE, bf16>(tl, tc, out, nullptr, rows_lane, rows_col, K, ldo, 1, s);
    return launch_tc<BN, SWAP, EPI_STORE, float>(tl, tc, out, nullptr, rows_lane, rows_col, K, ldo, 1, s);
}

}  // namespace

// One-time set-up of this translation unit on the current device: the error word.
TFF_API int tff_gemm_tc_init() {
    if (g_error_flag) return TFF_OK;
    if (!get_encode_fn()) return TFF_ERR_DRIVER;
    if (cudaMalloc(&g_error_flag, sizeof(int)) != cudaSuccess) return TFF_ERR_LAUNCH;
    if (cudaMemset(g_error_flag, 0, sizeof(int)) != cudaSuccess) return TFF_ERR_LAUNCH;
    return TFF_OK;
}

// Reads (and clears) the error word: non-zero when a bounded wait inside a kernel ran out.
// Synchronises the device.
TFF_API int tff_gemm_tc_error() {
    if (!g_error_flag) return 0;
    int v = 0;
    if (cudaMemcpy(&v, g_error_flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(g_error_flag, 0, sizeof(int));
    return v;
}

// out[M, N] (+)= A[M, K] * W[N, K]^T; A, W bfloat16.
//   swap    0: A rows on TMEM lanes (tiles 128 x bn over M x N); 1: W rows on lanes (tiles 128 x bn over N x M)
//   bn      16, 32, 64, 128 or 256
//   splits  number of K ranges (> 1 only with atomic = 1)
//   atomic  1: float32 atomic adds into ``out`` (which the caller has initialised); residual must be null
//   residual float32 [M, N] added to the product (may alias ``out``); out must be float32
TFF_API int tff_gemm_tc(const void* A, const void* W, void* out, int out_is_bf16, const float* residual,
                        int M, int N, int K, int swap, int bn, int splits, int atomic, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return TFF_OK;
    if (K <= 0 || splits < 1 || (splits > 1 && !atomic) || (atomic && residual)) return TFF_ERR_BAD_ARGUMENT;
    if (K % 8 != 0) return TFF_ERR_UNSUPPORTED;                         // TMA row pitch must be a multiple of 16 bytes
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return TFF_ERR_UNSUPPORTED;
    if (!g_error_flag) { const int st = tff_gemm_tc_init(); if (st != TFF_OK) return st; }
    const void* lane_ptr = swap ? W : A;
    const void* col_ptr = swap ? A : W;
    const int rows_lane = swap ? N : M, rows_col = swap ? M : N;
    CUtensorMap tl, tc;
    if (!get_tensor_map(lane_ptr, rows_lane, K, BM, &tl)) return TFF_ERR_DRIVER;
    if (!get_tensor_map(col_ptr, rows_col, K, bn, &tc)) return TFF_ERR_DRIVER;
#define TFF_CASE(BN_)                                                                                              \
    case BN_:                                                                                                      \
        return swap ? dispatch_epi<BN_, true>(tl, tc, out, out_is_bf16, residual, atomic, rows_lane, rows_col, K, N, splits, stream) \
                    : dispatch_epi<BN_, false>(tl, tc, out, out_is_bf16, residual, atomic, rows_lane, rows_col, K, N, splits, stream);
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
