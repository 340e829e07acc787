// The gate/up projection of a decode step as ONE kernel with the SwiGLU behind it and, for steps of at most 16
// tokens, the RMSNorm ahead of it:
//
//   y[m, n] = r[m] * sum_k bf16(x[m, k] * w_norm[k]) * W[n, k],   r[m] = rsqrt(mean_k x[m, k]^2 + eps)
//   act[m, i] = bf16(silu(y_gate[m, i]) * y_up[m, i])
//
// A decode layer is a chain of dependent kernels; the norm and the SwiGLU kernel move next to nothing and cost
// 4 and 6 us a layer at the margin (Qwen3-8B shape, 8 requests).  As one kernel the group is 3.5 us a layer
// faster at 8 requests and 5 at one (3.70 -> 3.55 ms and 3.28 -> 3.10 ms a step).  The q/k/v group was built
// the same way (its tail: per-head RMSNorm, rotation and cache write in the first CTA of a cluster of eight)
// and measured slower than its three separate kernels (3.82 against 3.70 ms a step): eight K blocks a CTA are
// too little work to carry two cluster barriers and a serial tail, so that group keeps its kernels.
//
// How the nonlinear tail gets whole sums although the K range is split (one pass of the weights through all
// SMs wants some 400 CTAs, and the product has about 200 tiles of 128 weight rows): the CTAs that share a
// tile form a thread-block cluster.  Each takes a slice of the K range, accumulates in tensor memory, and then
// leaves its 128 x 16 partial sums in its shared memory, from where the first CTA fetches them through distributed
// shared memory (ld.shared::cluster), together with each CTA's share of the rows' sums of squares, which comes for
// free from the x tiles it converts.  The first CTA then holds complete, still linear sums, applies r[m] and
// runs the tail.
//
// The activation operand is made in the kernel: the four warps that later run the epilogue (a CTA has one
// segment, so they would idle through the main loop) read x from global memory (L2), multiply by the norm's
// weight, round to bfloat16 and write the 128-byte-swizzled tile the tensor core reads; warp w takes the K
// blocks n with n % 4 == w and has the x of its next block in registers while it writes the current one, so
// eight loads of x are in flight a CTA.  (The separate norm kernel rounds (x * r) * w; here x * w is rounded
// and the float32 r multiplies the float32 sum: the same number of roundings.)
//   warp 0      TMA producer of the weight tiles (one lane)
//   warp 1      TMEM allocation, MMA issue (one lane)
//   warps 2-5   activation tiles; then partial sums out of tensor memory, the cluster reduction, the tail
// A stage is full when its weight tile has landed and its activation tile has been written.
// Rows that come normalised already (FOLD_NORM = false: a block arrangement that did not defer its norm) arrive as
// bfloat16 by TMA.  The kernel is a template on the number of token columns; 32 and 64 columns (steps of 17 to 64
// tokens, rows by TMA) were measured and are not instantiated: 7.05 against 6.85 ms a step at 64 requests, even at
// 32, although they save the SwiGLU kernel and the accumulators' float32 round trip.
// Every mbarrier wait is bounded; the two cluster barriers are reached by every thread whatever happened.
#include "tcgen05.cuh"

namespace {

using namespace tc5;

constexpr int C_THREADS = 192;
constexpr int C_CTAS_PER_SM = 3;
constexpr int C_W_BYTES = BM * BK * 2;                    // 16 KB weight tile

template <int BN> struct ClusterCfg {
    static constexpr int kStages = BN == 16 ? 4 : 3;
    static constexpr int kBBytes = BN * BK * 2;            // bfloat16 activation tile: 2, 4 or 8 KB
    static constexpr int kStageBytes = C_W_BYTES + kBBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
    static constexpr int kTmemCols = BN < 32 ? 32 : BN;
    static_assert(kStageBytes % 1024 == 0, "stages must keep the 1024-byte alignment of swizzled tiles");
    static_assert(C_CTAS_PER_SM * (kSmemBytes + 1024) <= 228 * 1024, "the CTAs meant to share an SM do not fit");
    static_assert(BM * BN * 4 + 5 * 16 * 4 <= kStages * kStageBytes, "the reduction buffer reuses the ring");
};

struct ClusterGemmParams {
    const float* x;                       // FOLD_NORM: [M, K] float32
    const float* norm_w; float eps;       // FOLD_NORM: input RMSNorm
    int M, N, K;
    bf16* act; int inter;                 // [M, inter] bfloat16 out
    int* error_flag;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA ``rank`` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int BN, bool FOLD_NORM>
__global__ void __launch_bounds__(C_THREADS, C_CTAS_PER_SM)
gemm_tc_cluster_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_h,
                       const ClusterGemmParams p) {
    static_assert(!FOLD_NORM || BN == 16, "the activation tile is made in the kernel for 16 token columns only");
    using Cfg = ClusterCfg<BN>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + STAGES * Cfg::kStageBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };                    // weights landed and activations there
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };        // the MMAs have read the stage
    const uint32_t tfull_bar = bars + 8u * (2 * STAGES);
    uint8_t* tail = gen_base + STAGES * Cfg::kStageBytes + 8 * (2 * STAGES + 1);
    volatile uint32_t* tmem_slot = (volatile uint32_t*)tail;
    volatile int* abort_flag = (volatile int*)(tail + 4);
    // after the main loop the ring is free: each CTA's holds its share, the first CTA's then the sums of the cluster
    float* red = reinterpret_cast<float*>(gen_base);                  // [128 features][BN tokens]
    float* sumsq = red + BM * BN;                                     // [16 tokens]          (FOLD_NORM)
    float* ss_part = sumsq + 16;                                      // [4 warps][16 tokens] (FOLD_NORM)
    const uint32_t red_addr = base, sumsq_addr = base + BM * BN * 4;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank(), csize = cluster_nctarank();
    const int tile = blockIdx.x / csize;
    const int kbt = (p.K + BK - 1) / BK;
    const int kb0 = (int)((long long)kbt * rank / csize), kb1 = (int)((long long)kbt * (rank + 1) / csize);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), FOLD_NORM ? 2 : 1); mbar_init(empty_bar(s), 1); }
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        if (!FOLD_NORM) asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_h) : "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    float my_ss = 0.f;                                   // converter: this lane's share of its row's sum of squares
    if (warp == 0) {
        if (lane == 0) {
            // ---------------------------------------------- TMA producer (the weights are older than the kernel ahead)
            if constexpr (FOLD_NORM) {
                for (int kb = kb0; kb < kb1; ++kb) {
                    const uint32_t n = kb - kb0;
                    const int s = n % STAGES;
                    if (n >= STAGES && !mbar_wait(empty_bar(s), (n / STAGES - 1) & 1, abort_flag)) break;
                    mbar_expect_tx(full_bar(s), C_W_BYTES);
                    tma_load_2d(base + s * Cfg::kStageBytes, &tm_w, full_bar(s), kb * BK, tile * BM);
                }
            } else {
                // weight tiles of the first ring before the wait for the kernel ahead, its activation rows after
                const int pre = min(STAGES, kb1 - kb0);
                for (int i = 0; i < pre; ++i) {
                    mbar_expect_tx(full_bar(i), Cfg::kStageBytes);
                    tma_load_2d(base + i * Cfg::kStageBytes, &tm_w, full_bar(i), (kb0 + i) * BK, tile * BM);
                }
                pdl_wait();
                for (int i = 0; i < pre; ++i)
                    tma_load_2d(base + i * Cfg::kStageBytes + C_W_BYTES, &tm_h, full_bar(i), (kb0 + i) * BK, 0);
                for (int kb = kb0 + pre; kb < kb1; ++kb) {
                    const uint32_t n = kb - kb0;
                    const int s = n % STAGES;
                    if (!mbar_wait(empty_bar(s), (n / STAGES - 1) & 1, abort_flag)) break;
                    mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
                    tma_load_2d(base + s * Cfg::kStageBytes, &tm_w, full_bar(s), kb * BK, tile * BM);
                    tma_load_2d(base + s * Cfg::kStageBytes + C_W_BYTES, &tm_h, full_bar(s), kb * BK, 0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // -------------------------------------------------------- MMA issuer
            constexpr uint32_t idesc = make_idesc(BM, BN);
            bool ok = true;
            for (int kb = kb0; kb < kb1 && ok; ++kb) {
                const uint32_t n = kb - kb0;
                const int s = n % STAGES;
                if (!mbar_wait(full_bar(s), (n / STAGES) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a_addr = base + s * Cfg::kStageBytes;
                const uint64_t adesc = make_smem_desc(a_addr);
                const uint64_t bdesc = make_smem_desc(a_addr + C_W_BYTES);
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk)
                    umma_bf16(tmem_base, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                              (kb > kb0 || kk > 0) ? 1u : 0u);
                umma_commit(empty_bar(s));
            }
            if (ok) umma_commit(tfull_bar);
        }
    } else if constexpr (FOLD_NORM) {
        // ------------------------------------------------------------ activation tiles (warps 2-5)
        // Lane (row, half): 32 consecutive K elements of token ``row``; out go four 16-byte chunks of the row's
        // 128-byte line of the bfloat16 tile, at ((half * 4 + c) XOR row % 8).
        const int cw = warp - 2;
        const int row = lane >> 1, half = lane & 1;
        const bool live = row < p.M;
        const float* xrow = p.x + (size_t)row * p.K;
        pdl_wait();                                        // x is what the kernel ahead wrote
        float4 nx[8];
        auto fetch = [&](int kb) {
            const int k0 = kb * BK + half * 32;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                nx[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live && kb < kb1 && k0 + 4 * i < p.K) nx[i] = *reinterpret_cast<const float4*>(xrow + k0 + 4 * i);
            }
        };
        fetch(kb0 + cw);
        bool ok = true;
        for (int kb = kb0 + cw; kb < kb1 && ok; kb += 4) {
            const uint32_t n = kb - kb0;
            const int s = n % STAGES;
            const int k0 = kb * BK + half * 32;
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 a = nx[i];
                my_ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
                float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
                if (k0 + 4 * i < p.K) w = __ldg(reinterpret_cast<const float4*>(p.norm_w + k0 + 4 * i));
                packed[2 * i] = pack2(a.x * w.x, a.y * w.y);
                packed[2 * i + 1] = pack2(a.z * w.z, a.w * w.w);
            }
            fetch(kb + 4);                                 // the next block of this warp, in flight while this one is written
            if (n >= STAGES) {
                bool free_now = true;
                if (lane == 0) free_now = mbar_wait(empty_bar(s), (n / STAGES - 1) & 1, abort_flag);
                free_now = __shfl_sync(0xffffffffu, free_now, 0);
                if (!free_now) { ok = false; break; }
            }
            const uint32_t btile = base + s * Cfg::kStageBytes + C_W_BYTES + (uint32_t)row * 128u;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t dst = btile + (uint32_t)((((half * 4 + c) ^ (row & 7)) & 7) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[4 * c]), "r"(packed[4 * c + 1]),
                             "r"(packed[4 * c + 2]), "r"(packed[4 * c + 3]) : "memory");
            }
            fence_async_smem();                             // the tensor core reads through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(full_bar(s));
        }
        my_ss += __shfl_xor_sync(0xffffffffu, my_ss, 1);   // both halves of the row
    }

    // ---------------------------------------------------------------- partial sums out of tensor memory
    const bool epi = warp >= 2;
    const int q = warp & 3;
    float acc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.f;
    if (epi && kb1 > kb0) {
        if (mbar_wait(tfull_bar, 0, abort_flag)) {
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c0 + j] = __uint_as_float(v[j]);
            }
        }
        tc_fence_before();
    }
    // ---------------------------------------------------------------- cluster reduction in the first CTA
    // Every CTA puts its share into its own shared memory (its ring is free by now); after the cluster barrier
    // the first CTA's epilogue threads fetch the others' shares over distributed shared memory, 16-byte loads,
    // and add them to what they hold in registers.  The others may not leave (their shared memory would go)
    // before that is done: they wait at the second barrier, at which the first CTA's threads arrive as soon as
    // they have read.
    __syncthreads();                                       // this CTA's ring is no longer read or written
    const int f = q * 32 + lane;                           // feature row of an epilogue thread
    if constexpr (FOLD_NORM) {
        if (epi && (lane & 1) == 0) ss_part[(warp - 2) * 16 + (lane >> 1)] = my_ss;
        __syncthreads();
        if (warp == 2 && lane < 16) my_ss = ss_part[lane] + ss_part[16 + lane] + ss_part[32 + lane] + ss_part[48 + lane];
    }
    if (rank != 0) {
        if (epi) {
            float4* mine = reinterpret_cast<float4*>(red + f * BN);
#pragma unroll
            for (int c = 0; c < BN / 4; ++c) mine[c] = make_float4(acc[4 * c], acc[4 * c + 1], acc[4 * c + 2], acc[4 * c + 3]);
        }
        if (FOLD_NORM && warp == 2 && lane < 16) sumsq[lane] = my_ss;
    }
    __syncwarp();
    cluster_sync_all();                                    // every share is in its CTA's shared memory
    if (rank == 0) {
        if (epi) {
            for (uint32_t r = 1; r < csize; ++r) {
                const uint32_t src = map_to_cta(red_addr + (uint32_t)(f * BN) * 4u, r);
#pragma unroll
                for (int c = 0; c < BN / 4; ++c) {
                    float4 t;
                    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w) : "r"(src + 16u * c) : "memory");
                    acc[4 * c] += t.x; acc[4 * c + 1] += t.y; acc[4 * c + 2] += t.z; acc[4 * c + 3] += t.w;
                }
            }
#pragma unroll
            for (int j = 0; j < BN; ++j) red[f * BN + j] = acc[j];
        }
        if (FOLD_NORM && warp == 2 && lane < 16) {
            // the rows' sums of squares: lane ``row`` of the first epilogue warp holds this CTA's share
            float ss = my_ss;
            for (uint32_t r = 1; r < csize; ++r) {
                float t;
                asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(t)
                             : "r"(map_to_cta(sumsq_addr + 4u * (uint32_t)lane, r)) : "memory");
                ss += t;
            }
            sumsq[lane] = ss;
        }
    }
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");      // done reading the others' memory
    if (rank != 0) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    __syncthreads();                                       // first CTA: sums and sums of squares are in place

    // ---------------------------------------------------------------- the tail, in the first CTA
    if (rank == 0 && epi && !*abort_flag) {
        pdl_wait();                                        // nothing is written before the kernel ahead has finished
        // features 0..63 of the tile are the gate, 64..127 the up projection of the same 64 channels
        const int et = threadIdx.x - 64;
        const float inv_k = 1.0f / (float)p.K;
        for (int idx = et; idx < p.M * 64; idx += 128) {
            const int j = idx >> 6, c = idx & 63;
            const int channel = tile * 64 + c;
            if (channel >= p.inter) continue;
            const float r = FOLD_NORM ? rsqrtf(sumsq[j] * inv_k + p.eps) : 1.0f;
            const float g = red[c * BN + j] * r, u = red[(64 + c) * BN + j] * r;
            p.act[(size_t)j * p.inter + channel] = __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * u);   // rounded to bfloat16 anyway
        }
    }
    // ------------------------------------------------------------------ teardown
    if (rank == 0) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // pairs with its arrive above
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);      // copies in flight land before the shared memory goes
        if (threadIdx.x == 0) atomicExch(p.error_flag, 1);
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

template <int BN, bool FOLD_NORM>
int launch_cluster_gemm(const CUtensorMap& tw, const CUtensorMap& th, const ClusterGemmParams& p, cudaStream_t stream) {
    using Cfg = ClusterCfg<BN>;
    auto kern = gemm_tc_cluster_kernel<BN, FOLD_NORM>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
            return TFF_ERR_LAUNCH;
        configured = true;
    }
    const int tiles = (p.N + BM - 1) / BM, kbt = (p.K + BK - 1) / BK;
    // CTAs of a tile: as many as fill the SMs' CTA slots once (as in gemm_tc.cu, not every slot is taken), at most
    // 8 (the portable cluster size) and at most one per K block
    static int cs_max = -1;
    if (cs_max < 0) { const char* e = getenv("TFFINFER_CLUSTER_MAX"); cs_max = e ? atoi(e) : 8; if (cs_max < 1 || cs_max > 8) cs_max = 8; }
    int cs = (int)(tff_decode_gemm_ctas(1ll << 40) / tiles);
    cs = cs < 1 ? 1 : (cs > cs_max ? cs_max : cs);
    if (cs > kbt) cs = kbt;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * cs)); cfg.blockDim = dim3(C_THREADS);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tff_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kern, tw, th, p) == cudaSuccess ? TFF_OK : TFF_ERR_LAUNCH;
}

}  // namespace

// gate/up projection of a decode step of at most 16 tokens with the norm ahead of it and its activation:
// act [M, I] bfloat16 = silu(gate) * up of RMSNorm(x) W^T; x [M, K] float32, W [2 I, K] bfloat16 with gate and up
// rows alternating in blocks of 64 (I a multiple of 64).  TFF_ERR_UNSUPPORTED for shapes it does not take.
TFF_API int tff_gemm_tc_cluster_swiglu(const float* x, const float* norm_w, float eps, const void* W, int M, int K,
                                       void* act, int inter, cudaStream_t stream) {
    if (M <= 0) return TFF_OK;
    if (inter <= 0 || !act || K <= 0 || !x || !norm_w || !W) return TFF_ERR_BAD_ARGUMENT;
    if (inter % 64 != 0 || M > 16 || K % 8 != 0) return TFF_ERR_UNSUPPORTED;
    if (((uintptr_t)W & 15) || ((uintptr_t)x & 15) || ((uintptr_t)norm_w & 15)) return TFF_ERR_UNSUPPORTED;
    ClusterGemmParams p = {};
    p.x = x; p.norm_w = norm_w; p.eps = eps; p.M = M; p.N = 2 * inter; p.K = K;
    p.act = (bf16*)act; p.inter = inter;
    p.error_flag = tff_device_error_flag();
    if (p.error_flag == nullptr) return TFF_ERR_LAUNCH;
    CUtensorMap tw;
    if (!tff_tensor_map_2d(W, p.N, K, BM, BK, 2, &tw)) return TFF_ERR_DRIVER;
    return launch_cluster_gemm<16, true>(tw, tw, p, stream);
}

// The same for activation rows that have been normalised already: h [M <= 16, K] bfloat16.
TFF_API int tff_gemm_tc_cluster_swiglu_bf16(const void* h, const void* W, int M, int K, void* act, int inter,
                                            cudaStream_t stream) {
    if (M <= 0) return TFF_OK;
    if (inter <= 0 || !act || K <= 0 || !h || !W) return TFF_ERR_BAD_ARGUMENT;
    if (inter % 64 != 0 || M > 16 || K % 8 != 0) return TFF_ERR_UNSUPPORTED;
    if (((uintptr_t)W & 15) || ((uintptr_t)h & 15)) return TFF_ERR_UNSUPPORTED;
    ClusterGemmParams p = {};
    p.M = M; p.N = 2 * inter; p.K = K;
    p.act = (bf16*)act; p.inter = inter;
    p.error_flag = tff_device_error_flag();
    if (p.error_flag == nullptr) return TFF_ERR_LAUNCH;
    CUtensorMap tw, th;
    if (!tff_tensor_map_2d(W, p.N, K, BM, BK, 2, &tw)) return TFF_ERR_DRIVER;
    if (!tff_tensor_map_2d(h, M, K, 16, BK, 2, &th)) return TFF_ERR_DRIVER;     // rows beyond M arrive as zeros
    return launch_cluster_gemm<16, false>(tw, th, p, stream);
}
