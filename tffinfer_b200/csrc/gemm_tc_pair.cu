// bfloat16 matrix product on pairs of SMs (tcgen05 cta_group::2), for prompt-sized M:
//   out[M, N] = A[M, K] * W[N, K]^T  (+ residual | SwiGLU), float32 accumulation in tensor memory.
//
// A cluster of two CTAs works on a 256 x 256 tile.  Each CTA holds 128 rows of A and HALF of the
// 256 weight rows of the tile in its shared memory (32 KB a stage instead of the 48 KB a single CTA
// needs for a 128 x 256 tile); one thread of the pair's first CTA issues tcgen05.mma.cta_group::2
// (M = 256, N = 256, K = 16), which reads both CTAs' operands and leaves rows 0-127 of the result in
// the first CTA's tensor memory and rows 128-255 in the second's.  With a third less to load per
// product the ring is six stages deep: the main loop of the single-CTA kernel is bound by the bytes
// it can keep in flight, this one much less so.  Each CTA then runs the same epilogue as the
// single-CTA kernel on its own 128 x 256 half.
//
//   warp 0      TMA producer (one lane) in both CTAs: its A rows and its half of the W rows; every
//               load reports its bytes to the FIRST CTA's "full" barrier of the stage
//   warp 1      TMEM allocation (both CTAs); in the first CTA, MMA issue (one lane); its commits go
//               to the "empty" and "accumulator full" barriers of both CTAs (multicast)
//   warps 2-5   epilogue in both CTAs; all eight warps of the pair arrive at the first CTA's
//               "accumulator empty" barrier
// No load is multicast.  The pair's two tiles are neighbours along M; pair tiles go round-robin
// over the clusters, rows fastest; the tiles of a last, partial wave can be cut along K as in
// gemm_tc.cu when the product is added to a float32 buffer.
// Every mbarrier wait is bounded as in gemm_tc.cu; the two cluster barriers (after set-up, before
// tear-down) are reached by every thread whatever happened in between.
// Every wait of this kernel lets the hardware suspend the warp: the four epilogue warps wait for an accumulator
// while the issuing threads on their schedulers work, and polled they took issue slots from those (the four
// products of a layer at 2048 tokens ran 4 % slower).
#define TFF_SUSPENDED_WAITS
#include <type_traits>
#include "gemm_epilogue.cuh"
#include "gemm_tc_pair.h"

namespace {

using namespace tc5;

constexpr int PBN = 256;                          // columns of the pair's tile
constexpr int HALF_N = PBN / 2;                   // weight rows a CTA loads
constexpr int P_STAGE_BYTES = BM * BK * 2 + HALF_N * BK * 2;      // 32 KB
constexpr int P_STAGES = 6;
constexpr int P_STAGING_BYTES = 4 * 2 * 4096;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + P_STAGING_BYTES + 1024 + 256;
constexpr int P_TMEM_COLS = 2 * PBN;              // two accumulator buffers of 256 columns

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the shared::cluster address of ``local`` (a shared::cta address) in CTA ``rank`` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    tc5::jitter();
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// a TMA load of one CTA of a pair; ``bar`` is a shared::cluster address and may lie in the other CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the products issued so far are done, at the barrier at this shared-memory offset in
// every CTA of the cluster named by ``mask``
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}

template <int EPI, typename TC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_a,     // activations [M, K], box 64 x 128
                    const __grid_constant__ CUtensorMap tm_w,     // weights [N, K], box 64 x 128 (half a tile's rows)
                    const __grid_constant__ CUtensorMap tm_out,   // output, boxes of 128 bytes x 32 rows
                    int rows_m, int rows_n, int K, int stream_k, int* error_flag,
                    const QkvEpilogue qkv) {                  // EPI_QKV only
    constexpr int STAGES = P_STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t staging = base + STAGES * P_STAGE_BYTES;
    const uint32_t bars = staging + P_STAGING_BYTES;
    // barriers: full[STAGES] (used in the first CTA), empty[STAGES], tmem_full[2], tmem_empty[2] (first CTA)
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + STAGES * P_STAGE_BYTES + P_STAGING_BYTES + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                 // 0: the CTA that issues the products
    const int cluster_id = (int)blockIdx.x >> 1, n_clusters = (int)gridDim.x >> 1;
    const int kbt = (K + BK - 1) / BK;
    const int n_m_pairs = (rows_m + 2 * BM - 1) / (2 * BM);
    const int n_col_tiles = (rows_n + PBN - 1) / PBN;
    const int n_tiles = n_m_pairs * n_col_tiles;             // tiles of the pair

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_out) : "memory");
    }
    __syncthreads();
    cluster_sync_all();                                       // both CTAs' barriers exist before either is touched from outside
    if (warp == 1) tmem_alloc_pair(smem_u32((const void*)tmem_slot), P_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------------ TMA producer (both CTAs)
            pdl_wait();
            SegIterSlices it(n_tiles, kbt, stream_k, cluster_id, n_clusters);
            uint32_t n = 0;
            bool ok = true;
            while (ok && it.next()) {
                const int arow = ((it.tile % n_m_pairs) * 2 + (int)rank) * BM;
                const int wrow = (it.tile / n_m_pairs) * PBN + (int)rank * HALF_N;
                for (int kb = it.kb0; kb < it.kb1; ++kb, ++n) {
                    const int s = n % STAGES;
                    const uint32_t round = n / STAGES;
                    if (round > 0 && !mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag)) { ok = false; break; }
                    const uint32_t first_full = map_to_cta(full_bar(s), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * P_STAGE_BYTES);     // both CTAs' tiles of the stage
                    const uint32_t a_dst = base + s * P_STAGE_BYTES;
                    tma_load_2d_pair(a_dst, &tm_a, first_full, kb * BK, arow);
                    tma_load_2d_pair(a_dst + BM * BK * 2, &tm_w, first_full, kb * BK, wrow);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // -------------------------------------------------------- MMA issuer (first CTA)
            constexpr uint32_t idesc = make_idesc(2 * BM, PBN);
            SegIterSlices it(n_tiles, kbt, stream_k, cluster_id, n_clusters);
            uint32_t n = 0, seg = 0;
            bool ok = true;
            while (ok && it.next()) {
                const uint32_t acc = seg & 1, use = seg >> 1;
                if (use > 0 && !mbar_wait(tempty_bar(acc), (use - 1) & 1, abort_flag)) break;   // both epilogues have drained it
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * PBN;
                for (int kb = it.kb0; kb < it.kb1; ++kb, ++n) {
                    const int s = n % STAGES;
                    const uint32_t round = n / STAGES;
                    if (!mbar_wait(full_bar(s), round & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = base + s * P_STAGE_BYTES;
                    const uint64_t adesc = make_smem_desc(a_addr);
                    const uint64_t bdesc = make_smem_desc(a_addr + BM * BK * 2);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk)
                        umma_bf16_pair(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                                       (kb > it.kb0 || kk > 0) ? 1u : 0u);
                    umma_commit_pair(empty_bar(s), 3);       // the stage is free in both CTAs once these products have read it
                }
                if (ok) umma_commit_pair(tfull_bar(acc), 3); // this segment's accumulators are complete in both CTAs
                ++seg;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs)
        const int q = warp & 3;
        pdl_wait();
        const uint32_t first_tempty[2] = {map_to_cta(tempty_bar(0), 0), map_to_cta(tempty_bar(1), 0)};
        SegIterSlices it(n_tiles, kbt, stream_k, cluster_id, n_clusters);
        uint32_t seg = 0, chunk_no = 0;
        while (it.next()) {
            const uint32_t acc = seg & 1, use = seg >> 1;
            if (!mbar_wait(tfull_bar(acc), use & 1, abort_flag)) break;
            tc_fence_after();
            const int lane_row0 = ((it.tile % n_m_pairs) * 2 + (int)rank) * BM, col_row0 = (it.tile / n_m_pairs) * PBN;
            const uint32_t t_addr = tmem_base + acc * PBN + ((uint32_t)(q * 32) << 16);
            const bool partial = stream_k && (it.kb1 - it.kb0) < kbt;
            if constexpr (EPI == EPI_QKV)
                epilogue_quarter_qkv(t_addr, lane, q, lane_row0, col_row0, qkv);
            else
                epilogue_quarter_tma<PBN, EPI, TC>(t_addr, staging + (uint32_t)((warp - 2) * 2) * 4096u, chunk_no, lane, q,
                                                   lane_row0, col_row0, partial, &tm_out);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(first_tempty[acc]);
            ++seg;
        }
        if (lane == 0) bulk_wait_read<0>();                   // staged rows must have been read before the CTA leaves
    }
    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);       // copies still in flight land before the memory is released
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        __syncthreads();
    }
    cluster_sync_all();                                       // neither CTA leaves while the other may still reach into it
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, P_TMEM_COLS);
    }
}

template <int EPI, typename TC>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to, int M, int N, int K, int stream_k,
                cudaStream_t stream, const QkvEpilogue& qkv = QkvEpilogue()) {
    auto kern = gemm_tc_pair_kernel<EPI, TC>;
    static int max_clusters = -1;                 // clusters of this kernel the device runs at a time
    if (max_clusters < 0) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES) != cudaSuccess)
            return TFF_ERR_LAUNCH;
        // SMs pair up inside a GPC, so fewer than half the SM count may be possible; a cluster that had to
        // wait for another to finish would double the time of this persistent kernel
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(tff_num_sms() / 2 * 2)); cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = P_SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = tff_num_sms() / 2; }
        if (n > tff_num_sms() / 2) n = tff_num_sms() / 2;
        max_clusters = n;
    }
    const long long n_tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + PBN - 1) / PBN);
    const long long units = stream_k ? n_tiles * ((K + BK - 1) / BK) : n_tiles;
    long long clusters = max_clusters;
    if (clusters <= 0) return TFF_ERR_LAUNCH;
    if (clusters > units) clusters = units;
    return tff_launch_pdl(kern, dim3((unsigned)(2 * clusters)), dim3(NUM_THREADS), (size_t)P_SMEM_BYTES, stream, ta, tw, to,
                          M, N, K, stream_k, tff_device_error_flag(), qkv);
}

}  // namespace

// The q/k/v projection of a prompt portion with everything up to the cache write in its epilogue:
//   [q | k | v] = A[M, K] * W[(nq + 2 nkv) * 128, K]^T; q and k heads normalised (weights q_w, k_w of 128, or null)
//   and rotated by ``table`` ((cos, sin)[max_pos][64], or null); q to q_out [M, nq * 128], k and v to the token's
//   slot of the paged cache (write_cache != 0).  Heads of 128 only; bfloat16 in and out.
TFF_API int tff_gemm_tc_qkv_rope(const void* A, const void* W, int M, int K, void* q_out, const float* q_w, const float* k_w,
                                 float eps, const float* table, int max_pos, const int* positions, const int* tok_req,
                                 const int* block_table, int table_width, void* cache, int cache_layers, int layer,
                                 int page_size, int write_cache, int nq, int nkv, cudaStream_t stream) {
    if (M <= 0) return TFF_OK;
    if (K <= 0 || nq <= 0 || nkv <= 0 || positions == nullptr || q_out == nullptr) return TFF_ERR_BAD_ARGUMENT;
    if (write_cache && (cache == nullptr || block_table == nullptr || tok_req == nullptr || page_size <= 0)) return TFF_ERR_BAD_ARGUMENT;
    if (K % 8 != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)q_out & 15) || ((uintptr_t)cache & 15) ||
        ((uintptr_t)q_w & 15) || ((uintptr_t)k_w & 15) || ((uintptr_t)table & 15))
        return TFF_ERR_UNSUPPORTED;
    if (tff_device_error_flag() == nullptr) return TFF_ERR_LAUNCH;
    const int N = (nq + 2 * nkv) * 128;
    CUtensorMap ta, tw;
    if (!tff_tensor_map_2d(A, M, K, BM, BK, 2, &ta)) return TFF_ERR_DRIVER;
    if (!tff_tensor_map_2d(W, N, K, 128, BK, 2, &tw)) return TFF_ERR_DRIVER;
    QkvEpilogue e;
    e.q_out = (bf16*)q_out; e.cache = (bf16*)cache; e.q_w = q_w; e.k_w = k_w; e.table = (const float2*)table;
    e.positions = positions; e.tok_req = tok_req; e.block_table = block_table;
    e.L = make_kv_layout(cache_layers, nkv, page_size > 0 ? page_size : 1, 128);
    e.eps = eps; e.table_width = table_width; e.layer = layer; e.write_cache = write_cache; e.nq = nq; e.nkv = nkv;
    e.T = M; e.max_pos = max_pos;
    return launch_pair<EPI_QKV, bf16>(ta, tw, ta, M, N, K, 0, stream, e);
}

int tff_gemm_tc_pair_launch(const CUtensorMap& tm_a, const CUtensorMap& tm_w_half, const CUtensorMap& tm_out, int epilogue,
                            int out_is_bf16, int M, int N, int K, int stream_k, cudaStream_t stream) {
    if (tff_device_error_flag() == nullptr) return TFF_ERR_LAUNCH;
    if (epilogue == EPI_SWIGLU) return launch_pair<EPI_SWIGLU, bf16>(tm_a, tm_w_half, tm_out, M, N, K, 0, stream);
    if (out_is_bf16) {
        if (epilogue != EPI_STORE || stream_k) return TFF_ERR_BAD_ARGUMENT;
        return launch_pair<EPI_STORE, bf16>(tm_a, tm_w_half, tm_out, M, N, K, 0, stream);
    }
    if (epilogue == EPI_ADD) return launch_pair<EPI_ADD, float>(tm_a, tm_w_half, tm_out, M, N, K, stream_k, stream);
    return launch_pair<EPI_STORE, float>(tm_a, tm_w_half, tm_out, M, N, K, stream_k, stream);
}
