// Decode attention over the paged cache: few query rows (one token, the query heads of one
// kv-head group packed into a 16-row tile) against a long run of keys, i.e. a stream of the
// cache through the SM.  Same contract and numerics as the keys mode of attention_bf16.cu;
// what differs is how the keys arrive:
//   warp 4      producer: one TMA box per page (its keys and values of the kv head, 8 KB with
//               16-token pages), issued by as many lanes as the block has pages, into a ring of
//               64-key stages guarded by mbarriers
//   warps 0-3   each takes 16 of the 64 keys of a stage: QK^T and PV on mma.sync m16n8k16,
//               float32 online softmax; the four partial results are merged through shared
//               memory at the end
// The cache is seen by TMA as a 4-D tensor (64 columns, head_dim/64 halves, rows, {K, V}) over the
// matrix [pages * layers * 2 * kv_heads * page_size, head_dim]; the 128-byte swizzle TMA applies is
// the one ldmatrix is then addressed with.
// Pages that are missing (given back by a sliding window, or beyond the sequence) are not
// fetched; value rows beyond the request's last key or before its window are cleared in shared
// memory, because a page's unused slots, and shared memory that was not written, may hold
// anything.
// Every mbarrier wait is bounded; when one runs out the CTA raises the library's error word.
#include "tcgen05.cuh"
#include "attention_common.h"

namespace {

// mbarrier, TMA and tensor-memory wrappers shared with the product kernels
using tc5::smem_u32;
using tc5::mbar_init;
using tc5::mbar_expect_tx;
using tc5::mbar_arrive;
using tc5::mbar_try_wait;
using tc5::mbar_wait;


constexpr int BLOCK_N = 64;
#ifndef TFF_DEC_STAGES
#define TFF_DEC_STAGES 3
#endif
#ifndef TFF_DEC_CTAS
#define TFF_DEC_CTAS 2
#endif
constexpr int NSTAGES = TFF_DEC_STAGES;
constexpr int NTHREADS = 160;

__device__ __forceinline__ void compute_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct DecodeParams {
    const bf16* q; int q_row_stride;
    const int* q_start; const int* pos_start; const int* req_ids;
    const int* block_table; int table_width;
    int cache_layers, layer, page_shift;         // page_size = 1 << page_shift
    bf16* out; float* part_o; float* part_ml; int num_splits;
    int nq, nkv; float scale_log2; int window;
    int* error_flag;
};

// Byte offset, inside a stage, of 16-byte chunk ``c`` of key row ``kr`` (0..63) of K (kv = 0) or V (kv = 1).
// A stage holds, page after page of the block, what one TMA box brings: [K | V][page_size rows][halves][128 B];
// the 16-byte chunks of every 128-byte line are XOR-swizzled by the line's index % 8 (TMA's 128-byte swizzle).
template <int D>
__device__ __forceinline__ uint32_t kv_off(int kr, int c, int kv, int page_shift) {
    constexpr int HF = D / 64;
    const int j = kr >> page_shift, r = kr & ((1 << page_shift) - 1);
    const int line = r * HF + (c >> 3);                          // 128-byte line inside the page's K (or V)
    return (uint32_t)((((j * 2 + kv) << page_shift) * HF + line) * 128 + ((((c & 7) ^ line) & 7) << 4));
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int x0, int x1, int x2, int x3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(x0), "r"(x1), "r"(x2), "r"(x3) : "memory");
}

template <int D>
__global__ void __launch_bounds__(NTHREADS, TFF_DEC_CTAS)
attn_decode_kernel(const __grid_constant__ CUtensorMap tm_cache, const DecodeParams p) {
    constexpr int CH = D / 8;
    constexpr int KV_BYTES = BLOCK_N * D * 2;                     // K (or V) of one stage
    constexpr int STAGE_BYTES = 2 * KV_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    // [ring: NSTAGES x (K | V)] [Q 16 x D] [barriers full[NSTAGES], empty[NSTAGES]] [abort]
    const uint32_t sQ = base + NSTAGES * STAGE_BYTES;
    uint8_t* gQ = gbase + NSTAGES * STAGE_BYTES;
    const uint32_t bars = sQ + 16 * D * 2;
    volatile int* abort_flag = (volatile int*)(gQ + 16 * D * 2 + 8 * 2 * NSTAGES);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (NSTAGES + s); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, split = blockIdx.x;
    const int G = p.nq / p.nkv;

    if (tid == 0) {
        for (int s = 0; s < NSTAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_cache) : "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    // What the kernel ahead wrote is the queries and the cache slots of the tokens this step brings; the
    // step's batch arrays and the keys of earlier steps are older.  The producer therefore asks for its
    // first stages before it waits for that kernel, the compute warps wait before they read the queries.

    const int b = p.req_ids ? p.req_ids[blockIdx.z] : (int)blockIdx.z;
    const int q0 = p.q_start[b];
    const int q_len = p.q_start[b + 1] - q0;
    const int rows_total = q_len * G;                              // <= 16 by the launcher's choice
    const int pos0 = p.pos_start[b];
    const int hi = pos0 + q_len - 1;
    const int lo_tile = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int kb_lo = lo_tile / BLOCK_N, kb_hi = hi / BLOCK_N;
    const int nblk = kb_hi - kb_lo + 1;
    const int per = (nblk + p.num_splits - 1) / p.num_splits;
    const int kb_begin = kb_lo + split * per;
    const int kb_end = min(kb_hi + 1, kb_begin + per);             // may be <= kb_begin: an empty split
    const int* table = p.block_table + (size_t)b * p.table_width;

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        const int ppb = BLOCK_N >> p.page_shift;                   // pages per 64-key block = boxes per stage (<= 8)
        const int j = lane;
        const uint32_t box_bytes = (uint32_t)(2 * D * 2) << p.page_shift;      // K and V of one page
        const int first_new_blk = pos0 / BLOCK_N;                  // key blocks from here on hold slots written just now
        bool waited = false;
        for (int blk = kb_begin; blk < kb_end; ++blk) {
            const int i = blk - kb_begin, s = i % NSTAGES;
            const uint32_t round = i / NSTAGES;
            bool ok = true;
            if (!waited && (blk >= first_new_blk || round > 0)) { pdl_wait(); waited = true; }
            if (round > 0) {
                if (lane == 0) ok = mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag);
                ok = __shfl_sync(0xffffffffu, ok, 0);
            }
            if (!ok) break;
            const int n0 = blk * BLOCK_N + (j << p.page_shift);
            int page = -1;
            if (lane < ppb && n0 <= hi) page = table[n0 >> p.page_shift];
            const bool valid = page >= 0;
            const unsigned mask = __ballot_sync(0xffffffffu, valid);
            if (lane == 0) mbar_expect_tx(full_bar(s), (uint32_t)__popc(mask) * box_bytes);
            __syncwarp();
            if (valid) {
                // first K row of (page, layer, kv head) in the cache seen as [rows, D]; the box brings its V too
                const long long row = (((long long)page * p.cache_layers + p.layer) * 2 * p.nkv + kvh) << p.page_shift;
                tma_load_4d(base + s * STAGE_BYTES + (uint32_t)j * box_bytes, &tm_cache, full_bar(s), 0, 0, (int)row, 0);
            }
        }
        return;
    }

    // ---------------------------------------------------------------- compute warps
    pdl_wait();
    // the query tile: packed rows (token, head of the group), chunks XOR-swizzled by row % 8
    for (int idx = tid; idx < 16 * CH; idx += 128) {
        const int row = idx / CH, chunk = idx % CH;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < rows_total)
            v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + row / G) * p.q_row_stride +
                                                (size_t)(kvh * G + row % G) * D + chunk * 8);
        *reinterpret_cast<uint4*>(gQ + row * (D * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4)) = v;
    }
    compute_barrier();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int chunk = kk * 2 + (lane >> 4);
        ldsm_x4(sQ + row * (D * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }

    const int key_off = warp * 16;
    const int r0 = lane >> 2, r1 = r0 + 8;
    const bool v0 = r0 < rows_total, v1 = r1 < rows_total;
    const int pr0 = pos0 + r0 / G, pr1 = pos0 + r1 / G;
    const int lo0 = p.window > 0 ? max(0, pr0 - p.window + 1) : 0;
    const int lo1 = p.window > 0 ? max(0, pr1 - p.window + 1) : 0;

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int blk = kb_begin; blk < kb_end; ++blk) {
        const int i = blk - kb_begin, s = i % NSTAGES;
        const uint32_t round = i / NSTAGES;
        if (!mbar_wait(full_bar(s), round & 1, abort_flag)) break;
        const uint32_t tS = base + s * STAGE_BYTES;
        if (blk == kb_hi || blk == kb_lo) {
            // This warp's value rows that no query row may see -- beyond the last key, or before
            // the window -- are cleared: their page slots may hold anything, and pages that were
            // not fetched leave whatever shared memory held.  (Such key rows only produce scores
            // that the mask discards.)
            uint8_t* gS = gbase + s * STAGE_BYTES;
            for (int idx = lane; idx < 16 * CH; idx += 32) {
                const int kr = key_off + idx / CH, c = idx % CH;
                const int n = blk * BLOCK_N + kr;
                if (n > hi || n < lo_tile)
                    *reinterpret_cast<uint4*>(gS + kv_off<D>(kr, c, 1, p.page_shift)) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        }
        // ------------------------------------------------------ S = Q K^T (16 rows x this warp's 16 keys)
        float sc[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t) { sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int kr = key_off + (lane & 7) + (lane >> 4) * 8;
            const int chunk = kk * 2 + ((lane >> 3) & 1);
            uint32_t b0, b1, b2, b3;
            ldsm_x4(tS + kv_off<D>(kr, chunk, 0, p.page_shift), b0, b1, b2, b3);
            mma_bf16(sc[0], qf[kk], b0, b1);
            mma_bf16(sc[1], qf[kk], b2, b3);
        }
        // ------------------------------------------- mask, online softmax
        const int nbase = blk * BLOCK_N + key_off + 2 * (lane & 3);
        float bm0 = -INFINITY, bm1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int n = nbase + nt * 8 + (e & 1);
                const bool up = e < 2;
                const bool ok = up ? (v0 && n <= pr0 && n >= lo0) : (v1 && n <= pr1 && n >= lo1);
                const float x = ok ? sc[nt][e] * p.scale_log2 : -INFINITY;
                sc[nt][e] = x;
                if (up) bm0 = fmaxf(bm0, x); else bm1 = fmaxf(bm1, x);
            }
        }
        bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 1)); bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 2));
        bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 1)); bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 2));
        const float mn0 = fmaxf(m0, bm0), mn1 = fmaxf(m1, bm1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float a0 = exp2f(m0 - ms0), a1 = exp2f(m1 - ms1);
        m0 = mn0; m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            sc[nt][0] = exp2f(sc[nt][0] - ms0); sc[nt][1] = exp2f(sc[nt][1] - ms0);
            sc[nt][2] = exp2f(sc[nt][2] - ms1); sc[nt][3] = exp2f(sc[nt][3] - ms1);
            ps0 += sc[nt][0] + sc[nt][1];
            ps1 += sc[nt][2] + sc[nt][3];
        }
        l0 = l0 * a0 + ps0;
        l1 = l1 * a1 + ps1;
#pragma unroll
        for (int i2 = 0; i2 < D / 8; ++i2) { o[i2][0] *= a0; o[i2][1] *= a0; o[i2][2] *= a1; o[i2][3] *= a1; }
        // -------------------------------------------------------- O += P V
        uint32_t a[4];
        a[0] = pack_bf16(sc[0][0], sc[0][1]);
        a[1] = pack_bf16(sc[0][2], sc[0][3]);
        a[2] = pack_bf16(sc[1][0], sc[1][1]);
        a[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
        for (int dn = 0; dn < D / 16; ++dn) {
            const int kr = key_off + (lane & 7) + ((lane >> 3) & 1) * 8;
            const int chunk = dn * 2 + (lane >> 4);
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(tS + kv_off<D>(kr, chunk, 1, p.page_shift), b0, b1, b2, b3);
            mma_bf16(o[2 * dn], a, b0, b1);
            mma_bf16(o[2 * dn + 1], a, b2, b3);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(s));          // this warp is done with the stage
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    compute_barrier();                                     // every warp has finished reading the ring
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);    // copies in flight land before the CTA leaves
        if (tid == 0) atomicExch(p.error_flag, 1);
        return;
    }
    // ---------------------------------------------- merge the four warps through shared memory
    float* mO = reinterpret_cast<float*>(gbase);           // [4][16][D] floats: 256 * D bytes <= one stage
    float* mM = reinterpret_cast<float*>(gbase + STAGE_BYTES);
    float* mL = mM + 64;
    if ((lane & 3) == 0) {
        mM[warp * 16 + r0] = m0; mM[warp * 16 + r1] = m1;
        mL[warp * 16 + r0] = l0; mL[warp * 16 + r1] = l1;
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int c = i * 8 + 2 * (lane & 3);
        *reinterpret_cast<float2*>(&mO[(warp * 16 + r0) * D + c]) = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2*>(&mO[(warp * 16 + r1) * D + c]) = make_float2(o[i][2], o[i][3]);
    }
    compute_barrier();
    for (int idx = tid; idx < 16 * D; idx += 128) {
        const int r = idx / D, c = idx % D;
        if (r >= rows_total) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mM[w * 16 + r]);
        const float Ms = M == -INFINITY ? 0.f : M;
        float acc = 0.f, lsum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = exp2f(mM[w * 16 + r] - Ms);
            acc += f * mO[(w * 16 + r) * D + c];
            lsum += f * mL[w * 16 + r];
        }
        const size_t grow = (size_t)(q0 + r / G) * p.nq + (kvh * G + r % G);
        if (p.num_splits == 1) {
            p.out[grow * D + c] = __float2bfloat16_rn(acc / lsum);
        } else {
            p.part_o[(grow * p.num_splits + split) * D + c] = acc;
            if (c == 0) {
                p.part_ml[(grow * p.num_splits + split) * 2] = M;
                p.part_ml[(grow * p.num_splits + split) * 2 + 1] = lsum;
            }
        }
    }
}

template <int D>
int launch_decode(const CUtensorMap& tm, const DecodeParams& p, int B, cudaStream_t stream) {
    constexpr int smem = NSTAGES * 2 * BLOCK_N * D * 2 + 16 * D * 2 + 8 * 2 * NSTAGES + 16 + 1024;
    auto kern = attn_decode_kernel<D>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return TFF_ERR_LAUNCH;
        configured = true;
    }
    return tff_launch_pdl(kern, dim3(p.num_splits, p.nkv, B), dim3(NTHREADS), (size_t)smem, stream, tm, p);
}

}  // namespace

// Launches the decode kernel (without the merge of the splits).  TFF_ERR_UNSUPPORTED when the
// shape is not one it takes (head size 64/128, page size 8/16/32/64, at most 16 packed rows).
int tff_attention_decode_launch(
    const void* q, const int* q_start, const int* pos_start, const int* req_ids, const int* block_table, int table_width,
    const void* cache, long long cache_pages, int cache_layers, int layer, int page_size,
    void* out, float* part_o, float* part_ml, int num_requests, int max_q_len, int num_splits,
    int nq, int nkv, int d, float scale, int window, cudaStream_t stream) {
    if (d != 64 && d != 128) return TFF_ERR_UNSUPPORTED;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return TFF_ERR_UNSUPPORTED;
    if ((long long)max_q_len * (nq / nkv) > 16 || cache_pages <= 0) return TFF_ERR_UNSUPPORTED;
    if (((uintptr_t)cache & 15) || ((uintptr_t)q & 15) || (nq * d) % 8) return TFF_ERR_UNSUPPORTED;
    const long long rows = cache_pages * cache_layers * 2 * nkv * page_size;
    if (rows >= (1ll << 31)) return TFF_ERR_UNSUPPORTED;
    CUtensorMap tm;
    if (!tff_tensor_map_kv_page(cache, rows, d, page_size, nkv, &tm)) return TFF_ERR_DRIVER;
    DecodeParams p;
    p.q = (const bf16*)q; p.q_row_stride = nq * d;
    p.q_start = q_start; p.pos_start = pos_start; p.req_ids = req_ids;
    p.block_table = block_table; p.table_width = table_width;
    p.cache_layers = cache_layers; p.layer = layer;
    p.page_shift = page_size == 8 ? 3 : page_size == 16 ? 4 : page_size == 32 ? 5 : 6;
    p.out = (bf16*)out; p.part_o = part_o; p.part_ml = part_ml; p.num_splits = num_splits;
    p.nq = nq; p.nkv = nkv; p.scale_log2 = scale * 1.4426950408889634f; p.window = window;
    p.error_flag = tff_device_error_flag();
    if (p.error_flag == nullptr) return TFF_ERR_LAUNCH;
    return d == 128 ? launch_decode<128>(tm, p, num_requests, stream) : launch_decode<64>(tm, p, num_requests, stream);
}
