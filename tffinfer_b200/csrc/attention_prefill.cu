// Prompt-portion attention over the paged cache on the 5th-generation tensor cores.
//
// A CTA takes one or two tiles of 128 packed query rows (row R of a request = token R / G, head
// kvh*G + R % G) of one (request, kv head) and walks the keys in blocks of 64, once for its tiles.
// Per tile:
//   S = Q K^T     tcgen05.mma, M = 128, N = 64, K = head size; both operands K-major in
//                 128-byte-swizzled shared memory; S (float32) in tensor memory, two buffers
//   softmax       four warps, one thread per row: S row from TMEM, causal/window mask by
//                 position, running maximum and sum in float32, probabilities to shared memory
//                 as bfloat16 (K-major, swizzled: the A operand of the next product)
//   O += P V      tcgen05.mma, M = 128, N = head size, K = 64; V is the B operand in
//                 MN-major form, exactly as TMA lays the pages down; O (float32) stays in
//                 tensor memory for the whole key walk
// O is rescaled only when a row's maximum has grown by more than 2^8 since the value the
// exponentials use (the probabilities then stay below 2^8, harmless in float32/bfloat16), so
// the read-modify-write of O in tensor memory is rare.
//   warp 0      TMA producer: one box per (page, 64-column half, K or V) into a ring of stages
//   warp 1      TMEM allocation (all 512 columns: O and two S buffers per tile), MMA issue (one lane)
//   warps 2-5   softmax, rescale, epilogue of the first tile (TMEM lane quarter = warp % 4)
//   warps 6-9   the same for the second tile
// What the schedule of the issuing thread rests on (measured on a B200): a product of this size
// occupies the tensor core for 48 (S, bound by the 6 KB of operands it reads from shared memory)
// or 64 cycles (PV), and issuing blocks while the one before runs; a run of products that starts
// on an idle tensor core costs about 175 cycles extra, and a barrier wait in between costs the
// thread 100 cycles and more.  So the thread waits on one barrier per key block (the probabilities
// of block j of its tiles; a softmax warp has looked after the keys of block j + 2) and then issues
// PV(j) and S(j + 2) for its tiles in one run; the softmax warps find S(j + 1) finished when they
// have written P(j), and with two tiles a CTA the run is twice as long for the same wait.
// CTAs are handed out longest walk first over all kv heads.
// Same contract as the rows mode of attention_bf16.cu, which it replaces when the page size
// is 8/16/32/64.  Every mbarrier wait is bounded; a timeout raises the library's error word.
// Every wait lets the hardware suspend the warp: the waiting warps share their schedulers with the softmax warps
// of the other tile, and polled they took issue slots from those (5 % of the kernel's time).
#define TFF_SUSPENDED_WAITS
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
using tc5::tma_load_2d;
using tc5::fence_async_smem;
using tc5::tmem_alloc;
using tc5::tmem_dealloc;
using tc5::umma_bf16;
using tc5::umma_commit;
using tc5::tc_fence_before;
using tc5::tc_fence_after;
using tc5::tmem_ld16;
using tc5::tmem_ld_wait;


constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 64;
constexpr int NSTAGES = 4;
constexpr float RESCALE_THRESHOLD = 8.0f;       // in log2 units

// the same for a whole warp: every lane gets the same answer
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}
// 2^x on the special-function unit (float32 in and out; 2^-inf = 0)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart.  ``lbo_bytes`` is
// the distance between successive 64-element blocks along the M/N extent of an MN-major operand
// (not used by K-major operands).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: float32 accumulate, bfloat16 operands, A K-major; B K-major or MN-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct PrefillParams {
    const bf16* q; int q_row_stride;
    const int* q_start; const int* pos_start; const int* req_ids;
    const int* block_table; int table_width;
    int cache_layers, layer, page_shift;
    bf16* out;
    int nq, nkv; float scale_log2; int window;
    int* error_flag;
};

// QT: query tiles per CTA.  Two when that still gives every SM a CTA, one otherwise.
template <int D, int QT>
__global__ void __launch_bounds__(64 + QT * 128, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_cache, const PrefillParams p) {
    constexpr int HF = D / 64;                                   // 64-column halves of a head
    constexpr int CH = D / 8;                                    // 16-byte chunks per row
    constexpr int KV_BYTES = BLOCK_N * D * 2;                    // K (or V) of one stage: [half][64 keys][128 B]
    constexpr int STAGE_BYTES = 2 * KV_BYTES;
    constexpr int Q_BYTES = BLOCK_M * D * 2;                     // one query tile: [half][128 rows][128 B]
    constexpr int P_BYTES = BLOCK_M * BLOCK_N * 2;               // one tile's probabilities: [128 rows][128 B]
    constexpr int TMEM_COLS = 512;                               // O of tile x at 128 x; S buffers at 256 + 128 x + 64 sb
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sQ = base + NSTAGES * STAGE_BYTES;            // two query tiles
    const uint32_t sP = sQ + QT * Q_BYTES;                       // one buffer per tile
    const uint32_t bars = sP + QT * P_BYTES;
    uint8_t* gQ = gbase + NSTAGES * STAGE_BYTES;
    uint8_t* gP = gQ + QT * Q_BYTES;
    // barriers: kv_full[NS], kv_empty[NS], p_full; per tile x: s_full[2], pv_done, q_ready
    auto kv_full = [&](int s) { return bars + 8u * s; };
    auto kv_empty = [&](int s) { return bars + 8u * (NSTAGES + s); };
    const uint32_t p_full = bars + 8u * (2 * NSTAGES);            // the probabilities of a block, of all tiles of the CTA
    auto s_full = [&](int x, int b) { return bars + 8u * (2 * NSTAGES + 1 + 4 * x + b); };
    auto pv_done = [&](int x) { return bars + 8u * (2 * NSTAGES + 1 + 4 * x + 2); };
    auto q_ready = [&](int x) { return bars + 8u * (2 * NSTAGES + 1 + 4 * x + 3); };
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gP + QT * P_BYTES + 8 * (2 * NSTAGES + 1 + 4 * QT));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // CTAs are handed out in the order x, y, z: all kv heads of the last rows (which see the most keys)
    // first, the shortest walks last, so that the SMs finish together
    const int kvh = blockIdx.x;
    const int pair = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int G = p.nq / p.nkv;
    const int ps = 1 << p.page_shift;

    if (tid == 0) {
        for (int s = 0; s < NSTAGES; ++s) { mbar_init(kv_full(s), 1); mbar_init(kv_empty(s), 1); }
        for (int x = 0; x < QT; ++x) {
            mbar_init(s_full(x, 0), 1); mbar_init(s_full(x, 1), 1);
            mbar_init(pv_done(x), 1); mbar_init(q_ready(x), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_cache) : "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    // request geometry (q_start and pos_start come with the step's batch, read after the dependency wait all the same)
    const int b = p.req_ids ? p.req_ids[blockIdx.z] : (int)blockIdx.z;
    const int q0 = p.q_start[b];
    const int q_len = p.q_start[b + 1] - q0;
    const int rows_total = q_len * G;
    const int row0 = pair * QT * BLOCK_M;                         // first packed row of the CTA
    const bool active = row0 < rows_total;                        // uniform over the CTA
    const int n_act = !active ? 0 : (row0 + BLOCK_M < rows_total ? QT : 1);   // query tiles of the CTA that have rows
    const int pos0 = p.pos_start[b];
    const int first_tok = row0 / G;
    const int last_tok = min(q_len - 1, (row0 + QT * BLOCK_M - 1) / G);
    const int hi = pos0 + last_tok;                               // last key any row of the CTA sees
    const int lo_cta = p.window > 0 ? max(0, pos0 + first_tok - p.window + 1) : 0;   // first key any row sees
    const int kb_lo = lo_cta / BLOCK_N, kb_hi = hi / BLOCK_N;
    const int nb = active ? kb_hi - kb_lo + 1 : 0;
    const int* table = p.block_table + (size_t)b * p.table_width;
    // the issuing thread waits on ONE barrier per key block: the four softmax warps of every tile that has
    // rows arrive there, the first of them only after it has also seen the keys of block j + 2 land
    if (tid == 0) {
        mbar_init(p_full, 4u * (uint32_t)(n_act > 0 ? n_act : 1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        const int ppb = BLOCK_N >> p.page_shift;
        const int nloads = ppb * HF * 2;                          // boxes per stage (<= 32)
        const int j = lane / (HF * 2), rem = lane % (HF * 2);
        const int kv = rem / HF, hf = rem % HF;
        for (int i = 0; i < nb; ++i) {
            const int s = i % NSTAGES;
            const uint32_t round = i / NSTAGES;
            bool ok = true;
            if (round > 0) {
                if (lane == 0) ok = mbar_wait(kv_empty(s), (round - 1) & 1, abort_flag);
                ok = __shfl_sync(0xffffffffu, ok, 0);
            }
            if (!ok) break;
            const int n0 = (kb_lo + i) * BLOCK_N + (j << p.page_shift);
            int page = -1;
            if (lane < nloads && n0 <= hi) page = table[n0 >> p.page_shift];
            const bool valid = page >= 0;
            const unsigned mask = __ballot_sync(0xffffffffu, valid);
            if (lane == 0) mbar_expect_tx(kv_full(s), (uint32_t)__popc(mask) * (uint32_t)(ps * 128));
            __syncwarp();
            if (valid) {
                const long long row = ((((long long)page * p.cache_layers + p.layer) * 2 + kv) * p.nkv + kvh) << p.page_shift;
                // stage layout: K then V, each [half][64 keys][128 B]
                const uint32_t dst = base + s * STAGE_BYTES + kv * KV_BYTES + hf * (BLOCK_N * 128) +
                                     (uint32_t)((j << p.page_shift) * 128);
                tma_load_2d(dst, &tm_cache, kv_full(s), hf * 64, (int)row);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        // Starting a run of products after the tensor core has gone idle costs about 175 cycles, so the
        // thread waits once per key block and then issues one long run: O_x += P_x(j) V_j for both tiles,
        // then S_x(j+2) = Q_x K_(j+2)^T for both.  S runs two blocks ahead of the softmax (two S buffers
        // per tile), so a tile's softmax warps find their next scores finished when they have written a
        // block's probabilities.  S_x(j+2) overwrites the buffer of S_x(j), which the softmax warps have
        // read before they announce P_x(j).
        if (lane == 0 && nb > 0) {
            constexpr uint32_t idesc_s = make_idesc(BLOCK_M, BLOCK_N, 0);
            constexpr uint32_t idesc_pv = make_idesc(BLOCK_M, D, 1);
            bool ok = true;
            for (int x = 0; x < n_act && ok; ++x) ok = mbar_wait(q_ready(x), 0, abort_flag);
            // descriptors are built once; a product costs one 64-bit add on each (the low bits of a
            // descriptor are the shared-memory address in units of 16 bytes)
            const uint64_t qdesc = make_smem_desc(sQ, 16);                         // + x * Q_BYTES
            const uint64_t kdesc = make_smem_desc(base, 16);                       // + stage * STAGE_BYTES
            const uint64_t vdesc = make_smem_desc(base + KV_BYTES, BLOCK_N * 128); // + stage * STAGE_BYTES
            const uint64_t pdesc = make_smem_desc(sP, 16);                         // + x * P_BYTES
            auto issue_s = [&](int jj) {                           // S_x(jj) for both tiles; K_jj has landed
                const int sb = jj & 1;
                const uint64_t kd = kdesc + (uint64_t)((jj % NSTAGES) * (STAGE_BYTES >> 4));
#pragma unroll
                for (int x = 0; x < QT; ++x) {
                    if (x < n_act) {
                        const uint64_t qd = qdesc + (uint64_t)(x * (Q_BYTES >> 4));
#pragma unroll
                        for (int kk = 0; kk < D / 16; ++kk) {
                            // Q: [half][128 rows][128 B], K: [half][64 keys][128 B]; 16 elements = 32 bytes along a row
                            const uint32_t qoff = ((kk / 4) * (BLOCK_M * 128) + (kk % 4) * 32) >> 4;
                            const uint32_t koff = ((kk / 4) * (BLOCK_N * 128) + (kk % 4) * 32) >> 4;
                            umma_bf16(tmem_base + 256 + x * 128 + sb * 64, qd + qoff, kd + koff, idesc_s, kk > 0 ? 1u : 0u);
                        }
                        umma_commit(s_full(x, sb));
                    }
                }
            };
            for (int jj = 0; jj < 2 && jj < nb && ok; ++jj) {
                ok = mbar_wait(kv_full(jj), 0, abort_flag);
                if (ok) { tc_fence_after(); issue_s(jj); }
            }
            for (int j = 0; j < nb && ok; ++j) {
                const int st = j % NSTAGES;
                ok = mbar_wait(p_full, j & 1, abort_flag);         // P_x(j) of every tile, and K, V of block j + 2
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = vdesc + (uint64_t)(st * (STAGE_BYTES >> 4));
#pragma unroll
                for (int x = 0; x < QT; ++x) {
                    if (x < n_act) {
                        const uint64_t pd = pdesc + (uint64_t)(x * (P_BYTES >> 4));
#pragma unroll
                        for (int kk = 0; kk < BLOCK_N / 16; ++kk)
                            umma_bf16(tmem_base + x * 128, pd + (uint64_t)(kk * 2), vd + (uint64_t)(kk * 128), idesc_pv,
                                      kk > 0 ? 1u : (j > 0 ? 1u : 0u));
                        umma_commit(pv_done(x));                   // O_x holds block j; the tile's P buffer is free
                    }
                }
                umma_commit(kv_empty(st));                         // K and V of the stage have been read
                if (j + 2 < nb) issue_s(j + 2);
            }
        }
    } else {
        // ------------------------------------------------- softmax / rescale / epilogue
        const int x = (warp - 2) >> 2;                             // query tile of this warp
        const int q = warp & 3;                                    // TMEM lane quarter this warp may touch
        const int r = q * 32 + lane;                               // row of the tile = TMEM lane
        const int R = row0 + x * BLOCK_M + r;
        const bool tile_active = x < n_act;
        const bool rv = tile_active && R < rows_total;
        const int pr = pos0 + R / G;
        const int lo_r = p.window > 0 ? max(0, pr - p.window + 1) : 0;
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t t_o = t_row + x * 128;
        // the query tile: this thread's row, 16-byte chunks XOR-swizzled by row % 8, one [128 x 128 B] block per half
        if (tile_active) {
            const bf16* src = p.q + (size_t)(q0 + R / G) * p.q_row_stride + (size_t)(kvh * G + R % G) * D;
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (rv) v = *reinterpret_cast<const uint4*>(src + c * 8);
                *reinterpret_cast<uint4*>(gQ + x * Q_BYTES + (c >> 3) * (BLOCK_M * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready(x));
        }
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        const int nb_x = tile_active ? nb : 0;
        for (int j = 0; j < nb_x && ok; ++j) {
            const int sb = j & 1, st = j % NSTAGES;
            const int blk = kb_lo + j;
            if (x == 0 && (blk == kb_hi || blk == kb_lo)) {
                // value rows no query row of the CTA may see (beyond the last key, before the first window):
                // cleared by the warps of tile 0, since page slots and unfetched shared memory may hold anything.
                // The stage has landed first; the product that reads it waits for these warps' probabilities.
                ok = mbar_wait_warp(kv_full(st), (j / NSTAGES) & 1, abort_flag);
                if (!ok) break;
                uint8_t* gV = gbase + st * STAGE_BYTES + KV_BYTES;
                for (int idx = tid - 64; idx < BLOCK_N * CH; idx += 128) {
                    const int kr = idx / CH, c = idx % CH;
                    const int n = blk * BLOCK_N + kr;
                    if (n > hi || n < lo_cta)
                        *reinterpret_cast<uint4*>(gV + (c >> 3) * (BLOCK_N * 128) + kr * 128 + (((c & 7) ^ (kr & 7)) << 4)) =
                            make_uint4(0u, 0u, 0u, 0u);
                }
                fence_async_smem();
            }
            ok = mbar_wait_warp(s_full(x, sb), (j >> 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            float s[BLOCK_N];
#pragma unroll
            for (int h = 0; h < BLOCK_N / 16; ++h) {
                uint32_t v[16];
                tmem_ld16(t_row + 256 + x * 128 + sb * 64 + h * 16, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) s[h * 16 + i] = __uint_as_float(v[i]);
            }
            tc_fence_before();                                     // the scores are in registers (see the MMA issuer)
            // Scores stay unscaled in registers; the scale (> 0) is folded into the exponent below.  Key
            // blocks that every row of the warp sees whole need no mask.
            // (four running maxima and, below, four partial sums: chains of 16 dependent operations, not 64)
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            const int n_first = blk * BLOCK_N;
            if (__all_sync(0xffffffffu, rv && n_first + BLOCK_N - 1 <= pr && n_first >= lo_r)) {
#pragma unroll
                for (int i = 0; i < BLOCK_N; ++i) m4[i & 3] = fmaxf(m4[i & 3], s[i]);
            } else {
#pragma unroll
                for (int i = 0; i < BLOCK_N; ++i) {
                    const int n = n_first + i;
                    const bool vis = rv && n <= pr && n >= lo_r;
                    s[i] = vis ? s[i] : -INFINITY;
                    m4[i & 3] = fmaxf(m4[i & 3], s[i]);
                }
            }
            const float m_raw = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            const float m_blk = m_raw * p.scale_log2;
            // lazy rescale: only when the maximum has grown by more than the threshold (warp-uniform decision)
            const bool grow = m_blk > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && m_blk > -INFINITY);
            // O_x must hold every earlier block before it is rescaled, and the product of the block before
            // this one must have read the tile's P buffer before it is written again
            if (j > 0) {
                ok = mbar_wait_warp(pv_done(x), (j - 1) & 1, abort_flag);
                if (!ok) break;
            }
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? m_blk : m_used;
                const float alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
                if (j > 0) {
                    tc_fence_after();
#pragma unroll 1
                    for (int c0 = 0; c0 < D; c0 += 16) {
                        uint32_t v[16];
                        tmem_ld16(t_o + c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * (grow ? alpha : 1.f));
                        tmem_st16(t_o + c0, v);
                    }
                    tmem_st_wait();
                    tc_fence_before();
                }
                if (grow) { l *= alpha; m_used = m_new; }
            }
            const float ms = m_used == -INFINITY ? 0.f : m_used;
            uint8_t* prow = gP + x * P_BYTES + r * 128;
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float e0 = ex2_approx(fmaf(s[c * 8 + 2 * i], p.scale_log2, -ms));
                    const float e1 = ex2_approx(fmaf(s[c * 8 + 2 * i + 1], p.scale_log2, -ms));
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
                    l4[i] += e0 + e1;
                    w[i] = *reinterpret_cast<uint32_t*>(&b2);
                }
                *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            fence_async_smem();
            if (warp == 2 && j + 2 < nb) {                          // on behalf of the issuing thread
                ok = mbar_wait_warp(kv_full((j + 2) % NSTAGES), ((j + 2) / NSTAGES) & 1, abort_flag);
                if (!ok) break;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        // ---------------------------------------------------------------- epilogue
        if (ok && nb_x > 0) ok = mbar_wait_warp(pv_done(x), (nb_x - 1) & 1, abort_flag);
        if (ok && nb_x > 0) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* orow = p.out + ((size_t)(q0 + R / G) * p.nq + (kvh * G + R % G)) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(t_o + c0, v);
                tmem_ld_wait();
                if (rv) {
                    uint32_t w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[2 * i]) * inv, __uint_as_float(v[2 * i + 1]) * inv);
                        w[i] = *reinterpret_cast<uint32_t*>(&b2);
                    }
                    *reinterpret_cast<uint4*>(orow + c0) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(orow + c0 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
    }
    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if (tid == 0) atomicExch(p.error_flag, 1);
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int D, int QT>
int launch_prefill(const CUtensorMap& tm, const PrefillParams& p, int q_tiles, int B, cudaStream_t stream) {
    constexpr int NTHREADS = 64 + QT * 128;
    constexpr int smem = NSTAGES * 2 * BLOCK_N * D * 2 + QT * BLOCK_M * D * 2 + QT * BLOCK_M * BLOCK_N * 2 +
                         8 * (2 * NSTAGES + 1 + 4 * QT) + 16 + 1024;
    static_assert(smem <= 227 * 1024, "shared memory of the prompt attention kernel");
    auto kern = attn_prefill_tc_kernel<D, QT>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return TFF_ERR_LAUNCH;
        configured = true;
    }
    return tff_launch_pdl(kern, dim3(p.nkv, q_tiles, B), dim3(NTHREADS), (size_t)smem, stream, tm, p);
}

}  // namespace

// Prompt-portion attention on tcgen05.  TFF_ERR_UNSUPPORTED when the shape is not one it takes
// (head size 64/128, page size 8/16/32/64).
int tff_attention_prefill_launch(
    const void* q, const int* q_start, const int* pos_start, const int* req_ids, const int* block_table, int table_width,
    const void* cache, long long cache_pages, int cache_layers, int layer, int page_size,
    void* out, int num_requests, int max_q_len, int nq, int nkv, int d, float scale, int window, cudaStream_t stream) {
    if (d != 64 && d != 128) return TFF_ERR_UNSUPPORTED;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return TFF_ERR_UNSUPPORTED;
    if (cache_pages <= 0 || !(scale > 0.f)) return TFF_ERR_UNSUPPORTED;     // the kernel folds a positive scale into the exponent
    if (((uintptr_t)cache & 15) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || (nq * d) % 8) return TFF_ERR_UNSUPPORTED;
    const long long rows = cache_pages * cache_layers * 2 * nkv * page_size;
    if (rows >= (1ll << 31) || num_requests > 65535 || (long long)max_q_len * (nq / nkv) > 65535ll * 256) return TFF_ERR_UNSUPPORTED;
    CUtensorMap tm;
    if (!tff_tensor_map_2d(cache, rows, d, page_size, 64, 2, &tm)) return TFF_ERR_DRIVER;
    PrefillParams p;
    p.q = (const bf16*)q; p.q_row_stride = nq * d;
    p.q_start = q_start; p.pos_start = pos_start; p.req_ids = req_ids;
    p.block_table = block_table; p.table_width = table_width;
    p.cache_layers = cache_layers; p.layer = layer;
    p.page_shift = page_size == 8 ? 3 : page_size == 16 ? 4 : page_size == 32 ? 5 : 6;
    p.out = (bf16*)out;
    p.nq = nq; p.nkv = nkv; p.scale_log2 = scale * 1.4426950408889634f; p.window = window;
    p.error_flag = tff_device_error_flag();
    if (p.error_flag == nullptr) return TFF_ERR_LAUNCH;
    const int G = nq / nkv;
    const int tiles = (max_q_len * G + BLOCK_M - 1) / BLOCK_M;
    const int pairs = (tiles + 1) / 2;
    // Two query tiles a CTA share one walk over the keys (a pair costs about 1.7 times a single tile) but
    // halve the number of CTAs: whichever fills the SMs in fewer rounds, weighed by that cost.
    const long long sms = tff_num_sms() > 0 ? tff_num_sms() : 1;
    const long long rounds2 = ((long long)pairs * nkv * num_requests + sms - 1) / sms;
    const long long rounds1 = ((long long)tiles * nkv * num_requests + sms - 1) / sms;
    if (rounds2 * 17 < rounds1 * 10)
        return d == 128 ? launch_prefill<128, 2>(tm, p, pairs, num_requests, stream)
                        : launch_prefill<64, 2>(tm, p, pairs, num_requests, stream);
    return d == 128 ? launch_prefill<128, 1>(tm, p, tiles, num_requests, stream)
                    : launch_prefill<64, 1>(tm, p, tiles, num_requests, stream);
}
