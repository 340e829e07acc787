// Prompt-portion attention over the paged cache on the 5th-generation tensor cores.
//
// A CTA takes one or two tiles of 128 packed query rows (row R of a request = token R / G, head
// kvh*G + R % G) of one (request, kv head) and walks the keys in blocks of 64, once for its tiles.
// Per tile:
//   S = Q K^T     tcgen05.mma, M = 128, N = 64, K = head size; Q is the A operand in TENSOR MEMORY
//                 (written there once by the tile's warps), K the B operand, K-major in
//                 128-byte-swizzled shared memory; S (float32) in tensor memory, one buffer
//   softmax       four warps, one thread per row: S row from TMEM (the buffer is given back as soon
//                 as the row is in registers), causal/window mask by position, running maximum and
//                 sum in float32, probabilities to shared memory as bfloat16 (K-major, swizzled:
//                 the A operand of the next product)
//   O += P V      tcgen05.mma, M = 128, N = head size, K = 64; V is the B operand in
//                 MN-major form, exactly as TMA lays the pages down; O (float32) stays in
//                 tensor memory for the whole key walk
// O is rescaled only when a row's maximum has grown by more than 2^8 since the value the
// exponentials use (the probabilities then stay below 2^8, harmless in float32/bfloat16), so
// the read-modify-write of O in tensor memory is rare.
//   warp 0      TMA producer: one box per (page, 64-column half, K or V) into a ring of stages
//   warp 1      TMEM allocation (512 columns: O of tile x at 128 x, S at 256 + 64 x, Q at 384 + 64 x);
//               issues the products of tile 0 (one lane)
//   warps 2-5   softmax, rescale, epilogue of the first tile (TMEM lane quarter = warp % 4)
//   warps 6-9   the same for the second tile
//   warp 10     issues the products of the second tile (one lane)
// What the schedule rests on (measured on a B200 with probes that only issue products): a
// 128 x 64 x 16 product with both operands in shared memory occupies the tensor core for 48 cycles
// (it reads 6 KB at 128 B/cycle), with A in tensor memory for the 32 its arithmetic takes; the PV
// product takes 64.  Issuing blocks while the product before runs, and a barrier wait by an issuing
// thread leaves the tensor core idle for 100-175 cycles unless another thread has products queued:
// so each tile has an issuing thread of its own (two threads keep the tensor core full, measured),
// and a tile's thread issues S(j + 1) as soon as the softmax warps have read S(j) into registers,
// PV(j) when they have written P(j).  S(j + 1) is therefore finished long before the softmax of
// block j is, and one S buffer a tile is enough; the columns that a second buffer took hold Q.
// P has two buffers a tile, so that the softmax of block j does not wait for PV(j - 1).
// With the products cheaper the kernel is bound by the exponentials: the special-function unit gives
// 16 a cycle and SM, a 64-key block of two tiles needs 1,024 cycles of it.  Left alone the two
// tiles fall into step (both in their exponential pass, each at half speed; then both in the rest of
// the loop with the unit idle), so the two warps that share a scheduler (the same lane quarter of
// the two tiles) take their exponential passes in turn, handing over through an mbarrier: one
// tile's waits, loads and maxima then run under the other tile's exponentials (8,192 tokens:
// 615 -> 547 us; with scale, subtraction and row sum on pairs of float32, fma.f32x2: 525).
// A cubic on the FMA pipe for part of the exponentials made it slower at every share tried.
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
constexpr int NSTAGES = 5;
#ifndef TURN_AFTER
#define TURN_AFTER 8          // of the 8 chunks of a block's exponentials, after which the other tile may begin its own
#endif
constexpr int BARS_PER_TILE = 7;
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
// The A operand from tensor memory (lane = row, one 32-bit column = two consecutive K elements), B from shared memory.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// Pairs of float32 in a 64-bit register: fma and add on a pair issue as one instruction on sm_100.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// maximum of three (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

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

#ifdef AP_TIMERS
__device__ long long ap_dbg[64];
#define AP_T(var) const long long var = clock64()
#define AP_ACC(slot, a, b) do { if (dbg_on) ap_dbg[slot] += (b) - (a); } while (0)
#else
#define AP_T(var)
#define AP_ACC(slot, a, b)
#endif

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
__global__ void __launch_bounds__(QT == 2 ? 352 : 192, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_cache, const PrefillParams p) {
    constexpr int HF = D / 64;                                   // 64-column halves of a head
    constexpr int CH = D / 8;                                    // 16-byte chunks per row
    constexpr int KV_BYTES = BLOCK_N * D * 2;                    // K (or V) of one stage: [half][64 keys][128 B]
    constexpr int STAGE_BYTES = 2 * KV_BYTES;
    constexpr int P_BYTES = BLOCK_M * BLOCK_N * 2;               // one tile's probabilities: [128 rows][128 B]
    constexpr int TMEM_COLS = 512;
    constexpr int NBARS = 2 * NSTAGES + BARS_PER_TILE * QT + 8;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sP = base + NSTAGES * STAGE_BYTES;            // two buffers per tile: [tile][block % 2]
    const uint32_t bars = sP + QT * 2 * P_BYTES;
    uint8_t* gP = gbase + NSTAGES * STAGE_BYTES;
    // barriers: kv_full[NS], kv_empty[NS]; per tile x: s_full, s_free, p_full[0], pv_done[2], q_ready, p_full[1]
    auto kv_full = [&](int s) { return bars + 8u * s; };
    auto kv_empty = [&](int s) { return bars + 8u * (NSTAGES + s); };
    auto s_full = [&](int x) { return bars + 8u * (2 * NSTAGES + BARS_PER_TILE * x); };
    auto s_free = [&](int x) { return bars + 8u * (2 * NSTAGES + BARS_PER_TILE * x + 1); };
    // P(j) reports to p_full(x, j % 2).  With one barrier a warp that took the short, unmasked path through two
    // blocks could arrive for block j + 1 before a warp on the masked path had arrived for block j, and PV(j)
    // went out with that warp's rows of P unwritten; a warp cannot be two blocks ahead (S(j + 2) is issued only
    // when every warp has read S(j + 1)), so two barriers taken in turn are enough.
    auto p_full = [&](int x, int b) { return bars + 8u * (2 * NSTAGES + BARS_PER_TILE * x + 2 + 4 * b); };
    // PV(j) reports to pv_done(x, j % 2): a waiter is then never more than one completion behind the barrier
    // it looks at, which a parity wait needs
    auto pv_done = [&](int x, int b) { return bars + 8u * (2 * NSTAGES + BARS_PER_TILE * x + 3 + b); };
    auto q_ready = [&](int x) { return bars + 8u * (2 * NSTAGES + BARS_PER_TILE * x + 5); };
    // whose turn it is at the special-function unit: the warps of the two tiles that share a scheduler (the same
    // lane quarter) take their exponential passes in turn
    auto turn = [&](int x, int q) { return bars + 8u * (2 * NSTAGES + BARS_PER_TILE * QT + 4 * x + q); };
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gP + QT * 2 * P_BYTES + 8 * NBARS);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // CTAs are handed out in the order x, y, z: all kv heads of the last rows (which see the most keys)
    // first, the shortest walks last, so that the SMs finish together
    const int kvh = blockIdx.x;
    const int pair = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int G = p.nq / p.nkv;
    const int ps = 1 << p.page_shift;

    if (tid == 0) {
        for (int s = 0; s < NSTAGES; ++s) mbar_init(kv_full(s), 1);
        for (int x = 0; x < QT; ++x) {
            mbar_init(s_full(x), 1); mbar_init(s_free(x), 4); mbar_init(p_full(x, 0), 4); mbar_init(p_full(x, 1), 4);
            mbar_init(pv_done(x, 0), 1); mbar_init(pv_done(x, 1), 1); mbar_init(q_ready(x), 4);
        }
        for (int i = 0; i < 8; ++i) mbar_init(turn(i >> 2, i & 3), 1);
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
    // a stage is free again when the PV products of every tile that has rows have read it
    if (tid == 0) {
        for (int s = 0; s < NSTAGES; ++s) mbar_init(kv_empty(s), (uint32_t)(n_act > 0 ? n_act : 1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int q = 0; q < 4; ++q) mbar_arrive(turn(0, q));      // the first tile begins
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
    } else if (warp == 1 || warp == 10) {
        // -------------------------------------------------------------- MMA issuers, one per tile
        const int x = warp == 1 ? 0 : 1;
        if (lane == 0 && x < n_act && nb > 0) {
            constexpr uint32_t idesc_s = make_idesc(BLOCK_M, BLOCK_N, 0);
            constexpr uint32_t idesc_pv = make_idesc(BLOCK_M, D, 1);
            const uint32_t t_o = tmem_base + x * 128, t_s = tmem_base + 256 + x * 64, t_q = tmem_base + 384 + x * 64;
            // descriptors are built once; a product costs one 64-bit add on each (the low bits of a
            // descriptor are the shared-memory address in units of 16 bytes)
            const uint64_t kdesc = make_smem_desc(base, 16);                       // + stage * STAGE_BYTES
            const uint64_t vdesc = make_smem_desc(base + KV_BYTES, BLOCK_N * 128); // + stage * STAGE_BYTES
            const uint64_t pdesc = make_smem_desc(sP + x * 2 * P_BYTES, 16);      // + (block % 2) * P_BYTES
            auto issue_s = [&](int jj) {                           // S(jj); K(jj) has landed, the S buffer is free
                const uint64_t kd = kdesc + (uint64_t)((jj % NSTAGES) * (STAGE_BYTES >> 4));
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    // Q: 16 elements of a row = 8 columns of tensor memory; K: [half][64 keys][128 B], 32 bytes along a row
                    const uint32_t koff = ((kk / 4) * (BLOCK_N * 128) + (kk % 4) * 32) >> 4;
                    umma_bf16_a_tmem(t_s, t_q + kk * 8, kd + koff, idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(s_full(x));
            };
#ifdef AP_TIMERS
            const bool dbg_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
            const int dslot = x * 8;
            if (dbg_on) for (int i = 0; i < 8; ++i) ap_dbg[dslot + i] = 0;
            const long long tm0 = clock64();
#endif
            bool ok = mbar_wait(q_ready(x), 0, abort_flag);
            if (ok) ok = mbar_wait(kv_full(0), 0, abort_flag);
            if (ok) { tc_fence_after(); issue_s(0); }
            for (int j = 0; j < nb && ok; ++j) {
                const int st = j % NSTAGES;
                AP_T(ta);
                if (j + 1 < nb) {
                    // S(j + 1): its keys have landed, and the tile's warps hold S(j) in registers
                    ok = mbar_wait(kv_full((j + 1) % NSTAGES), (uint32_t)((j + 1) / NSTAGES) & 1, abort_flag);
                    if (ok) ok = mbar_wait(s_free(x), (uint32_t)j & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    AP_T(ta2);
                    issue_s(j + 1);
                    AP_T(ta3);
                    AP_ACC(dslot + 1, ta, ta2); AP_ACC(dslot + 2, ta2, ta3);
                }
                AP_T(tb);
                ok = mbar_wait(p_full(x, j & 1), (uint32_t)(j >> 1) & 1, abort_flag);   // P(j) is in shared memory
                if (!ok) break;
                tc_fence_after();
                AP_T(tc);
                const uint64_t vd = vdesc + (uint64_t)(st * (STAGE_BYTES >> 4));
#pragma unroll
                for (int kk = 0; kk < BLOCK_N / 16; ++kk)
                    umma_bf16(t_o, pdesc + (uint64_t)((j & 1) * (P_BYTES >> 4) + kk * 2), vd + (uint64_t)(kk * 128), idesc_pv,
                              kk > 0 ? 1u : (j > 0 ? 1u : 0u));
                umma_commit(pv_done(x, j & 1));                    // O holds block j; that P buffer is free
                umma_commit(kv_empty(st));                         // this tile has read K and V of the stage
                AP_T(td);
                AP_ACC(dslot + 3, tb, tc); AP_ACC(dslot + 4, tc, td);
            }
#ifdef AP_TIMERS
            if (dbg_on) { ap_dbg[dslot + 0] = clock64() - tm0; ap_dbg[dslot + 5] = nb; }
#endif
        }
    } else if (warp >= 2 && warp <= 9) {
        // ------------------------------------------------- softmax / rescale / epilogue
        const int x = (warp - 2) >> 2;                             // query tile of this warp
        const int q = warp & 3;                                    // TMEM lane quarter this warp may touch
        const int r = q * 32 + lane;                               // row of the tile = TMEM lane
        const int tt = tid - 64 - x * 128;                         // 0..127 within the tile's warps
        const int R = row0 + x * BLOCK_M + r;
        const bool tile_active = x < n_act;
        const bool rv = tile_active && R < rows_total;
        const int pr = pos0 + R / G;
        const int lo_r = p.window > 0 ? max(0, pr - p.window + 1) : 0;
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t t_o = t_row + x * 128;
        const uint32_t t_s = t_row + 256 + x * 64;
        const uint32_t t_q = t_row + 384 + x * 64;
        // the query tile: this thread's row, two elements a column, into tensor memory
        if (tile_active) {
            const bf16* src = p.q + (size_t)(q0 + R / G) * p.q_row_stride + (size_t)(kvh * G + R % G) * D;
#pragma unroll
            for (int c16 = 0; c16 < D / 32; ++c16) {
                uint32_t v[16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint4 u = make_uint4(0u, 0u, 0u, 0u);
                    if (rv) u = *reinterpret_cast<const uint4*>(src + c16 * 32 + c * 8);
                    v[4 * c] = u.x; v[4 * c + 1] = u.y; v[4 * c + 2] = u.z; v[4 * c + 3] = u.w;
                }
                tmem_st16(t_q + c16 * 16, v);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready(x));
        }
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        const int nb_x = tile_active ? nb : 0;
#ifdef AP_TIMERS
        const bool dbg_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (warp == 2 || warp == 6) && lane == 0;
        const int dslot = 16 + x * 8;
        if (dbg_on) for (int i = 0; i < 8; ++i) ap_dbg[dslot + i] = 0;
        const long long ts0 = clock64();
#endif
        for (int j = 0; j < nb_x && ok; ++j) {
            const int st = j % NSTAGES;
            const int blk = kb_lo + j;
            if (blk == kb_hi || blk == kb_lo) {
                // value rows no query row of the CTA may see (beyond the last key, before the first window) are
                // cleared, since page slots and unfetched shared memory may hold anything; the warps of both tiles
                // do it (the same zeros), so that each tile's products wait for its own warps only.
                ok = mbar_wait_warp(kv_full(st), (j / NSTAGES) & 1, abort_flag);
                if (!ok) break;
                uint8_t* gV = gbase + st * STAGE_BYTES + KV_BYTES;
                for (int idx = tt; idx < BLOCK_N * CH; idx += 128) {
                    const int kr = idx / CH, c = idx % CH;
                    const int n = blk * BLOCK_N + kr;
                    if (n > hi || n < lo_cta)
                        *reinterpret_cast<uint4*>(gV + (c >> 3) * (BLOCK_N * 128) + kr * 128 + (((c & 7) ^ (kr & 7)) << 4)) =
                            make_uint4(0u, 0u, 0u, 0u);
                }
                fence_async_smem();
            }
            AP_T(sa);
            ok = mbar_wait_warp(s_full(x), (uint32_t)j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            AP_T(sb);
            float s[BLOCK_N];
            {
                uint32_t v[BLOCK_N];                               // the four loads are in flight together
#pragma unroll
                for (int h = 0; h < BLOCK_N / 16; ++h) tmem_ld16(t_s + h * 16, v + h * 16);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < BLOCK_N; ++i) s[i] = __uint_as_float(v[i]);
            }
            tc_fence_before();                                     // the scores are in registers: the buffer may
            __syncwarp();                                          // take the next block's
            if (lane == 0) mbar_arrive(s_free(x));
            AP_T(sc);
            // Scores stay unscaled in registers; the scale (> 0) is folded into the exponent below.  Key
            // blocks that every row of the warp sees whole need no mask.
            // (four running maxima and, below, four partial sums: chains of 16 dependent operations, not 64)
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            const int n_first = blk * BLOCK_N;
            if (__all_sync(0xffffffffu, rv && n_first + BLOCK_N - 1 <= pr && n_first >= lo_r)) {
#pragma unroll
                for (int i = 0; i < BLOCK_N; i += 2) m4[(i >> 1) & 3] = fmax3(m4[(i >> 1) & 3], s[i], s[i + 1]);
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
            // the product of the block before last must have read the P buffer that this block writes
            AP_T(sd);
            if (j > 1) {
                ok = mbar_wait_warp(pv_done(x, j & 1), (uint32_t)((j >> 1) - 1) & 1, abort_flag);
                if (!ok) break;
            }
            AP_T(se);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? m_blk : m_used;
                const float alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
                if (j > 0) {
                    // O must hold every earlier block before it is rescaled
                    ok = mbar_wait_warp(pv_done(x, (j - 1) & 1), (uint32_t)((j - 1) >> 1) & 1, abort_flag);
                    if (!ok) break;
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
            if (QT == 2 && n_act == 2) {
                // the exponentials of a block are bound by the special-function unit (16 a cycle and SM): side by side
                // the two tiles' passes take twice as long each and leave the unit idle while both tiles do the rest
                ok = mbar_wait_warp(turn(x, q), (uint32_t)j & 1, abort_flag);
                if (!ok) break;
            }
            AP_T(sf);
            uint8_t* prow = gP + (x * 2 + (j & 1)) * P_BYTES + r * 128;
            // scale, subtraction and the row's sum work on pairs of float32 (one instruction a pair)
            uint64_t lsum2[2] = {0ull, 0ull};
            const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), negms2 = pack2(-ms, -ms);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float a0, a1;
                    unpack2(fma2(pack2(s[c * 8 + 2 * i], s[c * 8 + 2 * i + 1]), scale2, negms2), a0, a1);
                    const float e0 = ex2_approx(a0), e1 = ex2_approx(a1);
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
                    lsum2[i & 1] = add2(lsum2[i & 1], pack2(e0, e1));
                    w[i] = *reinterpret_cast<uint32_t*>(&b2);
                }
                *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                if (c == TURN_AFTER - 1 && QT == 2 && n_act == 2) {
                    // the other tile's warp of this scheduler may begin its pass (handing over earlier, so that the
                    // passes overlap in part, was no faster: 3 of 8 chunks 531 us, 6: 525, 8: 522 at 8,192 tokens)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(turn(x ^ 1, q));
                }
            }
            {
                float s0, s1;
                unpack2(add2(lsum2[0], lsum2[1]), s0, s1);
                l += s0 + s1;
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(x, j & 1));
            AP_T(sg);
            AP_ACC(dslot + 1, sa, sb); AP_ACC(dslot + 2, sb, sc); AP_ACC(dslot + 3, sc, sd); AP_ACC(dslot + 4, sd, se);
            AP_ACC(dslot + 5, se, sf); AP_ACC(dslot + 6, sf, sg);
        }
#ifdef AP_TIMERS
        if (dbg_on) ap_dbg[dslot + 0] = clock64() - ts0;
#endif
        // ---------------------------------------------------------------- epilogue
        if (ok && nb_x > 0) ok = mbar_wait_warp(pv_done(x, (nb_x - 1) & 1), (uint32_t)((nb_x - 1) >> 1) & 1, abort_flag);
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
    constexpr int NTHREADS = QT == 2 ? 352 : 192;
    constexpr int smem = NSTAGES * 2 * BLOCK_N * D * 2 + QT * 2 * BLOCK_M * BLOCK_N * 2 +
                         8 * (2 * NSTAGES + BARS_PER_TILE * QT + 8) + 16 + 1024;
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

#ifdef AP_TIMERS
TFF_API int tff_debug_ap_pair_timers(long long* out) {
    return cudaMemcpyFromSymbol(out, ap_dbg, sizeof(long long) * 64) == cudaSuccess ? 0 : 1;
}
#endif

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
    // Two query tiles a CTA share one walk over the keys and take turns at the exponentials: a pair of tiles costs
    // 1.08 times what a single tile costs (512 new tokens behind 3,584 cached ones, 32/8 heads: 92 us as 128 CTAs
    // of one tile, 100 us as 64 CTAs of two).  So single tiles only while they all run at once, one an SM; as soon
    // as they would not, pairs (1,536 tokens from scratch: 61 us against 74 as single tiles; 2,816 tokens: 114
    // against 149; 1,536 behind 2,048 cached ones: 123 against 160).
    const long long sms = tff_num_sms() > 0 ? tff_num_sms() : 1;
    if ((long long)tiles * nkv * num_requests > sms)
        return d == 128 ? launch_prefill<128, 2>(tm, p, pairs, num_requests, stream)
                        : launch_prefill<64, 2>(tm, p, pairs, num_requests, stream);
    return d == 128 ? launch_prefill<128, 1>(tm, p, tiles, num_requests, stream)
                    : launch_prefill<64, 1>(tm, p, tiles, num_requests, stream);
}
