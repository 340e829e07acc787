// Causal grouped-query flash attention over the paged cache, bfloat16 operands, float32
// softmax statistics and output accumulators, for head sizes 64 and 128.
//
// One contract serves prompt portions and single decoded tokens (any mix in one launch):
// the G = nq/nkv query heads that share a kv head are packed with the tokens into rows,
// row R of a request = (token R / G, head kvh*G + R % G), so that a decode token with
// G = 4 is a 4-row tile and a 16-token portion a 64-row tile.  A CTA (4 warps) takes one
// tile of one (request, kv head) and one contiguous share of the keys ("split"):
//   rows mode   64 rows, each warp 16 of them against all 64 keys of a block (portions);
//   keys mode   16 rows, each warp all of them against 16 of the 64 keys of a block; the
//               warps' partial results are merged through shared memory (decode).
// Key/value blocks of 64 tokens, aligned to absolute positions, come through cp.async
// into a two-stage swizzled shared-memory ring, page by page through the block table.
// QK^T and PV run on mma.sync m16n8k16 (bf16 in, float32 out); the probabilities go
// from the score accumulators straight into the A fragments of the PV product.
// With more than one split the unnormalised partial (O, m, l) goes to a float32
// workspace and a second kernel merges the splits.
//
// Stands where the reference runs its SIMT kernel paged_flash_attention_fp16_8x32
// (src/kernel/cuda/paged_flash_attention.cu:877-1055: 8 queries x 32 keys x one GQA group,
// scale 1/sqrt(d) at :1158, online softmax :696-792), which is instantiated for 32/8/128 only.
#include "common.cuh"
#include "attention_common.h"

namespace {

constexpr int BLOCK_N = 64;
constexpr int NTHREADS = 128;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

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
// byte offset of 16-byte chunk ``chunk`` of row ``row`` in a tile with D bf16 per row
template <int D> __device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * (D * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
}

struct AttnParams {
    const bf16* q; int q_row_stride;
    const int* q_start; const int* pos_start; const int* req_ids;   // req_ids: rows of the per-request arrays (or null)
    const int* block_table; int table_width;
    const bf16* cache; KvLayout L; int layer;
    bf16* out; float* part_o; float* part_ml; int num_splits;
    int nq, nkv; float scale_log2; int window;
};

template <int D, bool KEYS_MODE>
__global__ void __launch_bounds__(NTHREADS)
attn_fwd_kernel(const AttnParams p) {
    constexpr int BLOCK_M = KEYS_MODE ? 16 : 64;
    constexpr int NT = KEYS_MODE ? 2 : 8;            // 8-key tiles per warp per block
    constexpr int CH = D / 8;                        // 16-byte chunks per row
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* sQ = smem;                                          // [BLOCK_M][D]
    uint8_t* sK = sQ + BLOCK_M * D * 2;                          // [2][64][D]
    uint8_t* sV = sK + 2 * BLOCK_N * D * 2;                      // [2][64][D]

    pdl_launch_dependents();          // the next kernel may become resident (it waits before it reads or writes)
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = p.req_ids ? p.req_ids[blockIdx.z] : (int)blockIdx.z, kvh = blockIdx.y;
    // later tiles see more keys: they are issued first
    const int tile = (int)(gridDim.x / p.num_splits) - 1 - (int)(blockIdx.x / p.num_splits);
    const int split = blockIdx.x % p.num_splits;
    const int G = p.nq / p.nkv;
    const int q0 = p.q_start[b];
    const int q_len = p.q_start[b + 1] - q0;
    const int rows_total = q_len * G;
    if (tile * BLOCK_M >= rows_total) return;
    const int pos0 = p.pos_start[b];
    const int first_tok = (tile * BLOCK_M) / G;
    const int last_tok = min(q_len - 1, (tile * BLOCK_M + BLOCK_M - 1) / G);
    const int hi = pos0 + last_tok;
    const int lo_tile = p.window > 0 ? max(0, pos0 + first_tok - p.window + 1) : 0;
    const int kb_lo = lo_tile / BLOCK_N, kb_hi = hi / BLOCK_N;
    const int nblk = kb_hi - kb_lo + 1;
    const int per = (nblk + p.num_splits - 1) / p.num_splits;
    const int kb_begin = kb_lo + split * per;
    const int kb_end = min(kb_hi + 1, kb_begin + per);           // may be <= kb_begin: an empty split
    const int* table = p.block_table + (size_t)b * p.table_width;
    const bf16* cache_k = p.cache + (size_t)p.layer * p.L.layer_stride + (size_t)kvh * p.L.head_stride;

    // ---------------------------------------------------------------- loads
    auto load_kv = [&](int blk, int stage) {
        uint8_t* dk = sK + stage * BLOCK_N * D * 2;
        uint8_t* dv = sV + stage * BLOCK_N * D * 2;
#pragma unroll
        for (int it = 0; it < BLOCK_N * CH / NTHREADS; ++it) {
            const int idx = tid + it * NTHREADS;
            const int row = idx / CH, chunk = idx % CH;
            const int n = blk * BLOCK_N + row;
            const bf16* src = p.cache;
            int bytes = 0;
            if (n <= hi) {
                const int page = table[n / p.L.page_size];
                if (page >= 0) {
                    src = cache_k + (size_t)page * p.L.page_stride + (size_t)(n % p.L.page_size) * D + chunk * 8;
                    bytes = 16;
                }
            }
            const uint32_t off = swz<D>(row, chunk);
            cp_async16(smem_u32(dk + off), src, bytes);
            cp_async16(smem_u32(dv + off), bytes ? src + p.L.kv_stride : src, bytes);
        }
    };
    // the query tile: packed rows (token, head of the group)
    for (int idx = tid; idx < BLOCK_M * CH; idx += NTHREADS) {
        const int row = idx / CH, chunk = idx % CH;
        const int R = tile * BLOCK_M + row;
        const bf16* src = p.q;
        int bytes = 0;
        if (R < rows_total) {
            src = p.q + (size_t)(q0 + R / G) * p.q_row_stride + (size_t)(kvh * G + R % G) * D + chunk * 8;
            bytes = 16;
        }
        cp_async16(smem_u32(sQ + swz<D>(row, chunk)), src, bytes);
    }
    if (kb_begin < kb_end) load_kv(kb_begin, 0);
    cp_async_commit();

    // ------------------------------------------------------- per-thread rows
    const int row_off = KEYS_MODE ? 0 : warp * 16;
    const int key_off = KEYS_MODE ? warp * 16 : 0;
    const int r0 = row_off + (lane >> 2), r1 = r0 + 8;            // rows of the tile this thread holds
    const int R0 = tile * BLOCK_M + r0, R1 = tile * BLOCK_M + r1;
    const bool v0 = R0 < rows_total, v1 = R1 < rows_total;
    const int pr0 = pos0 + R0 / G, pr1 = pos0 + R1 / G;           // positions of the rows' tokens
    const int lo0 = p.window > 0 ? max(0, pr0 - p.window + 1) : 0;
    const int lo1 = p.window > 0 ? max(0, pr1 - p.window + 1) : 0;

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    uint32_t qf[D / 16][4];

    for (int blk = kb_begin; blk < kb_end; ++blk) {
        const int stage = (blk - kb_begin) & 1;
        if (blk + 1 < kb_end) load_kv(blk + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (blk == kb_begin) {
            // query fragments once: matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15)
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int row = row_off + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int chunk = kk * 2 + (lane >> 4);
                ldsm_x4(smem_u32(sQ + swz<D>(row, chunk)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
            }
        }
        const uint8_t* tK = sK + stage * BLOCK_N * D * 2;
        const uint8_t* tV = sV + stage * BLOCK_N * D * 2;
        // ------------------------------------------------------ S = Q K^T
        float s[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                // matrices: (keys 0-7, k 0-7), (keys 0-7, k 8-15), (keys 8-15, k 0-7), (keys 8-15, k 8-15)
                const int row = key_off + np * 16 + (lane & 7) + (lane >> 4) * 8;
                const int chunk = kk * 2 + ((lane >> 3) & 1);
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_u32(tK + swz<D>(row, chunk)), b0, b1, b2, b3);
                mma_bf16(s[2 * np], qf[kk], b0, b1);
                mma_bf16(s[2 * np + 1], qf[kk], b2, b3);
            }
        }
        // ------------------------------------------- mask, online softmax
        const int nbase = blk * BLOCK_N + key_off + 2 * (lane & 3);
        float bm0 = -INFINITY, bm1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int n = nbase + nt * 8 + (e & 1);
                const bool up = e < 2;
                const bool ok = up ? (v0 && n <= pr0 && n >= lo0) : (v1 && n <= pr1 && n >= lo1);
                const float x = ok ? s[nt][e] * p.scale_log2 : -INFINITY;
                s[nt][e] = x;
                if (up) bm0 = fmaxf(bm0, x); else bm1 = fmaxf(bm1, x);
            }
        }
        bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 1)); bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 2));
        bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 1)); bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 2));
        const float mn0 = fmaxf(m0, bm0), mn1 = fmaxf(m1, bm1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float a0 = exp2f(m0 - ms0), a1 = exp2f(m1 - ms1);       // exp2(-inf) = 0 on the first block
        m0 = mn0; m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            s[nt][0] = exp2f(s[nt][0] - ms0); s[nt][1] = exp2f(s[nt][1] - ms0);
            s[nt][2] = exp2f(s[nt][2] - ms1); s[nt][3] = exp2f(s[nt][3] - ms1);
            ps0 += s[nt][0] + s[nt][1];
            ps1 += s[nt][2] + s[nt][3];
        }
        l0 = l0 * a0 + ps0;
        l1 = l1 * a1 + ps1;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
        // -------------------------------------------------------- O += P V
#pragma unroll
        for (int kc = 0; kc < NT / 2; ++kc) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kc][0], s[2 * kc][1]);
            a[1] = pack_bf16(s[2 * kc][2], s[2 * kc][3]);
            a[2] = pack_bf16(s[2 * kc + 1][0], s[2 * kc + 1][1]);
            a[3] = pack_bf16(s[2 * kc + 1][2], s[2 * kc + 1][3]);
#pragma unroll
            for (int dn = 0; dn < D / 16; ++dn) {
                // transposed matrices: (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
                const int row = key_off + kc * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int chunk = dn * 2 + (lane >> 4);
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(smem_u32(tV + swz<D>(row, chunk)), b0, b1, b2, b3);
                mma_bf16(o[2 * dn], a, b0, b1);
                mma_bf16(o[2 * dn + 1], a, b2, b3);
            }
        }
        __syncthreads();                       // the stage may be overwritten by the next iteration's load
    }
    cp_async_wait<0>();
    // row sums over the four lanes that share a row
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    if constexpr (KEYS_MODE) {
        // merge the four warps (same 16 rows, different keys) through shared memory
        __syncthreads();
        float* mO = reinterpret_cast<float*>(sK);                 // [4][16][D] floats (fits: 2*64*D*2 bytes >= 4*16*D*4)
        float* mM = reinterpret_cast<float*>(sV);                 // [4][16], then [4][16] for l
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
        __syncthreads();
        for (int idx = tid; idx < 16 * D; idx += NTHREADS) {
            const int r = idx / D, c = idx % D;
            const int R = r;                                       // tile 0 in keys mode
            if (R >= rows_total) continue;
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
            const size_t grow = (size_t)(q0 + R / G) * p.nq + (kvh * G + R % G);
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
    } else {
        const size_t g0 = (size_t)(q0 + R0 / G) * p.nq + (kvh * G + R0 % G);
        const size_t g1 = (size_t)(q0 + R1 / G) * p.nq + (kvh * G + R1 % G);
        if (p.num_splits == 1) {
            const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                const int c = i * 8 + 2 * (lane & 3);
                if (v0) *reinterpret_cast<uint32_t*>(&p.out[g0 * D + c]) = pack_bf16(o[i][0] * i0, o[i][1] * i0);
                if (v1) *reinterpret_cast<uint32_t*>(&p.out[g1 * D + c]) = pack_bf16(o[i][2] * i1, o[i][3] * i1);
            }
        } else {
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                const int c = i * 8 + 2 * (lane & 3);
                if (v0) *reinterpret_cast<float2*>(&p.part_o[(g0 * p.num_splits + split) * D + c]) = make_float2(o[i][0], o[i][1]);
                if (v1) *reinterpret_cast<float2*>(&p.part_o[(g1 * p.num_splits + split) * D + c]) = make_float2(o[i][2], o[i][3]);
            }
            if ((lane & 3) == 0) {
                if (v0) { p.part_ml[(g0 * p.num_splits + split) * 2] = m0; p.part_ml[(g0 * p.num_splits + split) * 2 + 1] = l0; }
                if (v1) { p.part_ml[(g1 * p.num_splits + split) * 2] = m1; p.part_ml[(g1 * p.num_splits + split) * 2 + 1] = l1; }
            }
        }
    }
}

// out[row, :] = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s, M = max_s m_s, for the rows
// (token, head) of the requests the launch covered: grid (nq * max_q_len, requests).
// the merge of up to MAXS splits of one output row: all statistics, then all partial outputs, are asked for at
// once (two round trips to memory, not two per split)
template <int D, int MAXS>
__device__ __forceinline__ void combine_row(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                            bf16* __restrict__ out, int num_splits, size_t row) {
    float2 ml[MAXS];
#pragma unroll
    for (int s = 0; s < MAXS; ++s)
        ml[s] = s < num_splits ? *reinterpret_cast<const float2*>(part_ml + (row * num_splits + s) * 2) : make_float2(-INFINITY, 0.f);
    float M = -INFINITY;
#pragma unroll
    for (int s = 0; s < MAXS; ++s) M = fmaxf(M, ml[s].x);
    const float Ms = M == -INFINITY ? 0.f : M;
    float f[MAXS], lsum = 0.f;
#pragma unroll
    for (int s = 0; s < MAXS; ++s) {
        f[s] = (s < num_splits && ml[s].y != 0.f) ? exp2f(ml[s].x - Ms) : 0.f;   // an empty split counts for nothing
        lsum += f[s] * ml[s].y;
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float po[MAXS];
#pragma unroll
        for (int s = 0; s < MAXS; ++s)                                      // (an empty split's O may be unwritten)
            po[s] = f[s] != 0.f ? part_o[(row * num_splits + s) * D + c] : 0.f;
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < MAXS; ++s) acc += f[s] * po[s];
        out[row * D + c] = __float2bfloat16_rn(acc / lsum);
    }
}

template <int D>
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, int num_splits, const int* __restrict__ q_start,
                                    const int* __restrict__ req_ids, int nq) {
    pdl_launch_dependents();          // the next kernel may become resident (it waits before it reads or writes)
    // the step's batch arrays are older than the kernel ahead: they are read before waiting for it
    const int b = req_ids ? req_ids[blockIdx.y] : (int)blockIdx.y;
    const int t = blockIdx.x / nq, h = blockIdx.x % nq;
    const int q0 = q_start[b];
    const int q_len = q_start[b + 1] - q0;
    pdl_wait();
    if (t >= q_len) return;
    const size_t row = (size_t)(q0 + t) * nq + h;
    if (num_splits <= 4) { combine_row<D, 4>(part_o, part_ml, out, num_splits, row); return; }
    if (num_splits <= 8) { combine_row<D, 8>(part_o, part_ml, out, num_splits, row); return; }
    if (num_splits <= 16) { combine_row<D, 16>(part_o, part_ml, out, num_splits, row); return; }
    float M = -INFINITY;
    for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[(row * num_splits + s) * 2]);
    const float Ms = M == -INFINITY ? 0.f : M;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float acc = 0.f, lsum = 0.f;
        for (int s = 0; s < num_splits; ++s) {
            const float l = part_ml[(row * num_splits + s) * 2 + 1];
            if (l == 0.f) continue;                                 // an empty split (its O may be unwritten)
            const float f = exp2f(part_ml[(row * num_splits + s) * 2] - Ms);
            acc += f * part_o[(row * num_splits + s) * D + c];
            lsum += f * l;
        }
        out[row * D + c] = __float2bfloat16_rn(acc / lsum);
    }
}

template <int D, bool KEYS_MODE>
int launch_attn(const AttnParams& p, int q_tiles, int B, cudaStream_t stream) {
    constexpr int BLOCK_M = KEYS_MODE ? 16 : 64;
    constexpr int smem = (BLOCK_M + 4 * BLOCK_N) * D * 2;
    auto kern = attn_fwd_kernel<D, KEYS_MODE>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return TFF_ERR_LAUNCH;
        configured = true;
    }
    dim3 grid(q_tiles * p.num_splits, p.nkv, B);
    return tff_launch_pdl(kern, grid, NTHREADS, smem, stream, p);
}

}  // namespace

// Bytes of float32 workspace needed for ``rows`` = tokens * nq rows and ``num_splits`` splits.
TFF_API long long tff_attention_bf16_workspace(int rows, int num_splits, int d) {
    if (num_splits <= 1) return 0;
    return (long long)rows * num_splits * (d + 2) * 4;
}

// q [T, nq*d] bf16 (normalised, rotated); out [T, nq*d] bf16.
//   max_q_len   largest number of new tokens any request brings (sizes the grid)
//   num_splits  shares of the key range per tile (> 1 needs ``workspace``)
// Returns TFF_ERR_UNSUPPORTED for head sizes other than 64 and 128.
static int attention_bf16_impl(
    const void* q, const int* q_start, const int* pos_start, const int* req_ids, const int* block_table, int table_width,
    const void* cache, long long cache_pages, int cache_layers, int layer, int page_size,
    void* out, void* workspace, int num_tokens, int num_requests, int max_q_len, int num_splits,
    int nq, int nkv, int d, float scale, int window, cudaStream_t stream) {
    if (num_tokens <= 0 || num_requests <= 0) return TFF_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || max_q_len <= 0 || num_splits < 1)
        return TFF_ERR_BAD_ARGUMENT;
    if (d != 64 && d != 128) return TFF_ERR_UNSUPPORTED;
    if (num_splits > 1 && workspace == nullptr) return TFF_ERR_BAD_ARGUMENT;
    if (num_requests > 65535 || nkv > 65535) return TFF_ERR_UNSUPPORTED;
    const int G = nq / nkv;
    AttnParams p;
    p.q = (const bf16*)q; p.q_row_stride = nq * d;
    p.q_start = q_start; p.pos_start = pos_start; p.req_ids = req_ids;
    p.block_table = block_table; p.table_width = table_width;
    p.cache = (const bf16*)cache; p.L = make_kv_layout(cache_layers, nkv, page_size, d); p.layer = layer;
    p.out = (bf16*)out;
    p.num_splits = num_splits;
    const long long rows = (long long)num_tokens * nq;
    p.part_o = (float*)workspace;
    p.part_ml = workspace ? (float*)workspace + rows * num_splits * d : nullptr;
    p.nq = nq; p.nkv = nkv;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.window = window;
    const bool keys_mode = (long long)max_q_len * G <= 16;
    const int block_m = keys_mode ? 16 : 64;
    const int q_tiles = (max_q_len * G + block_m - 1) / block_m;
    int st = TFF_ERR_UNSUPPORTED;
    if (keys_mode && cache_pages > 0)      // decode: keys streamed by TMA (attention_decode.cu), when it takes the shape
        st = tff_attention_decode_launch(q, q_start, pos_start, req_ids, block_table, table_width, cache, cache_pages,
                                         cache_layers, layer, page_size, out, p.part_o, p.part_ml, num_requests,
                                         max_q_len, num_splits, nq, nkv, d, scale, window, stream);
    if (!keys_mode && num_splits == 1 && cache_pages > 0)   // portions: tcgen05 kernel (attention_prefill.cu)
        st = tff_attention_prefill_launch(q, q_start, pos_start, req_ids, block_table, table_width, cache, cache_pages,
                                          cache_layers, layer, page_size, out, num_requests, max_q_len, nq, nkv, d,
                                          scale, window, stream);
    if (st == TFF_ERR_UNSUPPORTED) {
        if (d == 128) st = keys_mode ? launch_attn<128, true>(p, q_tiles, num_requests, stream)
                                     : launch_attn<128, false>(p, q_tiles, num_requests, stream);
        else st = keys_mode ? launch_attn<64, true>(p, q_tiles, num_requests, stream)
                            : launch_attn<64, false>(p, q_tiles, num_requests, stream);
    }
    if (st != TFF_OK) return st;
    if (num_splits > 1) {
        const dim3 cgrid((unsigned)(nq * max_q_len), (unsigned)num_requests);
        if (d == 128) return tff_launch_pdl(attn_combine_kernel<128>, cgrid, dim3(128), 0, stream,
                                            (const float*)p.part_o, (const float*)p.part_ml, p.out, num_splits,
                                            q_start, req_ids, nq);
        return tff_launch_pdl(attn_combine_kernel<64>, cgrid, dim3(64), 0, stream,
                              (const float*)p.part_o, (const float*)p.part_ml, p.out, num_splits, q_start, req_ids, nq);
    }
    return TFF_OK;
}

TFF_API int tff_attention_bf16(
    const void* q, const int* q_start, const int* pos_start, const int* block_table, int table_width,
    const void* cache, int cache_layers, int layer, int page_size,
    void* out, void* workspace, int num_tokens, int num_requests, int max_q_len, int num_splits,
    int nq, int nkv, int d, float scale, int window, cudaStream_t stream) {
    return attention_bf16_impl(q, q_start, pos_start, nullptr, block_table, table_width, cache, 0, cache_layers, layer,
                               page_size, out, workspace, num_tokens, num_requests, max_q_len, num_splits, nq, nkv, d,
                               scale, window, stream);
}

// The same with the number of pages of the cache tensor given, which lets decode-sized calls
// stream the keys with TMA (a tensor map needs the extent of what it describes).
// ``req_ids`` (may be null) lists the rows of q_start / pos_start / block_table the launch covers,
// num_requests of them; null means rows 0 .. num_requests-1.
TFF_API int tff_attention_bf16_paged(
    const void* q, const int* q_start, const int* pos_start, const int* req_ids, const int* block_table, int table_width,
    const void* cache, long long cache_pages, int cache_layers, int layer, int page_size,
    void* out, void* workspace, int num_tokens, int num_requests, int max_q_len, int num_splits,
    int nq, int nkv, int d, float scale, int window, cudaStream_t stream) {
    return attention_bf16_impl(q, q_start, pos_start, req_ids, block_table, table_width, cache, cache_pages, cache_layers,
                               layer, page_size, out, workspace, num_tokens, num_requests, max_q_len, num_splits, nq,
                               nkv, d, scale, window, stream);
}

// ------------------------------------------------------- allocation-free variant
// See no_alloc_api.h for who this is for and for its rules.
#include "no_alloc_api.h"
#include <mutex>

namespace {
// The scratch of the split-key merge, inside the library.  In host code this name is only
// a stand-in for the symbol, not a device address: the address each GPU gave it is looked
// up once per device with cudaGetSymbolAddress and that pointer is what kernels receive.
static __device__ __align__(256) float g_noalloc_scratch[TFF_ATTENTION_NOALLOC_SCRATCH_BYTES / 4];
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;
}  // namespace

// Bytes of the library's scratch array that a call would use, in 64-bit arithmetic throughout (the
// row count tokens * nq of a large batch does not fit an int): 0 when num_splits == 1, -1 when a count is
// not positive or the product does not fit 62 bits.  A pure function of its arguments; launches nothing.
long long tff_attention_bf16_noalloc_bytes(long long num_tokens, long long nq, long long num_splits, long long d) {
    if (num_tokens <= 0 || nq <= 0 || num_splits < 1 || d <= 0) return -1;
    if (num_splits == 1) return 0;
    const long long limit = 1LL << 62;
    long long v = num_tokens;
    const long long factors[4] = {nq, num_splits, d + 2, 4};
    for (long long f : factors) {
        if (v > limit / f) return -1;
        v *= f;
    }
    return v;
}

int tff_attention_bf16_noalloc(
    const void* q, const int* q_start, const int* pos_start, const int* block_table, int table_width,
    const void* cache, int cache_layers, int layer, int page_size,
    void* out, int num_tokens, int num_requests, int max_q_len, int num_splits,
    int nq, int nkv, int d, float scale, int window, cudaStream_t stream) {
    if (num_tokens <= 0 || num_requests <= 0) return TFF_OK;
    // every argument is checked here, before the size of the scratch is looked at and before anything is launched
    if (!q || !q_start || !pos_start || !block_table || !cache || !out) return TFF_ERR_BAD_ARGUMENT;
    if (num_splits < 1 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || d <= 0 || page_size <= 0 || table_width <= 0 ||
        max_q_len <= 0 || cache_layers <= 0 || layer < 0 || layer >= cache_layers || window < 0)
        return TFF_ERR_BAD_ARGUMENT;
    const long long need = tff_attention_bf16_noalloc_bytes(num_tokens, nq, num_splits, d);
    if (need < 0 || need > (long long)TFF_ATTENTION_NOALLOC_SCRATCH_BYTES) return TFF_ERR_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    if (num_splits > 1) {
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TFF_ERR_LAUNCH;
        std::lock_guard<std::mutex> g(g_noalloc_mu);
        if (g_noalloc_ptr[dev] == nullptr) {
            // set-up, once per device, with that device current
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return TFF_ERR_LAUNCH;
            g_noalloc_ptr[dev] = static_cast<float*>(p);
        }
        scratch = g_noalloc_ptr[dev];
    }
    return tff_attention_bf16(q, q_start, pos_start, block_table, table_width, cache, cache_layers, layer, page_size,
                              out, scratch, num_tokens, num_requests, max_q_len, num_splits, nq, nkv, d, scale,
                              window, stream);
}
