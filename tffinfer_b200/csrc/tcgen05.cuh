// Pieces shared by the tcgen05 kernels: PTX wrappers for mbarriers, TMA copies, tensor memory and
// tcgen05.mma, the shared-memory and instruction descriptors of a 128-byte-swizzled K-major bfloat16
// tile, and the iterator that deals (tile, K block) units to the CTAs of a persistent kernel.
#pragma once
#include "common.cuh"
#include "tma_host.h"

namespace tc5 {

constexpr int BM = 128;           // rows of the lane operand per tile
constexpr int BK = 64;            // K elements per stage: 128 bytes of bf16 = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

// ---------------------------------------------------------------- PTX wrappers
static __device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// A build for hunting faults of ordering: with -DTFF_JITTER=<ns> (TFFINFER_NVCC_FLAGS) every arrival at an mbarrier
// and every return from a wait is held back, about one time in three, by a pseudo-random pause of up to that many
// nanoseconds, so that warps which usually keep step fall out of it by more than a pipeline stage.  A kernel whose
// barriers are right gives the same results, only later; one that relied on the usual timing (a warp arriving for
// use n + 1 of a counted barrier before another has arrived for use n) fails its tests at once instead of one run
// in three.  Off, and free, in the normal build.
#ifdef TFF_JITTER
static __device__ __forceinline__ void jitter() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    uint32_t h = (uint32_t)t * 2654435761u ^ (threadIdx.x * 40503u + blockIdx.x * 9176u + blockIdx.y * 131u);
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    if (h % 3u == 0u) __nanosleep((h >> 8) % (uint32_t)(TFF_JITTER));
}
#else
static __device__ __forceinline__ void jitter() {}
#endif

static __device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
static __device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
static __device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    jitter();
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
static __device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait: at most ``limit`` polls.  Returns false when it gave up (the flag is then raised) or when
// another role already had.
static __device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                       uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i >= 64) {
            __nanosleep(32);
            if (*abort_flag) return false;
        }
    }
    *abort_flag = 1;
    return false;
}
// The same for warps that wait beside warps that compute: try_wait is given a time hint, so that the hardware
// suspends the waiting warp instead of letting it poll (a failed try_wait without a hint returns after 8 cycles,
// with a hint of 1 us after 1400; a suspended warp runs again 120 cycles after the arrival).  Polling warps take
// issue slots from the others on their scheduler: the softmax warps of the prompt attention ran 5 % slower
// beside them.  Bounded by time: about a second of SM clock.
constexpr long long WAIT_LIMIT_CYCLES = 1ll << 31;
static __device__ __forceinline__ uint32_t mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
    return ok;
}
static __device__ __forceinline__ bool mbar_wait_suspended(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait_hint(bar, parity, 2000u)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) break;
    }
    *abort_flag = 1;
    return false;
}
static __device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#ifdef TFF_SUSPENDED_WAITS
    const bool ok = mbar_wait_suspended(bar, parity, abort_flag);
#else
    const bool ok = mbar_wait_limit(bar, parity, abort_flag, WAIT_LIMIT);
#endif
    jitter();
    return ok;
}
static __device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(x), "r"(y) : "memory");
}
static __device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(tm), "r"(src), "r"(x), "r"(y) : "memory");
}
static __device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* tm, uint32_t src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(tm), "r"(src), "r"(x), "r"(y) : "memory");
}
static __device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
static __device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

static __device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
static __device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
static __device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
static __device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
static __device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
static __device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

static __device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
static __device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128
// bytes, groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1,
// layout type 2 (SWIZZLE_128B).  Addresses and offsets are in units of 16 bytes.
static __device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
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

// The segments of one CTA of a persistent kernel with G CTAs: which (tile, range of K blocks) it works
// on, in order.  Two dealers, kept apart so that the kernels that stream weights carry only the short one.
//
// SegIterShares (products that stream their weights once):
//   mode 0:  whole tiles c, c+G, c+2G, ...
//   mode 1:  the contiguous share [c*U/G, (c+1)*U/G) of the U = tiles * kb_per_tile (tile, K block)
//            units ("stream-K"): every CTA reads the same number of bytes
struct SegIterShares {
    int kbt, mode, stride;
    long long u, u_end;
    int tile, kb0, kb1;
    __device__ SegIterShares(int n_tiles, int kbt_, int mode_, int cta, int n_ctas)
        : kbt(kbt_), mode(mode_), stride(n_ctas) {
        if (mode) {
            const long long U = (long long)n_tiles * kbt;
            u = U * cta / n_ctas;
            u_end = U * (cta + 1) / n_ctas;
        } else {
            u = cta;
            u_end = n_tiles;
        }
    }
    __device__ bool next() {
        if (u >= u_end) return false;
        if (mode) {
            tile = (int)(u / kbt);
            kb0 = (int)(u % kbt);
            const long long left = u_end - u;
            kb1 = (long long)(kbt - kb0) < left ? kbt : kb0 + (int)left;
            u += kb1 - kb0;
        } else {
            tile = (int)u; kb0 = 0; kb1 = kbt;
            u += stride;
        }
        return true;
    }
};

// SegIterSlices (products with many tiles, bound by the tensor core):
//   mode 0:       whole tiles c, c+G, c+2G, ...
//   mode S >= 1:  the first floor(tiles / G) * G tiles as in mode 0; each tile of the last, partial wave
//                 is cut into max(S, 2) slices of its K range, and the (slice, tile) items, tiles fastest,
//                 go round-robin to the CTAs.  CTAs that run together then work on neighbouring tiles at
//                 the same K blocks, as in the whole waves, and share operands in L2; a partial wave of
//                 R tiles costs ceil(R*S/G)/S of a tile's time instead of a whole one.
struct SegIterSlices {
    int kbt, slices, stride, first_split, tail_tiles;
    long long u, u_end;
    int tile, kb0, kb1;
    bool whole;                      // still in the whole-tile part
    __device__ SegIterSlices(int n_tiles, int kbt_, int mode, int cta, int n_ctas)
        : kbt(kbt_), slices(mode == 1 ? 2 : mode), stride(n_ctas) {
        first_split = mode == 0 ? n_tiles : (n_tiles / n_ctas) * n_ctas;
        tail_tiles = n_tiles - first_split;
        whole = true;
        u = cta;
        u_end = first_split;
    }
    __device__ bool next() {
        if (whole) {
            if (u < u_end) {
                tile = (int)u; kb0 = 0; kb1 = kbt;
                u += stride;
                return true;
            }
            whole = false;
            u -= first_split;                                  // first item of this CTA: its index continues
            u_end = (long long)tail_tiles * slices;
        }
        while (u < u_end) {
            const int slice = (int)(u / tail_tiles);
            tile = first_split + (int)(u % tail_tiles);
            kb0 = (int)((long long)slice * kbt / slices);
            kb1 = (int)((long long)(slice + 1) * kbt / slices);
            u += stride;
            if (kb1 > kb0) return true;                        // more slices than K blocks: empty ones are skipped
        }
        return false;
    }
};

}  // namespace tc5
