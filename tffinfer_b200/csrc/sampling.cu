// Sampling over float32 logits [rows, vocab] on the device: one token id per row.
//   greedy       first maximum (ties go to the lowest id), as std::max_element does in
//                src/core/sampler/LLMSampler.cpp:43-45
//   temperature  logits scaled by 1/T (LLMSampler.cpp:36-41), softmax in float32, then
//                the inverse CDF at a uniform number u[row] in [0, 1) that the host
//                derives from (seed, request, step), so a request's tokens do not
//                depend on what else is in the batch.  Optional top-k / top-p / min-p
//                filters (the fields of SamplingConfig, LLMSampler.h:55-63) are applied
//                by a threshold on the scaled logit computed by a bisection, which runs
//                over the whole row at first and on a list of candidates in shared
//                memory as soon as that list is short.
#include "common.cuh"

namespace {

constexpr int NT = 1024;

// Two block sums for the price of one (two barriers): every thread gets both totals, added in an order fixed by NT.
__device__ __forceinline__ void block_sum2(float& x, float& y, float* smem /* >= 64 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    x = warp_sum(x); y = warp_sum(y);
    __syncthreads();
    if (lane == 0) { smem[warp] = x; smem[32 + warp] = y; }
    __syncthreads();
    x = warp_sum(lane < NT / 32 ? smem[lane] : 0.f);
    y = warp_sum(lane < NT / 32 ? smem[32 + lane] : 0.f);
}

__global__ void __launch_bounds__(NT)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float sval[32];
    __shared__ int sidx[32];
    pdl_launch_dependents();          // the next kernel may become resident (it waits before it reads or writes)
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += NT) {
        const float v = row[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    if (bi == 0x7fffffff) bi = threadIdx.x < vocab ? threadIdx.x : 0;   // all NaN/-inf in this thread's share
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = sval[lane]; bi = sidx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = bi;
    }
}

// Each thread owns a contiguous share of the vocabulary so that the cumulative sum
// runs in index order.
__global__ void __launch_bounds__(NT)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ uniform, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              int* __restrict__ out, int vocab, int cap) {
    extern __shared__ float2 cand[];             // ``cap`` candidates of the threshold search: (scaled logit, token id)
    __shared__ float red[64];
    __shared__ float part[NT];
    __shared__ int chosen;
    __shared__ float sh_a;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const float T = temperature[r];
    const int tid = threadIdx.x;
    if (tid == 0) chosen = -1;

    // maximum (also the greedy answer when T == 0)
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += NT) mx = fmaxf(mx, row[i]);
    mx = block_max<NT>(mx, red);
    if (!(T > 0.f)) {
        int bi = 0x7fffffff;
        for (int i = tid; i < vocab; i += NT) if (row[i] == mx && i < bi) bi = i;
        __shared__ int smin;
        if (tid == 0) smin = 0x7fffffff;
        __syncthreads();
        atomicMin(&smin, bi);
        __syncthreads();
        if (tid == 0) out[r] = smin == 0x7fffffff ? 0 : smin;
        return;
    }
    const float invT = 1.f / T;
    const int per = (vocab + NT - 1) / NT;
    const int lo = tid * per, hi = min(vocab, lo + per);

    // threshold on z = (x - max) / T below which tokens are dropped
    float cut = -INFINITY;
    const int k = top_k ? top_k[r] : 0;
    const float tp = top_p ? top_p[r] : 1.f;
    const float mp = min_p ? min_p[r] : 0.f;
    if (mp > 0.f) cut = fmaxf(cut, logf(mp));             // p_i >= min_p * p_max  <=>  z_i >= ln(min_p)
    bool among_candidates = false;                        // the tokens that can be kept are listed in shared memory
    int seg = 0;
    if ((k > 0 && k < vocab) || tp < 1.f) {
        // The threshold is the largest z at which a filter is still satisfied: at least k tokens at or above it
        // (top-k), or at least top_p of the mass (top-p); the filters intersect, so the final threshold is the
        // larger of the two, i.e. the largest one at which at least one active filter is still satisfied.  It is
        // found by halving an interval 40 times, each halving a count and a mass of the tokens above the midpoint.
        // Over the whole vocabulary that is 40 passes (151,936 logits: 1.5 ms a row, whatever the batch).  So the
        // halvings look at the whole row only until few tokens are left to decide about: either few lie at or above
        // the interval's lower end (logits as a trained model gives them: some ten passes), or few lie inside the
        // interval (a flat row, of which top-p keeps tens of thousands).  Those tokens -- the candidates -- go to
        // shared memory, and the remaining halvings run on them alone; in the first case so does the draw itself.
        // Rows whose candidates do not fit their slabs' stretches, or that have fewer than k tokens above -32, take
        // every halving over the whole row.  One row: 1.47 -> 0.13-0.33 ms; 256 rows: 3.2 -> 0.4-0.6 ms.
        // (The passes take the row strided, thread t the tokens t, t + NT, ..., four loads in flight: neighbouring
        // threads read neighbouring words.  A sum's order of additions is fixed by the row alone in every one of them.)
        const bool want_k = k > 0 && k < vocab, want_p = tp < 1.f;
        const int lane = tid & 31, warp = tid >> 5;
        auto above = [&](float mid, float& cnt, float& mass) {        // tokens with z >= mid: how many, their mass
            cnt = 0.f; mass = 0.f;
            for (int base = tid; base < vocab; base += 4 * NT) {
                float x[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) x[u] = base + u * NT < vocab ? row[base + u * NT] : -INFINITY;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float z = (x[u] - mx) * invT;
                    if (z >= mid) { cnt += 1.f; mass += expf(z); }
                }
            }
            block_sum2(cnt, mass, red);                               // the same totals in every thread
        };
        float tot = 0.f, cnt, mass;
        above(-INFINITY, cnt, tot);                                   // the whole row: total mass for top-p
        float a = -32.f, bnd = 0.f;                                   // invariant: kept(a) is enough, kept(bnd) may not be
        float cnt_a, cnt_b = 0.f, mass_b = 0.f;                       // tokens at or above a; at or above bnd, and their mass
        above(a, cnt_a, mass);
        int halvings = 40;
        // 0: every halving over the whole row.  1: the candidates are all tokens at or above a (few are kept: the search
        // and the draw run on them).  2: the candidates are the tokens of [a, bnd) (many are kept: the search runs on
        // them, on top of the count and the mass of the tokens above bnd; the draw takes the row once more).
        int mode = 0;
        seg = cap / 32;
        const float fits = (float)(seg * 12);                         // candidates spread over the 32 slabs: well under 32 * seg
        if ((want_k && cnt_a >= (float)k) || (want_p && mass >= tp * tot)) {
            while (halvings > 0 && cap >= 32) {
                if (cnt_a <= fits) { mode = 1; break; }
                if (cnt_a - cnt_b <= fits && bnd < 0.f) { mode = 2; break; }
                const float mid = 0.5f * (a + bnd);
                above(mid, cnt, mass);
                --halvings;
                if ((want_k && cnt >= (float)k) || (want_p && mass >= tp * tot)) { a = mid; cnt_a = cnt; }
                else { bnd = mid; cnt_b = cnt; mass_b = mass; }
            }
        } else {
            float zmin = 0.f;                                         // (fewer than k tokens above -32)
            for (int i = tid; i < vocab; i += NT) zmin = fminf(zmin, (row[i] - mx) * invT);
            a = -block_max<NT>(-zmin, red);
        }
        // the candidates, warp w those of its slab of the row, in index order, in its own stretch of the buffer
        int* seg_n = reinterpret_cast<int*>(part);                    // [32]
        if (mode != 0) {
            const float top = mode == 1 ? INFINITY : bnd;
            const int slab = (vocab + 31) / 32;
            const int s0 = warp * slab, s1 = min(vocab, s0 + slab);
            int n = 0;
            for (int base = s0; base < s1; base += 128) {
                float x[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) x[u] = base + u * 32 + lane < s1 ? row[base + u * 32 + lane] : -INFINITY;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float z = (x[u] - mx) * invT;
                    const bool is_c = z >= a && z < top;
                    const unsigned m = __ballot_sync(0xffffffffu, is_c);
                    if (is_c) {
                        const int pos = n + __popc(m & ((1u << lane) - 1u));
                        if (pos < seg) cand[warp * (seg + 1) + pos] = make_float2(z, __int_as_float(base + u * 32 + lane));
                    }
                    n += __popc(m);
                }
            }
            if (lane == 0) seg_n[warp] = n;
            __syncthreads();
            for (int w = 0; w < 32; ++w) if (seg_n[w] > seg) mode = 0;         // a slab with more than its stretch holds
        }
        if (mode != 0) {
            // one warp finishes the search alone, lane w on warp w's candidates, with shuffles and no barrier in the loop
            if (tid < 32) {
                const float2* mine = cand + tid * (seg + 1);
                const int n = seg_n[tid];
                const float c0 = mode == 2 ? cnt_b : 0.f, m0 = mode == 2 ? mass_b : 0.f;
                for (int it = 0; it < halvings; ++it) {
                    const float mid = 0.5f * (a + bnd);
                    if (mid <= a || mid >= bnd) break;             // float resolution reached
                    float c1 = 0.f, m1 = 0.f;
                    for (int c = 0; c < n; ++c) {
                        const float z = mine[c].x;
                        if (z >= mid) { c1 += 1.f; m1 += expf(z); }
                    }
                    c1 = c0 + warp_sum(c1); m1 = m0 + warp_sum(m1);
                    if ((want_k && c1 >= (float)k) || (want_p && m1 >= tp * tot)) a = mid; else bnd = mid;
                }
                if (tid == 0) sh_a = a;
            }
            __syncthreads();
            a = sh_a;
        } else {
            for (int it = 0; it < halvings; ++it) {
                const float mid = 0.5f * (a + bnd);
                above(mid, cnt, mass);
                if ((want_k && cnt >= (float)k) || (want_p && mass >= tp * tot)) a = mid; else bnd = mid;
            }
        }
        among_candidates = mode == 1;
        cut = fmaxf(cut, a);
        if (among_candidates) {
            // Every token that is kept is a candidate, and the candidates stand in index order (warp after warp, each
            // its slab of the row): the draw needs no further pass over the row.  One warp adds the kept masses 32
            // at a time, first for the total, then again until the running sum passes u * total.
            if (tid < 32) {
                float total_mass = 0.f;
                int pick = -1, last_kept = -1;
                for (int round = 0; round < 2 && pick < 0; ++round) {
                    const float target = uniform[r] * total_mass;      // (of the second round)
                    float running = 0.f;
                    for (int w = 0; w < 32 && pick < 0; ++w) {
                        for (int c0 = 0; c0 < seg_n[w] && pick < 0; c0 += 32) {
                            const int c = c0 + tid;
                            float e = 0.f;
                            int id = -1;
                            if (c < seg_n[w]) {
                                const float2 zc = cand[w * (seg + 1) + c];
                                if (zc.x >= cut) { e = expf(zc.x); id = __float_as_int(zc.y); }
                            }
                            float incl = e;                            // inclusive sum over the lanes
#pragma unroll
                            for (int o = 1; o < 32; o <<= 1) {
                                const float v = __shfl_up_sync(0xffffffffu, incl, o);
                                if (tid >= o) incl += v;
                            }
                            if (round == 1) {
                                const unsigned hit = __ballot_sync(0xffffffffu, id >= 0 && target < running + incl);
                                const unsigned kept = __ballot_sync(0xffffffffu, id >= 0);
                                if (hit) pick = __shfl_sync(0xffffffffu, id, __ffs(hit) - 1);
                                else if (kept) last_kept = __shfl_sync(0xffffffffu, id, 31 - __clz(kept));
                            }
                            running += __shfl_sync(0xffffffffu, incl, 31);
                        }
                    }
                    if (round == 0) total_mass = running;
                }
                if (pick < 0) pick = last_kept;                        // rounding left the target at the very end
                if (tid == 0) out[r] = pick >= 0 ? pick : 0;
            }
            return;
        }
        __syncthreads();                                   // ``part`` is used again below
    }

    float s = 0.f;
    for (int i = lo; i < hi; ++i) {
        const float z = (row[i] - mx) * invT;
        if (z >= cut) s += expf(z);
    }
    part[tid] = s;
    __syncthreads();
    // inclusive scan of the NT partial sums (Hillis-Steele; order fixed by NT)
    for (int off = 1; off < NT; off <<= 1) {
        const float v = tid >= off ? part[tid - off] : 0.f;
        __syncthreads();
        part[tid] += v;
        __syncthreads();
    }
    const float total = part[NT - 1];
    const float target = uniform[r] * total;
    const float before = tid > 0 ? part[tid - 1] : 0.f;
    if (lo < hi && before <= target && target < part[tid]) {
        float c = before;
        int pick = -1, last = -1;
        for (int i = lo; i < hi; ++i) {
            const float z = (row[i] - mx) * invT;
            if (z < cut) continue;
            last = i;
            c += expf(z);
            if (target < c) { pick = i; break; }
        }
        if (pick < 0) pick = last;
        if (pick >= 0) chosen = pick;
    }
    __syncthreads();
    if (tid == 0) {
        int c = chosen;
        if (c < 0) {                          // rounding left the target at the very end: take the maximum
            c = 0;
            for (int i = 0; i < vocab; ++i) if (row[i] == mx) { c = i; break; }
        }
        out[r] = c;
    }
}

}  // namespace

// Greedy choice with the vocabulary cut into shares, one CTA a share, for few rows of a large
// vocabulary (one CTA a row would leave the GPU idle).  The shares write (value, index) candidates
// into ``scratch`` (rows * shares pairs); the last share of a row to finish -- a ticket counter per
// row, reset for the next call -- picks the first maximum among them.
constexpr int ARGMAX_SHARES = 16;
__global__ void __launch_bounds__(256)
argmax_split_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab,
                    float* __restrict__ cand_val, int* __restrict__ cand_idx, unsigned* __restrict__ tickets) {
    __shared__ float sval[8];
    __shared__ int sidx[8];
    __shared__ bool last;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y, share = blockIdx.x;
    const int per = (vocab + ARGMAX_SHARES - 1) / ARGMAX_SHARES;
    const int lo = share * per, hi = min(vocab, lo + per);
    const float* row = logits + (size_t)r * vocab;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += 256) {
        const float v = row[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sval[w] > best || (sval[w] == best && sidx[w] < bi)) { best = sval[w]; bi = sidx[w]; }
        cand_val[r * ARGMAX_SHARES + share] = best;
        cand_idx[r * ARGMAX_SHARES + share] = bi;
        __threadfence();
        last = atomicAdd(&tickets[r], 1u) == ARGMAX_SHARES - 1;
    }
    __syncthreads();
    if (last && threadIdx.x == 0) {
        __threadfence();
        float b = -INFINITY;
        int id = 0x7fffffff;
        for (int s2 = 0; s2 < ARGMAX_SHARES; ++s2) {
            // what other CTAs wrote: read from the L2, never from a line this SM may hold
            const float v = __ldcg(&cand_val[r * ARGMAX_SHARES + s2]);
            const int i = __ldcg(&cand_idx[r * ARGMAX_SHARES + s2]);
            if (v > b || (v == b && i < id)) { b = v; id = i; }
        }
        out[r] = id == 0x7fffffff ? 0 : id;
        tickets[r] = 0;
    }
}

// ``scratch`` (may be null): (64 + 2 * 64 * 16) 32-bit words, the first 64 of them zero before the
// first call (the kernel leaves them zero); with it, up to 64 rows of a large vocabulary are searched
// by 16 CTAs each.
TFF_API int tff_argmax(const float* logits, int* out, int rows, int vocab, void* scratch, cudaStream_t stream) {
    if (rows <= 0) return TFF_OK;
    if (vocab <= 0) return TFF_ERR_BAD_ARGUMENT;
    if (scratch != nullptr && vocab >= 16384 && rows <= 64) {
        unsigned* tickets = (unsigned*)scratch;                       // 64 counters, zero between calls
        float* cand_val = (float*)(tickets + 64);                     // 64 x 16 values
        int* cand_idx = (int*)(cand_val + 64 * ARGMAX_SHARES);        // 64 x 16 indices
        return tff_launch_pdl(argmax_split_kernel, dim3(ARGMAX_SHARES, rows), dim3(256), 0, stream, logits, out, vocab,
                              cand_val, cand_idx, tickets);
    }
    return tff_launch_pdl(argmax_kernel, rows, NT, 0, stream, logits, out, vocab);
}

// temperature[r] <= 0 selects greedy for that row.  top_k / top_p / min_p may be null.
TFF_API int tff_sample(const float* logits, const float* temperature, const float* uniform,
                       const int* top_k, const float* top_p, const float* min_p,
                       int* out, int rows, int vocab, cudaStream_t stream) {
    if (rows <= 0) return TFF_OK;
    if (vocab <= 0 || temperature == nullptr || uniform == nullptr) return TFF_ERR_BAD_ARGUMENT;
    // with top-k or top-p: room for the candidates of the threshold search (8,192 of them; more shared memory would
    // leave the L1 too small for the passes in which every thread walks a contiguous share of the row, which rows
    // without candidates still take)
    constexpr int kCandBytes = 64 * 1024;
    size_t smem = 0;
    if (top_k != nullptr || top_p != nullptr) {
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kCandBytes) != cudaSuccess)
                return TFF_ERR_LAUNCH;
            configured = true;
        }
        smem = kCandBytes;
    }
    sample_kernel<<<rows, NT, smem, stream>>>(logits, temperature, uniform, top_k, top_p, min_p, out, vocab,
                                              (int)(smem / sizeof(float2)) - 64);     // 254 a warp, 255 apart: an odd stride
    return tff_launch_status();
}

// logits[row[i], token[i]] is divided by penalty[i] if positive, else multiplied
// (src/core/sampler/LLMSampler.cpp:21-34).  The (row, token) pairs are distinct.
__global__ void repetition_penalty_kernel(float* logits, const int* __restrict__ rows,
                                          const int* __restrict__ tokens, const float* __restrict__ penalty,
                                          int n, int vocab) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = tokens[i];
    if (t < 0 || t >= vocab) return;
    float* p = logits + (size_t)rows[i] * vocab + t;
    const float v = *p;
    *p = v > 0.f ? v / penalty[i] : v * penalty[i];
}

TFF_API int tff_repetition_penalty(float* logits, const int* rows, const int* tokens, const float* penalty,
                                   int n, int vocab, cudaStream_t stream) {
    if (n <= 0) return TFF_OK;
    repetition_penalty_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, rows, tokens, penalty, n, vocab);
    return tff_launch_status();
}
