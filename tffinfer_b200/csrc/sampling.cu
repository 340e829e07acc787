// Sampling over float32 logits [rows, vocab] on the device: one token id per row.
//   greedy       first maximum (ties go to the lowest id), as std::max_element does in
//                src/core/sampler/LLMSampler.cpp:43-45
//   temperature  logits scaled by 1/T (LLMSampler.cpp:36-41), softmax in float32, then
//                the inverse CDF at a uniform number u[row] in [0, 1) that the host
//                derives from (seed, request, step), so a request's tokens do not
//                depend on what else is in the batch.  Optional top-k / top-p / min-p
//                filters (the fields of SamplingConfig, LLMSampler.h:55-63) are applied
//                by a threshold on the scaled logit computed by a bisection.
#include "common.cuh"

namespace {

constexpr int NT = 1024;

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
              int* __restrict__ out, int vocab) {
    __shared__ float red[32];
    __shared__ float part[NT];
    __shared__ int chosen;
    __shared__ float sh_a, sh_b;
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
    if ((k > 0 && k < vocab) || tp < 1.f) {
        // total mass for top-p
        float tot = 0.f;
        for (int i = lo; i < hi; ++i) tot += expf((row[i] - mx) * invT);
        tot = block_sum<NT>(tot, red);
        // bisection on the threshold: keep the largest threshold whose kept set still
        // has >= k members (top-k) / mass >= top_p * total (top-p); 40 halvings of
        // [zmin, 0] reach float resolution.
        float a = -1e30f, bnd = 0.f;                       // invariant: kept(a) is enough, kept(bnd) may not be
        float zmin = 0.f;
        for (int i = lo; i < hi; ++i) zmin = fminf(zmin, (row[i] - mx) * invT);
        zmin = -block_max<NT>(-zmin, red);
        a = zmin;
        for (int it = 0; it < 40; ++it) {
            const float mid = 0.5f * (a + bnd);
            float cnt = 0.f, mass = 0.f;
            for (int i = lo; i < hi; ++i) {
                const float z = (row[i] - mx) * invT;
                if (z >= mid) { cnt += 1.f; mass += expf(z); }
            }
            cnt = block_sum<NT>(cnt, red);
            mass = block_sum<NT>(mass, red);
            // the filters intersect: the final threshold is the larger of the two, i.e. the
            // largest one at which at least one active filter is still satisfied
            bool enough = false;
            if (k > 0 && k < vocab) enough = enough || cnt >= (float)k;
            if (tp < 1.f) enough = enough || mass >= tp * tot;
            if (tid == 0) { if (enough) sh_a = mid, sh_b = bnd; else sh_a = a, sh_b = mid; }
            __syncthreads();
            a = sh_a; bnd = sh_b;
            __syncthreads();
        }
        cut = fmaxf(cut, a);
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
    sample_kernel<<<rows, NT, 0, stream>>>(logits, temperature, uniform, top_k, top_p, min_p, out, vocab);
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
