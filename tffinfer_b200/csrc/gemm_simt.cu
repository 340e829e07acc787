// C[M, N] = A[M, K] * W[N, K]^T (+ residual), accumulated in float32 with plain FMAs.
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced
// precision mode) and the product used whenever an operand is stored in float32.
// It stands in for the reference's dense fp32 GEMM (src/kernel/cuda/mat_mul.cu:151-660).
// Every output element adds its K products in the order k = 0 .. K-1, so its value
// does not depend on M, on the tile it falls in, or on what else is in the batch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* C,
                 const float* residual, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;          // tx -> N, ty -> M
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BK, kk = idx % BK;
            const int gk = k0 + kk;
            float a = 0.f, w = 0.f;
            if (gk < K) {
                if (m0 + r < M) a = to_f32<TA>(A[(size_t)(m0 + r) * K + gk]);
                if (n0 + r < N) w = to_f32<TW>(W[(size_t)(n0 + r) * K + gk]);
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (residual) v = residual[(size_t)m * N + n] + v;
            C[(size_t)m * N + n] = from_f32<TC>(v);
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch(const void* A, const void* W, void* C, const float* residual, int M, int N, int K, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_simt_kernel<TA, TW, TC><<<grid, 256, 0, s>>>((const TA*)A, (const TW*)W, (TC*)C, residual, M, N, K);
    return tff_launch_status();
}

}  // namespace

// dtype codes: 0 = float32, 1 = bfloat16.  ``residual`` (float32 [M, N], may alias C
// when C is float32) is added to the product when it is not null.
TFF_API int tff_gemm_simt(const void* A, int a_dt, const void* W, int w_dt, void* C, int c_dt,
                          const float* residual, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return TFF_OK;
    if (K <= 0) return TFF_ERR_BAD_ARGUMENT;
    if ((long long)((M + BM - 1) / BM) > 65535) return TFF_ERR_UNSUPPORTED;
    const int code = a_dt * 4 + w_dt * 2 + c_dt;
    switch (code) {
        case 0: return launch<float, float, float>(A, W, C, residual, M, N, K, stream);
        case 1: return launch<float, float, bf16>(A, W, C, residual, M, N, K, stream);
        case 2: return launch<float, bf16, float>(A, W, C, residual, M, N, K, stream);
        case 3: return launch<float, bf16, bf16>(A, W, C, residual, M, N, K, stream);
        case 4: return launch<bf16, float, float>(A, W, C, residual, M, N, K, stream);
        case 5: return launch<bf16, float, bf16>(A, W, C, residual, M, N, K, stream);
        case 6: return launch<bf16, bf16, float>(A, W, C, residual, M, N, K, stream);
        case 7: return launch<bf16, bf16, bf16>(A, W, C, residual, M, N, K, stream);
    }
    return TFF_ERR_BAD_ARGUMENT;
}
