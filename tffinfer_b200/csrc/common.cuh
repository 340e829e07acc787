// Shared device helpers for the sm_100a kernels of this package.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#define TFF_API extern "C" __attribute__((visibility("default")))

// Error codes returned by the host launchers (0 = launched).
enum TffStatus : int {
    TFF_OK = 0,
    TFF_ERR_BAD_ARGUMENT = -1,     // a size or pointer the kernel cannot take
    TFF_ERR_UNSUPPORTED = -2,      // a size outside what this kernel was written for
    TFF_ERR_LAUNCH = -3,           // cudaGetLastError() after the launch was not success
    TFF_ERR_DRIVER = -4,           // a driver entry point (tensor maps) is unavailable
};

static inline int tff_launch_status() {
    return cudaGetLastError() == cudaSuccess ? TFF_OK : TFF_ERR_LAUNCH;
}

// Programmatic dependent launch.  A kernel launched through tff_launch_pdl may become
// resident while its predecessor in the stream is still running; it must call pdl_wait()
// before it writes global memory or reads anything a predecessor wrote (constant inputs
// such as weights may be fetched earlier), and calls pdl_launch_dependents() once it no
// longer minds its own successor becoming resident.  TFFINFER_PDL=0 turns the launch
// attribute off (the device-side calls are then no-ops).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool tff_pdl_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("TFFINFER_PDL"); v = (e && e[0] == '0') ? 0 : 1; }
    return v != 0;
}

template <typename Kern, typename... Args>
static inline int tff_launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tff_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...) == cudaSuccess ? TFF_OK : TFF_ERR_LAUNCH;
}

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of NT threads (NT a multiple of 32, <= 1024).  The order of the
// additions is fixed by NT alone, so a row's result never depends on its neighbours.
template <int NT>
__device__ __forceinline__ float block_sum(float v, float* smem /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = (lane < NT / 32) ? smem[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
template <int NT>
__device__ __forceinline__ float block_max(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = (lane < NT / 32) ? smem[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// Geometry of one layer group's paged cache:
// tensor [pages, layers, 2 (K,V), kv_heads, page_size, head_dim], contiguous.
struct KvLayout {
    long long page_stride;    // elements between pages
    long long layer_stride;   // elements between layers
    long long kv_stride;      // elements between K and V
    long long head_stride;    // elements between kv heads (= page_size * head_dim)
    int page_size;
    int head_dim;
};
__host__ __device__ inline KvLayout make_kv_layout(int layers, int kv_heads, int page_size, int head_dim) {
    KvLayout L;
    L.page_size = page_size;
    L.head_dim = head_dim;
    L.head_stride = (long long)page_size * head_dim;
    L.kv_stride = L.head_stride * kv_heads;
    L.layer_stride = L.kv_stride * 2;
    L.page_stride = L.layer_stride * layers;
    return L;
}
