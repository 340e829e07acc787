#include "common.cuh"
#include "tma_host.h"
#include <mutex>
#include <unordered_map>

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

struct MapKey {
    const void* ptr; long long rows; long long cols; int box_rows; int box_cols; int elt;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols && elt == o.elt;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h ^= (size_t)k.rows * 0x9E3779B97F4A7C15ull; h ^= (size_t)k.cols * 0xC2B2AE3D27D4EB4Full;
        h ^= ((size_t)k.box_rows << 48) ^ ((size_t)k.box_cols << 40) ^ ((size_t)k.elt << 36);
        return h;
    }
};

int* g_error_flag = nullptr;
int g_num_sms = 0;
std::mutex g_mu;

}  // namespace

bool tff_tensor_map_2d(const void* ptr, long long rows, long long cols, int box_rows, int box_cols, int elt,
                       CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{ptr, rows, cols, box_rows, box_cols, elt};
    {
        std::lock_guard<std::mutex> g(g_mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return true; }
    }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * elt};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    if (enc(&m, elt == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
            const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    {
        std::lock_guard<std::mutex> g(g_mu);
        if (cache.size() > 4096) cache.clear();
        cache[key] = m;
    }
    *out = m;
    return true;
}

bool tff_tensor_map_kv_page(const void* cache, long long total_rows, int head_dim, int page_size, int kv_heads,
                            CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache_maps;
    const MapKey key{cache, total_rows, head_dim, page_size, kv_heads, -4};
    {
        std::lock_guard<std::mutex> g(g_mu);
        auto it = cache_maps.find(key);
        if (it != cache_maps.end()) { *out = it->second; return true; }
    }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    const int halves = head_dim / 64;
    const cuuint64_t dims[4] = {64, (cuuint64_t)halves, (cuuint64_t)total_rows, 2};
    const cuuint64_t strides[3] = {128, (cuuint64_t)head_dim * 2, (cuuint64_t)kv_heads * page_size * head_dim * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)halves, (cuuint32_t)page_size, 2};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMap m;
    if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(cache), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    {
        std::lock_guard<std::mutex> g(g_mu);
        if (cache_maps.size() > 256) cache_maps.clear();
        cache_maps[key] = m;
    }
    *out = m;
    return true;
}

int* tff_device_error_flag() {
    std::lock_guard<std::mutex> g(g_mu);
    if (g_error_flag) return g_error_flag;
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) { cudaFree(p); return nullptr; }
    g_error_flag = p;
    return g_error_flag;
}

int tff_num_sms() {
    std::lock_guard<std::mutex> g(g_mu);
    if (g_num_sms > 0) return g_num_sms;
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    g_num_sms = n;
    return n;
}

long long tff_decode_gemm_ctas(long long units) {
    static int x100 = -1;
    if (x100 < 0) { const char* v = getenv("TFFINFER_GEMM_CTAS_X100"); x100 = v ? atoi(v) : 275; if (x100 < 100 || x100 > 300) x100 = 275; }
    long long ctas = (long long)tff_num_sms() * x100 / 100;
    return ctas > units ? units : ctas;
}

// The SM count of the current device, for planners outside this library (they must cut work the way
// the launchers size their grids).
TFF_API int tff_sm_count() { return tff_num_sms(); }

// Copies the error word into pinned host memory in stream order (no synchronisation): the host looks at it
// when it reads the results of the same step.
TFF_API int tff_error_word_to_host_async(int* pinned_dst, cudaStream_t stream) {
    int* flag = tff_device_error_flag();
    if (!flag || !pinned_dst) return TFF_ERR_BAD_ARGUMENT;
    return cudaMemcpyAsync(pinned_dst, flag, sizeof(int), cudaMemcpyDeviceToHost, stream) == cudaSuccess ? TFF_OK : TFF_ERR_LAUNCH;
}

// Reads (and clears) the error word: non-zero when a bounded wait inside a kernel ran out.
// Synchronises the device.
TFF_API int tff_kernel_error() {
    int* flag = nullptr;
    {
        std::lock_guard<std::mutex> g(g_mu);
        flag = g_error_flag;
    }
    if (!flag) return 0;
    int v = 0;
    if (cudaMemcpy(&v, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(flag, 0, sizeof(int));
    return v;
}
