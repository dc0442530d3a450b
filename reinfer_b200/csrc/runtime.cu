// Error text of the last refused call (per host thread) and a version probe.
#include "common.cuh"
#include <stdarg.h>
#include <cuda.h>
#include <cudaTypedefs.h>
#include <mutex>
#include <unordered_map>

static thread_local char g_err[512] = "";

void rb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

extern "C" const char* rb_last_error() { return g_err; }

extern "C" int rb_abi_version() { return 1; }

int g_rb_pdl = 1;
// Programmatic dependent launch on (1) or off (0) for the kernels that support it; returns the old value.
extern "C" int rb_set_pdl(int on) { int old = g_rb_pdl; g_rb_pdl = on ? 1 : 0; return old; }

// Compute capability of the current device as major*10+minor, or a negative cudaError_t.
extern "C" int rb_device_cc() {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return -(int)e;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return -(int)e;
    e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) return -(int)e;
    return major * 10 + minor;
}

// ---- tensor maps -------------------------------------------------------------------------
// Encoded through the driver entry point (no link against libcuda) and cached.
static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
    });
    return fn;
}

struct MapKey {
    const void* ptr; long long rows, cols, ld; int box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.ld; h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};
// A tensor map depends only on (address, extents, row stride, box), so a cached one never goes stale.
int rb_tensor_map_bf16(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    auto enc = get_encode();
    if (!enc) RB_REFUSE("tensor map: the driver offers no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RB_REFUSE("tensor map: cuTensorMapEncodeTiled failed with %d (ptr %p rows %lld cols %lld ld %lld)", (int)r, ptr, rows, cols, ld);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
    return 0;
}


// A map over one layer's paged cache [pages, 2 (keys, values), kv_heads, page_size, 128] bfloat16 that brings the keys (or
// the values) of one (page, kv head) in ONE request, laid out for the tensor cores: the 128 dims of a key are split
// into two 64-dim halves and the keys into groups of eight, and the box arrives as [group][half][8 keys][64 dims] -
// 1,024-byte atoms of the 128-byte swizzle, a group's two halves side by side, groups 2,048 bytes apart.  So a tile
// of 64 keys from pages of any size (8, 16, 32, 64 tokens) has ONE layout, and a page costs one request instead
// of one per half (two per page with a plain 2-D map).  Dimensions, innermost first: 64 dims (2 bytes apart), 8
// keys (256 bytes), 2 halves (128 bytes), page_size / 8 groups (2,048 bytes), and (page, k|v, head) folded into one
// index of page_size * 256 bytes.  (The halves' stride is smaller than the keys': the driver asks only that strides
// are multiples of 16 bytes.)
int rb_tensor_map_kv_pages(const void* cache, long long num_pages, int kv_heads, int page_size, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache_maps;
    static std::mutex mu;
    MapKey key{cache, num_pages, kv_heads, page_size, -5};
    std::lock_guard<std::mutex> g(mu);
    auto it = cache_maps.find(key);
    if (it != cache_maps.end()) { *out = it->second; return 0; }
    auto enc = get_encode();
    if (!enc) RB_REFUSE("tensor map: the driver offers no cuTensorMapEncodeTiled");
    if (page_size < 8 || page_size % 8) RB_REFUSE("tensor map: pages of %d tokens (a multiple of 8 is needed)", page_size);
    const int groups = page_size / 8;
    cuuint64_t dims[5] = {64, 8, 2, (cuuint64_t)groups, (cuuint64_t)num_pages * 2ull * (cuuint64_t)kv_heads};
    cuuint64_t strides[4] = {256, 128, 2048, (cuuint64_t)page_size * 256ull};
    cuuint32_t box[5] = {64, 8, 2, (cuuint32_t)(groups < 8 ? groups : 8), 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RB_REFUSE("tensor map (cache pages): cuTensorMapEncodeTiled failed with %d (pages %lld heads %d page size %d)",
                                     (int)r, num_pages, kv_heads, page_size);
    if (cache_maps.size() > 1024) cache_maps.clear();
    cache_maps.emplace(key, *out);
    return 0;
}

// ---- the status word -------------------------------------------------------------------------
// One int per device in pinned host memory that is mapped into the device.  A kernel whose bounded wait gives up
// stores its code there (sm100.cuh: rb_raise), so the host learns of it with a plain load at a moment when it has
// waited for the step anyway (after the sampled tokens arrived), with no call into the device.  Made at the first
// call on a device, which also tells every translation unit where the word is.
extern "C" int rb_gemm_bind_status(int*);
extern "C" int rb_attn_bind_status(int*);
extern "C" int rb_attn_tc_bind_status(int*);
extern "C" int rb_selftest_bind_status(int*);
extern "C" int rb_gemm_error(int);
extern "C" int rb_attn_error(int);
extern "C" int rb_attn_tc_error(int);
extern "C" int rb_selftest_error(int);

#define RB_MAX_DEVICES 64
static int* g_status_host[RB_MAX_DEVICES] = {nullptr};
static std::mutex g_status_mu;

// The host address of the current device's status word (NULL on failure, with the reason in rb_last_error).
extern "C" int* rb_status_host() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= RB_MAX_DEVICES) { rb_set_error("status word: no current device"); return nullptr; }
    std::lock_guard<std::mutex> g(g_status_mu);
    if (g_status_host[dev]) return g_status_host[dev];
    int* host = nullptr;
    int* mapped = nullptr;
    cudaError_t e = cudaHostAlloc((void**)&host, 64, cudaHostAllocMapped);
    if (e == cudaSuccess) { *host = 0; e = cudaHostGetDevicePointer((void**)&mapped, host, 0); }
    if (e != cudaSuccess) { rb_set_error("status word: CUDA error %d", (int)e); return nullptr; }
    int rc = rb_gemm_bind_status(mapped);
    if (!rc) rc = rb_attn_bind_status(mapped);
    if (!rc) rc = rb_attn_tc_bind_status(mapped);
    if (!rc) rc = rb_selftest_bind_status(mapped);
    if (rc) { rb_set_error("status word: CUDA error %d while binding it", rc); return nullptr; }
    g_status_host[dev] = host;
    return host;
}

// Clear the status word and every unit's own word (synchronises the device); returns what the status word held.
extern "C" int rb_status_clear() {
    int* host = rb_status_host();
    if (!host) return -1;
    cudaDeviceSynchronize();
    const int v = *(volatile int*)host;
    *(volatile int*)host = 0;
    rb_gemm_error(1); rb_attn_error(1); rb_attn_tc_error(1); rb_selftest_error(1);
    return v;
}
