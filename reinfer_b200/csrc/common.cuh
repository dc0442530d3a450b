// Shared helpers of the hand-written sm_100a kernels: element types, conversions,
// deterministic reductions and the error convention of the C entry points.
//
// Every entry point is `extern "C" int rb_*(…, void* stream)`, takes raw device
// pointers, launches on the given stream and returns 0, a negative code for a
// refused argument (the text is kept per thread, see rb_last_error) or the
// positive cudaError_t of the launch.  No entry point allocates.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

enum RbDtype { RB_F32 = 0, RB_BF16 = 1 };

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Fixed-order warp reductions (butterfly: every lane ends with the same value, and
// the order of additions does not depend on anything but the lane count).
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

// Block sum over blockDim.x threads (a multiple of 32, at most 1024); `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = (lane < nw) ? red[lane] : 0.0f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = (lane < nw) ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// With -DRB_TIMELINE thread 0 of every CTA of a kernel that opens with RB_TL(id) appends a record
// {id << 32 | linear block index, start, end, mark} (mark: where the kernel calls RB_TL_MARK(), usually after its wait for the kernels before) (globaltimer, ns) to a buffer set through the translation
// unit's setter (RB_TL_SETTER): word 0 of the buffer counts records, word 1 holds the capacity, records of
// 4 words start at word 4.  A development aid for seeing how the kernels of a step overlap; off by default.
#ifdef RB_TIMELINE
static __device__ unsigned long long* g_rb_tl = nullptr;
struct RbTlScope {
    unsigned long long t0, aux;
    int id;
    __device__ __forceinline__ explicit RbTlScope(int id_) : aux(0), id(id_) { asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0)); }
    __device__ __forceinline__ void mark() { asm volatile("mov.u64 %0, %globaltimer;" : "=l"(aux)); }
    __device__ __forceinline__ ~RbTlScope() {
        unsigned long long* b = g_rb_tl;
        if (!b || threadIdx.x || threadIdx.y || threadIdx.z) return;
        unsigned long long t1;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        const unsigned long long slot = atomicAdd(b, 1ULL);
        if (slot >= b[1]) return;
        unsigned long long* r = b + 4 + slot * 4;
        r[0] = ((unsigned long long)id << 32) | (unsigned)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x);
        r[1] = t0; r[2] = t1; r[3] = aux;
    }
};
#define RB_TL(id) RbTlScope rb_tl_scope(id)
#define RB_TL_MARK() rb_tl_scope.mark()
#define RB_TL_SETTER(fn) extern "C" int fn(unsigned long long* buf) { return (int)cudaMemcpyToSymbol(g_rb_tl, &buf, sizeof(buf)); }
#else
#define RB_TL(id) do { } while (0)
#define RB_TL_MARK() do { } while (0)
#define RB_TL_SETTER(fn)
#endif

// Programmatic dependent launch.  A kernel launched through rb_launch() may begin while its
// predecessor in the stream is still running; it must call pdl_wait() before it touches any
// memory that a predecessor writes or reads.  pdl_trigger() lets the successor begin.  Both are
// no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- host side -----------------------------------------------------------
extern int g_rb_pdl;                      // 1: rb_launch() asks for programmatic stream serialization

template <typename... KArgs, typename... Args>
static inline int rb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rb_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
    return (int)cudaGetLastError();
}

// The same for a grid whose CTAs form clusters of the given shape (every grid dimension a multiple of the cluster's).
template <typename... KArgs, typename... Args>
static inline int rb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x; attr[0].val.clusterDim.y = cluster.y; attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rb_pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
    return (int)cudaGetLastError();
}

void rb_set_error(const char* fmt, ...);
#define RB_REFUSE(...) do { rb_set_error(__VA_ARGS__); return -1; } while (0)
#define RB_LAUNCH_RESULT() ((int)cudaGetLastError())

static inline int rb_ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }
