// Inline PTX for the sm_100a features the kernels use: mbarriers with bounded waits, TMA tile
// loads, tcgen05 (tensor memory, MMA, commit, loads), cluster barriers and distributed shared
// memory; and the host call that encodes a 2-D bfloat16 tensor map.
#pragma once
#include "common.cuh"
#include <cuda.h>

#define RB_SPIN_LIMIT (1u << 24)

// 0 ok; else (unit << 16 | 1 << 8 | where) of the first bounded wait that gave up.  One word per translation unit
// (device symbols are not shared between separately compiled files; a file names its unit with RB_UNIT before it
// includes this header) and, for the host, one word for all of them in pinned host memory that is mapped into the
// device (g_rb_status_host, bound by RB_STATUS_EXPORTS' binder): the kernel that gives up writes its code there as
// well, so the host sees it with a plain load, without a call into the device (runtime.cu: rb_status_host).
#ifndef RB_UNIT
#define RB_UNIT 0
#endif
static __device__ int g_rb_kernel_error = 0;
static __device__ int* g_rb_status_host = nullptr;

__device__ __forceinline__ void rb_raise(int where) {
    const int code = (RB_UNIT << 16) | (1 << 8) | where;
    if (atomicCAS(&g_rb_kernel_error, 0, code) == 0) {
        int* h = g_rb_status_host;
        if (h) { *(volatile int*)h = code; __threadfence_system(); }
    }
}

// The reader of this unit's word (synchronises the device; with reset != 0 the word is cleared) and the binder of
// the host's word.
#define RB_STATUS_EXPORTS(reader, binder)                                                                   \
    extern "C" int reader(int reset) {                                                                      \
        int v = 0;                                                                                          \
        if (cudaMemcpyFromSymbol(&v, g_rb_kernel_error, sizeof(int)) != cudaSuccess) return -1;              \
        if (reset && v) { int z = 0; cudaMemcpyToSymbol(g_rb_kernel_error, &z, sizeof(int)); }               \
        return v;                                                                                           \
    }                                                                                                       \
    extern "C" int binder(int* mapped) { return (int)cudaMemcpyToSymbol(g_rb_status_host, &mapped, sizeof(mapped)); }

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// *p += v in global memory with nothing coming back.
__device__ __forceinline__ void red_add_f32(float* p, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add_f32x4(float* p, float4 v) {       // p is 16-byte aligned
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// A look at the barrier that never suspends the thread (try_wait may, for a while, when the phase is not complete).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after RB_WAIT_NS nanoseconds of the global timer (or RB_SPIN_LIMIT polls,
// whichever comes first).  Returns false if the CTA is aborting, or if this wait gave up - then it
// raises the CTA's abort flag and records where in the error word.
#define RB_WAIT_NS 2000000000ull
__device__ __forceinline__ unsigned long long rb_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait_ns(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where,
                                             unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < RB_SPIN_LIMIT; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 63u) == 63u) {
            if (*abort_flag) return false;
            const unsigned long long now = rb_globaltimer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) break;
        }
    }
    *abort_flag = where;
    rb_raise(where);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where) {
    return mbar_wait_ns(bar, parity, abort_flag, where, RB_WAIT_NS);
}
// After a failed wait: let the copies that were issued into this CTA's shared memory land (bounded) before leaving.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = rb_globaltimer();
    while (!mbar_try(bar, parity)) if (rb_globaltimer() - t0 > RB_WAIT_NS / 4) break;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// Ask for bytes [base + lo, base + hi) to be brought into L2, in pieces of at most 32 KB; nothing waits for them.
// base is 16-byte aligned; the range is clipped to whole 16-byte units inside it.
__device__ __forceinline__ void l2_prefetch_range(const unsigned char* base, long long lo, long long hi) {
    for (long long o = lo; o < hi; o += 32768) {
        const long long left = hi - o;
        const uint32_t n = (uint32_t)(left < 32768 ? left : 32768) & ~15u;
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + o), "r"(n) : "memory");
    }
}
// This CTA's share (part of parts, 4 KB granules) of the first `bytes` bytes at base.
__device__ __forceinline__ void l2_prefetch_share(const void* base, long long bytes, int part, int parts) {
    if (!base || bytes <= 0) return;
    const long long per = (((bytes + parts - 1) / parts) + 4095) & ~4095LL;
    const long long lo = per * part;
    const long long hi = lo + per < bytes ? lo + per : bytes;
    if (lo < hi) l2_prefetch_range((const unsigned char*)base, lo, hi);
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Forms for a warp that stays converged and lets one lane issue (lead != 0 in that lane only).  A warp whose issuing
// lane runs alone inside a branch pays for it at every asynchronous instruction: measured on the persistent product,
// about a hundred cycles for each tcgen05.mma, tcgen05.commit and TMA request, whatever its size.
__device__ __forceinline__ void tc_mma_bf16_lead(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate, uint32_t lead) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(lead) : "memory");
}
__device__ __forceinline__ void tc_commit_lead(uint32_t bar, uint32_t lead) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar), "r"(lead) : "memory");
}
__device__ __forceinline__ void tma_load_2d_lead(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint32_t lead) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n\t}"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar), "r"(lead) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_lead(uint32_t bar, uint32_t bytes, uint32_t lead) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %2, 0;\n\t"
        "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}"
        ::"r"(bar), "r"(bytes), "r"(lead) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();                                       // .aligned: the whole warp must arrive together
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The two halves of a cluster barrier for a CTA that is done with its peers' shared memory before it is done with its
// own work: a thread arrives once the values it loaded from its peers are in its registers (`consumed` depends on every
// one of them, so the instruction cannot issue before they have come), goes on with work that touches no peer, and
// waits before it leaves - when the wait returns, every thread of the cluster has arrived, so nobody still reads this
// CTA's memory.  Not .aligned: threads of a warp may arrive from different places.
__device__ __forceinline__ void cluster_arrive_after(float consumed) {
    asm volatile("barrier.cluster.arrive.release;" ::"f"(consumed) : "memory");
}
__device__ __forceinline__ void cluster_wait_all() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}

// Shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart (SBO), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D float, A and B bfloat16, both K-major, M = 128, N = bn.
__host__ __device__ constexpr uint32_t make_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}


// Encode a tiled 2-D map of a bfloat16 matrix [rows, cols] with row stride `ld` elements; box = [box_rows, 64
// columns] (128 bytes), 128-byte swizzle, out-of-bounds elements read as zero.  Maps are cached by
// (address, extents, stride, box): a map depends on nothing else, so a cached one never goes stale.
int rb_tensor_map_bf16(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out);
// A map over a layer's paged cache that brings one (page, kv head)'s keys or values in one request, as
// [8-key group][64-dim half][8 keys][64 dims] (runtime.cu).
int rb_tensor_map_kv_pages(const void* cache, long long num_pages, int kv_heads, int page_size, CUtensorMap* out);

// One box of a 5-D map (coordinates innermost first) into shared memory, issued by the lane whose `lead` is not 0.
__device__ __forceinline__ void tma_load_5d_lead(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint32_t bar, uint32_t lead) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %8, 0;\n\t"
        "@q cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];\n\t}"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar), "r"(lead) : "memory");
}
// Shared-memory operand descriptor like make_smem_desc with the leading and stride offsets given (bytes).
__device__ __forceinline__ uint64_t make_smem_desc_lbo_sbo(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) |
           (1ull << 46) | (2ull << 61);
}
