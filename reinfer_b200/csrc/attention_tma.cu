// Split-K flash decoding over the paged cache with the tiles brought in by TMA.
//
// Same arithmetic and the same division of work as fa_decode_kernel (attention_mma.cu): the
// grouped query heads of one kv head are the rows of a 16-row tile, a request's keys are split
// across CTAs and, inside a CTA, across four warps (16 keys of each 64-key tile per warp),
// mma.sync m16n8k16 with an online softmax in float, merge in shared memory, then across CTAs.
// A fifth warp is the producer: it runs ahead of the four by the depth of the pipeline (full and
// empty mbarriers per stage), reading the block table 32 entries at a time.
// What differs is how keys and values reach shared memory: one layer of the cache is described
// to the TMA unit as a 2-D bfloat16 matrix [pages * 2 * kv_heads * page_size, head_dim], and one
// elected thread issues a box copy (cp.async.bulk.tensor) per page, per K/V and per 64-column
// half, completing on an mbarrier - a handful of instructions per 32 KB tile where the cp.async
// loader spends thousands, which is what held that kernel at a third of the memory bandwidth.
// Tiles land in the 128-byte swizzled layout, so ldmatrix needs no padding to avoid conflicts.
//
// A box copy brings whole pages.  Slots of the request's last page beyond its length hold
// whatever was there; the rows of the last tile at or beyond the length are therefore zeroed in
// shared memory before use, and shared memory is zeroed once at the start, so that nothing but
// the request's own keys and values ever reaches the arithmetic.
// Needs a page size that is a power of two >= 8 and head_dim % 8 == 0 (else fa_decode_kernel).
#define RB_UNIT 2
#include "sm100.cuh"
#include <stdlib.h>

#define FT_WARPS 4
#define FT_THREADS 160                       // four consumer warps and one producer warp
#define FT_BN 64
#define FT_HALF_BYTES (FT_BN * 128)          // 64 keys x 128 bytes

struct FtArgs {
    const bf16* q;
    const int* block_table;
    const int* cu_q;
    const int* kv_len;
    bf16* out;
    float* part_o;
    float* part_lse;
    int QH, KH, d, page_size, page_shift, max_pages, window;
    int Gc, chunks, first_entry, n_entries, n_splits;
    float scale_log2;
    const void* next_w;                     // decode: a range to call into L2 once this CTA's tiles are requested
    long long next_bytes;
    int cluster_merge;                      // decode: the CTAs of one (request, kv head) are a cluster and merge themselves
};

// With -DRB_TIMELINE a caller may hand the decode kernel a buffer of eight 64-bit words per CTA (linear block index) that
// get the global timer at: 0 the CTA's start, 1 shared memory zeroed, 2 the kernels before done, 3 the first tile landed,
// 4 the last tile used, 5 this CTA's part sent, 6 the cluster's barrier passed, 7 the end.
#ifdef RB_TIMELINE
__device__ unsigned long long* g_ft_trace = nullptr;
extern "C" int rb_fa_decode_trace(unsigned long long* buf) { return (int)cudaMemcpyToSymbol(g_ft_trace, &buf, sizeof(buf)); }
__device__ __forceinline__ unsigned long long ft_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define FT_T(slot) do { if (g_ft_trace) g_ft_trace[(size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + (slot)] = ft_now(); } while (0)
#else
#define FT_T(slot) do { } while (0)
#endif

struct FtShared {
    unsigned long long full[4];
    unsigned long long empty[4];
    int abort_flag;
};

__device__ __forceinline__ void ft_ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ft_ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ft_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ft_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// byte offset of 16-byte chunk `chunk` of row `row` in a tile of 64-column halves, 128-byte swizzle
__device__ __forceinline__ uint32_t ft_off(int row, int chunk, int half_bytes) {
    return (uint32_t)((chunk >> 3) * half_bytes + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// The end of the decode kernel: its four warps hold partial results (o, running maximum m, sum l) for the same 16 rows
// over different keys.  ft_merge_park puts them side by side in shared memory - rows of heads that exist only; a row is
// 8 floats longer than the head, so that the 8-byte stores of a warp's lanes fall into 32 different banks; sF gets
// [warp][16] maxima and, 64 floats on, sums.  After a barrier ft_merge_weights lets one thread per row turn them into
// each warp's share of the row (exp2(m_w - M) / L, in sF's first half) and the row's log-sum-exp; after another barrier a
// row's merged value for a dim is the sum over the warps of their value times their share: no exponential and no
// division per element.
template <int D>
__device__ __forceinline__ void ft_merge_park(float* sO, float* sF, const float (&o)[D / 8][4], const float (&m)[2], float (&l)[2],
                                              int Gc, int warp, int lane) {
    constexpr int SD = D + 8;
    const int row0 = lane >> 2;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        const int dim = j * 8 + 2 * (lane & 3);
        if (row0 < Gc) *reinterpret_cast<float2*>(sO + (warp * 16 + row0) * SD + dim) = make_float2(o[j][0], o[j][1]);
        if (row0 + 8 < Gc) *reinterpret_cast<float2*>(sO + (warp * 16 + row0 + 8) * SD + dim) = make_float2(o[j][2], o[j][3]);
    }
    if ((lane & 3) == 0) {
        sF[warp * 16 + row0] = m[0]; sF[warp * 16 + row0 + 8] = m[1];
        sF[FT_WARPS * 16 + warp * 16 + row0] = l[0]; sF[FT_WARPS * 16 + warp * 16 + row0 + 8] = l[1];
    }
}
__device__ __forceinline__ void ft_merge_weights(float* sF, float* sLse, int Gc) {
    const int row = threadIdx.x;
    if (row >= Gc) return;
    float mw[FT_WARPS], M = -INFINITY, L = 0.0f;
#pragma unroll
    for (int w = 0; w < FT_WARPS; ++w) { mw[w] = sF[w * 16 + row]; M = fmaxf(M, mw[w]); }
#pragma unroll
    for (int w = 0; w < FT_WARPS; ++w) {
        mw[w] = M > -INFINITY ? exp2f(mw[w] - M) : 0.0f;
        L += sF[FT_WARPS * 16 + w * 16 + row] * mw[w];
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
    for (int w = 0; w < FT_WARPS; ++w) sF[w * 16 + row] = mw[w] * inv;
    sLse[row] = L > 0.0f ? M + log2f(L) : -INFINITY;
}

// P5: the map is the 5-D one of runtime.cu (head size 128): ONE request brings a page's keys (or values) for this kv head,
// as [8-key group][64-dim half][8 keys][64 dims] - groups 2,048 bytes apart, a group's second half 1,024 bytes on - instead
// of one request per page and half into [half][64 keys][64 dims].
template <int HALVES, int NST, bool P5>
__global__ void __launch_bounds__(FT_THREADS)
fa_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const FtArgs a) {
    RB_TL(4);
    constexpr int D = HALVES * 64;
    constexpr int KV_BYTES = HALVES * FT_HALF_BYTES;           // one K (or V) tile
    constexpr int STAGE = 2 * KV_BYTES;
    constexpr int Q_HALF = 16 * 128;
    // byte offset of 16-byte chunk c of key `row` inside a key (or value) tile
    auto kv_off = [](int row, int c) -> uint32_t {
        return P5 ? (uint32_t)((row >> 3) * 2048 + (c >> 3) * 1024 + (row & 7) * 128 + (((c & 7) ^ (row & 7)) << 4))
                  : ft_off(row, c, FT_HALF_BYTES);
    };
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = smem;
    unsigned char* sQ = smem + NST * STAGE;
    FtShared* sh = (FtShared*)(sQ + HALVES * Q_HALF);
    const uint32_t stages_u = smem_u32(stages), sQ_u = smem_u32(sQ);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sh->abort_flag;

    if (threadIdx.x == 0) {
        FT_T(0);
        for (int s = 0; s < NST; ++s) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), FT_WARPS); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // shared memory starts at zero: rows that no copy fills are then finite
    for (int i = threadIdx.x; i < (NST * STAGE + HALVES * Q_HALF) / 16; i += FT_THREADS)
        reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeroing precedes the TMA writes
    __syncthreads();
    if (threadIdx.x == 0) FT_T(1);
    pdl_trigger();

    // The step's tables (lengths, block table) were complete before its first kernel began, and the keys of
    // earlier positions were written by earlier steps: both may be read while the kernels before this one still
    // run.  Only the query rows and the new token's key and value wait for them.
    // CTAs start in the order of their linear index: x (the kv head and chunk) fastest, then y (the entry).  A caller
    // that names its longest requests first thus has the CTAs with most keys begin first and the short ones fill
    // the slots as they come free - which is what balances a batch of unequal lengths.
    const int e = a.first_entry + blockIdx.y;
    const int kh = blockIdx.x / a.chunks, chunk = blockIdx.x % a.chunks;
    const int head0 = kh * (a.QH / a.KH) + chunk * a.Gc;
    const int split = blockIdx.z;
    const int kv_end = a.kv_len[e];
    const int pos = kv_end - 1;
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int tok = a.cu_q[e];
    const int* bt = a.block_table + (size_t)e * a.max_pages;
    const int t_lo = lo / FT_BN, t_hi = pos / FT_BN + 1;
    const int per = (t_hi - t_lo + a.n_splits - 1) / a.n_splits;
    const int t_begin = t_lo + split * per, t_end = min(t_hi, t_begin + per);
    const int n_tiles = max(0, t_end - t_begin);

    if (warp < FT_WARPS) {
        pdl_wait();
        RB_TL_MARK();
        if (threadIdx.x == 0) FT_T(2);
        // Q rows (row r = query head head0 + r) into the swizzled layout, by the consumer warps that read them
        for (int i = threadIdx.x; i < a.Gc * (a.d / 8); i += FT_WARPS * 32) {
            const int row = i / (a.d / 8), c = i % (a.d / 8);
            const uint4 v = *reinterpret_cast<const uint4*>(a.q + ((size_t)tok * a.QH + head0 + row) * a.d + c * 8);
            *reinterpret_cast<uint4*>(sQ + ft_off(row, c, Q_HALF)) = v;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(FT_WARPS * 32) : "memory");
    }

    const int box_rows = min(a.page_size, FT_BN);
    const int subs = FT_BN / box_rows;
    const int rows_per_page2 = 2 * a.KH * a.page_size;            // matrix rows of one page (K and V, all heads)
    int issued = 0;                                               // producer: tiles whose copies were issued

    const int row0 = lane >> 2;
    const int pos0 = row0 < a.Gc ? pos : -1, pos1 = row0 + 8 < a.Gc ? pos : -1;
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    const int koff = warp * 16;

    if (warp == FT_WARPS) {
        // ---- producer warp: runs ahead of the consumers by up to NST tiles --------------------
        // Block-table entries are fetched 32 at a time by the whole warp and handed to lane 0.
        int cached_first = 0, cached = -1;                        // page index of lane 0's entry; entry of this lane
        bool have = false, waited = false;
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % NST;
            const int k0 = (t_begin + it) * FT_BN;
            if (!waited && k0 + FT_BN > pos) { pdl_wait(); waited = true; }   // the tile with this step's key and value
            const int pi0 = k0 >> a.page_shift;
            const int need_last = (k0 + (subs - 1) * box_rows) >> a.page_shift;
            if (!have || need_last >= cached_first + 32) {
                cached_first = pi0;
                cached = (pi0 + lane < a.max_pages) ? bt[pi0 + lane] : -1;
                have = true;
            }
            int pages[8];
            int n_valid = 0;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int key = k0 + u * box_rows;
                const int idx = (key >> a.page_shift) - cached_first;
                const int pg = __shfl_sync(0xffffffffu, cached, idx & 31);
                pages[u] = (u < subs && key < kv_end) ? pg : -1;
                n_valid += pages[u] >= 0;
            }
            // every lane waits, lane 0's requests take effect (a lane alone inside a branch pays for each of them)
            const uint32_t lead = lane == 0 ? 1u : 0u;
            if (it >= NST && !mbar_wait(smem_u32(&sh->empty[s]), ((it / NST) & 1) ^ 1, abort_flag, 5)) break;
            const uint32_t full = smem_u32(&sh->full[s]);
            mbar_expect_tx_lead(full, (uint32_t)(n_valid * 2 * HALVES * box_rows * 128), lead);
            const uint32_t dst0 = stages_u + s * STAGE;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (pages[u] >= 0) {
                    const int key = k0 + u * box_rows;
                    if (P5) {
                        const int grp = (key & (a.page_size - 1)) >> 3, j = pages[u] * 2 * a.KH + kh;
                        const uint32_t dst = dst0 + (uint32_t)(u * (box_rows >> 3) * 2048);
                        tma_load_5d_lead(dst, &map_kv, 0, 0, 0, grp, j, full, lead);
                        tma_load_5d_lead(dst + KV_BYTES, &map_kv, 0, 0, 0, grp, j + a.KH, full, lead);
                    } else {
                        const int y = pages[u] * rows_per_page2 + kh * a.page_size + (key & (a.page_size - 1));
#pragma unroll
                        for (int h = 0; h < HALVES; ++h) {
                            tma_load_2d_lead(dst0 + h * FT_HALF_BYTES + u * box_rows * 128, &map_kv, h * 64, y, full, lead);
                            tma_load_2d_lead(dst0 + KV_BYTES + h * FT_HALF_BYTES + u * box_rows * 128, &map_kv, h * 64,
                                             y + a.KH * a.page_size, full, lead);
                        }
                    }
                }
            }
            issued = it + 1;
        }
        // this CTA's keys and values are all requested: while they arrive, are used and merged, and the kernels after
        // this one start up, memory would idle - the weights that the next product streams are called into L2 now
        // (by this warp, which has nothing left to do; the consumers' merge waits for nobody)
        if (lane == 0)
            l2_prefetch_share(a.next_w, a.next_bytes, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                              gridDim.x * gridDim.y * gridDim.z);
    } else {
        // ---- consumer warps --------------------------------------------------------------------
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % NST;
            if (!mbar_wait(smem_u32(&sh->full[s]), (it / NST) & 1, abort_flag, 4)) break;
            if (it == 0 && threadIdx.x == 0) FT_T(3);
            const uint32_t sK = stages_u + s * STAGE, sV = sK + KV_BYTES;
            const int k0 = (t_begin + it) * FT_BN;
            if (k0 + FT_BN > kv_end) {
                // the request's last tile: slots of its last page beyond its length hold foreign data
                for (int i = threadIdx.x; i < FT_BN * HALVES * 8; i += FT_WARPS * 32) {
                    const int row = i / (HALVES * 8), c = i % (HALVES * 8);
                    if (k0 + row >= kv_end) {
                        *reinterpret_cast<uint4*>(stages + s * STAGE + kv_off(row, c)) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(stages + s * STAGE + KV_BYTES + kv_off(row, c)) = make_uint4(0, 0, 0, 0);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // before a later copy refills this stage
                asm volatile("bar.sync 1, %0;" ::"n"(FT_WARPS * 32) : "memory");   // the four consumer warps
            }
            // S = Q K^T for this warp's 16 keys
            float sc[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f; }
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t qa[4], kb[4];
                ft_ldsm_x4(qa, sQ_u + ft_off((lane & 7) + 8 * ((lane >> 3) & 1), ks * 2 + (lane >> 4), Q_HALF));
                ft_ldsm_x4(kb, sK + kv_off(koff + (lane & 7) + 8 * (lane >> 4), ks * 2 + ((lane >> 3) & 1)));
                ft_mma(sc[0], qa, kb[0], kb[1]);
                ft_mma(sc[1], qa, kb[2], kb[3]);
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int key = k0 + koff + j * 8 + 2 * (lane & 3);
                sc[j][0] = (key >= lo && key <= pos0) ? sc[j][0] * a.scale_log2 : -INFINITY;
                sc[j][1] = (key + 1 >= lo && key + 1 <= pos0) ? sc[j][1] * a.scale_log2 : -INFINITY;
                sc[j][2] = (key >= lo && key <= pos1) ? sc[j][2] * a.scale_log2 : -INFINITY;
                sc[j][3] = (key + 1 >= lo && key + 1 <= pos1) ? sc[j][3] * a.scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
            const float b0 = mn0 == -INFINITY ? 0.0f : mn0, b1 = mn1 == -INFINITY ? 0.0f : mn1;
            const float c0 = exp2f(m[0] - b0), c1 = exp2f(m[1] - b1);
            m[0] = mn0; m[1] = mn1;
            uint32_t pa[4];
            {
                const float e0 = exp2f(sc[0][0] - b0), e1 = exp2f(sc[0][1] - b0), e2 = exp2f(sc[0][2] - b1), e3 = exp2f(sc[0][3] - b1);
                const float f0 = exp2f(sc[1][0] - b0), f1 = exp2f(sc[1][1] - b0), f2 = exp2f(sc[1][2] - b1), f3 = exp2f(sc[1][3] - b1);
                l[0] = l[0] * c0 + (e0 + e1) + (f0 + f1);
                l[1] = l[1] * c1 + (e2 + e3) + (f2 + f3);
                pa[0] = ft_pack(e0, e1); pa[1] = ft_pack(e2, e3); pa[2] = ft_pack(f0, f1); pa[3] = ft_pack(f2, f3);
            }
#pragma unroll
            for (int j = 0; j < D / 8; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                uint32_t vb[4];
                ft_ldsm_x4_trans(vb, sV + kv_off(koff + (lane & 7) + 8 * ((lane >> 3) & 1), dp * 2 + (lane >> 4)));
                ft_mma(o[2 * dp], pa, vb[0], vb[1]);
                ft_mma(o[2 * dp + 1], pa, vb[2], vb[3]);
            }
            // this warp is done with the stage: the producer may refill it once all four are
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->empty[s]));
        }
        if (threadIdx.x == 0) FT_T(4);
    }
    __syncthreads();
    const bool aborted = *abort_flag != 0;
    if (aborted) {
        // copies that were issued but never consumed still write this CTA's shared memory: wait for them
        if (threadIdx.x == FT_WARPS * 32)
            for (int it = max(0, issued - NST); it < issued; ++it)
                mbar_drain(smem_u32(&sh->full[it % NST]), (it / NST) & 1);
        __syncthreads();
        if (!a.cluster_merge) return;
    }
    if (a.cluster_merge) {
        // The splits of one (request, kv head) are the CTAs of a cluster (rank = split).  Each merges its four warps,
        // then writes its result - dims [r*dq, (r+1)*dq) to CTA r, its log-sum-exp to all - straight into the
        // receiving CTAs' shared memory; after one cluster barrier every CTA combines the parts that arrived for its
        // own dims (ascending split order, as the merge kernel does) and stores them.  Every thread of every CTA
        // reaches the barrier, whatever happened before; nobody reads remote memory after it.
        float* recv_o = reinterpret_cast<float*>(sQ + HALVES * Q_HALF + 256);   // [split][Gc][dq], behind FtShared
        float* recv_l = recv_o + 16 * D + 128;                                  // [split][16]
        const int dq = (a.d + a.n_splits - 1) / a.n_splits;
        if (!aborted && warp < FT_WARPS) {
            constexpr int SD = D + 8;
            float* sO = reinterpret_cast<float*>(stages);
            float* sF = sO + FT_WARPS * 16 * SD;                   // [warp][16]: a warp's share of a row, after ft_merge_weights
            float* sLse = sF + 2 * FT_WARPS * 16;                  // [16]
            ft_merge_park<D>(sO, sF, o, m, l, a.Gc, warp, lane);
            asm volatile("bar.sync 1, %0;" ::"n"(FT_WARPS * 32) : "memory");
            ft_merge_weights(sF, sLse, a.Gc);
            asm volatile("bar.sync 1, %0;" ::"n"(FT_WARPS * 32) : "memory");
            // a thread takes one dim of every row: its owner and the address there are found once
            for (int dim = threadIdx.x; dim < a.d; dim += FT_WARPS * 32) {
                const int owner = dim / dq, dl = dim - owner * dq;
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote)
                             : "r"(smem_u32(recv_o + (split * a.Gc) * dq + dl)), "r"((uint32_t)owner));
#pragma unroll 4
                for (int row = 0; row < a.Gc; ++row) {
                    float O = 0.0f;
#pragma unroll
                    for (int w = 0; w < FT_WARPS; ++w) O += sO[(w * 16 + row) * SD + dim] * sF[w * 16 + row];
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)(row * dq) * 4u), "f"(O) : "memory");
                }
            }
            // every row's log-sum-exp, to every CTA of the cluster
            for (int i = threadIdx.x; i < a.Gc * a.n_splits; i += FT_WARPS * 32) {
                const int row = i / a.n_splits, target = i - row * a.n_splits;
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote)
                             : "r"(smem_u32(recv_l + split * 16 + row)), "r"((uint32_t)target));
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(sLse[row]) : "memory");
            }
        }
        __syncwarp();
        if (threadIdx.x == 0) FT_T(5);
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (threadIdx.x == 0) FT_T(6);
        if (aborted || warp == FT_WARPS) return;
        for (int i = threadIdx.x; i < a.Gc * dq; i += FT_WARPS * 32) {
            const int row = i / dq, dl = i - row * dq;
            const int dim = split * dq + dl;
            if (dim >= a.d) continue;
            float M = -INFINITY;
            for (int s2 = 0; s2 < a.n_splits; ++s2) M = fmaxf(M, recv_l[s2 * 16 + row]);
            float W = 0.0f, O = 0.0f;
            if (M > -INFINITY) {
                for (int s2 = 0; s2 < a.n_splits; ++s2) {
                    const float w = exp2f(recv_l[s2 * 16 + row] - M);
                    W += w;
                    O += w * recv_o[(s2 * a.Gc + row) * dq + dl];
                }
            }
            a.out[((size_t)tok * a.QH + head0 + row) * a.d + dim] = __float2bfloat16_rn(W > 0.0f ? O / W : 0.0f);
        }
        if (threadIdx.x == 0) FT_T(7);
        return;
    }
    if (warp == FT_WARPS) return;                              // the producer has no part in the merge
    // merge the four warps (fixed order), then store or hand to the merge kernel
    constexpr int SD = D + 8;
    float* sO = reinterpret_cast<float*>(stages);              // [warp][16][D + 8]
    float* sF = sO + FT_WARPS * 16 * SD;
    float* sLse = sF + 2 * FT_WARPS * 16;
    ft_merge_park<D>(sO, sF, o, m, l, a.Gc, warp, lane);
    asm volatile("bar.sync 1, %0;" ::"n"(FT_WARPS * 32) : "memory");
    ft_merge_weights(sF, sLse, a.Gc);
    asm volatile("bar.sync 1, %0;" ::"n"(FT_WARPS * 32) : "memory");
    for (int dim = threadIdx.x; dim < a.d; dim += FT_WARPS * 32) {
#pragma unroll 4
        for (int row = 0; row < a.Gc; ++row) {
            float O = 0.0f;
#pragma unroll
            for (int w = 0; w < FT_WARPS; ++w) O += sO[(w * 16 + row) * SD + dim] * sF[w * 16 + row];
            const int head = head0 + row;
            if (a.n_splits == 1) {
                a.out[((size_t)tok * a.QH + head) * a.d + dim] = __float2bfloat16_rn(O);
            } else {
                const size_t pi = ((size_t)(tok - a.cu_q[a.first_entry]) * a.QH + head) * a.n_splits + split;
                a.part_o[pi * a.d + dim] = O;
                if (dim == 0) a.part_lse[pi] = sLse[row];
            }
        }
    }
}

// ------------------------------------------------------------------------------- prefill
// Entries that bring several tokens.  A CTA owns 64 rows = 64/Gc tokens x Gc grouped query heads of one
// kv head; each of the four consumer warps owns 16 rows and walks all 64 keys of every tile; the fifth
// warp feeds the tiles by TMA as in the decode kernel.  Reads every page of the request, those that
// earlier steps wrote included.  Q fragments stay in registers for head sizes up to 128.
template <int HALVES, int NST>
__global__ void __launch_bounds__(FT_THREADS)
fa_prefill_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const FtArgs a) {
    RB_TL(10);
    constexpr int D = HALVES * 64;
    constexpr int KV_BYTES = HALVES * FT_HALF_BYTES;
    constexpr int STAGE = 2 * KV_BYTES;
    constexpr int Q_HALF = 64 * 128;                           // 64 rows x 128 bytes
    constexpr bool Q_IN_REGS = HALVES <= 2;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = smem;
    unsigned char* sQ = smem + NST * STAGE;
    FtShared* sh = (FtShared*)(sQ + HALVES * Q_HALF);
    const uint32_t stages_u = smem_u32(stages), sQ_u = smem_u32(sQ);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sh->abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), FT_WARPS); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < (NST * STAGE + HALVES * Q_HALF) / 16; i += FT_THREADS)
        reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    pdl_trigger();
    pdl_wait();

    const int tpt = FT_BN / a.Gc;                              // tokens per CTA (64 rows)
    int tile = blockIdx.x, e = a.first_entry, q_len = 0;
    for (; e < a.first_entry + a.n_entries; ++e) {
        q_len = a.cu_q[e + 1] - a.cu_q[e];
        const int nt = (q_len + tpt - 1) / tpt;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e >= a.first_entry + a.n_entries) return;              // uniform: the whole CTA leaves
    const int q0 = tile * tpt;
    const int n_tok = min(tpt, q_len - q0);
    const int kh = blockIdx.y / a.chunks, chunk = blockIdx.y % a.chunks;
    const int head0 = kh * (a.QH / a.KH) + chunk * a.Gc;
    const int kv_end = a.kv_len[e];
    const int start_pos = kv_end - q_len;
    const int tok_base = a.cu_q[e] + q0;
    const int* bt = a.block_table + (size_t)e * a.max_pages;
    const int pos_min = start_pos + q0, pos_max = start_pos + q0 + n_tok - 1;
    const int lo_min = a.window > 0 ? max(0, pos_min - a.window + 1) : 0;
    const int t_begin = lo_min / FT_BN, t_end = pos_max / FT_BN + 1;
    const int n_tiles = t_end - t_begin;

    for (int i = threadIdx.x; i < n_tok * a.Gc * (a.d / 8); i += FT_THREADS) {
        const int row = i / (a.d / 8), c = i % (a.d / 8);
        const int ti = row / a.Gc, g = row % a.Gc;
        const uint4 v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(tok_base + ti) * a.QH + head0 + g) * a.d + c * 8);
        *reinterpret_cast<uint4*>(sQ + ft_off(row, c, Q_HALF)) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    const int box_rows = min(a.page_size, FT_BN);
    const int subs = FT_BN / box_rows;
    const int rows_per_page2 = 2 * a.KH * a.page_size;
    int issued = 0;

    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    const int r0 = (warp & 3) * 16 + (lane >> 2), r1 = r0 + 8;
    const int ti0 = r0 / a.Gc, ti1 = r1 / a.Gc;

    if (warp == FT_WARPS) {
        int cached_first = 0, cached = -1;
        bool have = false;
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % NST;
            const int k0 = (t_begin + it) * FT_BN;
            const int pi0 = k0 >> a.page_shift;
            const int need_last = (k0 + (subs - 1) * box_rows) >> a.page_shift;
            if (!have || need_last >= cached_first + 32) {
                cached_first = pi0;
                cached = (pi0 + lane < a.max_pages) ? bt[pi0 + lane] : -1;
                have = true;
            }
            int pages[8];
            int n_valid = 0;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int key = k0 + u * box_rows;
                const int pg = __shfl_sync(0xffffffffu, cached, ((key >> a.page_shift) - cached_first) & 31);
                pages[u] = (u < subs && key < kv_end) ? pg : -1;
                n_valid += pages[u] >= 0;
            }
            bool ok = true;
            if (lane == 0) {
                if (it >= NST) ok = mbar_wait(smem_u32(&sh->empty[s]), ((it / NST) & 1) ^ 1, abort_flag, 7);
                if (ok) {
                    const uint32_t full = smem_u32(&sh->full[s]);
                    mbar_expect_tx(full, (uint32_t)(n_valid * 2 * HALVES * box_rows * 128));
                    const uint32_t dst0 = stages_u + s * STAGE;
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        if (pages[u] >= 0) {
                            const int key = k0 + u * box_rows;
                            const int y = pages[u] * rows_per_page2 + kh * a.page_size + (key & (a.page_size - 1));
#pragma unroll
                            for (int h = 0; h < HALVES; ++h) {
                                tma_load_2d(dst0 + h * FT_HALF_BYTES + u * box_rows * 128, &map_kv, h * 64, y, full);
                                tma_load_2d(dst0 + KV_BYTES + h * FT_HALF_BYTES + u * box_rows * 128, &map_kv, h * 64,
                                            y + a.KH * a.page_size, full);
                            }
                        }
                    }
                    issued = it + 1;
                }
            }
            if (!__shfl_sync(0xffffffffu, (int)ok, 0)) break;
        }
    } else {
        const int pos0 = ti0 < n_tok ? start_pos + q0 + ti0 : -1, pos1 = ti1 < n_tok ? start_pos + q0 + ti1 : -1;
        const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0, lo1 = a.window > 0 ? max(0, pos1 - a.window + 1) : 0;
        // keys beyond the last row of this warp are masked for all its rows: it may skip those tiles
        const int warp_last_tok = min(n_tok - 1, (warp * 16 + 15) / a.Gc);
        const int warp_t_end = (warp * 16) / a.Gc < n_tok ? (start_pos + q0 + warp_last_tok) / FT_BN + 1 : 0;
        uint32_t qreg[Q_IN_REGS ? D / 16 : 1][4];
        if (Q_IN_REGS) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ft_ldsm_x4(qreg[ks], sQ_u + ft_off(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), ks * 2 + (lane >> 4), Q_HALF));
        }
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % NST;
            if (!mbar_wait(smem_u32(&sh->full[s]), (it / NST) & 1, abort_flag, 6)) break;
            const uint32_t sK = stages_u + s * STAGE, sV = sK + KV_BYTES;
            const int k0 = (t_begin + it) * FT_BN;
            if (k0 + FT_BN > kv_end) {
                for (int i = threadIdx.x; i < FT_BN * HALVES * 8; i += FT_WARPS * 32) {
                    const int row = i / (HALVES * 8), c = i % (HALVES * 8);
                    if (k0 + row >= kv_end) {
                        *reinterpret_cast<uint4*>(stages + s * STAGE + ft_off(row, c, FT_HALF_BYTES)) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(stages + s * STAGE + KV_BYTES + ft_off(row, c, FT_HALF_BYTES)) = make_uint4(0, 0, 0, 0);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, %0;" ::"n"(FT_WARPS * 32) : "memory");
            }
            if (t_begin + it < warp_t_end) {
                float sc[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f; }
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t qa[4];
                    if (Q_IN_REGS) { qa[0] = qreg[ks][0]; qa[1] = qreg[ks][1]; qa[2] = qreg[ks][2]; qa[3] = qreg[ks][3]; }
                    else ft_ldsm_x4(qa, sQ_u + ft_off(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), ks * 2 + (lane >> 4), Q_HALF));
#pragma unroll
                    for (int jp = 0; jp < 4; ++jp) {
                        uint32_t kb[4];
                        ft_ldsm_x4(kb, sK + ft_off(jp * 16 + (lane & 7) + 8 * (lane >> 4), ks * 2 + ((lane >> 3) & 1), FT_HALF_BYTES));
                        ft_mma(sc[2 * jp], qa, kb[0], kb[1]);
                        ft_mma(sc[2 * jp + 1], qa, kb[2], kb[3]);
                    }
                }
                const bool need_mask = (k0 + FT_BN - 1 > min(pos0 < 0 ? -1 : pos0, pos1 < 0 ? -1 : pos1)) || (a.window > 0);
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int key = k0 + j * 8 + 2 * (lane & 3);
                    if (need_mask) {
                        sc[j][0] = (key >= lo0 && key <= pos0) ? sc[j][0] * a.scale_log2 : -INFINITY;
                        sc[j][1] = (key + 1 >= lo0 && key + 1 <= pos0) ? sc[j][1] * a.scale_log2 : -INFINITY;
                        sc[j][2] = (key >= lo1 && key <= pos1) ? sc[j][2] * a.scale_log2 : -INFINITY;
                        sc[j][3] = (key + 1 >= lo1 && key + 1 <= pos1) ? sc[j][3] * a.scale_log2 : -INFINITY;
                    } else {
                        sc[j][0] *= a.scale_log2; sc[j][1] *= a.scale_log2; sc[j][2] *= a.scale_log2; sc[j][3] *= a.scale_log2;
                    }
                    mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
                    mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
                const float b0 = mn0 == -INFINITY ? 0.0f : mn0, b1 = mn1 == -INFINITY ? 0.0f : mn1;
                const float c0 = exp2f(m[0] - b0), c1 = exp2f(m[1] - b1);
                m[0] = mn0; m[1] = mn1;
                float sum0 = 0.0f, sum1 = 0.0f;
                uint32_t p[8][2];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float e0 = exp2f(sc[j][0] - b0), e1 = exp2f(sc[j][1] - b0);
                    const float e2 = exp2f(sc[j][2] - b1), e3 = exp2f(sc[j][3] - b1);
                    sum0 += e0 + e1; sum1 += e2 + e3;
                    p[j][0] = ft_pack(e0, e1);
                    p[j][1] = ft_pack(e2, e3);
                }
                l[0] = l[0] * c0 + sum0;
                l[1] = l[1] * c1 + sum1;
#pragma unroll
                for (int j = 0; j < D / 8; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint32_t pa[4] = {p[2 * kk][0], p[2 * kk][1], p[2 * kk + 1][0], p[2 * kk + 1][1]};
#pragma unroll
                    for (int dp = 0; dp < D / 16; ++dp) {
                        uint32_t vb[4];
                        ft_ldsm_x4_trans(vb, sV + ft_off(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dp * 2 + (lane >> 4), FT_HALF_BYTES));
                        ft_mma(o[2 * dp], pa, vb[0], vb[1]);
                        ft_mma(o[2 * dp + 1], pa, vb[2], vb[3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->empty[s]));
        }
    }
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == FT_WARPS * 32)
            for (int it = max(0, issued - NST); it < issued; ++it)
                mbar_drain(smem_u32(&sh->full[it % NST]), (it / NST) & 1);
        __syncthreads();
        return;
    }
    if (warp == FT_WARPS) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    const float inv0 = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv1 = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        const int dim = j * 8 + 2 * (lane & 3);
        if (dim >= a.d) continue;
        if (ti0 < n_tok)
            *reinterpret_cast<uint32_t*>(a.out + ((size_t)(tok_base + ti0) * a.QH + head0 + r0 % a.Gc) * a.d + dim) = ft_pack(o[j][0] * inv0, o[j][1] * inv0);
        if (ti1 < n_tok)
            *reinterpret_cast<uint32_t*>(a.out + ((size_t)(tok_base + ti1) * a.QH + head0 + r1 % a.Gc) * a.d + dim) = ft_pack(o[j][2] * inv1, o[j][3] * inv1);
    }
}

// out[t, h, :] = sum_s w_s o_s / sum_s w_s,  w_s = 2^(lse_s - max lse), splits in ascending order
constexpr int FT_MERGE_UNROLL = 16;
__global__ void ft_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, bf16* __restrict__ out,
                                int first_tok, int QH, int d, int n_splits) {
    RB_TL(5);
    pdl_trigger(); pdl_wait();
    RB_TL_MARK();
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t base = ((size_t)t * QH + h) * n_splits;
    bf16* orow = out + ((size_t)(first_tok + t) * QH + h) * d;
    if (n_splits <= FT_MERGE_UNROLL) {
        // the usual case: every load of a thread is issued before the first is used (one trip to L2, not two)
        for (int dim = threadIdx.x; dim < d; dim += blockDim.x) {
            float l[FT_MERGE_UNROLL], o[FT_MERGE_UNROLL];
#pragma unroll
            for (int s = 0; s < FT_MERGE_UNROLL; ++s) {
                l[s] = s < n_splits ? part_lse[base + s] : -INFINITY;
                o[s] = s < n_splits ? part_o[(base + s) * d + dim] : 0.0f;
            }
            float M = -INFINITY;
#pragma unroll
            for (int s = 0; s < FT_MERGE_UNROLL; ++s) M = fmaxf(M, l[s]);
            float W = 0.0f, O = 0.0f;
            if (M > -INFINITY) {
#pragma unroll
                for (int s = 0; s < FT_MERGE_UNROLL; ++s) {
                    if (s < n_splits) {
                        const float w = exp2f(l[s] - M);
                        W += w;
                        O += w * o[s];
                    }
                }
            }
            orow[dim] = __float2bfloat16_rn(W > 0.0f ? O / W : 0.0f);
        }
        return;
    }
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_lse[base + s]);
    for (int dim = threadIdx.x; dim < d; dim += blockDim.x) {
        float W = 0.0f, O = 0.0f;
        if (M > -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float w = exp2f(part_lse[base + s] - M);
                W += w;
                O += w * part_o[(base + s) * d + dim];
            }
        }
        orow[dim] = __float2bfloat16_rn(W > 0.0f ? O / W : 0.0f);
    }
}

#define FT_MAX_CLUSTER 16                   // splits that merge themselves inside one cluster
template <int HALVES, int NST>
constexpr size_t ft_decode_smem() {
    return (size_t)NST * 2 * HALVES * FT_HALF_BYTES + HALVES * 16 * 128 + 256 +
           (size_t)(16 * HALVES * 64 + 128 + FT_MAX_CLUSTER * 16) * sizeof(float) + 1024;
}

// How many CTAs of the decode kernel for this head size can be resident at once as clusters of n (0: such clusters
// cannot be launched here).
template <int HALVES, int NST, bool P5>
static int ft_cluster_slots(int n) {
    constexpr size_t smem = ft_decode_smem<HALVES, NST>();
    if (cudaFuncSetAttribute(fa_decode_tma_kernel<HALVES, NST, P5>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(fa_decode_tma_kernel<HALVES, NST, P5>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, n); cfg.blockDim = dim3(FT_THREADS); cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = n;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, fa_decode_tma_kernel<HALVES, NST, P5>, &cfg) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return clusters * n;
}
extern "C" int rb_fa_decode_cluster_slots(int d, int n) {
    if (n < 2 || n > FT_MAX_CLUSTER) return 0;
    if (d == 128) return ft_cluster_slots<2, 3, true>(n);
    if (d <= 64) return ft_cluster_slots<1, 4, false>(n);
    if (d <= 128) return ft_cluster_slots<2, 3, false>(n);
    return ft_cluster_slots<4, 2, false>(n);
}

template <int HALVES, int NST, bool P5 = false>
static int ft_launch(const CUtensorMap& map, const FtArgs& a, cudaStream_t s) {
    constexpr size_t pipe = (size_t)NST * 2 * HALVES * FT_HALF_BYTES;
    constexpr size_t merge = ((size_t)FT_WARPS * 16 * (HALVES * 64 + 8 + 2) + 16) * sizeof(float);
    static_assert(merge <= pipe, "the merge buffers reuse the stages");
    static_assert(sizeof(FtShared) <= 256, "the cluster's receive buffers start 256 bytes behind the barriers");
    // stages, Q, barriers, and what the other splits of a cluster send: [split][Gc][dq] results + [split][16] log-sum-exps
    constexpr size_t smem = ft_decode_smem<HALVES, NST>();
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fa_decode_tma_kernel<HALVES, NST, P5>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        // clusters of more than 8 CTAs (up to 16 splits merge themselves) are not portable: the kernel has to allow them
        e = cudaFuncSetAttribute(fa_decode_tma_kernel<HALVES, NST, P5>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    const dim3 grid(a.KH * a.chunks, a.n_entries, a.n_splits);
    if (a.cluster_merge)
        return rb_launch_cluster(fa_decode_tma_kernel<HALVES, NST, P5>, grid, dim3(FT_THREADS), dim3(1, 1, a.n_splits), smem, s, map, a);
    return rb_launch(fa_decode_tma_kernel<HALVES, NST, P5>, grid, dim3(FT_THREADS), smem, s, map, a);
}

// As rb_fa_decode, with `cache` the layer's [num_pages, 2, KH, page_size, d] array described to TMA.
extern "C" int rb_fa_decode_tma(const void* q, const void* cache, long long num_pages, const int* block_table, const int* cu_q,
                                const int* kv_len, void* out, float* part_o, float* part_lse, int first_entry, int n_entries,
                                int first_tok, int n_splits, int QH, int KH, int d, int page_size, int max_pages, int window,
                                float scale, const void* next_w, long long next_bytes, void* stream) {
    if (n_entries <= 0) return 0;
    if ((uintptr_t)next_w & 15) RB_REFUSE("attention: the range to prefetch must start on a 16-byte boundary");
    if (QH <= 0 || KH <= 0 || QH % KH) RB_REFUSE("attention: %d query heads over %d kv heads", QH, KH);
    if (d <= 0 || d % 8 || d > 256) RB_REFUSE("attention (TMA): head_dim %d is not a multiple of 8 up to 256", d);
    int shift = -1;
    for (int s = 3; s < 16; ++s) if ((1 << s) == page_size) shift = s;
    if (shift < 0) RB_REFUSE("attention (TMA): page size %d is not a power of two >= 8", page_size);
    if (n_splits < 1 || n_splits > 65535) RB_REFUSE("attention: %d splits", n_splits);
    if (n_entries > 65535) RB_REFUSE("attention: %d decoding entries in one launch (at most 65535)", n_entries);
    // up to 16 splits are the CTAs of a cluster, which merge their results themselves; more go through scratch and a merge kernel
    static const char* cl_env = getenv("REINFER_B200_ATTN_CLUSTER");                // "0": always the merge kernel (for comparison)
    const bool cluster_merge = n_splits >= 2 && n_splits <= FT_MAX_CLUSTER && n_splits <= d && !(cl_env && cl_env[0] == '0') && part_o == nullptr;
    if (n_splits > 1 && !cluster_merge && (!part_o || !part_lse)) RB_REFUSE("attention: decoding in %d splits needs its scratch", n_splits);
    if (((uintptr_t)cache & 15) || ((uintptr_t)q & 15)) RB_REFUSE("attention (TMA): operands must be 16-byte aligned");
    FtArgs a{};
    a.q = (const bf16*)q; a.block_table = block_table; a.cu_q = cu_q; a.kv_len = kv_len; a.out = (bf16*)out;
    a.part_o = part_o; a.part_lse = part_lse; a.QH = QH; a.KH = KH; a.d = d; a.page_size = page_size; a.page_shift = shift;
    a.max_pages = max_pages; a.window = window;
    const int G = QH / KH;
    a.Gc = 1;
    for (int c = 16; c >= 1; --c) if (G % c == 0) { a.Gc = c; break; }
    a.chunks = G / a.Gc; a.first_entry = first_entry; a.n_entries = n_entries; a.n_splits = n_splits;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.next_w = next_w; a.next_bytes = next_bytes;
    a.cluster_merge = cluster_merge ? 1 : 0;
    CUtensorMap map;
    const int box_rows = page_size < FT_BN ? page_size : FT_BN;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (d == 128) {                                    // heads of exactly 128: a page's keys in one request
        if (rb_tensor_map_kv_pages(cache, num_pages, KH, page_size, &map)) return -1;
        rc = ft_launch<2, 3, true>(map, a, s);
    } else {
        if (rb_tensor_map_bf16(cache, num_pages * 2LL * KH * page_size, d, d, box_rows, &map)) return -1;
        if (d <= 64) rc = ft_launch<1, 4>(map, a, s);
        else if (d <= 128) rc = ft_launch<2, 3>(map, a, s);
        else rc = ft_launch<4, 2>(map, a, s);
    }
    if (rc || n_splits == 1 || cluster_merge) return rc;
    return rb_launch(ft_merge_kernel, dim3(n_entries, QH), dim3(128), 0, s, (const float*)part_o, (const float*)part_lse,
                     (bf16*)out, first_tok, QH, d, n_splits);
}

template <int HALVES, int NST>
static int ft_launch_prefill(const CUtensorMap& map, const FtArgs& a, int n_tiles, cudaStream_t s) {
    constexpr size_t smem = (size_t)NST * 2 * HALVES * FT_HALF_BYTES + HALVES * 64 * 128 + sizeof(FtShared) + 1024;
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fa_prefill_tma_kernel<HALVES, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    return rb_launch(fa_prefill_tma_kernel<HALVES, NST>, dim3(n_tiles, a.KH * a.chunks), dim3(FT_THREADS), smem, s, map, a);
}

// As rb_fa_prefill, with the key/value tiles brought in by TMA (page size a power of two >= 8).
extern "C" int rb_fa_prefill_tma(const void* q, const void* cache, long long num_pages, const int* block_table, const int* cu_q,
                                 const int* kv_len, void* out, int first_entry, int n_entries, int n_tiles, int QH, int KH, int d,
                                 int page_size, int max_pages, int window, float scale, void* stream) {
    if (n_entries <= 0 || n_tiles <= 0) return 0;
    if (QH <= 0 || KH <= 0 || QH % KH) RB_REFUSE("attention: %d query heads over %d kv heads", QH, KH);
    if (d <= 0 || d % 8 || d > 256) RB_REFUSE("attention (TMA): head_dim %d is not a multiple of 8 up to 256", d);
    int shift = -1;
    for (int s = 3; s < 16; ++s) if ((1 << s) == page_size) shift = s;
    if (shift < 0) RB_REFUSE("attention (TMA): page size %d is not a power of two >= 8", page_size);
    if (((uintptr_t)cache & 15) || ((uintptr_t)q & 15)) RB_REFUSE("attention (TMA): operands must be 16-byte aligned");
    FtArgs a{};
    a.q = (const bf16*)q; a.block_table = block_table; a.cu_q = cu_q; a.kv_len = kv_len; a.out = (bf16*)out;
    a.QH = QH; a.KH = KH; a.d = d; a.page_size = page_size; a.page_shift = shift; a.max_pages = max_pages; a.window = window;
    const int G = QH / KH;
    a.Gc = 1;
    for (int c = 16; c >= 1; --c) if (G % c == 0) { a.Gc = c; break; }
    a.chunks = G / a.Gc; a.first_entry = first_entry; a.n_entries = n_entries; a.n_splits = 1;
    a.scale_log2 = scale * 1.4426950408889634f;
    CUtensorMap map;
    const int box_rows = page_size < FT_BN ? page_size : FT_BN;
    if (rb_tensor_map_bf16(cache, num_pages * 2LL * KH * page_size, d, d, box_rows, &map)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    if (d <= 64) return ft_launch_prefill<1, 4>(map, a, n_tiles, s);
    if (d <= 128) return ft_launch_prefill<2, 2>(map, a, n_tiles, s);     // 82 KB: two CTAs per SM
    return ft_launch_prefill<4, 2>(map, a, n_tiles, s);
}

RB_STATUS_EXPORTS(rb_attn_error, rb_attn_bind_status)

RB_TL_SETTER(rb_attn_step_timeline)
