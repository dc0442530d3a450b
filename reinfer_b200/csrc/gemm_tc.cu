// The tensor-core matrix product of the bfloat16 path, written for sm_100a:
//     C[T,N] (=|+=) X[T,K] * W[N,K]^T        X, W bfloat16 K-major; accumulation in float
// TMA (cp.async.bulk.tensor) stages 128-byte-swizzled tiles of both operands in shared
// memory, one elected thread issues tcgen05.mma (kind::f16, bf16 inputs) with the
// accumulator in tensor memory, four warps read it back with tcgen05.ld and store.
//
// The operands are always swapped: the WEIGHT rows ride the instruction's M (128 output
// features per CTA) and the TOKENS ride its N (16..256).  One kernel therefore serves a
// 2,048-token prompt portion (N = 256) and a single decoded token (N = 16, operands
// padded by TMA's out-of-bounds zero fill), and in the accumulator a thread owns one
// output feature, so a warp's stores for one token are 32 consecutive features.
// Small token counts give few CTAs, so K is split across CTAs (grid.z).  Up to 8 splits form
// a thread-block cluster: every CTA parks its accumulator in its own shared memory and the
// CTAs share out the tile's tokens, each adding all ranks' partial sums for its tokens over
// distributed shared memory in rank order, and storing them.
// More splits than that go through a float workspace and a second kernel that adds in split
// order.  Either way the order is fixed and there are no atomics (the reference's two-phase
// gemv does the same, crates/cuda/kernels/gemm_m1.cu:106-123).  The reference's products are cublasGemmEx
// and scalar gemv kernels (crates/cuda/src/gemm.rs:226-372).
//
// Every wait on an mbarrier is bounded (two seconds of the global timer): after that the CTA raises
// an abort flag, its roles leave their loops, outstanding TMA loads are waited for (again
// bounded), tensor memory is freed, and an error word in global memory tells the host.
#define RB_UNIT 1
#include "sm100.cuh"
#ifndef RB_SPLIT_BARRIER
#define RB_SPLIT_BARRIER 1     // development: 0 = every thread arrives at the cluster's second barrier only after its stores
#endif
#include <stdlib.h>

#define TC_BM 128            // output features per CTA (MMA M)
#define TC_BK 64             // K elements per stage (128 bytes: one swizzle row)
#define TC_THREADS 192       // warp 0: TMA, warp 1: MMA + tensor memory, warps 2..5: epilogue

// With -DRB_TIMELINE every CTA writes globaltimer stamps of its phases (ns) to a buffer given by
// rb_gemm_timeline(): [cta][8] = start, set-up done, first tile landed, all MMAs issued, accumulator
// ready, epilogue stored/parked, cluster reduction done, end.  A development aid, off by default.
#ifdef RB_TIMELINE
__device__ unsigned long long* g_tc_timeline = nullptr;
__device__ __forceinline__ unsigned long long tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TL(slot) do { if (g_tc_timeline) g_tc_timeline[(size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + (slot)] = tl_now(); } while (0)
extern "C" int rb_gemm_timeline(unsigned long long* buf) {
    return (int)cudaMemcpyToSymbol(g_tc_timeline, &buf, sizeof(buf));
}
// The persistent kernels also write, per CTA and per tile they take (at most `g_tc_tile_cap` of them), ten words to the
// buffer of rb_gemm_tile_trace(): MMA thread: tile begun (ns), cycles it waited for operand stages, last product issued
// (ns), cycles its commits took; epilogue: accumulator ready (ns), accumulator drained (ns);
// producer: first request of the tile issued (ns), cycles it waited for free stages; MMA thread again: cycles from
// tile begun to last product issued, cycles its products took to issue.  Ten words a tile.
__device__ unsigned long long* g_tc_tiles = nullptr;
__device__ int g_tc_tile_cap = 0;
#define TT(local, slot, value) do { if (g_tc_tiles && (local) < g_tc_tile_cap) g_tc_tiles[((size_t)blockIdx.x * g_tc_tile_cap + (local)) * 10 + (slot)] = (value); } while (0)
extern "C" int rb_gemm_tile_trace(unsigned long long* buf, int cap) {
    cudaError_t e = cudaMemcpyToSymbol(g_tc_tiles, &buf, sizeof(buf));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_tc_tile_cap, &cap, sizeof(cap));
    return (int)e;
}
#else
#define TL(slot) do { } while (0)
#define TT(local, slot, value) do { } while (0)
#endif

struct TcShared {                        // after the operand stages, in dynamic shared memory
    unsigned long long full[12];
    unsigned long long empty[12];
    unsigned long long acc_full;
    uint32_t tmem_base;
    int abort_flag;
    float row_scale[256];                // the factor that each token's results are multiplied by (1 if none)
};

// What a product over one token tile may be told beside its operands.
struct TcExtra {
    // A range that the CTAs call into L2 once their own weights have arrived (null: none).
    const void* next_w;
    long long next_bytes;
    // The rows of X lack a factor: row t stands for X[t,:] / sqrt(sum_p row_sumsq[t, p] * inv_width + eps) - an
    // RMS norm whose division is left to this product's epilogue, where it costs one multiplication per
    // result (null: X is complete).  The parts are added in ascending order.
    const float* row_sumsq;
    int sumsq_parts;
    float inv_width, eps;
    // An accumulating product (out_mode 2) that is reduced inside a cluster may also prepare the rows for the RMS norm
    // that reads the sum next (null: no): prep_rows [T, N] bfloat16 gets (C + product) * prep_w per feature - the norm
    // without its division - and prep_sumsq [T, N / 128] the sum of squares of the new C over each tile's 128
    // features, from which the product that reads the rows forms their factor (row_sumsq there).
    const void* prep_w;
    int prep_w_f32;
    bf16* prep_rows;
    float* prep_sumsq;
    // The product is the attention's q/k/v projection with heads of 128 (a tile of 128 features is one head), reduced
    // inside a cluster: the CTAs do the per-head work on their sums themselves (h_q_out null: no) - the RMS norm of
    // query and key heads with h_q_w / h_k_w (null: none), the half-split rotation by positions[t] * inv_freq, queries
    // to h_q_out [T, QH, 128], keys and values into the slot h_kv_slot[t] of the layer's cache pages (what
    // qknorm_rope_append of elementwise.cu does on the stored projection; the sums are rounded to bfloat16 first, as
    // they are there).
    bf16* h_q_out;
    bf16* h_cache;
    const int* h_kv_slot;
    const int* h_positions;
    const float* h_inv_freq;
    const void* h_q_w;
    const void* h_k_w;
    int h_w_f32, h_QH, h_KH, h_page;
    float h_eps;
};

// Cosines, sines and norm weights of the four features f4 .. f4 + 3 of a query or key head for token t (heads in the
// cluster's reduction; weights 1 where the heads have no norm).
__device__ __forceinline__ void head_angles_weights(const TcExtra& ex, bool is_q, int t, int f4, float* c, float* s, float* w) {
    const void* wv = is_q ? ex.h_q_w : ex.h_k_w;
    const float pos = (float)ex.h_positions[t];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        w[i] = !wv ? 1.0f : ex.h_w_f32 ? ((const float*)wv)[f4 + i] : __bfloat162float(((const bf16*)wv)[f4 + i]);
        sincosf(pos * ex.h_inv_freq[(f4 & 63) + i], &s[i], &c[i]);
    }
}

// out_mode 0: C = acc as bf16; 1: C = acc as float; 2: C(float) += acc; 3: workspace partial (float, [split][T][N]).
// csplit > 1: the grid.z CTAs of one tile are a cluster; out_mode (0..2) is applied to the sum over the cluster.
// DUAL: W holds two matrices of N rows each (gate rows, then up rows); the CTA multiplies the same token tile
// with the matching 128 rows of both into two accumulators and stores silu(gate) * up as bfloat16
// (the reference's fused_cast_swiglu_f16, crates/cuda/kernels/dense_kernels.cu:236-248, as a GEMM epilogue).
template <int BN, int STAGES, bool DUAL>
__global__ void __launch_bounds__(TC_THREADS, (BN <= 64 ? 2 : 1))
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               void* __restrict__ C, float* __restrict__ ws, int T, int N, int K, long long ldc, int out_mode,
               int kb_per_split, int csplit, const TcExtra ex) {
    RB_TL(DUAL ? 7 : 6);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr uint32_t W1_BYTES = TC_BM * TC_BK * 2;                // 16 KB per weight tile
    constexpr uint32_t W_BYTES = (DUAL ? 2 : 1) * W1_BYTES;
    constexpr uint32_t X_BYTES = BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES;            // multiples of 1024 (BN >= 16 -> 2 KB)
    constexpr uint32_t ACC_COLS = (DUAL ? 2 : 1) * BN;
    constexpr uint32_t TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    TcShared* sh = (TcShared*)(smem + (size_t)STAGES * STAGE_BYTES);
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * BN, n0 = blockIdx.y * TC_BM, split = blockIdx.z;
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    const int kb0 = split * kb_per_split;
    const int nkb = min(kb_per_split, total_kb - kb0);
    volatile int* abort_flag = &sh->abort_flag;

    if (threadIdx.x == 0) {
        TL(0);
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), 1); }
        mbar_init(smem_u32(&sh->acc_full), 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    if (threadIdx.x == 0) TL(1);
    int issued = 0;                                   // producer: k-blocks whose loads were issued
    // heads in the cluster's reduction: what an epilogue thread needs for its first token, fetched while the weights stream
    float hp_c[4] = {1.f, 1.f, 1.f, 1.f}, hp_s[4] = {0.f, 0.f, 0.f, 0.f}, hp_w[4] = {1.f, 1.f, 1.f, 1.f};
    int hp_slot = -1;
    // an accumulating product reduced by its cluster: the old sums of this thread's first two tokens, fetched likewise
    float4 pre_a = make_float4(0.f, 0.f, 0.f, 0.f), pre_b = pre_a;

    // The two issuing warps stay converged (every lane walks the loop and waits at the barriers) and lane 0 issues
    // through predicated instructions: an issuing lane alone inside a branch pays about a hundred cycles more for
    // every asynchronous instruction.
    const uint32_t lead = lane == 0 ? 1u : 0u;
    if (warp == 0) {
        // Weights never change, so their first tiles are fetched at once, while the kernels
        // before this one may still be running; the activations wait for them to finish.
        pdl_trigger();
        const int pre = min(nkb, STAGES);
        for (int kb = 0; kb < pre; ++kb) {
            const uint32_t full = smem_u32(&sh->full[kb]);
            mbar_expect_tx_lead(full, STAGE_BYTES, lead);
            tma_load_2d_lead(smem_base + kb * STAGE_BYTES, &map_w, (kb0 + kb) * TC_BK, n0, full, lead);
            if (DUAL) tma_load_2d_lead(smem_base + kb * STAGE_BYTES + W1_BYTES, &map_w, (kb0 + kb) * TC_BK, N + n0, full, lead);
        }
        pdl_wait();
        if (lead) RB_TL_MARK();
        for (int kb = 0; kb < pre; ++kb)
            tma_load_2d_lead(smem_base + kb * STAGE_BYTES + W_BYTES, &map_x, (kb0 + kb) * TC_BK, t0, smem_u32(&sh->full[kb]), lead);
        issued = pre;
        for (int kb = pre; kb < nkb; ++kb) {
            const int s = kb % STAGES;
            const uint32_t round = kb / STAGES;
            if (!mbar_wait(smem_u32(&sh->empty[s]), (round & 1) ^ 1, abort_flag, 1)) break;
            const uint32_t full = smem_u32(&sh->full[s]);
            mbar_expect_tx_lead(full, STAGE_BYTES, lead);
            const uint32_t dst = smem_base + s * STAGE_BYTES;
            const int kx = (kb0 + kb) * TC_BK;
            tma_load_2d_lead(dst, &map_w, kx, n0, full, lead);
            if (DUAL) tma_load_2d_lead(dst + W1_BYTES, &map_w, kx, N + n0, full, lead);
            tma_load_2d_lead(dst + W_BYTES, &map_x, kx, t0, full, lead);
            issued = kb + 1;
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = make_idesc(BN);
        bool ok = true;
        bool landed = false;                                     // the next stage's barrier is looked at while this stage's products are issued
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int s = kb % STAGES;
            const uint32_t round = kb / STAGES;
            if (!landed) {
                ok = mbar_wait(smem_u32(&sh->full[s]), round & 1, abort_flag, 2);   // TMA's bytes, seen through the barrier
                if (!ok) break;
            }
            if (kb == 0 && lead) TL(2);
            const uint32_t a = smem_base + s * STAGE_BYTES;
            const uint64_t da = make_smem_desc(a), db = make_smem_desc(a + W_BYTES);
            const uint64_t da2 = make_smem_desc(a + W1_BYTES);
            tc_mma_bf16_lead(tmem, da, db, idesc, kb != 0, lead);
            if (DUAL) tc_mma_bf16_lead(tmem + BN, da2, db, idesc, kb != 0, lead);
            landed = kb + 1 < nkb && mbar_test(smem_u32(&sh->full[(kb + 1) % STAGES]), (uint32_t)((kb + 1) / STAGES) & 1);
#pragma unroll
            for (int k = 1; k < TC_BK / 16; ++k) {               // 32 bytes further along K inside the swizzled row
                tc_mma_bf16_lead(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, 1, lead);
                if (DUAL) tc_mma_bf16_lead(tmem + BN, da2 + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, 1, lead);
            }
            tc_commit_lead(smem_u32(&sh->empty[s]), lead);       // frees the stage when these MMAs are done
        }
        if (ok) tc_commit_lead(smem_u32(&sh->acc_full), lead);
        if (lead) TL(3);
    } else {
        // epilogue: warp w may read tensor-memory lanes 32*(w%4) .. +31
        const int q = warp & 3;
        const int feat = n0 + q * 32 + lane;
        if (!DUAL && ex.h_q_out && csplit > 1) {
            // positions, slots, norm weights and frequencies come from before the step: nothing here waits
            const int et = threadIdx.x - 64, f4 = (et & 31) * 4, cb = split + (et >> 5) * csplit, hh = blockIdx.y;
            if (cb < BN && t0 + cb < T) {
                hp_slot = ex.h_kv_slot ? ex.h_kv_slot[t0 + cb] : -1;
                if (hh < ex.h_QH + ex.h_KH) head_angles_weights(ex, hh < ex.h_QH, t0 + cb, f4, hp_c, hp_s, hp_w);
            }
        }
        pdl_wait();                                            // C may still be in use by the kernels before
        if (!DUAL && csplit > 1 && out_mode == 2 && (ldc & 3) == 0 && ((uintptr_t)C & 15) == 0) {
            const int et = threadIdx.x - 64, f4 = (et & 31) * 4, cb0 = split + (et >> 5) * csplit, cb1 = cb0 + 4 * csplit;
            if (n0 + f4 + 3 < N) {
                if (cb0 < BN && t0 + cb0 < T) pre_a = *reinterpret_cast<const float4*>((const float*)C + (size_t)(t0 + cb0) * ldc + n0 + f4);
                if (cb1 < BN && t0 + cb1 < T) pre_b = *reinterpret_cast<const float4*>((const float*)C + (size_t)(t0 + cb1) * ldc + n0 + f4);
            }
        }
        for (int idx = threadIdx.x - 64; idx < BN; idx += 128) {
            float f = 1.0f;
            if (ex.row_sumsq && t0 + idx < T) {
                float ssq = 0.0f;
                for (int p = 0; p < ex.sumsq_parts; ++p) ssq += ex.row_sumsq[(size_t)(t0 + idx) * ex.sumsq_parts + p];
                f = 1.0f / sqrtf(ssq * ex.inv_width + ex.eps);
            }
            sh->row_scale[idx] = f;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");         // the four epilogue warps
        if (mbar_wait(smem_u32(&sh->acc_full), 0, abort_flag, 3)) {
            tc_fence_after();
            if (threadIdx.x == 64) TL(4);
            // All of this CTA's weights have arrived.  While the product drains (the cluster's reduction, the
            // stores) and the kernels after it start up, memory would idle: the weights that the next product
            // streams are called into L2 now.
            if (threadIdx.x == 64)
                l2_prefetch_share(ex.next_w, ex.next_bytes, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                                  gridDim.x * gridDim.y * gridDim.z);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (t0 + c0 >= T) break;                               // warp-uniform
                uint32_t r[16], r2[16];
                tc_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
                if (DUAL) tc_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(BN + c0), r2);
                tc_ld_wait();
                if (csplit == 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float f = sh->row_scale[c0 + j];
                        r[j] = __float_as_uint(__uint_as_float(r[j]) * f);
                        if (DUAL) r2[j] = __float_as_uint(__uint_as_float(r2[j]) * f);
                    }
                }
                if (csplit > 1) {                              // park the accumulator(s) for the cluster's reduction
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        reinterpret_cast<float*>(smem)[(c0 + j) * TC_BM + q * 32 + lane] = __uint_as_float(r[j]);
                        if (DUAL) reinterpret_cast<float*>(smem)[(BN + c0 + j) * TC_BM + q * 32 + lane] = __uint_as_float(r2[j]);
                    }
                } else if (feat < N) {
                    const int nt = min(16, T - t0 - c0);        // tokens of this chunk that exist
                    if (DUAL) {
                        bf16* cp = (bf16*)C + (size_t)(t0 + c0) * ldc + feat;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float g = __uint_as_float(r[j]), u = __uint_as_float(r2[j]);
                            if (j < nt) cp[(size_t)j * ldc] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
                        }
                    } else if (out_mode == 2) {
                        // read-modify-write of the float residual: all loads first, so that their
                        // latencies overlap instead of queueing behind the stores
                        float* cp = (float*)C + (size_t)(t0 + c0) * ldc + feat;
                        float old[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) old[j] = j < nt ? cp[(size_t)j * ldc] : 0.0f;
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (j < nt) cp[(size_t)j * ldc] = old[j] + __uint_as_float(r[j]);
                    } else if (out_mode == 0) {
                        bf16* cp = (bf16*)C + (size_t)(t0 + c0) * ldc + feat;
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (j < nt) cp[(size_t)j * ldc] = __float2bfloat16_rn(__uint_as_float(r[j]));
                    } else if (out_mode == 1) {
                        float* cp = (float*)C + (size_t)(t0 + c0) * ldc + feat;
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (j < nt) cp[(size_t)j * ldc] = __uint_as_float(r[j]);
                    } else {
                        float* cp = ws + ((size_t)split * T + t0 + c0) * N + feat;
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (j < nt) cp[(size_t)j * N] = __uint_as_float(r[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) TL(5);
    if (*abort_flag && threadIdx.x == 0) {
        // loads that were issued but never consumed still write this CTA's shared memory: wait for them
        for (int kb = max(0, issued - STAGES); kb < issued; ++kb) {
            const uint32_t bar = smem_u32(&sh->full[kb % STAGES]);
            const uint32_t parity = (kb / STAGES) & 1;
            mbar_drain(bar, parity);
        }
    }
    __syncthreads();
    if (csplit > 1) {
        // every CTA of the cluster reaches both barriers, whatever happened before
        cluster_sync_all();                                    // all accumulators are parked
        // The second barrier (nobody leaves while its memory is being read) is split: a thread arrives as soon as its last
        // loads from the peers are in its registers, stores its results, and waits only then.
        bool arrived = false;
        if (warp >= 2 && !*abort_flag) {
            // reduce-scatter: CTA `split` sums and stores the tokens c = split, split + csplit, ...  A thread
            // takes four neighbouring features (one 16-byte load per rank over distributed shared memory),
            // 32 threads a token, the four epilogue warps four tokens at once; every rank's partial sums are
            // fetched before the first is added, and they are added in rank order.
            const int et = threadIdx.x - 64;                       // 0..127
            const int f4 = (et & 31) * 4, tsub = et >> 5;
            const int feat = n0 + f4;
            if (!DUAL && feat + 3 < N && (ldc & 3) == 0 && ((uintptr_t)C & 15) == 0 && out_mode != 0) {
                // float results, four whole features: two tokens a trip (their partial sums from every rank and, for
                // an accumulating product, the residual's old values are all on their way before the first is used)
                float* Cf = (float*)C;
                for (int cb0 = split + tsub * csplit; cb0 < BN && t0 + cb0 < T; cb0 += 8 * csplit) {
                    const int cb1 = cb0 + 4 * csplit;
                    const bool two = cb1 < BN && t0 + cb1 < T;
                    float4 pa[8], pb[8];
                    const uint32_t m0 = smem_base + (uint32_t)(cb0 * TC_BM + f4) * 4, m1 = smem_base + (uint32_t)(cb1 * TC_BM + f4) * 4;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        pa[r] = r < csplit ? ld_cluster_f32x4(m0, (uint32_t)r) : make_float4(0.f, 0.f, 0.f, 0.f);
                        pb[r] = (two && r < csplit) ? ld_cluster_f32x4(m1, (uint32_t)r) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    float4* d0 = reinterpret_cast<float4*>(Cf + (size_t)(t0 + cb0) * ldc + feat);
                    float4* d1 = reinterpret_cast<float4*>(Cf + (size_t)(t0 + cb1) * ldc + feat);
                    float4 oa = make_float4(0.f, 0.f, 0.f, 0.f), ob = oa;
                    if (out_mode == 2) {
                        if (cb0 == split + tsub * csplit) { oa = pre_a; ob = pre_b; }      // fetched while the weights streamed
                        else { oa = *d0; if (two) ob = *d1; }
                    }
                    float4 va = pa[0], vb = pb[0];
#pragma unroll
                    for (int r = 1; r < 8; ++r) {
                        va.x += pa[r].x; va.y += pa[r].y; va.z += pa[r].z; va.w += pa[r].w;
                        vb.x += pb[r].x; vb.y += pb[r].y; vb.z += pb[r].z; vb.w += pb[r].w;
                    }
                    if (RB_SPLIT_BARRIER && !(cb0 + 8 * csplit < BN && t0 + cb0 + 8 * csplit < T)) {           // this thread's last trip
                        cluster_arrive_after(va.x + va.y + va.z + va.w + vb.x + vb.y + vb.z + vb.w);
                        arrived = true;
                    }
                    const float fa = sh->row_scale[cb0], fb = two ? sh->row_scale[cb1] : 0.0f;
                    const float4 na = make_float4(oa.x + va.x * fa, oa.y + va.y * fa, oa.z + va.z * fa, oa.w + va.w * fa);
                    const float4 nb = make_float4(ob.x + vb.x * fb, ob.y + vb.y * fb, ob.z + vb.z * fb, ob.w + vb.w * fb);
                    *d0 = na;
                    if (two) *d1 = nb;
                    if (ex.prep_rows) {
                        // the warp holds the tile's 128 features of one token (two tokens): the next norm's rows and
                        // this tile's part of the sum of squares
                        float4 w;
                        if (ex.prep_w_f32) w = *reinterpret_cast<const float4*>((const float*)ex.prep_w + feat);
                        else {
                            const uint2 wb = *reinterpret_cast<const uint2*>((const bf16*)ex.prep_w + feat);
                            const float2 w01 = __bfloat1622float2(*(const __nv_bfloat162*)&wb.x), w23 = __bfloat1622float2(*(const __nv_bfloat162*)&wb.y);
                            w = make_float4(w01.x, w01.y, w23.x, w23.y);
                        }
                        float sa = na.x * na.x + na.y * na.y + na.z * na.z + na.w * na.w;
                        float sb = nb.x * nb.x + nb.y * nb.y + nb.z * nb.z + nb.w * nb.w;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            sa += __shfl_xor_sync(0xffffffffu, sa, o);
                            sb += __shfl_xor_sync(0xffffffffu, sb, o);
                        }
                        const int parts = N / TC_BM;
                        const __nv_bfloat162 a01 = __floats2bfloat162_rn(na.x * w.x, na.y * w.y), a23 = __floats2bfloat162_rn(na.z * w.z, na.w * w.w);
                        *reinterpret_cast<uint2*>(ex.prep_rows + (size_t)(t0 + cb0) * N + feat) = make_uint2(*(const uint32_t*)&a01, *(const uint32_t*)&a23);
                        if (lane == 0) ex.prep_sumsq[(size_t)(t0 + cb0) * parts + blockIdx.y] = sa;
                        if (two) {
                            const __nv_bfloat162 b01 = __floats2bfloat162_rn(nb.x * w.x, nb.y * w.y), b23 = __floats2bfloat162_rn(nb.z * w.z, nb.w * w.w);
                            *reinterpret_cast<uint2*>(ex.prep_rows + (size_t)(t0 + cb1) * N + feat) = make_uint2(*(const uint32_t*)&b01, *(const uint32_t*)&b23);
                            if (lane == 0) ex.prep_sumsq[(size_t)(t0 + cb1) * parts + blockIdx.y] = sb;
                        }
                    }
                }
            } else
            for (int cb = split + tsub * csplit; cb < BN && t0 + cb < T; cb += 4 * csplit) {
                float4 part[8], part2[8];
                const uint32_t mine = smem_base + (uint32_t)(cb * TC_BM + f4) * 4;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    part[r] = r < csplit ? ld_cluster_f32x4(mine, (uint32_t)r) : make_float4(0.f, 0.f, 0.f, 0.f);
                    if (DUAL) part2[r] = r < csplit ? ld_cluster_f32x4(mine + (uint32_t)BN * TC_BM * 4, (uint32_t)r) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                float v[4] = {part[0].x, part[0].y, part[0].z, part[0].w};
#pragma unroll
                for (int r = 1; r < 8; ++r) { v[0] += part[r].x; v[1] += part[r].y; v[2] += part[r].z; v[3] += part[r].w; }
                float u[4] = {0.f, 0.f, 0.f, 0.f};
                if (DUAL) {
                    u[0] = part2[0].x; u[1] = part2[0].y; u[2] = part2[0].z; u[3] = part2[0].w;
#pragma unroll
                    for (int r = 1; r < 8; ++r) { u[0] += part2[r].x; u[1] += part2[r].y; u[2] += part2[r].z; u[3] += part2[r].w; }
                }
                if (RB_SPLIT_BARRIER && !(cb + 4 * csplit < BN && t0 + cb + 4 * csplit < T)) {                 // this thread's last trip
                    cluster_arrive_after(v[0] + v[1] + v[2] + v[3] + u[0] + u[1] + u[2] + u[3]);
                    arrived = true;
                }
                const float f = sh->row_scale[cb];
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] *= f;
                if (!DUAL && ex.h_q_out) {
                    // the warp holds one head of token t: lanes 0-15 the low half (four features each), lane ^ 16 the partner
                    const int t = t0 + cb, hh = blockIdx.y;
                    const int kind = hh < ex.h_QH ? 0 : hh < ex.h_QH + ex.h_KH ? 1 : 2;
                    const bool first = cb == split + tsub * csplit;          // what was fetched before the weights arrived
                    const int slot = first ? hp_slot : ex.h_kv_slot ? ex.h_kv_slot[t] : -1;
                    if (!first && kind < 2) head_angles_weights(ex, kind == 0, t, f4, hp_c, hp_s, hp_w);
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
                    bf16* dst = nullptr;
                    if (kind == 0) dst = ex.h_q_out + ((size_t)t * ex.h_QH + hh) * 128;
                    else if (slot >= 0) {
                        const int page = slot / ex.h_page, off = slot % ex.h_page;
                        const int kh = kind == 1 ? hh - ex.h_QH : hh - ex.h_QH - ex.h_KH;
                        dst = ex.h_cache + ((((size_t)page * 2 + (kind - 1)) * ex.h_KH + kh) * ex.h_page + off) * 128;
                    }
                    float o[4] = {v[0], v[1], v[2], v[3]};
                    if (kind < 2) {
                        if (kind == 0 ? ex.h_q_w : ex.h_k_w) {
                            float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
                            for (int sft = 16; sft > 0; sft >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sft);
                            const float rstd = 1.0f / sqrtf(ss / 128.0f + ex.h_eps);
#pragma unroll
                            for (int i = 0; i < 4; ++i) v[i] = v[i] * rstd * hp_w[i];
                        }
                        const bool low = f4 < 64;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
                            o[i] = low ? v[i] * hp_c[i] - other * hp_s[i] : other * hp_s[i] + v[i] * hp_c[i];
                        }
                    }
                    if (dst) {
                        const __nv_bfloat162 p01 = __floats2bfloat162_rn(o[0], o[1]), p23 = __floats2bfloat162_rn(o[2], o[3]);
                        *reinterpret_cast<uint2*>(dst + f4) = make_uint2(*(const uint32_t*)&p01, *(const uint32_t*)&p23);
                    }
                    continue;
                }
                if (DUAL) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] = v[i] / (1.0f + expf(-v[i])) * (u[i] * f);
                }
                const size_t at = (size_t)(t0 + cb) * ldc + feat;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (feat + i >= N) break;
                    if (DUAL || out_mode == 0) ((bf16*)C)[at + i] = __float2bfloat16_rn(v[i]);
                    else if (out_mode == 1) ((float*)C)[at + i] = v[i];
                    else ((float*)C)[at + i] += v[i];
                }
            }
        }
        if (threadIdx.x == 64) TL(6);
        if (!arrived) cluster_arrive_after(0.0f);              // threads that read nothing (or gave up) arrive here
        cluster_wait_all();                                    // nobody leaves while its memory is being read
    }
    if (threadIdx.x == 0) TL(7);
    if (warp == 1) {
        __syncwarp();                                   // .sync.aligned: the MMA lane rejoins its warp first
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------ persistent
// The same product for many tokens (prompt portions): one CTA per SM walks the output tiles
// (tile = blockIdx.x, + gridDim.x, ...; token tiles fastest, so that CTAs running side by side share a
// weight tile in L2).  Two accumulators in tensor memory alternate: while the four epilogue warps read
// one back and store it, the MMA thread already fills the other with the next tile, and the TMA thread
// keeps the shared-memory ring full across tile borders - neither the epilogue nor the pipeline's fill
// and drain leave the tensor cores idle as they do with one CTA per tile.
struct TcPersistShared {
    unsigned long long full[8];
    unsigned long long empty[8];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    __align__(16) float head_w[2][128];      // MODE 3: the q and k norm weights
};

// MODE 3 of the persistent kernel: the product is the attention's q/k/v projection with heads of 128, and a tile's 256
// features are two whole heads of its 128 tokens.  The epilogue then does what a kernel of its own did on the rounded
// projection (elementwise.cu, qknorm_rope_append): per head the RMS norm over its 128 features with the q or k weights,
// the half-split rotation by the step's table of cosines and sines, and the store - query heads to q_out [T, QH, 128],
// key and value heads into the token's slot of the layer's cache pages.  A thread holds its token's whole head in its
// accumulator lane, so norm and rotation need no exchange; and the projection never goes to memory.
struct TcHeads {
    bf16* q_out;
    bf16* cache;                 // the layer's [pages, 2, KH, page_size, 128]
    const int* kv_slot;          // [T] page * page_size + offset of each token, -1: store no key or value
    const float2* cs_table;      // [T, 64] (cos, sin) of each token's angles
    const void* q_w;             // [128] norm weights (w_f32: float, else bfloat16)
    const void* k_w;
    int w_f32, QH, KH, page_size;
    float eps;
};

// Rows that lack their factor, for the token-lane forms of the persistent kernel (MODE 1 .. 3; row_sumsq null: rows are
// complete): token t stands for X[t,:] / sqrt(sum_p row_sumsq[t, p] * inv_width + eps), and its lane multiplies its
// results by that - the norm's division behind the product, as in TcExtra.
struct TcRows {
    const float* row_sumsq;
    int sumsq_parts;
    float inv_width, eps;
};

template <int BN, int STAGES, int MODE, int ROWS = 2 * TC_BM>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                          void* __restrict__ C, int T, int N, int K, long long ldc, int out_mode, int t_tiles, int n_tiles,
                          TcHeads hd, TcRows rs) {
    // MODE 0: a tile is 128 features (the M operand) x BN tokens.  MODE 1 (the gated pair) and MODE 2: a tile is 128
    // tokens (the M operand) x ROWS weight rows (the N operand; a multiple of 32 up to 256): ROWS / 2 gate rows and the
    // ROWS / 2 up rows of the same features, or ROWS features.  A lane of the accumulator is then a token, and the
    // epilogue writes 16 features of it at a time.  Fewer rows leave room for a stage more.
    constexpr bool DUAL = MODE == 1, FLIP = MODE != 0, HEADS = MODE == 3;
    static_assert(!HEADS || ROWS == 2 * TC_BM, "two heads of 128 a tile");
    static_assert(ROWS % 32 == 0 && ROWS >= 32 && ROWS <= 2 * TC_BM, "rows of the N operand");
    constexpr int FEATS = (MODE == 2 || MODE == 3) ? ROWS : MODE == 1 ? ROWS / 2 : TC_BM;   // features per tile
    RB_TL(DUAL ? 9 : 8);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr uint32_t W1_BYTES = (FLIP ? ROWS / 2 : TC_BM) * TC_BK * 2;     // the gate rows (DUAL), or half of the rows
    constexpr uint32_t W_BYTES = (FLIP ? 2 : 1) * W1_BYTES;
    static_assert(W1_BYTES % 1024 == 0, "the second box starts on a swizzle atom");
    constexpr uint32_t X_BYTES = BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES;
    static_assert(!FLIP || BN == 128, "with the tokens as the M operand a tile has 128 of them");
    constexpr uint32_t ACC_COLS = FLIP ? 2 * TC_BM : BN;          // columns of one accumulator stage (ROWS of them used)
    static_assert(2 * ACC_COLS <= 512, "two accumulator stages must fit tensor memory");
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS <= 32 ? 32 : 2 * ACC_COLS <= 64 ? 64 : 2 * ACC_COLS <= 128 ? 128 : 2 * ACC_COLS <= 256 ? 256 : 512;
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    TcPersistShared* sh = (TcPersistShared*)(smem + (size_t)STAGES * STAGE_BYTES);
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = t_tiles * n_tiles;
    const int nkb = (K + TC_BK - 1) / TC_BK;
    volatile int* abort_flag = &sh->abort_flag;
    if (*(volatile int*)&g_rb_kernel_error) return;               // an earlier launch gave up: fail fast, the host will see the word

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&sh->acc_full[a]), 1); mbar_init(smem_u32(&sh->acc_empty[a]), 4); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    uint32_t issued = 0;                                // producer: k-blocks (over all its tiles) whose loads were issued

    // The two issuing warps stay converged: every lane walks the loop and waits at the barriers, lane 0 alone issues
    // (predicated instructions).  Stage index and parity are counters, barrier addresses and operand descriptors are
    // sums with constants.
    const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
    const uint32_t lead = lane == 0 ? 1u : 0u;
    if (warp == 0) {
        pdl_trigger();
        pdl_wait();
        bool ok = true;
        uint32_t s = 0, ph = 1;                           // a stage's first use finds it free
        [[maybe_unused]] int plocal = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++plocal) {
            const int t0 = (tile % t_tiles) * BN, n0 = (tile / t_tiles) * FEATS;
            [[maybe_unused]] long long waited = 0;
            for (int kb = 0; kb < nkb; ++kb) {
#ifdef RB_TIMELINE
                const long long c0 = clock64();
#endif
                ok = mbar_wait(empty0 + 8 * s, ph, abort_flag, 11);
#ifdef RB_TIMELINE
                waited += clock64() - c0;
                if (kb == 0 && lead) TT(plocal, 6, tl_now());
#endif
                if (!ok) break;
                const uint32_t full = full0 + 8 * s;
                mbar_expect_tx_lead(full, STAGE_BYTES, lead);
                const uint32_t dst = smem_base + s * STAGE_BYTES;
                tma_load_2d_lead(dst, &map_w, kb * TC_BK, n0, full, lead);      // MODE 2: the map's box has ROWS rows, MODE 1: ROWS / 2
                if (DUAL) tma_load_2d_lead(dst + W1_BYTES, &map_w, kb * TC_BK, N + n0, full, lead);
                tma_load_2d_lead(dst + W_BYTES, &map_x, kb * TC_BK, t0, full, lead);
                ++issued;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            if (lead) TT(plocal, 7, (unsigned long long)waited);
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = make_idesc(FLIP ? ROWS : BN);
        const uint64_t dw0 = make_smem_desc(smem_base), dx0 = make_smem_desc(smem_base + W_BYTES);
        bool ok = true;
        uint32_t s = 0, ph = 0;
        int local = 0;
        // Whether the next stage has landed is asked while this stage's products are being issued, so that the
        // answer's latency is not part of the serial loop; only an answer of "not yet" leads to a wait.
        bool landed = false;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
            const int a = local & 1;
            ok = mbar_wait(smem_u32(&sh->acc_empty[a]), ((uint32_t)(local >> 1) & 1) ^ 1, abort_flag, 12);   // drained by the epilogue
            if (!ok) break;
#ifdef RB_TIMELINE
            if (lead) TT(local, 0, tl_now());
            long long waited = 0, t_mma = 0, t_commit = 0;
            const long long cb = clock64();
#endif
            tc_fence_after();
            const uint32_t acc = tmem + (uint32_t)a * ACC_COLS;
            for (int kb = 0; kb < nkb; ++kb) {
                if (!landed) {
#ifdef RB_TIMELINE
                    const long long c0 = clock64();
#endif
                    ok = mbar_wait(full0 + 8 * s, ph, abort_flag, 13);   // TMA's bytes, seen through the barrier: no tcgen05 fence is due
#ifdef RB_TIMELINE
                    waited += clock64() - c0;
#endif
                    if (!ok) break;
                }
                const uint64_t off = (uint64_t)(s * (STAGE_BYTES >> 4));     // the address field counts 16-byte units
                const uint64_t da = dw0 + off, db = dx0 + off;
                const uint32_t s_next = s + 1 == STAGES ? 0 : s + 1, ph_next = s + 1 == STAGES ? ph ^ 1 : ph;
#ifdef RB_TIMELINE
                const long long c1 = clock64();
#endif
                if (FLIP) tc_mma_bf16_lead(acc, db, da, idesc, kb != 0, lead);
                else tc_mma_bf16_lead(acc, da, db, idesc, kb != 0, lead);
                landed = mbar_test(full0 + 8 * s_next, ph_next);
#pragma unroll
                for (int k = 1; k < TC_BK / 16; ++k) {
                    if (FLIP) tc_mma_bf16_lead(acc, db + (uint64_t)(k * 2), da + (uint64_t)(k * 2), idesc, 1, lead);
                    else tc_mma_bf16_lead(acc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, 1, lead);
                }
#ifdef RB_TIMELINE
                const long long c2 = clock64();
#endif
                tc_commit_lead(empty0 + 8 * s, lead);
#ifdef RB_TIMELINE
                t_mma += c2 - c1;
                t_commit += clock64() - c2;
#endif
                s = s_next; ph = ph_next;
            }
            if (ok) tc_commit_lead(smem_u32(&sh->acc_full[a]), lead);
#ifdef RB_TIMELINE
            if (lead) { TT(local, 1, (unsigned long long)waited); TT(local, 2, tl_now()); TT(local, 8, (unsigned long long)(clock64() - cb)); TT(local, 9, (unsigned long long)t_mma); TT(local, 3, (unsigned long long)t_commit); }
#endif
        }
    } else {
        const int q = warp & 3;
        pdl_wait();
        int local = 0;
        const bool vec_ok = (ldc % 8 == 0) && (((uintptr_t)C & 15) == 0);
        if (HEADS) {                                               // the norm weights, once, for the four epilogue warps
            const int i = threadIdx.x - 64;                        // 0..127
            sh->head_w[0][i] = hd.w_f32 ? ((const float*)hd.q_w)[i] : __bfloat162float(((const bf16*)hd.q_w)[i]);
            sh->head_w[1][i] = hd.w_f32 ? ((const float*)hd.k_w)[i] : __bfloat162float(((const bf16*)hd.k_w)[i]);
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
            const int a = local & 1;
            const int t0 = (tile % t_tiles) * BN, n0 = (tile / t_tiles) * FEATS;
            if (!mbar_wait(smem_u32(&sh->acc_full[a]), (uint32_t)(local >> 1) & 1, abort_flag, 14)) break;
#ifdef RB_TIMELINE
            if (warp == 2 && lane == 0) TT(local, 4, tl_now());
#endif
            tc_fence_after();
            const uint32_t acc = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)a * ACC_COLS;
            float rf = 1.0f;                                       // the factor that this lane's token still lacks
            if (FLIP && rs.row_sumsq && t0 + q * 32 + lane < T) {
                const float* parts = rs.row_sumsq + (size_t)(t0 + q * 32 + lane) * rs.sumsq_parts;
                float ssq = 0.0f;
                for (int p = 0; p < rs.sumsq_parts; ++p) ssq += parts[p];
                rf = 1.0f / sqrtf(ssq * rs.inv_width + rs.eps);
            }
            if (DUAL) {
                // a lane is a token; columns 0..FEATS-1 hold its gate features, the next FEATS the up features of the same tile
                const int tok = t0 + q * 32 + lane;
                bf16* row = (bf16*)C + (size_t)tok * ldc + n0;
#pragma unroll 1
                for (int c0 = 0; c0 < FEATS; c0 += 16) {
                    if (n0 + c0 >= N) break;
                    uint32_t r[16], r2[16];
                    tc_ld16(acc + (uint32_t)c0, r);
                    tc_ld16(acc + (uint32_t)(FEATS + c0), r2);
                    tc_ld_wait();
                    if (tok < T) {
                        uint32_t o[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float g0 = __uint_as_float(r[2 * j]) * rf, u0 = __uint_as_float(r2[2 * j]) * rf;
                            const float g1 = __uint_as_float(r[2 * j + 1]) * rf, u1 = __uint_as_float(r2[2 * j + 1]) * rf;
                            const __nv_bfloat162 v = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
                            o[j] = *(const uint32_t*)&v;
                        }
                        if (vec_ok && n0 + c0 + 16 <= N) {
                            *(uint4*)(row + c0) = make_uint4(o[0], o[1], o[2], o[3]);
                            *(uint4*)(row + c0 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                        } else {
                            const bf16* ov = (const bf16*)o;
#pragma unroll
                            for (int j = 0; j < 16; ++j) if (n0 + c0 + j < N) row[c0 + j] = ov[j];
                        }
                    }
                }
            } else if (HEADS) {
                const int tok = t0 + q * 32 + lane;
                const bool live = tok < T;
                const int slot = live && hd.kv_slot ? hd.kv_slot[tok] : -1;
                const float2* cs = hd.cs_table + (size_t)(live ? tok : 0) * 64;
#pragma unroll 1
                for (int hh = 0; hh < 2; ++hh) {
                    const int head = n0 / 128 + hh;                       // of QH + 2 KH heads: queries, keys, values
                    if (head >= hd.QH + 2 * hd.KH) break;
                    const uint32_t hcol = acc + (uint32_t)(hh * 128);
                    const int kind = head < hd.QH ? 0 : head < hd.QH + hd.KH ? 1 : 2;
                    bf16* dst = nullptr;
                    if (kind == 0) {
                        if (live) dst = hd.q_out + ((size_t)tok * hd.QH + head) * 128;
                    } else if (slot >= 0) {
                        const int kh = head - hd.QH - (kind == 2 ? hd.KH : 0);
                        const size_t page = (size_t)(slot / hd.page_size), off = (size_t)(slot % hd.page_size);
                        dst = hd.cache + (((page * 2 + (kind == 2 ? 1 : 0)) * hd.KH + kh) * hd.page_size + off) * 128;
                    }
                    if (kind == 2) {
#pragma unroll 1
                        for (int c0 = 0; c0 < 128; c0 += 16) {
                            uint32_t r[16];
                            tc_ld16(hcol + (uint32_t)c0, r);
                            tc_ld_wait();
                            if (!dst) continue;
                            uint32_t o[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]) * rf, __uint_as_float(r[2 * j + 1]) * rf);
                                o[j] = *(const uint32_t*)&v;
                            }
                            *(uint4*)(dst + c0) = make_uint4(o[0], o[1], o[2], o[3]);
                            *(uint4*)(dst + c0 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                        }
                        continue;
                    }
                    // the head as the separate kernel sees it: rounded to bfloat16 first
                    float ss = 0.0f;
#pragma unroll 1
                    for (int c0 = 0; c0 < 128; c0 += 16) {
                        uint32_t r[16];
                        tc_ld16(hcol + (uint32_t)c0, r);
                        tc_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float v = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[j]) * rf));
                            ss = fmaf(v, v, ss);
                        }
                    }
                    const float rstd = 1.0f / sqrtf(ss / 128.0f + hd.eps);
                    const float4* wv = reinterpret_cast<const float4*>(sh->head_w[kind]);
                    const float4* cs4 = reinterpret_cast<const float4*>(cs);       // two (cos, sin) pairs each
#pragma unroll 1
                    for (int c0 = 0; c0 < 64; c0 += 16) {
                        uint32_t lo[16], hi[16];
                        tc_ld16(hcol + (uint32_t)c0, lo);
                        tc_ld16(hcol + (uint32_t)(64 + c0), hi);
                        float4 ang[8];                                      // this token's 16 angles of the chunk
#pragma unroll
                        for (int j = 0; j < 8; ++j) ang[j] = cs4[c0 / 2 + j];
                        tc_ld_wait();
                        if (!dst) continue;
                        uint32_t ol[8], oh[8];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {                       // four features of each half a trip
                            const float4 wl = wv[c0 / 4 + j], wh = wv[16 + c0 / 4 + j];
                            const float wls[4] = {wl.x, wl.y, wl.z, wl.w}, whs[4] = {wh.x, wh.y, wh.z, wh.w};
                            const float cc[4] = {ang[2 * j].x, ang[2 * j].z, ang[2 * j + 1].x, ang[2 * j + 1].z};
                            const float sn[4] = {ang[2 * j].y, ang[2 * j].w, ang[2 * j + 1].y, ang[2 * j + 1].w};
                            float xo[4], yo[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const float x = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lo[4 * j + u]) * rf)) * rstd * wls[u];
                                const float y = __bfloat162float(__float2bfloat16_rn(__uint_as_float(hi[4 * j + u]) * rf)) * rstd * whs[u];
                                xo[u] = x * cc[u] - y * sn[u];             // low half: x c - y s
                                yo[u] = x * sn[u] + y * cc[u];             // high half: y c + x s
                            }
                            const __nv_bfloat162 p0 = __floats2bfloat162_rn(xo[0], xo[1]), p1 = __floats2bfloat162_rn(xo[2], xo[3]);
                            const __nv_bfloat162 r0 = __floats2bfloat162_rn(yo[0], yo[1]), r1 = __floats2bfloat162_rn(yo[2], yo[3]);
                            ol[2 * j] = *(const uint32_t*)&p0; ol[2 * j + 1] = *(const uint32_t*)&p1;
                            oh[2 * j] = *(const uint32_t*)&r0; oh[2 * j + 1] = *(const uint32_t*)&r1;
                        }
                        *(uint4*)(dst + c0) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
                        *(uint4*)(dst + c0 + 8) = make_uint4(ol[4], ol[5], ol[6], ol[7]);
                        *(uint4*)(dst + 64 + c0) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
                        *(uint4*)(dst + 64 + c0 + 8) = make_uint4(oh[4], oh[5], oh[6], oh[7]);
                    }
                }
            } else if (FLIP) {
                // a lane is a token; its 256 columns are 256 features
                const int tok = t0 + q * 32 + lane;
                const bool vec4 = (ldc % 4 == 0) && (((uintptr_t)C & 15) == 0);
#pragma unroll 1
                for (int c0 = 0; c0 < FEATS; c0 += 16) {
                    if (n0 + c0 >= N) break;
                    uint32_t r[16];
                    tc_ld16(acc + (uint32_t)c0, r);
                    tc_ld_wait();
                    if (tok >= T) continue;
                    if (rs.row_sumsq) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * rf);
                    }
                    const bool whole = n0 + c0 + 16 <= N;
                    if (out_mode == 0) {
                        bf16* row = (bf16*)C + (size_t)tok * ldc + n0 + c0;
                        uint32_t o[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                            o[j] = *(const uint32_t*)&v;
                        }
                        if (vec_ok && whole) {
                            *(uint4*)row = make_uint4(o[0], o[1], o[2], o[3]);
                            *(uint4*)(row + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                        } else {
                            const bf16* ov = (const bf16*)o;
#pragma unroll
                            for (int j = 0; j < 16; ++j) if (n0 + c0 + j < N) row[j] = ov[j];
                        }
                    } else {
                        float* row = (float*)C + (size_t)tok * ldc + n0 + c0;
                        if (vec4 && whole) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                             __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                                if (out_mode == 2) red_add_f32x4(row + 4 * j, v);
                                else *(float4*)(row + 4 * j) = v;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (n0 + c0 + j < N) row[j] = (out_mode == 2 ? row[j] : 0.0f) + __uint_as_float(r[j]);
                        }
                    }
                }
            } else {
            const int feat = n0 + q * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (t0 + c0 >= T) break;
                uint32_t r[16];
                tc_ld16(acc + (uint32_t)c0, r);
                tc_ld_wait();
                if (feat < N) {
                    const int nt = min(16, T - t0 - c0);
                    if (out_mode == 2) {
                        // one addition per element, done where the element lives (a reduction without a return value):
                        // the same sum as load, add, store, without the load's way back
                        float* cp = (float*)C + (size_t)(t0 + c0) * ldc + feat;
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (j < nt) red_add_f32(cp + (size_t)j * ldc, __uint_as_float(r[j]));
                    } else if (out_mode == 0) {
                        bf16* cp = (bf16*)C + (size_t)(t0 + c0) * ldc + feat;
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (j < nt) cp[(size_t)j * ldc] = __float2bfloat16_rn(__uint_as_float(r[j]));
                    } else {
                        float* cp = (float*)C + (size_t)(t0 + c0) * ldc + feat;
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (j < nt) cp[(size_t)j * ldc] = __uint_as_float(r[j]);
                    }
                }
            }
            }
            // this warp has read its quarter of the accumulator: the MMA thread may refill it once all four have
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[a]));
#ifdef RB_TIMELINE
            if (warp == 2 && lane == 0) TT(local, 5, tl_now());
#endif
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        for (uint32_t it = issued > STAGES ? issued - STAGES : 0; it < issued; ++it) {
            const uint32_t bar = smem_u32(&sh->full[it % STAGES]);
            const uint32_t parity = (it / STAGES) & 1;
            mbar_drain(bar, parity);
        }
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();                                   // .sync.aligned: the MMA lane rejoins its warp first
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

template <int BN, int STAGES, int MODE, int ROWS = 2 * TC_BM>
static int launch_tc_persistent(const CUtensorMap& mw, const CUtensorMap& mx, void* C, int T, int N, int K, long long ldc,
                                int mode, cudaStream_t s, const TcHeads& hd = TcHeads{}, const TcRows& rs = TcRows{}) {
    constexpr size_t smem = (size_t)STAGES * ((MODE ? ROWS : TC_BM) * TC_BK * 2 + BN * TC_BK * 2) + sizeof(TcPersistShared) + 1024;
    static_assert(smem <= 232448, "stages beyond the shared memory of an SM");
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, STAGES, MODE, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    const int t_tiles = rb_ceil_div(T, BN), n_tiles = rb_ceil_div(N, (MODE == 2 || MODE == 3) ? ROWS : MODE == 1 ? ROWS / 2 : TC_BM);
    const int total = t_tiles * n_tiles;
    const int grid = total < sms ? total : sms;
    return rb_launch(gemm_tc_persistent_kernel<BN, STAGES, MODE, ROWS>, dim3(grid), dim3(TC_THREADS), smem, s, mw, mx, C, T, N, K, ldc,
                     mode, t_tiles, n_tiles, hd, rs);
}

// The gated pair over 65 .. 128 tokens (a decode step of that many requests): one tile per CTA, 128 tokens (the M
// operand; rows beyond T are zero-filled by TMA) x 64 gate + 64 up weight rows (the N operand), the whole depth K, three
// stages of 32 KB - two CTAs fit an SM, and F / 64 CTAs stream the weights (192 at the 8B shape, where 128-row tiles
// gave 96 CTAs on 148 SMs with eight products to issue per k-step: 4.4 TB/s).  A lane of the accumulator is a token;
// its row factor (the deferred RMS norm) multiplies gate and up before the activation.  The weights' first stages are
// requested before the kernels in front of this one have finished, the tokens after.
struct TcStreamShared {
    unsigned long long full[4];
    unsigned long long empty[4];
    unsigned long long acc_full;
    uint32_t tmem_base;
    int abort_flag;
};
#define TCS_ROWS 64                      // gate rows (and up rows) per tile
template <int STAGES, int XROWS>
__global__ void __launch_bounds__(TC_THREADS, 2)
gemm_tc_gated_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                            bf16* __restrict__ act, int T, int F, int K, long long ldc, TcExtra ex) {
    RB_TL(7);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr uint32_t W1_BYTES = TCS_ROWS * TC_BK * 2;            // the gate rows of a stage; the up rows follow
    constexpr uint32_t W_BYTES = 2 * W1_BYTES;
    // XROWS tokens are fetched (64 when there are no more: the product still reads 128 rows, the 64 beyond lie in
    // the next stage's weights or in the slack behind the last stage - whatever they hold lands in accumulator lanes of
    // tokens that do not exist and is never read)
    constexpr uint32_t X_BYTES = XROWS * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * TCS_ROWS;
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    TcStreamShared* sh = (TcStreamShared*)(smem + (size_t)STAGES * STAGE_BYTES + (128 - XROWS) * TC_BK * 2);
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TCS_ROWS;
    const int nkb = (K + TC_BK - 1) / TC_BK;
    volatile int* abort_flag = &sh->abort_flag;
    if (*(volatile int*)&g_rb_kernel_error) return;               // an earlier launch gave up: fail fast, the host will see the word

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), 1); }
        mbar_init(smem_u32(&sh->acc_full), 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
    const uint32_t lead = lane == 0 ? 1u : 0u;                     // the issuing warps stay converged; lane 0's instructions take effect
    int issued = 0;

    if (warp == 0) {
        pdl_trigger();
        const int pre = min(nkb, STAGES);
        for (int kb = 0; kb < pre; ++kb) {                         // the weights never change: fetched at once
            const uint32_t full = full0 + 8 * kb;
            mbar_expect_tx_lead(full, STAGE_BYTES, lead);
            tma_load_2d_lead(smem_base + kb * STAGE_BYTES, &map_w, kb * TC_BK, n0, full, lead);
            tma_load_2d_lead(smem_base + kb * STAGE_BYTES + W1_BYTES, &map_w, kb * TC_BK, F + n0, full, lead);
        }
        pdl_wait();
        if (lead) RB_TL_MARK();
        for (int kb = 0; kb < pre; ++kb)
            tma_load_2d_lead(smem_base + kb * STAGE_BYTES + W_BYTES, &map_x, kb * TC_BK, 0, full0 + 8 * kb, lead);
        issued = pre;
        for (int kb = pre; kb < nkb; ++kb) {
            const int s = kb % STAGES;
            if (!mbar_wait(empty0 + 8 * s, ((uint32_t)(kb / STAGES) & 1) ^ 1, abort_flag, 31)) break;
            const uint32_t full = full0 + 8 * s, dst = smem_base + s * STAGE_BYTES;
            mbar_expect_tx_lead(full, STAGE_BYTES, lead);
            tma_load_2d_lead(dst, &map_w, kb * TC_BK, n0, full, lead);
            tma_load_2d_lead(dst + W1_BYTES, &map_w, kb * TC_BK, F + n0, full, lead);
            tma_load_2d_lead(dst + W_BYTES, &map_x, kb * TC_BK, 0, full, lead);
            issued = kb + 1;
        }
        // this CTA's weights are on their way: the weights that the next product streams are called into L2
        if (lead) l2_prefetch_share(ex.next_w, ex.next_bytes, blockIdx.x, gridDim.x);
    } else if (warp == 1) {
        constexpr uint32_t idesc = make_idesc(2 * TCS_ROWS);
        const uint64_t dw0 = make_smem_desc(smem_base), dx0 = make_smem_desc(smem_base + W_BYTES);
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % STAGES;
            ok = mbar_wait(full0 + 8 * s, (uint32_t)(kb / STAGES) & 1, abort_flag, 32);
            if (!ok) break;
            const uint64_t off = (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k)                   // the tokens are the M operand, the 128 weight rows the N operand
                tc_mma_bf16_lead(tmem, dx0 + off + (uint64_t)(k * 2), dw0 + off + (uint64_t)(k * 2), idesc, (kb | k) != 0, lead);
            tc_commit_lead(empty0 + 8 * s, lead);
        }
        if (ok) tc_commit_lead(smem_u32(&sh->acc_full), lead);
    } else {
        const int q = warp & 3;
        const int tok = q * 32 + lane;
        pdl_wait();
        float f = 1.0f;                                            // this token's row factor
        if (ex.row_sumsq && tok < T) {
            float ssq = 0.0f;
            for (int p = 0; p < ex.sumsq_parts; ++p) ssq += ex.row_sumsq[(size_t)tok * ex.sumsq_parts + p];
            f = 1.0f / sqrtf(ssq * ex.inv_width + ex.eps);
        }
        const bool vec_ok = (ldc % 8 == 0) && (((uintptr_t)act & 15) == 0);
        if (mbar_wait(smem_u32(&sh->acc_full), 0, abort_flag, 33)) {
            tc_fence_after();
            const uint32_t acc = tmem + ((uint32_t)(q * 32) << 16);
            bf16* row = act + (size_t)tok * ldc + n0;
#pragma unroll 1
            for (int c0 = 0; c0 < TCS_ROWS; c0 += 16) {
                if (n0 + c0 >= F) break;
                uint32_t r[16], r2[16];
                tc_ld16(acc + (uint32_t)c0, r);
                tc_ld16(acc + (uint32_t)(TCS_ROWS + c0), r2);
                tc_ld_wait();
                if (tok >= T) continue;
                uint32_t o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float g0 = __uint_as_float(r[2 * j]) * f, u0 = __uint_as_float(r2[2 * j]) * f;
                    const float g1 = __uint_as_float(r[2 * j + 1]) * f, u1 = __uint_as_float(r2[2 * j + 1]) * f;
                    const __nv_bfloat162 v = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
                    o[j] = *(const uint32_t*)&v;
                }
                if (vec_ok && n0 + c0 + 16 <= F) {
                    *(uint4*)(row + c0) = make_uint4(o[0], o[1], o[2], o[3]);
                    *(uint4*)(row + c0 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                } else {
                    const bf16* ov = (const bf16*)o;
#pragma unroll
                    for (int j = 0; j < 16; ++j) if (n0 + c0 + j < F) row[c0 + j] = ov[j];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        for (int kb = max(0, issued - STAGES); kb < issued; ++kb)
            mbar_drain(smem_u32(&sh->full[kb % STAGES]), (uint32_t)(kb / STAGES) & 1);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

template <int STAGES, int XROWS>
static int launch_tc_gated_stream(const void* X, const void* Wgu, void* act, int T, int F, int K, long long ldx, long long ldw,
                                  long long ldc, const TcExtra& ex, cudaStream_t s) {
    constexpr size_t smem = (size_t)STAGES * (2 * TCS_ROWS * TC_BK * 2 + XROWS * TC_BK * 2) + (128 - XROWS) * TC_BK * 2 +
                            sizeof(TcStreamShared) + 1024;
    static_assert(smem <= 113 * 1024, "two CTAs to an SM");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_gated_stream_kernel<STAGES, XROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        (void)cudaFuncSetAttribute(gemm_tc_gated_stream_kernel<STAGES, XROWS>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = true;
    }
    CUtensorMap mw, mx;
    if (rb_tensor_map_bf16(Wgu, 2LL * F, K, ldw, TCS_ROWS, &mw)) return -1;
    if (rb_tensor_map_bf16(X, T, K, ldx, XROWS, &mx)) return -1;
    return rb_launch(gemm_tc_gated_stream_kernel<STAGES, XROWS>, dim3(rb_ceil_div(F, TCS_ROWS)), dim3(TC_THREADS), smem, s, mw, mx,
                     (bf16*)act, T, F, K, ldc, ex);
}

// Sum of the split partials in split order, then store / accumulate.  mode as OUT_MODE 0..2.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ C, int T, int N, long long ldc,
                                     int splits, int mode) {
    pdl_trigger(); pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)T * N) return;
    const int t = (int)(i / N), n = (int)(i % N);
    float v = 0.0f;
    for (int s = 0; s < splits; ++s) v += ws[(size_t)s * T * N + i];
    if (mode == 0) ((bf16*)C)[(size_t)t * ldc + n] = __float2bfloat16_rn(v);
    else if (mode == 1) ((float*)C)[(size_t)t * ldc + n] = v;
    else ((float*)C)[(size_t)t * ldc + n] += v;
}

// ------------------------------------------------------------------ host side
// How many CTAs of this kernel can be resident at once when launched as clusters of `sp` (1: no cluster).
// The occupancy calls answer one CTA per SM for the tensor-core kernels themselves although two are resident
// (256 CTAs were seen to start within a microsecond), so a twin with the same threads, launch bounds and shared
// memory is asked instead; its cluster count knows how clusters of two CTAs per SM tile the GPCs.
template <int MINB>
__global__ void __launch_bounds__(TC_THREADS, MINB) tc_occupancy_twin(int* p) {
    extern __shared__ unsigned char twin_smem[];
    if (p) p[threadIdx.x] = twin_smem[threadIdx.x];
}
template <int BN, int STAGES, bool DUAL>
static int tc_capacity(int sp, size_t smem) {
    static int cache[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    if (cache[sp]) return cache[sp];
    constexpr int MINB = BN <= 64 ? 2 : 1;                          // the kernel's __launch_bounds__
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    (void)cudaFuncSetAttribute(tc_occupancy_twin<MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int n = 0;
    if (sp == 1) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tc_occupancy_twin<MINB>, TC_THREADS, smem) == cudaSuccess)
            n = (per_sm > MINB ? MINB : per_sm) * sms;
    } else {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, sp); cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = sp;
        cfg.attrs = attr; cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, tc_occupancy_twin<MINB>, &cfg) == cudaSuccess) n = clusters * sp;
    }
    (void)cudaGetLastError();
    if (n <= 0) n = sms / sp * sp;                                  // unknown: one CTA per SM
    cache[sp] = n;
    return n;
}

// A weight-streaming launch (one token tile).  Estimate, for every split count that leaves >= 4 k-blocks per
// CTA, waves x (fixed cost + the time its resident CTAs need to stream their share) and take the least.  The
// capacity is what the device says can be resident as clusters of that size - fewer than SMs x CTAs/SM when
// clusters do not tile the GPCs.  caps (optional, 9 ints) receives the capacities that were used.
template <int BN, int STAGES, bool DUAL>
static int tc_choose_splits(int tiles, int total_kb, size_t smem, int* caps) {
    const double kb_us = (double)(TC_BM * TC_BK * 2 * (DUAL ? 2 : 1)) / 6.5e6;   // one k-block of weights at 6.5 TB/s
    double best = 1e30;
    int splits = 1;
    for (int sp = 1; sp <= 8 && total_kb / sp >= 4; ++sp) {
        // a tenth of the slots stays free: the kernels after this one then find room to start early and fetch
        // their own first tiles while this one drains (measured inside whole decode steps)
        const int cap = tc_capacity<BN, STAGES, DUAL>(sp, smem) * 9 / 10;
        if (caps) caps[sp] = cap;
        const long long ctas = (long long)tiles * sp;
        const long long waves = (ctas + cap - 1) / cap;
        const long long resident = ctas < cap ? ctas : cap;
        const double kbs = (double)rb_ceil_div(total_kb, sp);
        const double shared_us = kbs * kb_us * (double)resident;        // all resident CTAs at the device's bandwidth
        const double alone_us = kbs * kb_us * 6.5e6 / 30e3;              // one CTA's pipeline sustains about 30 GB/s
        const double cost = (double)waves * (6.0 + (sp > 1 ? 3.0 : 0.0) + (shared_us > alone_us ? shared_us : alone_us));
        if (cost < best - 0.25) { best = cost; splits = sp; }
    }
    return splits;
}

// REINFER_B200_GEMM_SPLITS="NxK:S,NxK:S,..." fixes the cluster split of products with these weight shapes (N counts
// both matrices of a gated pair), for tuning; anything else is chosen by the model above.
static int tc_env_splits(int N, int K) {
    static const char* env = getenv("REINFER_B200_GEMM_SPLITS");
    if (!env) return 0;
    for (const char* p = env; *p;) {
        int n = 0, k = 0, sp = 0;
        if (sscanf(p, "%dx%d:%d", &n, &k, &sp) == 3 && n == N && k == K && sp >= 1 && sp <= 8) return sp;
        while (*p && *p != ',') ++p;
        if (*p == ',') ++p;
    }
    return 0;
}

// want_splits: 0 = choose; > 0 = that many through a cluster (at most 8); < 0 = that many through the workspace.
template <int BN, int STAGES, bool DUAL>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, void* C, float* ws, long long ws_floats, int T, int N, int K,
                     long long ldc, int mode, int want_splits, const TcExtra& ex, cudaStream_t s,
                     bool keep_partials = false) {
    constexpr size_t smem = (size_t)STAGES * ((DUAL ? 2 : 1) * TC_BM * TC_BK * 2 + BN * TC_BK * 2) + sizeof(TcShared) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        // the whole of the SM's memory as shared memory, so that two CTAs of the small-tile kernels fit beside each other
        (void)cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, DUAL>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = true;
    }
    const int total_kb = rb_ceil_div(K, TC_BK);
    const int t_tiles = rb_ceil_div(T, BN), n_tiles = rb_ceil_div(N, TC_BM);
    const int tiles = t_tiles * n_tiles;
    // a cluster's CTAs park their accumulators ([tokens][128] floats, twice for DUAL) in the operand stages
    constexpr size_t park_bytes = (size_t)(DUAL ? 2 : 1) * BN * TC_BM * sizeof(float);
    constexpr bool can_park = park_bytes <= (size_t)STAGES * ((DUAL ? 2 : 1) * TC_BM * TC_BK * 2 + BN * TC_BK * 2);
    int splits = 1;
    bool via_ws = false;
    if (want_splits > 0) { splits = want_splits; via_ws = !can_park; }
    else if (want_splits < 0) { splits = -want_splits; via_ws = true; }
    else if (t_tiles == 1 && can_park) {
        splits = tc_env_splits(DUAL ? 2 * N : N, K);
        if (!splits) splits = tc_choose_splits<BN, STAGES, DUAL>(tiles, total_kb, smem, nullptr);
    }
    if (splits > total_kb) splits = total_kb;
    int kb_per_split = rb_ceil_div(total_kb, splits);
    splits = rb_ceil_div(total_kb, kb_per_split);                   // no empty split
    if (splits > 8) via_ws = true;                                  // larger than a portable cluster
    if (DUAL && via_ws) { splits = 1; via_ws = false; kb_per_split = total_kb; }   // two accumulators never go through the workspace
    if (via_ws) {
        while (splits > 1 && (!ws || (long long)splits * T * N > ws_floats)) --splits;
        kb_per_split = rb_ceil_div(total_kb, splits);
        splits = rb_ceil_div(total_kb, kb_per_split);
    }
    const int csplit = (splits > 1 && !via_ws) ? splits : 1;
    if (keep_partials && !via_ws) RB_REFUSE("gemm: partial sums go through the workspace");
    const int out_mode = ((splits > 1 || keep_partials) && via_ws) ? 3 : mode;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(t_tiles, n_tiles, splits);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (csplit > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = csplit;
        ++na;
    }
    if (g_rb_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, STAGES, DUAL>, mw, mx, C, ws, T, N, K, ldc, out_mode, kb_per_split, csplit, ex);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
    int rc = RB_LAUNCH_RESULT();
    if (rc) return rc;
    if (splits > 1 && via_ws && !keep_partials) {
        const long long total = (long long)T * N;
        return rb_launch(splitk_reduce_kernel, dim3(rb_ceil_div(total, 256)), dim3(256), 0, s, (const float*)ws, C, T, N, ldc, splits, mode);
    }
    return 0;
}

static int g_tc_persistent = 1;
// Schedule of products with several token tiles: 0 = one CTA per tile, 1 = persistent CTAs.  Returns the old value.
extern "C" int rb_set_gemm_persistent(int mode) { int old = g_tc_persistent; g_tc_persistent = mode ? 1 : 0; return old; }

static int g_tc_token_lanes = 1;
// Persistent products of several token tiles: 1 = a token per accumulator lane (128 tokens x 256 features a tile),
// 0 = a feature per lane (128 features x 256 or 128 tokens).  Returns the old value.
extern "C" int rb_set_gemm_token_lanes(int v) { int old = g_tc_token_lanes; g_tc_token_lanes = v ? 1 : 0; return old; }

static int g_tc_gated_stream = 1;
// The gated pair over 65 .. 128 tokens: 1 = the streaming kernel with a token per lane (64 + 64 weight rows a CTA),
// 0 = the kernel with a feature per lane (128 + 128 rows a CTA).  Returns the old value.
extern "C" int rb_set_gemm_gated_stream(int v) { int old = g_tc_gated_stream; g_tc_gated_stream = v ? 1 : 0; return old; }

static int g_tc_tile_feats = 0;
// Weight rows per tile of the token-lane forms: 0 = chosen per product, 256 (four stages) or 224 (five).  Returns the old value.
extern "C" int rb_set_gemm_tile_features(int v) {
    int old = g_tc_tile_feats;
    g_tc_tile_feats = (v == 256 || v == 224) ? v : 0;
    return old;
}

static int tc_bn(int T) { return T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256; }

// The extras of a launch from the entry points' arguments (-1 and a message if they make no sense).
static TcRows tc_rows(const TcExtra& ex) {
    TcRows rs{};
    rs.row_sumsq = ex.row_sumsq; rs.sumsq_parts = ex.sumsq_parts; rs.inv_width = ex.inv_width; rs.eps = ex.eps;
    return rs;
}

// Weight rows per tile of the token-lane persistent product of T tokens and N features: 256 in four stages, or 224 in
// five.  A 64-deep k-step costs a tile about 600 cycles with four stages in flight whatever its width (the operands'
// latency sets the pace, not their bytes) and about 500 with five (then issuing the step's products does); the narrower
// tile wins where its count does not add a round over the SMs.
static int tc_token_lane_rows(int T, int N) {
    if (g_tc_tile_feats) return g_tc_tile_feats;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int t_tiles = rb_ceil_div(T, 128);
    const double c256 = 600.0 * rb_ceil_div((long long)rb_ceil_div(N, 256) * t_tiles, sms);
    const double c224 = 500.0 * rb_ceil_div((long long)rb_ceil_div(N, 224) * t_tiles, sms);
    return c224 < c256 ? 224 : 256;
}

// Whether a product over T tokens applies row factors (rows that lack their RMS factor) in its epilogue: the streaming
// kernels always do, the persistent ones in their token-lane forms.
extern "C" int rb_gemm_row_scale_ok(int T) { return T <= 256 || (g_tc_persistent && g_tc_token_lanes) ? 1 : 0; }

static int tc_extra(TcExtra* ex, const void* next_w, long long next_bytes, const float* row_sumsq, int sumsq_parts,
                    int norm_width, float norm_eps, int T) {
    if ((uintptr_t)next_w & 15) RB_REFUSE("gemm: the range to prefetch must start on a 16-byte boundary");
    if (row_sumsq && (sumsq_parts < 1 || sumsq_parts > 1024 || norm_width < 1))
        RB_REFUSE("gemm: a row factor from %d parts over a width of %d", sumsq_parts, norm_width);
    if (row_sumsq && !rb_gemm_row_scale_ok(T)) RB_REFUSE("gemm: row factors over %d tokens need the token-lane persistent product", T);
    ex->next_w = next_w; ex->next_bytes = next_w ? next_bytes : 0;
    ex->row_sumsq = row_sumsq; ex->sumsq_parts = sumsq_parts;
    ex->inv_width = row_sumsq ? 1.0f / (float)norm_width : 0.0f; ex->eps = norm_eps;
    ex->prep_w = nullptr; ex->prep_w_f32 = 0; ex->prep_rows = nullptr; ex->prep_sumsq = nullptr;
    ex->h_q_out = nullptr; ex->h_cache = nullptr; ex->h_kv_slot = nullptr; ex->h_positions = nullptr; ex->h_inv_freq = nullptr;
    ex->h_q_w = ex->h_k_w = nullptr; ex->h_w_f32 = 0; ex->h_QH = ex->h_KH = 0; ex->h_page = 1; ex->h_eps = 0.0f;
    return 0;
}

// X [T,K] bf16 (row stride ldx), W [N,K] bf16 (row stride ldw), C [T,N] bf16 or float (row stride ldc).
// ws: float workspace of ws_floats elements for split-K partials beyond a cluster (may be null).
extern "C" int rb_gemm_bf16(const void* X, const void* W, void* C, int c_dtype, int accumulate, int T, int N, int K,
                            long long ldx, long long ldw, long long ldc, float* ws, long long ws_floats,
                            int force_splits, const void* next_w, long long next_bytes,
                            const float* row_sumsq, int sumsq_parts, int norm_width, float norm_eps, void* stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0) RB_REFUSE("gemm: K=%d", K);
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15))
        RB_REFUSE("gemm: TMA needs 16-byte aligned operands and row strides (ldx %lld, ldw %lld)", ldx, ldw);
    if (accumulate && c_dtype != RB_F32) RB_REFUSE("gemm: accumulation needs a float destination");
    if (c_dtype != RB_F32 && c_dtype != RB_BF16) RB_REFUSE("gemm: destination dtype %d", c_dtype);
    TcExtra ex;
    if (tc_extra(&ex, next_w, next_bytes, row_sumsq, sumsq_parts, norm_width, norm_eps, T)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int mode = accumulate ? 2 : (c_dtype == RB_F32 ? 1 : 0);
    const int bn = tc_bn(T);
    CUtensorMap mw, mx;
    if (rb_tensor_map_bf16(W, N, K, ldw, TC_BM, &mw)) return -1;
    if (T > 256 && force_splits == 0 && g_tc_persistent) {          // several token tiles: the persistent schedule
        // Token tiles of 256 or of 128: whichever needs less time for its rounds over the SMs.  A 128 x 128 tile
        // reads as many operand bytes from shared memory per MMA as a 128 x 256 one for half the work, so its
        // rounds count 1.36 times their width; the wider tile wins ties (the weights are read once less often).
        // A token per accumulator lane (128 tokens x 256 features a tile): a lane writes 32 bytes of its row at a time
        // (stored results) or adds 16 bytes at a time where they live (added results), which keeps the one epilogue that
        // nothing hides, the last, short.  rb_set_gemm_token_lanes(0) runs the form with a feature per lane instead.
        const bool flip = g_tc_token_lanes != 0;
        if (flip) {
            const bool narrow = tc_token_lane_rows(T, N) == 224;
            if (rb_tensor_map_bf16(W, N, K, ldw, narrow ? 224 : 256, &mw)) return -1;
            if (rb_tensor_map_bf16(X, T, K, ldx, 128, &mx)) return -1;
            if (narrow) return launch_tc_persistent<128, 5, 2, 224>(mw, mx, C, T, N, K, ldc, mode, s, TcHeads{}, tc_rows(ex));
            return launch_tc_persistent<128, 4, 2, 256>(mw, mx, C, T, N, K, ldc, mode, s, TcHeads{}, tc_rows(ex));
        }
        if (row_sumsq) RB_REFUSE("gemm: row factors over %d tokens need the token-lane persistent product", T);
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long n_tiles = rb_ceil_div(N, TC_BM);
        const double c256 = (double)rb_ceil_div((long long)rb_ceil_div(T, 256) * n_tiles, sms) * 256.0;
        const double c128 = (double)rb_ceil_div((long long)rb_ceil_div(T, 128) * n_tiles, sms) * 128.0 * 1.36;
        if (c128 < c256) {
            if (rb_tensor_map_bf16(X, T, K, ldx, 128, &mx)) return -1;
            return launch_tc_persistent<128, 5, 0>(mw, mx, C, T, N, K, ldc, mode, s);
        }
#ifdef RB_TIMELINE
        if (const char* v = getenv("REINFER_B200_TRACE_TILE")) {     // "BN,STAGES": other pipelines, to be compared in the tile trace
            int tb = 0, ts = 0;
            if (sscanf(v, "%d,%d", &tb, &ts) == 2) {
                if (rb_tensor_map_bf16(X, T, K, ldx, tb, &mx)) return -1;
                if (tb == 256 && ts == 2) return launch_tc_persistent<256, 2, 0>(mw, mx, C, T, N, K, ldc, mode, s);
                if (tb == 256 && ts == 3) return launch_tc_persistent<256, 3, 0>(mw, mx, C, T, N, K, ldc, mode, s);
                if (tb == 128 && ts == 3) return launch_tc_persistent<128, 3, 0>(mw, mx, C, T, N, K, ldc, mode, s);
                if (tb == 128 && ts == 4) return launch_tc_persistent<128, 4, 0>(mw, mx, C, T, N, K, ldc, mode, s);
                if (tb == 128 && ts == 6) return launch_tc_persistent<128, 6, 0>(mw, mx, C, T, N, K, ldc, mode, s);
                if (tb == 64 && ts == 4) return launch_tc_persistent<64, 4, 0>(mw, mx, C, T, N, K, ldc, mode, s);
                if (tb == 64 && ts == 8) return launch_tc_persistent<64, 8, 0>(mw, mx, C, T, N, K, ldc, mode, s);
                RB_REFUSE("REINFER_B200_TRACE_TILE=%s is not instantiated", v);
            }
        }
#endif
        if (rb_tensor_map_bf16(X, T, K, ldx, 256, &mx)) return -1;
        return launch_tc_persistent<256, 4, 0>(mw, mx, C, T, N, K, ldc, mode, s);
    }
    if (row_sumsq && T > 256) RB_REFUSE("gemm: row factors over %d tokens need the token-lane persistent product", T);
    if (rb_tensor_map_bf16(X, T, K, ldx, bn, &mx)) return -1;
    switch (bn) {
        case 16: return launch_tc<16, 6, false>(mw, mx, C, ws, ws_floats, T, N, K, ldc, mode, force_splits, ex, s);
        case 32: return launch_tc<32, 5, false>(mw, mx, C, ws, ws_floats, T, N, K, ldc, mode, force_splits, ex, s);
        case 64: return launch_tc<64, 4, false>(mw, mx, C, ws, ws_floats, T, N, K, ldc, mode, force_splits, ex, s);
        case 128: return launch_tc<128, 5, false>(mw, mx, C, ws, ws_floats, T, N, K, ldc, mode, force_splits, ex, s);
        default: return launch_tc<256, 4, false>(mw, mx, C, ws, ws_floats, T, N, K, ldc, mode, force_splits, ex, s);
    }
}

// C (float, [T, N], row stride ldc) += X W^T for one token tile, reduced inside a cluster, with the rows of the RMS norm
// that reads C next prepared by the same CTAs: prep_rows [T, N] bfloat16 = new C * norm_w (the norm without its
// division), prep_sumsq [T, N / 128] = the new C's sum of squares by tiles of 128 features.  One token tile, N a
// multiple of 128; refused otherwise (the caller then runs the product and the norm one after the other).  (Over several
// token tiles the same in the persistent product's epilogue was measured: no faster at the 8B shape, 5 % slower at 4B -
// the lanes have to load the old sums where they now only send additions, and the last tile's epilogue hides behind nothing.)
extern "C" int rb_gemm_bf16_residual_norm(const void* X, const void* W, float* C, int T, int N, int K, long long ldx, long long ldw,
                                          long long ldc, const void* norm_w, int norm_w_dtype, void* prep_rows, float* prep_sumsq,
                                          const void* next_w, long long next_bytes, const float* row_sumsq, int sumsq_parts,
                                          int norm_width, float norm_eps, void* stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0) RB_REFUSE("gemm: K=%d", K);
    if (T > 256) RB_REFUSE("gemm_residual_norm: one token tile (%d tokens)", T);
    if (N % TC_BM || K < 2 * TC_BK)
        RB_REFUSE("gemm_residual_norm: features in tiles of 128, two blocks of K at least (N %d, K %d)", N, K);
    if ((ldc & 3) || ((uintptr_t)C & 15) || ((uintptr_t)prep_rows & 7) || ((uintptr_t)norm_w & 15))
        RB_REFUSE("gemm_residual_norm: 16-byte aligned sum and weight, rows 8-byte aligned (ldc %lld)", ldc);
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15))
        RB_REFUSE("gemm: TMA needs 16-byte aligned operands and row strides (ldx %lld, ldw %lld)", ldx, ldw);
    if (!norm_w || !prep_rows || !prep_sumsq) RB_REFUSE("gemm: the norm's weight and both of its outputs are needed");
    if (norm_w_dtype != RB_F32 && norm_w_dtype != RB_BF16) RB_REFUSE("gemm: norm weight of dtype %d", norm_w_dtype);
    TcExtra ex;
    if (tc_extra(&ex, next_w, next_bytes, row_sumsq, sumsq_parts, norm_width, norm_eps, T)) return -1;
    ex.prep_w = norm_w; ex.prep_w_f32 = norm_w_dtype == RB_F32; ex.prep_rows = (bf16*)prep_rows; ex.prep_sumsq = prep_sumsq;
    cudaStream_t s = (cudaStream_t)stream;
    const int bn = tc_bn(T);
    CUtensorMap mw, mx;
    if (rb_tensor_map_bf16(W, N, K, ldw, TC_BM, &mw)) return -1;
    if (rb_tensor_map_bf16(X, T, K, ldx, bn, &mx)) return -1;
    // the cluster's size as the plain product would choose it, but never one CTA alone: the reduction's code does the norm's part
    const int total_kb = rb_ceil_div(K, TC_BK), tiles = rb_ceil_div(N, TC_BM);
    int sp = tc_env_splits(N, K);
    switch (bn) {
#define RB_CASE(BN_, ST_) \
        case BN_: { \
            constexpr size_t smem = (size_t)ST_ * (TC_BM * TC_BK * 2 + BN_ * TC_BK * 2) + sizeof(TcShared) + 1024; \
            if (!sp) sp = tc_choose_splits<BN_, ST_, false>(tiles, total_kb, smem, nullptr); \
            if (sp < 2) sp = 2; \
            return launch_tc<BN_, ST_, false>(mw, mx, C, nullptr, 0, T, N, K, ldc, 2, sp, ex, s); }
        RB_CASE(16, 6) RB_CASE(32, 5) RB_CASE(64, 4) RB_CASE(128, 5)
        default: RB_CASE(256, 4)
#undef RB_CASE
    }
}

// The q/k/v projection of a decode step's few rows with the per-head work done by the cluster that reduces it (heads of
// 128, the whole head rotated; see TcExtra): X [T, K] bf16, W [(QH + 2 KH) * 128, K] bf16.  One token tile.
extern "C" int rb_gemm_qkv_heads_stream(const void* X, const void* W, int T, int K, long long ldx, long long ldw, int QH, int KH,
                                        void* q_out, void* cache, const int* kv_slot, const int* positions, const float* inv_freq,
                                        const void* q_w, const void* k_w, int w_dtype, float eps, int page_size,
                                        const void* next_w, long long next_bytes, const float* row_sumsq, int sumsq_parts,
                                        int norm_width, float norm_eps, void* stream) {
    if (T <= 0) return 0;
    if (T > 256 || K < 2 * TC_BK) RB_REFUSE("gemm_qkv_heads_stream: one token tile and two blocks of K at least (T %d, K %d)", T, K);
    if (QH <= 0 || KH <= 0 || page_size <= 0) RB_REFUSE("gemm_qkv_heads_stream: heads %d/%d, page %d", QH, KH, page_size);
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15))
        RB_REFUSE("gemm: TMA needs 16-byte aligned operands and row strides (ldx %lld, ldw %lld)", ldx, ldw);
    if (!q_out || !positions || !inv_freq || (!cache && kv_slot)) RB_REFUSE("gemm_qkv_heads_stream: q_out, positions, inv_freq (and a cache for the slots) are needed");
    if (((uintptr_t)q_out & 7) || ((uintptr_t)cache & 7)) RB_REFUSE("gemm_qkv_heads_stream: destinations must be 8-byte aligned");
    if ((q_w == nullptr) != (k_w == nullptr)) RB_REFUSE("gemm_qkv_heads_stream: q and k norm weights come together");
    if (q_w && w_dtype != RB_F32 && w_dtype != RB_BF16) RB_REFUSE("gemm_qkv_heads_stream: norm weights of dtype %d", w_dtype);
    TcExtra ex;
    if (tc_extra(&ex, next_w, next_bytes, row_sumsq, sumsq_parts, norm_width, norm_eps, T)) return -1;
    ex.h_q_out = (bf16*)q_out; ex.h_cache = (bf16*)cache; ex.h_kv_slot = kv_slot; ex.h_positions = positions; ex.h_inv_freq = inv_freq;
    ex.h_q_w = q_w; ex.h_k_w = k_w; ex.h_w_f32 = w_dtype == RB_F32; ex.h_QH = QH; ex.h_KH = KH; ex.h_page = page_size; ex.h_eps = eps;
    cudaStream_t s = (cudaStream_t)stream;
    const int N = (QH + 2 * KH) * 128;
    const int bn = tc_bn(T);
    CUtensorMap mw, mx;
    if (rb_tensor_map_bf16(W, N, K, ldw, TC_BM, &mw)) return -1;
    if (rb_tensor_map_bf16(X, T, K, ldx, bn, &mx)) return -1;
    const int total_kb = rb_ceil_div(K, TC_BK), tiles = rb_ceil_div(N, TC_BM);
    int sp = tc_env_splits(N, K);
    switch (bn) {
#define RB_CASE(BN_, ST_) \
        case BN_: { \
            constexpr size_t smem = (size_t)ST_ * (TC_BM * TC_BK * 2 + BN_ * TC_BK * 2) + sizeof(TcShared) + 1024; \
            if (!sp) sp = tc_choose_splits<BN_, ST_, false>(tiles, total_kb, smem, nullptr); \
            if (sp < 2) sp = 2; \
            return launch_tc<BN_, ST_, false>(mw, mx, nullptr, nullptr, 0, T, N, K, N, 0, sp, ex, s); }
        RB_CASE(16, 6) RB_CASE(32, 5) RB_CASE(64, 4) RB_CASE(128, 5)
        default: RB_CASE(256, 4)
#undef RB_CASE
    }
}

// How many partial sums rb_gemm_bf16_partials leaves for T tokens, N features and K: as many splits of K as
// keep most resident CTA slots busy (two CTAs per SM for up to 64 tokens, else one) with at least four
// 64-wide blocks of K each.  No cluster is involved, so nothing limits the count but the work.
extern "C" int rb_gemm_partials_plan(int T, int N, int K) {
    if (T <= 0 || N <= 0 || K <= 0) return 1;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int bn = tc_bn(T);
    // four fifths of the slots: the kernels after this one then find room to start early and fetch their own
    // first tiles while this one drains (measured inside whole decode steps; REINFER_B200_PARTIAL_FILL for tuning)
    static const char* fill_env = getenv("REINFER_B200_PARTIAL_FILL");
    const double fill = fill_env ? atof(fill_env) : 0.8;
    const int slots = (int)(sms * (bn <= 64 ? 2 : 1) * (fill > 0.05 && fill <= 1.0 ? fill : 0.8));
    const int tiles = rb_ceil_div(T, bn) * rb_ceil_div(N, TC_BM), total_kb = rb_ceil_div(K, TC_BK);
    int sp = slots / tiles;
    if (sp > total_kb / 4) sp = total_kb / 4;
    if (sp > 32) sp = 32;
    if (sp < 1) sp = 1;
    const int per = rb_ceil_div(total_kb, sp);
    return rb_ceil_div(total_kb, per);
}

// partials[s][T][N] (float) = X[:, K-range s] W[:, K-range s]^T for the `splits` ranges of K that
// rb_gemm_partials_plan names: the product without its last sum, which the kernel that reads the result
// forms on the way (the residual sum and norm, the head norm) - no CTA waits for another.
extern "C" int rb_gemm_bf16_partials(const void* X, const void* W, float* partials, int splits, int T, int N, int K,
                                     long long ldx, long long ldw, const void* next_w, long long next_bytes,
                                     const float* row_sumsq, int sumsq_parts, int norm_width, float norm_eps, void* stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0) RB_REFUSE("gemm: K=%d", K);
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15))
        RB_REFUSE("gemm: TMA needs 16-byte aligned operands and row strides (ldx %lld, ldw %lld)", ldx, ldw);
    if (T > 256) RB_REFUSE("gemm: partial sums are for one token tile (%d tokens)", T);
    TcExtra ex;
    if (tc_extra(&ex, next_w, next_bytes, row_sumsq, sumsq_parts, norm_width, norm_eps, T)) return -1;
    if (splits != rb_gemm_partials_plan(T, N, K)) RB_REFUSE("gemm: %d partial sums where the plan names %d", splits, rb_gemm_partials_plan(T, N, K));
    cudaStream_t s = (cudaStream_t)stream;
    const int bn = tc_bn(T);
    CUtensorMap mw, mx;
    if (rb_tensor_map_bf16(W, N, K, ldw, TC_BM, &mw)) return -1;
    if (rb_tensor_map_bf16(X, T, K, ldx, bn, &mx)) return -1;
    const long long wsf = (long long)splits * T * N;
    switch (bn) {
        case 16: return launch_tc<16, 6, false>(mw, mx, nullptr, partials, wsf, T, N, K, N, 1, -splits, ex, s, true);
        case 32: return launch_tc<32, 5, false>(mw, mx, nullptr, partials, wsf, T, N, K, N, 1, -splits, ex, s, true);
        case 64: return launch_tc<64, 4, false>(mw, mx, nullptr, partials, wsf, T, N, K, N, 1, -splits, ex, s, true);
        case 128: return launch_tc<128, 5, false>(mw, mx, nullptr, partials, wsf, T, N, K, N, 1, -splits, ex, s, true);
        default: return launch_tc<256, 4, false>(mw, mx, nullptr, partials, wsf, T, N, K, N, 1, -splits, ex, s, true);
    }
}

// The attention's q/k/v projection over a prompt portion with everything that follows it per head: X [T, K] bf16,
// W [(QH + 2 KH) * 128, K] bf16 (query heads, key heads, value heads); q_out [T, QH, 128] gets the normalised and
// rotated queries, the layer's cache pages the keys (normalised, rotated) and the values of every token whose kv_slot
// is not negative.  Heads of 128, the whole head rotated, several token tiles (T > 256): the caller takes the
// two-kernel way otherwise.
extern "C" int rb_gemm_qkv_heads(const void* X, const void* W, int T, int K, long long ldx, long long ldw, int QH, int KH,
                                 void* q_out, void* cache, const int* kv_slot, const void* cs_table, const void* q_w,
                                 const void* k_w, int w_dtype, float eps, int page_size,
                                 const float* row_sumsq, int sumsq_parts, int norm_width, float norm_eps, void* stream) {
    if (T <= 256) RB_REFUSE("gemm_qkv_heads: %d tokens (more than 256: the persistent product)", T);
    if (QH <= 0 || KH <= 0 || K <= 0 || page_size <= 0) RB_REFUSE("gemm_qkv_heads: heads %d/%d, K %d, page %d", QH, KH, K, page_size);
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15))
        RB_REFUSE("gemm_qkv_heads: TMA needs 16-byte aligned operands and row strides (ldx %lld, ldw %lld)", ldx, ldw);
    if (!q_out || !cache || !cs_table || !q_w || !k_w) RB_REFUSE("gemm_qkv_heads: q_out, cache, table and both norm weights are needed");
    if (((uintptr_t)q_out & 15) || ((uintptr_t)cache & 15)) RB_REFUSE("gemm_qkv_heads: destinations must be 16-byte aligned");
    if (w_dtype != RB_F32 && w_dtype != RB_BF16) RB_REFUSE("gemm_qkv_heads: norm weights of dtype %d", w_dtype);
    TcHeads hd{};
    hd.q_out = (bf16*)q_out; hd.cache = (bf16*)cache; hd.kv_slot = kv_slot; hd.cs_table = (const float2*)cs_table;
    hd.q_w = q_w; hd.k_w = k_w; hd.w_f32 = w_dtype == RB_F32; hd.QH = QH; hd.KH = KH; hd.page_size = page_size; hd.eps = eps;
    const int N = (QH + 2 * KH) * 128;
    CUtensorMap mw, mx;
    if (rb_tensor_map_bf16(W, N, K, ldw, 256, &mw)) return -1;
    if (rb_tensor_map_bf16(X, T, K, ldx, 128, &mx)) return -1;
    TcExtra ex;
    if (tc_extra(&ex, nullptr, 0, row_sumsq, sumsq_parts, norm_width, norm_eps, T)) return -1;
    return launch_tc_persistent<128, 4, 3, 256>(mw, mx, nullptr, T, N, K, 0, 0, (cudaStream_t)stream, hd, tc_rows(ex));
}

// act[T,F] (bfloat16) = silu(X Wg^T) * (X Wu^T) for Wgu = [Wg; Wu] of shape [2F, K]: one product with two
// accumulators and the activation in the epilogue.  Splits (at most 8) reduce inside a cluster.
extern "C" int rb_gemm_bf16_swiglu(const void* X, const void* Wgu, void* act, int T, int F, int K,
                                   long long ldx, long long ldw, long long ldc, int force_splits,
                                   const void* next_w, long long next_bytes,
                                   const float* row_sumsq, int sumsq_parts, int norm_width, float norm_eps, void* stream) {
    if (T <= 0 || F <= 0) return 0;
    if (K <= 0) RB_REFUSE("gemm_swiglu: K=%d", K);
    if (force_splits < 0 || force_splits > 8) RB_REFUSE("gemm_swiglu: %d splits (0 = choose, at most a cluster of 8)", force_splits);
    TcExtra ex;
    if (tc_extra(&ex, next_w, next_bytes, row_sumsq, sumsq_parts, norm_width, norm_eps, T)) return -1;
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)Wgu & 15))
        RB_REFUSE("gemm_swiglu: TMA needs 16-byte aligned operands and row strides (ldx %lld, ldw %lld)", ldx, ldw);
    cudaStream_t s = (cudaStream_t)stream;
    const int bn = tc_bn(T);
    CUtensorMap mw, mx;
    if (rb_tensor_map_bf16(Wgu, 2LL * F, K, ldw, TC_BM, &mw)) return -1;
    if (T > 256 && g_tc_persistent) {                               // tiles of 128 tokens x (128 gate + 128 up) weight rows
        // (112 + 112 rows in five stages were measured too: 292 against 290 us at the 8B shape, 154 against 149 at 4B)
        if (rb_tensor_map_bf16(X, T, K, ldx, 128, &mx)) return -1;
        return launch_tc_persistent<128, 4, 1, 256>(mw, mx, act, T, F, K, ldc, 0, s, TcHeads{}, tc_rows(ex));
    }
    if (row_sumsq && T > 256) RB_REFUSE("gemm_swiglu: row factors over %d tokens need the persistent product", T);
    // 65 .. 128 tokens: F / 64 CTAs, two to an SM.  (For 33 .. 64 tokens the same kernel, also with 64-token stages of
    // 24 KB, is faster alone - 40 against 44 us at the 8B shape - but the decode step around it is not: 9.86 against
    // 9.78 ms at batch 64; its 192 CTAs leave the product after it no SM to start on early.)
    if (T > 64 && T <= 128 && force_splits == 0 && g_tc_gated_stream)
        return launch_tc_gated_stream<3, 128>(X, Wgu, act, T, F, K, ldx, ldw, ldc, ex, s);
    if (rb_tensor_map_bf16(X, T, K, ldx, bn, &mx)) return -1;
    switch (bn) {
        case 16: return launch_tc<16, 3, true>(mw, mx, act, nullptr, 0, T, F, K, ldc, 0, force_splits, ex, s);
        case 32: return launch_tc<32, 3, true>(mw, mx, act, nullptr, 0, T, F, K, ldc, 0, force_splits, ex, s);
        case 64: return launch_tc<64, 4, true>(mw, mx, act, nullptr, 0, T, F, K, ldc, 0, force_splits, ex, s);
        case 128: return launch_tc<128, 4, true>(mw, mx, act, nullptr, 0, T, F, K, ldc, 0, force_splits, ex, s);
        default: return launch_tc<256, 3, true>(mw, mx, act, nullptr, 0, T, F, K, ldc, 0, force_splits, ex, s);
    }
}

// What the decode product (T <= 16) would choose for N output features and K: out[0] = splits, out[1..8] = the
// resident-CTA capacity the device reports for clusters of that size.  For tests and tuning.
extern "C" int rb_gemm_plan(int N, int K, int dual, int* out) {
    const int tiles = rb_ceil_div(N, TC_BM), total_kb = rb_ceil_div(K, TC_BK);
    int caps[9] = {0};
    if (dual) {
        constexpr size_t smem = (size_t)3 * (2 * TC_BM * TC_BK * 2 + 16 * TC_BK * 2) + sizeof(TcShared) + 1024;
        cudaFuncSetAttribute(gemm_tc_kernel<16, 3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(gemm_tc_kernel<16, 3, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        out[0] = tc_choose_splits<16, 3, true>(tiles, total_kb, smem, caps);
    } else {
        constexpr size_t smem = (size_t)6 * (TC_BM * TC_BK * 2 + 16 * TC_BK * 2) + sizeof(TcShared) + 1024;
        cudaFuncSetAttribute(gemm_tc_kernel<16, 6, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(gemm_tc_kernel<16, 6, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        out[0] = tc_choose_splits<16, 6, false>(tiles, total_kb, smem, caps);
    }
    for (int i = 1; i <= 8; ++i) out[i] = caps[i];
    return 0;
}

// The error word of the tensor-core kernels (0 = none); synchronises the device.  With reset != 0 it is cleared.
RB_STATUS_EXPORTS(rb_gemm_error, rb_gemm_bind_status)

RB_TL_SETTER(rb_gemm_step_timeline)
