// Paged causal flash attention for prompt portions on the fifth-generation tensor cores.
//
// The formulas are the reference's attention (crates/cuda/kernels/dense_kernels.cu:173-231: scores, causal
// mask, softmax in float, weighted sum of the values), tiled as flash attention: a CTA owns 128 rows
// (128 / Gc tokens x the Gc grouped query heads of one kv head) and walks the request's keys in tiles of 64.
// For every tile
//     S = Q K^T          tcgen05.mma, 128 x 64 x 128, operands in shared memory, S in tensor memory
//     P = exp2(S - max)  128 threads, one row each (tcgen05.ld gives a thread its whole row: the row maximum
//                        and sum need no shuffles), P rounded to bfloat16 into shared memory
//     O += P V           tcgen05.mma, 128 x 128 x 64, accumulated in tensor memory over all tiles: P and O are scaled
//                        to a maximum that follows the true one only when it rose by more than 2^8 (then the row's
//                        thread rescales its lane of O in tensor memory, which is rare), so the rows read O once, at the end
// Warp 0 feeds key/value tiles by TMA exactly as the mma.sync kernels do (one box per page, key/value and
// 64-column half onto a full/empty mbarrier ring); warp 1 allocates tensor memory and issues the MMAs;
// warps 4-11 are the softmax rows.  Q [rows][d], K [keys][d] and P [rows][keys] are K-major operands (the
// descriptor form of the GEMM); V [keys][d] is used as it lands, as an MN-major operand (instruction
// descriptor bit 16; in the shared-memory descriptor the leading offset steps to the second 64 dims, the stride
// offset to the next 8 keys) - nothing is transposed.
//
// Two tiles are in flight: S, P and the P V accumulator exist twice, and so do the rows - two groups of four
// warps take the even and the odd tiles, each with its own running maximum, sum and O, which are combined at the end
// (as the splits of flash decoding are).  While one group waits for its MMA the other computes, and every
// scheduler of the SM has two warps to choose from.  The MMA warp computes the scores of tile i+1 before the
// weighted sum of tile i.  Registers follow the roles (setmaxnreg): 40 for the control warps, 232 for the rows - what
// the control warps give up (128 x 128) must cover what the rows take (256 x 64), for the registers come from the
// CTA's own allocation and a request for more than it holds waits for ever.
//
// Head size 128, page size a power of two >= 8.  Every wait is bounded (2 s); a CTA that gives up raises the
// error word, lets its copies land, frees its tensor memory and leaves.
#define RB_UNIT 3
#include "sm100.cuh"
#include <stdlib.h>

#define FC_BN 64                              // keys per tile
#define FC_ROWS 128                           // query rows per CTA
#define FC_D 128
#define FC_THREADS 384                        // a control group (TMA warp, MMA warp, two idle) and two groups of four row warps
#define FC_NST 5
#define FC_KHALF (FC_BN * 128)                // 64 keys x 128 bytes: one 64-column half of a key (or value) tile
#define FC_KV_BYTES (2 * FC_KHALF)            // a key tile: two halves
#define FC_STAGE (2 * FC_KV_BYTES)            // keys and values
#define FC_QHALF (FC_ROWS * 128)              // 128 rows x 128 bytes
#define FC_RESCALE 8.0f                       // O is brought to a new maximum only when it rose by more than this (log2)
#define FC_TMEM_COLS 512                      // S of two tiles: columns 0..127; P V of two tiles: 128..383

struct FcArgs {
    const bf16* q;
    const int* block_table;
    const int* cu_q;
    const int* kv_len;
    bf16* out;
    int QH, KH, page_size, page_shift, max_pages, window;
    int Gc, chunks, first_entry, n_entries;
    float scale_log2;
};

struct FcShared {
    unsigned long long full[FC_NST];
    unsigned long long empty[FC_NST];
    unsigned long long s_full[2], p_full[2], o_full[2];
    uint32_t tmem_base;
    int abort_flag;
};

// byte offset of 16-byte chunk c (8 elements) of row `row` in a K-major tile of 128-byte rows with the 128-byte
// swizzle; chunks 8.. lie in the next 64-column half, half_bytes further
__device__ __forceinline__ uint32_t fc_off(int row, int c, int half_bytes) {
    return (uint32_t)((c >> 3) * half_bytes + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}
// Sixteen 32-bit columns of this warp's 32 lanes back into tensor memory (the counterpart of tc_ld16).
__device__ __forceinline__ void fc_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void fc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 2^x by the special-function unit alone (one instruction; exp2f adds range handling around it).  The arguments
// here are <= 0 or -inf, where it is accurate to two units in the last place - far inside bfloat16's rounding of P.
__device__ __forceinline__ float fc_ex2(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t fc_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// The bounded wait of sm100.cuh with a pause between polls: here up to twelve warps wait for one another on one SM,
// and a warp that polls without pause takes issue slots from the warps it waits for.
__device__ __forceinline__ bool fc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where) {
    if (mbar_try(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < RB_SPIN_LIMIT; ++it) {
        __nanosleep(40);
        if (mbar_try(bar, parity)) return true;
        if ((it & 63u) == 63u) {
            if (*abort_flag) return false;
            const unsigned long long now = rb_globaltimer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > RB_WAIT_NS) break;
        }
    }
    *abort_flag = where;
    rb_raise(where);
    return false;
}

__global__ void __launch_bounds__(FC_THREADS, 1)
fa_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_kv, const FcArgs a) {
    RB_TL(11);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = smem;                                  // [FC_NST][K half 0, K half 1, V half 0, V half 1]
    unsigned char* sQ = stages + FC_NST * FC_STAGE;                // two halves of [128 rows][64 dims]
    unsigned char* sP = sQ + 2 * FC_QHALF;                         // two of [128 rows][64 keys]
    FcShared* sh = (FcShared*)(sP + 2 * FC_QHALF);
    const uint32_t stages_u = smem_u32(stages), sQ_u = smem_u32(sQ), sP_u = smem_u32(sP);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sh->abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < FC_NST; ++s) {
            mbar_init(smem_u32(&sh->full[s]), 1);
            mbar_init(smem_u32(&sh->empty[s]), 2);                 // the MMA warp's commits: scores done (keys), P V done (values)
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&sh->s_full[b]), 1);
            mbar_init(smem_u32(&sh->p_full[b]), 4);                // one arrival per row warp
            mbar_init(smem_u32(&sh->o_full[b]), 1);
        }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(FC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Nothing that a copy or a thread of this CTA did not write reaches the results: value rows at or beyond the
    // request's length are zeroed before use, scores of such keys and of rows without a token are replaced by
    // -inf whatever they are, P and V^T are written whole before they are read.
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    pdl_trigger();
    pdl_wait();

    // which rows: heavy tiles (late in a request: more keys) first
    const int tpt = FC_ROWS / a.Gc;                                // tokens per CTA
    int tile = (int)gridDim.y - 1 - (int)blockIdx.y, e = a.first_entry, q_len = 0;   // CTAs start in order of x, then y
    for (; e < a.first_entry + a.n_entries; ++e) {
        q_len = a.cu_q[e + 1] - a.cu_q[e];
        const int nt = (q_len + tpt - 1) / tpt;
        if (tile < nt) break;
        tile -= nt;
    }
    const bool none = e >= a.first_entry + a.n_entries;            // uniform: a tile beyond the last entry
    int n_tiles = 0, q0 = 0, n_tok = 0, kv_end = 0, start_pos = 0, tok_base = 0, t_begin = 0, head0 = 0, kh = 0;
    const int* bt = a.block_table;
    if (!none) {
        q0 = tile * tpt;
        n_tok = min(tpt, q_len - q0);
        kh = blockIdx.x / a.chunks;
        head0 = kh * (a.QH / a.KH) + (blockIdx.x % a.chunks) * a.Gc;
        kv_end = a.kv_len[e];
        start_pos = kv_end - q_len;
        tok_base = a.cu_q[e] + q0;
        bt = a.block_table + (size_t)e * a.max_pages;
        const int pos_min = start_pos + q0, pos_max = start_pos + q0 + n_tok - 1;
        const int lo_min = a.window > 0 ? max(0, pos_min - a.window + 1) : 0;
        t_begin = lo_min / FC_BN;
        n_tiles = pos_max / FC_BN + 1 - t_begin;
        // Q rows (row r = token r / Gc, grouped head r % Gc) into the swizzled K-major layout
        for (int i = threadIdx.x; i < n_tok * a.Gc * (FC_D / 8); i += FC_THREADS) {
            const int row = i / (FC_D / 8), c = i % (FC_D / 8);
            const uint4 v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(tok_base + row / a.Gc) * a.QH + head0 + row % a.Gc) * FC_D + c * 8);
            *reinterpret_cast<uint4*>(sQ + fc_off(row, c, FC_QHALF)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    int issued = 0;                                                // producer: tiles whose copies were issued
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");           // the control group gives registers up ...
    if (warp == 0) {
        // ---- producer: runs ahead by up to FC_NST tiles; block-table entries 32 at a time -------------------
        const int box_rows = min(a.page_size, FC_BN);
        const int subs = FC_BN / box_rows;
        const int rows_per_page2 = 2 * a.KH * a.page_size;         // matrix rows of one page (K and V, all heads)
        int cached_first = 0, cached = -1;
        bool have = false;
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % FC_NST;
            const int k0 = (t_begin + it) * FC_BN;
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
                if (it >= FC_NST) ok = fc_wait(smem_u32(&sh->empty[s]), ((it / FC_NST) & 1) ^ 1, abort_flag, 11);
                if (ok) {
                    const uint32_t full = smem_u32(&sh->full[s]);
                    mbar_expect_tx(full, (uint32_t)(n_valid * 4 * box_rows * 128));
                    const uint32_t dst0 = stages_u + s * FC_STAGE;
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        if (pages[u] >= 0) {
                            const int key = k0 + u * box_rows;
                            const int y = pages[u] * rows_per_page2 + kh * a.page_size + (key & (a.page_size - 1));
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                tma_load_2d(dst0 + h * FC_KHALF + u * box_rows * 128, &map_kv, h * 64, y, full);
                                tma_load_2d(dst0 + FC_KV_BYTES + h * FC_KHALF + u * box_rows * 128, &map_kv, h * 64,
                                            y + a.KH * a.page_size, full);
                            }
                        }
                    }
                    issued = it + 1;
                }
            }
            if (!__shfl_sync(0xffffffffu, (int)ok, 0)) break;
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----------------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(FC_BN);
            // S(i) = Q K(i)^T into score buffer i & 1: d = 128 is two 64-column halves of four 16-wide steps each
            auto scores = [&](int i) -> bool {
                const int s = i % FC_NST;
                if (!fc_wait(smem_u32(&sh->full[s]), (i / FC_NST) & 1, abort_flag, 12)) return false;
                tc_fence_after();
                const uint32_t sK = stages_u + s * FC_STAGE;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint64_t dq = make_smem_desc(sQ_u + h * FC_QHALF), dk = make_smem_desc(sK + h * FC_KHALF);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc_mma_bf16(tmem + (uint32_t)((i & 1) * FC_BN), dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s, (h | k) != 0);
                }
                tc_commit(smem_u32(&sh->s_full[i & 1]));
                tc_commit(smem_u32(&sh->empty[s]));                // the keys of this stage are read once these MMAs are done ...
                return true;
            };
            bool ok = n_tiles > 0 && scores(0);
            for (int it = 0; it < n_tiles && ok; ++it) {
                // the scores of the next tile while the rows work on this one (its buffer was read two tiles ago)
                if (it + 1 < n_tiles) ok = scores(it + 1);
                if (!ok) break;
                // O_tile(it) = P V once the rows have written P and V^T (the accumulator was read two tiles ago)
                if (!fc_wait(smem_u32(&sh->p_full[it & 1]), (it >> 1) & 1, abort_flag, 13)) break;
                tc_fence_after();
                // P [rows][keys] is a K-major operand; V [keys][d] as it lies in the stage is an MN-major one: a key's 64
                // dims (128 bytes) contiguous, keys 128 bytes apart, groups of 8 keys 1024 bytes apart (SBO), the second
                // 64 dims a half tile further (LBO); an MMA takes 16 keys = 2048 bytes
                const uint64_t dp = make_smem_desc(sP_u + (it & 1) * FC_QHALF);
                const uint32_t sVs = stages_u + (it % FC_NST) * FC_STAGE + FC_KV_BYTES;
                const uint64_t dv = (uint64_t)((sVs >> 4) & 0x3FFFu) | ((uint64_t)(FC_KHALF >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
                constexpr uint32_t idesc_mn = make_idesc(FC_D) | (1u << 16);       // B is MN-major
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc_mma_bf16(tmem + (uint32_t)(2 * FC_BN + (it & 1) * FC_D), dp + (uint64_t)(k * 2), dv + (uint64_t)(k * (2048 >> 4)), idesc_mn, (it >= 2) || k != 0);
                tc_commit(smem_u32(&sh->o_full[it & 1]));
                tc_commit(smem_u32(&sh->empty[it % FC_NST]));      // ... and its values once these are
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");      // ... and the rows take them
        // ---- softmax rows: thread = row = tensor-memory lane; group g takes tiles g, g + 2, ... ---------------------
        const int g = (warp - 4) >> 2;
        const int quad = warp & 3;                                 // the lanes this warp may read: 32 * (warp % 4) ..
        const int row = quad * 32 + lane;
        const int et = quad * 32 + lane;                           // 0..127 inside the group
        const int ti = row / a.Gc;
        const bool live = !none && ti < n_tok;
        const int pos = live ? start_pos + q0 + ti : -1;
        const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
        // m: the maximum that P and O are scaled to (it follows the true maximum only in steps larger than
        // FC_RESCALE, so that O can stay in tensor memory and be accumulated by the MMA itself); l: the sum in that scale
        float m = -INFINITY, l = 0.0f;
        const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
        const uint32_t s_col = (uint32_t)(g * FC_BN), o_col = (uint32_t)(2 * FC_BN + g * FC_D);
        unsigned char* sPg = sP + g * FC_QHALF;
        bool ok = true;
        for (int it = g; it < n_tiles; it += 2) {
            const int s = it % FC_NST;
            const uint32_t par = (uint32_t)((it >> 1) & 1);
            const int k0 = (t_begin + it) * FC_BN;
            if (k0 + FC_BN > kv_end) {
                // the request's last tile: slots of its last page beyond its length hold foreign data - the values
                // there are zeroed before the tensor core multiplies them (by P = 0, but 0 x NaN is NaN)
                if (!fc_wait(smem_u32(&sh->full[s]), (it / FC_NST) & 1, abort_flag, 14)) { ok = false; break; }
                unsigned char* sV = stages + s * FC_STAGE + FC_KV_BYTES;
                for (int i = et; i < FC_BN * 16; i += FC_ROWS) {
                    const int r = i / 16, c = i % 16;
                    if (k0 + r >= kv_end) *reinterpret_cast<uint4*>(sV + fc_off(r, c, FC_KHALF)) = make_uint4(0, 0, 0, 0);
                }
            }
            // S: this row's 64 scores in one go (one wait for tensor memory); maxima and sums in four independent chains
            if (!fc_wait(smem_u32(&sh->s_full[g]), par, abort_flag, 15)) { ok = false; break; }
            tc_fence_after();
            const bool edge = k0 + FC_BN - 1 > pos || k0 < lo;     // the tile crosses this row's causal edge or window
            uint32_t sr[FC_BN];
#pragma unroll
            for (int c = 0; c < FC_BN / 16; ++c) tc_ld16(lane_base + s_col + (uint32_t)(c * 16), sr + c * 16);
            tc_ld_wait();
            if (edge) {
#pragma unroll
                for (int j = 0; j < FC_BN; ++j) {
                    const int key = k0 + j;
                    if (key < lo || key > pos) sr[j] = 0xff800000u;            // -inf
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < FC_BN; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sr[j]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;   // the scale is positive
            // the scale follows the maximum at once while the row has nothing yet (m = -inf: O and l are zero), else
            // only when the maximum rose by more than FC_RESCALE - P then stays below 2^FC_RESCALE, which bfloat16
            // and the float accumulators hold as well as values below 1
            float alpha = 1.0f;
            if (m == -INFINITY) m = mx;
            else if (mx > m + FC_RESCALE) { alpha = fc_ex2(m - mx); m = mx; }
            const bool rescale = __any_sync(0xffffffffu, alpha != 1.0f);
            // the product before this one (same accumulator, same P buffer) must be done before either is touched
            if (it >= 2) {
                if (!fc_wait(smem_u32(&sh->o_full[g]), par ^ 1, abort_flag, 16)) { ok = false; break; }
                tc_fence_after();
            }
            if (rescale && it >= 2) {
                // rare: O = O * alpha in tensor memory, every lane of the warp with its own factor (1 for most)
#pragma unroll
                for (int c = 0; c < FC_D / 32; ++c) {
                    uint32_t ov[32];
                    tc_ld16(lane_base + o_col + (uint32_t)(c * 32), ov);
                    tc_ld16(lane_base + o_col + (uint32_t)(c * 32 + 16), ov + 16);
                    tc_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
                    fc_st16(lane_base + o_col + (uint32_t)(c * 32), ov);
                    fc_st16(lane_base + o_col + (uint32_t)(c * 32 + 16), ov + 16);
                }
                fc_st_wait();
            }
            const float base = m == -INFINITY ? 0.0f : m;
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < FC_BN / 8; ++c) {
                float p[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) { p[j] = fc_ex2(fmaf(__uint_as_float(sr[c * 8 + j]), a.scale_log2, -base)); sum4[j & 3] += p[j]; }
                uint4 pk;
                pk.x = fc_pack(p[0], p[1]); pk.y = fc_pack(p[2], p[3]); pk.z = fc_pack(p[4], p[5]); pk.w = fc_pack(p[6], p[7]);
                *reinterpret_cast<uint4*>(sPg + fc_off(row, c, 0)) = pk;
            }
            l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // P (and zeroed value rows) before the tensor core reads them
            tc_fence_before();                                     // S is read, O (if touched) written: the MMA may go on
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->p_full[g]));
        }
        // the row of O, once the group's last product is done
        float o[FC_D];
#pragma unroll
        for (int j = 0; j < FC_D; ++j) o[j] = 0.0f;
        const int n_mine = n_tiles > g ? (n_tiles - g + 1) / 2 : 0;
        if (ok && n_mine > 0 && fc_wait(smem_u32(&sh->o_full[g]), (uint32_t)((n_mine - 1) & 1), abort_flag, 17)) {
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < FC_D / 64; ++c) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) tc_ld16(lane_base + o_col + (uint32_t)(c * 64 + q4 * 16), reinterpret_cast<uint32_t*>(o) + c * 64 + q4 * 16);
                tc_ld_wait();
            }
            tc_fence_before();
        }
        // The two groups' results for a row are combined like two splits: group 1 hands its maximum, sum and O over
        // through the (now idle) stages, group 0 adds and stores.  Both reach the barrier whatever happened before.
        float* xo = reinterpret_cast<float*>(stages);              // [128 rows][128] + [128] m + [128] l: 66.5 KB of the ring's 160
        asm volatile("bar.sync 3, %0;" ::"n"(2 * FC_ROWS) : "memory");          // both groups are done with the ring
        if (g == 1) {
#pragma unroll
            for (int j = 0; j < FC_D; ++j) xo[j * FC_ROWS + row] = o[j];        // column-major: neighbouring rows, neighbouring words
            xo[FC_D * FC_ROWS + row] = m;
            xo[FC_D * FC_ROWS + FC_ROWS + row] = l;
        }
        asm volatile("bar.sync 3, %0;" ::"n"(2 * FC_ROWS) : "memory");
        if (g == 0 && live && !*abort_flag) {
            const float m1 = xo[FC_D * FC_ROWS + row], l1 = xo[FC_D * FC_ROWS + FC_ROWS + row];
            const float M = fmaxf(m, m1);
            const float base = M == -INFINITY ? 0.0f : M;
            const float f0 = fc_ex2(m - base), f1 = fc_ex2(m1 - base);
            const float L = l * f0 + l1 * f1;
            const float inv = L > 0.0f ? 1.0f / L : 0.0f;
            const float w0 = f0 * inv, w1 = f1 * inv;
            bf16* dst = a.out + ((size_t)(tok_base + ti) * a.QH + head0 + row % a.Gc) * FC_D;
#pragma unroll
            for (int c = 0; c < FC_D / 8; ++c) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = o[c * 8 + j] * w0 + xo[(c * 8 + j) * FC_ROWS + row] * w1;
                uint4 pk;
                pk.x = fc_pack(v[0], v[1]); pk.y = fc_pack(v[2], v[3]); pk.z = fc_pack(v[4], v[5]); pk.w = fc_pack(v[6], v[7]);
                reinterpret_cast<uint4*>(dst)[c] = pk;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // copies that were issued but never consumed still write this CTA's shared memory: wait for them
        for (int it = max(0, issued - FC_NST); it < issued; ++it)
            mbar_drain(smem_u32(&sh->full[it % FC_NST]), (it / FC_NST) & 1);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(FC_TMEM_COLS) : "memory");
    }
}

// q [T, QH, 128] bfloat16; cache: one layer's [num_pages, 2, KH, page_size, 128]; entries first_entry .. bring
// cu_q[e+1] - cu_q[e] tokens each and hold kv_len[e] tokens after this step.  n_tiles: the sum over these
// entries of ceil(tokens / (128 / Gc)), Gc = the largest of 16, 8, 4, 2, 1 that divides QH / KH.
extern "C" int rb_fa_prefill_tc(const void* q, const void* cache, long long num_pages, const int* block_table, const int* cu_q,
                                const int* kv_len, void* out, int first_entry, int n_entries, int n_tiles, int QH, int KH, int d,
                                int page_size, int max_pages, int window, float scale, void* stream) {
    if (n_entries <= 0 || n_tiles <= 0) return 0;
    if (QH <= 0 || KH <= 0 || QH % KH) RB_REFUSE("attention: %d query heads over %d kv heads", QH, KH);
    if (d != FC_D) RB_REFUSE("attention (tcgen05): head_dim %d, only 128 is built", d);
    int shift = -1;
    for (int s = 3; s < 16; ++s) if ((1 << s) == page_size) shift = s;
    if (shift < 0) RB_REFUSE("attention (tcgen05): page size %d is not a power of two >= 8", page_size);
    if (((uintptr_t)cache & 15) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15)) RB_REFUSE("attention (tcgen05): operands must be 16-byte aligned");
    FcArgs a{};
    a.q = (const bf16*)q; a.block_table = block_table; a.cu_q = cu_q; a.kv_len = kv_len; a.out = (bf16*)out;
    a.QH = QH; a.KH = KH; a.page_size = page_size; a.page_shift = shift; a.max_pages = max_pages; a.window = window;
    const int G = QH / KH;
    a.Gc = 1;
    for (int c = 16; c >= 1; c >>= 1) if (G % c == 0) { a.Gc = c; break; }
    a.chunks = G / a.Gc; a.first_entry = first_entry; a.n_entries = n_entries;
    a.scale_log2 = scale * 1.4426950408889634f;
    CUtensorMap map;
    const int box_rows = page_size < FC_BN ? page_size : FC_BN;
    if (rb_tensor_map_bf16(cache, num_pages * 2LL * KH * page_size, d, d, box_rows, &map)) return -1;
    constexpr size_t smem = (size_t)FC_NST * FC_STAGE + 4 * FC_QHALF + sizeof(FcShared) + 1024;
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fa_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    if (n_tiles > 65535) RB_REFUSE("attention (tcgen05): %d row tiles in one launch", n_tiles);
    return rb_launch(fa_prefill_tc_kernel, dim3(KH * a.chunks, n_tiles), dim3(FC_THREADS), smem, (cudaStream_t)stream, map, a);
}

// The group of query heads that share a CTA's rows, as rb_fa_prefill_tc chooses it (for the caller's tile count).
extern "C" int rb_fa_prefill_tc_group(int QH, int KH) {
    if (QH <= 0 || KH <= 0 || QH % KH) return 0;
    const int G = QH / KH;
    for (int c = 16; c >= 1; c >>= 1) if (G % c == 0) return c;
    return 1;
}

// The error word of this file's kernels (0 = none); synchronises the device.  With reset != 0 it is cleared.
RB_STATUS_EXPORTS(rb_attn_tc_error, rb_attn_tc_bind_status)

RB_TL_SETTER(rb_attn_tc_step_timeline)
