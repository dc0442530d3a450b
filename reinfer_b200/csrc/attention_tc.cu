// Paged causal flash attention for prompt portions on the fifth-generation tensor cores.
//
// The formulas are the reference's attention (crates/cuda/kernels/dense_kernels.cu:173-231: scores, causal
// mask, softmax in float, weighted sum of the values), tiled as flash attention.  A CTA owns 256 query rows: two
// row tiles A and B of 128 rows each (a row = a token x one of the Gc grouped query heads of one kv head; tile B
// holds the tokens after tile A's), and walks the request's keys in tiles of 64.  Both row tiles use every key
// tile that comes in, so a key tile is fetched once for 256 rows.  For every key tile j and row tile t
//     S_t = Q_t K^T        tcgen05.mma, 128 x 64 x 128, operands in shared memory, S in tensor memory (two buffers
//                          per row tile)
//     P_t = exp2(S_t - m)  128 threads, one row each (tcgen05.ld gives a thread its whole row: the row maximum and
//                          sum need no shuffles), P rounded to bfloat16 into shared memory (two buffers per row tile)
//     O_t += P_t V         tcgen05.mma, 128 x 128 x 64, accumulated in tensor memory over all key tiles: P and O are
//                          scaled to a maximum that follows the true one only when it rose by more than 2^8 (then the
//                          row's thread rescales its lane of O in tensor memory, which is rare), so the rows read O once
// Warp 0 feeds key/value tiles by TMA: ONE request brings the keys (or the values) of a page for this kv head, laid
// out as [8-key group][64-dim half][8 keys][64 dims] whatever the page size is (the 5-D map of runtime.cu).  Warp 1
// allocates tensor memory and issues the scores of tile A, warp 3 those of tile B, warp 2 the weighted sums; warps 4-7 are the rows of tile A,
// warps 8-11 the rows of tile B.  Q [rows][d], K [keys][d] and P [rows][keys] are K-major operands; V [keys][d] is
// used as it lands, as an MN-major operand (instruction descriptor bit 16; in the shared-memory descriptor the
// leading offset steps to the second 64 dims, the stride offset to the next 8 keys) - nothing is transposed.
//
// What runs ahead of what.  A hand-over through an mbarrier that a tcgen05.commit arrives at costs well over a
// thousand clocks from one side's last instruction to the other side's first (measured: the bare skeleton of such
// hand-overs, with no copy, product or arithmetic in it, ran at 1,700 clocks a key tile).  So no such hand-over may
// lie on the rows' path from one key tile to the next.  The scores of tile j+2 are issued as soon as the rows have
// taken the scores of tile j out of tensor memory (they say so at once, before they exponentiate) - not when P(j) is
// done - by an issuer of their own, so the rows find the next scores waiting; the weighted sums have their own issuer
// and nothing but the row's last read of O and the reuse of a P buffer two tiles later waits for them.  (Keeping P in
// tensor memory over the scores it came from - the A operand of the product may lie there - was built and measured:
// it ties the scores' buffer to the product's completion and was no faster.)
// What bounds a key tile now (the kernel's own trace, -DRB_TIMELINE: lane 0 of every warp adds up its waits and its
// work): of the 2,100 cycles a key tile takes, a row warp works 1,970 (the issuers wait for it): 1,270 in P (64
// scale-and-subtract, exponential, sum, 32 conversions, 8 stores a row), of which 760 are the exponentials' (two row
// warps share a scheduler's special-function unit).  With the exponentials taken out the tile still takes 1,900: then
// the rows wait for the scores, whose issuer needs 900 cycles for a tile's 8 products and 2 commits.  Both sides are
// that close, so neither alone buys much.  Built, measured, left out: two threads per row (half the chain each, the
// row's maximum agreed through shared memory: 690 against 623 us at 8,192 tokens); a part of the exponentials as a
// cubic on the FMA pipe (3 of 8: 671 us, 1 of 2: 724 - nine instructions for one); P rounded by integer instructions
// instead of the conversion (no change).
// Registers follow the roles (setmaxnreg): 88 for the control warps, 208 for the rows - what the control warps give up
// (128 threads x 80) must cover what the rows take (256 threads x 40), for the registers come from the CTA's own
// allocation (384 x 168) and a request for more than it holds waits for ever.
//
// Head size 128, page size a power of two >= 8.  Every wait is bounded (2 s); a CTA that gives up raises the
// error word, lets its copies land, frees its tensor memory and leaves; CTAs that start after that leave at once.
#define RB_UNIT 3
#include "sm100.cuh"
#include <stdlib.h>

#define FC_BN 64                              // keys per tile
#define FC_ROWS 128                           // query rows per row tile
#define FC_TILES 2                            // row tiles per CTA
#define FC_D 128
#define FC_THREADS 384                        // a control group (TMA warp, MMA warp, two idle) and two groups of four row warps
#define FC_NST 3
#define FC_KV_BYTES (FC_BN * 256)             // a key (or value) tile: 64 keys x 256 bytes, as 8 groups of [2 halves][8 keys][128 bytes]
#define FC_GROUP 2048                         // bytes from one 8-key group to the next
#define FC_HALF 1024                          // bytes from a group's first 64 dims to its second
#define FC_STAGE (2 * FC_KV_BYTES)            // keys and values
#define FC_QHALF (FC_ROWS * 128)              // 128 rows x 128 bytes: one 64-column half of a Q tile, or one P buffer
#define FC_RESCALE 8.0f                       // O is brought to a new maximum only when it rose by more than this (log2)
#define FC_TMEM_COLS 512                      // S: columns 0..255 (tile A buffers 0, 1; tile B buffers 0, 1); O_A 256..383; O_B 384..511

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
    unsigned long long s_full[FC_TILES][2], s_free[FC_TILES][2], p_full[FC_TILES][2], o_full[FC_TILES][2];
    uint32_t tmem_base;
    int abort_flag;
};

// byte offset of 16-byte chunk c (8 elements) of row `row` in a K-major tile of 128-byte rows with the 128-byte
// swizzle; chunks 8.. lie in the next 64-column half, half_bytes further
__device__ __forceinline__ uint32_t fc_off(int row, int c, int half_bytes) {
    return (uint32_t)((c >> 3) * half_bytes + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}
// the same for a key/value tile as the 5-D map lays it out: [8-key group][half][8 keys][128 bytes]
__device__ __forceinline__ uint32_t fc_kv_off(int key, int c) {
    return (uint32_t)((key >> 3) * FC_GROUP + (c >> 3) * FC_HALF + (key & 7) * 128 + (((c & 7) ^ (key & 7)) << 4));
}
// Sixteen 32-bit columns of this warp's 32 lanes back into tensor memory (the counterpart of tc_ld16).
__device__ __forceinline__ void fc_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void fc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// An issuing warp runs its loop with all lanes (addresses and descriptors are the same in all of them, so they live in
// uniform registers) and one lane issues: the instruction carries the predicate itself, no branch surrounds it.  A loop
// run by one lane alone cost well over a hundred clocks per MMA in moving its operands into uniform registers, and
// the tensor pipe waited for the issuing thread.
__device__ __forceinline__ void fc_mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate, uint32_t lead) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(lead) : "memory");
}
__device__ __forceinline__ void fc_commit_lead(uint32_t bar, uint32_t lead) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar), "r"(lead) : "memory");
}

// 2^x by the special-function unit alone: one instruction (exp2f adds range handling around it, and so does
// ex2.approx without .ftz: a compare and two multiplications per call for results below 2^-126, which are flushed to
// zero here - P is rounded to bfloat16 anyway).  The arguments are <= 0 or -inf, where it is accurate to two units in
// the last place.
__device__ __forceinline__ float fc_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t fc_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// try_wait with a suspend-time hint: the thread sleeps in the barrier unit until the phase completes or the time is
// up, and issues nothing meanwhile.  (A bare poll loop spins: a waiting warp was seen to execute a fifth of all the
// kernel's instructions, taking issue slots from the row warps on its scheduler.)
__device__ __forceinline__ bool fc_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
    return ok != 0;
}
// The bounded wait of sm100.cuh on top of it.
__device__ __forceinline__ bool fc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where) {
    if (fc_try(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < RB_SPIN_LIMIT; ++it) {
        if (fc_try(bar, parity)) return true;
        if ((it & 7u) == 7u) {
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

// With -DRB_TIMELINE lane 0 of every warp adds up, over the key tiles of its CTA, the cycles it spent in each of its
// waits and in its own work, into the buffer of rb_fa_tc_trace(): [warp][8] sums over all CTAs (atomics) and, in word 7
// of a warp's row, the number of (CTA, key tile) pairs counted.  A development aid: where a key tile's time goes.
#ifdef RB_TIMELINE
__device__ unsigned long long* g_fc_trace = nullptr;
extern "C" int rb_fa_tc_trace(unsigned long long* buf) { return (int)cudaMemcpyToSymbol(g_fc_trace, &buf, sizeof(buf)); }
#define FC_T0() const long long fc_t0 = clock64()
#define FC_ADD(slot) do { fc_acc[slot] += clock64() - fc_t0; } while (0)
#define FC_FLUSH(n) do { if (g_fc_trace && lane == 0) { for (int q = 0; q < 7; ++q) atomicAdd(g_fc_trace + warp * 8 + q, (unsigned long long)fc_acc[q]); \
                         atomicAdd(g_fc_trace + warp * 8 + 7, (unsigned long long)(n)); } } while (0)
#else
#define FC_T0() do { } while (0)
#define FC_ADD(slot) do { } while (0)
#define FC_FLUSH(n) do { } while (0)
#endif

__global__ void __launch_bounds__(FC_THREADS, 1)
fa_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_kv, const FcArgs a) {
    RB_TL(11);
    if (*(volatile int*)&g_rb_kernel_error) return;                // an earlier wait gave up: fail fast, the host sees the word
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = smem;                                  // [FC_NST][keys, values]
    unsigned char* sQ = stages + FC_NST * FC_STAGE;                // [row tile][two halves of [128 rows][64 dims]]
    unsigned char* sP = sQ + FC_TILES * 2 * FC_QHALF;              // [row tile][buffer][128 rows][64 keys]
    FcShared* sh = (FcShared*)(sP + FC_TILES * 2 * FC_QHALF);
    const uint32_t stages_u = smem_u32(stages), sQ_u = smem_u32(sQ), sP_u = smem_u32(sP);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sh->abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < FC_NST; ++s) {
            mbar_init(smem_u32(&sh->full[s]), 1);
            mbar_init(smem_u32(&sh->empty[s]), 3);                 // the issuers' commits: scores of either row tile done (keys), P V done (values)
        }
        for (int t = 0; t < FC_TILES; ++t)
            for (int b = 0; b < 2; ++b) {
                mbar_init(smem_u32(&sh->s_full[t][b]), 1);
                mbar_init(smem_u32(&sh->s_free[t][b]), 4);         // one arrival per row warp: the scores are in registers
                mbar_init(smem_u32(&sh->p_full[t][b]), 4);         // one arrival per row warp: P is written
                mbar_init(smem_u32(&sh->o_full[t][b]), 1);
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
    // -inf whatever they are, P is written whole before it is read.
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    pdl_trigger();
    pdl_wait();

    // which rows: heavy CTAs (late in a request: more keys) first
    const int tpt = FC_ROWS / a.Gc;                                // tokens per row tile
    const int tpc = FC_TILES * tpt;                                // tokens per CTA
    int tile = (int)gridDim.y - 1 - (int)blockIdx.y, e = a.first_entry, q_len = 0;   // CTAs start in order of x, then y
    for (; e < a.first_entry + a.n_entries; ++e) {
        q_len = a.cu_q[e + 1] - a.cu_q[e];
        const int nt = (q_len + tpc - 1) / tpc;
        if (tile < nt) break;
        tile -= nt;
    }
    const bool none = e >= a.first_entry + a.n_entries;            // uniform: a CTA beyond the last entry
    int n_tiles = 0, q0 = 0, n_tok = 0, kv_end = 0, start_pos = 0, tok_base = 0, t_begin = 0, head0 = 0, kh = 0;
    const int* bt = a.block_table;
    if (!none) {
        q0 = tile * tpc;
        n_tok = min(tpc, q_len - q0);                              // tokens of this CTA: the first tpt in tile A, the rest in B
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
        // Q rows (row r of the CTA = token r / Gc, grouped head r % Gc; rows 128.. are tile B) into the swizzled K-major layout
        for (int i = threadIdx.x; i < n_tok * a.Gc * (FC_D / 8); i += FC_THREADS) {
            const int row = i / (FC_D / 8), c = i % (FC_D / 8);
            const uint4 v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(tok_base + row / a.Gc) * a.QH + head0 + row % a.Gc) * FC_D + c * 8);
            *reinterpret_cast<uint4*>(sQ + (row >> 7) * 2 * FC_QHALF + fc_off(row & 127, c, FC_QHALF)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    int issued = 0;                                                // producer: tiles whose copies were issued
    [[maybe_unused]] long long fc_acc[7] = {0, 0, 0, 0, 0, 0, 0};
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");           // the control group gives registers up ...
    if (warp == 0) {
        // ---- producer: runs ahead by up to FC_NST tiles; block-table entries 32 at a time -------------------
        const int box_keys = min(a.page_size, FC_BN);              // keys that one request brings
        const int subs = FC_BN / box_keys;
        int cached_first = 0, cached = -1;
        bool have = false;
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % FC_NST;
            const int k0 = (t_begin + it) * FC_BN;
            const int pi0 = k0 >> a.page_shift;
            const int need_last = (k0 + (subs - 1) * box_keys) >> a.page_shift;
            if (!have || need_last >= cached_first + 32) {
                cached_first = pi0;
                cached = (pi0 + lane < a.max_pages) ? bt[pi0 + lane] : -1;
                have = true;
            }
            int pages[8];
            int n_valid = 0;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int key = k0 + u * box_keys;
                const int pg = __shfl_sync(0xffffffffu, cached, ((key >> a.page_shift) - cached_first) & 31);
                pages[u] = (u < subs && key < kv_end) ? pg : -1;
                n_valid += pages[u] >= 0;
            }
            // every lane waits, lane 0's requests take effect (a lane alone inside a branch pays for each of them)
            const uint32_t lead = lane == 0 ? 1u : 0u;
            { FC_T0(); if (it >= FC_NST && !fc_wait(smem_u32(&sh->empty[s]), ((it / FC_NST) & 1) ^ 1, abort_flag, 11)) break; FC_ADD(0); }
            FC_T0();
            const uint32_t full = smem_u32(&sh->full[s]);
            mbar_expect_tx_lead(full, (uint32_t)(n_valid * 2 * box_keys * 256), lead);
            const uint32_t dst0 = stages_u + s * FC_STAGE;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (pages[u] >= 0) {
                    const int key = k0 + u * box_keys;
                    const int grp = (key & (a.page_size - 1)) >> 3;          // first 8-key group inside the page
                    const int j = pages[u] * 2 * a.KH + kh;                 // (page, keys, head); values: + KH
                    const uint32_t dst = dst0 + (uint32_t)(u * (box_keys >> 3) * FC_GROUP);
                    tma_load_5d_lead(dst, &map_kv, 0, 0, 0, grp, j, full, lead);
                    tma_load_5d_lead(dst + FC_KV_BYTES, &map_kv, 0, 0, 0, grp, j + a.KH, full, lead);
                }
            }
            issued = it + 1;
            FC_ADD(1);
        }
        FC_FLUSH(n_tiles);
    } else if (warp == 1 || warp == 3) {
        // ---- issuers of the scores, one warp per row tile: every lane runs the loop, lane 0's instructions take effect
        // S_t(i) = Q_t K(i)^T into score buffer i & 1 of row tile t, as soon as the keys have landed and the rows
        // have taken the scores of two tiles ago out of that buffer: the scores run ahead of the rows, whatever the
        // products P V are doing.  d = 128 is two 64-column halves of four 16-wide steps each; the keys' 8-row groups
        // lie 2,048 bytes apart, their second half 1,024 bytes on.  (One warp for both tiles had 16 products and 3
        // commits to issue per key tile, about 65 cycles each: more than the products take to run.)
        const uint32_t lead = lane == 0 ? 1u : 0u;
        const int t = warp == 1 ? 0 : 1;
        constexpr uint32_t idesc_s = make_idesc(FC_BN);
        const uint64_t dq0 = make_smem_desc(sQ_u + (t * 2) * FC_QHALF), dq1 = make_smem_desc(sQ_u + (t * 2 + 1) * FC_QHALF);
        for (int i = 0; i < n_tiles; ++i) {
            const int s = i % FC_NST;
            { FC_T0(); if (!fc_wait(smem_u32(&sh->full[s]), (i / FC_NST) & 1, abort_flag, 12)) break; FC_ADD(0); }
            { FC_T0(); if (i >= 2 && !fc_wait(smem_u32(&sh->s_free[t][i & 1]), (uint32_t)(((i >> 1) & 1) ^ 1), abort_flag, 20)) break; FC_ADD(1); }
            FC_T0();
            tc_fence_after();
            const uint32_t sK = stages_u + s * FC_STAGE;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint64_t dq = h ? dq1 : dq0;
                const uint64_t dk = make_smem_desc_lbo_sbo(sK + h * FC_HALF, 16, FC_GROUP);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    fc_mma_ss(tmem + (uint32_t)((t * 2 + (i & 1)) * FC_BN), dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s,
                              (h | k) != 0, lead);
            }
            fc_commit_lead(smem_u32(&sh->s_full[t][i & 1]), lead);
            fc_commit_lead(smem_u32(&sh->empty[s]), lead);         // the keys of this stage are read once these MMAs are done ...
            FC_ADD(2);
        }
        FC_FLUSH(n_tiles);
    } else if (warp == 2) {
        // ---- issuer of the weighted sums: O_t += P_t V once the rows of tile t have written P -----------------------
        const uint32_t lead = lane == 0 ? 1u : 0u;
        constexpr uint32_t idesc_mn = make_idesc(FC_D) | (1u << 16);           // B is MN-major
        bool ok = true;
        for (int it = 0; it < n_tiles && ok; ++it) {
            const uint32_t sVs = stages_u + (it % FC_NST) * FC_STAGE + FC_KV_BYTES;
            // V [keys][d] as it lies in the stage is an MN-major operand: a key's 64 dims (128 bytes) contiguous, keys
            // 128 bytes apart, groups of 8 keys 2,048 bytes apart (SBO), the second 64 dims 1,024 bytes on (LBO); an
            // MMA takes 16 keys = two groups.  (The values landed with the keys, which the scores waited for.)
            const uint64_t dv = make_smem_desc_lbo_sbo(sVs, FC_HALF, FC_GROUP);
#pragma unroll
            for (int t = 0; t < FC_TILES; ++t) {
                { FC_T0(); if (!fc_wait(smem_u32(&sh->p_full[t][it & 1]), (it >> 1) & 1, abort_flag, 13)) { ok = false; break; } FC_ADD(0); }
                FC_T0();
                tc_fence_after();
                const uint64_t dp = make_smem_desc(sP_u + (t * 2 + (it & 1)) * FC_QHALF);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    fc_mma_ss(tmem + (uint32_t)(FC_TILES * 2 * FC_BN + t * FC_D), dp + (uint64_t)(k * 2),
                              dv + (uint64_t)(k * ((2 * FC_GROUP) >> 4)), idesc_mn, (it > 0) || k != 0, lead);
                fc_commit_lead(smem_u32(&sh->o_full[t][it & 1]), lead);
                FC_ADD(2);
            }
            if (!ok) break;
            fc_commit_lead(smem_u32(&sh->empty[it % FC_NST]), lead);   // ... and its values once these are
        }
        FC_FLUSH(n_tiles);
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");      // ... and the rows take them
        // ---- softmax rows: thread = row = tensor-memory lane; group t owns row tile t through all key tiles ----------
        const int t = (warp - 4) >> 2;
        const int quad = warp & 3;                                 // the lanes this warp may read: 32 * (warp % 4) ..
        const int row = quad * 32 + lane;                          // row of the tile
        const int ti = t * tpt + row / a.Gc;                       // token of the CTA
        const bool live = !none && ti < n_tok;
        const int pos = live ? start_pos + q0 + ti : -1;
        const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
        // m: the maximum that P and O are scaled to (it follows the true maximum only in steps larger than
        // FC_RESCALE, so that O can stay in tensor memory and be accumulated by the MMA itself); l: the sum in that scale
        float m = -INFINITY, l = 0.0f;
        const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
        const uint32_t o_col = (uint32_t)(FC_TILES * 2 * FC_BN + t * FC_D);
        bool ok = true;
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % FC_NST, b = it & 1;
            const uint32_t par = (uint32_t)((it >> 1) & 1);
            const int k0 = (t_begin + it) * FC_BN;
            if (t == 0 && k0 + FC_BN > kv_end) {
                // the request's last tile: slots of its last page beyond its length hold foreign data - the values
                // there are zeroed before the tensor core multiplies them (by P = 0, but 0 x NaN is NaN).  The rows of
                // tile A do it; the product of tile B is issued behind A's, so it sees the zeros too.
                if (!fc_wait(smem_u32(&sh->full[s]), (it / FC_NST) & 1, abort_flag, 14)) { ok = false; break; }
                unsigned char* sV = stages + s * FC_STAGE + FC_KV_BYTES;
                for (int i = row; i < FC_BN * 16; i += FC_ROWS) {
                    const int r = i / 16, c = i % 16;
                    if (k0 + r >= kv_end) *reinterpret_cast<uint4*>(sV + fc_kv_off(r, c)) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeros, before the tensor core reads the values
            }
            // S: this row's 64 scores in one go (one wait for tensor memory); maxima and sums in four independent chains
            { FC_T0(); if (!fc_wait(smem_u32(&sh->s_full[t][b]), par, abort_flag, 15)) { ok = false; break; } FC_ADD(0); }
#ifdef RB_TIMELINE
            const long long fc_tile0 = clock64();
#endif
            tc_fence_after();
            const bool edge = k0 + FC_BN - 1 > pos || k0 < lo;     // the tile crosses this row's causal edge or window
            uint32_t sr[FC_BN];
            const uint32_t s_col = (uint32_t)((t * 2 + b) * FC_BN);
#pragma unroll
            for (int c = 0; c < FC_BN / 16; ++c) tc_ld16(lane_base + s_col + (uint32_t)(c * 16), sr + c * 16);
            tc_ld_wait();
#ifdef RB_TIMELINE
            fc_acc[1] += clock64() - fc_tile0;
#endif
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->s_free[t][b]));          // this buffer may take the scores of tile it + 2
            if (edge) {
#pragma unroll
                for (int j = 0; j < FC_BN; ++j) {
                    const int key = k0 + j;
                    if (key < lo || key > pos) sr[j] = 0xff800000u;            // -inf
                }
            }
            // this P buffer was read by the product of two key tiles ago, which must be done before it is written again
            if (it >= 2) {
                FC_T0();
                if (!fc_wait(smem_u32(&sh->o_full[t][b]), par ^ 1, abort_flag, 16)) { ok = false; break; }
                FC_ADD(2);
            }
            unsigned char* sPb = sP + (t * 2 + b) * FC_QHALF;
            // P = 2^(S * scale - base), rounded to bfloat16, into the buffer; and its row sum
            auto emit = [&](float base) -> float {
                float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int c = 0; c < FC_BN / 8; ++c) {
                    float p[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) { p[j] = fc_ex2(fmaf(__uint_as_float(sr[c * 8 + j]), a.scale_log2, -base)); sum4[j & 3] += p[j]; }
                    uint4 pk;
                    pk.x = fc_pack(p[0], p[1]); pk.y = fc_pack(p[2], p[3]); pk.z = fc_pack(p[4], p[5]); pk.w = fc_pack(p[6], p[7]);
                    *reinterpret_cast<uint4*>(sPb + fc_off(row, c, 0)) = pk;
                }
                return (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            };
            // The scale m follows the true maximum only when that rose by more than FC_RESCALE (P then stays below
            // 2^FC_RESCALE, which bfloat16 and the float accumulators hold as well as values below 1).  So in nearly every
            // tile the old scale stays, and the exponentials need not wait for this tile's maximum: both are computed side
            // by side, and only a warp in which some row's scale has to move (always in a row's first tile) does its
            // exponentials again.
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#ifdef RB_TIMELINE
            const long long fc_c3 = clock64();
#endif
#pragma unroll
            for (int j = 0; j < FC_BN; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sr[j]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;   // the scale is positive
            float sum = 0.0f;
#ifdef RB_TIMELINE
            const long long fc_c5 = clock64();
            fc_acc[3] += fc_c5 - fc_c3;
#endif
            if (it > 0) sum = emit(m == -INFINITY ? 0.0f : m);
#ifdef RB_TIMELINE
            fc_acc[5] += clock64() - fc_c5;
#endif
            const bool moves = (m == -INFINITY) ? (mx != -INFINITY) : (mx > m + FC_RESCALE);
            if (it == 0 || __any_sync(0xffffffffu, moves)) {
                float alpha = 1.0f;
                if (m == -INFINITY) m = mx;
                else if (moves) { alpha = fc_ex2(m - mx); m = mx; }
                if (it >= 1 && __any_sync(0xffffffffu, alpha != 1.0f)) {
                    // rare: O = O * alpha in tensor memory, every lane of the warp with its own factor (1 for most); the
                    // product of the key tile before (the last one that can have been issued) must have landed in O first
                    if (!fc_wait(smem_u32(&sh->o_full[t][b ^ 1]), (uint32_t)(((it - 1) >> 1) & 1), abort_flag, 18)) { ok = false; break; }
                    tc_fence_after();
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
                l *= alpha;
                sum = emit(m == -INFINITY ? 0.0f : m);
            }
            l += sum;
#ifdef RB_TIMELINE
            const long long fc_c6 = clock64();
#endif
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // P (and zeroed value rows) before the tensor core reads them
            tc_fence_before();                                     // O (if touched) is written: the product may go on
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->p_full[t][b]));
#ifdef RB_TIMELINE
            fc_acc[6] += clock64() - fc_c6;
            fc_acc[4] += clock64() - fc_tile0;
#endif
        }
        FC_FLUSH(n_tiles);
        // the row of O, once the tile's last products are done (the last one on each of the two barriers)
        if (ok && n_tiles > 0) {
            const int last = n_tiles - 1;
            ok = fc_wait(smem_u32(&sh->o_full[t][last & 1]), (uint32_t)((last >> 1) & 1), abort_flag, 17);
            if (ok && last >= 1) ok = fc_wait(smem_u32(&sh->o_full[t][(last - 1) & 1]), (uint32_t)(((last - 1) >> 1) & 1), abort_flag, 19);
        }
        if (ok && n_tiles > 0 && !*abort_flag) {
            // (the loads from tensor memory are the whole warp's: every lane takes part, only live rows store)
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            bf16* dst = a.out + ((size_t)(tok_base + (live ? ti : 0)) * a.QH + head0 + row % a.Gc) * FC_D;
#pragma unroll
            for (int c = 0; c < FC_D / 32; ++c) {
                uint32_t ov[32];
                tc_ld16(lane_base + o_col + (uint32_t)(c * 32), ov);
                tc_ld16(lane_base + o_col + (uint32_t)(c * 32 + 16), ov + 16);
                tc_ld_wait();
                if (!live) continue;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint4 pk;
                    pk.x = fc_pack(__uint_as_float(ov[q4 * 8 + 0]) * inv, __uint_as_float(ov[q4 * 8 + 1]) * inv);
                    pk.y = fc_pack(__uint_as_float(ov[q4 * 8 + 2]) * inv, __uint_as_float(ov[q4 * 8 + 3]) * inv);
                    pk.z = fc_pack(__uint_as_float(ov[q4 * 8 + 4]) * inv, __uint_as_float(ov[q4 * 8 + 5]) * inv);
                    pk.w = fc_pack(__uint_as_float(ov[q4 * 8 + 6]) * inv, __uint_as_float(ov[q4 * 8 + 7]) * inv);
                    reinterpret_cast<uint4*>(dst)[c * 4 + q4] = pk;
                }
            }
            tc_fence_before();
        } else if (ok && live && n_tiles == 0) {
            // a row without a single key (cannot happen for a causal row, which sees itself): zeros
            bf16* dst = a.out + ((size_t)(tok_base + ti) * a.QH + head0 + row % a.Gc) * FC_D;
            for (int c = 0; c < FC_D / 8; ++c) reinterpret_cast<uint4*>(dst)[c] = make_uint4(0, 0, 0, 0);
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
// entries of ceil(tokens / (256 / Gc)), Gc = the largest of 16, 8, 4, 2, 1 that divides QH / KH.
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
    if (rb_tensor_map_kv_pages(cache, num_pages, KH, page_size, &map)) return -1;
    constexpr size_t smem = (size_t)FC_NST * FC_STAGE + FC_TILES * 4 * FC_QHALF + sizeof(FcShared) + 1024;
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fa_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    if (n_tiles > 65535) RB_REFUSE("attention (tcgen05): %d row tiles in one launch", n_tiles);
    return rb_launch(fa_prefill_tc_kernel, dim3(KH * a.chunks, n_tiles), dim3(FC_THREADS), smem, (cudaStream_t)stream, map, a);
}

// The group of query heads that share a CTA's rows, as rb_fa_prefill_tc chooses it, and the rows of a CTA (for the
// caller's count of CTAs: a CTA takes rows / group tokens).
extern "C" int rb_fa_prefill_tc_group(int QH, int KH) {
    if (QH <= 0 || KH <= 0 || QH % KH) return 0;
    const int G = QH / KH;
    for (int c = 16; c >= 1; c >>= 1) if (G % c == 0) return c;
    return 1;
}
extern "C" int rb_fa_prefill_tc_rows() { return FC_TILES * FC_ROWS; }

// The error word of this file's kernels (0 = none); synchronises the device.  With reset != 0 it is cleared.
RB_STATUS_EXPORTS(rb_attn_tc_error, rb_attn_tc_bind_status)

RB_TL_SETTER(rb_attn_tc_step_timeline)
