// Flash attention over the paged cache for the bfloat16 path: one kernel body in two
// shapes.  Keys and values are brought page by page into shared memory with cp.async
// (16-byte copies, zero fill for what lies outside the request), scores and the
// probability-weighted values go through mma.sync m16n8k16 (bf16 in, float out), the
// softmax is online and in float (exp2 of scores pre-multiplied by scale*log2 e).
//
//  * PREFILL (entries that bring more than one token): a CTA owns 64 rows = 64/Gc tokens
//    x Gc query heads of one kv head (grouped heads share every K/V tile they read), each
//    warp 16 rows, all warps walk the same 64-key tiles from the request's pages -
//    including the pages that EARLIER steps wrote, which the reference's prefill kernel
//    cannot read (it attends to the fresh K/V of one call only,
//    bin/reinfer/src/sched_loop.rs:188-195; crates/cuda/src/fmha.rs:711-729).
//  * DECODE (one token): the Gc query heads of a kv head are the rows of ONE 16-row tile;
//    the request's keys are split across CTAs (grid.z) and inside a CTA across the four
//    warps (16 keys of each 64-key tile per warp); warps merge in shared memory, CTAs
//    through a scratch buffer and a small merge kernel, in fixed order.  (The reference
//    runs one CTA per query head over the whole context and re-reads K/V per head,
//    crates/cuda/kernels/decode_flash_kernels.cu:167-369.)
//
// Head sizes: the template is instantiated for 32, 64, 128 and 256; a head size that is a
// multiple of 8 below the next instance is zero-padded in shared memory.
#include "common.cuh"

#define FA_WARPS 4
#define FA_THREADS (FA_WARPS * 32)
#define FA_BN 64                       // keys per tile
#define FA_BM 64                       // rows per prefill CTA

struct FaArgs {
    const bf16* q;                     // [T, QH, d]
    const bf16* cache;                 // one layer: [page][2][KH][page_size][d]
    const int* block_table;            // [entries, max_pages]
    const int* cu_q;                   // [entries + 1]
    const int* kv_len;                 // [entries] length of the request after this step
    bf16* out;                         // [T, QH, d]
    float* part_o;                     // decode: [tokens, QH, splits, d] normalised partial outputs
    float* part_lse;                   // decode: [tokens, QH, splits] log2 of the partial softmax sums
    int QH, KH, d, page_size, max_pages, window;
    int page_shift;                    // log2(page_size), or -1 if it is no power of two
    int Gc, chunks;                    // query heads per row tile (divides QH/KH, <= 16), tiles per kv head
    int first_entry, n_entries;        // entries this launch covers: [first_entry, first_entry + n_entries)
    int n_splits;
    float scale_log2;
};

// ---------------------------------------------------------------- small PTX wrappers
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int D> struct FaSmem {
    static constexpr int STRIDE = D * 2 + 16;                 // bytes per row: 16 bytes of padding keep ldmatrix conflict-free
    static constexpr int TILE = FA_BN * STRIDE;               // one K or V tile
    static constexpr int STAGE = 2 * TILE;
};

// Copy keys [k0, k0+64) of kv head `kh` (K and V) of the request whose block-table row is `bt`
// into one stage.  Rows at or beyond `kv_end`, rows in pages that were given back (id < 0) and
// the padding dims d..D are zero-filled, so nothing that is not the request's own data is read.
// A thread always copies the same 16-byte column of rows r0, r0 + RPI, ...; with a page size that
// is a power of two (page_shift >= 0) the page of a row costs a shift and a mask.
template <int D>
__device__ __forceinline__ void fa_load_tile(unsigned char* stage, const FaArgs& a, const int* bt, int kh, int k0, int kv_end) {
    constexpr int CPR = D / 8;                                // 16-byte chunks per row
    constexpr int RPI = FA_THREADS / CPR;                     // rows per pass over the tile
    static_assert(FA_THREADS % CPR == 0 && FA_BN % RPI == 0, "tile shape");
    const int c = threadIdx.x % CPR, r0 = threadIdx.x / CPR;
    const bool col_ok = c * 8 < a.d;
    const size_t head_stride = (size_t)a.page_size * a.d;
    const size_t page_stride = 2 * (size_t)a.KH * head_stride;
    const bf16* base = a.cache + (size_t)kh * head_stride + c * 8;
    const size_t v_off = (size_t)a.KH * head_stride;
    unsigned char* dst0 = stage + r0 * FaSmem<D>::STRIDE + c * 16;
#pragma unroll
    for (int i = 0; i < FA_BN / RPI; ++i) {
        const int key = k0 + r0 + i * RPI;
        const bf16* src = a.cache;
        int bytes = 0;
        if (col_ok && key < kv_end) {
            int pi, off;
            if (a.page_shift >= 0) { pi = key >> a.page_shift; off = key & (a.page_size - 1); }
            else { pi = key / a.page_size; off = key - pi * a.page_size; }
            const int page = pi < a.max_pages ? bt[pi] : -1;
            if (page >= 0) { src = base + (size_t)page * page_stride + (size_t)off * a.d; bytes = 16; }
        }
        unsigned char* dst = dst0 + i * RPI * FaSmem<D>::STRIDE;
        cp_async16(dst, src, bytes);
        cp_async16(dst + FaSmem<D>::TILE, bytes ? src + v_off : src, bytes);
    }
}

// One 64-key tile for one warp: scores of its 16 rows against NT n-tiles of 8 keys starting at
// key `koff` of the tile, online softmax, and the P V update.
//   pos0/pos1, lo0/lo1: last and first visible key of row lane/4 and row lane/4 + 8.
template <int D, int NT>
__device__ __forceinline__ void fa_tile(const unsigned char* sQ, const unsigned char* sK, const unsigned char* sV,
                                        int koff, int k0_abs, int pos0, int pos1, int lo0, int lo1, float scale_log2,
                                        float (&o)[D / 8][4], float (&m)[2], float (&l)[2]) {
    constexpr int STRIDE = FaSmem<D>::STRIDE;
    const int lane = threadIdx.x & 31;
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t qa[4];
        ldsm_x4(qa, sQ + ((lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + (ks * 16 + 8 * (lane >> 4)) * 2);
#pragma unroll
        for (int jp = 0; jp < NT / 2; ++jp) {
            uint32_t kb[4];
            ldsm_x4(kb, sK + (koff + jp * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + (ks * 16 + 8 * ((lane >> 3) & 1)) * 2);
            mma_bf16(s[2 * jp], qa, kb[0], kb[1]);
            mma_bf16(s[2 * jp + 1], qa, kb[2], kb[3]);
        }
    }
    // scale, mask, row maxima
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int key = k0_abs + koff + j * 8 + 2 * (lane & 3);
        s[j][0] = (key >= lo0 && key <= pos0) ? s[j][0] * scale_log2 : -INFINITY;
        s[j][1] = (key + 1 >= lo0 && key + 1 <= pos0) ? s[j][1] * scale_log2 : -INFINITY;
        s[j][2] = (key >= lo1 && key <= pos1) ? s[j][2] * scale_log2 : -INFINITY;
        s[j][3] = (key + 1 >= lo1 && key + 1 <= pos1) ? s[j][3] * scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
        mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const float base0 = mn0 == -INFINITY ? 0.0f : mn0, base1 = mn1 == -INFINITY ? 0.0f : mn1;   // a row that saw no key yet
    const float c0 = exp2f(m[0] - base0), c1 = exp2f(m[1] - base1);
    m[0] = mn0; m[1] = mn1;
    float sum0 = 0.0f, sum1 = 0.0f;
    uint32_t p[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const float e0 = exp2f(s[j][0] - base0), e1 = exp2f(s[j][1] - base0);
        const float e2 = exp2f(s[j][2] - base1), e3 = exp2f(s[j][3] - base1);
        sum0 += e0 + e1; sum1 += e2 + e3;
        p[j][0] = pack_bf16(e0, e1);
        p[j][1] = pack_bf16(e2, e3);
    }
    l[0] = l[0] * c0 + sum0;                                   // per-thread partial sums; joined at the end
    l[1] = l[1] * c1 + sum1;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        const uint32_t pa[4] = {p[2 * kk][0], p[2 * kk][1], p[2 * kk + 1][0], p[2 * kk + 1][1]};
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            uint32_t vb[4];
            ldsm_x4_trans(vb, sV + (koff + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + (dp * 16 + 8 * (lane >> 4)) * 2);
            mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
            mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
        }
    }
}

// Load `rows` rows of Q (row r = token q_tok0 + r / Gc, head head0 + r % Gc) into shared memory, zero beyond.
template <int D>
__device__ __forceinline__ void fa_load_q(unsigned char* sQ, const FaArgs& a, int tok_base, int n_tok, int head0, int n_rows_smem) {
    constexpr int CPR = D / 8;
    for (int i = threadIdx.x; i < n_rows_smem * CPR; i += FA_THREADS) {
        const int row = i / CPR, c = i % CPR;
        const int ti = row / a.Gc, g = row % a.Gc;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (ti < n_tok && c * 8 < a.d)
            v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(tok_base + ti) * a.QH + head0 + g) * a.d + c * 8);
        *reinterpret_cast<uint4*>(sQ + row * FaSmem<D>::STRIDE + c * 16) = v;
    }
}

// ------------------------------------------------------------------------ prefill
template <int D>
__global__ void __launch_bounds__(FA_THREADS)
fa_prefill_kernel(const FaArgs a) {
    constexpr int NST = 2;
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_trigger(); pdl_wait();
    unsigned char* sQ = smem;
    unsigned char* stages = smem + FA_BM * FaSmem<D>::STRIDE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tpt = FA_BM / a.Gc;                              // tokens per CTA
    // which (entry, first token) is this CTA's?  entries are few: a linear walk
    int tile = blockIdx.x, e = a.first_entry, q_len = 0;
    for (; e < a.first_entry + a.n_entries; ++e) {
        q_len = a.cu_q[e + 1] - a.cu_q[e];
        const int nt = (q_len + tpt - 1) / tpt;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e >= a.first_entry + a.n_entries) return;
    const int q0 = tile * tpt;
    const int n_tok = min(tpt, q_len - q0);
    const int kh = blockIdx.y / a.chunks, chunk = blockIdx.y % a.chunks;
    const int head0 = kh * (a.QH / a.KH) + chunk * a.Gc;
    const int kv_end = a.kv_len[e];
    const int start_pos = kv_end - q_len;
    const int* bt = a.block_table + (size_t)e * a.max_pages;

    fa_load_q<D>(sQ, a, a.cu_q[e] + q0, n_tok, head0, FA_BM);
    const int pos_min = start_pos + q0, pos_max = start_pos + q0 + n_tok - 1;
    const int lo_min = a.window > 0 ? max(0, pos_min - a.window + 1) : 0;
    const int t_begin = lo_min / FA_BN, t_end = pos_max / FA_BN + 1;

    // this thread's two rows
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int ti0 = r0 / a.Gc, ti1 = r1 / a.Gc;
    const int pos0 = ti0 < n_tok ? start_pos + q0 + ti0 : -1, pos1 = ti1 < n_tok ? start_pos + q0 + ti1 : -1;
    const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0, lo1 = a.window > 0 ? max(0, pos1 - a.window + 1) : 0;
    // keys beyond the last row of this WARP are masked for all its rows: the warp may stop early
    const int warp_last_tok = min(n_tok - 1, (warp * 16 + 15) / a.Gc);
    const int warp_t_end = (warp * 16) / a.Gc < n_tok ? (start_pos + q0 + warp_last_tok) / FA_BN + 1 : 0;

    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    fa_load_tile<D>(stages, a, bt, kh, t_begin * FA_BN, kv_end);
    cp_async_commit();
    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) % NST;
        cp_async_wait<0>();
        __syncthreads();                                       // tile t has landed; tile t-1 is no longer read
        if (t + 1 < t_end) fa_load_tile<D>(stages + ((buf + 1) % NST) * FaSmem<D>::STAGE, a, bt, kh, (t + 1) * FA_BN, kv_end);
        cp_async_commit();
        if (t < warp_t_end) {
            const unsigned char* sK = stages + buf * FaSmem<D>::STAGE;
            fa_tile<D, FA_BN / 8>(sQ + warp * 16 * FaSmem<D>::STRIDE, sK, sK + FaSmem<D>::TILE, 0, t * FA_BN,
                                  pos0, pos1, lo0, lo1, a.scale_log2, o, m, l);
        }
    }
    cp_async_wait<0>();
    // join the four threads of a row, normalise, store
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    const float inv0 = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv1 = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
    const int tok_base = a.cu_q[e] + q0;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        const int dim = j * 8 + 2 * (lane & 3);
        if (dim >= a.d) continue;
        if (ti0 < n_tok)
            *reinterpret_cast<uint32_t*>(a.out + ((size_t)(tok_base + ti0) * a.QH + head0 + r0 % a.Gc) * a.d + dim) = pack_bf16(o[j][0] * inv0, o[j][1] * inv0);
        if (ti1 < n_tok)
            *reinterpret_cast<uint32_t*>(a.out + ((size_t)(tok_base + ti1) * a.QH + head0 + r1 % a.Gc) * a.d + dim) = pack_bf16(o[j][2] * inv1, o[j][3] * inv1);
    }
}

// ------------------------------------------------------------------------- decode
template <int D, int NST>
__global__ void __launch_bounds__(FA_THREADS)
fa_decode_kernel(const FaArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_trigger(); pdl_wait();
    unsigned char* sQ = smem;                                  // 16 rows
    unsigned char* stages = smem + 16 * FaSmem<D>::STRIDE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = a.first_entry + blockIdx.x;                  // a decode entry brings one token: token index = cu_q[e]
    const int kh = blockIdx.y / a.chunks, chunk = blockIdx.y % a.chunks;
    const int head0 = kh * (a.QH / a.KH) + chunk * a.Gc;
    const int split = blockIdx.z;
    const int kv_end = a.kv_len[e];
    const int pos = kv_end - 1;
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int tok = a.cu_q[e];
    const int* bt = a.block_table + (size_t)e * a.max_pages;
    const int t_lo = lo / FA_BN, t_hi = pos / FA_BN + 1;
    const int per = (t_hi - t_lo + a.n_splits - 1) / a.n_splits;
    const int t_begin = t_lo + split * per, t_end = min(t_hi, t_begin + per);

    fa_load_q<D>(sQ, a, tok, 1, head0, 16);
    const int row0 = lane >> 2;                                // rows >= Gc are padding
    const int pos0 = row0 < a.Gc ? pos : -1, pos1 = row0 + 8 < a.Gc ? pos : -1;
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

#pragma unroll
    for (int i = 0; i < NST - 1; ++i) {
        if (t_begin + i < t_end) fa_load_tile<D>(stages + i * FaSmem<D>::STAGE, a, bt, kh, (t_begin + i) * FA_BN, kv_end);
        cp_async_commit();
    }
    for (int t = t_begin; t < t_end; ++t) {
        const int it = t - t_begin;
        cp_async_wait<NST - 2>();
        __syncthreads();
        if (t + NST - 1 < t_end)
            fa_load_tile<D>(stages + ((it + NST - 1) % NST) * FaSmem<D>::STAGE, a, bt, kh, (t + NST - 1) * FA_BN, kv_end);
        cp_async_commit();
        const unsigned char* sK = stages + (it % NST) * FaSmem<D>::STAGE;
        fa_tile<D, 2>(sQ, sK, sK + FaSmem<D>::TILE, warp * 16, t * FA_BN, pos0, pos1, lo, lo, a.scale_log2, o, m, l);
    }
    cp_async_wait<0>();
    __syncthreads();                                           // the stages are free: reuse them for the merge
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    float* sO = reinterpret_cast<float*>(stages);              // [warp][16][D]
    float* sM = sO + FA_WARPS * 16 * D;                        // [warp][16]
    float* sL = sM + FA_WARPS * 16;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        const int dim = j * 8 + 2 * (lane & 3);
        sO[(warp * 16 + row0) * D + dim] = o[j][0]; sO[(warp * 16 + row0) * D + dim + 1] = o[j][1];
        sO[(warp * 16 + row0 + 8) * D + dim] = o[j][2]; sO[(warp * 16 + row0 + 8) * D + dim + 1] = o[j][3];
    }
    if ((lane & 3) == 0) {
        sM[warp * 16 + row0] = m[0]; sM[warp * 16 + row0 + 8] = m[1];
        sL[warp * 16 + row0] = l[0]; sL[warp * 16 + row0 + 8] = l[1];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.Gc * a.d; i += FA_THREADS) {
        const int row = i / a.d, dim = i % a.d;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < FA_WARPS; ++w) M = fmaxf(M, sM[w * 16 + row]);
        float L = 0.0f, O = 0.0f;
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < FA_WARPS; ++w) {
                const float f = exp2f(sM[w * 16 + row] - M);   // a warp that saw no key: exp2(-inf) = 0
                L += sL[w * 16 + row] * f;
                O += sO[(w * 16 + row) * D + dim] * f;
            }
        }
        const float val = L > 0.0f ? O / L : 0.0f;
        const int head = head0 + row;
        if (a.n_splits == 1) {
            a.out[((size_t)tok * a.QH + head) * a.d + dim] = __float2bfloat16_rn(val);
        } else {
            const size_t pi = ((size_t)(tok - a.cu_q[a.first_entry]) * a.QH + head) * a.n_splits + split;
            a.part_o[pi * a.d + dim] = val;
            if (dim == 0) a.part_lse[pi] = L > 0.0f ? M + log2f(L) : -INFINITY;
        }
    }
}

// out[t, h, :] = sum_s w_s o_s / sum_s w_s,  w_s = 2^(lse_s - max lse), splits in ascending order
__global__ void fa_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, bf16* __restrict__ out,
                                int first_tok, int QH, int d, int n_splits) {
    pdl_trigger(); pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t base = ((size_t)t * QH + h) * n_splits;
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
        out[((size_t)(first_tok + t) * QH + h) * d + dim] = __float2bfloat16_rn(W > 0.0f ? O / W : 0.0f);
    }
}

// --------------------------------------------------------------------- host side
static int fa_shift(int n) {
    for (int s = 0; s < 31; ++s) if ((1 << s) == n) return s;
    return -1;
}
static int fa_group_chunk(int G) {                             // largest divisor of G that is <= 16
    for (int c = 16; c >= 1; --c) if (G % c == 0) return c;
    return 1;
}

template <int D>
static int fa_launch_prefill(const FaArgs& a, int n_tiles, cudaStream_t s) {
    const size_t smem = (size_t)FA_BM * FaSmem<D>::STRIDE + 2 * FaSmem<D>::STAGE;
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fa_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    return rb_launch(fa_prefill_kernel<D>, dim3(n_tiles, a.KH * a.chunks), dim3(FA_THREADS), smem, s, a);
}
template <int D, int NST>
static int fa_launch_decode(const FaArgs& a, cudaStream_t s) {
    const size_t pipe = (size_t)NST * FaSmem<D>::STAGE;
    const size_t merge = (size_t)FA_WARPS * 16 * (D + 2) * sizeof(float);
    const size_t smem = 16 * FaSmem<D>::STRIDE + (pipe > merge ? pipe : merge);
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fa_decode_kernel<D, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    return rb_launch(fa_decode_kernel<D, NST>, dim3(a.n_entries, a.KH * a.chunks, a.n_splits), dim3(FA_THREADS), smem, s, a);
}

static int fa_check(int QH, int KH, int d, int page_size, int max_pages) {
    if (QH <= 0 || KH <= 0 || QH % KH) RB_REFUSE("attention: %d query heads over %d kv heads", QH, KH);
    if (d <= 0 || d % 8 || d > 256) RB_REFUSE("attention (tensor cores): head_dim %d is not a multiple of 8 up to 256", d);
    if (page_size <= 0 || max_pages <= 0) RB_REFUSE("attention: page_size %d max_pages %d", page_size, max_pages);
    return 0;
}

// Entries [first_entry, first_entry + n_entries) bring q_len >= 1 tokens each; n_tiles = sum over them of
// ceil(q_len / (64 / Gc)) with Gc = rb_fa_group_chunk(QH / KH).
extern "C" int rb_fa_group_chunk(int G) { return fa_group_chunk(G); }

extern "C" int rb_fa_prefill(const void* q, const void* cache, const int* block_table, const int* cu_q, const int* kv_len,
                             void* out, int first_entry, int n_entries, int n_tiles, int QH, int KH, int d, int page_size,
                             int max_pages, int window, float scale, void* stream) {
    if (n_entries <= 0 || n_tiles <= 0) return 0;
    if (fa_check(QH, KH, d, page_size, max_pages)) return -1;
    FaArgs a{};
    a.q = (const bf16*)q; a.cache = (const bf16*)cache; a.block_table = block_table; a.cu_q = cu_q; a.kv_len = kv_len;
    a.out = (bf16*)out; a.QH = QH; a.KH = KH; a.d = d; a.page_size = page_size; a.page_shift = fa_shift(page_size); a.max_pages = max_pages; a.window = window;
    a.Gc = fa_group_chunk(QH / KH); a.chunks = (QH / KH) / a.Gc; a.first_entry = first_entry; a.n_entries = n_entries;
    a.n_splits = 1; a.scale_log2 = scale * 1.4426950408889634f;
    cudaStream_t s = (cudaStream_t)stream;
    if (d <= 32) return fa_launch_prefill<32>(a, n_tiles, s);
    if (d <= 64) return fa_launch_prefill<64>(a, n_tiles, s);
    if (d <= 128) return fa_launch_prefill<128>(a, n_tiles, s);
    return fa_launch_prefill<256>(a, n_tiles, s);
}

// Decode entries [first_entry, first_entry + n_entries): one token each.  With n_splits > 1 the scratch
// part_o [n_entries*QH*n_splits*d] and part_lse [n_entries*QH*n_splits] (floats) must be given.
extern "C" int rb_fa_decode(const void* q, const void* cache, const int* block_table, const int* cu_q, const int* kv_len,
                            void* out, float* part_o, float* part_lse, int first_entry, int n_entries, int first_tok,
                            int n_splits, int QH, int KH, int d, int page_size, int max_pages, int window, float scale,
                            void* stream) {
    if (n_entries <= 0) return 0;
    if (fa_check(QH, KH, d, page_size, max_pages)) return -1;
    if (n_splits < 1 || n_splits > 65535) RB_REFUSE("attention: %d splits", n_splits);
    if (n_splits > 1 && (!part_o || !part_lse)) RB_REFUSE("attention: split decoding needs its scratch");
    FaArgs a{};
    a.q = (const bf16*)q; a.cache = (const bf16*)cache; a.block_table = block_table; a.cu_q = cu_q; a.kv_len = kv_len;
    a.out = (bf16*)out; a.part_o = part_o; a.part_lse = part_lse;
    a.QH = QH; a.KH = KH; a.d = d; a.page_size = page_size; a.page_shift = fa_shift(page_size); a.max_pages = max_pages; a.window = window;
    a.Gc = fa_group_chunk(QH / KH); a.chunks = (QH / KH) / a.Gc; a.first_entry = first_entry; a.n_entries = n_entries;
    a.n_splits = n_splits; a.scale_log2 = scale * 1.4426950408889634f;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (d <= 32) rc = fa_launch_decode<32, 3>(a, s);
    else if (d <= 64) rc = fa_launch_decode<64, 3>(a, s);
    else if (d <= 128) rc = fa_launch_decode<128, 3>(a, s);
    else rc = fa_launch_decode<256, 2>(a, s);
    if (rc || n_splits == 1) return rc;
    return rb_launch(fa_merge_kernel, dim3(n_entries, QH), dim3(128), 0, s, (const float*)part_o, (const float*)part_lse,
                     (bf16*)out, first_tok, QH, d, n_splits);
}
