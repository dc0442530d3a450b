// The plain attention over the paged cache: any number of new tokens per request,
// causal, grouped heads, optional window.  One warp per (token, query head) walks the
// keys of its request in ascending order, in blocks of 32 that are aligned to absolute
// positions, with one online-softmax update per block.  The sequence of operations for
// a token depends only on its position (and the window), never on how the request was
// cut into steps, on the batch, or on the page size - so this kernel gives the same
// bits under every cut.  It is the attention of the 32-bit path and the yardstick of
// the faster bfloat16 kernels.
// (reference semantics: crates/cuda/kernels/decode_gqa_kernels.cu:99-136 page lookup
//  page[t/block_len]; decode_flash_kernels.cu:212-349 max/exp/sum/PV in f32.)
#include "common.cuh"

#define RA_WARPS 4
#define RA_MAX_D 512

// q        [T, QH, d]
// cache    one layer: [page][2][KH][page_size][d]
// block_table [rows, max_pages] (page id of the i-th page of a request's row)
// tok_row  [T] row of block_table for token t;  positions [T] absolute position of token t
// A token at position p attends keys max(0, p-window+1) .. p  (window <= 0: all of them).
template <typename TA, typename TC>
__global__ void __launch_bounds__(RA_WARPS * 32)
paged_attention_ref_kernel(const TA* __restrict__ q, const TC* __restrict__ cache,
                           const int* __restrict__ block_table, const int* __restrict__ tok_row,
                           const int* __restrict__ positions, TA* __restrict__ out,
                           int QH, int KH, int d, int page_size, int max_pages, int window, float scale) {
    extern __shared__ float qs_all[];                         // RA_WARPS * d floats
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int hq = blockIdx.y * RA_WARPS + warp;
    if (hq >= QH) return;                                     // no block-wide barrier below
    float* qs = qs_all + warp * d;
    const TA* qp = q + ((size_t)t * QH + hq) * d;
    for (int i = lane; i < d; i += 32) qs[i] = to_f32(qp[i]);
    __syncwarp();
    const int kh = hq / (QH / KH);
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* bt = block_table + (size_t)tok_row[t] * max_pages;
    const size_t head_stride = (size_t)page_size * d;         // one (page, k|v, head) tile
    const size_t page_stride = 2 * (size_t)KH * head_stride;

    constexpr int NACC = RA_MAX_D / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;

    for (int b0 = (lo / 32) * 32; b0 <= pos; b0 += 32) {
        const int key = b0 + lane;
        bool valid = key >= lo && key <= pos;
        float s = -INFINITY;
        const TC* vrow = nullptr;
        const int page = (valid && key / page_size < max_pages) ? bt[key / page_size] : -1;
        valid = valid && page >= 0;                            // a page that is not held: an inert padding row
        if (valid) {
            const int off = key % page_size;
            const TC* krow = cache + (size_t)page * page_stride + (size_t)kh * head_stride + (size_t)off * d;
            vrow = krow + (size_t)KH * head_stride;
            float dot = 0.0f;
            for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(krow[i]), dot);
            s = dot * scale;
        }
        const float bm = warp_max(s);
        if (bm == -INFINITY) continue;                         // no key in this block (warp-uniform)
        const float m_new = fmaxf(m, bm);
        const float corr = expf(m - m_new);                    // first block: exp(-inf) = 0
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const unsigned long long vj = __shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
            if (vj == 0ull) continue;                          // warp-uniform
            const TC* vr = (const TC*)vj;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int dim = lane + 32 * i;
                if (dim < d) acc[i] = fmaf(pj, to_f32(vr[dim]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    TA* op = out + ((size_t)t * QH + hq) * d;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int dim = lane + 32 * i;
        if (dim < d) op[dim] = from_f32<TA>(acc[i] * inv);
    }
}

extern "C" int rb_paged_attention_ref(const void* q, const void* cache, int dtype,
                                      const int* block_table, const int* tok_row, const int* positions,
                                      void* out, int n_tokens, int QH, int KH, int d, int page_size,
                                      int max_pages, int window, float scale, void* stream) {
    if (n_tokens <= 0) return 0;
    if (QH <= 0 || KH <= 0 || QH % KH != 0) RB_REFUSE("attention: %d query heads over %d kv heads", QH, KH);
    if (d <= 0 || d > RA_MAX_D) RB_REFUSE("attention: head_dim %d (supported: 1..%d)", d, RA_MAX_D);
    if (page_size <= 0 || max_pages <= 0) RB_REFUSE("attention: page_size %d max_pages %d", page_size, max_pages);
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, rb_ceil_div(QH, RA_WARPS));
    const size_t smem = (size_t)RA_WARPS * d * sizeof(float);
    if (dtype == RB_F32)
        paged_attention_ref_kernel<float, float><<<grid, RA_WARPS * 32, smem, s>>>(
            (const float*)q, (const float*)cache, block_table, tok_row, positions, (float*)out,
            QH, KH, d, page_size, max_pages, window, scale);
    else if (dtype == RB_BF16)
        paged_attention_ref_kernel<bf16, bf16><<<grid, RA_WARPS * 32, smem, s>>>(
            (const bf16*)q, (const bf16*)cache, block_table, tok_row, positions, (bf16*)out,
            QH, KH, d, page_size, max_pages, window, scale);
    else RB_REFUSE("attention: dtype %d", dtype);
    return RB_LAUNCH_RESULT();
}
