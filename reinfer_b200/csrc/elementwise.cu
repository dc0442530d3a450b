// Row-wise kernels: embedding gather, RMSNorm with the residual sum fused in,
// per-head q/k RMSNorm + rotary encoding + append to the paged cache, SwiGLU.
// All arithmetic is 32-bit; only loads and stores see the storage type.
// The residual stream is float in both precisions of the model.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// x[t,:] = E[ids[t],:]   (reference: crates/cuda/kernels/dense_kernels.cu:329-336)
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                    const int* __restrict__ slot_token, const int* __restrict__ entry_slot,
                                    const int* __restrict__ tok_entry, float* __restrict__ out, int h, int vocab) {
    pdl_trigger(); pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    // a negative id stands for "the token that the sampler drew for this request in the step before": it is in
    // the request's slot on the device, so the host need not have seen it yet
    if (id < 0 && slot_token) id = slot_token[entry_slot[tok_entry[t]]];
    const bool ok = (id >= 0 && id < vocab);          // the host refuses other ids before launching
    const TW* row = table + (size_t)(ok ? id : 0) * h;
    float* o = out + (size_t)t * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) o[i] = ok ? to_f32(row[i]) : 0.0f;
}

// slot_token [slots], entry_slot [entries], tok_entry [tokens]: all three, or none (then every id must be >= 0).
extern "C" int rb_embed_gather(const void* table, int table_dtype, const int* ids, const int* slot_token,
                               const int* entry_slot, const int* tok_entry, float* out,
                               int n_tokens, int h, int vocab, void* stream) {
    if (n_tokens <= 0) return 0;
    if (h <= 0 || vocab <= 0) RB_REFUSE("embed_gather: hidden=%d vocab=%d", h, vocab);
    if (slot_token && (!entry_slot || !tok_entry)) RB_REFUSE("embed_gather: tokens from slots need the slot of each entry and the entry of each token");
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = h >= 1024 ? 256 : 128;
    if (table_dtype == RB_F32)
        return rb_launch(embed_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)table, ids,
                         slot_token, entry_slot, tok_entry, out, h, vocab);
    if (table_dtype == RB_BF16)
        return rb_launch(embed_gather_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, (const bf16*)table, ids,
                         slot_token, entry_slot, tok_entry, out, h, vocab);
    RB_REFUSE("embed_gather: table dtype %d", table_dtype);
}

// ------------------------------------------------------------------ RMSNorm
// Optional residual sum first:  x[r,:] += delta[r,:]  (x is float, written back), then
// out[r,:] = x * (1/sqrt(mean(x^2)+eps)) * w       (dense_kernels.cu:59-88, 257-296).
// With row_idx the input row of output row r is row_idx[r] (gather of the rows whose
// logits are wanted); a residual sum is not combined with row_idx.
// One block per row; each thread sums its strided elements in ascending order and the
// block tree is fixed, so a row's result does not depend on the other rows.
template <typename TD, typename TW, typename TO, int PER>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_delta, long long delta_stride,
                                   const TW* __restrict__ w, TO* __restrict__ out,
                                   const int* __restrict__ row_idx, int h, float eps) {
    RB_TL(2);
    __shared__ float red[32];
    pdl_trigger();
    // the norm's weights never change: they are fetched while the kernels before this one still run
    float wv[PER > 0 ? PER : 1];
    if (PER > 0) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            wv[k] = i < h ? to_f32(w[i]) : 0.0f;
        }
    }
    pdl_wait();
    RB_TL_MARK();
    const int r = blockIdx.x;
    const size_t in_row = row_idx ? (size_t)row_idx[r] : (size_t)r;
    float* xr = x + in_row * h;
    const TD* dr = delta ? delta + in_row * h : nullptr;
    const bool keep = delta && !row_idx;              // gathered rows are read once more by nobody: x stays as it is
    // each thread keeps its strided elements in registers (PER of them; PER == 0: rows too wide, re-read)
    float v[PER > 0 ? PER : 1];
    float ss = 0.0f;
    if (PER > 0) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            float t = 0.0f;
            if (i < h) {
                t = xr[i];
                if (delta) {
                    for (int p = 0; p < n_delta; ++p) t += to_f32(dr[(size_t)p * delta_stride + i]);   // ascending: a fixed order
                    if (keep) xr[i] = t;
                }
            }
            v[k] = t;
            ss += t * t;
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            float t = xr[i];
            if (delta) {
                for (int p = 0; p < n_delta; ++p) t += to_f32(dr[(size_t)p * delta_stride + i]);
                xr[i] = t;
            }
            ss += t * t;
        }
    }
    const float total = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(total / (float)h + eps);
    TO* orow = out + (size_t)r * h;
    if (PER > 0) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < h) orow[i] = from_f32<TO>(v[k] * rstd * wv[k]);
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x)
            orow[i] = from_f32<TO>(xr[i] * rstd * to_f32(w[i]));
    }
}

template <typename TD, typename TW, typename TO>
static int launch_add_rmsnorm_k(float* x, const TD* delta, int n_delta, long long delta_stride, const TW* w, TO* out,
                                const int* row_idx, int rows, int h, float eps, cudaStream_t s) {
    // the summation order (thread stride, then the block tree) depends on h only, never on the batch
    if (h <= 512) return rb_launch(add_rmsnorm_kernel<TD, TW, TO, 4>, dim3(rows), dim3(128), 0, s, x, delta, n_delta, delta_stride, w, out, row_idx, h, eps);
    if (h <= 2048) return rb_launch(add_rmsnorm_kernel<TD, TW, TO, 8>, dim3(rows), dim3(256), 0, s, x, delta, n_delta, delta_stride, w, out, row_idx, h, eps);
    if (h <= 8192) return rb_launch(add_rmsnorm_kernel<TD, TW, TO, 8>, dim3(rows), dim3(1024), 0, s, x, delta, n_delta, delta_stride, w, out, row_idx, h, eps);
    if (delta && row_idx) RB_REFUSE("rmsnorm: rows of %d elements cannot combine a residual sum with a row gather", h);
    return rb_launch(add_rmsnorm_kernel<TD, TW, TO, 0>, dim3(rows), dim3(1024), 0, s, x, delta, n_delta, delta_stride, w, out, row_idx, h, eps);
}

// The same for a few rows of 16-bit activations (a decode step), where one CTA per row would be bound by what one
// SM can pull from L2 - above all when delta is a stack of partial sums.  A row is shared by a cluster of RN_CL
// CTAs: each takes a contiguous share of the columns (16-byte loads, all of a thread's loads in flight at once),
// forms its part of the sum of squares in a fixed order, and the parts are exchanged through distributed shared
// memory and added in rank order - so a row's result depends on h alone, not on the other rows.
constexpr int RN_CL = 4, RN_THREADS = 256, RN_VPER = 4;
template <typename TW>
__global__ void __launch_bounds__(RN_THREADS)
add_rmsnorm_cluster_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta, long long delta_stride,
                           const TW* __restrict__ w, bf16* __restrict__ out, const int* __restrict__ row_idx, int h, float eps) {
    RB_TL(2);
    __shared__ float red[32];
    __shared__ float part_ss[RN_CL];
    pdl_trigger();
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int share = h / RN_CL;                              // columns of this CTA, a multiple of 4
    const int c0 = (int)rank * share;
    // the norm's weights never change: they are fetched while the kernels before this one still run
    float4 wv[RN_VPER];
#pragma unroll
    for (int k = 0; k < RN_VPER; ++k) {
        const int i = (threadIdx.x + k * RN_THREADS) * 4;
        wv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < share) { wv[k].x = to_f32(w[c0 + i]); wv[k].y = to_f32(w[c0 + i + 1]); wv[k].z = to_f32(w[c0 + i + 2]); wv[k].w = to_f32(w[c0 + i + 3]); }
    }
    pdl_wait();
    RB_TL_MARK();
    const int r = blockIdx.y;
    const size_t in_row = row_idx ? (size_t)row_idx[r] : (size_t)r;
    float* xr = x + in_row * h + c0;
    const float* dr = delta ? delta + in_row * h + c0 : nullptr;
    const bool keep = delta && !row_idx;
    float4 v[RN_VPER];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < RN_VPER; ++k) {
        const int i = (threadIdx.x + k * RN_THREADS) * 4;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < share) {
            t = *reinterpret_cast<const float4*>(xr + i);
            if (delta) {
                for (int p0 = 0; p0 < n_delta; p0 += 8) {      // eight partial sums in flight, added in ascending order
                    float4 d[8];
#pragma unroll
                    for (int p = 0; p < 8; ++p)
                        d[p] = p0 + p < n_delta ? *reinterpret_cast<const float4*>(dr + (size_t)(p0 + p) * delta_stride + i)
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int p = 0; p < 8; ++p) if (p0 + p < n_delta) { t.x += d[p].x; t.y += d[p].y; t.z += d[p].z; t.w += d[p].w; }
                }
                if (keep) *reinterpret_cast<float4*>(xr + i) = t;
            }
        }
        v[k] = t;
        ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
    }
    const float mine = block_sum(ss, red);
    // every CTA writes its part into the slot of its rank in every CTA of the cluster (its own included); after
    // the one barrier each reads its own shared memory only, so nobody has to outlive its peers
    if (threadIdx.x < RN_CL) {
        uint32_t remote;
        const uint32_t local = (uint32_t)__cvta_generic_to_shared(&part_ss[rank]);
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((uint32_t)threadIdx.x));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(mine) : "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    float total = 0.0f;
#pragma unroll
    for (int c = 0; c < RN_CL; ++c) total += part_ss[c];     // rank order: the same sum in every CTA of the row
    const float rstd = 1.0f / sqrtf(total / (float)h + eps);
    bf16* orow = out + (size_t)r * h + c0;                  // 8-byte aligned: h and the share are multiples of 4
#pragma unroll
    for (int k = 0; k < RN_VPER; ++k) {
        const int i = (threadIdx.x + k * RN_THREADS) * 4;
        if (i < share) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v[k].x * rstd * wv[k].x, v[k].y * rstd * wv[k].y);
            const __nv_bfloat162 hi = __floats2bfloat162_rn(v[k].z * rstd * wv[k].z, v[k].w * rstd * wv[k].w);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo); pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(orow + i) = pk;
        }
    }
}

// Many rows of 16-bit activations (a prompt portion): one CTA per row with 16-byte loads and stores, every load of
// a thread in flight before the first is used.  (The 32-bit path keeps the scalar kernel above, whose sums do not
// depend on how many rows a step brings.)
constexpr int RV_THREADS = 256;
template <typename TW, int VPER>
__global__ void __launch_bounds__(RV_THREADS)
add_rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta, long long delta_stride,
                       const TW* __restrict__ w, bf16* __restrict__ out, int h, float eps) {
    RB_TL(2);
    __shared__ float red[32];
    pdl_trigger(); pdl_wait();
    RB_TL_MARK();
    const size_t row = (size_t)blockIdx.x * h;
    float4 v[VPER];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < VPER; ++k) {
        const int i = (threadIdx.x + k * RV_THREADS) * 4;
        v[k] = i < h ? *reinterpret_cast<const float4*>(x + row + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (delta) {
        for (int p = 0; p < n_delta; ++p) {                        // ascending: a fixed order
#pragma unroll
            for (int k = 0; k < VPER; ++k) {
                const int i = (threadIdx.x + k * RV_THREADS) * 4;
                if (i < h) {
                    const float4 d = *reinterpret_cast<const float4*>(delta + (size_t)p * delta_stride + row + i);
                    v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
                }
            }
        }
#pragma unroll
        for (int k = 0; k < VPER; ++k) {
            const int i = (threadIdx.x + k * RV_THREADS) * 4;
            if (i < h) *reinterpret_cast<float4*>(x + row + i) = v[k];
        }
    }
#pragma unroll
    for (int k = 0; k < VPER; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    const float total = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(total / (float)h + eps);
#pragma unroll
    for (int k = 0; k < VPER; ++k) {
        const int i = (threadIdx.x + k * RV_THREADS) * 4;
        if (i < h) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v[k].x * rstd * to_f32(w[i]), v[k].y * rstd * to_f32(w[i + 1]));
            const __nv_bfloat162 hi = __floats2bfloat162_rn(v[k].z * rstd * to_f32(w[i + 2]), v[k].w * rstd * to_f32(w[i + 3]));
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo); pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(out + row + i) = pk;
        }
    }
}
template <typename TW>
static int launch_add_rmsnorm_vec(float* x, const float* delta, int n_delta, long long delta_stride, const TW* w, bf16* out,
                                  int rows, int h, float eps, cudaStream_t s) {
    const int vper = rb_ceil_div(h, RV_THREADS * 4);
    if (vper <= 1) return rb_launch(add_rmsnorm_vec_kernel<TW, 1>, dim3(rows), dim3(RV_THREADS), 0, s, x, delta, n_delta, delta_stride, w, out, h, eps);
    if (vper <= 2) return rb_launch(add_rmsnorm_vec_kernel<TW, 2>, dim3(rows), dim3(RV_THREADS), 0, s, x, delta, n_delta, delta_stride, w, out, h, eps);
    if (vper <= 4) return rb_launch(add_rmsnorm_vec_kernel<TW, 4>, dim3(rows), dim3(RV_THREADS), 0, s, x, delta, n_delta, delta_stride, w, out, h, eps);
    return rb_launch(add_rmsnorm_vec_kernel<TW, 8>, dim3(rows), dim3(RV_THREADS), 0, s, x, delta, n_delta, delta_stride, w, out, h, eps);
}

// An RMS norm whose division is left to the product that reads it:  x[r,:] += sum_p delta[p][r,:] (ascending),
// y[r,:] = bfloat16(x[r,:] * w), and sumsq[r, c] = the sum of x^2 over the columns of chunk c (RS_COLS columns a
// chunk).  The reader multiplies its results for row r by 1/sqrt(sum_c sumsq[r,c] / h + eps), which is the same
// number as normalising first (a row's factor is a scalar that passes through a product) - and so no CTA here
// needs another CTA's sum: a decode step's few rows spread over rows x chunks CTAs, each one trip to L2.
constexpr int RS_THREADS = 256, RS_COLS = RS_THREADS * 4;
template <typename TW>
__global__ void __launch_bounds__(RS_THREADS)
residual_rowscale_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta, long long delta_stride,
                         const TW* __restrict__ w, bf16* __restrict__ y, float* __restrict__ sumsq, int h) {
    RB_TL(2);
    __shared__ float red[32];
    pdl_trigger();
    const int i = (blockIdx.x * RS_THREADS + threadIdx.x) * 4;      // h is a multiple of 4
    const bool in = i < h;
    float4 wv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (in) { wv.x = to_f32(w[i]); wv.y = to_f32(w[i + 1]); wv.z = to_f32(w[i + 2]); wv.w = to_f32(w[i + 3]); }
    pdl_wait();
    RB_TL_MARK();
    const size_t row = (size_t)blockIdx.y * h;
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    if (in) {
        t = *reinterpret_cast<const float4*>(x + row + i);
        if (delta) {
            const float* dr = delta + row + i;
            for (int p0 = 0; p0 < n_delta; p0 += 8) {          // eight partial sums in flight, added in ascending order
                float4 d[8];
#pragma unroll
                for (int p = 0; p < 8; ++p)
                    d[p] = p0 + p < n_delta ? *reinterpret_cast<const float4*>(dr + (size_t)(p0 + p) * delta_stride)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int p = 0; p < 8; ++p) if (p0 + p < n_delta) { t.x += d[p].x; t.y += d[p].y; t.z += d[p].z; t.w += d[p].w; }
            }
            *reinterpret_cast<float4*>(x + row + i) = t;
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(t.x * wv.x, t.y * wv.y);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(t.z * wv.z, t.w * wv.w);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo); pk.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(y + row + i) = pk;
    }
    const float ss = block_sum(t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w, red);
    if (threadIdx.x == 0) sumsq[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = ss;
}

// How many chunks (parts of a row's sum of squares) rb_residual_rowscale writes for rows of h elements.
extern "C" int rb_rowscale_parts(int h) { return h > 0 ? rb_ceil_div(h, RS_COLS) : 0; }

extern "C" int rb_residual_rowscale(float* x, const float* delta, int n_delta, long long delta_stride, const void* w, int w_dtype,
                                    void* y, float* sumsq, int rows, int h, void* stream) {
    if (rows <= 0) return 0;
    if (h <= 0 || h % 4) RB_REFUSE("rowscale: width %d is not a multiple of 4", h);
    if (delta && (n_delta < 1 || n_delta > 64 || delta_stride % 4)) RB_REFUSE("rowscale: %d partial sums, %lld apart", n_delta, delta_stride);
    if ((((uintptr_t)x | (uintptr_t)delta) & 15) || ((uintptr_t)y & 7)) RB_REFUSE("rowscale: operands must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(rb_ceil_div(h, RS_COLS), rows);
    if (w_dtype == RB_F32)
        return rb_launch(residual_rowscale_kernel<float>, grid, dim3(RS_THREADS), 0, s, x, delta, n_delta, delta_stride,
                         (const float*)w, (bf16*)y, sumsq, h);
    if (w_dtype == RB_BF16)
        return rb_launch(residual_rowscale_kernel<bf16>, grid, dim3(RS_THREADS), 0, s, x, delta, n_delta, delta_stride,
                         (const bf16*)w, (bf16*)y, sumsq, h);
    RB_REFUSE("rowscale: weight dtype %d", w_dtype);
}

template <typename TD, typename TW>
static int launch_add_rmsnorm_o(float* x, const void* delta, int n_delta, long long delta_stride, const void* w, void* out, int out_dtype,
                                const int* row_idx, int rows, int h, float eps, cudaStream_t s) {
    if (out_dtype == RB_F32)
        return launch_add_rmsnorm_k<TD, TW, float>(x, (const TD*)delta, n_delta, delta_stride, (const TW*)w, (float*)out, row_idx, rows, h, eps, s);
    if (out_dtype == RB_BF16)
        return launch_add_rmsnorm_k<TD, TW, bf16>(x, (const TD*)delta, n_delta, delta_stride, (const TW*)w, (bf16*)out, row_idx, rows, h, eps, s);
    RB_REFUSE("rmsnorm: out dtype %d", out_dtype);
}

// delta: n_delta partial sums of x's shape, delta_stride elements apart (n_delta == 1: one plain addend); they
// are added to x in ascending order.  With row_idx the sums are formed for the gathered rows only and x is left
// as it was (the pass ends there).
extern "C" int rb_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_delta, long long delta_stride,
                              const void* w, int w_dtype, void* out, int out_dtype, const int* row_idx, int rows, int h,
                              float eps, void* stream) {
    if (rows <= 0) return 0;
    if (h <= 0) RB_REFUSE("rmsnorm: width %d", h);
    if (delta && (n_delta < 1 || n_delta > 64)) RB_REFUSE("rmsnorm: %d partial sums", n_delta);
    cudaStream_t s = (cudaStream_t)stream;
    const int dd = delta ? delta_dtype : RB_F32;
    // a stack of partial sums for a decode step's few rows of 16-bit activations: a cluster per row (the whole
    // 32-bit path keeps the one kernel, whose sums do not depend on how many rows a step brings)
    if (out_dtype == RB_BF16 && dd == RB_F32 && delta && n_delta > 1 && rows <= 64 && h % (4 * RN_CL) == 0 && h / RN_CL <= RN_THREADS * 4 * RN_VPER &&
        ((((uintptr_t)x | (uintptr_t)delta) & 15) == 0) && (((uintptr_t)out) & 7) == 0 && delta_stride % 4 == 0) {
        if (w_dtype == RB_F32)
            return rb_launch_cluster(add_rmsnorm_cluster_kernel<float>, dim3(RN_CL, rows), dim3(RN_THREADS), dim3(RN_CL, 1, 1), 0, s, x,
                                     (const float*)delta, n_delta, delta_stride, (const float*)w, (bf16*)out, row_idx, h, eps);
        if (w_dtype == RB_BF16)
            return rb_launch_cluster(add_rmsnorm_cluster_kernel<bf16>, dim3(RN_CL, rows), dim3(RN_THREADS), dim3(RN_CL, 1, 1), 0, s, x,
                                     (const float*)delta, n_delta, delta_stride, (const bf16*)w, (bf16*)out, row_idx, h, eps);
    }
    if (out_dtype == RB_BF16 && dd == RB_F32 && !row_idx && rows > 64 && h % 4 == 0 && h <= RV_THREADS * 4 * 8 &&
        ((((uintptr_t)x | (uintptr_t)delta) & 15) == 0) && (((uintptr_t)out) & 7) == 0 && (!delta || delta_stride % 4 == 0)) {
        if (w_dtype == RB_F32) return launch_add_rmsnorm_vec<float>(x, (const float*)delta, n_delta, delta_stride, (const float*)w, (bf16*)out, rows, h, eps, s);
        if (w_dtype == RB_BF16) return launch_add_rmsnorm_vec<bf16>(x, (const float*)delta, n_delta, delta_stride, (const bf16*)w, (bf16*)out, rows, h, eps, s);
    }
    if (dd == RB_F32 && w_dtype == RB_F32) return launch_add_rmsnorm_o<float, float>(x, delta, n_delta, delta_stride, w, out, out_dtype, row_idx, rows, h, eps, s);
    if (dd == RB_F32 && w_dtype == RB_BF16) return launch_add_rmsnorm_o<float, bf16>(x, delta, n_delta, delta_stride, w, out, out_dtype, row_idx, rows, h, eps, s);
    if (dd == RB_BF16 && w_dtype == RB_F32) return launch_add_rmsnorm_o<bf16, float>(x, delta, n_delta, delta_stride, w, out, out_dtype, row_idx, rows, h, eps, s);
    if (dd == RB_BF16 && w_dtype == RB_BF16) return launch_add_rmsnorm_o<bf16, bf16>(x, delta, n_delta, delta_stride, w, out, out_dtype, row_idx, rows, h, eps, s);
    RB_REFUSE("rmsnorm: dtypes delta=%d weight=%d", delta_dtype, w_dtype);
}

// x[r,:] += delta[r,:]  (the last residual sum of a layer when nothing follows to fuse it into)
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n) {
    pdl_trigger(); pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += to_f32(delta[i]);
}
extern "C" int rb_residual_add(float* x, const void* delta, int delta_dtype, long long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = rb_ceil_div(n, 256);
    if (delta_dtype == RB_F32) residual_add_kernel<float><<<blocks, 256, 0, s>>>(x, (const float*)delta, (size_t)n);
    else if (delta_dtype == RB_BF16) residual_add_kernel<bf16><<<blocks, 256, 0, s>>>(x, (const bf16*)delta, (size_t)n);
    else RB_REFUSE("residual_add: dtype %d", delta_dtype);
    return RB_LAUNCH_RESULT();
}

// ------------------------------------------- q/k head norm + rotation + cache append
// Input  qkv[t, (QH+2KH)*d]: q heads, then k heads, then v heads of token t.
// q: optional RMSNorm over the head row (weight qw[d]), rotation, -> q_out[t, QH, d]
// k: optional RMSNorm (kw[d]), rotation, -> cache K at slot kv_slot[t]
// v: copy -> cache V at the same slot
// (reference order: dense_kernels.cu:92-123 norm, :127-170 rotation, :302-318 append;
//  the reference also multiplies q by 1/sqrt(d) here, engine.rs:4150-4160 - that scale is
//  applied to the scores inside the attention kernels instead, so q is rounded once less).
// Rotation pairs (p, p+rot/2) for p < rot/2, angle = pos * inv_freq[p]; dims >= rot pass through.
// Cache layout of one layer: [page][2 (k,v)][KH][page_size][d]; slot = page*page_size + offset;
// slot < 0 means "do not store" (a layer that reads another layer's cache).
// With k_out given, k goes to k_out[t, KH, d] instead of the cache and v is left alone
// (the path of a position encoding that is not a plain rotation: it is applied between
// this kernel and rb_kv_append).  KH may be 0 (rotation of q alone).
// One warp per (token, head row).
template <typename TA, typename TW, typename TC>
__global__ void qknorm_rope_append_kernel(const TA* __restrict__ qkv, const TW* __restrict__ qw,
                                          const TW* __restrict__ kw, const float* __restrict__ inv_freq,
                                          const int* __restrict__ positions, const int* __restrict__ kv_slot,
                                          TA* __restrict__ q_out, TA* __restrict__ k_out,
                                          TC* __restrict__ cache, int n_tokens, int QH, int KH, int d, int rot, int page_size,
                                          float eps) {
    pdl_trigger(); pdl_wait();
    const int heads = QH + 2 * KH;
    const long long wglobal = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wglobal >= (long long)n_tokens * heads) return;
    const int t = (int)(wglobal / heads);
    const int hh = (int)(wglobal % heads);
    const TA* src = qkv + ((size_t)t * heads + hh) * d;
    const int slot = kv_slot ? kv_slot[t] : -1;

    if (hh >= QH + KH) {                                   // a value head: plain copy into the cache
        if (slot < 0 || k_out) return;
        const int kh = hh - QH - KH;
        const int page = slot / page_size, off = slot % page_size;
        TC* dst = cache + ((((size_t)page * 2 + 1) * KH + kh) * page_size + off) * d;
        for (int i = lane; i < d; i += 32) dst[i] = from_f32<TC>(to_f32(src[i]));
        return;
    }
    const bool is_q = hh < QH;
    const TW* w = is_q ? qw : kw;
    if (!is_q && !k_out && slot < 0) return;
    // 1/rms over the whole head row
    float rstd = 1.0f;
    if (w) {
        float ss = 0.0f;
        for (int i = lane; i < d; i += 32) { float v = to_f32(src[i]); ss += v * v; }
        ss = warp_sum(ss);
        rstd = 1.0f / sqrtf(ss / (float)d + eps);
    }
    const int half = rot >> 1;
    const float pos = positions ? (float)positions[t] : 0.0f;   // no rotation: no positions
    TA* qdst = is_q ? q_out + ((size_t)t * QH + hh) * d : nullptr;
    TC* kdst = nullptr;
    TA* kdst_a = (!is_q && k_out) ? k_out + ((size_t)t * KH + (hh - QH)) * d : nullptr;
    if (!is_q && !k_out) {
        const int kh = hh - QH;
        const int page = slot / page_size, off = slot % page_size;
        kdst = cache + ((((size_t)page * 2 + 0) * KH + kh) * page_size + off) * d;
    }
    for (int p = lane; p < half; p += 32) {
        float a = to_f32(src[p]), b = to_f32(src[p + half]);
        if (w) { a = a * rstd * to_f32(w[p]); b = b * rstd * to_f32(w[p + half]); }
        float sn, cs;
        sincosf(pos * inv_freq[p], &sn, &cs);
        const float ra = a * cs - b * sn, rb = a * sn + b * cs;
        if (is_q) { qdst[p] = from_f32<TA>(ra); qdst[p + half] = from_f32<TA>(rb); }
        else if (kdst_a) { kdst_a[p] = from_f32<TA>(ra); kdst_a[p + half] = from_f32<TA>(rb); }
        else { kdst[p] = from_f32<TC>(ra); kdst[p + half] = from_f32<TC>(rb); }
    }
    for (int i = rot + lane; i < d; i += 32) {             // dims beyond the rotated part
        float a = to_f32(src[i]);
        if (w) a = a * rstd * to_f32(w[i]);
        if (is_q) qdst[i] = from_f32<TA>(a);
        else if (kdst_a) kdst_a[i] = from_f32<TA>(a);
        else kdst[i] = from_f32<TC>(a);
    }
}

// The angles' cosines and sines of a step, once for all layers and heads: cs[t, p] = (cos, sin)(pos[t] * inv_freq[p]).
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cs, int n_tokens, int half) {
    pdl_trigger(); pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * half) return;
    const int t = i / half, p = i % half;
    float sn, c;
    sincosf((float)positions[t] * inv_freq[p], &sn, &c);
    cs[i] = make_float2(c, sn);
}
extern "C" int rb_rope_table(const int* positions, const float* inv_freq, void* cs, int n_tokens, int half, void* stream) {
    if (n_tokens <= 0 || half <= 0) return 0;
    return rb_launch(rope_table_kernel, dim3(rb_ceil_div((long long)n_tokens * half, 256)), dim3(256), 0, (cudaStream_t)stream,
                     positions, inv_freq, (float2*)cs, n_tokens, half);
}

// The same operation for the common layout - bfloat16 activations and cache, the whole head rotated, head_dim a
// multiple of 128 - with 4-byte loads and stores (a lane owns element pairs 2l, 2l+1 of both halves) and 16-byte
// copies of the value rows; cosines and sines come from the step's table when one is given.
template <typename TW>
__global__ void qknorm_rope_append_vec_kernel(const bf16* __restrict__ qkv, const TW* __restrict__ qw, const TW* __restrict__ kw,
                                              const float* __restrict__ inv_freq, const float2* __restrict__ cs_table,
                                              const int* __restrict__ positions, const int* __restrict__ kv_slot,
                                              bf16* __restrict__ q_out, bf16* __restrict__ cache,
                                              int n_tokens, int QH, int KH, int d, int page_size, float eps) {
    RB_TL(3);
    pdl_trigger();
    // Everything that does not come from the kernels before this one - the step's positions and slots, the
    // norm weights, the angles - is fetched and computed while they still run; only qkv (and a table of
    // cosines that an earlier kernel of this step wrote) waits for them.
    const int heads = QH + 2 * KH;
    const long long wglobal = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wglobal >= (long long)n_tokens * heads) return;
    const int t = (int)(wglobal / heads);
    const int hh = (int)(wglobal % heads);
    const bf16* src = qkv + ((size_t)t * heads + hh) * d;
    const int slot = kv_slot ? kv_slot[t] : -1;
    if (hh >= QH + KH) {
        if (slot < 0) return;
        const int kh = hh - QH - KH;
        const int page = slot / page_size, off = slot % page_size;
        bf16* dst = cache + ((((size_t)page * 2 + 1) * KH + kh) * page_size + off) * d;
        pdl_wait();
        RB_TL_MARK();
        for (int i = lane; i < d / 8; i += 32)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
        return;
    }
    const bool is_q = hh < QH;
    if (!is_q && slot < 0) return;
    const TW* w = is_q ? qw : kw;
    const int half = d >> 1;
    bf16* dst;
    if (is_q) dst = q_out + ((size_t)t * QH + hh) * d;
    else {
        const int page = slot / page_size, off = slot % page_size;
        dst = cache + ((((size_t)page * 2 + 0) * KH + (hh - QH)) * page_size + off) * d;
    }
    // this lane's pairs: elements p, p+1 with p = 2*lane + 64*i, and their partners half further
    const int n_it = half / 64;                               // head_dim <= 512
    float wa0[4], wa1[4], wb0[4], wb1[4], c0[4], s0[4], c1[4], s1[4];
    const float pos = (float)positions[t];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        wa0[i] = wa1[i] = wb0[i] = wb1[i] = 1.0f;
        c0[i] = c1[i] = 1.0f; s0[i] = s1[i] = 0.0f;
        if (i < n_it) {
            const int p = 2 * lane + 64 * i;
            if (w) { wa0[i] = to_f32(w[p]); wa1[i] = to_f32(w[p + 1]); wb0[i] = to_f32(w[p + half]); wb1[i] = to_f32(w[p + half + 1]); }
            if (!cs_table) {
                sincosf(pos * inv_freq[p], &s0[i], &c0[i]);
                sincosf(pos * inv_freq[p + 1], &s1[i], &c1[i]);
            }
        }
    }
    pdl_wait();
    RB_TL_MARK();
    float a0[4], a1[4], b0[4], b1[4];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (i < n_it) {
            const int p = 2 * lane + 64 * i;
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + p));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + p + half));
            a0[i] = lo.x; a1[i] = lo.y; b0[i] = hi.x; b1[i] = hi.y;
            ss += lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y;
            if (cs_table) {
                const float4 v = *reinterpret_cast<const float4*>(cs_table + (size_t)t * half + p);
                c0[i] = v.x; s0[i] = v.y; c1[i] = v.z; s1[i] = v.w;
            }
        }
    }
    float rstd = 1.0f;
    if (w) {
        ss = warp_sum(ss);
        rstd = 1.0f / sqrtf(ss / (float)d + eps);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (i < n_it) {
            const int p = 2 * lane + 64 * i;
            float x0 = a0[i], x1 = a1[i], y0 = b0[i], y1 = b1[i];
            if (w) {
                x0 = x0 * rstd * wa0[i]; x1 = x1 * rstd * wa1[i];
                y0 = y0 * rstd * wb0[i]; y1 = y1 * rstd * wb1[i];
            }
            *reinterpret_cast<__nv_bfloat162*>(dst + p) = __floats2bfloat162_rn(x0 * c0[i] - y0 * s0[i], x1 * c1[i] - y1 * s1[i]);
            *reinterpret_cast<__nv_bfloat162*>(dst + p + half) = __floats2bfloat162_rn(x0 * s0[i] + y0 * c0[i], x1 * s1[i] + y1 * c1[i]);
        }
    }
}

// The same for many tokens (a prompt portion) and heads of 128: a warp takes one token and a group of up to
// QG_HEADS heads of one kind (query, key or value).  A lane owns four neighbouring elements of a head (one 8-byte
// load and store per head); the partner of a rotation pair (p, p + 64) sits in lane ^ 16 and comes by shuffle.  The
// token's slot, cosines, sines and the norm's weights are fetched once per group, and the loads of all its heads
// are in flight together.
constexpr int QG_HEADS = 4;
template <typename TW>
__global__ void __launch_bounds__(128)
qknorm_rope_append_d128_kernel(const bf16* __restrict__ qkv, const TW* __restrict__ qw, const TW* __restrict__ kw,
                               const float* __restrict__ inv_freq, const float2* __restrict__ cs_table,
                               const int* __restrict__ positions, const int* __restrict__ kv_slot,
                               bf16* __restrict__ q_out, bf16* __restrict__ cache,
                               int n_tokens, int QH, int KH, int page_size, float eps) {
    RB_TL(3);
    pdl_trigger(); pdl_wait();
    RB_TL_MARK();
    constexpr int d = 128, half = 64;
    const int qg = (QH + QG_HEADS - 1) / QG_HEADS, kg = (KH + QG_HEADS - 1) / QG_HEADS;
    const int groups = qg + 2 * kg;
    const long long wglobal = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wglobal >= (long long)n_tokens * groups) return;
    const int t = (int)(wglobal / groups), g = (int)(wglobal % groups);
    const int kind = g < qg ? 0 : (g < qg + kg ? 1 : 2);          // query, key, value
    const int h0 = (kind == 0 ? g : kind == 1 ? g - qg : g - qg - kg) * QG_HEADS;
    const int nh = min(QG_HEADS, (kind == 0 ? QH : KH) - h0);
    const bf16* src0 = qkv + ((size_t)t * (QH + 2 * KH) + (kind == 0 ? 0 : kind == 1 ? QH : QH + KH) + h0) * d + 4 * lane;
    // every load of the warp is independent of the others: all are issued before the first is used
    uint2 raw[QG_HEADS];
#pragma unroll
    for (int j = 0; j < QG_HEADS; ++j) raw[j] = j < nh ? *reinterpret_cast<const uint2*>(src0 + (size_t)j * d) : make_uint2(0u, 0u);
    const int slot = kv_slot ? kv_slot[t] : -1;
    const int p = (4 * lane) & (half - 1);                        // the pair index of this lane's first element
    const TW* w = kind == 0 ? qw : kw;
    float wv[4] = {1.f, 1.f, 1.f, 1.f}, c[4], sn[4];
    if (kind != 2) {
        if (w) {
#pragma unroll
            for (int i = 0; i < 4; ++i) wv[i] = to_f32(w[4 * lane + i]);
        }
        if (cs_table) {
            const float4 a = *reinterpret_cast<const float4*>(cs_table + (size_t)t * half + p);
            const float4 b = *reinterpret_cast<const float4*>(cs_table + (size_t)t * half + p + 2);
            c[0] = a.x; sn[0] = a.y; c[1] = a.z; sn[1] = a.w; c[2] = b.x; sn[2] = b.y; c[3] = b.z; sn[3] = b.w;
        } else {
            const float pos = (float)positions[t];
#pragma unroll
            for (int i = 0; i < 4; ++i) sincosf(pos * inv_freq[p + i], &sn[i], &c[i]);
        }
    }
    if (kind != 0 && slot < 0) return;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    // low half (lanes 0..15): x c - y s;  high half: y c + x s
#pragma unroll
    for (int j = 0; j < QG_HEADS; ++j) {
        if (j >= nh) break;
        bf16* dst = kind == 0 ? q_out + ((size_t)t * QH + h0 + j) * d
                              : cache + ((((size_t)page * 2 + (kind == 2 ? 1 : 0)) * KH + h0 + j) * page_size + off) * d;
        if (kind == 2) { *reinterpret_cast<uint2*>(dst + 4 * lane) = raw[j]; continue; }
        const float2 v01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[j].x));
        const float2 v23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[j].y));
        float v[4] = {v01.x, v01.y, v23.x, v23.y};
        if (w) {
            const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
            const float rstd = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = v[i] * rstd * wv[i];
        }
        float o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
            o[i] = lane < 16 ? v[i] * c[i] - other * sn[i] : other * sn[i] + v[i] * c[i];
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo); pk.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst + 4 * lane) = pk;
    }
}

extern "C" int rb_qknorm_rope_append(const void* qkv, int act_dtype, const void* qw, const void* kw, int w_dtype,
                                     const float* inv_freq, const void* cs_table, const int* positions, const int* kv_slot,
                                     void* q_out, void* k_out, void* cache, int cache_dtype,
                                     int n_tokens, int QH, int KH, int d, int rot, int page_size, float eps,
                                     void* stream) {
    if (n_tokens <= 0) return 0;
    if (QH < 0 || KH < 0 || QH + KH <= 0 || d <= 0) RB_REFUSE("qknorm_rope_append: heads %d/%d head_dim %d", QH, KH, d);
    if (KH > 0 && !k_out && !cache) RB_REFUSE("qknorm_rope_append: neither a cache nor a k destination");
    if (rot < 0 || rot > d || (rot & 1)) RB_REFUSE("qknorm_rope_append: rotated width %d of head_dim %d", rot, d);
    if ((qw == nullptr) != (kw == nullptr)) RB_REFUSE("qknorm_rope_append: q and k norm weights come together");
    if (cache_dtype != act_dtype) RB_REFUSE("qknorm_rope_append: cache dtype %d differs from activations %d", cache_dtype, act_dtype);
    if (rot > 0 && (!inv_freq || !positions)) RB_REFUSE("qknorm_rope_append: rotation needs inv_freq and positions");
    cudaStream_t s = (cudaStream_t)stream;
    const long long warps = (long long)n_tokens * (QH + 2 * KH);
    const int blocks = rb_ceil_div(warps, 4);
    if (act_dtype == RB_BF16 && !k_out && cache && KH > 0 && rot == d && d % 128 == 0 && d <= 512 &&
        (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)cache) & 15) == 0) {
        if (n_tokens > 64 && d == 128) {                              // a prompt portion: a warp per token and group of heads
            const long long gw = (long long)n_tokens * (rb_ceil_div(QH, QG_HEADS) + 2 * rb_ceil_div(KH, QG_HEADS));
            const int gb = rb_ceil_div(gw, 4);
            if (w_dtype == RB_F32)
                return rb_launch(qknorm_rope_append_d128_kernel<float>, dim3(gb), dim3(128), 0, s, (const bf16*)qkv, (const float*)qw,
                                 (const float*)kw, inv_freq, (const float2*)cs_table, positions, kv_slot, (bf16*)q_out, (bf16*)cache,
                                 n_tokens, QH, KH, page_size, eps);
            return rb_launch(qknorm_rope_append_d128_kernel<bf16>, dim3(gb), dim3(128), 0, s, (const bf16*)qkv, (const bf16*)qw,
                             (const bf16*)kw, inv_freq, (const float2*)cs_table, positions, kv_slot, (bf16*)q_out, (bf16*)cache,
                             n_tokens, QH, KH, page_size, eps);
        }
        if (w_dtype == RB_F32)
            return rb_launch(qknorm_rope_append_vec_kernel<float>, dim3(blocks), dim3(128), 0, s, (const bf16*)qkv, (const float*)qw,
                             (const float*)kw, inv_freq, (const float2*)cs_table, positions, kv_slot, (bf16*)q_out, (bf16*)cache,
                             n_tokens, QH, KH, d, page_size, eps);
        return rb_launch(qknorm_rope_append_vec_kernel<bf16>, dim3(blocks), dim3(128), 0, s, (const bf16*)qkv, (const bf16*)qw,
                         (const bf16*)kw, inv_freq, (const float2*)cs_table, positions, kv_slot, (bf16*)q_out, (bf16*)cache,
                         n_tokens, QH, KH, d, page_size, eps);
    }
#define RB_QK(TA, TW) return rb_launch(qknorm_rope_append_kernel<TA, TW, TA>, dim3(blocks), dim3(128), 0, s, \
        (const TA*)qkv, (const TW*)qw, (const TW*)kw, inv_freq, positions, kv_slot, (TA*)q_out, (TA*)k_out, (TA*)cache, \
        n_tokens, QH, KH, d, rot, page_size, eps)
    if (act_dtype == RB_F32 && w_dtype == RB_F32) RB_QK(float, float);
    if (act_dtype == RB_F32 && w_dtype == RB_BF16) RB_QK(float, bf16);
    if (act_dtype == RB_BF16 && w_dtype == RB_F32) RB_QK(bf16, float);
    if (act_dtype == RB_BF16 && w_dtype == RB_BF16) RB_QK(bf16, bf16);
#undef RB_QK
    RB_REFUSE("qknorm_rope_append: dtypes act=%d weight=%d", act_dtype, w_dtype);
}

// Append given k [T,KH,d] (row stride k_stride elements) and v (row stride v_stride) to the cache
// (crates/cuda/kernels/dense_kernels.cu:302-318).  One warp per (token, kv head).
template <typename TA>
__global__ void kv_append_kernel(const TA* __restrict__ k, long long k_stride, const TA* __restrict__ v,
                                 long long v_stride, const int* __restrict__ kv_slot, TA* __restrict__ cache,
                                 int n_tokens, int KH, int d, int page_size) {
    pdl_trigger(); pdl_wait();
    const long long wglobal = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wglobal >= (long long)n_tokens * KH) return;
    const int t = (int)(wglobal / KH), kh = (int)(wglobal % KH);
    const int slot = kv_slot[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot % page_size;
    TA* kd = cache + ((((size_t)page * 2 + 0) * KH + kh) * page_size + off) * d;
    TA* vd = cache + ((((size_t)page * 2 + 1) * KH + kh) * page_size + off) * d;
    const TA* ks = k + (size_t)t * k_stride + (size_t)kh * d;
    const TA* vs = v + (size_t)t * v_stride + (size_t)kh * d;
    for (int i = lane; i < d; i += 32) { kd[i] = ks[i]; vd[i] = vs[i]; }
}
extern "C" int rb_kv_append(const void* k, long long k_stride, const void* v, long long v_stride,
                            const int* kv_slot, void* cache, int dtype, int n_tokens, int KH, int d,
                            int page_size, void* stream) {
    if (n_tokens <= 0) return 0;
    if (KH <= 0 || d <= 0 || page_size <= 0) RB_REFUSE("kv_append: kv heads %d head_dim %d page %d", KH, d, page_size);
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = rb_ceil_div((long long)n_tokens * KH, 4);
    if (dtype == RB_F32) kv_append_kernel<float><<<blocks, 128, 0, s>>>((const float*)k, k_stride, (const float*)v, v_stride, kv_slot, (float*)cache, n_tokens, KH, d, page_size);
    else if (dtype == RB_BF16) kv_append_kernel<bf16><<<blocks, 128, 0, s>>>((const bf16*)k, k_stride, (const bf16*)v, v_stride, kv_slot, (bf16*)cache, n_tokens, KH, d, page_size);
    else RB_REFUSE("kv_append: dtype %d", dtype);
    return RB_LAUNCH_RESULT();
}

// ------------------------------------------------------------------- SwiGLU
// out[t,f] = g/(1+exp(-g)) * u,  g = gu[t,f], u = gu[t,F+f]   (dense_kernels.cu:202-214)
template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int F, size_t total) {
    pdl_trigger(); pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / F;
    const int f = (int)(i % F);
    const float g = to_f32(gu[t * 2 * F + f]);
    const float u = to_f32(gu[t * 2 * F + F + f]);
    out[i] = from_f32<TA>(g / (1.0f + expf(-g)) * u);
}
extern "C" int rb_swiglu(const void* gu, void* out, int dtype, int n_tokens, int F, void* stream) {
    if (n_tokens <= 0) return 0;
    if (F <= 0) RB_REFUSE("swiglu: width %d", F);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)n_tokens * F;
    const int blocks = rb_ceil_div((long long)total, 256);
    if (dtype == RB_F32) return rb_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, F, total);
    if (dtype == RB_BF16) return rb_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, F, total);
    RB_REFUSE("swiglu: dtype %d", dtype);
}

RB_TL_SETTER(rb_elementwise_step_timeline)
