// Row-wise kernels: embedding gather, RMSNorm with the residual sum fused in,
// per-head q/k RMSNorm + rotary encoding + append to the paged cache, SwiGLU.
// All arithmetic is 32-bit; only loads and stores see the storage type.
// The residual stream is float in both precisions of the model.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// x[t,:] = E[ids[t],:]   (reference: crates/cuda/kernels/dense_kernels.cu:329-336)
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int h, int vocab) {
    pdl_trigger(); pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    const bool ok = (id >= 0 && id < vocab);          // the host refuses such ids before launching
    const TW* row = table + (size_t)(ok ? id : 0) * h;
    float* o = out + (size_t)t * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) o[i] = ok ? to_f32(row[i]) : 0.0f;
}

extern "C" int rb_embed_gather(const void* table, int table_dtype, const int* ids, float* out,
                               int n_tokens, int h, int vocab, void* stream) {
    if (n_tokens <= 0) return 0;
    if (h <= 0 || vocab <= 0) RB_REFUSE("embed_gather: hidden=%d vocab=%d", h, vocab);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = h >= 1024 ? 256 : 128;
    if (table_dtype == RB_F32)
        return rb_launch(embed_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)table, ids, out, h, vocab);
    if (table_dtype == RB_BF16)
        return rb_launch(embed_gather_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, (const bf16*)table, ids, out, h, vocab);
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
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                   const TW* __restrict__ w, TO* __restrict__ out,
                                   const int* __restrict__ row_idx, int h, float eps) {
    __shared__ float red[32];
    pdl_trigger(); pdl_wait();
    const int r = blockIdx.x;
    const size_t in_row = row_idx ? (size_t)row_idx[r] : (size_t)r;
    float* xr = x + in_row * h;
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
                if (delta) { t += to_f32(delta[in_row * h + i]); xr[i] = t; }
            }
            v[k] = t;
            ss += t * t;
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            float t = xr[i];
            if (delta) { t += to_f32(delta[in_row * h + i]); xr[i] = t; }
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
            if (i < h) orow[i] = from_f32<TO>(v[k] * rstd * to_f32(w[i]));
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x)
            orow[i] = from_f32<TO>(xr[i] * rstd * to_f32(w[i]));
    }
}

template <typename TD, typename TW, typename TO>
static int launch_add_rmsnorm_k(float* x, const TD* delta, const TW* w, TO* out, const int* row_idx, int rows, int h,
                                float eps, cudaStream_t s) {
    // the summation order (thread stride, then the block tree) depends on h only, never on the batch
    if (h <= 512) return rb_launch(add_rmsnorm_kernel<TD, TW, TO, 4>, dim3(rows), dim3(128), 0, s, x, delta, w, out, row_idx, h, eps);
    if (h <= 2048) return rb_launch(add_rmsnorm_kernel<TD, TW, TO, 8>, dim3(rows), dim3(256), 0, s, x, delta, w, out, row_idx, h, eps);
    if (h <= 8192) return rb_launch(add_rmsnorm_kernel<TD, TW, TO, 8>, dim3(rows), dim3(1024), 0, s, x, delta, w, out, row_idx, h, eps);
    return rb_launch(add_rmsnorm_kernel<TD, TW, TO, 0>, dim3(rows), dim3(1024), 0, s, x, delta, w, out, row_idx, h, eps);
}

template <typename TD, typename TW>
static int launch_add_rmsnorm_o(float* x, const void* delta, const void* w, void* out, int out_dtype,
                                const int* row_idx, int rows, int h, float eps, cudaStream_t s) {
    if (out_dtype == RB_F32)
        return launch_add_rmsnorm_k<TD, TW, float>(x, (const TD*)delta, (const TW*)w, (float*)out, row_idx, rows, h, eps, s);
    if (out_dtype == RB_BF16)
        return launch_add_rmsnorm_k<TD, TW, bf16>(x, (const TD*)delta, (const TW*)w, (bf16*)out, row_idx, rows, h, eps, s);
    RB_REFUSE("rmsnorm: out dtype %d", out_dtype);
}

extern "C" int rb_add_rmsnorm(float* x, const void* delta, int delta_dtype, const void* w, int w_dtype,
                              void* out, int out_dtype, const int* row_idx, int rows, int h, float eps,
                              void* stream) {
    if (rows <= 0) return 0;
    if (h <= 0) RB_REFUSE("rmsnorm: width %d", h);
    if (delta && row_idx) RB_REFUSE("rmsnorm: a residual sum cannot be combined with a row gather");
    cudaStream_t s = (cudaStream_t)stream;
    const int dd = delta ? delta_dtype : RB_F32;
    if (dd == RB_F32 && w_dtype == RB_F32) return launch_add_rmsnorm_o<float, float>(x, delta, w, out, out_dtype, row_idx, rows, h, eps, s);
    if (dd == RB_F32 && w_dtype == RB_BF16) return launch_add_rmsnorm_o<float, bf16>(x, delta, w, out, out_dtype, row_idx, rows, h, eps, s);
    if (dd == RB_BF16 && w_dtype == RB_F32) return launch_add_rmsnorm_o<bf16, float>(x, delta, w, out, out_dtype, row_idx, rows, h, eps, s);
    if (dd == RB_BF16 && w_dtype == RB_BF16) return launch_add_rmsnorm_o<bf16, bf16>(x, delta, w, out, out_dtype, row_idx, rows, h, eps, s);
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
// multiple of 64 - with 4-byte loads and stores (a lane owns element pairs 2l, 2l+1 of both halves) and 16-byte
// copies of the value rows; cosines and sines come from the step's table when one is given.
template <typename TW>
__global__ void qknorm_rope_append_vec_kernel(const bf16* __restrict__ qkv, const TW* __restrict__ qw, const TW* __restrict__ kw,
                                              const float* __restrict__ inv_freq, const float2* __restrict__ cs_table,
                                              const int* __restrict__ positions, const int* __restrict__ kv_slot,
                                              bf16* __restrict__ q_out, bf16* __restrict__ cache,
                                              int n_tokens, int QH, int KH, int d, int page_size, float eps) {
    pdl_trigger(); pdl_wait();
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
    float a0[4], a1[4], b0[4], b1[4];                         // head_dim <= 512
    float ss = 0.0f;
    const int n_it = half / 64;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (i < n_it) {
            const int p = 2 * lane + 64 * i;
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + p));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + p + half));
            a0[i] = lo.x; a1[i] = lo.y; b0[i] = hi.x; b1[i] = hi.y;
            ss += lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y;
        }
    }
    float rstd = 1.0f;
    if (w) {
        ss = warp_sum(ss);
        rstd = 1.0f / sqrtf(ss / (float)d + eps);
    }
    const float pos = (float)positions[t];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (i < n_it) {
            const int p = 2 * lane + 64 * i;
            float x0 = a0[i], x1 = a1[i], y0 = b0[i], y1 = b1[i];
            if (w) {
                x0 = x0 * rstd * to_f32(w[p]); x1 = x1 * rstd * to_f32(w[p + 1]);
                y0 = y0 * rstd * to_f32(w[p + half]); y1 = y1 * rstd * to_f32(w[p + half + 1]);
            }
            float c0, s0, c1, s1;
            if (cs_table) {
                const float4 v = *reinterpret_cast<const float4*>(cs_table + (size_t)t * half + p);
                c0 = v.x; s0 = v.y; c1 = v.z; s1 = v.w;
            } else {
                sincosf(pos * inv_freq[p], &s0, &c0);
                sincosf(pos * inv_freq[p + 1], &s1, &c1);
            }
            *reinterpret_cast<__nv_bfloat162*>(dst + p) = __floats2bfloat162_rn(x0 * c0 - y0 * s0, x1 * c1 - y1 * s1);
            *reinterpret_cast<__nv_bfloat162*>(dst + p + half) = __floats2bfloat162_rn(x0 * s0 + y0 * c0, x1 * s1 + y1 * c1);
        }
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
    if (act_dtype == RB_BF16 && !k_out && cache && KH > 0 && rot == d && d % 64 == 0 && d <= 512 &&
        (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)cache) & 15) == 0) {
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
