// Token choice on the GPU, one thread block per row of logits, any number of rows
// per launch.  Chain and meanings follow the reference's sampler
// (crates/cuda/kernels/sampler_kernel.cu:20-24, 157-397):
//   repetition / frequency / presence penalties over the request's recent tokens
//   -> temperature (divide) -> min_p -> top_k -> top_p -> Gumbel-max draw,
// and temperature <= 0 means greedy with no random number consumed.
// Differences, on purpose: a tie of the maximum goes to the FIRST (smallest) id
// everywhere (the reference's engine takes the first, its sampler kernel the last,
// engine.rs:6512-6520 vs sampler_kernel.cu:4-11); rows are independent blocks instead
// of one block per launch.
//
// The draw is a pure function of (seed, step, token id): noise(v) = -ln(-ln(u)),
// u = top 24 bits of mix(base ^ mix(v)), base = the step-th output of a SplitMix64
// stream started at `seed` (sampler_kernel.cu:61-77; crates/scheduler/src/rng.rs:12-50).
// So a request's tokens do not depend on what else is in the batch.
//
// The penalised, temperature-scaled logits of a row live in a scratch row `work`
// ([rows, vocab] floats, given by the caller); the logits themselves are not changed.
// Non-finite logits never win (stored as -FLT_MAX); a row without any finite logit
// gives token -1.
#include "common.cuh"
#include <float.h>

#define SP_THREADS 1024

struct RbSampleParams {          // one per row; mirrored by ctypes in sampling/sampler.py
    float temperature;           // <= 0: greedy
    int top_k;                   // <= 0 or >= vocab: off
    float top_p;                 // <= 0 or >= 1: off
    float min_p;                 // <= 0: off
    float repeat_penalty;        // <= 1: off      l > 0 ? l / r : l * r
    float frequency_penalty;     // l -= count * f
    float presence_penalty;      // l -= p (once, if the token occurred)
    int hist_len;                // valid entries of this row's history (<= hist_cap)
    unsigned long long seed;
    unsigned long long step;     // index of this draw in the request's stream
    const int2* bias;            // bias_len pairs (token id, float bits): added to the logits first of all
    int bias_len;
    int hist_window;             // slot records only: the history is a ring of this many tokens (0: none is kept)
};

__device__ __forceinline__ unsigned long long sp_mix(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float sp_gumbel(unsigned long long base, unsigned v) {
    const float u = (float)(sp_mix(base ^ sp_mix((unsigned long long)v)) >> 40) * (1.0f / 16777216.0f);
    return -logf(-logf(u));                                   // u == 0 -> -inf: never wins
}
// larger key = larger value; equal values: smaller id first (sampler_kernel.cu:88-93)
__device__ __forceinline__ unsigned long long sp_key(float val, unsigned id) {
    const unsigned bits = __float_as_uint(val);
    const unsigned asc = (bits >> 31) ? ~bits : (bits ^ 0x80000000u);
    return ((unsigned long long)asc << 32) | (0xFFFFFFFFu - id);
}

// best (value, smallest id) over the block; all threads get the result
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sval, int* sidx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sval[wid] = v; sidx[wid] = idx; }
    __syncthreads();
    float rv = sval[lane]; int ri = sidx[lane];               // SP_THREADS / 32 == 32 warps
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, rv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, ri, o);
        if (ov > rv || (ov == rv && oi < ri)) { rv = ov; ri = oi; }
    }
    v = rv; idx = ri;
}
__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    unsigned long long r = red[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

// One row: the token for logits `lg` under the record P, with `hist` the recent tokens (P.hist_len of them, in
// any order) and `w` a scratch row of vocab floats.  Every thread of the block returns the same token (-1: no
// finite logit).
__device__ int sample_row(const float* __restrict__ lg, const RbSampleParams& P, const int* __restrict__ hist,
                          float* __restrict__ w, int vocab) {
    __shared__ float sval[32];
    __shared__ int sidx[32];
    __shared__ float red[32];
    __shared__ unsigned long long red64[32];
    const int tid = threadIdx.x;

    const bool penalties = P.hist_len > 0 &&
        (P.repeat_penalty > 1.0f || P.frequency_penalty != 0.0f || P.presence_penalty != 0.0f);
    const bool greedy = !(P.temperature > 0.0f);
    const bool biased = P.bias_len > 0 && P.bias != nullptr;

    if (greedy && !penalties && !biased) {                     // no scratch needed
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int i = tid; i < vocab; i += SP_THREADS) {
            const float v = lg[i];
            if (isfinite(v) && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
        }
        block_argmax(bv, bi, sval, sidx);
        return (bi == 0x7fffffff) ? -1 : bi;
    }

    for (int i = tid; i < vocab; i += SP_THREADS) {
        const float v = lg[i];
        w[i] = isfinite(v) ? v : -FLT_MAX;
    }
    __syncthreads();
    if (biased) {
        // logit_bias comes first in the chain (sampler_kernel.cu:20-24,198-205); ids are distinct, one thread each
        for (int j = tid; j < P.bias_len; j += SP_THREADS) {
            const int2 b = P.bias[j];
            if (b.x >= 0 && b.x < vocab && w[b.x] != -FLT_MAX) w[b.x] += __int_as_float(b.y);
        }
        __syncthreads();
    }
    if (penalties) {
        // one thread per history entry; the first occurrence of a token applies the penalty
        for (int j = tid; j < P.hist_len; j += SP_THREADS) {
            const int tok = hist[j];
            if (tok < 0 || tok >= vocab) continue;
            int count = 0; bool first = true;
            for (int k = 0; k < P.hist_len; ++k) {
                if (hist[k] == tok) { ++count; if (k < j) first = false; }
            }
            if (!first) continue;
            float l = w[tok];
            if (l == -FLT_MAX) continue;
            l -= (float)count * P.frequency_penalty + P.presence_penalty;        // sampler_kernel.cu:213-215
            if (P.repeat_penalty > 1.0f) l = l > 0.0f ? l / P.repeat_penalty : l * P.repeat_penalty;  // :207-218
            w[tok] = l;
        }
        __syncthreads();
    }
    if (greedy) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int i = tid; i < vocab; i += SP_THREADS) {
            const float v = w[i];
            if (v != -FLT_MAX && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
        }
        block_argmax(bv, bi, sval, sidx);
        return (bi == 0x7fffffff) ? -1 : bi;
    }

    // temperature, maximum
    const float inv_t = 1.0f / P.temperature;
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += SP_THREADS) {
        float v = w[i];
        if (v != -FLT_MAX) { v *= inv_t; w[i] = v; mx = fmaxf(mx, v); }
    }
    mx = block_max(mx, red);
    if (!(mx > -INFINITY)) return -1;
    __syncthreads();

    // survivors are {i : key(i) >= key_floor and w[i] >= val_floor}
    float val_floor = -FLT_MAX * 0.5f;                         // above the -FLT_MAX sentinel
    if (P.min_p > 0.0f) val_floor = fmaxf(val_floor, mx + logf(P.min_p));     // prob >= max_prob * min_p
    unsigned long long key_floor = 0ull;
    if (P.top_k > 0 && P.top_k < vocab) {
        // largest tau with count(key >= tau) >= k, by bisection over the 64 key bits
        unsigned long long tau = 0ull;
        for (int bit = 63; bit >= 0; --bit) {
            const unsigned long long cand = tau | (1ull << bit);
            unsigned long long c = 0;
            for (int i = tid; i < vocab; i += SP_THREADS) {
                const float v = w[i];
                c += (v >= val_floor && sp_key(v, (unsigned)i) >= cand) ? 1ull : 0ull;
            }
            c = block_sum_u64(c, red64);
            if (c >= (unsigned long long)P.top_k) tau = cand;
        }
        key_floor = tau;
    }
    float e_floor = 0.0f;                                      // survivors also need exp(w - mx) >= e_floor
    if (P.top_p > 0.0f && P.top_p < 1.0f) {
        // mass of the survivors, then the largest theta with sum_{e >= theta} e >= p * mass,
        // by bisection over the bits of the (positive) float e = exp(w - mx); a tie at the
        // boundary keeps its whole group (sampler_kernel.cu:320-362)
        float zs = 0.0f;
        for (int i = tid; i < vocab; i += SP_THREADS) {
            const float v = w[i];
            if (v >= val_floor && sp_key(v, (unsigned)i) >= key_floor) zs += expf(v - mx);
        }
        zs = block_sum(zs, red);
        const float target = P.top_p * zs;
        unsigned theta = 0u;
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned cand = theta | (1u << bit);
            const float th = __uint_as_float(cand);
            float acc = 0.0f;
            for (int i = tid; i < vocab; i += SP_THREADS) {
                const float v = w[i];
                if (v >= val_floor && sp_key(v, (unsigned)i) >= key_floor) {
                    const float e = expf(v - mx);
                    if (e >= th) acc += e;
                }
            }
            acc = block_sum(acc, red);
            if (acc >= target) theta = cand;
        }
        e_floor = __uint_as_float(theta);
    }
    const unsigned long long stream = sp_mix(P.seed + (P.step + 1ull) * 0x9E3779B97F4A7C15ull);
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += SP_THREADS) {
        const float v = w[i];
        if (v >= val_floor && sp_key(v, (unsigned)i) >= key_floor && expf(v - mx) >= e_floor) {
            const float g = v + sp_gumbel(stream, (unsigned)i);
            if (g > bv || (g == bv && i < bi)) { bv = g; bi = i; }
        }
    }
    block_argmax(bv, bi, sval, sidx);
    if (bi == 0x7fffffff) {                                   // every survivor drew u == 0: take the mode
        bv = -INFINITY;
        for (int i = tid; i < vocab; i += SP_THREADS) {
            const float v = w[i];
            if (v != -FLT_MAX && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
        }
        block_argmax(bv, bi, sval, sidx);
    }
    return (bi == 0x7fffffff) ? -1 : bi;
}

__global__ void __launch_bounds__(SP_THREADS)
sample_kernel(const float* __restrict__ logits, long long ld_logits, const int* __restrict__ row_idx,
              const RbSampleParams* __restrict__ params, const int* __restrict__ history, int hist_cap,
              float* __restrict__ work, int* __restrict__ out_tokens, int vocab) {
    const int r = blockIdx.x;
    const RbSampleParams P = params[r];
    const float* lg = logits + (size_t)(row_idx ? row_idx[r] : r) * ld_logits;
    const int tok = sample_row(lg, P, history + (size_t)r * hist_cap, work + (size_t)r * vocab, vocab);
    if (threadIdx.x == 0) out_tokens[r] = tok;
}

// The same choice with everything about the request taken from its slot on the device: row r of the logits belongs
// to the request in slot row_slot[r]; its record (parameters, seed, count of draws so far) and its ring of recent
// tokens are rows of the slot tables.  The kernel writes the token into the slot (where the next step's embedding
// finds it), appends it to the ring, counts the draw, and reports the token in out_tokens[r] for the host.  The
// host writes a slot's record when the request is admitted and never again, so a decode step needs no upload for
// its sampler and the launch can live in a captured graph.  Two rows of one launch must not name the same slot
// (but for the slot that belongs to nobody, which rows of padding share: what they leave there is never read).
__global__ void __launch_bounds__(SP_THREADS)
sample_slots_kernel(const float* __restrict__ logits, long long ld_logits, const int* __restrict__ row_slot,
                    RbSampleParams* __restrict__ slot_params, int* __restrict__ slot_history, int hist_cap,
                    int* __restrict__ slot_token, float* __restrict__ work, int* __restrict__ out_tokens, int vocab) {
    pdl_trigger(); pdl_wait();
    const int r = blockIdx.x;
    const int s = row_slot[r];
    const RbSampleParams P = slot_params[s];
    int* hist = slot_history + (size_t)s * hist_cap;
    const int tok = sample_row(logits + (size_t)r * ld_logits, P, hist, work + (size_t)r * vocab, vocab);
    __syncthreads();                                        // every thread has read the ring before it changes
    if (threadIdx.x == 0) {
        out_tokens[r] = tok;
        slot_token[s] = tok;
        slot_params[s].step = P.step + 1ull;
        const int window = P.hist_window < hist_cap ? P.hist_window : hist_cap;
        if (window > 0 && tok >= 0) {
            hist[(int)(P.step % (unsigned long long)window)] = tok;      // the n-th draw lives at n mod window
            if (P.hist_len < window) slot_params[s].hist_len = P.hist_len + 1;
        }
    }
}

// logits [*, ld_logits] floats; row r of the launch reads logits row row_idx[r] (or r);
// params [rows]; history [rows, hist_cap] recent tokens of each row's request;
// work [rows, vocab] floats of scratch; out_tokens [rows].
extern "C" int rb_sample(const float* logits, long long ld_logits, const int* row_idx, const void* params,
                         const int* history, int hist_cap, float* work, int* out_tokens,
                         int rows, int vocab, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) RB_REFUSE("sample: vocab %d", vocab);
    if (!work) RB_REFUSE("sample: the scratch rows are missing");
    sample_kernel<<<rows, SP_THREADS, 0, (cudaStream_t)stream>>>(
        logits, ld_logits, row_idx, (const RbSampleParams*)params, history, hist_cap, work, out_tokens, vocab);
    return RB_LAUNCH_RESULT();
}

// logits [rows, ld_logits] floats; row_slot [rows]; slot_params [slots] records; slot_history [slots, hist_cap];
// slot_token [slots]; work [rows, vocab] floats of scratch; out_tokens [rows].
extern "C" int rb_sample_slots(const float* logits, long long ld_logits, const int* row_slot, void* slot_params,
                               int* slot_history, int hist_cap, int* slot_token, float* work, int* out_tokens,
                               int rows, int vocab, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || hist_cap <= 0) RB_REFUSE("sample_slots: vocab %d, history of %d", vocab, hist_cap);
    if (!row_slot || !slot_params || !slot_history || !slot_token || !work || !out_tokens)
        RB_REFUSE("sample_slots: a table is missing");
    return rb_launch(sample_slots_kernel, dim3(rows), dim3(SP_THREADS), 0, (cudaStream_t)stream, logits, ld_logits, row_slot,
                     (RbSampleParams*)slot_params, slot_history, hist_cap, slot_token, work, out_tokens, vocab);
}

extern "C" int rb_sample_params_size() { return (int)sizeof(RbSampleParams); }

// ------------------------------------------------------------------------------------------
// The sampler for callers that must not allocate (declared and described in sampler_static.h).
// Its scratch rows are this file-scope array in device memory.  In host code the array's name
// is only a handle; its device address comes from cudaGetSymbolAddress, looked up once per
// device with that device current, and it is that address the kernel receives.
#include "sampler_static.h"
#include <atomic>
#include <mutex>

static __device__ __align__(256) float g_sample_static_scratch[RB_SAMPLE_STATIC_FLOATS];

#define RB_SAMPLE_STATIC_MAX_DEVICES 64
static std::atomic<float*> g_sample_static_addr[RB_SAMPLE_STATIC_MAX_DEVICES];     // zero-initialised: not looked up yet
static std::mutex g_sample_static_mu;                                              // taken by a device's first call only

extern "C" int rb_sample_static(const float* logits, long long ld_logits, const int* row_idx, const void* params,
                                const int* history, int hist_cap, int* out_tokens, int rows, int vocab, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) RB_REFUSE("sample_static: vocab %d", vocab);
    if ((unsigned long long)rows * (unsigned long long)vocab > (unsigned long long)RB_SAMPLE_STATIC_FLOATS)
        RB_REFUSE("sample_static: %d rows x %d entries need %llu floats of scratch; the built-in array holds %u "
                  "(use rb_sample with a buffer of your own)", rows, vocab,
                  (unsigned long long)rows * (unsigned long long)vocab, (unsigned)RB_SAMPLE_STATIC_FLOATS);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= RB_SAMPLE_STATIC_MAX_DEVICES) RB_REFUSE("sample_static: device index %d", dev);
    float* scratch = g_sample_static_addr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {                                   // first call on this device: look the address up
        std::lock_guard<std::mutex> g(g_sample_static_mu);
        scratch = g_sample_static_addr[dev].load(std::memory_order_relaxed);
        if (scratch == nullptr) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_sample_static_scratch);
            if (e != cudaSuccess) return (int)e;
            scratch = (float*)p;
            g_sample_static_addr[dev].store(scratch, std::memory_order_release);
        }
    }
    sample_kernel<<<rows, SP_THREADS, 0, (cudaStream_t)stream>>>(
        logits, ld_logits, row_idx, (const RbSampleParams*)params, history, hist_cap, scratch, out_tokens, vocab);
    return RB_LAUNCH_RESULT();
}
