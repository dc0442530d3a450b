// Random tensors from a counter: element i is a fixed function of (base, i), the same one that
// reinfer_b200/weights/random.py evaluates on the CPU.  mix() and GOLDEN are SplitMix64's
// (the reference's crates/scheduler/src/rng.rs:12-30).
//
//   a, b   = mix(base + (2i+1) GOLDEN), mix(base + (2i+2) GOLDEN)
//   u1, u2 = ((a >> 11) + 1) * 2^-53,  (b >> 11) * 2^-53
//   value  = float32(mean + std * sqrt(-2 ln u1) * cos(2 pi u2))      in float64, no fused multiply-add,
//            then rounded to the tensor's dtype (nearest even)
//   integer tables: a >> 49
#include "common.cuh"

#define RB_GOLDEN 0x9E3779B97F4A7C15ull

__device__ __forceinline__ unsigned long long rnd_mix(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long long n, unsigned long long base, double mean, double std) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned long long k = base + 2ull * (unsigned long long)i * RB_GOLDEN;
        const unsigned long long a = rnd_mix(k + RB_GOLDEN), b = rnd_mix(k + 2ull * RB_GOLDEN);
        const double u1 = __dmul_rn((double)((a >> 11) + 1ull), 0x1p-53);
        const double u2 = __dmul_rn((double)(b >> 11), 0x1p-53);
        const double r = sqrt(__dmul_rn(-2.0, log(u1)));
        const double x = __dmul_rn(r, cos(__dmul_rn(6.283185307179586, u2)));
        const double v = __dadd_rn(__dmul_rn(x, std), mean);
        out[i] = from_f32<T>(__double2float_rn(v));
    }
}

__global__ void random_ints_kernel(int* __restrict__ out, long long n, unsigned long long base) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned long long a = rnd_mix(base + (2ull * (unsigned long long)i + 1ull) * RB_GOLDEN);
        out[i] = (int)(a >> 49);
    }
}

extern "C" int rb_random_normal(void* out, int dtype, long long n, unsigned long long base, double mean, double std,
                                void* stream) {
    if (n <= 0) return 0;
    if (dtype != RB_F32 && dtype != RB_BF16) RB_REFUSE("random_normal: dtype %d", dtype);
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    const int grid = (int)(blocks < 148 * 16 ? blocks : 148 * 16);
    if (dtype == RB_F32)
        random_normal_kernel<float><<<grid, threads, 0, (cudaStream_t)stream>>>((float*)out, n, base, mean, std);
    else
        random_normal_kernel<bf16><<<grid, threads, 0, (cudaStream_t)stream>>>((bf16*)out, n, base, mean, std);
    return RB_LAUNCH_RESULT();
}

extern "C" int rb_random_ints(int* out, long long n, unsigned long long base, void* stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    const int grid = (int)(blocks < 148 * 16 ? blocks : 148 * 16);
    random_ints_kernel<<<grid, threads, 0, (cudaStream_t)stream>>>(out, n, base);
    return RB_LAUNCH_RESULT();
}
