// A wait that is meant to run out, for tests of the error path: one CTA initialises an mbarrier that nobody
// ever arrives at and waits on it through the same bounded wait as the product kernels (mbar_wait_ns of
// sm100.cuh), with the limit taken from the argument.  The wait gives up, the error word of this unit and the
// host's status word receive (4 << 16 | 1 << 8 | 77), and the kernel returns; the context stays usable.  It uses
// no TMA, no tensor memory and no cluster.  The reference turns the same condition into
// EngineError::BarrierTimeout / SyncTimeout (crates/cuda/src/engine.rs:3697-3737, 3849-3897).
#define RB_UNIT 4
#include "sm100.cuh"

#define RB_SELFTEST_WHERE 77

__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns, int* gave_up) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait_ns(smem_u32(&bar), 0, &abort_flag, RB_SELFTEST_WHERE, limit_ns);
        if (gave_up) *gave_up = ok ? 0 : 1;
    }
}

// limit_ns: how long the wait may last (at most one second is accepted); gave_up: one int in device memory that
// receives 1 when the wait ran out (may be NULL).
extern "C" int rb_test_bounded_wait(unsigned long long limit_ns, int* gave_up, void* stream) {
    if (limit_ns == 0 || limit_ns > 1000000000ull) RB_REFUSE("test_bounded_wait: limit of %llu ns (1 .. 1e9)", limit_ns);
    bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit_ns, gave_up);
    return RB_LAUNCH_RESULT();
}

RB_STATUS_EXPORTS(rb_selftest_error, rb_selftest_bind_status)
