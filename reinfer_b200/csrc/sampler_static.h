/* rb_sample_static: the GPU sampler for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference (LeonRust/reinfer allocates its
 * sampler's device buffers when the sampler is built); it exists for users of this library.
 *
 * Who needs it.  The ordinary entry point, rb_sample, asks its caller for a scratch buffer of
 * rows x vocab floats in device memory.  Some callers have no way to get one at the moment
 * they want a token: code that runs between the kernels of a latency-critical loop, where
 * cudaMalloc would stall the whole device while it maps memory; a plug-in inside another
 * program that owns every byte of the GPU through its own pool and hands none out.  For them
 * the scratch lives inside the library: one array in device memory, of fixed size, that every
 * GPU holds from the moment it loads the library until the process exits.
 *
 * It is an ordinary host function all the same: it makes CUDA runtime calls (cudaGetDevice, a
 * kernel launch, and cudaGetSymbolAddress at the first call on a device), and that first call takes
 * a mutex.  So it is not for a cudaLaunchHostFunc callback or a signal handler, where runtime
 * calls are not allowed at all.  After the first call on a device the address is read with one
 * atomic load and no lock is taken.
 *
 * Limits.  rows * vocab <= RB_SAMPLE_STATIC_FLOATS (2,097,152 floats = 8 MiB per GPU): for
 * example 8 rows of a 262,144-entry vocabulary or 13 rows of Qwen3's 151,936.  Anything larger
 * is refused with an error (return value -1, text from rb_last_error()); nothing is launched.
 *
 * What it does not do.  It calls no cudaMalloc, cudaFree or other allocating routine, neither
 * of CUDA nor of any library.  The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) and remembers it; make that first call on each device outside any
 * stream capture.  Later calls only launch the kernel.
 *
 * Sharing.  All calls on a device use the same array.  It keeps whatever the last call left
 * there; the sampler rewrites every element of a row before it reads it, so nothing has to be
 * cleared between calls.  Two calls whose kernels may run at the same time on one GPU (other
 * streams, other host threads) would overwrite each other's rows: run them in one stream, or
 * wait for the first before launching the second.
 *
 * Arguments and result are those of rb_sample without the scratch pointer:
 *   logits      [*, ld_logits] float32 in device memory
 *   row_idx     [rows] which logits row each output row reads, or NULL for 0..rows-1
 *   params      [rows] RbSampleParams records (see sampler.cu) in device memory
 *   history     [rows, hist_cap] recent token ids for the penalties, or NULL
 *   out_tokens  [rows] int32 in device memory; -1 for a row without a finite logit
 * Returns 0, -1 for a refused argument, or the positive cudaError_t of the launch or look-up.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define RB_SAMPLE_STATIC_FLOATS (2u << 20)

int rb_sample_static(const float* logits, long long ld_logits, const int* row_idx, const void* params,
                     const int* history, int hist_cap, int* out_tokens, int rows, int vocab, void* stream);

#ifdef __cplusplus
}
#endif
