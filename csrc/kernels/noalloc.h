// C entry point for callers that are not allowed to allocate device memory.
//
// This has no counterpart in the reference extension.
//
// Who needs it: code that runs where cudaMalloc / cudaFree (or any allocating
// library call, torch's caching allocator included) is off limits -- for
// example a plugin called from inside someone else's stream-ordered pipeline
// that has handed out its whole memory budget up front, a real-time loop that
// may not take the allocator's locks or trigger its implicit device
// synchronisation, or a host process that loads this library through dlopen /
// ctypes and owns every buffer itself.  Such callers bring the input, the
// optional residual and the output buffer; the only other memory the TernGrad
// compressor needs is its small min/max reduction scratch, and that lives in
// a fixed device array inside this library (16 KB per GPU that loads the
// library, of which the reduction state uses about 8 KB; held until the process
// exits).
//
// Rules of use:
//  * The first call on each device looks up the device address of the built-in
//    scratch (the device must be current, which it is when its pointers are
//    passed).  Make that first call outside any stream capture.
//  * All calls on one device share the one scratch array.  Two calls whose
//    kernels may overlap on the GPU (different streams without an ordering
//    between them) race on it; order them, or use the allocating API, which
//    keeps one scratch per stream.
//  * n may not exceed HIPRESS_NOALLOC_MAX_ELEMS; out_bytes must be exactly
//    10 + ceil(n / (8 / bitwidth)).
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HIPRESS_NOALLOC_MAX_ELEMS 2147483647LL  /* payload sizes are 32-bit in the wire format */
#define HIPRESS_NOALLOC_SCRATCH_BYTES 16384     /* size of the built-in device scratch */

/* Return codes */
#define HIPRESS_OK 0
#define HIPRESS_ERR_ARGUMENT 1   /* null pointer, bad bitwidth, wrong out_bytes */
#define HIPRESS_ERR_TOO_LARGE 2  /* n > HIPRESS_NOALLOC_MAX_ELEMS */
#define HIPRESS_ERR_CUDA 3       /* a CUDA call failed; see hipress_noalloc_last_error() */

/* TernGrad-style min-max quantisation of `grad` (n floats, device memory) into
 * `out` (device memory, out_bytes bytes), same payload as the allocating
 * entry point.  `residual` may be NULL; when given it is added to the gradient
 * before quantisation and receives the quantisation error.  `stream` is a
 * cudaStream_t (NULL = default stream).  Allocates nothing. */
__attribute__((visibility("default")))
int hipress_terngrad_compress_noalloc(const float* grad, float* residual, long long n, int bitwidth,
                                      int enable_random, unsigned long long seed, unsigned char* out,
                                      long long out_bytes, void* stream);

/* Text of the last CUDA error seen by the function above in this thread. */
__attribute__((visibility("default")))
const char* hipress_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
