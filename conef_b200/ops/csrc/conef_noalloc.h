// Allocation-free LAMB step.
//
// This entry point has no counterpart in the reference project: it exists for
// callers of this library that are not allowed to allocate device memory at the
// point where they run the optimizer.  Typical cases are a training loop whose
// memory is handed out once by an external pool or arena (so a cudaMalloc in the
// middle of a step would bypass the pool's accounting or fail its budget), a host
// thread that must not take the allocator's locks, and embedders that link this
// library from plain C/C++ without PyTorch, where no caching allocator exists to
// provide the small scratch buffer that conef_lamb_step() expects from its caller.
//
// conef_lamb_step() needs 1 + 2 * ntensors floats of scratch for the squared
// norms it accumulates.  conef_lamb_step_noalloc() keeps that scratch in a fixed
// array inside the library (static device memory, CONEF_NOALLOC_MAX_TENSORS
// tensors at most, about 32 KB, resident on every GPU that loads the library
// until the process exits).  The caller still passes every input and output:
// the tensor table, the chunk table and the hyper-parameters, exactly as for
// conef_lamb_step().
//
// Rules of use
//   * ntensors > CONEF_NOALLOC_MAX_TENSORS is rejected (non-zero return code and
//     a message in conef_last_error()); nothing is launched in that case.
//   * The first call on a device looks up the device address of the scratch
//     array (cudaGetSymbolAddress, with that device current) and remembers it.
//     Make that first call outside of any CUDA stream capture.  Several host threads
//     may make it at once: each looks the address up and stores the same value.
//   * The function calls no cudaMalloc / cudaFree and no allocating library
//     routine.  It enqueues one memset and the same three kernels as
//     conef_lamb_step() on `stream`.
//   * All calls on a device share the one scratch array, which keeps the values
//     of the last call.  The part a call uses is cleared at its start; two calls
//     whose kernels can overlap on the GPU (different streams without ordering
//     between them) race on it and must be serialised by the caller.
#pragma once
#include "conef.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CONEF_NOALLOC_MAX_TENSORS 4096

int conef_lamb_step_noalloc(const ConefLambTensor* tensors, int ntensors, const int2* chunks, int nchunks,
                            int chunk_elems, float lr, float beta1, float beta2, float eps, int step,
                            int bias_correction, float grad_scale, float max_grad_norm,
                            cudaStream_t stream);

#ifdef __cplusplus
}
#endif
