/* Allocation-free entry point of libb200llm.so.
 *
 * This function has no counterpart in the reference (tanbo24/Create-LLM-by-Cupy): there every
 * kernel gets its temporaries from CuPy's memory pool. It exists for callers that are not allowed
 * to allocate device memory at the moment they need the RMSNorm backward: a serving or training
 * loop that has handed the whole device to its own arena and treats any further cudaMalloc as a
 * bug, a real-time step that cannot afford cudaMalloc's implicit device synchronisation, or a
 * host thread that must not take the allocator lock.
 *
 * The regular entry point, b200_rmsnorm_bwd, needs a caller-provided fp32 scratch block for the
 * per-CTA partial sums of dgamma. This variant is the same computation with that scratch taken
 * from a fixed array compiled into the library:
 *
 *   - the array is B200_NOALLOC_RMS_ROWS x B200_NOALLOC_RMS_MAX_H floats (about 4.75 MiB); every
 *     GPU that loads the library holds it until the process exits;
 *   - hidden sizes above B200_NOALLOC_RMS_MAX_H are refused (cudaErrorInvalidValue and a message
 *     on stderr), as is a device with so many SMs that the partial rows would not fit;
 *   - the first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress, with that device current). Under lazy module loading that look-up may
 *     also be the moment the driver loads the module that holds the array, i.e. when the 4.75 MiB are
 *     actually taken from the device. Make that first call at start-up and outside of any stream
 *     capture; later calls on the same device do no set-up and change no memory accounting;
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine. Inputs and outputs are
 *     the caller's;
 *   - all calls on one device share the array and it keeps the previous call's contents. The
 *     function clears what has to start from zero itself, but two calls that overlap on the GPU
 *     (different streams, no ordering between them) race on it: serialise them.
 *
 * Arguments are those of b200_rmsnorm_bwd without `partial`:
 *   dy, x [M, H] bf16; gamma [H] bf16; rstd [M] fp32; add [M, H] bf16 or NULL (added to dx);
 *   dx [M, H] bf16 out; dgamma [H] bf16 out (+= when accumulate_dgamma != 0).
 * Returns 0 or a cudaError_t value.
 */
#pragma once
#include <cuda_runtime.h>

#define B200_NOALLOC_RMS_ROWS 304
#define B200_NOALLOC_RMS_MAX_H 4096

#ifdef __cplusplus
extern "C" {
#endif

int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const void* rstd, const void* add,
                             void* dx, void* dgamma, int M, int H, int accumulate_dgamma, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
