// Column sum of a bf16 matrix for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of this library whose
// code runs where cudaMalloc is off limits: inside a memory pool that someone else owns (an
// inference server that hands out fixed arenas), in a real-time control loop that may not take the
// driver's allocation locks, or in a plug-in whose host forbids allocations after start-up. The
// regular entry point (the torch binding `column_sum`) allocates an fp32 accumulator and its output
// through torch on every call; this one uses a fixed scratch array that lives inside the library.
//
// Contract
//   * The caller passes the input and the output; nothing is allocated or freed, by the CUDA
//     runtime or by any library, at any call.
//   * The fp32 scratch is a file-scope device array of WX_NOALLOC_MAX_COLS floats (256 KB). Every
//     GPU that loads the library holds that array until the process exits.
//   * `cols` above WX_NOALLOC_MAX_COLS is refused with WX_NOALLOC_ERR_TOO_WIDE; nothing is launched.
//   * The first call on a device looks up the scratch array's device address (once per device,
//     with that device current). Make that first call before any stream capture begins.
//   * Row slices are added into the scratch with float atomics, so the last bits of a sum can differ
//     from run to run (the regular entry point reduces in a fixed order and is bit-reproducible).
//   * All calls share the one scratch array and it keeps the last call's contents, so every call
//     starts by clearing the part it uses. Two calls that overlap on the GPU (different streams,
//     or different host threads) race on it: serialise them.
#pragma once
#include <cuda_runtime.h>

#define WX_NOALLOC_MAX_COLS 65536

#define WX_NOALLOC_OK 0
#define WX_NOALLOC_ERR_BAD_ARG (-1)    // null pointer, negative size, ld < cols, or input not 4-byte aligned
#define WX_NOALLOC_ERR_TOO_WIDE (-2)   // cols > WX_NOALLOC_MAX_COLS
#define WX_NOALLOC_ERR_SETUP (-3)      // the scratch address could not be resolved on this device
// Positive return values are cudaError_t codes from the launches.

#ifdef __cplusplus
extern "C" {
#endif

// out[c] = sum_r x[r, c], accumulated in fp32, written as bf16.
//   x    device pointer, bf16, `rows` x `cols`, row pitch `ld` elements (ld >= cols)
//   out  device pointer, bf16, `cols` elements
// Runs on `stream`; the device that owns `x` must be current.
int wx_column_sum_bf16_noalloc(const void* x, long ld, void* out, int rows, int cols, cudaStream_t stream);

// Human-readable text for a return value of the function above.
const char* wx_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
