// An entry point of the tensor-core product that allocates nothing.
//
// It has no counterpart in ktfth/smolmoe-c99 (a CPU program whose heap is a counted budget,
// src/util.h:81-89); it exists for callers of this library that cannot allocate device memory
// at the moment of the call: code that runs inside someone else's memory budget (a plug-in of
// a host application that owns the GPU's memory), code on a path where cudaMalloc's implicit
// device-wide synchronisation is not acceptable, or a process that has handed all free memory
// to a pool and has no allocator of its own to ask.
//
// sm_gemm_tc_static computes the same product as sm_gemm_tc (see kernels.h: mode 0 store
// with bias, 1 accumulate into a float output, 2 act(gate) * up). Where sm_gemm_tc wants a
// workspace from its caller for shapes whose reduction is split over several CTAs, this one
// uses a fixed array that is part of the library's image on every GPU that loads it:
// SM_GEMM_TC_STATIC_SCRATCH_BYTES (4 MiB) of device memory per GPU, held until the process
// exits. The caller passes only inputs and outputs (device pointers) and a stream.
//
//    4 MiB covers what decoding needs at the model sizes this library is measured on (most products need
//    none: up to 8 splits of K are added up inside a cluster); the planner's worst cases reach about 10 MB.
//  * A shape that needs more scratch than the array holds is refused with status 1 and a
//    message from sm_last_error() that names the bytes needed and the limit; nothing runs.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress,
//    with that device current) and remembers it. Make that first call at start-up: outside
//    any stream capture, and before the stretch of the program in which nothing may be
//    allocated. Where the CUDA runtime loads modules lazily, that first call is also when
//    this library's module, and with it the 4 MiB array, comes to lie on the device (an
//    allocation and a synchronisation by the runtime, once). Later calls on the same device
//    do no set-up.
//  * After that, no call allocates or frees: no cudaMalloc, cudaFree, or library routine that
//    does.
//  * All calls on a device share the one array, and it keeps whatever the last call left in
//    it. Nothing in it has to start at zero (every partial sum that is read was written by
//    the same call), so it is never cleared. Two calls whose kernels may run at the same time
//    (different streams, or one stream without ordering between them) race on it: keep calls
//    on one stream, or order them with events.
//  * `error` may be null; then a word beside the scratch array receives the code of a
//    bounded wait that ran out. sm_gemm_tc_static_error() reads it and, if it was set, clears
//    it: an error is reported once.
#pragma once

#include <stddef.h>

#define SM_GEMM_TC_STATIC_SCRATCH_BYTES ((size_t)4 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, or non-zero with a message for sm_last_error(). Pointers are device pointers;
// x [T, K] and w bfloat16; bias_dt / out_dt: 0 float32, 1 bfloat16; stream: a cudaStream_t.
int sm_gemm_tc_static(const void* x, const void* w, const void* bias, int bias_dt, void* out, int out_dt, int T, int N,
                      int K, int mode, int up_offset, int* error, void* stream);

// The error word used when `error` was null, read back to the host (synchronises the device)
// and cleared if it was set. -1: the read itself failed (see sm_last_error()).
int sm_gemm_tc_static_error(void);

#ifdef __cplusplus
}
#endif
