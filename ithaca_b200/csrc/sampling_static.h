// ik_sample_static: sampling for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (SwankyMan88/ithaca samples on the
// host, src/chat.cpp:124-145); it is an addition of this library.
//
// Who needs it.  ik_sample works on a penalised copy of the logits and asks its caller for
// that scratch ([rows, V] floats).  Some callers cannot supply it: a host program that handed
// the whole device to its own arena at start-up and has nothing left to cudaMalloc from; a
// latency-critical loop in which cudaMalloc / cudaFree are off limits because they may stall
// every stream of the device; a caller from C or another language that links this library
// alone and has no tensor allocator to lean on.  For them the scratch lives inside the
// library, in a file-scope device array of fixed size.
//
// What it costs.  The array holds IK_SAMPLE_STATIC_MAX_FLOATS floats (8 MiB).  Every GPU on
// which this library is loaded keeps that much device memory for the array until the process
// exits, whether or not the entry point is ever called.
//
// Limits and rules.
//  * rows * V must not exceed IK_SAMPLE_STATIC_MAX_FLOATS (for instance 16 rows of a
//    128,256-entry vocabulary).  A larger request is refused: the call returns
//    IK_SAMPLE_STATIC_TOO_LARGE, prints one line to stderr that names both numbers, and
//    launches nothing.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress,
//    with that device current) and remembers it per device.  Make that first call outside
//    any stream capture.
//  * It calls no cudaMalloc, cudaFree or other allocating routine, of CUDA or of torch.
//  * All calls share the one array, and it keeps what the last call left in it.  Nothing in
//    it has to start at zero: each call first overwrites the rows * V floats it is going to
//    read.  Two calls that overlap on the GPU (different streams, or different host threads
//    without ordering between their launches) race on the array; order them on one stream
//    or with events.
//  * Arguments, rule and result are those of ik_sample (sampling.cu) without the `work`
//    pointer; for the same inputs it returns the same ids.
#pragma once
#include <cuda_runtime.h>

#define IK_SAMPLE_STATIC_MAX_FLOATS (2 * 1024 * 1024)
#define IK_SAMPLE_STATIC_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C"
#endif
int ik_sample_static(const float* logits, int ldl, int* out, int rows, int V, float temperature, int top_k,
                     float top_p, float rep_pen, const int* recent, int n_recent, unsigned long long seed,
                     const int* streams, const int* counters, cudaStream_t stream);
