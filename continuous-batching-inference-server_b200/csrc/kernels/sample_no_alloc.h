// Sampling for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project (its sampler is a host loop,
// src/server_demo.cpp:70-74); it is an addition of this library.
//
// Who needs it: code that picks next tokens from places where asking the CUDA allocator for memory
// is not an option: a serving loop that has already handed every remaining byte of the GPU to the
// key/value cache, a latency-critical thread that cannot afford the device-wide synchronisation a
// cudaMalloc or cudaFree may cause, or a host program that links this library without torch and
// owns no allocator of its own.  The ordinary entry point, cbis_sample(), leaves the scratch memory
// of the chunked argmax to its caller; this one brings its own, a fixed array inside the library.
//
// Limits and rules:
//   * at most CBIS_SAMPLE_NO_ALLOC_MAX_ROWS rows per call (any vocabulary size); more is refused
//     with CBIS_ERR_TOO_LARGE and nothing is launched;
//   * the scratch array (about 132 KB) lives in every GPU that loads the library until the process
//     ends; all calls share it and it keeps what the last call left, so two calls whose kernels may
//     run at the same time on one GPU (different streams) race: keep them in one stream or order
//     them yourself;
//   * the first call on each device looks the array's device address up (with that device current);
//     make that first call before starting any stream capture;
//   * it calls no cudaMalloc, cudaFree or any routine that allocates.
#pragma once

#define CBIS_SAMPLE_NO_ALLOC_MAX_ROWS 256

#ifdef __cplusplus
extern "C" {
#endif

// logits: [R, ld >= V] float on the current device; temperature[R] (<= 0: greedy) and keys[R] (one
// 64-bit key per draw) may be null for greedy sampling; out: int[R].  Returns 0, a negative CBIS_ERR_*
// status, or a CUDA error code.
int cbis_sample_no_alloc(const float* logits, int ld, const float* temperature, const unsigned long long* keys,
                         int* out, int R, int V, void* stream);

#ifdef __cplusplus
}
#endif
