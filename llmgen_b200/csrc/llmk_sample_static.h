// Sampling for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference: its sampler always receives scratch from
// the executor's workspace (src/executor.zig:717-753).  It exists for users of this library who
// may not call cudaMalloc (or any allocating routine) at the point where they sample: a plugin
// inside a host application whose own runtime owns all device memory, or code on a path where
// allocation is forbidden.  They still pass the logits, temperatures, seed and the output ids; the
// scratch for the blocks' candidates and the rows' ticket counters is a fixed array inside the library.
//
//   int llmk_sample_static(int* out, const float* logits, long long ld, const float* temps,
//                          const unsigned long long* seed, int n_rows, int V, void* stream);
//
//   out     int32 [n_rows], device: the sampled ids
//   logits  float32 [n_rows, V] with row stride ld, device
//   temps   float32 [n_rows], device: <= 0 greedy (ties to the smaller id), > 0 Gumbel-max
//   seed    one 64-bit step seed, device
//   stream  a cudaStream_t
//
// Returns 0, or non-zero with a message in llmk_last_error().  Same results as llmk_sample.
//
// Limits and rules:
//   * at most LLMK_SAMPLE_STATIC_MAX_ROWS rows a call; more is refused with an error, nothing runs;
//   * the array (65 KiB) stays on every GPU that loads the library until the process ends;
//   * the first call on a device looks the array's address up (cudaGetSymbolAddress, that device
//     current); make that first call outside any stream capture;
//   * calls share the array: do not let two of them overlap on the GPU (one stream, or order
//     them with events); nothing needs clearing between calls (the counters in it start at zero
//     and every call leaves them at zero);
//   * no cudaMalloc, cudaFree or other allocating call is made.
#pragma once

#define LLMK_SAMPLE_STATIC_MAX_ROWS 256

#ifdef __cplusplus
extern "C" {
#endif
int llmk_sample_static_max_rows(void);
int llmk_sample_static(int* out, const float* logits, long long ld, const float* temps,
                       const unsigned long long* seed, int n_rows, int V, void* stream);
#ifdef __cplusplus
}
#endif
