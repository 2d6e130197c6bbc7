// llm_sample_no_alloc: token choice for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference engine (which samples on the CPU with a
// plain argmax, src/engine.cpp:52-58); it exists for users of this library only.
//
// Who needs it: a host program that has already handed every free byte of the GPU to its own
// pools (this engine's page pool is sized that way by default, so a later cudaMalloc can fail or
// fragment what is left), or a latency-bound loop that must never enter the CUDA allocator, which
// may synchronise the whole device. The regular entry point, llm_sample, leaves the scratch for
// its two-stage argmax to the caller, who normally gets it from an allocator. This variant brings
// its own: a fixed array that lives in the library's device image, so every GPU that loads the
// library holds LLM_SAMPLE_NO_ALLOC_SCRATCH_BYTES of it until the process exits.
//
// Contract
//   * Same inputs, outputs and results as llm_sample; the caller still owns logits, the per-row
//     parameters and `out`. Nothing is allocated or freed, by this function or by anything it calls.
//   * Limits: n_rows <= LLM_SAMPLE_NO_ALLOC_MAX_ROWS; the vocabulary is scanned in at most 64 chunks
//     per row whatever its size. Larger requests are refused with LLM_ERR_ARG and a message.
//   * The first call on a device looks up the array's device address (once per device, with that
//     device current) before it launches anything; make that first call before any stream capture
//     begins on that device. Later calls only launch.
//   * All calls on a device share the one array. Each call overwrites the part it uses before
//     reading it, so nothing has to be cleared between calls; but two calls whose kernels can
//     overlap on the GPU (different streams without an ordering between them) race on it. Keep
//     calls on one stream, or order them with events.
#pragma once

#include <cuda_runtime.h>

#define LLM_SAMPLE_NO_ALLOC_MAX_ROWS 256
#define LLM_SAMPLE_NO_ALLOC_MAX_CHUNKS 64
// two 4-byte words (best value, best index) per row and chunk
#define LLM_SAMPLE_NO_ALLOC_SCRATCH_BYTES (2 * 4 * LLM_SAMPLE_NO_ALLOC_MAX_ROWS * LLM_SAMPLE_NO_ALLOC_MAX_CHUNKS)

#ifdef __cplusplus
extern "C" {
#endif

// logits: float32 [n_rows, ld] on the device (ld >= vocab); temperature/seeds/draws: one per row on
// the device, temperature may be null (all greedy); out: int32 [n_rows] on the device.
// Returns 0, or a non-zero code with the text in llm_last_error().
int llm_sample_no_alloc(const float* logits, long long ld, const float* temperature, const int* seeds, const int* draws,
                        int* out, int n_rows, int vocab, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
