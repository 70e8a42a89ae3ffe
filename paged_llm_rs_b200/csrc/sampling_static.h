// pllm_sample_static: choose the next token for a few rows of logits without
// allocating anything, for callers that cannot call cudaMalloc (see the notes at its
// definition in sampling.cu).  It has no counterpart in the reference
// (nicoNaeg/paged-llm-rs samples on the host, crates/pagedllm/src/sampler.rs).
//
//   logits       float32 [n_rows, vocab] on the device, rows row_stride floats apart
//   temperature  float32 [n_rows] on the device; <= 0 means the first maximum
//   uniform      float32 [n_rows] on the device, each in [0, 1): the draw of a row
//   tokens       int32 [n_rows] on the device, written
//
// Returns 0, a negative refusal (-2 size, -4 beyond the limits below) or a cudaError_t.
// Same kernels and same result as pllm_sample; the scratch memory between its two
// launches is a fixed array of PLLM_STATIC_SAMPLE_FLOATS floats in the library image
// instead of a buffer from the caller.  Calls must not overlap on the GPU.  The first
// call on a device should come before any stream capture.  The array that is used is
// the CURRENT device's (cudaGetDevice at the call): ``stream`` must be a stream of that
// device, or the kernels would be given another GPU's array.
#pragma once

#include <cuda_runtime_api.h>   // cudaStream_t: this header can be included on its own

#define PLLM_STATIC_SAMPLE_MAX_ROWS 64
#define PLLM_STATIC_SAMPLE_MAX_VOCAB (1 << 20)
// rows * ceil(vocab / 4096) * 4 floats: exactly what 64 rows of 2^20 logits need (256 KiB)
#define PLLM_STATIC_SAMPLE_FLOATS (64 * 1024)

#ifdef __cplusplus
extern "C"
#endif
int pllm_sample_static(const float* logits, int n_rows, int vocab, long long row_stride, const float* temperature,
                       const float* uniform, int* tokens, cudaStream_t stream);
