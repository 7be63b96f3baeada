// api_util.cuh - conventions shared by the extern "C" entry points.
//
// Every entry point is stream-ordered and never synchronises, allocates or
// reads device memory on the host; it validates its arguments, launches, and
// returns 0 or one of the error codes in q4k_common.cuh. A failed device-side
// bounded wait raises the library's status word, which sgr_status() reads.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "sager_b200.h"   // the public prototypes: definitions must agree with them
#include "sager_b200_diag.h"

#define SGR_API extern "C" __attribute__((visibility("default")))

namespace sgr {

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// Device address of the library's status word on the current device.
int* status_word();

// One Q4_K matrix over n_tok Q8_K rows on the int8 tensor-core kernel of the grouped GEMM
// (grouped_gemm_i8.cu): y[t][r], fp16. xq 16-byte aligned.
int gemm_i8_dense(const void* w, const void* xq, uint16_t* y, int n_tok, int n_rows, int k, cudaStream_t stream);

}  // namespace sgr
