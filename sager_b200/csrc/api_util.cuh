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

}  // namespace sgr
