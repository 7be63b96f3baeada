// quantize.cu - fp16 activations -> Q8_K blocks on the device.
//
// Arithmetic of the reference's quantize_q8_k_kernel (src/kernels/cuda/
// q4_k.cu:94-130): per 256 values amax = max(1e-30, |x|), d = amax/127,
// id = 1/d, q = clamp(rint(x*id), +-127), bsums[s] = sum of 32 codes. The
// result is bit-identical to the host quantiser on fp16-representable inputs,
// which is the gate the reference's own CUDA test applies. One warp per block:
// a lane converts 8 consecutive values from one 16-byte load.
#include "api_util.cuh"
#include "quantize_dev.cuh"

namespace sgr {
namespace {

constexpr int kQuantWarps = 4;

__global__ void __launch_bounds__(kQuantWarps * 32)
quantize_q8_k_kernel(const uint16_t* __restrict__ x, unsigned char* __restrict__ out,
                     long long n_blocks, const int* __restrict__ d_rows, int row_mult) {
  const long long b = static_cast<long long>(blockIdx.x) * kQuantWarps + (threadIdx.x >> 5);
  long long live = n_blocks;
  if (d_rows != nullptr) {
    const long long elems = static_cast<long long>(*d_rows) * row_mult;
    live = min(live, (elems + kQK - 1) / kQK);
  }
  if (b >= live) return;
  quantize_block_f16(x + b * kQK, out + b * kX8, threadIdx.x & 31);
}

}  // namespace
}  // namespace sgr

using namespace sgr;

SGR_API int sgr_quantize_q8_k(const uint16_t* x_f16, void* out, long long n, void* stream) {
  if (n <= 0) return kOk;
  if (!x_f16 || !out || n % kQK != 0) return kErrArg;
  if ((reinterpret_cast<uintptr_t>(out) & 3u) || (reinterpret_cast<uintptr_t>(x_f16) & 1u))
    return kErrAlign;
  const long long nblk = n / kQK;
  quantize_q8_k_kernel<<<static_cast<unsigned>((nblk + kQuantWarps - 1) / kQuantWarps),
                         kQuantWarps * 32, 0, as_stream(stream)>>>(
      x_f16, static_cast<unsigned char*>(out), nblk, nullptr, 0);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// Device-count variant (q4_k.cu:1869-1924 of the reference): the live element
// count is (*d_rows) * row_mult, read on the device; n_max bounds the grid and
// is denominated in Q8_K blocks.
SGR_API int sgr_quantize_q8_k_n(const uint16_t* x_f16, void* out, const int* d_rows, int row_mult,
                                int n_max, void* stream) {
  if (n_max <= 0) return kOk;
  if (!x_f16 || !out || !d_rows || row_mult <= 0) return kErrArg;
  if ((reinterpret_cast<uintptr_t>(out) & 3u) || (reinterpret_cast<uintptr_t>(x_f16) & 1u))
    return kErrAlign;
  quantize_q8_k_kernel<<<(n_max + kQuantWarps - 1) / kQuantWarps, kQuantWarps * 32, 0,
                         as_stream(stream)>>>(x_f16, static_cast<unsigned char*>(out), n_max, d_rows,
                                              row_mult);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}
