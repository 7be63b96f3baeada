// quantize.cu - fp16 activations -> Q8_K blocks on the device.
//
// Arithmetic of the reference's quantize_q8_k_kernel (src/kernels/cuda/
// q4_k.cu:94-130): per 256 values amax = max(1e-30, |x|), d = amax/127,
// id = 1/d, q = clamp(rint(x*id), +-127), bsums[s] = sum of 32 codes. The
// result is bit-identical to the host quantiser on fp16-representable inputs,
// which is the gate the reference's own CUDA test applies. One warp per block:
// a lane converts 8 consecutive values from one 16-byte load.
#include "api_util.cuh"
#include "q4k_common.cuh"

namespace sgr {
namespace {

constexpr int kQuantWarps = 4;

__device__ __forceinline__ void quantize_block(const uint16_t* __restrict__ x,
                                               unsigned char* __restrict__ out, int lane) {
  float v[8];
  if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[lane];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = h2f(static_cast<uint16_t>(w[i] & 0xFFFFu));
      v[2 * i + 1] = h2f(static_cast<uint16_t>(w[i] >> 16));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = h2f(x[lane * 8 + i]);
  }
  float a = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(v[i]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, off));
  const float amax = fmaxf(1e-30f, a);
  const float d = amax / 127.f;
  const float id = d > 0.f ? 1.f / d : 0.f;
  int q[8];
  int sum = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    q[i] = max(-127, min(127, static_cast<int>(rintf(v[i] * id))));
    sum += q[i];
  }
  // four lanes hold one 32-value sub-block
  sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
  sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
  const int sum_hi = __shfl_down_sync(0xFFFFFFFFu, sum, 4);   // next sub-block's sum
  uint32_t* o32 = reinterpret_cast<uint32_t*>(out);           // block is 4-byte aligned
  if (lane == 0) o32[0] = __float_as_uint(d);
  o32[1 + 2 * lane] = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) |
                      (static_cast<uint32_t>(q[3] & 0xFF) << 24);
  o32[2 + 2 * lane] = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) |
                      (static_cast<uint32_t>(q[7] & 0xFF) << 24);
  if ((lane & 7) == 0) {                                      // lanes 0, 8, 16, 24
    o32[65 + (lane >> 3)] = (static_cast<uint32_t>(sum) & 0xFFFFu) |
                            (static_cast<uint32_t>(sum_hi) << 16);
  }
}

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
  quantize_block(x + b * kQK, out + b * kX8, threadIdx.x & 31);
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
