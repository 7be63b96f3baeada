// quantize_dev.cuh - one warp quantises 256 fp16 values into a packed Q8_K block
// (arithmetic of the reference's quantize_q8_k_kernel, src/kernels/cuda/q4_k.cu:94-130).
#pragma once

#include "q4k_common.cuh"

namespace sgr {

// out16 (optional): the same block once more in the padded 288-byte form
// [d | 12 bytes | 256 codes | 8 int16 sums], every part 16-byte aligned.
__device__ __forceinline__ void quantize_block_f16(const uint16_t* __restrict__ x,
                                               unsigned char* __restrict__ out, int lane,
                                               unsigned char* __restrict__ out16 = nullptr) {
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
  if (out16 != nullptr) {
    uint32_t* p32 = reinterpret_cast<uint32_t*>(out16);
    if (lane == 0) p32[0] = __float_as_uint(d);
    p32[4 + 2 * lane] = o32[1 + 2 * lane];
    p32[5 + 2 * lane] = o32[2 + 2 * lane];
    if ((lane & 7) == 0) p32[68 + (lane >> 3)] = o32[65 + (lane >> 3)];
  }
}

}  // namespace sgr
