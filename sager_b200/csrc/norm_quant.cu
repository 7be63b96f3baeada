// norm_quant.cu - RMS norm fused with the Q8_K activation quantiser: the step
// that produces the MoE half's input rows (xn fp16 and their Q8_K blocks) from the
// residual stream. Replaces rmsnorm_quant_f16 of the reference
// (src/kernels/cuda/mmq.cu:533-641; call site src/core/session.cpp:1020-1023) and is
// held to its contract: bit-identical to the RMS norm followed by the quantiser.
//
// What fixes the bits:
//   sum of squares  thread t of a b-thread block (b = n rounded up to 32, at most
//                   1024) adds x[t]^2, x[t + b]^2, ... with FMA; a warp folds with
//                   shfl_down 16..1; thread 0 adds the warp sums in warp order
//   scale           rsqrtf(sum / n + eps)
//   out[i]          f16((f32(x[i]) * scale) * f32(w[i]))
//   Q8_K blocks     of the fp16 values just written: amax (order-free), d = amax/127,
//                   id = 1/d, codes rint(v * id) clamped to +-127, int16 sub-block sums
// Only the first line constrains the shape of the kernel; it is kept (one CTA per
// row, the same thread-to-element map). The quantiser runs warp-per-block on the
// normalised row held in shared memory instead of the reference's 256-thread
// groups with four CTA barriers per block.
#include "api_util.cuh"
#include "quantize_dev.cuh"

namespace sgr {
namespace {

__global__ void __launch_bounds__(1024) rmsnorm_quant_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ x,
                                                            const uint16_t* __restrict__ w,
                                                            unsigned char* __restrict__ xq, int n, float eps) {
  extern __shared__ __align__(16) uint16_t row_sh[];        // the normalised row, fp16
  __shared__ float red[32];
  pdl_wait();                                               // x comes from the previous kernel
  pdl_launch_dependents();
  const int tid = threadIdx.x, stride = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5;
  const size_t row = static_cast<size_t>(blockIdx.x) * n;
  float acc = 0.f;
  for (int i = tid; i < n; i += stride) {
    const float v = h2f(x[row + i]);
    acc = fmaf(v, v, acc);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xFFFFFFFFu, acc, off);
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    const int nw = (blockDim.x + 31) / 32;
    for (int i = 0; i < nw; ++i) s += red[i];
    red[0] = rsqrtf(s / static_cast<float>(n) + eps);
  }
  __syncthreads();
  const float scale = red[0];
  for (int i = tid; i < n; i += stride) {
    const uint16_t h = f2h(h2f(x[row + i]) * scale * h2f(w[i]));
    out[row + i] = h;
    row_sh[i] = h;
  }
  __syncthreads();
  const int nb = n / kQK;
  for (int blk = warp; blk < nb; blk += (blockDim.x >> 5))
    quantize_block_f16(row_sh + blk * kQK, xq + (static_cast<size_t>(blockIdx.x) * nb + blk) * kX8, lane);
}

}  // namespace
}  // namespace sgr

using namespace sgr;

// cuda_ops.hpp:149-151 of the reference. n must be a multiple of 256 (the reference falls back to
// its unfused norm kernel otherwise; that kernel is not part of this library).
SGR_API int sgr_rmsnorm_quant_f16(uint16_t* out, const uint16_t* x, const uint16_t* w, void* xq, int n, float eps,
                                  int n_rows, void* stream) {
  if (n_rows <= 0) return kOk;
  if (!out || !x || !w || !xq || n <= 0) return kErrArg;
  if (n % kQK != 0 || n > 16384) return kErrUnsupported;
  if (reinterpret_cast<uintptr_t>(xq) & 3u) return kErrAlign;
  int b = ((n + 31) / 32) * 32;
  if (b > 1024) b = 1024;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(n_rows);
  cfg.blockDim = dim3(b);
  cfg.dynamicSmemBytes = static_cast<size_t>(n) * 2;
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, rmsnorm_quant_kernel, out, x, w, static_cast<unsigned char*>(xq), n, eps) == cudaSuccess
             ? kOk
             : kErrLaunch;
}
