// router_dev.cuh - warp-level pieces of the router shared by router.cu and the
// fused layer: the lane-strided logit dot and the softmax / top-k selection.
// The arithmetic contracts are stated at the top of router.cu.
#pragma once

#include "q4k_common.cuh"

namespace sgr {

// One warp, one weight row, up to TT tokens whose fp16 rows sit in shared
// memory (xs[t*k + i]). Returns lane 0's tree sums in out[t].
template <int TT>
__device__ __forceinline__ void router_row_dot(const float* __restrict__ wrow,
                                               const uint16_t* __restrict__ xs, int k, int nt,
                                               int lane, float (&out)[TT]) {
  float acc[TT];
#pragma unroll
  for (int t = 0; t < TT; ++t) acc[t] = 0.f;
  int i = lane;
  // 32 independent loads in flight (a 2048-wide row is two round trips to memory),
  // FMAs issued in ascending index order
  for (; i + 31 * 32 < k; i += 32 * 32) {
    float wv[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) wv[j] = __ldg(wrow + i + j * 32);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
#pragma unroll
      for (int t = 0; t < TT; ++t)
        if (t < nt) acc[t] = fmaf(wv[j], h2f(xs[t * k + i + j * 32]), acc[t]);
    }
  }
  for (; i + 7 * 32 < k; i += 8 * 32) {
    float wv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) wv[j] = __ldg(wrow + i + j * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int t = 0; t < TT; ++t)
        if (t < nt) acc[t] = fmaf(wv[j], h2f(xs[t * k + i + j * 32]), acc[t]);
    }
  }
  for (; i < k; i += 32) {
    const float wv = __ldg(wrow + i);
#pragma unroll
    for (int t = 0; t < TT; ++t)
      if (t < nt) acc[t] = fmaf(wv, h2f(xs[t * k + i]), acc[t]);
  }
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    float a = acc[t];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) a += __shfl_down_sync(0xFFFFFFFFu, a, off);
    out[t] = a;
  }
}

// Softmax + top-k of one row by one warp. `prob` is n_expert floats of shared
// memory that already hold the logits; it is overwritten.
__device__ __forceinline__ void router_select_warp(float* prob, int n_expert, int k, int* out_idx,
                                                   float* out_w, float shared_w, bool write_shared,
                                                   int lane) {
  float mx = -1e30f;
  for (int i = lane; i < n_expert; i += 32) mx = fmaxf(mx, prob[i]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
  for (int i = lane; i < n_expert; i += 32) prob[i] = expf(prob[i] - mx);
  __syncwarp();
  float z = 0.f;
  if (lane == 0) {
    int i = 0;
    for (; i + 8 <= n_expert; i += 8) {           // loads batched, adds strictly in order
      float e[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = prob[i + j];
#pragma unroll
      for (int j = 0; j < 8; ++j) z += e[j];
    }
    for (; i < n_expert; ++i) z += prob[i];
  }
  z = __shfl_sync(0xFFFFFFFFu, z, 0);
  for (int i = lane; i < n_expert; i += 32) prob[i] = prob[i] / z;
  __syncwarp();

  // Every lane learns each pick (butterfly reduction); lane kk keeps pick kk in
  // registers, so the results reach global memory once, in parallel, already
  // renormalised. wsum is added in pick order in every lane (same rounding as the
  // reference's serial sum).
  float wsum = 0.f;
  float my_w = 0.f;
  int my_i = 0;
  // up to 256 experts: a lane keeps its eight probabilities in registers
  const bool in_regs = n_expert <= 256;
  float pr[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) pr[j] = (in_regs && lane + 32 * j < n_expert) ? prob[lane + 32 * j] : -1.f;
  for (int kk = 0; kk < k; ++kk) {
    float bv = -1.f;
    int bi = -1;
    if (in_regs) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float p = pr[j];
        if (p == p && p > bv) { bv = p; bi = lane + 32 * j; }
      }
    } else {
      for (int i = lane; i < n_expert; i += 32) {
        const float p = prob[i];
        if (p == p && p > bv) { bv = p; bi = i; }    // ascending scan: first strict max
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
      const bool take = (oi >= 0) && (bi < 0 || ov > bv || (ov == bv && oi < bi));
      if (take) { bv = ov; bi = oi; }
    }
    if (bi < 0) bi = kk % n_expert;                // nothing valid: deterministic filler
    if (in_regs) {
      if ((bi & 31) == lane) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j == (bi >> 5)) pr[j] = -1.f;
      }
    } else if (lane == 0) {
      prob[bi] = -1.f;
    }
    wsum += bv;
    if (k <= 32) {
      if (lane == kk) { my_w = bv; my_i = bi; }
    } else if (lane == 0) {
      out_idx[kk] = bi;
      out_w[kk] = bv;
    }
    __syncwarp();
  }
  if (k <= 32) {
    if (lane < k) {
      out_idx[lane] = my_i;
      out_w[lane] = wsum > 0.f ? my_w / wsum : my_w;
    }
  } else if (lane == 0 && wsum > 0.f) {
    for (int kk = 0; kk < k; ++kk) out_w[kk] /= wsum;
  }
  if (lane == 0 && write_shared) out_w[k] = shared_w;
}

}  // namespace sgr
