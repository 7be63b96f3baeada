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

// The router dot of two expert rows (one warp) against NT token rows, everything in shared
// memory as fp32: the rows' weights as they lie in global memory, the activations k-major
// in planes of four token rows, xs[(t / 4) * 4 * k + kk * 4 + t % 4] (NT = 1, 2:
// xs[kk * NT + t]). A lane's activations of one k are one 16-byte load per plane and serve
// both rows. The loop is kept small on purpose: it runs once per CTA, and long unrolled
// code would spend its time in instruction fetch. The FMAs of a (row, lane, token) chain
// run in the same order as in router_row_dot, so the logits are bit-identical.
template <int NT>
__device__ __forceinline__ void router_fma_k2(float w0, float w1, const float* __restrict__ xs, int k, int kk,
                                              float (&acc)[2][NT]) {
  if (NT >= 4) {
#pragma unroll
    for (int p = 0; p < NT / 4; ++p) {
      const float4 a = *reinterpret_cast<const float4*>(xs + static_cast<size_t>(p) * 4 * k + static_cast<size_t>(kk) * 4);
      const float v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        acc[0][(4 * p + t) % NT] = fmaf(w0, v[t], acc[0][(4 * p + t) % NT]);
        acc[1][(4 * p + t) % NT] = fmaf(w1, v[t], acc[1][(4 * p + t) % NT]);
      }
    }
  } else if (NT == 2) {
    const float2 a = *reinterpret_cast<const float2*>(xs + static_cast<size_t>(kk) * 2);
    acc[0][0] = fmaf(w0, a.x, acc[0][0]); acc[0][1 % NT] = fmaf(w0, a.y, acc[0][1 % NT]);
    acc[1][0] = fmaf(w1, a.x, acc[1][0]); acc[1][1 % NT] = fmaf(w1, a.y, acc[1][1 % NT]);
  } else {
    const float a = xs[kk];
    acc[0][0] = fmaf(w0, a, acc[0][0]);
    acc[1][0] = fmaf(w1, a, acc[1][0]);
  }
}

template <int NT>
__device__ __forceinline__ void router_rows2_dot_kmajor(const float* __restrict__ w0s, const float* __restrict__ w1s,
                                                        const float* __restrict__ xs, int k, int lane,
                                                        float (&out)[2][NT]) {
  float acc[2][NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) acc[0][t] = acc[1][t] = 0.f;
#pragma unroll 4
  for (int kk = lane; kk < k; kk += 32) router_fma_k2<NT>(w0s[kk], w1s[kk], xs, k, kk, acc);
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      float a = acc[r][t];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) a += __shfl_down_sync(0xFFFFFFFFu, a, off);
      out[r][t] = a;
    }
}

// Softmax + top-k of one row by one warp. `prob` is n_expert floats of shared
// memory that already hold the logits; it is overwritten.
__device__ __forceinline__ void router_select_warp(float* prob, int n_expert, int k, int* out_idx,
                                                   float* out_w, float shared_w, bool write_shared,
                                                   int lane) {
  if (n_expert <= 256 && k <= 32) {
    // Up to 256 experts: a lane keeps its eight values (experts lane, lane + 32, ...) in
    // registers from the logits to the picks. Same arithmetic as the general path below.
    float pr[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) pr[j] = lane + 32 * j < n_expert ? prob[lane + 32 * j] : -1e30f;
    float mx = -1e30f;
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, pr[j]);
    {                                            // warp maximum through an order-preserving integer key
      const int b = __float_as_int(mx);
      const int key = b ^ ((b >> 31) & 0x7FFFFFFF);
      const int mk = __reduce_max_sync(0xFFFFFFFFu, key);
      mx = __int_as_float(mk ^ ((mk >> 31) & 0x7FFFFFFF));
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      pr[j] = expf(pr[j] - mx);
      if (lane + 32 * j < n_expert) prob[lane + 32 * j] = pr[j];
    }
    __syncwarp();
    float z = 0.f;
    if (lane == 0) {                             // strictly in index order, loads ahead of the adds
      int i = 0;
#pragma unroll 4
      for (; i + 8 <= n_expert; i += 8) {
        const float4 a = *reinterpret_cast<const float4*>(prob + i), b = *reinterpret_cast<const float4*>(prob + i + 4);
        z += a.x; z += a.y; z += a.z; z += a.w; z += b.x; z += b.y; z += b.z; z += b.w;
      }
      for (; i < n_expert; ++i) z += prob[i];
    }
    z = __shfl_sync(0xFFFFFFFFu, z, 0);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p = pr[j] / z;
      pr[j] = (lane + 32 * j < n_expert && p == p) ? p : -1.f;     // absent or NaN: never picked
    }
    float wsum = 0.f, my_w = 0.f;
    int my_i = 0;
    for (int kk = 0; kk < k; ++kk) {
      // this lane's best (lowest j on ties), then the warp's: largest value, lowest index
      float bv = pr[0];
      int bj = 0;
#pragma unroll
      for (int j = 1; j < 8; ++j)
        if (pr[j] > bv) { bv = pr[j]; bj = j; }
      const int vmax = __reduce_max_sync(0xFFFFFFFFu, __float_as_int(bv));      // values are >= 0 or -1
      const int cand = __float_as_int(bv) == vmax ? lane + 32 * bj : 0x7FFFFFFF;
      int bi = __reduce_min_sync(0xFFFFFFFFu, cand);
      float best = __int_as_float(vmax);
      if (best < 0.f) bi = kk % n_expert;          // nothing valid: deterministic filler
      if ((bi & 31) == lane && best >= 0.f) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j == (bi >> 5)) pr[j] = -1.f;
      }
      wsum += best;
      if (lane == kk) { my_w = best; my_i = bi; }
    }
    if (lane < k) {
      out_idx[lane] = my_i;
      out_w[lane] = wsum > 0.f ? my_w / wsum : my_w;
    }
    if (lane == 0 && write_shared) out_w[k] = shared_w;
    return;
  }
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
