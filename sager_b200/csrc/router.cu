// router.cu - router logits (fp32 W x fp16 x) and the softmax / top-k selection.
//
// Arithmetic contracts restated from the reference:
//  * logits (src/kernels/cuda/q4_k.cu:133-149, 285-303, 1439-1495): lane l of a
//    warp accumulates w[i]*x[i] for i = l, l+32, ... ascending with one FMA per
//    term, then the shuffle-down tree 16,8,4,2,1. Kept exactly, so logits are
//    bit-identical to the reference kernels' and routing cannot flip.
//  * selection (src/kernels/cuda/moe.cu:25-85, 165-234; mmq.cu:420-510):
//    mx = max logit, z = sum of expf(l - mx) added serially in index order,
//    p = expf(l - mx)/z, K greedy argmax passes on p (NaN never picked, ties to
//    the lower index, picked entries masked with -1, an empty pass yields
//    kk % E), weights renormalised by the sum of the picked p, slot K =
//    shared_w. The exponentials are evaluated in parallel, the sum keeps the
//    serial order, the argmax is a warp reduction with the same tie rule.
#include <cooperative_groups.h>

#include "api_util.cuh"
#include "router_dev.cuh"

namespace cg = cooperative_groups;

namespace sgr {

namespace {

constexpr int kRouterTok = 8;     // tokens per CTA of the logits kernel

// grid (ceil(n_rows / warps), ceil(n_tokens / kRouterTok)); dynamic smem = nt*k fp16
template <int TT>
__global__ void router_logits_kernel(const float* __restrict__ w, const uint16_t* __restrict__ x,
                                     float* __restrict__ y, int n_rows, int k, int n_tokens) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint16_t* xs = reinterpret_cast<uint16_t*>(smem);
  const int tok0 = blockIdx.y * TT;
  const int nt = min(TT, n_tokens - tok0);
  for (int i = threadIdx.x; i < nt * k; i += blockDim.x) xs[i] = x[static_cast<size_t>(tok0) * k + i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  float out[TT];
  router_row_dot<TT>(w + static_cast<size_t>(row) * k, xs, k, nt, lane, out);
  if (lane == 0) {
#pragma unroll
    for (int t = 0; t < TT; ++t)
      if (t < nt) y[static_cast<size_t>(tok0 + t) * n_rows + row] = out[t];
  }
}

int launch_logits(const float* w, const uint16_t* x, float* y, int n_rows, int k, int n_tokens,
                  cudaStream_t stream) {
  if (n_tokens <= 0 || n_rows <= 0) return kOk;
  if (!w || !x || !y || k <= 0) return kErrArg;
  if (n_tokens == 1) {
    const int warps = 2;                           // 2 MB of W spread over >= 128 CTAs at E=256
    const size_t smem = static_cast<size_t>(k) * 2;
    if (smem > 48 * 1024) return kErrUnsupported;
    router_logits_kernel<1><<<dim3((n_rows + warps - 1) / warps, 1), warps * 32, smem, stream>>>(
        w, x, y, n_rows, k, 1);
  } else {
    const int warps = 4;
    const size_t smem = static_cast<size_t>(kRouterTok) * k * 2;
    if (smem > 48 * 1024) return kErrUnsupported;
    router_logits_kernel<kRouterTok>
        <<<dim3((n_rows + warps - 1) / warps, (n_tokens + kRouterTok - 1) / kRouterTok), warps * 32,
           smem, stream>>>(w, x, y, n_rows, k, n_tokens);
  }
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// one warp per row, 4 rows per CTA; dynamic smem = 4 * n_expert floats
constexpr int kTopkWarps = 4;
__global__ void router_topk_kernel(const float* __restrict__ logits, int* __restrict__ idx,
                                   float* __restrict__ weight, int n_expert, int k, int stride,
                                   int n_rows, float shared_w) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kTopkWarps + warp;
  if (row >= n_rows) return;
  float* prob = reinterpret_cast<float*>(smem) + static_cast<size_t>(warp) * n_expert;
  for (int i = lane; i < n_expert; i += 32) prob[i] = logits[static_cast<size_t>(row) * n_expert + i];
  __syncwarp();
  router_select_warp(prob, n_expert, k, idx + static_cast<size_t>(row) * stride,
                     weight + static_cast<size_t>(row) * stride, shared_w, true, lane);
}

// Fused single-token router: a cluster of 8 CTAs splits the rows of W, every
// CTA drops its logits into the leader's shared memory through DSMEM, and after
// one cluster barrier the leader's first warp selects. One launch, no global
// scratch. Slot K of `weight` is left untouched, as the reference's
// router_topk_fused does (mmq.cu:459-510).
constexpr int kFusedCluster = 8;
constexpr int kFusedThreads = 512;
__global__ void __cluster_dims__(kFusedCluster, 1, 1) __launch_bounds__(kFusedThreads)
router_topk_fused_kernel(const float* __restrict__ w, const uint16_t* __restrict__ x,
                         int* __restrict__ idx, float* __restrict__ weight, int n_expert, int k_used,
                         int hidden) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint16_t* xs = reinterpret_cast<uint16_t*>(smem);
  float* logits = reinterpret_cast<float*>(smem + ((static_cast<size_t>(hidden) * 2 + 15) & ~size_t(15)));
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = x[i];
  __syncthreads();
  float* leader_logits = cluster.map_shared_rank(logits, 0);
  const int lane = threadIdx.x & 31;
  const int gwarp = rank * (kFusedThreads / 32) + (threadIdx.x >> 5);
  for (int row = gwarp; row < n_expert; row += kFusedCluster * (kFusedThreads / 32)) {
    float out[1];
    router_row_dot<1>(w + static_cast<size_t>(row) * hidden, xs, hidden, 1, lane, out);
    if (lane == 0) leader_logits[row] = out[0];
  }
  cluster.sync();
  if (rank == 0 && threadIdx.x < 32)
    router_select_warp(logits, n_expert, k_used, idx, weight, 0.f, false, lane);
}

}  // namespace
}  // namespace sgr

using namespace sgr;

SGR_API int sgr_gemv_f32_out_f16x(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows,
                                  int k, void* stream) {
  return launch_logits(w_f32, x_f16, y, n_rows, k, 1, as_stream(stream));
}
SGR_API int sgr_gemv_f32_out_f16x_batched(const float* w_f32, const uint16_t* x_f16, float* y,
                                          int n_rows, int k, int n_tokens, void* stream) {
  return launch_logits(w_f32, x_f16, y, n_rows, k, n_tokens, as_stream(stream));
}
SGR_API int sgr_gemv_f32_out_f16x_mtok(const float* w_f32, const uint16_t* x_f16, float* y,
                                       int n_rows, int k, int n_tokens, void* stream) {
  return launch_logits(w_f32, x_f16, y, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_router_topk_batched(const float* logits, int* idx, float* weight, int n_expert,
                                    int n_expert_used, int idx_stride, int n_rows, float shared_w,
                                    void* stream) {
  if (n_rows <= 0) return kOk;
  if (!logits || !idx || !weight || n_expert <= 0 || n_expert_used <= 0 ||
      idx_stride < n_expert_used + 1)
    return kErrArg;
  const size_t smem = static_cast<size_t>(kTopkWarps) * n_expert * sizeof(float);
  if (smem > 48 * 1024) return kErrUnsupported;
  router_topk_kernel<<<(n_rows + kTopkWarps - 1) / kTopkWarps, kTopkWarps * 32, smem,
                       as_stream(stream)>>>(logits, idx, weight, n_expert, n_expert_used,
                                            idx_stride, n_rows, shared_w);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}

SGR_API int sgr_router_topk(const float* logits, int* idx, float* weight, int n_expert,
                            int n_expert_used, float shared_w, void* stream) {
  return sgr_router_topk_batched(logits, idx, weight, n_expert, n_expert_used, n_expert_used + 1, 1,
                                 shared_w, stream);
}

SGR_API int sgr_router_topk_fused(const float* w_f32, const uint16_t* x_f16, int* idx, float* weight,
                                  int n_expert, int n_expert_used, int hidden, void* stream) {
  if (!w_f32 || !x_f16 || !idx || !weight || n_expert <= 0 || n_expert_used <= 0 || hidden <= 0)
    return kErrArg;
  const size_t smem = ((static_cast<size_t>(hidden) * 2 + 15) & ~size_t(15)) +
                      static_cast<size_t>(n_expert) * sizeof(float);
  if (smem > 48 * 1024) return kErrUnsupported;
  router_topk_fused_kernel<<<kFusedCluster, kFusedThreads, smem, as_stream(stream)>>>(
      w_f32, x_f16, idx, weight, n_expert, n_expert_used, hidden);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}
