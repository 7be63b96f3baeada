// moe_prefill.cu - one MoE layer over a prefill chunk behind one call.
//
// The sequence is the one Session::moe_dispatch_device of the reference runs for a
// chunk (src/core/session.cpp:2482-3030): quantize_q8_k -> gemv_f32_out_f16x_mtok ->
// router_topk_batched -> moe_dispatch_scan -> gather_rows_q8_n -> gate / up ->
// silu_mul_f16_n -> quantize_q8_k_n -> down -> scatter_routed_f16 -> shared expert
// (gemv2 mtok, silu_mul, quantize, gemv mtok, strided copy into slot K of the combine
// slab) -> moe_combine_batched_f16, on the caller's scratch buffers
// (src/core/session.cpp:207-257). The last three steps - scatter into the combine slab, the
// shared rows' copy into its slot K, the combine over the slab - are one kernel here that reads
// the grouped rows and the shared rows where they lie (same sums in the same order; the slab,
// 75 MB written and read back for a 2048-row chunk, is not touched). The routed expert projections run on the int8
// tensor-core grouped GEMM (grouped_gemm_i8.cu) where the reference dequantises to fp16
// and calls a library GEMM per expert (src/core/session.cpp:2643-2760); every other
// step is the launcher the reference calls. Stream-ordered, no host synchronisation,
// nothing allocated: legal inside stream capture.
#include <algorithm>

#include "api_util.cuh"
#include "q4k_common.cuh"

using namespace sgr;

namespace {
// x[row] += sum_k w[row][k] * y_grouped[gslot[row][k]] (k = 0 .. K-1, in this order; a route that was
// not computed, gslot < 0, adds nothing) + w[row][K] * sh_y[row] (when there is a shared expert):
// scatter_routed_f16 + the strided copy + moe_combine_batched_f16 of the reference's sequence
// (src/core/session.cpp:2890-2930) without the slab in between. fp32 sums, one rounding to fp16.
// grid (rows, column chunks), 128 threads, 8 columns per thread; dynamic smem: (K+1) floats + K ints.
__global__ void combine_grouped_kernel(uint16_t* __restrict__ x, const uint16_t* __restrict__ y_grouped,
                                       const int* __restrict__ gslot, const uint16_t* __restrict__ sh_y,
                                       const float* __restrict__ weight, int K, int H) {
  extern __shared__ float wsm[];       // [K+1] weights of this row, then [K] grouped slots
  int* slot_sm = reinterpret_cast<int*>(wsm + K + 1);
  const int row = blockIdx.x;
  for (int kk = threadIdx.x; kk <= K; kk += blockDim.x) {
    wsm[kk] = weight[static_cast<size_t>(row) * (K + 1) + kk];
    if (kk < K) slot_sm[kk] = gslot[static_cast<size_t>(row) * K + kk];
  }
  __syncthreads();
  uint16_t* o = x + static_cast<size_t>(row) * H;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < H / 8; j += gridDim.y * blockDim.x) {
    const uint4 rv = reinterpret_cast<const uint4*>(o)[j];
    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
    float acc[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) { acc[2 * q] = h2f(rw[q] & 0xFFFF); acc[2 * q + 1] = h2f(rw[q] >> 16); }
    for (int k0 = 0; k0 < K; k0 += 4) {             // four routes' rows requested together
      uint4 yv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int gs = k0 + u < K ? slot_sm[k0 + u] : -1;
        yv[u] = gs >= 0 ? __ldg(reinterpret_cast<const uint4*>(y_grouped + static_cast<size_t>(gs) * H) + j)
                        : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (k0 + u < K && slot_sm[k0 + u] >= 0) {
          const float w = wsm[k0 + u];
          const uint32_t yw[4] = {yv[u].x, yv[u].y, yv[u].z, yv[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            acc[2 * q] += w * h2f(yw[q] & 0xFFFF);
            acc[2 * q + 1] += w * h2f(yw[q] >> 16);
          }
        }
      }
    }
    if (sh_y != nullptr) {
      const float w = wsm[K];
      const uint4 sv = __ldg(reinterpret_cast<const uint4*>(sh_y + static_cast<size_t>(row) * H) + j);
      const uint32_t yw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += w * h2f(yw[q] & 0xFFFF);
        acc[2 * q + 1] += w * h2f(yw[q] >> 16);
      }
    }
    uint32_t ow[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) ow[q] = f2h(acc[2 * q]) | (static_cast<uint32_t>(f2h(acc[2 * q + 1])) << 16);
    reinterpret_cast<uint4*>(o)[j] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}
}  // namespace

SGR_API int sgr_moe_layer_prefill(const sgr_moe_prefill* a, void* stream) {
  if (a == nullptr) return kErrArg;
  if (a->n <= 0) return kOk;
  const int n = a->n, H = a->hidden, F = a->n_ff, E = a->n_expert, K = a->n_used;
  if (H <= 0 || H % kQK || F <= 0 || F % kQK || E <= 0 || K <= 0 || K > E || a->n_max < n) return kErrGeometry;
  if (!a->xn || !a->x_f16 || !a->w_tab || !a->xq || !a->route_idx || !a->route_w || !a->gslot || !a->grows ||
      !a->off || !a->toff || !a->meta || !a->mail || !a->mail_n || !a->xqg || !a->g || !a->u || !a->hq ||
      !a->y_grouped || !a->expert_y)
    return kErrArg;
  if (!a->logits_in && (!a->router_w || !a->logits)) return kErrArg;
  const bool shared = a->shared_gate && a->shared_up && a->shared_down;
  if (shared && (!a->sh_g || !a->sh_u || !a->sh_q || !a->sh_y)) return kErrArg;
  const long long ts = a->tab_stride > 0 ? a->tab_stride : E;
  if (ts < E) return kErrArg;
  const int tok_per = a->tok_per > 0 ? a->tok_per : 16;
  const void* const* tab_g = a->w_tab;
  const void* const* tab_u = a->w_tab + ts;
  const void* const* tab_d = a->w_tab + 2 * ts;
  const long long R = static_cast<long long>(a->n_max) * K;
  if (R > 0x7FFFFFFF / (F / kQK)) return kErrUnsupported;
  int rc;
#define SGR_STEP(call) do { rc = (call); if (rc != kOk) return rc; } while (0)
  SGR_STEP(sgr_quantize_q8_k(a->xn, a->xq, static_cast<long long>(n) * H, stream));
  const float* logits = a->logits_in;
  if (logits == nullptr) {
    SGR_STEP(sgr_gemv_f32_out_f16x_mtok(a->router_w, a->xn, a->logits, E, H, n, stream));
    logits = a->logits;
  }
  SGR_STEP(sgr_router_topk_batched(logits, a->route_idx, a->route_w, E, K, K + 1, n,
                                   shared ? a->shared_w : 0.f, stream));
  SGR_STEP(sgr_moe_dispatch_scan(a->route_idx, a->route_w, a->gslot, a->grows, a->off, a->toff, a->meta,
                                 a->mail, a->mail_n, n, K, E, tok_per, stream));
  SGR_STEP(sgr_gather_rows_q8_n(a->xqg, a->xq, a->grows, a->meta, static_cast<int>(R), H / kQK, stream));
  SGR_STEP(sgr_moe_grouped_gemm_i8(tab_g, a->off, a->xqg, a->g, F, H, E, stream));
  SGR_STEP(sgr_moe_grouped_gemm_i8(tab_u, a->off, a->xqg, a->u, F, H, E, stream));
  SGR_STEP(sgr_silu_mul_f16_n(a->g, a->g, a->u, a->meta, static_cast<int>(R), F, stream));
  SGR_STEP(sgr_quantize_q8_k_n(a->g, a->hq, a->meta, F, static_cast<int>(R * (F / kQK)), stream));
  SGR_STEP(sgr_moe_grouped_gemm_i8(tab_d, a->off, a->hq, a->y_grouped, H, F, E, stream));
  // the combine reads the grouped rows in place when every buffer allows 16-byte accesses
  const bool direct = (H & 7) == 0 && K <= 1024 &&
                      ((reinterpret_cast<uintptr_t>(a->x_f16) | reinterpret_cast<uintptr_t>(a->y_grouped) |
                        (shared ? reinterpret_cast<uintptr_t>(a->sh_y) : 0)) & 15u) == 0;
  if (!direct) SGR_STEP(sgr_scatter_routed_f16(a->expert_y, a->y_grouped, a->gslot, n, K, H, stream));
  if (shared) {
    // the shared expert is one expert that every row visits: the same tensor-core kernel as the routed
    // ones when its row buffers allow 16-byte reads (the multi-token GEMV of the reference's sequence,
    // gemv2_q4_k_q8_f16out_mtok, took 0.42 ms for gate and up of a 2048-row chunk)
    const bool tc = ((reinterpret_cast<uintptr_t>(a->xq) | reinterpret_cast<uintptr_t>(a->sh_q)) & 15u) == 0;
    if (tc) {
      SGR_STEP(gemm_i8_dense(a->shared_gate, a->xq, a->sh_g, n, F, H, as_stream(stream)));
      SGR_STEP(gemm_i8_dense(a->shared_up, a->xq, a->sh_u, n, F, H, as_stream(stream)));
    } else {
      SGR_STEP(sgr_gemv2_q4_k_q8_f16out_mtok(a->shared_gate, a->shared_up, a->xq, a->sh_g, a->sh_u, F, H, n, stream));
    }
    SGR_STEP(sgr_silu_mul_f16(a->sh_g, a->sh_g, a->sh_u, n, F, stream));
    SGR_STEP(sgr_quantize_q8_k(a->sh_g, a->sh_q, static_cast<long long>(n) * F, stream));
    if (tc) {
      SGR_STEP(gemm_i8_dense(a->shared_down, a->sh_q, a->sh_y, n, H, F, as_stream(stream)));
    } else {
      SGR_STEP(sgr_gemv_q4_k_q8_f16out_mtok(a->shared_down, a->sh_q, a->sh_y, H, F, n, stream));
    }
    if (a->shared_gate_w != nullptr) {           // scalar gate sigmoid(w_sg . x) on the shared rows (layer.cpp:128-134)
      if (a->sgate == nullptr) return kErrArg;
      SGR_STEP(sgr_gemv_f32_out_f16x_batched(a->shared_gate_w, a->xn, a->sgate, 1, H, n, stream));
      SGR_STEP(sgr_sigmoid_gate_scalar_batched_f16(a->sh_y, a->sgate, n, H, stream));
    }
    // slot K of every row of the combine slab (the reference's strided copy, src/core/session.cpp:2911-2916)
    if (!direct && cudaMemcpy2DAsync(a->expert_y + static_cast<size_t>(K) * H, static_cast<size_t>(K + 1) * H * 2, a->sh_y,
                          static_cast<size_t>(H) * 2, static_cast<size_t>(H) * 2, n, cudaMemcpyDeviceToDevice,
                          as_stream(stream)) != cudaSuccess)
      return kErrLaunch;
  }
  if (direct) {
    const int chunks = std::max(1, std::min((H / 8 + 127) / 128, (4 * 148 + n - 1) / n));
    combine_grouped_kernel<<<dim3(n, chunks), 128, (2 * K + 1) * sizeof(float), as_stream(stream)>>>(
        a->x_f16, a->y_grouped, a->gslot, shared ? a->sh_y : nullptr, a->route_w, K, H);
    if (cudaPeekAtLastError() != cudaSuccess) return kErrLaunch;
  } else {
    SGR_STEP(sgr_moe_combine_batched_f16(a->x_f16, a->expert_y, a->route_w, K, H, n, stream));
  }
#undef SGR_STEP
  return kOk;
}
