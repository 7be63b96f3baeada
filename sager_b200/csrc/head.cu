// head.cu - the LM head of a decode step on weights kept in the model's own 6-bit
// format, and the candidate selection that follows it: gemv_q6_k_q8 / gemv_q6_k_q8_smx
// (src/kernels/cuda/q4_k.cu:1564-1658 and src/kernels/cuda/mmq.cu:890-986 of the
// reference) and the two-phase top-k (src/kernels/cuda/sampling.cu:162-289).
//
// Q6_K super-block, 210 bytes / 256 weights (llama.cpp's block_q6_K, as
// src/core/weights.cpp:168-209 of the reference reads it): ql[128] | qh[64] | sc int8[16] |
// d fp16. Sub-group t = 0..15 holds the 16 weights n*128 + qslot*32 + is*16 + j
// (n = t >> 3, qslot = (t & 7) >> 1, is = t & 1, j < 16) with
//   q = ((ql[n*64 + (qslot & 1)*32 + is*16 + j] >> (qslot & 2 ? 4 : 0)) & 15)
//       | (((qh[n*32 + is*16 + j] >> 2*qslot) & 3) << 4)            in 0..63, zero point 32,
// and its term of the row's dot product is  xd * d * sc[t] * (sum q*x - 32 * sum x).
// The integer sums are exact; the fp32 terms of a row are added in another order than in the
// reference's one-warp-per-row kernels, so logits agree to fp32 rounding.
//
// The head is the largest matrix of a step (151,936 x 2048: 255 MB), so the GEMV is a
// persistent kernel: one CTA per SM, a producer warp streaming stages of whole rows (1680
// contiguous bytes each at k = 2048) into a shared-memory ring with bulk copies, eight
// consumer warps. A lane owns one sub-group: sixteen 6-bit weights are two 16-byte runs of ql
// and qh, read as words (blocks start on 2-byte boundaries only: odd blocks are realigned with a
// funnel shift), turned into four packed words with two mask operations each and fed to dp4a.
// The activation row is staged once per CTA with its sixteen 16-column sums per block.
#include "api_util.cuh"
#include "q4k_common.cuh"

namespace sgr {
namespace {

constexpr int kQ6 = 210;                     // bytes per Q6_K super-block
constexpr int kHeadWarps = 8;
constexpr int kHeadThreads = kHeadWarps * 32 + 32;
constexpr int kHeadStages = 4;
constexpr int kHeadStageBytes = 48 * 1024;   // whole rows, at most this many bytes per stage

struct HeadArgs {
  const unsigned char* w;
  const unsigned char* xq;   // one packed Q8_K row
  float* y;
  int n_rows, nb;
  int rows_per_stage;
  int* status;
};

// staged activations: codes [nb][256] int8, 16-column sums [nb][16] int32, scales [nb] fp32
__host__ __device__ inline size_t head_x_bytes(int nb) { return static_cast<size_t>(nb) * (256 + 64 + 4); }

__global__ void __launch_bounds__(kHeadThreads, 1) gemv_q6_stream_kernel(const HeadArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kHeadStages;
  unsigned char* ring = smem + 128;
  const int nb = a.nb;
  const int row_bytes = nb * kQ6;
  const int stage_bytes = (a.rows_per_stage * row_bytes + 127) & ~127;
  int8_t* xs = reinterpret_cast<int8_t*>(ring + static_cast<size_t>(kHeadStages) * stage_bytes);
  int* xsum = reinterpret_cast<int*>(xs + static_cast<size_t>(nb) * 256);
  float* xd = reinterpret_cast<float*>(xsum + nb * 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_stages = (a.n_rows + a.rows_per_stage - 1) / a.rows_per_stage;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kHeadStages; ++i) {
      mbar_init(full + i, 1);
      mbar_init(empty + i, kHeadWarps);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  bool ok = true;
  if (warp == kHeadWarps) {                    // producer: the weights do not depend on the previous kernel
    if (lane == 0) {
      int it = 0;
      for (int st = blockIdx.x; st < n_stages; st += gridDim.x, ++it) {
        const int s = it % kHeadStages;
        if (it >= kHeadStages && !mbar_wait(empty + s, ((it / kHeadStages) - 1) & 1)) {
          ok = false;
          break;
        }
        const int r0 = st * a.rows_per_stage;
        const int nr = min(a.rows_per_stage, a.n_rows - r0);
        const uint32_t bytes = static_cast<uint32_t>(nr) * row_bytes;
        mbar_expect_tx(full + s, bytes);
        bulk_g2s(ring + static_cast<size_t>(s) * stage_bytes, a.w + static_cast<size_t>(r0) * row_bytes, bytes, full + s);
      }
    }
  } else {
    pdl_wait();
    pdl_launch_dependents();
    // stage the activation row: codes, per-16-column sums, block scales
    const int ctid = threadIdx.x;
    for (int i = ctid; i < nb * 64; i += kHeadWarps * 32) {
      const int blk = i >> 6, wi = i & 63;
      reinterpret_cast<uint32_t*>(xs)[blk * 64 + wi] =
          reinterpret_cast<const uint32_t*>(a.xq + static_cast<size_t>(blk) * kX8 + 4)[wi];
    }
    for (int i = ctid; i < nb; i += kHeadWarps * 32)
      xd[i] = *reinterpret_cast<const float*>(a.xq + static_cast<size_t>(i) * kX8);
    asm volatile("bar.sync 1, %0;" ::"n"(kHeadWarps * 32) : "memory");
    for (int i = ctid; i < nb * 16; i += kHeadWarps * 32) {
      const uint4 c = *reinterpret_cast<const uint4*>(xs + static_cast<size_t>(i) * 16);
      int s = __dp4a(static_cast<int>(c.x), 0x01010101, 0);
      s = __dp4a(static_cast<int>(c.y), 0x01010101, s);
      s = __dp4a(static_cast<int>(c.z), 0x01010101, s);
      s = __dp4a(static_cast<int>(c.w), 0x01010101, s);
      xsum[i] = s;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kHeadWarps * 32) : "memory");

    // a lane owns sub-group (lane & 15) of two blocks per pass: lanes 0-15 block 2p, lanes 16-31 block 2p+1
    const int t = lane & 15;
    const int qslot = (t & 7) >> 1, is = t & 1, n_half = t >> 3;
    const int ql_off = n_half * 64 + (qslot & 1) * 32 + is * 16;
    const int qh_off = 128 + n_half * 32 + is * 16;
    const int nib = (qslot & 2) ? 4 : 0, hshift = qslot * 2;
    const int colbase = n_half * 128 + qslot * 32 + is * 16;
    int it = 0;
    for (int st = blockIdx.x; st < n_stages && ok; st += gridDim.x, ++it) {
      const int s = it % kHeadStages;
      ok = mbar_wait(full + s, (it / kHeadStages) & 1);
      if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
      const int r0 = st * a.rows_per_stage;
      const int nr = min(a.rows_per_stage, a.n_rows - r0);
      const unsigned char* stage = ring + static_cast<size_t>(s) * stage_bytes;
      for (int r = warp; r < nr; r += kHeadWarps) {
        const unsigned char* roww = stage + static_cast<size_t>(r) * row_bytes;
        float acc = 0.f;
        for (int b0 = 0; b0 < nb; b0 += 2) {
          const int blk = b0 + (lane >> 4);
          if (blk < nb) {
            const unsigned char* blk6 = roww + blk * kQ6;
            // sixteen bytes of ql and of qh as aligned words, realigned when the block starts 2 bytes in
            const uintptr_t pl = reinterpret_cast<uintptr_t>(blk6 + ql_off), ph = reinterpret_cast<uintptr_t>(blk6 + qh_off);
            const uint32_t* wl = reinterpret_cast<const uint32_t*>(pl & ~static_cast<uintptr_t>(3));
            const uint32_t* wh = reinterpret_cast<const uint32_t*>(ph & ~static_cast<uintptr_t>(3));
            const unsigned sl = static_cast<unsigned>(pl & 3u) * 8u, sh = static_cast<unsigned>(ph & 3u) * 8u;
            uint32_t l[5], h[5];
#pragma unroll
            for (int i = 0; i < 5; ++i) { l[i] = wl[i]; h[i] = wh[i]; }
            const uint4 xc = *reinterpret_cast<const uint4*>(xs + blk * 256 + colbase);
            const uint32_t xw[4] = {xc.x, xc.y, xc.z, xc.w};
            int isum = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t lw = __funnelshift_r(l[i], l[i + 1], sl);
              const uint32_t hw = __funnelshift_r(h[i], h[i + 1], sh);
              const uint32_t q = ((lw >> nib) & 0x0F0F0F0Fu) | (((hw >> hshift) & 0x03030303u) << 4);
              isum = __dp4a(static_cast<int>(q), static_cast<int>(xw[i]), isum);
            }
            const int sc = static_cast<int8_t>(blk6[192 + t]);
            const float d = h2f(*reinterpret_cast<const uint16_t*>(blk6 + 208));
            acc += xd[blk] * d * static_cast<float>(sc) * static_cast<float>(isum - 32 * xsum[blk * 16 + t]);
          }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xFFFFFFFFu, acc, off);
        if (lane == 0) a.y[r0 + r] = acc;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_one(empty + s);
    }
  }
  if (!ok && lane == 0 && a.status != nullptr) atomicExch(a.status, 1);
}

// Matrices whose base is not 16-byte aligned (no bulk copies) or that are tiny: a warp per row
// straight from global memory, bytes read one at a time where alignment demands it.
__global__ void gemv_q6_direct_kernel(const HeadArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.n_rows) return;
  const unsigned char* roww = a.w + static_cast<size_t>(row) * a.nb * kQ6;
  float acc = 0.f;
  for (int sg = lane; sg < a.nb * 16; sg += 32) {
    const int blk = sg >> 4, t = sg & 15;
    const int qslot = (t & 7) >> 1, is = t & 1, n_half = t >> 3;
    const unsigned char* blk6 = roww + static_cast<size_t>(blk) * kQ6;
    const unsigned char* ql = blk6 + n_half * 64 + (qslot & 1) * 32 + is * 16;
    const unsigned char* qh = blk6 + 128 + n_half * 32 + is * 16;
    const int nib = (qslot & 2) ? 4 : 0, hshift = qslot * 2;
    const unsigned char* xb = a.xq + static_cast<size_t>(blk) * kX8;
    const int8_t* xc = reinterpret_cast<const int8_t*>(xb + 4) + n_half * 128 + qslot * 32 + is * 16;
    int isum = 0, xs = 0;
    for (int j = 0; j < 16; ++j) {
      const int q = ((ql[j] >> nib) & 0xF) | (((qh[j] >> hshift) & 3) << 4);
      isum += q * xc[j];
      xs += xc[j];
    }
    const float d = h2f(static_cast<uint16_t>(blk6[208] | (blk6[209] << 8)));
    acc += *reinterpret_cast<const float*>(xb) * d * static_cast<float>(static_cast<int8_t>(blk6[192 + t])) *
           static_cast<float>(isum - 32 * xs);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xFFFFFFFFu, acc, off);
  if (lane == 0) a.y[row] = acc;
}

template <typename Kern>
int launch_head(Kern kern, dim3 grid, int threads, size_t smem, cudaStream_t stream, const HeadArgs& a) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, a) == cudaSuccess ? kOk : kErrLaunch;
}

int gemv_q6(const void* w, const void* xq, float* y, int n_rows, int k, cudaStream_t stream) {
  if (n_rows <= 0) return kOk;
  if (!w || !xq || !y || k <= 0 || k % kQK != 0) return kErrArg;
  if (reinterpret_cast<uintptr_t>(xq) & 3u) return kErrAlign;
  HeadArgs a{};
  a.w = static_cast<const unsigned char*>(w);
  a.xq = static_cast<const unsigned char*>(xq);
  a.y = y;
  a.n_rows = n_rows;
  a.nb = k / kQK;
  a.status = status_word();
  const int row_bytes = a.nb * kQ6;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return kErrLaunch;
  // bulk copies need 16-byte aligned sources of 16-byte multiples: whole rows when the row is one
  const bool streamable = (reinterpret_cast<uintptr_t>(w) & 15u) == 0 && row_bytes % 16 == 0 &&
                          row_bytes <= kHeadStageBytes && n_rows >= 4 * sms;
  if (!streamable) return launch_head(gemv_q6_direct_kernel, dim3((n_rows + 7) / 8), 256, 0, stream, a);
  a.rows_per_stage = kHeadStageBytes / row_bytes;
  const int stage_bytes = (a.rows_per_stage * row_bytes + 127) & ~127;
  const size_t smem = 128 + static_cast<size_t>(kHeadStages) * stage_bytes + head_x_bytes(a.nb);
  if (smem > 227 * 1024) return launch_head(gemv_q6_direct_kernel, dim3((n_rows + 7) / 8), 256, 0, stream, a);
  if (cudaFuncSetAttribute(gemv_q6_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
      cudaSuccess)
    return kErrLaunch;
  return launch_head(gemv_q6_stream_kernel, dim3(sms), kHeadThreads, smem, stream, a);
}

// ---- two-phase top-k ---------------------------------------------------------------------
// Contract (src/kernels/cuda/sampling.cu:109-153, 173-289 of the reference): the k largest values
// in descending order, equal values in ascending index order; a value that is not greater than
// -3.4e38 (that sentinel, -inf, NaN) is never picked, and when fewer than k values qualify the rest
// of the output is (-3.4e38, -1). k is capped at 64. The logits are not modified.
//
// Phase 1: one WARP per 2048-value segment, the segment in registers (64 values per lane, value i
// of lane l is element 32 * i + l, so a lane's values ascend in index). A round is two warp
// reductions - the largest order-preserving key, then the lowest index holding it - and only the
// winning lane rescans its registers. No shared memory, no CTA barrier. Phase 2: one CTA merges
// the segments' candidates the same way, eight warps first, then one.
constexpr float kTopkNone = -3.4e38f;
constexpr int kTopkSeg = 2048;               // the reference's segment size: the caller's scratch is sized by it
constexpr int kTopkPerLane = kTopkSeg / 32;

__device__ __forceinline__ int order_key(float v) {
  const int b = __float_as_int(v + 0.f);         // -0 -> +0: equal values must have equal keys
  return b ^ ((b >> 31) & 0x7FFFFFFF);
}

// One warp selects the top k of the values it holds in registers: v[i] with global index gi(i).
// get_index(i) must ascend with i inside a lane. Results go to out_v/out_i[0..k).
template <int PER, typename IndexOf>
__device__ __forceinline__ void warp_topk(float (&v)[PER], IndexOf index_of, int k, float* out_v, int* out_i, int lane) {
  // the lane's best: value key and slot (lowest slot on ties = lowest index)
  int best_key = order_key(kTopkNone), best_slot = -1;
  auto rescan = [&]() {
    best_key = order_key(kTopkNone);
    best_slot = -1;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int key = order_key(v[i]);
      if (v[i] > kTopkNone && key > best_key) { best_key = key; best_slot = i; }
    }
  };
  rescan();
  for (int it = 0; it < k; ++it) {
    const int top = __reduce_max_sync(0xFFFFFFFFu, best_key);
    const int cand = (best_slot >= 0 && best_key == top) ? index_of(best_slot) : 0x7FFFFFFF;
    const int win = __reduce_min_sync(0xFFFFFFFFu, cand);
    if (win == 0x7FFFFFFF) {                       // nothing left that qualifies
      if (lane == 0) { out_v[it] = kTopkNone; out_i[it] = -1; }
      continue;
    }
    if (cand == win) {                             // exactly one lane
      float val = kTopkNone;
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (i == best_slot) { val = v[i]; v[i] = kTopkNone; }
      out_v[it] = val;
      out_i[it] = win;
      rescan();
    }
  }
}

__global__ void __launch_bounds__(256) topk_seg_kernel(const float* __restrict__ logits, float* __restrict__ seg_v,
                                                      int* __restrict__ seg_i, int n, int k) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int seg = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int base = seg * kTopkSeg;
  if (base >= n) return;
  float v[kTopkPerLane];
#pragma unroll
  for (int i = 0; i < kTopkPerLane; ++i) {
    const int gi = base + 32 * i + lane;
    const float x = gi < n ? __ldg(logits + gi) : kTopkNone;
    v[i] = x > kTopkNone ? x : kTopkNone;          // NaN and anything at or below the sentinel never qualify
  }
  warp_topk<kTopkPerLane>(v, [&](int i) { return base + 32 * i + lane; }, k,
                          seg_v + static_cast<size_t>(seg) * k, seg_i + static_cast<size_t>(seg) * k, lane);
}

// m candidates (value, index), -1 index = empty. Eight warps each reduce a slice to k, then warp 0
// reduces those 8k to the final k. Candidates of a segment are already in output order, and a warp
// holds its slice in index-ascending order only if that is how they are laid out - so here a lane's
// tie rule uses the candidates' own indices, not their slots.
constexpr int kMergePerLane = 24;              // 8 warps x 32 lanes x 24 = 6144 candidates per pass

template <int PER>
__device__ __forceinline__ void warp_topk_pairs(float (&v)[PER], int (&gi)[PER], int k, float* out_v, int* out_i, int lane) {
  int best_key = order_key(kTopkNone), best_idx = 0x7FFFFFFF, best_slot = -1;
  auto rescan = [&]() {
    best_key = order_key(kTopkNone);
    best_idx = 0x7FFFFFFF;
    best_slot = -1;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int key = order_key(v[i]);
      if (gi[i] >= 0 && v[i] > kTopkNone && (key > best_key || (key == best_key && gi[i] < best_idx))) {
        best_key = key; best_idx = gi[i]; best_slot = i;
      }
    }
  };
  rescan();
  for (int it = 0; it < k; ++it) {
    const int top = __reduce_max_sync(0xFFFFFFFFu, best_key);
    const int cand = (best_slot >= 0 && best_key == top) ? best_idx : 0x7FFFFFFF;
    const int win = __reduce_min_sync(0xFFFFFFFFu, cand);
    if (win == 0x7FFFFFFF) {
      if (lane == 0) { out_v[it] = kTopkNone; out_i[it] = -1; }
      continue;
    }
    if (cand == win) {
      float val = kTopkNone;
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (i == best_slot) { val = v[i]; gi[i] = -1; }
      out_v[it] = val;
      out_i[it] = win;
      rescan();
    }
  }
}

__global__ void __launch_bounds__(256) topk_merge_kernel(const float* __restrict__ seg_v, const int* __restrict__ seg_i,
                                                        float* __restrict__ out_v, int* __restrict__ out_i, int m, int k) {
  __shared__ float sv[2][8 * 64];
  __shared__ int si[2][8 * 64];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // passes of 6144 candidates; the running best k of earlier passes ride along as candidates of warp 0
  int carried = 0;                               // entries of sv[0] / si[0] that hold the running result
  for (int p0 = 0; p0 < m || p0 == 0; p0 += 8 * 32 * kMergePerLane) {
    float v[kMergePerLane];
    int gi[kMergePerLane];
#pragma unroll
    for (int i = 0; i < kMergePerLane; ++i) {
      const int c = p0 + (warp * kMergePerLane + i) * 32 + lane;
      const bool in = c < m;
      v[i] = in ? seg_v[c] : kTopkNone;
      gi[i] = in ? seg_i[c] : -1;
    }
    warp_topk_pairs<kMergePerLane>(v, gi, k, sv[1] + warp * 64, si[1] + warp * 64, lane);
    __syncthreads();
    if (warp == 0) {
      // 8 x k fresh candidates plus the carried k: at most 9 * 64 = 576 -> 18 per lane
      float fv[18];
      int fi[18];
#pragma unroll
      for (int i = 0; i < 18; ++i) {
        const int c = i * 32 + lane;             // 0..511 fresh (warp c / 64, entry c % 64), 512.. carried
        if (c < 512) {
          const int w = c >> 6, e = c & 63;
          fv[i] = e < k ? sv[1][w * 64 + e] : kTopkNone;
          fi[i] = e < k ? si[1][w * 64 + e] : -1;
        } else {
          const int e = c - 512;
          fv[i] = e < carried ? sv[0][e] : kTopkNone;
          fi[i] = e < carried ? si[0][e] : -1;
        }
      }
      __syncwarp();
      warp_topk_pairs<18>(fv, fi, k, sv[0], si[0], lane);
      carried = k;
    }
    __syncthreads();
    carried = k;
  }
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    out_v[i] = sv[0][i];
    out_i[i] = si[0][i];
  }
}

}  // namespace
}  // namespace sgr

using namespace sgr;

// cuda_ops.hpp:48-49 of the reference.
SGR_API int sgr_gemv_q6_k_q8(const void* w_q6, const void* x_q8, float* y, int n_rows, int k, void* stream) {
  return gemv_q6(w_q6, x_q8, y, n_rows, k, as_stream(stream));
}

// cuda_ops.hpp:181-182 of the reference: the variant with the activations staged in shared memory.
// Here every path stages them; the two entry points are the same kernel and agree to the bit.
SGR_API int sgr_gemv_q6_k_q8_smx(const void* w_q6, const void* x_q8, float* y, int n_rows, int k, void* stream) {
  return gemv_q6(w_q6, x_q8, y, n_rows, k, as_stream(stream));
}

// cuda_ops.hpp:436-438 of the reference. seg_v / seg_i hold ceil(n / 2048) * k candidates between the
// phases; a scratch that is smaller is refused (the reference then falls back to a single-block kernel
// that overwrites the logits).
SGR_API int sgr_topk_select_f32_2p(const float* logits, float* seg_v, int* seg_i, int seg_slots, float* out_v,
                                   int* out_i, int n, int k, void* stream) {
  if (k <= 0 || n <= 0) return kOk;
  if (!logits || !seg_v || !seg_i || !out_v || !out_i) return kErrArg;
  if (k > 64) k = 64;
  const int nseg = (n + kTopkSeg - 1) / kTopkSeg;
  if (static_cast<long long>(nseg) * k > seg_slots) return kErrUnsupported;
  cudaStream_t s = as_stream(stream);
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.stream = s;
  cfg.blockDim = dim3(64);                        // two segments per CTA: the segments spread over the SMs
  cfg.gridDim = dim3((nseg + 1) / 2);
  if (cudaLaunchKernelEx(&cfg, topk_seg_kernel, logits, seg_v, seg_i, n, k) != cudaSuccess) return kErrLaunch;
  cfg.blockDim = dim3(256);
  cfg.gridDim = dim3(1);
  return cudaLaunchKernelEx(&cfg, topk_merge_kernel, static_cast<const float*>(seg_v), static_cast<const int*>(seg_i),
                            out_v, out_i, nseg * k, k) == cudaSuccess
             ? kOk
             : kErrLaunch;
}
