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
// eight consumer warps of four rows each. A lane owns a quarter of a block (64 weights, four sub-groups): two
// 16-byte runs of ql and one of qh, read as words (blocks start on 2-byte boundaries only: odd
// blocks are realigned with a funnel shift), each ql word giving two packed words of 6-bit values
// and each qh word serving four of them, fed to dp4a; a row of k = 2048 is one pass of a warp.
// The activation row is staged once per CTA with its sixteen 16-column sums per block.
#include "api_util.cuh"
#include "q4k_common.cuh"

namespace sgr {
namespace {

constexpr int kQ6 = 210;                     // bytes per Q6_K super-block
constexpr int kHeadWarps = 8;
constexpr int kHeadRows = 4;                  // rows a warp works on at once
constexpr int kHeadThreads = kHeadWarps * 32 + 32;
constexpr int kHeadStages = 4;
constexpr int kHeadStageBytes = 54 * 1024;   // whole rows, at most this many bytes per stage (and at most 32 rows)

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

    // A lane owns a quarter of a block: the sixteen columns (n, is) of all four qslots, i.e. the
    // 16-byte runs ql[n*64 + is*16 ..], ql[n*64 + 32 + is*16 ..] and qh[n*32 + is*16 ..], which hold
    // the sub-groups t = n*8 + 2*qslot + is, qslot = 0..3 (64 weights, four scales). A row of
    // k = 2048 is one pass of the warp. Blocks start on 2-byte boundaries only: the runs are read
    // as five aligned words each and realigned with a funnel shift (by 0 or 16 bits).
    int it = 0;
    for (int st = blockIdx.x; st < n_stages && ok; st += gridDim.x, ++it) {
      const int s = it % kHeadStages;
      ok = mbar_wait(full + s, (it / kHeadStages) & 1);
      if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
      const int r0 = st * a.rows_per_stage;
      const int nr = min(a.rows_per_stage, a.n_rows - r0);
      const unsigned char* stage = ring + static_cast<size_t>(s) * stage_bytes;
      // four rows of the stage per warp and pass (rows warp, warp + 8, ...): their loads are in flight
      // together, the activation words are fetched once for the four, and one transposing reduction
      // (six shuffles) replaces four of five
      for (int rb = warp; rb < nr; rb += kHeadWarps * kHeadRows) {
        const unsigned char* roww[kHeadRows];
#pragma unroll
        for (int i = 0; i < kHeadRows; ++i)
          roww[i] = stage + static_cast<size_t>(min(rb + i * kHeadWarps, nr - 1)) * row_bytes;
        float acc[kHeadRows];
#pragma unroll
        for (int i = 0; i < kHeadRows; ++i) acc[i] = 0.f;
        for (int u = lane; u < nb * 4; u += 32) {
          const int blk = u >> 2, n_half = (u >> 1) & 1, is = u & 1;
          const int off0 = blk * kQ6 + n_half * 64 + is * 16, offh = blk * kQ6 + 128 + n_half * 32 + is * 16;
          const int8_t* xcol = xs + blk * 256 + n_half * 128 + is * 16;
          const uint4 x0 = *reinterpret_cast<const uint4*>(xcol), x1 = *reinterpret_cast<const uint4*>(xcol + 32);
          const uint4 x2 = *reinterpret_cast<const uint4*>(xcol + 64), x3 = *reinterpret_cast<const uint4*>(xcol + 96);
          const uint32_t xa[4] = {x0.x, x0.y, x0.z, x0.w}, xb[4] = {x1.x, x1.y, x1.z, x1.w};
          const uint32_t xc[4] = {x2.x, x2.y, x2.z, x2.w}, xe[4] = {x3.x, x3.y, x3.z, x3.w};
          const int* xsp = xsum + blk * 16 + n_half * 8 + is;
          // the zero point: every sum starts at -32 * (sum of the sub-group's activations)
          const int z0 = -32 * xsp[0], z1 = -32 * xsp[2], z2 = -32 * xsp[4], z3 = -32 * xsp[6];
          const float xdb = xd[blk];
#pragma unroll
          for (int i = 0; i < kHeadRows; ++i) {
            const unsigned char* blk6 = roww[i] + blk * kQ6;
            const uintptr_t p0 = reinterpret_cast<uintptr_t>(roww[i] + off0);
            const uintptr_t ph = reinterpret_cast<uintptr_t>(roww[i] + offh);
            const unsigned sh = static_cast<unsigned>(p0 & 3u) * 8u;      // the three runs share the block's alignment
            const uint32_t* w0 = reinterpret_cast<const uint32_t*>(p0 & ~static_cast<uintptr_t>(3));
            const uint32_t* w1 = w0 + 8;                                   // 32 bytes on
            const uint32_t* wh = reinterpret_cast<const uint32_t*>(ph & ~static_cast<uintptr_t>(3));
            uint32_t l0[5], l1[5], hh[5];
#pragma unroll
            for (int j = 0; j < 5; ++j) { l0[j] = w0[j]; l1[j] = w1[j]; hh[j] = wh[j]; }
            const int8_t* scp = reinterpret_cast<const int8_t*>(blk6 + 192 + n_half * 8 + is);
            const int sc0 = scp[0], sc1 = scp[2], sc2 = scp[4], sc3 = scp[6];
            const float d = h2f(*reinterpret_cast<const uint16_t*>(blk6 + 208));
            int i0 = z0, i1 = z1, i2 = z2, i3 = z3;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t a0 = __funnelshift_r(l0[j], l0[j + 1], sh);
              const uint32_t a1 = __funnelshift_r(l1[j], l1[j + 1], sh);
              const uint32_t hw = __funnelshift_r(hh[j], hh[j + 1], sh);
              const uint32_t q0 = (a0 & 0x0F0F0F0Fu) | ((hw << 4) & 0x30303030u);
              const uint32_t q1 = (a1 & 0x0F0F0F0Fu) | ((hw << 2) & 0x30303030u);
              const uint32_t q2 = ((a0 >> 4) & 0x0F0F0F0Fu) | (hw & 0x30303030u);
              const uint32_t q3 = ((a1 >> 4) & 0x0F0F0F0Fu) | ((hw >> 2) & 0x30303030u);
              i0 = __dp4a(static_cast<int>(q0), static_cast<int>(xa[j]), i0);
              i1 = __dp4a(static_cast<int>(q1), static_cast<int>(xb[j]), i1);
              i2 = __dp4a(static_cast<int>(q2), static_cast<int>(xc[j]), i2);
              i3 = __dp4a(static_cast<int>(q3), static_cast<int>(xe[j]), i3);
            }
            // |sc * i| < 2^7 * 2^18 and four of them: the scaled sum of the quarter block is exact in int32
            acc[i] += xdb * d * static_cast<float>(sc0 * i0 + sc1 * i1 + sc2 * i2 + sc3 * i3);
          }
        }
        static_assert(kHeadRows == 4, "the reduction below transposes four rows");
        // lanes 0-15 take rows 0 and 1, lanes 16-31 rows 2 and 3; then lanes with bit 3 clear the first of the two
        const bool hi16 = (lane & 16) != 0, hi8 = (lane & 8) != 0;
        float s0 = hi16 ? acc[2] : acc[0], s1 = hi16 ? acc[3] : acc[1];
        s0 += __shfl_xor_sync(0xFFFFFFFFu, hi16 ? acc[0] : acc[2], 16);
        s1 += __shfl_xor_sync(0xFFFFFFFFu, hi16 ? acc[1] : acc[3], 16);
        float t = hi8 ? s1 : s0;
        t += __shfl_xor_sync(0xFFFFFFFFu, hi8 ? s0 : s1, 8);
        t += __shfl_xor_sync(0xFFFFFFFFu, t, 4);
        t += __shfl_xor_sync(0xFFFFFFFFu, t, 2);
        t += __shfl_xor_sync(0xFFFFFFFFu, t, 1);
        const int row = rb + (lane >> 3) * kHeadWarps;          // lanes 8i .. 8i+7 hold row i of the pass
        if ((lane & 7) == 0 && row < nr) a.y[r0 + row] = t;
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
  a.rows_per_stage = std::min(kHeadWarps * kHeadRows, kHeadStageBytes / row_bytes);
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
// Both phases merge sorted runs: a candidate becomes one 64-bit word - the value's order-preserving
// key above the complement of its index - so that descending order of the words IS the output order
// (larger value first, lower index first among equals) and an entry that never qualifies is the word
// 0. A run is 64 words in descending order held by one warp; the 64 largest of two runs are a
// lane-wise maximum against the reversed partner plus a six-step bitonic merge, all in shuffles.
// Phase 1: a CTA of 32 warps per 2048-value segment, each warp sorts 64 values, five rounds of
// pairwise selection leave the segment's best 64. Phase 2: one CTA does the same over the segments'
// candidate lists (up to 128 segments). Values are read back from the logits by index, so what is
// returned are the caller's own bits. (Selection by repeated arg-max - a warp per segment, k rounds
// of two warp reductions and a rescan - is kept for more than 128 segments; it took 110 us for
// 151,936 logits and k = 40, as slow as the reference's kernels.)
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

__device__ __forceinline__ unsigned long long topk_word(float x, int index) {
  if (!(x > kTopkNone)) return 0ull;             // NaN and anything at or below the sentinel never qualify
  const unsigned key = static_cast<unsigned>(order_key(x)) ^ 0x80000000u;
  return (static_cast<unsigned long long>(key) << 32) | static_cast<unsigned>(~index);
}

// A run of 64 words lives in one warp: lane l holds elements l and l + 32 (x[0], x[1]).
__device__ __forceinline__ unsigned long long shfl64(unsigned long long v, int src) {
  const unsigned lo = __shfl_sync(0xFFFFFFFFu, static_cast<unsigned>(v), src);
  const unsigned hi = __shfl_sync(0xFFFFFFFFu, static_cast<unsigned>(v >> 32), src);
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}
// One compare-exchange step at distance `stride` < 32 inside both halves; desc0 / desc1: the direction
// of this lane's element in x[0] / x[1]
__device__ __forceinline__ void run_step(unsigned long long (&x)[2], int stride, bool desc0, bool desc1, int lane) {
  const bool lower = (lane & stride) == 0;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const unsigned long long y = shfl64(x[j], lane ^ stride);
    const bool keep_max = lower == (j == 0 ? desc0 : desc1);
    x[j] = keep_max ? (x[j] > y ? x[j] : y) : (x[j] < y ? x[j] : y);
  }
}
// Bitonic run (first half descending, second ascending, or any bitonic order) -> descending run
__device__ __forceinline__ void run_merge_desc(unsigned long long (&x)[2], int lane) {
  const unsigned long long a = x[0], b = x[1];
  x[0] = a > b ? a : b;
  x[1] = a > b ? b : a;
#pragma unroll
  for (int stride = 16; stride > 0; stride >>= 1) run_step(x, stride, true, true, lane);
}
// Any 64 words -> descending run
__device__ __forceinline__ void run_sort_desc(unsigned long long (&x)[2], int lane) {
#pragma unroll
  for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      // element index i = lane + 32 j: bit `size` of i is bit `size` of the lane below 32, and j at 32
      const bool d0 = size < 32 ? (lane & size) == 0 : true;
      const bool d1 = size < 32 ? (lane & size) == 0 : false;
      run_step(x, stride, d0, d1, lane);
    }
  }
  run_merge_desc(x, lane);
}
// The 64 largest words of two descending runs, as a descending run: element i of the one against
// element 63 - i of the other leaves a bitonic run that holds them.
__device__ __forceinline__ void run_select(unsigned long long (&a)[2], const unsigned long long (&b)[2], int lane) {
  const unsigned long long b1 = shfl64(b[1], 31 - lane), b0 = shfl64(b[0], 31 - lane);
  a[0] = a[0] > b1 ? a[0] : b1;
  a[1] = a[1] > b0 ? a[1] : b0;
  run_merge_desc(a, lane);
}

// grid: one CTA of 32 warps per segment. Every warp sorts 64 values, then five rounds halve the runs.
__global__ void __launch_bounds__(1024) topk_seg_sort_kernel(const float* __restrict__ logits, float* __restrict__ seg_v,
                                                            int* __restrict__ seg_i, int n, int k) {
  __shared__ unsigned long long runs[32][64];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int base = blockIdx.x * kTopkSeg + warp * 64;
  unsigned long long x[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int gi = base + lane + 32 * j;
    x[j] = gi < n ? topk_word(__ldg(logits + gi), gi) : 0ull;
  }
  run_sort_desc(x, lane);
  runs[warp][lane] = x[0];
  runs[warp][lane + 32] = x[1];
  for (int r = 0; r < 5; ++r) {
    __syncthreads();
    if (warp < (16 >> r)) {
      const int sa = warp << (r + 1), sb = sa + (1 << r);
      unsigned long long a[2] = {runs[sa][lane], runs[sa][lane + 32]};
      const unsigned long long b[2] = {runs[sb][lane], runs[sb][lane + 32]};
      run_select(a, b, lane);
      runs[sa][lane] = a[0];
      runs[sa][lane + 32] = a[1];
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const unsigned long long w = runs[0][j];
    const int gi = w != 0ull ? static_cast<int>(~static_cast<unsigned>(w)) : -1;
    seg_i[static_cast<size_t>(blockIdx.x) * k + j] = gi;
    seg_v[static_cast<size_t>(blockIdx.x) * k + j] = gi >= 0 ? __ldg(logits + gi) : kTopkNone;
  }
}

// One CTA merges the candidates of up to 128 segments: a segment's k candidates are a descending run
// already. The first round reads pairs of runs from global memory, six more halve the 64 that remain.
__global__ void __launch_bounds__(1024) topk_merge_sort_kernel(const float* __restrict__ logits,
                                                              const float* __restrict__ seg_v,
                                                              const int* __restrict__ seg_i, float* __restrict__ out_v,
                                                              int* __restrict__ out_i, int nseg, int k) {
  __shared__ unsigned long long runs[64][64];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto load_run = [&](int seg, unsigned long long (&x)[2]) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int e = lane + 32 * j;
      x[j] = 0ull;
      if (seg < nseg && e < k) {
        const int gi = seg_i[static_cast<size_t>(seg) * k + e];
        if (gi >= 0) x[j] = topk_word(seg_v[static_cast<size_t>(seg) * k + e], gi);
      }
    }
  };
  for (int pr = warp; pr < 64; pr += 32) {
    unsigned long long a[2], b[2];
    load_run(2 * pr, a);
    load_run(2 * pr + 1, b);
    run_select(a, b, lane);
    runs[pr][lane] = a[0];
    runs[pr][lane + 32] = a[1];
  }
  for (int r = 0; r < 6; ++r) {
    __syncthreads();
    if (warp < (32 >> r)) {
      const int sa = warp << (r + 1), sb = sa + (1 << r);
      unsigned long long a[2] = {runs[sa][lane], runs[sa][lane + 32]};
      const unsigned long long b[2] = {runs[sb][lane], runs[sb][lane + 32]};
      run_select(a, b, lane);
      runs[sa][lane] = a[0];
      runs[sa][lane + 32] = a[1];
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const unsigned long long w = runs[0][j];
    const int gi = w != 0ull ? static_cast<int>(~static_cast<unsigned>(w)) : -1;
    out_i[j] = gi;
    out_v[j] = gi >= 0 ? __ldg(logits + gi) : kTopkNone;
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
  if (nseg <= 128) {
    cfg.blockDim = dim3(1024);
    cfg.gridDim = dim3(nseg);
    if (cudaLaunchKernelEx(&cfg, topk_seg_sort_kernel, logits, seg_v, seg_i, n, k) != cudaSuccess) return kErrLaunch;
    cfg.gridDim = dim3(1);
    return cudaLaunchKernelEx(&cfg, topk_merge_sort_kernel, logits, static_cast<const float*>(seg_v),
                              static_cast<const int*>(seg_i), out_v, out_i, nseg, k) == cudaSuccess
               ? kOk
               : kErrLaunch;
  }
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
