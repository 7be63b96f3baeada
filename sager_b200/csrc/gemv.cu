// gemv.cu - the Q4_K x Q8_K GEMV family behind the reference's launchers
// (src/kernels/cuda/q4_k.cu:1534-1562, 1660-1849, 1926-1985 and
// src/kernels/cuda/mmq.cu:368-378 of the reference): dense single-row and
// multi-token, pointer-table, host-plan grouped and device-plan grouped with
// the null-pointer mailbox. One kernel template, four planners; all of them
// end in tile_run (tile.cuh).
#include "api_util.cuh"
#include "tile.cuh"

namespace sgr {
namespace {

enum Mode : int { kDense = 0, kPtrs = 1, kGrouped = 2, kTab = 3, kMulti = 4 };

struct GemvArgs {
  const unsigned char* w[2];            // dense: matrix bases
  const unsigned char* const* tab[2];   // ptrs / grouped / tab: per-job or per-expert bases
  const unsigned char* xq;              // packed Q8_K rows, nb blocks each
  void* y[2];
  int n_rows, nb, n_tokens, tok_tile, rows_per, n_expert;
  const int *off, *m, *tile_base, *job_of_tile;   // grouped (host plan)
  const int *toff, *meta;                          // tab (device plan)
  int *mail, *mail_n;
  int* status;
  uint16_t* res;                        // dense, one token, fp16 out: residual row updated in place
  // multi: up to three matrices of the same k with their own outputs, one token row
  const unsigned char* wm[3];
  uint16_t* ym[3];
  int rows_cum[3];                      // rows of matrices 0..m inclusive
};

// last e with toff[e] <= tile (toff is the E+1 exclusive prefix of tiles per expert)
__device__ __forceinline__ int expert_of_tile(const int* toff, int n_expert, int tile) {
  int lo = 0, hi = n_expert - 1, res = n_expert - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) >> 1;
    if (toff[mid + 1] <= tile) lo = mid + 1;
    else { res = mid; hi = mid - 1; }
  }
  return res;
}

template <bool F16>
__device__ __forceinline__ void store_out(void* y, size_t i, float v) {
  if constexpr (F16) reinterpret_cast<uint16_t*>(y)[i] = f2h(v);
  else reinterpret_cast<float*>(y)[i] = v;
}
// fp16 store followed by the residual add of the rounded value (add_kernel's semantics,
// src/kernels/cuda/mmq.cu:870-876 of the reference): res = f16(f32(res) + f32(f16(v)))
__device__ __forceinline__ void store_out_resadd(uint16_t* y, uint16_t* res, size_t i, float v) {
  const uint16_t h = f2h(v);
  y[i] = h;
  res[i] = f2h(h2f(res[i]) + h2f(h));
}

template <int NMAT, int TT, int MODE, bool F16>
__global__ void __launch_bounds__(kTileThreads) gemv_tile_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int nb = a.nb;
  const int rc = tile_rows(nb);
  int row0 = blockIdx.x * rc;
  // plans and pointer tables may come from the kernel before this one; matrices named in the
  // arguments are fixed, so their copies start first and the wait sits just before the
  // activations are read (tile_run_staged's before_x hook)
  if constexpr (MODE != kDense && MODE != kMulti) {
    pdl_wait();
    pdl_launch_dependents();
  }
  int mat = 0;                           // multi: which matrix this CTA works on
  const size_t row_bytes = static_cast<size_t>(nb) * kW4;
  const size_t xrow_bytes = static_cast<size_t>(nb) * kX8;

  const unsigned char* wsrc[NMAT];
  int nrows, ntok;
  size_t xbase;          // first activation row of this tile
  size_t ybase;          // output row index of token slot 0 (multiplied by n_rows below)
  int ncols = a.n_rows;  // output row length

  if constexpr (MODE == kDense) {
    nrows = min(rc, a.n_rows - row0);
    const int tok0 = blockIdx.y * a.tok_tile;
    ntok = min(a.tok_tile, a.n_tokens - tok0);
#pragma unroll
    for (int m = 0; m < NMAT; ++m) wsrc[m] = a.w[m] + row0 * row_bytes;
    xbase = tok0;
    ybase = tok0;
  } else if constexpr (MODE == kMulti) {
    // tiles of matrix 0, then of matrix 1, then of matrix 2
    const int t0 = (a.rows_cum[0] + rc - 1) / rc;
    const int t1 = t0 + (a.rows_cum[1] - a.rows_cum[0] + rc - 1) / rc;
    int tile = blockIdx.x, rows_m = a.rows_cum[0];
    if (tile >= t1) { mat = 2; tile -= t1; rows_m = a.rows_cum[2] - a.rows_cum[1]; }
    else if (tile >= t0) { mat = 1; tile -= t0; rows_m = a.rows_cum[1] - a.rows_cum[0]; }
    row0 = tile * rc;
    nrows = min(rc, rows_m - row0);
    ntok = 1;
    wsrc[0] = (mat == 0 ? a.wm[0] : (mat == 1 ? a.wm[1] : a.wm[2])) + row0 * row_bytes;
    xbase = 0;
    ybase = 0;
    ncols = 0;
  } else if constexpr (MODE == kPtrs) {
    // y[e * rows_per + r]; every expert reads the SAME activation row, as the
    // reference kernel does (q4_k.cu:184-213 indexes xq[blk] only).
    const int e = blockIdx.y;
    nrows = min(rc, a.rows_per - row0);
    ntok = 1;
    wsrc[0] = a.tab[0][e] + row0 * row_bytes;
    xbase = 0;
    ybase = 0;
    ncols = 0;
  } else if constexpr (MODE == kGrouped) {
    const int job = a.job_of_tile[blockIdx.y];
    const int joff = a.off[job];
    const int tok0 = (blockIdx.y - a.tile_base[job]) * a.tok_tile;
    ntok = min(a.tok_tile, a.m[job] - tok0);
    nrows = min(rc, a.n_rows - row0);
    if (ntok <= 0) return;
#pragma unroll
    for (int m = 0; m < NMAT; ++m) wsrc[m] = a.tab[m][job] + row0 * row_bytes;
    xbase = joff + tok0;
    ybase = joff + tok0;
  } else {
    if (static_cast<int>(blockIdx.y) >= a.meta[1]) return;      // meta = {rows, tiles, bad}
    const int e = expert_of_tile(a.toff, a.n_expert, blockIdx.y);
    const int joff = a.off[e];
    const int tok0 = (blockIdx.y - a.toff[e]) * a.tok_tile;
    ntok = min(a.tok_tile, a.off[e + 1] - joff - tok0);
    nrows = min(rc, a.n_rows - row0);
    if (ntok <= 0) return;
    bool absent = false;
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
      const unsigned char* base = a.tab[m][e];
      absent = absent || (base == nullptr);
      wsrc[m] = base + row0 * row_bytes;
    }
    if (absent) {
      // Absent expert: its rows read as zero in the combine; the gate/up launch
      // posts the expert id once per tile for the host-side patch
      // (q4_k.cu:697-710 of the reference).
      for (int i = threadIdx.x; i < nrows * ntok; i += kTileThreads) {
        const int r = i % nrows, t = i / nrows;
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
          reinterpret_cast<uint16_t*>(a.y[m])[static_cast<size_t>(joff + tok0 + t) * a.n_rows + row0 + r] = 0;
      }
      if (a.mail != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        const int mi = atomicAdd(a.mail_n, 1);
        if (mi < a.n_expert) a.mail[mi] = e;
      }
      return;
    }
    xbase = joff + tok0;
    ybase = joff + tok0;
  }
  if (nrows <= 0 || ntok <= 0) return;

  tile_run_staged<NMAT, TT>(
      smem, wsrc, nrows, nb, ntok,
      [] {
        if constexpr (MODE == kDense || MODE == kMulti) {
          pdl_wait();
          pdl_launch_dependents();
        }
      },
      [&](const XTile& xt, int t0, int nt) {
        xtile_stage(xt, nt, [&](int t) { return a.xq + (xbase + t0 + t) * xrow_bytes; }, threadIdx.x, kTileThreads);
      },
      [&](int r, int t, const float (&v)[NMAT]) {
        if constexpr (MODE == kMulti) {
          uint16_t* ym = mat == 0 ? a.ym[0] : (mat == 1 ? a.ym[1] : a.ym[2]);
          ym[row0 + r] = f2h(v[0]);
          return;
        }
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          size_t oi;
          if constexpr (MODE == kPtrs) oi = static_cast<size_t>(blockIdx.y) * a.rows_per + row0 + r;
          else oi = (ybase + t) * ncols + row0 + r;
          if constexpr (MODE == kDense && F16 && NMAT == 1) {
            if (a.res != nullptr) {
              store_out_resadd(reinterpret_cast<uint16_t*>(a.y[0]), a.res, oi, v[0]);
              continue;
            }
          }
          store_out<F16>(a.y[m], oi, v[m]);
        }
      },
      a.status);
}

// Every launch of the family may start while the kernel before it in the stream drains
// (programmatic dependent launch); the kernels wait for that kernel's results themselves,
// just before they first read anything it could have written.
template <typename Kern>
int launch_dependent(Kern kern, dim3 grid, int threads, size_t smem, cudaStream_t stream, const GemvArgs& a) {
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

template <int NMAT, int TT, int MODE, bool F16>
int launch_tile(const GemvArgs& a, dim3 grid, cudaStream_t stream) {
  const size_t smem = tile_smem(NMAT, a.nb, TT);
  if (smem > 200 * 1024) return kErrUnsupported;
  auto kern = gemv_tile_kernel<NMAT, TT, MODE, F16>;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return kErrLaunch;
  }
  return launch_dependent(kern, grid, kTileThreads, smem, stream, a);
}

// ---- dense matrices far larger than the machine (the LM head): a persistent kernel ----------
// One CTA per SM walks stages of 256 consecutive super-blocks (36,864 contiguous bytes: a
// whole number of rows when nb divides 256), each stage one bulk copy into a five-deep
// ring issued by a producer warp. Thread t of the eight consumer warps owns block t of the
// stage: a quarter-warp reads eight consecutive 144-byte blocks, 16 bytes per lane per
// load, which spreads over all 32 banks without padding. The activations (at most four
// token rows) are staged once per CTA. The nb lanes of a row meet by shuffle.
constexpr int kStreamBlocks = 256;                       // super-blocks per stage = consumer threads
constexpr int kStreamStageBytes = kStreamBlocks * kW4;   // 36,864
constexpr int kStreamStages = 5;
constexpr int kStreamThreads = kStreamBlocks + 32;       // + the producer warp
inline size_t stream_gemv_smem(int nb, int tt) {
  return 128 + static_cast<size_t>(kStreamStages) * kStreamStageBytes + xtile_bytes(tt, nb);
}

template <int TT, bool F16>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_stream_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kStreamStages;
  unsigned char* ring = smem + 128;
  const int nb = a.nb;
  const XTile xt = xtile_at(ring + kStreamStages * kStreamStageBytes, TT, nb);
  const long long total_blocks = static_cast<long long>(a.n_rows) * nb;
  const int n_stages = static_cast<int>((total_blocks + kStreamBlocks - 1) / kStreamBlocks);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStreamStages; ++i) {
      mbar_init(full + i, 1);
      mbar_init(empty + i, kStreamBlocks / 32);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  bool ok = true;
  if (warp == kStreamBlocks / 32) {                      // producer
    if (lane == 0) {
      int it = 0;
      for (int st = blockIdx.x; st < n_stages; st += gridDim.x, ++it) {
        const int s = it % kStreamStages;
        if (it >= kStreamStages && !mbar_wait(empty + s, ((it / kStreamStages) - 1) & 1)) {
          ok = false;
          break;
        }
        const long long b0 = static_cast<long long>(st) * kStreamBlocks;
        const long long nblk = total_blocks - b0 < kStreamBlocks ? total_blocks - b0 : kStreamBlocks;
        const uint32_t bytes = static_cast<uint32_t>(nblk) * kW4;
        mbar_expect_tx(full + s, bytes);
        bulk_g2s(ring + s * kStreamStageBytes, a.w[0] + b0 * kW4, bytes, full + s);
      }
    }
  } else {
    pdl_wait();                                          // the weight stream above is already running
    pdl_launch_dependents();
    xtile_stage(xt, a.n_tokens, [&](int t) { return a.xq + static_cast<size_t>(t) * nb * kX8; },
                threadIdx.x, kStreamBlocks);
    asm volatile("bar.sync 1, %0;" ::"n"(kStreamBlocks) : "memory");
    const int blk = threadIdx.x & (nb - 1);              // nb is a power of two <= 16
    int it = 0;
    for (int st = blockIdx.x; st < n_stages && ok; st += gridDim.x, ++it) {
      const int s = it % kStreamStages;
      ok = mbar_wait(full + s, (it / kStreamStages) & 1);
      if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
      const long long b = static_cast<long long>(st) * kStreamBlocks + threadIdx.x;
      float acc[1][TT];
#pragma unroll
      for (int t = 0; t < TT; ++t) acc[0][t] = 0.f;
      if (b < total_blocks) {
        const uint4* wb[1] = {reinterpret_cast<const uint4*>(ring + s * kStreamStageBytes + threadIdx.x * kW4)};
        block_dot<1, TT>(wb, xt, blk, a.n_tokens, acc);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_one(empty + s);          // this warp has read its blocks
#pragma unroll
      for (int t = 0; t < TT; ++t) acc[0][t] = reduce_lanes(acc[0][t], nb);
      if (blk == 0 && b < total_blocks) {
        const long long row = b / nb;
#pragma unroll
        for (int t = 0; t < TT; ++t)
          if (t < a.n_tokens) {
            if constexpr (F16 && TT == 1) {
              if (a.res != nullptr) {
                store_out_resadd(reinterpret_cast<uint16_t*>(a.y[0]), a.res, static_cast<size_t>(row), acc[0][t]);
                continue;
              }
            }
            store_out<F16>(a.y[0], static_cast<size_t>(t) * a.n_rows + row, acc[0][t]);
          }
      }
    }
  }
  if (!ok && lane == 0 && a.status != nullptr) atomicExch(a.status, 1);
}

template <int TT, bool F16>
int launch_stream(const GemvArgs& a, int sms, cudaStream_t stream) {
  const size_t smem = stream_gemv_smem(a.nb, TT);
  auto kern = gemv_stream_kernel<TT, F16>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
      cudaSuccess)
    return kErrLaunch;
  return launch_dependent(kern, dim3(sms), kStreamThreads, smem, stream, a);
}

// The persistent kernel pays off when every SM gets several stages.
inline int stream_sms(const GemvArgs& a) {
  if (a.n_tokens > 4 || a.nb > 16 || (a.nb & (a.nb - 1)) != 0) return 0;
  if (reinterpret_cast<uintptr_t>(a.w[0]) & 15u) return 0;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return 0;
  const long long stages = (static_cast<long long>(a.n_rows) * a.nb + kStreamBlocks - 1) / kStreamBlocks;
  return stages >= 8LL * sms ? sms : 0;
}

// ---- small dense matrices, two to four token rows (a verify window) ------------------------
// Fewer tiles than SMs: latency decides, not bandwidth, and staging through shared memory
// only adds to it. One lane per 32-byte nibble group (two sub-blocks) straight from global
// memory, no barriers. The integer partial sums of a super-block meet exactly by shuffle
// over its four lanes, its fp32 term is formed once, and the terms of a row are added in
// the order of the tile kernels' shuffle tree.
constexpr int kDirectThreads = 128;

template <int NMAT, int TT, bool F16>
__global__ void __launch_bounds__(kDirectThreads) gemv_direct_kernel(const GemvArgs a) {
  const int nb = a.nb;
  const int groups = nb * 4;
  const int lpr = groups < 32 ? groups : 32;               // lanes per row (a power of two >= 4)
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (kDirectThreads / 32) + (threadIdx.x >> 5);
  const int row_raw = warp * (32 / lpr) + lane / lpr;
  const int row = min(row_raw, a.n_rows - 1);              // every lane runs the same loops
  const int lr = lane & (lpr - 1);
  const int nt = a.n_tokens;
  float acc[NMAT][TT];
#pragma unroll
  for (int m = 0; m < NMAT; ++m)
#pragma unroll
    for (int t = 0; t < TT; ++t) acc[m][t] = 0.f;
  bool waited = false;                     // the previous kernel is awaited once the first weights are requested
  for (int gi = lr; gi < groups; gi += lpr) {
    const int blk = gi >> 2, g = gi & 3;
    float d[NMAT], dmin[NMAT];
    uint32_t lo[NMAT][8], hi[NMAT][8];
    int sc_lo[NMAT], sc_hi[NMAT], mn_lo[NMAT], mn_hi[NMAT];
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
      const unsigned char* wb = a.w[m] + (static_cast<size_t>(row) * nb + blk) * kW4;
      const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(wb));
      const uint4 q0 = __ldg(reinterpret_cast<const uint4*>(wb + 16 + 32 * g));
      const uint4 q1 = __ldg(reinterpret_cast<const uint4*>(wb + 32 + 32 * g));
      d[m] = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x & 0xFFFFu)));
      dmin[m] = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x >> 16)));
      const Scales6 s6 = unpack_scales6(hdr.y, hdr.z, hdr.w);
      const uint32_t scw = g < 2 ? s6.sc[0] : s6.sc[1], mnw = g < 2 ? s6.mn[0] : s6.mn[1];
      sc_lo[m] = (scw >> (16 * (g & 1))) & 0xFF;
      sc_hi[m] = (scw >> (16 * (g & 1) + 8)) & 0xFF;
      mn_lo[m] = (mnw >> (16 * (g & 1))) & 0xFF;
      mn_hi[m] = (mnw >> (16 * (g & 1) + 8)) & 0xFF;
      const uint32_t raw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        lo[m][i] = raw[i] & 0x0F0F0F0Fu;
        hi[m][i] = (raw[i] >> 4) & 0x0F0F0F0Fu;
      }
    }
    if (!waited) {
      pdl_wait();
      pdl_launch_dependents();
      waited = true;
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      if (t < nt) {
        const unsigned char* xb = a.xq + (static_cast<size_t>(t) * nb + blk) * kX8;
        const uint32_t* xc = reinterpret_cast<const uint32_t*>(xb + 4 + 64 * g);
        uint32_t xv[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) xv[i] = __ldg(xc + i);
        const uint32_t bs = __ldg(reinterpret_cast<const uint32_t*>(xb + 260 + 4 * g));   // two int16 sums
        const float xd = __ldg(reinterpret_cast<const float*>(xb));
        const int bs_lo = static_cast<int16_t>(bs & 0xFFFFu), bs_hi = static_cast<int16_t>(bs >> 16);
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          int dl = 0, dh = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dl = __dp4a(static_cast<int>(lo[m][i]), static_cast<int>(xv[i]), dl);
            dh = __dp4a(static_cast<int>(hi[m][i]), static_cast<int>(xv[8 + i]), dh);
          }
          int isum = sc_lo[m] * dl + sc_hi[m] * dh;
          int msum = mn_lo[m] * bs_lo + mn_hi[m] * bs_hi;
          isum += __shfl_xor_sync(0xFFFFFFFFu, isum, 1);
          msum += __shfl_xor_sync(0xFFFFFFFFu, msum, 1);
          isum += __shfl_xor_sync(0xFFFFFFFFu, isum, 2);
          msum += __shfl_xor_sync(0xFFFFFFFFu, msum, 2);
          if (g == 0) acc[m][t] += xd * (d[m] * static_cast<float>(isum) - dmin[m] * static_cast<float>(msum));
        }
      }
    }
  }
  if (!waited) {
    pdl_wait();
    pdl_launch_dependents();
  }
#pragma unroll
  for (int m = 0; m < NMAT; ++m)
#pragma unroll
    for (int t = 0; t < TT; ++t) acc[m][t] = reduce_lanes(acc[m][t], lpr);
  if (lr == 0 && row_raw < a.n_rows) {
#pragma unroll
    for (int t = 0; t < TT; ++t)
      if (t < nt) {
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
          store_out<F16>(a.y[m], static_cast<size_t>(t) * a.n_rows + row_raw, acc[m][t]);
      }
  }
}

template <int NMAT, bool F16>
int launch_direct(const GemvArgs& a, cudaStream_t stream) {
  const int lpr = a.nb * 4 < 32 ? a.nb * 4 : 32;
  const int rows_per_cta = (kDirectThreads / 32) * (32 / lpr);
  const int grid = (a.n_rows + rows_per_cta - 1) / rows_per_cta;
  if (a.n_tokens == 2) return launch_dependent(gemv_direct_kernel<NMAT, 2, F16>, dim3(grid), kDirectThreads, 0, stream, a);
  return launch_dependent(gemv_direct_kernel<NMAT, 4, F16>, dim3(grid), kDirectThreads, 0, stream, a);
}

// Two to four token rows over a matrix of at most a few tiles per SM, 16-byte aligned.
template <int NMAT>
inline bool direct_fits(const GemvArgs& a) {
  if (a.n_tokens < 2 || a.n_tokens > 4 || (a.nb & (a.nb - 1)) != 0) return false;
  for (int m = 0; m < NMAT; ++m)
    if (reinterpret_cast<uintptr_t>(a.w[m]) & 15u) return false;
  return static_cast<long long>(a.n_rows) * a.nb <= 148LL * 4 * kStreamBlocks;
}

// tokens per CTA of the dense multi-token kernels (walked in sub-tiles of 8)
constexpr int kDenseTokTile = 16;

template <int NMAT, bool F16>
int launch_dense(const void* w0, const void* w1, const void* xq, void* y0, void* y1, int n_rows,
                 int k, int n_tokens, cudaStream_t stream, uint16_t* res = nullptr) {
  if (n_tokens <= 0 || n_rows <= 0) return kOk;
  if (!w0 || !xq || !y0 || (NMAT == 2 && (!w1 || !y1)) || k <= 0 || k % kQK != 0) return kErrArg;
  if (reinterpret_cast<uintptr_t>(xq) & 3u) return kErrAlign;
  GemvArgs a{};
  a.w[0] = static_cast<const unsigned char*>(w0);
  a.w[1] = static_cast<const unsigned char*>(w1);
  a.xq = static_cast<const unsigned char*>(xq);
  a.y[0] = y0;
  a.y[1] = y1;
  a.n_rows = n_rows;
  a.nb = k / kQK;
  a.n_tokens = n_tokens;
  a.status = status_word();
  a.res = res;
  const int rc = tile_rows(a.nb);
  if constexpr (NMAT == 1) {
    if (const int sms = stream_sms(a)) {
      if (n_tokens == 1) return launch_stream<1, F16>(a, sms, stream);
      if (n_tokens == 2) return launch_stream<2, F16>(a, sms, stream);
      return launch_stream<4, F16>(a, sms, stream);
    }
  }
  if (direct_fits<NMAT>(a)) return launch_direct<NMAT, F16>(a, stream);
  if (n_tokens == 1) {
    a.tok_tile = 1;
    return launch_tile<NMAT, 1, kDense, F16>(a, dim3((n_rows + rc - 1) / rc, 1), stream);
  }
  if (n_tokens <= 4) {              // a verify window: dp4a over four token slots beats the MMA fragment set-up
    a.tok_tile = 4;
    return launch_tile<NMAT, 4, kDense, F16>(a, dim3((n_rows + rc - 1) / rc, 1), stream);
  }
  a.tok_tile = kDenseTokTile;
  return launch_tile<NMAT, 8, kDense, F16>(
      a, dim3((n_rows + rc - 1) / rc, (n_tokens + kDenseTokTile - 1) / kDenseTokTile), stream);
}

template <int NMAT>
int launch_grouped(const void* const* t0, const void* const* t1, const int* off, const int* m,
                   const int* tile_base, const int* job_of_tile, int n_tiles, const void* xq,
                   void* y0, void* y1, int n_rows, int k, int tok_per, cudaStream_t stream) {
  if (n_tiles <= 0) return kOk;
  if (!t0 || (NMAT == 2 && (!t1 || !y1)) || !off || !m || !tile_base || !job_of_tile || !xq ||
      !y0 || n_rows <= 0 || k <= 0 || k % kQK != 0 || tok_per <= 0)
    return kErrArg;
  if (reinterpret_cast<uintptr_t>(xq) & 3u) return kErrAlign;
  GemvArgs a{};
  a.tab[0] = reinterpret_cast<const unsigned char* const*>(t0);
  a.tab[1] = reinterpret_cast<const unsigned char* const*>(t1);
  a.off = off; a.m = m; a.tile_base = tile_base; a.job_of_tile = job_of_tile;
  a.xq = static_cast<const unsigned char*>(xq);
  a.y[0] = y0; a.y[1] = y1;
  a.n_rows = n_rows; a.nb = k / kQK; a.tok_tile = tok_per;
  a.status = status_word();
  const int rc = tile_rows(a.nb);
  const dim3 grid((n_rows + rc - 1) / rc, n_tiles);
  return tok_per == 1 ? launch_tile<NMAT, 1, kGrouped, true>(a, grid, stream)
                      : launch_tile<NMAT, 8, kGrouped, true>(a, grid, stream);
}

template <int NMAT>
int launch_tab(const void* const* t0, const void* const* t1, const int* off, const int* toff,
               const int* meta, int* mail, int* mail_n, int tiles_max, const void* xq, void* y0,
               void* y1, int n_rows, int k, int n_expert, int tok_per, cudaStream_t stream) {
  if (tiles_max <= 0) return kOk;
  if (!t0 || (NMAT == 2 && (!t1 || !y1)) || !off || !toff || !meta || !xq || !y0 || n_rows <= 0 ||
      k <= 0 || k % kQK != 0 || tok_per <= 0 || n_expert <= 0 || (mail && !mail_n))
    return kErrArg;
  if (reinterpret_cast<uintptr_t>(xq) & 3u) return kErrAlign;
  GemvArgs a{};
  a.tab[0] = reinterpret_cast<const unsigned char* const*>(t0);
  a.tab[1] = reinterpret_cast<const unsigned char* const*>(t1);
  a.off = off; a.toff = toff; a.meta = meta; a.mail = mail; a.mail_n = mail_n;
  a.xq = static_cast<const unsigned char*>(xq);
  a.y[0] = y0; a.y[1] = y1;
  a.n_rows = n_rows; a.nb = k / kQK; a.tok_tile = tok_per; a.n_expert = n_expert;
  a.status = status_word();
  const int rc = tile_rows(a.nb);
  const dim3 grid((n_rows + rc - 1) / rc, tiles_max);
  return tok_per == 1 ? launch_tile<NMAT, 1, kTab, true>(a, grid, stream)
                      : launch_tile<NMAT, 8, kTab, true>(a, grid, stream);
}

// Raw int32 sub-block dots of token 0: out[(r*nb + blk)*8 + s]. Parity probe for
// the integer unit every kernel shares (block_dot).
__global__ void subblock_dots_kernel(const unsigned char* w, const unsigned char* xq, int* out,
                                     int n_rows, int nb) {
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* wsm = smem;                       // one block per thread
  const XTile xt = xtile_at(smem + static_cast<size_t>(blockDim.x) * kW4, 1, nb);
  xtile_stage(xt, 1, [&](int) { return xq; }, threadIdx.x, blockDim.x);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;   // (row, blk) pair
  const bool live = i < n_rows * nb;
  if (live) {
    const unsigned char* src = w + static_cast<size_t>(i) * kW4;
    for (int b = 0; b < kW4 / 2; ++b)
      reinterpret_cast<uint16_t*>(wsm + threadIdx.x * kW4)[b] = reinterpret_cast<const uint16_t*>(src)[b];
  }
  __syncthreads();
  if (!live) return;
  float acc[1][1] = {{0.f}};
  int dots[8];
  const uint4* wb[1] = {reinterpret_cast<const uint4*>(wsm + threadIdx.x * kW4)};
  block_dot<1, 1>(wb, xt, i % nb, 1, acc, dots);
  for (int s = 0; s < 8; ++s) out[static_cast<size_t>(i) * 8 + s] = dots[s];
}

}  // namespace
}  // namespace sgr

using namespace sgr;

SGR_API int sgr_gemv_q4_k_q8(const void* w, const void* x_q8, float* y, int n_rows, int k,
                             void* stream) {
  return launch_dense<1, false>(w, nullptr, x_q8, y, nullptr, n_rows, k, 1, as_stream(stream));
}

SGR_API int sgr_gemv_q4_k_q8_f16out(const void* w, const void* x_q8, uint16_t* y, int n_rows, int k,
                                    void* stream) {
  return launch_dense<1, true>(w, nullptr, x_q8, y, nullptr, n_rows, k, 1, as_stream(stream));
}

// cuda_ops.hpp:169-171 of the reference: the fp16 GEMV and, on the rounded result, the residual add.
// Same kernels as sgr_gemv_q4_k_q8_f16out, so y is bit-identical to it and res_inout to an add after it.
SGR_API int sgr_gemv_q4_k_q8_f16out_resadd(const void* w, const void* x_q8, uint16_t* y, uint16_t* res_inout,
                                           int n_rows, int k, void* stream) {
  if (n_rows > 0 && !res_inout) return kErrArg;
  return launch_dense<1, true>(w, nullptr, x_q8, y, nullptr, n_rows, k, 1, as_stream(stream), res_inout);
}

namespace {
// cuda_ops.hpp:156-164 of the reference: two or three projections of one token row in one launch.
int launch_multi(int nmat, const void* const (&w)[3], const void* xq, uint16_t* const (&y)[3], const int (&rows)[3],
                 int k, cudaStream_t stream) {
  int total = 0;
  for (int m = 0; m < nmat; ++m) {
    if (rows[m] < 0) return kErrArg;
    total += rows[m];
  }
  if (total == 0) return kOk;
  if (!xq || k <= 0 || k % kQK != 0) return kErrArg;
  for (int m = 0; m < nmat; ++m)
    if (rows[m] > 0 && (!w[m] || !y[m])) return kErrArg;
  if (reinterpret_cast<uintptr_t>(xq) & 3u) return kErrAlign;
  GemvArgs a{};
  int cum = 0, tiles = 0;
  a.nb = k / kQK;
  const int rc = tile_rows(a.nb);
  for (int m = 0; m < 3; ++m) {
    const int r = m < nmat ? rows[m] : 0;
    a.wm[m] = m < nmat ? static_cast<const unsigned char*>(w[m]) : nullptr;
    a.ym[m] = m < nmat ? y[m] : nullptr;
    cum += r;
    a.rows_cum[m] = cum;
    tiles += (r + rc - 1) / rc;
  }
  a.xq = static_cast<const unsigned char*>(xq);
  a.n_rows = total;
  a.n_tokens = 1;
  a.tok_tile = 1;
  a.status = status_word();
  return launch_tile<1, 1, kMulti, true>(a, dim3(tiles, 1), stream);
}
}  // namespace

SGR_API int sgr_gemv2m_q4_k_q8_f16out(const void* w1, const void* w2, const void* xq, uint16_t* y1, uint16_t* y2,
                                      int rows1, int rows2, int k, int slot, void* stream) {
  (void)slot;                              // the reference keys a per-layer parameter block by it; nothing to key here
  const void* const w[3] = {w1, w2, nullptr};
  uint16_t* const y[3] = {y1, y2, nullptr};
  const int rows[3] = {rows1, rows2, 0};
  return launch_multi(2, w, xq, y, rows, k, as_stream(stream));
}

SGR_API int sgr_gemv3m_q4_k_q8_f16out(const void* w1, const void* w2, const void* w3, const void* xq, uint16_t* y1,
                                      uint16_t* y2, uint16_t* y3, int rows1, int rows2, int rows3, int k, int slot,
                                      void* stream) {
  (void)slot;
  const void* const w[3] = {w1, w2, w3};
  uint16_t* const y[3] = {y1, y2, y3};
  const int rows[3] = {rows1, rows2, rows3};
  return launch_multi(3, w, xq, y, rows, k, as_stream(stream));
}

SGR_API int sgr_gemv_q4_k_q8_batched(const void* w, const void* x_q8, float* y, int n_rows, int k,
                                     int n_tokens, void* stream) {
  return launch_dense<1, false>(w, nullptr, x_q8, y, nullptr, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_gemv_q4_k_q8_f16out_batched(const void* w, const void* x_q8, uint16_t* y,
                                            int n_rows, int k, int n_tokens, void* stream) {
  return launch_dense<1, true>(w, nullptr, x_q8, y, nullptr, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_gemv_q4_k_q8_f16out_mtok(const void* w, const void* xq, uint16_t* y, int n_rows,
                                         int k, int n_tokens, void* stream) {
  return launch_dense<1, true>(w, nullptr, xq, y, nullptr, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_mmq_q4_k_q8_f16out(const void* w, const void* xq, uint16_t* y, int n_rows, int k,
                                   int n_tokens, void* stream) {
  return launch_dense<1, true>(w, nullptr, xq, y, nullptr, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_gemv2_q4_k_q8_f16out_mtok(const void* wg, const void* wu, const void* xq,
                                          uint16_t* yg, uint16_t* yu, int n_rows, int k,
                                          int n_tokens, void* stream) {
  return launch_dense<2, true>(wg, wu, xq, yg, yu, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_mmq2_q4_k_q8_f16out(const void* wg, const void* wu, const void* xq, uint16_t* yg,
                                    uint16_t* yu, int n_rows, int k, int n_tokens, void* stream) {
  return launch_dense<2, true>(wg, wu, xq, yg, yu, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_gemv_ptrs_q4_k_q8_f16out(const void* const* ptrs, const void* x_q8, uint16_t* y,
                                         int n_ptrs, int rows_per, int k, void* stream) {
  if (n_ptrs <= 0 || rows_per <= 0) return kOk;
  if (!ptrs || !x_q8 || !y || k <= 0 || k % kQK != 0) return kErrArg;
  if (reinterpret_cast<uintptr_t>(x_q8) & 3u) return kErrAlign;
  GemvArgs a{};
  a.tab[0] = reinterpret_cast<const unsigned char* const*>(ptrs);
  a.xq = static_cast<const unsigned char*>(x_q8);
  a.y[0] = y;
  a.rows_per = rows_per;
  a.n_rows = rows_per;
  a.nb = k / kQK;
  a.tok_tile = 1;
  a.status = status_word();
  const int rc = tile_rows(a.nb);
  return launch_tile<1, 1, kPtrs, true>(a, dim3((rows_per + rc - 1) / rc, n_ptrs), as_stream(stream));
}

SGR_API int sgr_gemv_grouped2_q4_k_q8_f16out_mtok(const void* const* wg, const void* const* wu,
                                                  const int* off, const int* m,
                                                  const int* tile_base, const int* job_of_tile,
                                                  int n_tiles, const void* xq, uint16_t* yg,
                                                  uint16_t* yu, int n_rows, int k, int tok_per,
                                                  void* stream) {
  return launch_grouped<2>(wg, wu, off, m, tile_base, job_of_tile, n_tiles, xq, yg, yu, n_rows, k,
                           tok_per, as_stream(stream));
}

SGR_API int sgr_gemv_grouped_q4_k_q8_f16out_mtok(const void* const* w, const int* off, const int* m,
                                                 const int* tile_base, const int* job_of_tile,
                                                 int n_tiles, const void* xq, uint16_t* y,
                                                 int n_rows, int k, int tok_per, void* stream) {
  return launch_grouped<1>(w, nullptr, off, m, tile_base, job_of_tile, n_tiles, xq, y, nullptr,
                           n_rows, k, tok_per, as_stream(stream));
}

SGR_API int sgr_gemv_grouped2_tab_q4_k_q8_f16out_mtok(
    const void* const* wg_tab, const void* const* wu_tab, const int* off, const int* toff,
    const int* meta, int* mail, int* mail_n, int tiles_max, const void* xq, uint16_t* yg,
    uint16_t* yu, int n_rows, int k, int n_expert, int tok_per, void* stream) {
  return launch_tab<2>(wg_tab, wu_tab, off, toff, meta, mail, mail_n, tiles_max, xq, yg, yu, n_rows,
                       k, n_expert, tok_per, as_stream(stream));
}

SGR_API int sgr_gemv_grouped_tab_q4_k_q8_f16out_mtok(const void* const* w_tab, const int* off,
                                                     const int* toff, const int* meta,
                                                     int tiles_max, const void* xq, uint16_t* y,
                                                     int n_rows, int k, int n_expert, int tok_per,
                                                     void* stream) {
  return launch_tab<1>(w_tab, nullptr, off, toff, meta, nullptr, nullptr, tiles_max, xq, y, nullptr,
                       n_rows, k, n_expert, tok_per, as_stream(stream));
}

SGR_API int sgr_q4k_subblock_dots(const void* w, const void* x_q8, int* out, int n_rows, int k,
                                  void* stream) {
  if (!w || !x_q8 || !out || n_rows <= 0 || k <= 0 || k % kQK != 0) return kErrArg;
  if (reinterpret_cast<uintptr_t>(x_q8) & 3u) return kErrAlign;
  const int nb = k / kQK;
  const int threads = 128;
  const size_t smem = static_cast<size_t>(threads) * kW4 + xtile_bytes(1, nb);
  if (smem > 48 * 1024) return kErrUnsupported;
  subblock_dots_kernel<<<(n_rows * nb + threads - 1) / threads, threads, smem, as_stream(stream)>>>(
      static_cast<const unsigned char*>(w), static_cast<const unsigned char*>(x_q8), out, n_rows, nb);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}
