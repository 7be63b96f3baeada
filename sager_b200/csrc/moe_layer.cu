// moe_layer.cu - one MoE layer of a decode step (1..64 token rows) in three
// launches chained with programmatic dependent launch:
//
//   route    : Q8_K-quantise the rows, router logits, softmax/top-k, and - in the
//              last CTA to finish - the expert-major plan of the layer
//   gate_up  : for every (expert, 16-token tile, 16-row chunk): gate and up
//              projections and SwiGLU, fp32 h rows
//   down     : for every (expert, tile, 64-row chunk): Q8_K-quantise h in the
//              prologue, down projection, fp32 y rows; the last CTA to finish a
//              row chunk adds residual + sum_k w_k * y_k + shared expert
//
// It replaces the launch sequence of the reference's device-dispatch path
// (Session::moe_dispatch_device, src/core/session.cpp:2482-3030: quantize_q8_k,
// gemv_f32_out_f16x_mtok, router_topk_batched, moe_dispatch_scan,
// gather_rows_q8_n, gemv_grouped2_tab, silu_mul_f16_n, quantize_q8_k_n,
// gemv_grouped_tab, scatter_routed_f16, the shared-expert chain and
// moe_combine_batched_f16) and keeps its contracts: [3][E] pointer table with
// null = absent expert (zero contribution + mailbox), route_idx / route_w rows of
// stride K+1 with slot K = shared expert, bounds-invalid ids silence their row.
// Arithmetic follows the CPU expert FFN (src/kernels/cpu/q4_avx2.cpp:175-196):
// g, u, h and y stay fp32 and h is quantised from fp32, so the result tracks the
// AVX2 path more closely than the reference's fp16-staged device path does.
//
// Every weight byte is read once: the weight rows of a CTA arrive by one TMA
// bulk copy, the down kernel issues its copies before it waits for gate_up, and
// the route kernel prefetches the router matrix into L2 before it waits for the
// previous layer.
#include <algorithm>

#include "api_util.cuh"
#include "quantize_dev.cuh"
#include "router_dev.cuh"
#include "tile.cuh"

namespace sgr {

namespace {

constexpr int kMaxRows = 64;       // token rows per call (row masks are 64-bit)
constexpr int kTokTile = 16;       // token rows per CTA of the expert kernels
constexpr int kRouteTok = 8;       // token rows per CTA of the route kernel
constexpr int kRouteWarps = 4;

struct LayerDev {
  int n, H, FF, E, K, nbh, nbf;
  int e_lo, e_hi, sh_lo, sh_hi;
  int add_residual, routing_given;
  float shared_w;
  const uint16_t* xn;
  const unsigned char* xq_in;
  const float* router_w;
  const float* bias;
  const unsigned char* const* tab;
  const unsigned char* sh[3];
  uint16_t* x_f16;
  float* out_f32;
  int* idx;
  float* w;
  int* mail;
  int* mail_n;
  // workspace
  unsigned char* xq;
  float* logits;
  int* off;        // [E+1] exclusive prefix of routed rows per expert
  int* tile_e;     // [max_tiles] expert of a tile (E = shared expert)
  int* tile_t0;    // [max_tiles] first row of the tile inside its expert
  int* meta;       // {routed rows, tiles incl. shared, bad ids, -}
  int* gslot;      // [n*K] grouped slot of a route, -1 = not computed here
  int* grows;      // [n*K] source row of a grouped slot
  unsigned* cnt;   // [0..7] route tiles, [8] route tiles done, [16..] down row chunks
  float* hbuf;     // [(n_max*K + n_max)][FF]
  float* ybuf;     // [(n_max*K + n_max)][H]
  int n_max;
  int* status;
};

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct WsLayout {
  size_t xq, logits, off, tile_e, tile_t0, meta, gslot, grows, cnt, hbuf, ybuf, total;
};
inline WsLayout ws_layout(int n_max, int H, int FF, int E, int K) {
  WsLayout l{};
  size_t p = 0;
  const size_t rows = static_cast<size_t>(n_max) * K + n_max;
  const size_t tiles = static_cast<size_t>(n_max) * K + n_max;
  auto take = [&](size_t bytes) { const size_t at = p; p = align_up(p + bytes, 256); return at; };
  l.xq = take(static_cast<size_t>(n_max) * (H / kQK) * kX8);
  l.logits = take(static_cast<size_t>(n_max) * E * 4);
  l.off = take(static_cast<size_t>(E + 2) * 4);
  l.tile_e = take(tiles * 4);
  l.tile_t0 = take(tiles * 4);
  l.meta = take(16);
  l.gslot = take(static_cast<size_t>(n_max) * K * 4);
  l.grows = take(static_cast<size_t>(n_max) * K * 4);
  l.cnt = take((16 + static_cast<size_t>(H) / 64 + 1) * 4);
  l.hbuf = take(rows * FF * 4);
  l.ybuf = take(rows * H * 4);
  l.total = p;
  return l;
}

// ---- plan ------------------------------------------------------------------------
// One CTA (128 threads). Row sets per expert are 64-bit masks, so the slot of a
// route inside its expert is a popcount: the plan is deterministic (ascending
// row order) and needs no sort. Routes to experts outside [e_lo, e_hi) are left
// to their owner (gslot = -1); ids outside [0, E) silence their row as in
// moe_dispatch_scan (moe.cu:385-398 of the reference).
__device__ void build_plan(const LayerDev& L, unsigned char* smem) {
  unsigned long long* mask = reinterpret_cast<unsigned long long*>(smem);       // [E]
  int* scan_rows = reinterpret_cast<int*>(smem + static_cast<size_t>(L.E) * 8);   // [128]
  int* scan_tiles = scan_rows + 128;                                              // [128]
  __shared__ int bad_sh;
  const int tid = threadIdx.x;
  const int total = L.n * L.K;
  if (tid == 0) bad_sh = 0;
  for (int e = tid; e < L.E; e += blockDim.x) mask[e] = 0ull;
  __syncthreads();
  for (int i = tid; i < total; i += blockDim.x) {
    const int r = i / L.K, kk = i - r * L.K;
    const int e = __ldcg(L.idx + static_cast<size_t>(r) * (L.K + 1) + kk);
    if (e < 0 || e >= L.E) {
      for (int q = 0; q <= L.K; ++q) L.w[static_cast<size_t>(r) * (L.K + 1) + q] = 0.f;
      atomicAdd(&bad_sh, 1);
    } else if (e >= L.e_lo && e < L.e_hi) {
      atomicOr(&mask[e], 1ull << r);
    }
  }
  __syncthreads();
  // exclusive prefixes of rows and tiles over experts: each thread owns a run of experts
  const int per = (L.E + blockDim.x - 1) / blockDim.x;
  const int e0 = tid * per, e1 = min(L.E, e0 + per);
  int rows = 0, tiles = 0;
  for (int e = e0; e < e1; ++e) {
    const int c = __popcll(mask[e]);
    rows += c;
    tiles += (c + kTokTile - 1) / kTokTile;
  }
  scan_rows[tid] = rows;
  scan_tiles[tid] = tiles;
  __syncthreads();
  if (tid == 0) {
    int ar = 0, at = 0;
    for (int i = 0; i < static_cast<int>(blockDim.x); ++i) {
      const int r = scan_rows[i], t = scan_tiles[i];
      scan_rows[i] = ar;
      scan_tiles[i] = at;
      ar += r;
      at += t;
    }
    // shared expert: tiles over the rows [sh_lo, sh_hi), appended after the routed ones
    int sh_tiles = 0;
    if (L.sh[0] != nullptr && L.sh_hi > L.sh_lo) {
      sh_tiles = (L.sh_hi - L.sh_lo + kTokTile - 1) / kTokTile;
      for (int i = 0; i < sh_tiles; ++i) {
        L.tile_e[at + i] = L.E;
        L.tile_t0[at + i] = i * kTokTile;
      }
    }
    L.off[L.E] = ar;
    L.meta[0] = ar;
    L.meta[1] = at + sh_tiles;
    L.meta[2] = bad_sh;
    L.meta[3] = at;
    if (L.mail_n != nullptr) *L.mail_n = 0;
  }
  __syncthreads();
  {
    int ar = scan_rows[tid], at = scan_tiles[tid];
    for (int e = e0; e < e1; ++e) {
      const int c = __popcll(mask[e]);
      L.off[e] = ar;
      for (int t0 = 0; t0 < c; t0 += kTokTile) {
        L.tile_e[at] = e;
        L.tile_t0[at] = t0;
        ++at;
      }
      ar += c;
    }
  }
  __syncthreads();
  for (int i = tid; i < total; i += blockDim.x) {
    const int r = i / L.K, kk = i - r * L.K;
    const int e = __ldcg(L.idx + static_cast<size_t>(r) * (L.K + 1) + kk);
    int pos = -1;
    if (e >= L.e_lo && e < L.e_hi && e >= 0 && e < L.E) {
      pos = L.off[e] + __popcll(mask[e] & ((1ull << r) - 1ull));
      L.grows[pos] = r;
    }
    L.gslot[i] = pos;
  }
}

constexpr size_t plan_smem(int E) { return static_cast<size_t>(E) * 8 + 2 * 128 * 4; }

// ---- launch 1: route ------------------------------------------------------------------
// grid (ceil(E / 4), ceil(n / 8)), 128 threads. Dynamic smem: max(8 rows of fp16 x,
// 4*E floats for the selection, plan scratch).
__global__ void __launch_bounds__(kRouteWarps * 32) route_kernel(const LayerDev L) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int last_sh;
  uint16_t* xs = reinterpret_cast<uint16_t*>(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok0 = blockIdx.y * kRouteTok;
  const int nt = min(kRouteTok, L.n - tok0);
  const int row = blockIdx.x * kRouteWarps + warp;

  // The router matrix does not depend on the previous layer: pull this warp's row
  // towards L2 while the previous kernel drains.
  if (row < L.E && blockIdx.y == 0) {
    const char* wr = reinterpret_cast<const char*>(L.router_w + static_cast<size_t>(row) * L.H);
    for (int b = lane * 128; b < L.H * 4; b += 32 * 128)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(wr + b));
  }
  pdl_wait();
  pdl_launch_dependents();

  for (int i = tid; i < nt * L.H / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(xs)[i] =
        reinterpret_cast<const uint4*>(L.xn + static_cast<size_t>(tok0) * L.H)[i];
  __syncthreads();

  if (L.xq_in == nullptr) {
    for (int b = blockIdx.x * kRouteWarps + warp; b < nt * L.nbh; b += gridDim.x * kRouteWarps) {
      const int t = b / L.nbh, blk = b - t * L.nbh;
      quantize_block_f16(xs + static_cast<size_t>(t) * L.H + blk * kQK,
                         L.xq + (static_cast<size_t>(tok0 + t) * L.nbh + blk) * kX8, lane);
    }
  }
  if (row < L.E) {
    float out[kRouteTok];
    router_row_dot<kRouteTok>(L.router_w + static_cast<size_t>(row) * L.H, xs, L.H, nt, lane, out);
    if (lane == 0) {
      const float b = L.bias != nullptr ? L.bias[row] : 0.f;
#pragma unroll
      for (int t = 0; t < kRouteTok; ++t)
        if (t < nt) L.logits[static_cast<size_t>(tok0 + t) * L.E + row] = out[t] + b;
    }
  }
  // last CTA of this token tile selects
  __threadfence();
  __syncthreads();
  if (tid == 0) last_sh = atomicAdd(&L.cnt[blockIdx.y], 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (!last_sh) return;
  __threadfence();
  float* prob = reinterpret_cast<float*>(smem) + static_cast<size_t>(warp) * L.E;
  for (int t = warp; t < nt; t += kRouteWarps) {
    for (int i = lane; i < L.E; i += 32) prob[i] = __ldcg(L.logits + static_cast<size_t>(tok0 + t) * L.E + i);
    __syncwarp();
    router_select_warp(prob, L.E, L.K, L.idx + static_cast<size_t>(tok0 + t) * (L.K + 1),
                       L.w + static_cast<size_t>(tok0 + t) * (L.K + 1), L.shared_w, true, lane);
    __syncwarp();
  }
  // last token tile plans
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    L.cnt[blockIdx.y] = 0u;
    last_sh = atomicAdd(&L.cnt[8], 1u) == gridDim.y - 1 ? 1 : 0;
  }
  __syncthreads();
  if (!last_sh) return;
  __threadfence();
  if (tid == 0) L.cnt[8] = 0u;
  build_plan(L, smem);
}

// Routing supplied by the caller (expert-parallel owner side): plan only.
__global__ void __launch_bounds__(128) plan_kernel(const LayerDev L) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_launch_dependents();
  build_plan(L, smem);
}

// ---- shared decode of a tile index -------------------------------------------------------
struct TileRef {
  int e;        // expert, E = shared
  int ntok;     // rows in this tile
  int hrow0;    // first row of the tile in hbuf / ybuf
  int p0;       // first grouped slot (routed) or first token row (shared)
};
__device__ __forceinline__ bool decode_tile(const LayerDev& L, int tile, TileRef* t) {
  if (tile >= L.meta[1]) return false;
  t->e = L.tile_e[tile];
  const int t0 = L.tile_t0[tile];
  if (t->e == L.E) {
    t->ntok = min(kTokTile, L.sh_hi - L.sh_lo - t0);
    t->p0 = L.sh_lo + t0;
    t->hrow0 = L.n_max * L.K + L.sh_lo + t0;
  } else {
    const int o = L.off[t->e];
    t->ntok = min(kTokTile, L.off[t->e + 1] - o - t0);
    t->p0 = o + t0;
    t->hrow0 = o + t0;
  }
  return t->ntok > 0;
}

// ---- launch 2: gate + up + SwiGLU ------------------------------------------------------------
// grid (FF / tile_rows(nbh), max tiles), 128 threads
template <int TT>
__global__ void __launch_bounds__(kTileThreads) gate_up_kernel(const LayerDev L) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_launch_dependents();
  TileRef t;
  if (!decode_tile(L, blockIdx.y, &t)) return;
  const int rc = tile_rows(L.nbh);
  const int row0 = blockIdx.x * rc;
  const int nrows = min(rc, L.FF - row0);
  const size_t row_bytes = static_cast<size_t>(L.nbh) * kW4;
  const bool shared = t.e == L.E;
  const unsigned char* wg = shared ? L.sh[0] : L.tab[t.e];
  const unsigned char* wu = shared ? L.sh[1] : L.tab[L.E + t.e];
  const unsigned char* wd = shared ? L.sh[2] : L.tab[2 * L.E + t.e];
  if (wg == nullptr || wu == nullptr || wd == nullptr) {
    // absent expert: the down kernel writes zero rows; post the id once per tile
    if (L.mail != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && !shared) {
      const int mi = atomicAdd(L.mail_n, 1);
      if (mi < L.E) L.mail[mi] = t.e;
    }
    return;
  }
  const unsigned char* wsrc[2] = {wg + row0 * row_bytes, wu + row0 * row_bytes};
  const unsigned char* xq = L.xq_in != nullptr ? L.xq_in : L.xq;
  const size_t xrow_bytes = static_cast<size_t>(L.nbh) * kX8;
  tile_run<2, TT>(
      smem, wsrc, nrows, L.nbh, t.ntok,
      [&](int i) {
        const int r = shared ? t.p0 + i : L.grows[t.p0 + i];
        return xq + r * xrow_bytes;
      },
      [&](int r, int t0, int nt, float (&res)[2][TT]) {
#pragma unroll
        for (int i = 0; i < TT; ++i)
          if (i < nt) {
            const float g = res[0][i], u = res[1][i];
            L.hbuf[static_cast<size_t>(t.hrow0 + t0 + i) * L.FF + row0 + r] = g / (1.f + expf(-g)) * u;
          }
      },
      L.status);
}

// Q8_K-quantise fp32 rows straight into a staged tile (one warp per 256 values;
// arithmetic of src/kernels/cpu/q4_avx2.cpp:77-94 in the reference).
__device__ __forceinline__ void stage_quantized_f32(const XTile& xt, int nt, const float* src,
                                                    size_t row_stride) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int job = warp; job < nt * xt.nb; job += kTileThreads / 32) {
    const int t = job / xt.nb, blk = job - t * xt.nb;
    const float4* p = reinterpret_cast<const float4*>(src + t * row_stride + blk * kQK) + lane * 2;
    const float4 a = __ldcg(p), b = __ldcg(p + 1);
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    const float amax = fmaxf(1e-30f, m);
    const float d = amax / 127.f;
    const float id = d > 0.f ? 1.f / d : 0.f;
    int q[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      q[i] = max(-127, min(127, static_cast<int>(rintf(v[i] * id))));
      sum += q[i];
    }
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    int8_t* qs = xt.qs + (static_cast<size_t>(t) * xt.nb + blk) * kXqStride + lane * 8;
    reinterpret_cast<uint32_t*>(qs)[0] = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) |
                                         (static_cast<uint32_t>(q[3] & 0xFF) << 24);
    reinterpret_cast<uint32_t*>(qs)[1] = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) |
                                         (static_cast<uint32_t>(q[7] & 0xFF) << 24);
    if ((lane & 3) == 0) xt.bs[(static_cast<size_t>(t) * xt.nb + blk) * 8 + (lane >> 2)] = static_cast<int16_t>(sum);
    if (lane == 0) xt.d[t * xt.nb + blk] = d;
  }
}

// ---- launch 3: down projection + combine ---------------------------------------------------------
// grid (H / tile_rows(nbf), max tiles), 128 threads
template <int TT>
__global__ void __launch_bounds__(kTileThreads) down_kernel(const LayerDev L) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int last_sh;
  const int rc = tile_rows(L.nbf);
  const int row0 = blockIdx.x * rc;
  const int nrows = min(rc, L.H - row0);
  const size_t row_bytes = static_cast<size_t>(L.nbf) * kW4;
  // The plan is final here: this grid starts only after every gate_up CTA passed
  // its own wait on the route kernel.
  const int n_tiles = L.meta[1];
  TileRef t;
  const bool live = decode_tile(L, blockIdx.y, &t);
  if (!live && !(blockIdx.y == 0 && n_tiles == 0)) return;

  if (live) {
    const bool shared = t.e == L.E;
    const unsigned char* wg = shared ? L.sh[0] : L.tab[t.e];
    const unsigned char* wu = shared ? L.sh[1] : L.tab[L.E + t.e];
    const unsigned char* wd = shared ? L.sh[2] : L.tab[2 * L.E + t.e];
    if (wg == nullptr || wu == nullptr || wd == nullptr) {
      for (int i = threadIdx.x; i < nrows * t.ntok; i += kTileThreads)
        L.ybuf[static_cast<size_t>(t.hrow0 + i / nrows) * L.H + row0 + i % nrows] = 0.f;
      pdl_wait();
    } else {
      const unsigned char* wsrc[1] = {wd + row0 * row_bytes};
      tile_run_staged<1, TT>(
          smem, wsrc, nrows, L.nbf, t.ntok, [] { pdl_wait(); },
          [&](const XTile& xt, int t0, int nt) {
            stage_quantized_f32(xt, nt, L.hbuf + static_cast<size_t>(t.hrow0 + t0) * L.FF, L.FF);
          },
          [&](int r, int t0, int nt, float (&res)[1][TT]) {
#pragma unroll
            for (int i = 0; i < TT; ++i)
              if (i < nt) L.ybuf[static_cast<size_t>(t.hrow0 + t0 + i) * L.H + row0 + r] = res[0][i];
          },
          L.status);
    }
  } else {
    pdl_wait();
  }
  pdl_launch_dependents();

  // last CTA of this row chunk blends
  const unsigned expected = n_tiles > 0 ? static_cast<unsigned>(n_tiles) : 1u;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_sh = atomicAdd(&L.cnt[16 + blockIdx.x], 1u) == expected - 1 ? 1 : 0;
  __syncthreads();
  if (!last_sh) return;
  __threadfence();
  if (threadIdx.x == 0) L.cnt[16 + blockIdx.x] = 0u;
  const bool has_shared = L.sh[0] != nullptr && L.sh[1] != nullptr && L.sh[2] != nullptr;
  for (int i = threadIdx.x; i < nrows * L.n; i += kTileThreads) {
    const int tk = i / nrows, r = row0 + i % nrows;
    const size_t o = static_cast<size_t>(tk) * L.H + r;
    float acc = (L.add_residual && L.x_f16 != nullptr) ? h2f(L.x_f16[o]) : 0.f;
    const float* wr = L.w + static_cast<size_t>(tk) * (L.K + 1);
    for (int kk = 0; kk < L.K; ++kk) {
      const int gs = L.gslot[tk * L.K + kk];
      if (gs >= 0) acc += __ldcg(wr + kk) * __ldcg(L.ybuf + static_cast<size_t>(gs) * L.H + r);
    }
    if (has_shared && tk >= L.sh_lo && tk < L.sh_hi)
      acc += __ldcg(wr + L.K) * __ldcg(L.ybuf + static_cast<size_t>(L.n_max * L.K + tk) * L.H + r);
    if (L.out_f32 != nullptr) L.out_f32[o] = acc;
    if (L.x_f16 != nullptr && L.add_residual) L.x_f16[o] = f2h(acc);
  }
}

template <typename Kern>
int launch_pdl(Kern kern, dim3 grid, int threads, size_t smem, cudaStream_t stream,
               const LayerDev& L) {
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return kErrLaunch;
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
  return cudaLaunchKernelEx(&cfg, kern, L) == cudaSuccess ? kOk : kErrLaunch;
}

}  // namespace
}  // namespace sgr

using namespace sgr;

SGR_API size_t sgr_moe_layer_workspace_bytes(int n_max, int hidden, int n_ff, int n_expert,
                                             int n_used) {
  if (n_max <= 0 || n_max > kMaxRows || hidden <= 0 || hidden % kQK || n_ff <= 0 || n_ff % kQK ||
      n_expert <= 0 || n_used <= 0)
    return 0;
  return ws_layout(n_max, hidden, n_ff, n_expert, n_used).total;
}

SGR_API int sgr_moe_layer_workspace_init(void* workspace, size_t bytes, void* stream) {
  if (!workspace || bytes == 0) return kErrArg;
  return cudaMemsetAsync(workspace, 0, bytes, as_stream(stream)) == cudaSuccess ? kOk : kErrLaunch;
}

SGR_API int sgr_moe_layer_decode(const sgr_moe_layer* a, void* stream) {
  if (a == nullptr) return kErrArg;
  if (a->n <= 0) return kOk;
  if (a->hidden <= 0 || a->hidden % kQK || a->n_ff <= 0 || a->n_ff % kQK || a->n_expert <= 0 ||
      a->n_used <= 0 || a->n_used > a->n_expert || a->n_max < a->n || a->n_max > kMaxRows)
    return kErrGeometry;
  if (a->n_expert > 1024 || a->hidden > 8192 || a->n_ff > 8192) return kErrUnsupported;
  if (!a->w_tab || !a->route_idx || !a->route_w || !a->workspace || (!a->x_f16 && !a->out_f32))
    return kErrArg;
  if (!a->routing_given && (!a->xn || !a->router_w)) return kErrArg;
  if (a->routing_given && !a->xq_in && !a->xn) return kErrArg;
  if (a->mail && !a->mail_n) return kErrArg;
  const WsLayout lay = ws_layout(a->n_max, a->hidden, a->n_ff, a->n_expert, a->n_used);
  if (a->workspace_bytes < lay.total) return kErrArg;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 255u) ||
      (a->xn && (reinterpret_cast<uintptr_t>(a->xn) & 15u)) ||
      (a->xq_in && (reinterpret_cast<uintptr_t>(a->xq_in) & 3u)))
    return kErrAlign;

  LayerDev L{};
  L.n = a->n; L.H = a->hidden; L.FF = a->n_ff; L.E = a->n_expert; L.K = a->n_used;
  L.nbh = a->hidden / kQK; L.nbf = a->n_ff / kQK;
  L.e_lo = a->expert_lo; L.e_hi = a->expert_hi > 0 ? a->expert_hi : a->n_expert;
  L.sh_lo = a->shared_lo; L.sh_hi = a->shared_hi > 0 ? a->shared_hi : a->n;
  if (L.e_lo < 0 || L.e_hi > L.E || L.e_lo > L.e_hi || L.sh_lo < 0 || L.sh_hi > L.n || L.sh_lo > L.sh_hi)
    return kErrGeometry;
  L.add_residual = a->no_residual ? 0 : 1;
  L.routing_given = a->routing_given;
  L.shared_w = a->shared_w;
  L.xn = a->xn;
  L.xq_in = static_cast<const unsigned char*>(a->xq_in);
  L.router_w = a->router_w;
  L.bias = a->router_bias;
  L.tab = reinterpret_cast<const unsigned char* const*>(a->w_tab);
  L.sh[0] = static_cast<const unsigned char*>(a->shared_gate);
  L.sh[1] = static_cast<const unsigned char*>(a->shared_up);
  L.sh[2] = static_cast<const unsigned char*>(a->shared_down);
  if (!L.sh[0] || !L.sh[1] || !L.sh[2]) L.sh[0] = L.sh[1] = L.sh[2] = nullptr;
  L.x_f16 = a->x_f16;
  L.out_f32 = a->out_f32;
  L.idx = a->route_idx;
  L.w = a->route_w;
  L.mail = a->mail;
  L.mail_n = a->mail_n;
  unsigned char* ws = static_cast<unsigned char*>(a->workspace);
  L.xq = ws + lay.xq;
  L.logits = reinterpret_cast<float*>(ws + lay.logits);
  L.off = reinterpret_cast<int*>(ws + lay.off);
  L.tile_e = reinterpret_cast<int*>(ws + lay.tile_e);
  L.tile_t0 = reinterpret_cast<int*>(ws + lay.tile_t0);
  L.meta = reinterpret_cast<int*>(ws + lay.meta);
  L.gslot = reinterpret_cast<int*>(ws + lay.gslot);
  L.grows = reinterpret_cast<int*>(ws + lay.grows);
  L.cnt = reinterpret_cast<unsigned*>(ws + lay.cnt);
  L.hbuf = reinterpret_cast<float*>(ws + lay.hbuf);
  L.ybuf = reinterpret_cast<float*>(ws + lay.ybuf);
  L.n_max = a->n_max;
  L.status = status_word();
  cudaStream_t s = as_stream(stream);

  int rc;
  if (!a->routing_given) {
    const size_t smem = std::max<size_t>(
        std::max<size_t>(static_cast<size_t>(kRouteTok) * L.H * 2, static_cast<size_t>(kRouteWarps) * L.E * 4),
        plan_smem(L.E));
    rc = launch_pdl(route_kernel, dim3((L.E + kRouteWarps - 1) / kRouteWarps, (L.n + kRouteTok - 1) / kRouteTok),
                    kRouteWarps * 32, smem, s, L);
  } else {
    if (!a->xq_in) return kErrArg;
    rc = launch_pdl(plan_kernel, dim3(1), 128, plan_smem(L.E), s, L);
  }
  if (rc != kOk) return rc;

  const int local_e = L.e_hi - L.e_lo;
  const int routed_tiles = std::min(L.n * L.K, local_e + L.n * L.K / kTokTile);
  const int max_tiles = std::max(1, routed_tiles + (L.sh_hi - L.sh_lo + kTokTile - 1) / kTokTile);
  const dim3 g2((L.FF + tile_rows(L.nbh) - 1) / tile_rows(L.nbh), max_tiles);
  const dim3 g3((L.H + tile_rows(L.nbf) - 1) / tile_rows(L.nbf), max_tiles);
  if (L.n == 1) {
    rc = launch_pdl(gate_up_kernel<1>, g2, kTileThreads, tile_smem(2, L.nbh, 1), s, L);
    if (rc != kOk) return rc;
    return launch_pdl(down_kernel<1>, g3, kTileThreads, tile_smem(1, L.nbf, 1), s, L);
  }
  rc = launch_pdl(gate_up_kernel<4>, g2, kTileThreads, tile_smem(2, L.nbh, 4), s, L);
  if (rc != kOk) return rc;
  return launch_pdl(down_kernel<4>, g3, kTileThreads, tile_smem(1, L.nbf, 4), s, L);
}
