// moe_layer.cu - one MoE layer of a decode step (1..64 token rows) in two
// launches chained with programmatic dependent launch:
//
//   route   : Q8_K-quantise the rows, router logits, softmax/top-k, and - in the
//             last CTA to finish - the expert-major plan of the layer (tiles of up
//             to 16 rows per expert)
//   experts : a persistent kernel, one CTA per SM. Work items are (tile, row chunk)
//             pairs: first every gate/up item (16 rows of gate and of up for one
//             tile: SwiGLU, fp32 h rows), then every down item (64 rows of the down
//             matrix: Q8_K-quantise h, fp32 y rows). A producer warp streams the
//             weight rows of the CTA's items through a ring of shared-memory
//             stages with TMA bulk copies, several items ahead of the eight
//             consumer warps, which run int8 tensor-core MMAs on them. Down items
//             wait (bounded) for the gate/up items of their tile; their weights are
//             already in flight by then. The last CTA to finish a 64-row chunk of
//             the output adds residual + sum_k w_k * y_k + shared expert.
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
// Every weight byte is read once, and the weight stream never stops at the
// gate/up -> down dependency. The route kernel prefetches the router matrix into
// L2 before it waits for the previous layer.
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <mutex>

#include "api_util.cuh"
#include "quantize_dev.cuh"
#include "router_dev.cuh"
#include "tile.cuh"

namespace sgr {

namespace {

constexpr int kMaxRows = 64;       // token rows per call (row masks are 64-bit)
constexpr int kTokTile = 8;        // token rows per tile of the item kernel (one MMA n-tile)
constexpr int kMaxGrid = 192;            // most CTAs the expert kernels are launched with
constexpr int kTmapSlots = 6;            // patched TMA descriptor sets per CTA of the row-streaming kernel
constexpr int kTokenKernelMaxRows = 3;   // layers of up to this many token rows run as one persistent launch
                                         // (measured per layer, us: 26.6 / 36.1 / 44.7 against 30.1 / 39.6 / 47.3 for
                                         // route + expert kernel; at 4 rows 57 against 50)
constexpr int kRowsKernelMinRows = 4;    // layers of at least this many token rows run the row-streaming kernel
                                         // (measured: 4 rows 8 % faster, 8 rows 16 %, 2 rows slower)
constexpr int kRouteTok = 8;       // token rows per CTA of the route kernel
constexpr int kRouteWarps = 8;
constexpr int kRouteRows = 2 * kRouteWarps;   // experts per CTA of the route kernel: two rows per warp

constexpr int kTeams = 2;                         // consumer teams, items alternate between them
constexpr int kTeamWarps = 8;
constexpr int kTeamThreads = kTeamWarps * 32;
constexpr int kConsumers = kTeams * kTeamThreads;
constexpr int kProducerWarps = 4;
constexpr int kStreamThreads = kConsumers + kProducerWarps * 32;
constexpr int kStages = 4;
constexpr unsigned kSpinLimit = 1u << 22;         // bounded waits: give up, raise the status word

struct LayerDev {
  int n, H, FF, E, K, nbh, nbf;
  int e_lo, e_hi, sh_lo, sh_hi;
  int add_residual, routing_given, skip_plan;
  int plan_in_kernel;  // the row-streaming kernel builds the plan itself, in shared memory, from the routing
  // a second workspace whose counters this call's route stage re-arms (expert parallelism: the owner call that follows)
  unsigned *rearm_cnt, *rearm_tile_cnt, *rearm_blk_cnt, *rearm_ready;
  int* rearm_mail_n;
  int rearm_tiles;
  int rstride;     // elements between consecutive rows of idx / w (K+1 when packed)
  int xq_stride;   // bytes between consecutive Q8_K rows
  float shared_w;
  const uint16_t* xn;
  const unsigned char* xq_in;
  const float* router_w;
  const float* bias;
  const unsigned char* const* tab;
  long long tab_stride;   // pointers between the gate, up and down slices of the table (E when packed)
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
  int4* rec;       // [max_tiles] {expert (E = shared), rows, first h/y row, first slot / token row}
  int* meta;       // {routed rows, tiles incl. shared, bad ids, routed tiles}
  int* gslot;      // [n*K] grouped slot of a route, -1 = not computed here
  int* grows;      // [n*K] source row of a grouped slot
  unsigned* cnt;   // [0..7] route tiles, [8] route tiles done, [9] expert kernel grid barrier, [10] next group
  unsigned* tile_cnt;  // [max_tiles] finished gate/up items per tile
  unsigned* blk_cnt;   // [max_tiles][nbf] row-streaming kernel: warps done with a 256-wide block of h
  unsigned* ready;     // [max_tiles] row-streaming kernel: quantised blocks of h published
  unsigned char* hq;   // [(n_max*K + n_max)][nbf] Q8_K rows of h, 288-byte blocks (row-streaming kernel)
  int tok_tile;        // token rows per tile: 8 (item kernel) or 16 (row-streaming kernel)
  unsigned char* xq16; // the quantised rows once more in 288-byte blocks (row-streaming kernel)
  int xq16_stride;     // bytes between its rows (nbh * 288 in the workspace; the record stride for padded records)
  int xq_padded;       // the caller's xq_in / xq_out rows are in 288-byte blocks already
  int grid;            // CTAs of the expert kernel
  const unsigned* wait_flags;   // expert parallelism over peer memory: arrival words to wait for before planning
  const unsigned* wait_step;
  int wait_count, wait_mul, wait_add;
  unsigned wait_limit;          // polls before a wait for arrival words gives up
  // expert parallelism, exchanges done by the layer's own kernels over peer memory:
  //   home side (route without plan): the records just written (rows of ep_rec bytes at ep_src) go to
  //   slot ep_dst[p] of every peer p < ep_world, then the peers' arrival words ep_flags[p] are set;
  //   owner side: row t of the result goes to ep_out[t / ep_home] + (t % ep_home) * H (the home rank's
  //   buffer) instead of out_f32, then the home ranks' arrival words ep_flags[p] are set.
  void* const* ep_dst;
  unsigned* const* ep_flags;
  float* const* ep_out;
  const unsigned char* ep_src;
  const unsigned* ep_step;
  int ep_world, ep_rec, ep_home, ep_mul, ep_add;
  unsigned char* tmaps;   // [grid][kTmapSlots][3][128] row-streaming kernel: patched TMA descriptors
  // TMA descriptors (placeholder address) of a gate / up matrix and of a down matrix. Only ever
  // read with constant indices: a dynamic index would make every thread keep a local-memory
  // copy of the whole argument block.
  alignas(64) uint32_t tmap_gu[32];
  alignas(64) uint32_t tmap_dn[32];
  float* hbuf;     // [(n_max*K + n_max)][FF]
  float* ybuf;     // [(n_max*K + n_max)][H]
  int n_max;
  int* status;
};


__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct WsLayout {
  size_t xq, logits, off, rec, meta, gslot, grows, cnt, tile_cnt, blk_cnt, ready, hbuf, ybuf, hq, xq16, tmaps, total;
  size_t items_total;   // what the item kernel needs: everything up to and including ybuf
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
  l.rec = take(tiles * 16);
  l.meta = take(16);
  l.gslot = take(static_cast<size_t>(n_max) * K * 4);
  l.grows = take(static_cast<size_t>(n_max) * K * 4);
  l.cnt = take((16 + static_cast<size_t>(H) / 16 + 1) * 4);
  l.tile_cnt = take(tiles * 4);
  l.blk_cnt = take(tiles * (FF / kQK) * 4);
  l.ready = take(tiles * 4);
  l.hbuf = take(rows * FF * 4);
  l.ybuf = take(rows * H * 4);
  l.items_total = p;
  l.hq = take(rows * (FF / kQK) * 288);     // padded Q8_K blocks (rs::kHq)
  l.xq16 = take(static_cast<size_t>(n_max) * (H / kQK) * 288);
  l.tmaps = take(static_cast<size_t>(kMaxGrid) * kTmapSlots * 3 * 128);
  l.total = p;
  return l;
}

// ---- plan ------------------------------------------------------------------------
// One CTA. Row sets per expert are 64-bit masks, so the slot of a
// route inside its expert is a popcount: the plan is deterministic (ascending
// row order) and needs no sort. Routes to experts outside [e_lo, e_hi) are left
// to their owner (gslot = -1); ids outside [0, E) silence their row as in
// moe_dispatch_scan (moe.cu:385-398 of the reference).
// Release a step's peer stores to every rank: ONE system-scope fence, then the arrival words as relaxed
// stores that go out back to back. (A release store per word would wait, word after word, for the
// stores before it to be acknowledged over NVLink: measured about 2.5 us per peer, 35 us per layer on
// eight ranks.) The caller has observed every storing thread's stores (barrier / acquire-release count).
__device__ __forceinline__ void set_arrival_words(unsigned* const* flags, int world, unsigned v) {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  for (int p = 0; p < world; ++p)
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flags[p]), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned atom_add_acq_rel(unsigned* p, unsigned v) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}

__device__ __forceinline__ void reset_tile_counters(const LayerDev& L, int tid, int nthr) {
  const int tiles = L.n_max * L.K + L.n_max;
  for (int i = tid; i < tiles; i += nthr) {
    L.tile_cnt[i] = 0u;
    L.ready[i] = 0u;
  }
  for (int i = tid; i < tiles * L.nbf; i += nthr) L.blk_cnt[i] = 0u;
}

// Rows [t0, t0 + nt) of caller-provided packed Q8_K rows, once more in 288-byte blocks.
__device__ __forceinline__ void pad_xq_rows(const LayerDev& L, int t0, int nt, int tid, int nthr) {
  const int words = kX8 / 4;
  for (int i = tid; i < nt * L.nbh * words; i += nthr) {
    const int tb = i / words, w = i - tb * words;
    const int t = tb / L.nbh, blk = tb - t * L.nbh;
    const uint32_t v = reinterpret_cast<const uint32_t*>(L.xq_in + static_cast<size_t>(t0 + t) * L.xq_stride + blk * kX8)[w];
    uint32_t* o = reinterpret_cast<uint32_t*>(L.xq16 + static_cast<size_t>(t0 + t) * L.xq16_stride + blk * 288);
    o[w == 0 ? 0 : w + 3] = v;
  }
}

__device__ void build_plan(const LayerDev& L, unsigned char* smem) {
  unsigned long long* mask = reinterpret_cast<unsigned long long*>(smem);       // [E]
  int* scan_rows = reinterpret_cast<int*>(smem + static_cast<size_t>(L.E) * 8);   // [65] warp totals, prefixes, total
  int* scan_tiles = scan_rows + 128;                                              // [65]
  int* scan_heavy = scan_rows + 256;                                              // [65]
  int* off_sh = scan_rows + 384;                                                  // [E] copy of L.off for the last pass
  __shared__ int bad_sh;
  const int tid = threadIdx.x;
  const int total = L.n * L.K;
  const int TT = L.tok_tile;
  if (tid == 0) bad_sh = 0;
  for (int e = tid; e < L.E; e += blockDim.x) mask[e] = 0ull;
  __syncthreads();
  int my_e = 0;                               // this thread's first route, kept for the last pass
  for (int i = tid; i < total; i += blockDim.x) {
    const int r = i / L.K, kk = i - r * L.K;
    const int e = __ldcg(L.idx + static_cast<size_t>(r) * L.rstride + kk);
    if (i == tid) my_e = e;
    if (e < 0 || e >= L.E) {
      for (int q = 0; q <= L.K; ++q) L.w[static_cast<size_t>(r) * L.rstride + q] = 0.f;
      atomicAdd(&bad_sh, 1);
    } else if (e >= L.e_lo && e < L.e_hi) {
      atomicOr(&mask[e], 1ull << r);
    }
  }
  __syncthreads();
  // exclusive prefixes of rows and tiles over experts: each thread owns a run of experts
  const int per = (L.E + blockDim.x - 1) / blockDim.x;
  const int e0 = tid * per, e1 = min(L.E, e0 + per);
  // Tile order: the shared expert's tiles, then the routed tiles of more than half a tile's rows
  // ("heavy"), then the rest, each class in expert order. The expert kernels hand work out in tile
  // order; tiles of many rows take longest, in the dot products and in the requantisation of h that
  // must finish before their down projection can start, so they go first and the light ones fill the end.
  auto is_heavy = [&](int rows_in_tile) { return 2 * rows_in_tile > TT; };
  int rows = 0, tiles = 0, heavy = 0;
  for (int e = e0; e < e1; ++e) {
    const int c = __popcll(mask[e]);
    rows += c;
    tiles += (c + TT - 1) / TT;
    heavy += c / TT + (is_heavy(c % TT) ? 1 : 0);
  }
  // exclusive scan over the threads: inside the warps with shuffles, across the warps by warp 0
  {
    const int lane = tid & 31, wp = tid >> 5, nw = (blockDim.x + 31) >> 5;
    int ir = rows, it = tiles, ih = heavy;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int ur = __shfl_up_sync(0xFFFFFFFFu, ir, off), ut = __shfl_up_sync(0xFFFFFFFFu, it, off);
      const int uh = __shfl_up_sync(0xFFFFFFFFu, ih, off);
      if (lane >= off) { ir += ur; it += ut; ih += uh; }
    }
    if (lane == 31) { scan_rows[wp] = ir; scan_tiles[wp] = it; scan_heavy[wp] = ih; }
    __syncthreads();
    if (wp == 0) {
      int wr = lane < nw ? scan_rows[lane] : 0, wt = lane < nw ? scan_tiles[lane] : 0;
      int wh = lane < nw ? scan_heavy[lane] : 0;
      const int own_r = wr, own_t = wt, own_h = wh;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int ur = __shfl_up_sync(0xFFFFFFFFu, wr, off), ut = __shfl_up_sync(0xFFFFFFFFu, wt, off);
        const int uh = __shfl_up_sync(0xFFFFFFFFu, wh, off);
        if (lane >= off) { wr += ur; wt += ut; wh += uh; }
      }
      scan_rows[32 + lane] = wr - own_r;          // exclusive prefix of the warps
      scan_tiles[32 + lane] = wt - own_t;
      scan_heavy[32 + lane] = wh - own_h;
      if (lane == 31) { scan_rows[64] = wr; scan_tiles[64] = wt; scan_heavy[64] = wh; }
    }
    __syncthreads();
    rows = scan_rows[32 + wp] + ir - rows;        // this thread's exclusive prefixes
    tiles = scan_tiles[32 + wp] + it - tiles;
    heavy = scan_heavy[32 + wp] + ih - heavy;
  }
  const int sh_tiles = (L.sh[0] != nullptr && L.sh_hi > L.sh_lo) ? (L.sh_hi - L.sh_lo + TT - 1) / TT : 0;
  const int heavy_total = scan_heavy[64];
  if (tid == 0) {
    const int ar = scan_rows[64], at = scan_tiles[64];
    // shared expert: tiles over the rows [sh_lo, sh_hi), ahead of the routed ones
    for (int i = 0; i < sh_tiles; ++i) {
      const int t0 = i * TT;
      L.rec[i] = make_int4(L.E, min(TT, L.sh_hi - L.sh_lo - t0),
                           L.n_max * L.K + L.sh_lo + t0, L.sh_lo + t0);
    }
    L.off[L.E] = ar;
    L.meta[0] = ar;
    L.meta[1] = at + sh_tiles;
    L.meta[2] = bad_sh;
    L.meta[3] = sh_tiles;                 // first routed tile
    if (L.mail_n != nullptr) *L.mail_n = 0;
    L.cnt[9] = 0u;                        // grid barrier of the expert kernel
    L.cnt[10] = static_cast<unsigned>(L.grid);   // row-streaming kernel: next group to hand out
  }
  reset_tile_counters(L, tid, blockDim.x);
  __syncthreads();
  {
    int ar = rows;
    int at_heavy = sh_tiles + heavy, at_light = sh_tiles + heavy_total + (tiles - heavy);
    for (int e = e0; e < e1; ++e) {
      const int c = __popcll(mask[e]);
      L.off[e] = ar;
      off_sh[e] = ar;
      for (int t0 = 0; t0 < c; t0 += TT) {
        const int ct = min(TT, c - t0);
        const int at = is_heavy(ct) ? at_heavy++ : at_light++;
        L.rec[at] = make_int4(e, ct, ar + t0, ar + t0);
      }
      ar += c;
    }
  }
  __syncthreads();
  for (int i = tid; i < total; i += blockDim.x) {
    const int r = i / L.K, kk = i - r * L.K;
    const int e = i == tid ? my_e : __ldcg(L.idx + static_cast<size_t>(r) * L.rstride + kk);
    int pos = -1;
    if (e >= L.e_lo && e < L.e_hi && e >= 0 && e < L.E) {
      pos = off_sh[e] + __popcll(mask[e] & ((1ull << r) - 1ull));
      L.grows[pos] = r;
    }
    L.gslot[i] = pos;
  }
}

inline size_t plan_smem(int E, int, int) { return static_cast<size_t>(E) * 12 + 3 * 128 * 4; }

// ---- launch 1: route ------------------------------------------------------------------
// grid (ceil(E / 16), ceil(n / 8)), 256 threads: a CTA computes the logits of sixteen
// experts (two per warp) for a tile of up to eight token rows. The tile's activations are
// staged in shared memory as fp32, k-major (see router_rows2_dot_kmajor), so that a
// lane's values of one k for four rows are one vector load that serves both expert rows.
// Dynamic smem: H * (8 + 16) floats (activations, router rows; the selection and the plan reuse it).
template <int NT>
__device__ __forceinline__ void route_tile_logits(const LayerDev& L, float* xs, const float* ws, int tok0, int nt,
                                                   int row0, int warp, int lane) {
  // stage: lane = one k of a 32-wide chunk, all rows of the tile (rows beyond nt read as
  // zero); four chunks per pass, so that all loads of a pass are in flight together
  for (int c0 = warp; c0 < L.H / 32; c0 += 4 * kRouteWarps) {
    uint16_t raw[4][NT];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = (c0 + u * kRouteWarps) * 32 + lane;
#pragma unroll
      for (int t = 0; t < NT; ++t)
        raw[u][t] = (t < nt && k < L.H) ? L.xn[static_cast<size_t>(tok0 + t) * L.H + k] : static_cast<uint16_t>(0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = (c0 + u * kRouteWarps) * 32 + lane;
      if (k >= L.H) continue;
      if (NT >= 4) {
#pragma unroll
        for (int p = 0; p < NT / 4; ++p)
          *reinterpret_cast<float4*>(xs + static_cast<size_t>(p) * 4 * L.H + static_cast<size_t>(k) * 4) =
              make_float4(h2f(raw[u][(4 * p) % NT]), h2f(raw[u][(4 * p + 1) % NT]), h2f(raw[u][(4 * p + 2) % NT]),
                          h2f(raw[u][(4 * p + 3) % NT]));
      } else if (NT == 2) {
        *reinterpret_cast<float2*>(xs + static_cast<size_t>(k) * 2) = make_float2(h2f(raw[u][0]), h2f(raw[u][1 % NT]));
      } else {
        xs[k] = h2f(raw[u][0]);
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");     // this warp's two router rows have landed
  __syncthreads();
  float out[2][NT];
  router_rows2_dot_kmajor<NT>(ws + static_cast<size_t>(2 * warp) * L.H, ws + static_cast<size_t>(2 * warp + 1) * L.H, xs,
                              L.H, lane, out);
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (row0 + r < L.E) {
        const float b = L.bias != nullptr ? L.bias[row0 + r] : 0.f;
#pragma unroll
        for (int t = 0; t < NT; ++t)
          if (t < nt) L.logits[static_cast<size_t>(tok0 + t) * L.E + row0 + r] = out[r][t] + b;
      }
    }
  }
}

__global__ void __launch_bounds__(kRouteWarps * 32) route_kernel(const LayerDev L) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int last_sh;
  float* xs = reinterpret_cast<float*>(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok0 = blockIdx.y * kRouteTok;
  const int nt = min(kRouteTok, L.n - tok0);
  const int row0 = blockIdx.x * kRouteRows + 2 * warp;

  // this warp's two router rows do not depend on the previous layer: they are on their
  // way into shared memory (asynchronous copies) before the wait for that layer ends
  float* ws = xs + static_cast<size_t>(kRouteTok) * L.H;              // [16 rows][H]
  {
    const float* w0 = L.router_w + static_cast<size_t>(min(row0, L.E - 1)) * L.H;
    const float* w1 = L.router_w + static_cast<size_t>(min(row0 + 1, L.E - 1)) * L.H;
    float* d0 = ws + static_cast<size_t>(2 * warp) * L.H;
    float* d1 = d0 + L.H;
    if ((reinterpret_cast<uintptr_t>(L.router_w) & 15u) == 0) {
      for (int c = lane * 4; c < L.H; c += 128) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(d0 + c)), "l"(w0 + c) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(d1 + c)), "l"(w1 + c) : "memory");
      }
    } else {
      for (int c = lane; c < L.H; c += 32) {
        d0[c] = __ldg(w0 + c);
        d1[c] = __ldg(w1 + c);
      }
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  if (L.plan_in_kernel && !L.skip_plan && blockIdx.x == 0 && blockIdx.y == 0) {
    // the expert kernel builds its plan itself: all it needs from here are fresh counters (the
    // previous kernel on this workspace has finished)
    reset_tile_counters(L, tid, blockDim.x);
    if (tid == 0) {
      L.cnt[9] = 0u;
      L.cnt[10] = static_cast<unsigned>(L.grid);
      if (L.mail_n != nullptr) *L.mail_n = 0;
    }
  }
  if (L.rearm_cnt != nullptr && blockIdx.x == 0 && blockIdx.y == 0) {
    // the owner call that follows this one on the stream plans inside its expert kernel: its
    // workspace is idle now (every earlier kernel of the stream has finished) and gets fresh counters
    for (int i = tid; i < L.rearm_tiles; i += blockDim.x) {
      L.rearm_tile_cnt[i] = 0u;
      L.rearm_ready[i] = 0u;
    }
    for (int i = tid; i < L.rearm_tiles * L.nbf; i += blockDim.x) L.rearm_blk_cnt[i] = 0u;
    if (tid == 0) {
      L.rearm_cnt[9] = 0u;
      L.rearm_cnt[10] = static_cast<unsigned>(L.grid);
      if (L.rearm_mail_n != nullptr) *L.rearm_mail_n = 0;
    }
  }

  // Q8_K rows of the tile (packed, and padded for the row-streaming kernel): block
  // b of the tile goes to warp b / gridDim.x of CTA b % gridDim.x
  if (L.xq_in != nullptr) {
    if (blockIdx.x == 0 && L.tok_tile != kTokTile && !L.xq_padded) pad_xq_rows(L, tok0, nt, tid, blockDim.x);
  } else {
    const int b = warp * gridDim.x + blockIdx.x;
    if (b < nt * L.nbh) {
      const int t = b / L.nbh, blk = b - t * L.nbh;
      quantize_block_f16(L.xn + static_cast<size_t>(tok0 + t) * L.H + blk * kQK,
                         L.xq + static_cast<size_t>(tok0 + t) * L.xq_stride + blk * kX8, lane,
                         (L.tok_tile == kTokTile && !L.xq_padded)
                             ? nullptr
                             : L.xq16 + static_cast<size_t>(tok0 + t) * L.xq16_stride + blk * 288);
    }
    // more blocks than warps in the tile's CTAs (small expert counts): the rest in a loop
    for (int b2 = b + kRouteWarps * gridDim.x; b2 < nt * L.nbh; b2 += kRouteWarps * gridDim.x) {
      const int t = b2 / L.nbh, blk = b2 - t * L.nbh;
      quantize_block_f16(L.xn + static_cast<size_t>(tok0 + t) * L.H + blk * kQK,
                         L.xq + static_cast<size_t>(tok0 + t) * L.xq_stride + blk * kX8, lane,
                         (L.tok_tile == kTokTile && !L.xq_padded)
                             ? nullptr
                             : L.xq16 + static_cast<size_t>(tok0 + t) * L.xq16_stride + blk * 288);
    }
  }
  if (nt > 4) route_tile_logits<8>(L, xs, ws, tok0, nt, row0, warp, lane);
  else if (nt > 2) route_tile_logits<4>(L, xs, ws, tok0, nt, row0, warp, lane);
  else if (nt > 1) route_tile_logits<2>(L, xs, ws, tok0, nt, row0, warp, lane);
  else route_tile_logits<1>(L, xs, ws, tok0, nt, row0, warp, lane);
  // last CTA of this token tile selects (the counter's release covers the logits of all
  // warps, which the barrier ordered before it; its acquire covers the reads that follow)
  __syncthreads();
  if (tid == 0) last_sh = atom_add_acq_rel(&L.cnt[blockIdx.y], 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (!last_sh) return;
  if (tid == 0) L.cnt[blockIdx.y] = 0u;       // every CTA of the tile has counted in: ready for the next launch
  float* prob = reinterpret_cast<float*>(smem) + static_cast<size_t>(warp % kRouteTok) * L.E;
  for (int t = warp; t < nt; t += kRouteWarps) {
    for (int i = lane; i < L.E; i += 32) prob[i] = __ldcg(L.logits + static_cast<size_t>(tok0 + t) * L.E + i);
    __syncwarp();
    router_select_warp(prob, L.E, L.K, L.idx + static_cast<size_t>(tok0 + t) * L.rstride,
                       L.w + static_cast<size_t>(tok0 + t) * L.rstride, L.shared_w, true, lane);
    __syncwarp();
  }
  if (L.skip_plan) {
    if (L.ep_dst == nullptr) return;
    // Home side of an expert-parallel layer: this tile's records (quantised rows written by every
    // CTA of the tile, ids and weights written above) go straight into every owner's receive slot
    // with 16-byte peer stores; the last tile to finish sets the owners' arrival words.
    __syncthreads();
    {
      // (a thread's pieces are fetched once, four at a time, and then stored to every peer: one round
      //  trip to L2 per pass instead of one per piece and peer - 28 us per layer on eight ranks otherwise)
      const size_t tile_off = static_cast<size_t>(tok0) * L.ep_rec;
      const int n16 = nt * L.ep_rec / 16;
      const uint4* src = reinterpret_cast<const uint4*>(L.ep_src + tile_off);
      for (int base = 0; base < n16; base += 4 * blockDim.x) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = base + j * blockDim.x + tid;
          v[j] = i < n16 ? __ldcg(src + i) : make_uint4(0u, 0u, 0u, 0u);
        }
        for (int p = 0; p < L.ep_world; ++p) {
          uint4* dst = reinterpret_cast<uint4*>(static_cast<unsigned char*>(L.ep_dst[p]) + tile_off);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = base + j * blockDim.x + tid;
            if (i < n16) dst[i] = v[j];
          }
        }
      }
    }
    // Ordering: the CTA barrier makes every thread's peer stores observed by thread 0; its
    // acquire-release count chains the tiles' CTAs; the last CTA's one system-scope fence before the
    // arrival words is cumulative over all of that. One fence per exchange, not one per thread or per
    // word: each waits for the outstanding NVLink stores to be acknowledged (about 5 us measured).
    __syncthreads();
    if (tid == 0) {
      if (atom_add_acq_rel(&L.cnt[8], 1u) == gridDim.y - 1) {     // every tile's records are on their way
        L.cnt[8] = 0u;
        const unsigned v = *L.ep_step * L.ep_mul + L.ep_add;
        set_arrival_words(L.ep_flags, L.ep_world, v);
      }
    }
    return;
  }
  if (L.plan_in_kernel) return;
  // last token tile plans
  __syncthreads();
  if (tid == 0) last_sh = atom_add_acq_rel(&L.cnt[8], 1u) == gridDim.y - 1 ? 1 : 0;
  __syncthreads();
  if (!last_sh) return;
  if (tid == 0) L.cnt[8] = 0u;
  build_plan(L, smem);
}

// Bounded wait until n arrival words (written by peers over NVLink) reach `want`: at most
// `limit` polls, 64 ns apart, per word (sgr_ep_set_wait_limit).
__device__ __forceinline__ bool wait_arrivals(const unsigned* flags, int n, unsigned want, int tid, unsigned limit) {
  bool ok = true;
  if (tid < n) {
    unsigned it = 0, v;
    do {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + tid) : "memory");
    } while (static_cast<int>(v - want) < 0 && ++it < limit && (__nanosleep(64), true));
    ok = static_cast<int>(v - want) >= 0;
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Routing supplied by the caller (expert-parallel owner side): plan only.
__global__ void __launch_bounds__(256) plan_kernel(const LayerDev L) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_launch_dependents();
  if (L.wait_flags != nullptr &&
      !wait_arrivals(L.wait_flags, L.wait_count, *L.wait_step * L.wait_mul + L.wait_add, threadIdx.x, L.wait_limit) &&
      threadIdx.x == 0)
    atomicExch(L.status, 8);                  // a peer's records did not arrive: the plan below reads the rows
                                              // of an earlier step (valid memory, wrong step)
  if (L.tok_tile != kTokTile && !L.xq_padded) pad_xq_rows(L, 0, L.n, threadIdx.x, blockDim.x);
  build_plan(L, smem);
}

// ---- launch 2: the persistent expert kernel ----------------------------------------------
struct ItemDesc {
  int kind;     // 0 gate/up, 1 down
  int mode;     // 0 weights arrive by TMA, 1 expert absent, 2 unaligned: consumers copy
  int tile, chunk;
  int e, ntok, hrow0, p0;
  int row0, nrows;
  int pad[2];
};

struct StreamGeom {
  int rows_gu, rows_dn;          // rows of one matrix per item
  int ws_gu, ws_dn;              // shared-memory row strides
  int chunks_gu, chunks_dn;
  int stage_bytes;
  int x_bytes;                   // one team's activation tile
};
__host__ __device__ inline StreamGeom stream_geom(int H, int FF) {
  StreamGeom g;
  const int nbh = H / kQK, nbf = FF / kQK;
  g.rows_gu = tile_rows(nbh);
  g.rows_dn = tile_rows(nbf);
  // Padded row strides where eight rows would otherwise share a bank group: those
  // tiles arrive as one bulk copy per row. A warp issues its bulk copies one after
  // another (about 60 cycles each), so the rows are spread over the producer warps.
  g.ws_gu = tile_wstride(nbh);
  g.ws_dn = tile_wstride(nbf);
  g.chunks_gu = (FF + g.rows_gu - 1) / g.rows_gu;
  g.chunks_dn = (H + g.rows_dn - 1) / g.rows_dn;
  const int a = 2 * g.rows_gu * g.ws_gu, b = g.rows_dn * g.ws_dn;
  g.stage_bytes = ((a > b ? a : b) + 127) & ~127;
  const int xa = static_cast<int>(xtile_bytes(kTokTile, nbh)), xb = static_cast<int>(xtile_bytes(kTokTile, nbf));
  g.x_bytes = ((xa > xb ? xa : xb) + 127) & ~127;
  return g;
}
constexpr int kStreamHdr = 512;                                          // barriers, flags, item descriptors
constexpr int kTeamRed = 2 * kTeamWarps * 2 * 128 * 4;                   // two buffers of [warp][matrix][128] floats
inline size_t stream_smem(int H, int FF) {
  const StreamGeom g = stream_geom(H, FF);
  return kStreamHdr + static_cast<size_t>(kStages) * g.stage_bytes + kTeams * (g.x_bytes + kTeamRed);
}


__device__ __forceinline__ void team_sync(int team) {
  asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "n"(kTeamThreads) : "memory");
}
__device__ __forceinline__ void consumers_sync() {
  asm volatile("bar.sync 3, %0;" ::"n"(kConsumers) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Q8_K-quantise fp32 rows straight into a staged tile (one warp per 256 values;
// arithmetic of src/kernels/cpu/q4_avx2.cpp:77-94 in the reference).
__device__ __forceinline__ void stage_quantized_f32(const XTile& xt, int nt, const float* src,
                                                    size_t row_stride, int warp, int nwarps) {
  const int lane = threadIdx.x & 31;
  for (int job = warp; job < nt * xt.nb; job += nwarps) {
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
    int8_t* qs = xt.qs + static_cast<size_t>(t) * xt.tok_stride + blk * kXqStride + lane * 8;
    reinterpret_cast<uint32_t*>(qs)[0] = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) |
                                         (static_cast<uint32_t>(q[3] & 0xFF) << 24);
    reinterpret_cast<uint32_t*>(qs)[1] = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) |
                                         (static_cast<uint32_t>(q[7] & 0xFF) << 24);
    const int sum_next = __shfl_down_sync(0xFFFFFFFFu, sum, 4);      // the next sub-block's sum
    if ((lane & 7) == 0)
      xt.put_sum_pair(t, blk, lane >> 3,
                      (static_cast<uint32_t>(sum) & 0xFFFFu) | (static_cast<uint32_t>(sum_next) << 16));
    if (lane == 0) xt.d[t * xt.nb + blk] = d;
  }
}

// One team (eight warps) on one item. The (16-row group, super-block) units go
// round the team's warps; every warp leaves its partial sums in shared memory,
// the stage is released, and after one team barrier all 256 threads add the
// partials of their output element in warp order (reproducible) and emit it.
//   emit(row, token, v[NMAT])
template <int NMAT, typename Emit>
__device__ __forceinline__ void item_compute(const LayerDev& L, const unsigned char* w, int wstride,
                                             int mat_stride, const XTile& xt, float* red, int nrows,
                                             int nb, int ntok, int team, uint64_t* release, Emit emit) {
  const int tw = (threadIdx.x >> 5) & (kTeamWarps - 1), lane = threadIdx.x & 31;
  const int ttid = threadIdx.x & (kTeamThreads - 1);
  const int groups = (nrows + 15) / 16;
  const int units = groups * nb;
  int grp, blk0, bstep, contrib;
  bool active;
  if (units <= kTeamWarps) {              // one unit per warp
    active = tw < units;
    grp = tw / nb;
    blk0 = tw - grp * nb;
    bstep = nb;
    contrib = nb;
  } else {                                // a single group (host-checked): blocks go round the warps
    active = tw < min(kTeamWarps, nb);
    grp = 0;
    blk0 = tw;
    bstep = kTeamWarps;
    contrib = min(kTeamWarps, nb);
  }
  if (active) {
    float acc[NMAT][1][4];
    warp_mma_rows<NMAT, 1>(w, wstride, mat_stride, xt, grp * 16, nrows, nb, blk0, bstep, acc);
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) red[(tw * 2 + m) * 128 + j * 32 + lane] = acc[m][0][j];
  }
  __syncwarp();
  if (lane == 0) mbar_arrive(release);     // this warp no longer reads the weight stage
  team_sync(team);
  // element q of a group: fragment slot j = q / 32 of lane q % 32
  const int per_group = units <= kTeamWarps ? nb : 0;       // warps of group g start at g * per_group
  for (int o = ttid; o < groups * 128; o += kTeamThreads) {
    const int g = o >> 7, q = o & 127;
    const int j = q >> 5, ln = q & 31;
    const int r = g * 16 + (ln >> 2) + (j >> 1) * 8, t = 2 * (ln & 3) + (j & 1);
    if (r < nrows && t < ntok) {
      float v[NMAT];
      const int w0 = g * per_group;
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        float a = red[(w0 * 2 + m) * 128 + q];
        for (int p = 1; p < contrib; ++p) a += red[((w0 + p) * 2 + m) * 128 + q];
        v[m] = a;
      }
      emit(r, t, v);
    }
  }
}

// The same item for tiles of one or two token rows: dp4a, one thread per
// (row, matrix, super-block) task, shuffle reduction over the lanes of a row -
// no shared-memory partials and no team barrier. Needs NMAT * lanes-per-row <= 32.
template <int NMAT, typename Emit>
__device__ __forceinline__ void item_compute_dp4a(const unsigned char* w, int wstride, int mat_stride,
                                                  const XTile& xt, int nrows, int nb, int ntok,
                                                  uint64_t* release, Emit emit) {
  const int ttid = threadIdx.x & (kTeamThreads - 1), lane = threadIdx.x & 31;
  const int lpr = next_pow2_cap32(nb);
  const int tasks = nrows * NMAT * lpr;
  for (int base = 0; base < tasks; base += kTeamThreads) {     // uniform trip count
    const int t = base + ttid;
    const int lr = t & (lpr - 1);
    const int rm = t / lpr;
    const int m = NMAT == 2 ? (rm & 1) : 0;
    const int row = NMAT == 2 ? (rm >> 1) : rm;
    float acc[1][2] = {{0.f, 0.f}};
    if (t < tasks) {
      for (int blk = lr; blk < nb; blk += lpr) {
        const uint4* wb[1] = {reinterpret_cast<const uint4*>(w + m * mat_stride + row * wstride + blk * kW4)};
        block_dot<1, 2>(wb, xt, blk, ntok, acc);
      }
    }
    float v0 = reduce_lanes(acc[0][0], lpr), v1 = reduce_lanes(acc[0][1], lpr);
    float u0 = 0.f, u1 = 0.f;
    if (NMAT == 2) {                       // the up row's lanes follow the gate row's
      u0 = __shfl_down_sync(0xFFFFFFFFu, v0, lpr);
      u1 = __shfl_down_sync(0xFFFFFFFFu, v1, lpr);
    }
    if (t < tasks && lr == 0 && m == 0) {
      float a[NMAT], b[NMAT];
      a[0] = v0; b[0] = v1;
      if (NMAT == 2) { a[NMAT - 1] = u0; b[NMAT - 1] = u1; }
      emit(row, 0, a);
      if (ntok > 1) emit(row, 1, b);
    }
  }
  __syncwarp();
  if (lane == 0) mbar_arrive(release);
}

// residual + sum_k w_k * y_k + shared expert for output rows [row0, row0+nrows), tokens [t_lo, t_hi)
// The same blend as combine_rows over the whole layer, two columns per thread and every thread of the
// grid at work: the routes of a token (slot, weight) are fetched eight at a time and their y rows
// requested together, so an output costs two round trips to L2 instead of two per expert. Terms are
// added in combine_rows' order (residual, experts in slot order, shared expert), so both give the same bits.
__device__ __forceinline__ void combine_flat(const LayerDev& L, int gtid, int gthreads, const int* gslot, bool gslot_shared) {
  const bool has_shared = L.sh[0] != nullptr;
  const int half = L.H >> 1;
  for (int idx = gtid; idx < L.n * half; idx += gthreads) {
    const int tk = idx / half, r = (idx - tk * half) * 2;
    const size_t o = static_cast<size_t>(tk) * L.H + r;
    float a0 = 0.f, a1 = 0.f;
    if (L.add_residual && L.x_f16 != nullptr) {
      const uint32_t xv = *reinterpret_cast<const uint32_t*>(L.x_f16 + o);
      a0 = h2f(static_cast<uint16_t>(xv & 0xFFFFu));
      a1 = h2f(static_cast<uint16_t>(xv >> 16));
    }
    const float* wr = L.w + static_cast<size_t>(tk) * L.rstride;
    for (int k0 = 0; k0 < L.K; k0 += 8) {
      int gs[8];
      float w[8];
      float2 y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool in = k0 + j < L.K;
        gs[j] = in ? (gslot_shared ? gslot[tk * L.K + k0 + j] : __ldcg(gslot + tk * L.K + k0 + j)) : -1;
        w[j] = in ? __ldcg(wr + k0 + j) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        y[j] = gs[j] >= 0 ? __ldcg(reinterpret_cast<const float2*>(L.ybuf + static_cast<size_t>(gs[j]) * L.H + r))
                          : make_float2(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (gs[j] >= 0) {
          a0 += w[j] * y[j].x;
          a1 += w[j] * y[j].y;
        }
      }
    }
    if (has_shared && tk >= L.sh_lo && tk < L.sh_hi) {
      const float ws = __ldcg(wr + L.K);
      const float2 ys = __ldcg(reinterpret_cast<const float2*>(L.ybuf + static_cast<size_t>(L.n_max * L.K + tk) * L.H + r));
      a0 += ws * ys.x;
      a1 += ws * ys.y;
    }
    if (L.ep_out != nullptr)
      *reinterpret_cast<float2*>(L.ep_out[tk / L.ep_home] + static_cast<size_t>(tk % L.ep_home) * L.H + r) = make_float2(a0, a1);
    else if (L.out_f32 != nullptr)
      *reinterpret_cast<float2*>(L.out_f32 + o) = make_float2(a0, a1);
    if (L.x_f16 != nullptr && L.add_residual)
      *reinterpret_cast<uint32_t*>(L.x_f16 + o) = static_cast<uint32_t>(f2h(a0)) | (static_cast<uint32_t>(f2h(a1)) << 16);
  }
}

__device__ __forceinline__ void combine_rows(const LayerDev& L, int row0, int nrows, int t_lo, int t_hi,
                                             int tid, int nthr) {
  const bool has_shared = L.sh[0] != nullptr;
  for (int i = tid; i < nrows * (t_hi - t_lo); i += nthr) {
    const int tk = t_lo + i / nrows, r = row0 + i % nrows;
    const size_t o = static_cast<size_t>(tk) * L.H + r;
    float acc = (L.add_residual && L.x_f16 != nullptr) ? h2f(L.x_f16[o]) : 0.f;
    const float* wr = L.w + static_cast<size_t>(tk) * L.rstride;
    for (int kk = 0; kk < L.K; ++kk) {
      const int gs = __ldcg(L.gslot + tk * L.K + kk);
      if (gs >= 0) acc += __ldcg(wr + kk) * __ldcg(L.ybuf + static_cast<size_t>(gs) * L.H + r);
    }
    if (has_shared && tk >= L.sh_lo && tk < L.sh_hi)
      acc += __ldcg(wr + L.K) * __ldcg(L.ybuf + static_cast<size_t>(L.n_max * L.K + tk) * L.H + r);
    if (L.ep_out != nullptr) L.ep_out[tk / L.ep_home][static_cast<size_t>(tk % L.ep_home) * L.H + r] = acc;
    else if (L.out_f32 != nullptr) L.out_f32[o] = acc;
    if (L.x_f16 != nullptr && L.add_residual) L.x_f16[o] = f2h(acc);
  }
}

#include "expert_rows.cuh"
#include "token_layer.cuh"

__global__ void __launch_bounds__(kStreamThreads, 1) expert_stream_kernel(const LayerDev L) {
  extern __shared__ __align__(16) unsigned char smem[];
  const StreamGeom G = stream_geom(L.H, L.FF);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kStages;
  int* flag = reinterpret_cast<int*>(smem + 128);                 // broadcast slots
  ItemDesc* desc = reinterpret_cast<ItemDesc*>(smem + 256);
  unsigned char* stages = smem + kStreamHdr;
  unsigned char* team_base = stages + static_cast<size_t>(kStages) * G.stage_bytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kTeamWarps);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  pdl_wait();                       // plan, routing and quantised rows come from the route kernel
  pdl_launch_dependents();

  const int n_tiles = L.meta[1];
  const long long n_gu = static_cast<long long>(n_tiles) * G.chunks_gu;
  const long long n_dn = static_cast<long long>(n_tiles) * G.chunks_dn;
  const int gu_lo = static_cast<int>(n_gu * blockIdx.x / gridDim.x);
  const int gu_cnt = static_cast<int>(n_gu * (blockIdx.x + 1) / gridDim.x) - gu_lo;
  const int dn_lo = static_cast<int>(n_dn * blockIdx.x / gridDim.x);
  const int dn_cnt = static_cast<int>(n_dn * (blockIdx.x + 1) / gridDim.x) - dn_lo;
  const int n_items = gu_cnt + dn_cnt;
  const size_t rb_h = static_cast<size_t>(L.nbh) * kW4, rb_f = static_cast<size_t>(L.nbf) * kW4;

  if (warp >= kConsumers / 32) {
    // ---------------- producer warps ----------------
    // All of them walk the same item list; the first one also publishes the item
    // descriptor and arms the stage's barrier, every one issues its share of the rows.
    const int pw = warp - kConsumers / 32;
    int cached_tile = -1;
    int4 rc = make_int4(0, 0, 0, 0);
    const unsigned char *w0 = nullptr, *w1 = nullptr, *w2 = nullptr;
    for (int i = 0; i < n_items; ++i) {
      const int s = i % kStages;
      const unsigned ph = (i / kStages) & 1;
      const int kind = i < gu_cnt ? 0 : 1;
      const int id = kind == 0 ? gu_lo + i : dn_lo + (i - gu_cnt);
      const int chunks = kind == 0 ? G.chunks_gu : G.chunks_dn;
      const int tile = id / chunks, chunk = id - tile * chunks;
      if (tile != cached_tile) {                  // consecutive items share their tile
        rc = __ldcg(L.rec + tile);
        const bool shared = rc.x == L.E;
        w0 = shared ? L.sh[0] : L.tab[rc.x];
        w1 = shared ? L.sh[1] : L.tab[L.tab_stride + rc.x];
        w2 = shared ? L.sh[2] : L.tab[2 * L.tab_stride + rc.x];
        cached_tile = tile;
      }
      if (!mbar_wait(&empty[s], ph ^ 1u)) {
        if (lane == 0) atomicExch(L.status, 2);
        return;
      }
      const bool absent = w0 == nullptr || w1 == nullptr || w2 == nullptr;
      const bool aligned = ((reinterpret_cast<uintptr_t>(w0) | reinterpret_cast<uintptr_t>(w1) |
                             reinterpret_cast<uintptr_t>(w2)) & 15u) == 0;
      const int rows_per = kind == 0 ? G.rows_gu : G.rows_dn;
      const int row0 = chunk * rows_per;
      const int nrows = min(rows_per, (kind == 0 ? L.FF : L.H) - row0);
      const int mode = absent ? 1 : (aligned ? 0 : 2);
      if (lane == 0 && pw == 0) {
        ItemDesc d;
        d.kind = kind; d.mode = mode; d.tile = tile; d.chunk = chunk;
        d.e = rc.x; d.ntok = rc.y; d.hrow0 = rc.z; d.p0 = rc.w;
        d.row0 = row0; d.nrows = nrows; d.pad[0] = d.pad[1] = 0;
        desc[s] = d;
        const uint32_t bytes = mode != 0 ? 0u
                               : static_cast<uint32_t>(nrows) * static_cast<uint32_t>(kind == 0 ? 2 * rb_h : rb_f);
        mbar_expect_tx(&full[s], bytes);
      }
      __syncwarp();
      if (mode == 0) {
        unsigned char* st = stages + static_cast<size_t>(s) * G.stage_bytes;
        if (kind == 0) {
          const int ms = G.rows_gu * G.ws_gu;
          if (G.ws_gu == static_cast<int>(rb_h)) {
            if (pw == 0 && lane < 2) bulk_g2s(st + lane * ms, (lane == 0 ? w0 : w1) + row0 * rb_h,
                                              static_cast<uint32_t>(nrows * rb_h), &full[s]);
          } else {
            // copy j of 2*nrows goes to warp j % kProducerWarps, lane j / kProducerWarps
            for (int j = pw + kProducerWarps * lane; j < 2 * nrows; j += kProducerWarps * 32) {
              const int m = j / nrows, r = j - m * nrows;
              bulk_g2s(st + m * ms + r * G.ws_gu, (m == 0 ? w0 : w1) + (row0 + r) * rb_h,
                       static_cast<uint32_t>(rb_h), &full[s]);
            }
          }
        } else {
          if (G.ws_dn == static_cast<int>(rb_f)) {
            if (pw == 0 && lane == 0)
              bulk_g2s(st, w2 + row0 * rb_f, static_cast<uint32_t>(nrows * rb_f), &full[s]);
          } else {
            for (int r = pw + kProducerWarps * lane; r < nrows; r += kProducerWarps * 32)
              bulk_g2s(st + r * G.ws_dn, w2 + (row0 + r) * rb_f, static_cast<uint32_t>(rb_f), &full[s]);
          }
        }
      }
    }
    return;
  }

  // ---------------- consumer teams ----------------
  const int team = warp / kTeamWarps, tw = warp - team * kTeamWarps, ttid = tid - team * kTeamThreads;
  unsigned char* xbase = team_base + static_cast<size_t>(team) * (G.x_bytes + kTeamRed);
  float* red = reinterpret_cast<float*>(xbase + G.x_bytes);
  const unsigned char* xq = L.xq_in != nullptr ? L.xq_in : L.xq;
  int cur_kind = -1, cur_tile = -1, pending = 0, parity = 0;
  XTile xt = xtile_at(xbase, kTokTile, L.nbh);
  bool ok = true;
  // publish the gate/up chunks this team finished for its current tile
  auto publish = [&]() {
    if (cur_kind == 0 && pending > 0) {
      __threadfence();
      team_sync(team);
      if (ttid == 0) atomicAdd(L.tile_cnt + cur_tile, static_cast<unsigned>(pending));
    }
    pending = 0;
  };
  for (int i = team; i < n_items && ok; i += kTeams) {
    const int s = i % kStages;
    const unsigned ph = (i / kStages) & 1;
    if (!mbar_wait(&full[s], ph)) {
      if (ttid == 0) atomicExch(L.status, 3);
      ok = false;                              // the whole team sees the same expiry
      break;
    }
    const ItemDesc d = desc[s];
    unsigned char* st = stages + static_cast<size_t>(s) * G.stage_bytes;
    if (d.kind != cur_kind || d.tile != cur_tile) {
      publish();
      team_sync(team);                         // previous activation tile fully consumed
      cur_kind = d.kind;
      cur_tile = d.tile;
      if (d.kind == 0) {
        xt = xtile_at(xbase, kTokTile, L.nbh);
        const bool shared = d.e == L.E;
        xtile_stage(xt, d.ntok,
                    [&](int t) {
                      const int r = shared ? d.p0 + t : __ldcg(L.grows + d.p0 + t);
                      return xq + static_cast<size_t>(r) * L.xq_stride;
                    },
                    ttid, kTeamThreads);
      } else {
        xt = xtile_at(xbase, kTokTile, L.nbf);
        if (ttid == 0) {                       // wait for the gate/up items of this tile
          unsigned it = 0;
          while (ld_acquire(L.tile_cnt + d.tile) < static_cast<unsigned>(G.chunks_gu) && ++it < kSpinLimit)
            __nanosleep(32);
          flag[team] = it < kSpinLimit ? 1 : 0;
        }
        team_sync(team);
        if (!flag[team]) {
          if (ttid == 0) atomicExch(L.status, 4);
          ok = false;
          break;
        }
        if (d.mode != 1)
          stage_quantized_f32(xt, d.ntok, L.hbuf + static_cast<size_t>(d.hrow0) * L.FF, L.FF, tw, kTeamWarps);
      }
      team_sync(team);
    }
    if (d.mode == 2) {                         // unaligned weights: copy them here
      if (d.kind == 0) {
        const bool shared = d.e == L.E;
        const unsigned char* w0 = shared ? L.sh[0] : L.tab[d.e];
        const unsigned char* w1 = shared ? L.sh[1] : L.tab[L.tab_stride + d.e];
        for (int r = 0; r < d.nrows; ++r) {
          copy_unaligned(st + r * G.ws_gu, w0 + (d.row0 + r) * rb_h, static_cast<int>(rb_h), ttid, kTeamThreads);
          copy_unaligned(st + G.rows_gu * G.ws_gu + r * G.ws_gu, w1 + (d.row0 + r) * rb_h,
                         static_cast<int>(rb_h), ttid, kTeamThreads);
        }
      } else {
        const unsigned char* w2 = d.e == L.E ? L.sh[2] : L.tab[2 * L.tab_stride + d.e];
        for (int r = 0; r < d.nrows; ++r)
          copy_unaligned(st + r * G.ws_dn, w2 + (d.row0 + r) * rb_f, static_cast<int>(rb_f), ttid, kTeamThreads);
      }
      team_sync(team);
    }
    if (d.mode == 1) {                         // absent expert: zero rows, one mail per tile
      if (d.kind == 0) {
        if (d.chunk == 0 && ttid == 0 && L.mail != nullptr && d.e != L.E) {
          const int mi = atomicAdd(L.mail_n, 1);
          if (mi < L.E) L.mail[mi] = d.e;
        }
      } else {
        for (int j = ttid; j < d.nrows * d.ntok; j += kTeamThreads)
          L.ybuf[static_cast<size_t>(d.hrow0 + j / d.nrows) * L.H + d.row0 + j % d.nrows] = 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    } else if (d.ntok <= 2 && 2 * next_pow2_cap32(L.nbh) <= 32) {
      if (d.kind == 0)
        item_compute_dp4a<2>(st, G.ws_gu, G.rows_gu * G.ws_gu, xt, d.nrows, L.nbh, d.ntok, &empty[s],
                             [&](int r, int t, const float (&v)[2]) {
                               const float g = v[0], u = v[1];
                               L.hbuf[static_cast<size_t>(d.hrow0 + t) * L.FF + d.row0 + r] =
                                   g / (1.f + expf(-g)) * u;
                             });
      else
        item_compute_dp4a<1>(st, G.ws_dn, 0, xt, d.nrows, L.nbf, d.ntok, &empty[s],
                             [&](int r, int t, const float (&v)[1]) {
                               L.ybuf[static_cast<size_t>(d.hrow0 + t) * L.H + d.row0 + r] = v[0];
                             });
    } else if (d.kind == 0) {
      // partial sums alternate between two buffers: a warp may start the next item
      // while another thread of the team still adds up this one
      item_compute<2>(L, st, G.ws_gu, G.rows_gu * G.ws_gu, xt, red + (parity ^= 1) * (kTeamRed / 8), d.nrows,
                      L.nbh, d.ntok, team, &empty[s],
                      [&](int r, int t, const float (&v)[2]) {
                        const float g = v[0], u = v[1];
                        L.hbuf[static_cast<size_t>(d.hrow0 + t) * L.FF + d.row0 + r] = g / (1.f + expf(-g)) * u;
                      });
    } else {
      item_compute<1>(L, st, G.ws_dn, 0, xt, red + (parity ^= 1) * (kTeamRed / 8), d.nrows, L.nbf, d.ntok,
                      team, &empty[s],
                      [&](int r, int t, const float (&v)[1]) {
                        L.ybuf[static_cast<size_t>(d.hrow0 + t) * L.H + d.row0 + r] = v[0];
                      });
    }
    if (d.kind == 0) ++pending;
  }
  if (ok) publish();

  // ---- all down rows written everywhere: blend ------------------------------------------------
  __threadfence();
  consumers_sync();
  if (tid == 0) {
    atomicAdd(&L.cnt[9], 1u);
    unsigned it = 0;
    while (ld_acquire(&L.cnt[9]) < gridDim.x && ++it < kSpinLimit) __nanosleep(32);
    flag[2] = it < kSpinLimit ? 1 : 0;
  }
  consumers_sync();
  if (!flag[2]) {
    if (tid == 0) atomicExch(L.status, 5);
    return;
  }
  const int tgroups = (L.n + 15) / 16;
  for (int job = blockIdx.x; job < G.chunks_dn * tgroups; job += gridDim.x) {
    const int c = job / tgroups, tg = job - c * tgroups;
    combine_rows(L, c * G.rows_dn, min(G.rows_dn, L.H - c * G.rows_dn), tg * 16, min(L.n, tg * 16 + 16), tid,
                 kConsumers);
  }
}

// Scratch of the allocation-free entry point (sgr_moe_layer_decode_static): the
// same layout a caller-provided workspace has, held by every device that loads
// the library until the process exits.
constexpr size_t kStaticWsBytes = 2u << 20;
static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes];
constexpr int kStaticMaxDevices = 64;
unsigned char* g_static_ws_addr[kStaticMaxDevices];     // per-device address of g_static_ws

// Re-arms the counters the plan normally resets, for launches of the expert kernel
// alone on a workspace that already ran once.
__global__ void rearm_kernel(const LayerDev L) {
  pdl_wait();
  pdl_launch_dependents();
  reset_tile_counters(L, threadIdx.x, blockDim.x);
  if (threadIdx.x == 0) {
    L.cnt[9] = 0u;
    L.cnt[10] = static_cast<unsigned>(L.grid);
  }
}

// x[i] = f16( f32(x[i]) + sum_p parts[p][i] ), p ascending: the home rank's last step of
// an expert-parallel layer (partial sums of every owner rank, received row-aligned).
__global__ void ep_reduce_add_kernel(uint16_t* __restrict__ x, const float* __restrict__ parts,
                                     int n_parts, size_t part_stride, size_t count) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float acc = h2f(x[i]);
    for (int p = 0; p < n_parts; ++p) acc += parts[p * part_stride + i];
    x[i] = f2h(acc);
  }
}

// ep_reduce_add_kernel after the arrival words of all parts have reached `want` (every CTA waits).
// A CTA whose wait runs out raises status 8 and leaves its share of x as it was.
__global__ void ep_reduce_add_wait_kernel(uint16_t* __restrict__ x, const float* __restrict__ parts,
                                          int n_parts, size_t part_stride, size_t count, const unsigned* flags,
                                          const unsigned* step, int mul, int add, unsigned limit, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  if (!wait_arrivals(flags, n_parts, *step * mul + add, threadIdx.x, limit)) {
    if (threadIdx.x == 0) atomicExch(status, 8);
    return;
  }
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float acc = h2f(x[i]);
    for (int p0 = 0; p0 < n_parts; p0 += 8) {     // eight ranks' terms requested together, added in rank order
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = p0 + j < n_parts ? __ldcg(parts + (p0 + j) * part_stride + i) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (p0 + j < n_parts) acc += v[j];
    }
    x[i] = f2h(acc);
  }
}

// Copies to every peer, then (last CTA to finish) the arrival words. grid (chunks, world).
__global__ void ep_push_kernel(const unsigned char* __restrict__ src, size_t src_stride, size_t bytes,
                               void* const* __restrict__ dst, unsigned* const* __restrict__ flags, int world,
                               const unsigned* step, int mul, int add, unsigned* scratch) {
  pdl_wait();
  pdl_launch_dependents();
  const int p = blockIdx.y;
  const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(p) * src_stride);
  uint4* d = reinterpret_cast<uint4*>(dst[p]);
  const size_t n16 = bytes / 16;
  const size_t per = (n16 + gridDim.x - 1) / gridDim.x;
  const size_t lo = per * blockIdx.x, hi = lo + per < n16 ? lo + per : n16;
  for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) d[i] = s[i];
  // the CTA barrier makes the stores observed by thread 0, its acquire-release count chains the CTAs,
  // and the last CTA's system-scope fence before the arrival words is cumulative over all of it
  __syncthreads();
  if (threadIdx.x != 0) return;
  if (atom_add_acq_rel(scratch, 1u) != gridDim.x * gridDim.y - 1) return;
  *scratch = 0u;
  const unsigned v = *step * mul + add;
  set_arrival_words(flags, world, v);
}

__global__ void ep_step_kernel(unsigned* step) {
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) *step += 1u;
}


// A 2-D TMA descriptor over a Q4_K matrix seen as bytes, [rows][row_bytes], with boxes of
// one super-block column (144 bytes) x 128 rows, encoded for a placeholder address: the
// expert kernel patches the real base address in on the device. Encoded once per
// geometry (cuTensorMapEncodeTiled, reached through the runtime's driver entry point).
bool matrix_tmap(int row_bytes, int rows, const void* placeholder, uint32_t* out128) {
  struct Entry { int row_bytes, rows; unsigned char bytes[128]; };
  static std::mutex mu;
  static Entry cache[16];
  static int n_cache = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_cache; ++i)
    if (cache[i].row_bytes == row_bytes && cache[i].rows == rows) {
      std::memcpy(out128, cache[i].bytes, 128);
      return true;
    }
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  if (encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        fn == nullptr || qres != cudaDriverEntryPointSuccess)
      return false;
    encode = reinterpret_cast<EncodeFn>(fn);
  }
  CUtensorMap tm;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kW4), 128u};
  const cuuint32_t estr[2] = {1u, 1u};
  if (encode(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(placeholder), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  static_assert(sizeof(CUtensorMap) == 128, "descriptor size");
  std::memcpy(out128, &tm, 128);
  if (n_cache < 16) {
    cache[n_cache].row_bytes = row_bytes;
    cache[n_cache].rows = rows;
    std::memcpy(cache[n_cache].bytes, &tm, 128);
    ++n_cache;
  }
  return true;
}

// Polls (64 ns apart) after which a kernel that waits for a peer's arrival words gives up.
std::atomic<unsigned> g_wait_limit{1u << 22};

template <typename Kern>
int launch_pdl(Kern kern, dim3 grid, int threads, size_t smem, cudaStream_t stream,
               const LayerDev& L) {
  if (smem > 32 * 1024 &&     // (static shared memory counts towards the 48 KB default limit)
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

// Diagnostics (sager_b200_diag.h): where a region of the workspace starts, so that a test can read
// the intermediate rows a finished call left there. which: 0 fp32 h rows, 1 fp32 y rows, 2 gslot,
// 3 grows, 4 plan records, 5 meta.
SGR_API long long sgr_moe_layer_workspace_offset(int n_max, int hidden, int n_ff, int n_expert, int n_used,
                                                 int which) {
  if (sgr_moe_layer_workspace_bytes(n_max, hidden, n_ff, n_expert, n_used) == 0) return -1;
  const WsLayout l = ws_layout(n_max, hidden, n_ff, n_expert, n_used);
  switch (which) {
    case 0: return static_cast<long long>(l.hbuf);
    case 1: return static_cast<long long>(l.ybuf);
    case 2: return static_cast<long long>(l.gslot);
    case 3: return static_cast<long long>(l.grows);
    case 4: return static_cast<long long>(l.rec);
    case 5: return static_cast<long long>(l.meta);
    default: return -1;
  }
}

SGR_API int sgr_moe_layer_workspace_init(void* workspace, size_t bytes, void* stream) {
  if (!workspace || bytes == 0) return kErrArg;
  return cudaMemsetAsync(workspace, 0, bytes, as_stream(stream)) == cudaSuccess ? kOk : kErrLaunch;
}

SGR_API int sgr_moe_layer_decode_stages(const sgr_moe_layer* a, int stages, void* stream) {
  if (a == nullptr || (stages & 7) == 0) return kErrArg;   // bit 3 (8): route without the plan; bits 4, 5: kernel choice
  if (a->n <= 0) return kOk;
  if (a->hidden <= 0 || a->hidden % kQK || a->n_ff <= 0 || a->n_ff % kQK || a->n_expert <= 0 ||
      a->n_used <= 0 || a->n_used > a->n_expert || a->n_max < a->n || a->n_max > kMaxRows)
    return kErrGeometry;
  if (a->n_expert > 1024 || a->hidden > 8192 || a->n_ff > 8192) return kErrUnsupported;
  if (!a->w_tab || !a->route_idx || !a->route_w || !a->workspace || (!a->x_f16 && !a->out_f32 && !a->ep_out))
    return kErrArg;
  if (!a->routing_given && (!a->xn || !a->router_w)) return kErrArg;
  if (a->routing_given && !a->xq_in && !a->xn) return kErrArg;
  if (a->mail && !a->mail_n) return kErrArg;
  const WsLayout lay = ws_layout(a->n_max, a->hidden, a->n_ff, a->n_expert, a->n_used);
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 255u) ||
      (a->xn && (reinterpret_cast<uintptr_t>(a->xn) & 15u)) ||
      (a->xq_in && (reinterpret_cast<uintptr_t>(a->xq_in) & 3u)) ||
      (a->x_f16 && (reinterpret_cast<uintptr_t>(a->x_f16) & 3u)) ||          // the blend moves two columns at a time
      (a->out_f32 && (reinterpret_cast<uintptr_t>(a->out_f32) & 7u)))
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
  L.skip_plan = (stages & 8) ? 1 : 0;
  L.rstride = a->route_stride > 0 ? a->route_stride : a->n_used + 1;
  L.xq_stride = a->xq_stride > 0 ? a->xq_stride : (a->hidden / kQK) * kX8;
  if (L.rstride < a->n_used + 1 || L.xq_stride < (a->hidden / kQK) * kX8 || (L.xq_stride & 3)) return kErrArg;
  L.shared_w = a->shared_w;
  L.xn = a->xn;
  L.xq_in = static_cast<const unsigned char*>(a->xq_in);
  L.router_w = a->router_w;
  L.bias = a->router_bias;
  L.tab = reinterpret_cast<const unsigned char* const*>(a->w_tab);
  L.tab_stride = a->tab_stride > 0 ? a->tab_stride : a->n_expert;
  if (L.tab_stride < a->n_expert) return kErrArg;
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
  L.xq = a->xq_out != nullptr ? static_cast<unsigned char*>(a->xq_out) : ws + lay.xq;
  if (reinterpret_cast<uintptr_t>(L.xq) & 3u) return kErrAlign;
  L.logits = reinterpret_cast<float*>(ws + lay.logits);
  L.off = reinterpret_cast<int*>(ws + lay.off);
  L.rec = reinterpret_cast<int4*>(ws + lay.rec);
  L.tile_cnt = reinterpret_cast<unsigned*>(ws + lay.tile_cnt);
  L.blk_cnt = reinterpret_cast<unsigned*>(ws + lay.blk_cnt);
  L.ready = reinterpret_cast<unsigned*>(ws + lay.ready);
  L.hq = ws + lay.hq;
  L.xq16 = ws + lay.xq16;
  L.xq16_stride = L.nbh * 288;
  L.xq_padded = a->xq_padded ? 1 : 0;
  L.tmaps = ws + lay.tmaps;
  L.meta = reinterpret_cast<int*>(ws + lay.meta);
  L.gslot = reinterpret_cast<int*>(ws + lay.gslot);
  L.grows = reinterpret_cast<int*>(ws + lay.grows);
  L.cnt = reinterpret_cast<unsigned*>(ws + lay.cnt);
  L.hbuf = reinterpret_cast<float*>(ws + lay.hbuf);
  L.ybuf = reinterpret_cast<float*>(ws + lay.ybuf);
  L.n_max = a->n_max;
  // (null: the address lookup failed - a first call on this device made inside stream capture, or a
  // device ordinal beyond the table; the kernels write through this pointer when a wait gives up)
  L.status = status_word();
  if (L.status == nullptr) return kErrLaunch;
  L.wait_flags = a->wait_flags; L.wait_step = a->wait_step;
  L.wait_count = a->wait_count; L.wait_mul = a->wait_mul; L.wait_add = a->wait_add;
  L.wait_limit = g_wait_limit.load(std::memory_order_relaxed);
  if (L.wait_flags != nullptr && (!a->routing_given || !L.wait_step || L.wait_count < 0 || L.wait_count > 128)) return kErrArg;
  if (a->ep_dst != nullptr || a->ep_out != nullptr) {
    if (!a->ep_flags || !a->ep_step || a->ep_world <= 0 || a->ep_world > 64) return kErrArg;
    if (a->ep_dst != nullptr) {              // home side: route without plan, records at xq_out
      if ((stages & 15) != 9 || a->xq_out == nullptr || a->ep_rec_bytes <= 0 || (a->ep_rec_bytes & 15) ||
          (reinterpret_cast<uintptr_t>(a->xq_out) & 15u))
        return kErrArg;
      L.ep_dst = a->ep_dst;
      L.ep_src = static_cast<const unsigned char*>(a->xq_out);
      L.ep_rec = a->ep_rec_bytes;
    } else {                                 // owner side
      if (!a->routing_given || a->ep_home_rows <= 0 || !a->no_residual) return kErrArg;
      L.ep_out = a->ep_out;
      L.ep_home = a->ep_home_rows;
    }
    L.ep_flags = a->ep_flags;
    L.ep_step = a->ep_step;
    L.ep_world = a->ep_world;
    L.ep_mul = a->ep_mul;
    L.ep_add = a->ep_add;
  }
  // Which expert kernel: the row-streaming one pays once a layer has enough tiles to
  // give every SM whole groups (bit 4 of `stages` forces it, bit 5 forces the item
  // kernel; both stages of a split call must be given the same bits).
  // (a workspace sized for the item kernel only keeps the item kernel)
  const bool use_rows = (stages & 32) ? false
                        : ((stages & 16) ? true
                                         : a->n >= kRowsKernelMinRows && a->workspace_bytes >= lay.total);
  if (a->ep_out != nullptr && !use_rows) return kErrUnsupported;   // the peer stores live in the row-streaming kernel's tail
  L.tok_tile = use_rows ? rs::kTok : kTokTile;
  if (a->workspace_bytes < (use_rows ? lay.total : lay.items_total)) return kErrArg;
  if (L.xq_padded) {
    // rows in 288-byte blocks travel between ranks: the row-streaming kernel reads them in place
    // (given routing), or the route stage writes them instead of the packed rows (xq_out)
    const int stride = a->xq_stride > 0 ? a->xq_stride : L.nbh * 288;
    if (stride < L.nbh * 288 || (stride & 15)) return kErrArg;
    if (a->xq_in != nullptr) {
      if (!use_rows || (reinterpret_cast<uintptr_t>(a->xq_in) & 15u)) return kErrUnsupported;
      L.xq16 = const_cast<unsigned char*>(static_cast<const unsigned char*>(a->xq_in));
      L.xq16_stride = stride;
    } else if (a->xq_out != nullptr) {
      if (reinterpret_cast<uintptr_t>(a->xq_out) & 15u) return kErrAlign;
      L.xq16 = static_cast<unsigned char*>(a->xq_out);
      L.xq16_stride = stride;
      L.xq = ws + lay.xq;                      // the packed rows stay in the workspace
      L.xq_stride = L.nbh * kX8;
    }
  }
  // the row-streaming kernel plans for itself when the routing is this call's own and the plan fits
  // the shared memory set aside for it
  const bool plan_fits = L.E <= rs::kPlanExperts && a->n_max * a->n_used <= rs::kPlanRoutes;
  L.plan_in_kernel = (use_rows && !a->routing_given && plan_fits) ? 1 : 0;
  if (stages & 128) {
    // owner side of an expert-parallel layer without a plan launch: routing given in records of padded
    // blocks, counters re-armed by the home call's route stage (rearm_workspace of that call)
    if ((stages & 7) != 6 || !use_rows || !a->routing_given || !a->xq_in || !L.xq_padded || !plan_fits) return kErrUnsupported;
    L.plan_in_kernel = 1;
  }
  if (a->rearm_workspace != nullptr) {
    if (!(stages & 1) || a->routing_given || a->rearm_n_max <= 0 || a->rearm_n_max > kMaxRows ||
        (reinterpret_cast<uintptr_t>(a->rearm_workspace) & 255u))
      return kErrArg;
    const WsLayout lay2 = ws_layout(a->rearm_n_max, a->hidden, a->n_ff, a->n_expert, a->n_used);
    unsigned char* ws2 = static_cast<unsigned char*>(a->rearm_workspace);
    L.rearm_cnt = reinterpret_cast<unsigned*>(ws2 + lay2.cnt);
    L.rearm_tile_cnt = reinterpret_cast<unsigned*>(ws2 + lay2.tile_cnt);
    L.rearm_blk_cnt = reinterpret_cast<unsigned*>(ws2 + lay2.blk_cnt);
    L.rearm_ready = reinterpret_cast<unsigned*>(ws2 + lay2.ready);
    L.rearm_tiles = a->rearm_n_max * a->n_used + a->rearm_n_max;
    L.rearm_mail_n = a->rearm_mail_n;
  }
  if (use_rows && (!matrix_tmap(L.nbh * kW4, L.FF, a->workspace, L.tmap_gu) ||
                   !matrix_tmap(L.nbf * kW4, L.H, a->workspace, L.tmap_dn)))
    return kErrUnsupported;
  {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return kErrLaunch;
    L.grid = std::min(sms, kMaxGrid);
  }
  cudaStream_t s = as_stream(stream);

  // A few token rows, whole layer on this device, all stages in one call: the single
  // persistent launch (token_layer.cuh). Bit 6 of `stages` keeps the two-launch path.
  if ((stages & 7) == 7 && !(stages & (8 | 16 | 32 | 64)) && a->n <= kTokenKernelMaxRows && a->n * a->n_used <= 32 &&
      !a->routing_given && a->xq_in == nullptr && a->xq_out == nullptr && a->wait_flags == nullptr &&
      a->ep_dst == nullptr && a->ep_out == nullptr &&
      L.e_lo == 0 && L.e_hi == L.E && L.sh_lo == 0 && L.sh_hi == L.n && L.nbh <= 16 && L.nbf <= 16 &&
      a->workspace_bytes >= lay.items_total) {
    const tk::Geom g = tk::geom(tk::kMaxTok, L.H, L.FF, L.E, L.grid);
    if (g.total <= 227 * 1024 && g.rows_per_cta <= tk::kWarps)
      return launch_pdl(tk::token_layer_kernel, dim3(L.grid), tk::kThreads, g.total, s, L);
  }

  int rc = kOk;
  if (!(stages & 1)) {
    // plan, xq and routing are taken from the workspace as a previous call left them
  } else if (!a->routing_given) {
    const size_t smem = std::max<size_t>(
        std::max<size_t>(static_cast<size_t>(kRouteTok + kRouteRows) * L.H * 4, static_cast<size_t>(kRouteTok) * L.E * 4),
        plan_smem(L.E, L.n_max, L.K));
    if (smem > 200 * 1024) return kErrUnsupported;
    rc = launch_pdl(route_kernel, dim3((L.E + kRouteRows - 1) / kRouteRows, (L.n + kRouteTok - 1) / kRouteTok),
                    kRouteWarps * 32, smem, s, L);
  } else {
    if (!a->xq_in) return kErrArg;
    rc = launch_pdl(plan_kernel, dim3(1), 256, plan_smem(L.E, L.n_max, L.K), s, L);
  }
  if (rc != kOk) return rc;

  if ((stages & 6) && use_rows) {
    const int sms = L.grid;
    if (!(stages & 1) && !(stages & 128)) {
      rc = launch_pdl(rearm_kernel, dim3(1), 256, 0, s, L);
      if (rc != kOk) return rc;
    }
    rc = launch_pdl(rs::expert_rows_kernel, dim3(sms), rs::kThreads, rs::kSmem, s, L);
  } else if (stages & 6) {
    // geometry the consumer mapping was written for: a tile of rows is one 16-row
    // group, or at most eight (group, super-block) units
    const StreamGeom g = stream_geom(L.H, L.FF);
    auto units_ok = [](int rows, int nb) { const int grp = (rows + 15) / 16; return grp == 1 || grp * nb <= kTeamWarps; };
    if (!units_ok(g.rows_gu, L.nbh) || !units_ok(g.rows_dn, L.nbf)) return kErrUnsupported;
    const size_t smem = stream_smem(L.H, L.FF);
    if (smem > 227 * 1024) return kErrUnsupported;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return kErrLaunch;
    if (!(stages & 1)) {
      rc = launch_pdl(rearm_kernel, dim3(1), 256, 0, s, L);
      if (rc != kOk) return rc;
    }
    rc = launch_pdl(expert_stream_kernel, dim3(sms), kStreamThreads, smem, s, L);
  }
  return rc;
}


SGR_API int sgr_moe_layer_decode(const sgr_moe_layer* a, void* stream) {
  return sgr_moe_layer_decode_stages(a, 7, stream);
}

SGR_API int sgr_ep_reduce_add_f16(uint16_t* x_f16, const float* parts, int n_parts,
                                  long long part_stride, long long count, void* stream) {
  if (count <= 0 || n_parts <= 0) return kOk;
  if (!x_f16 || !parts || part_stride < count) return kErrArg;
  const int blocks = static_cast<int>(std::min<long long>((count + 255) / 256, 148 * 4));
  ep_reduce_add_kernel<<<blocks, 256, 0, as_stream(stream)>>>(x_f16, parts, n_parts,
                                                            static_cast<size_t>(part_stride),
                                                            static_cast<size_t>(count));
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}

namespace {
template <typename... Args>
int launch_pdl_args(void (*kern)(Args...), dim3 grid, int threads, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...) == cudaSuccess ? kOk : kErrLaunch;
}
}  // namespace

SGR_API int sgr_ep_push(const void* src, long long src_stride, long long bytes, void* const* dst,
                        unsigned* const* flags, int world, const unsigned* step, int mul, int add,
                        unsigned* scratch, void* stream) {
  if (world <= 0 || bytes <= 0) return kOk;
  if (!src || !dst || !flags || !step || !scratch || world > 64 || src_stride < 0) return kErrArg;
  if ((reinterpret_cast<uintptr_t>(src) & 15u) || (bytes & 15) || (src_stride & 15)) return kErrAlign;
  const int chunks = static_cast<int>(std::min<long long>(16, (bytes + 4095) / 4096));
  return launch_pdl_args(ep_push_kernel, dim3(chunks, world), 256, as_stream(stream),
                         static_cast<const unsigned char*>(src), static_cast<size_t>(src_stride),
                         static_cast<size_t>(bytes), dst, flags, world, step, mul, add, scratch);
}

SGR_API int sgr_ep_reduce_add_f16_wait(uint16_t* x_f16, const float* parts, int n_parts, long long part_stride,
                                       long long count, const unsigned* flags, const unsigned* step, int mul,
                                       int add, void* stream) {
  if (count <= 0 || n_parts <= 0) return kOk;
  if (!x_f16 || !parts || part_stride < count || !flags || !step || n_parts > 128) return kErrArg;
  const int blocks = static_cast<int>(std::min<long long>((count + 255) / 256, 148 * 2));
  int* status = status_word();
  if (status == nullptr) return kErrLaunch;
  return launch_pdl_args(ep_reduce_add_wait_kernel, dim3(blocks), 256, as_stream(stream), x_f16, parts, n_parts,
                         static_cast<size_t>(part_stride), static_cast<size_t>(count), flags, step, mul, add,
                         g_wait_limit.load(std::memory_order_relaxed), status);
}

SGR_API int sgr_ep_set_wait_limit(int polls) {
  if (polls <= 0) return kErrArg;
  g_wait_limit.store(static_cast<unsigned>(polls), std::memory_order_relaxed);
  return kOk;
}

SGR_API int sgr_ep_step_advance(unsigned* step, void* stream) {
  if (!step) return kErrArg;
  return launch_pdl_args(ep_step_kernel, dim3(1), 32, as_stream(stream), step);
}

SGR_API size_t sgr_moe_layer_static_limit(void) { return kStaticWsBytes; }

// The fused layer for callers that may not allocate device memory. `workspace`
// and `workspace_bytes` of the argument block are ignored: the scratch is the
// library's own file-scope device array of sgr_moe_layer_static_limit() bytes.
// In host code that array's name is only a stand-in, so the first call on a
// device asks the runtime for the array's device address (with that device
// current), and every later call reuses it; that first call must therefore be
// made outside stream capture. Nothing here calls cudaMalloc, cudaFree or any
// allocating library routine. All calls on a device share the one array and it
// keeps what the previous call left: the counters that must start at zero are
// cleared on the stream before the kernels run, and two calls that overlap on the
// GPU (different streams, or graphs replayed concurrently) would race on it.
SGR_API int sgr_moe_layer_decode_static(const sgr_moe_layer* a, void* stream) {
  if (a == nullptr) return kErrArg;
  if (a->n <= 0) return kOk;
  if (a->hidden <= 0 || a->hidden % kQK || a->n_ff <= 0 || a->n_ff % kQK || a->n_expert <= 0 ||
      a->n_used <= 0 || a->n_max < a->n || a->n_max > kMaxRows)
    return kErrGeometry;
  const WsLayout lay = ws_layout(a->n_max, a->hidden, a->n_ff, a->n_expert, a->n_used);
  // The whole layout must fit, so that the call picks its expert kernel exactly as a call on a
  // caller's workspace of sgr_moe_layer_workspace_bytes() does.
  if (lay.total > kStaticWsBytes) return kErrStaticLimit;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return kErrLaunch;
  if (g_static_ws_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_ws) != cudaSuccess || p == nullptr) return kErrLaunch;
    g_static_ws_addr[dev] = static_cast<unsigned char*>(p);
  }
  unsigned char* ws = g_static_ws_addr[dev];
  // what must start at zero: the counters of the route and expert kernels, [cnt, hbuf) of the layout
  // (cnt, tile_cnt, blk_cnt, ready are adjacent)
  if (cudaMemsetAsync(ws + lay.cnt, 0, lay.hbuf - lay.cnt, as_stream(stream)) != cudaSuccess)
    return kErrLaunch;
  sgr_moe_layer b = *a;
  b.workspace = ws;
  b.workspace_bytes = kStaticWsBytes;
  return sgr_moe_layer_decode_stages(&b, 7, stream);
}
