// token_layer.cuh - one MoE layer for one to four token rows in ONE persistent launch
// (part of moe_layer.cu, which defines LayerDev, the workspace and the helpers used here).
//
// The single-token layer is latency-bound: 18 MB of weights are 3 us of HBM time, and
// every dependent step around them - a launch, a global round trip, a grid-wide
// barrier - costs about as much again. This kernel keeps the chain as short as the data
// dependencies allow. One CTA per SM, eight consumer warps and a producer warp:
//
//   before the previous kernel's results are needed (programmatic dependent launch):
//     the CTA's router rows and its share of the shared expert's gate / up / down rows
//     are already on their way into shared memory - none of them depends on routing
//   phase 1  Q8_K-quantise the rows (every CTA, redundantly: 4 KB per row), logits of the
//            CTA's experts (one warp per expert row, the reference kernel's FMA order, so
//            logits are bit-identical), grid barrier
//   phase 2  every CTA selects redundantly from the n x E logits (one warp per row) and
//            builds the same list of tiles (distinct experts, each with the set of rows
//            routed to it). The producer warp then issues EVERY weight byte this CTA will
//            need as bulk copies (TMA): its pairs of the routed gate / up rows AND its
//            rows of the down matrices, so the down weights arrive while gate / up
//            computes and the second half of the layer never waits for memory
//   phase 3  gate / up dots (dp4a, integer sub-block dots exact), SwiGLU, fp32 h rows to
//            global memory, grid barrier
//   phase 4  every CTA quantises the h rows it needs (all of them: a few KB from L2),
//            runs the down dots for its H / grid output rows of EVERY tile, and - since
//            all of a row's expert contributions are then in this CTA - adds
//            residual + sum_k w_k * y_k + shared in place. No third barrier.
//
// Work split: gate / up by pairs (a flat range of (tile, pair) per CTA), down by output
// rows. Contracts are those of the two-launch path: null table entry = absent expert
// (zero contribution, id mailed), weight pointers may be only 2-byte aligned (then the
// producer copies with plain loads), routing written to route_idx / route_w.
#pragma once

namespace tk {

constexpr int kMaxTok = 4;                 // token rows per call
constexpr int kWarps = 8;                  // consumer warps
constexpr int kConsumers = kWarps * 32;
constexpr int kThreads = kConsumers + 32;  // + producer warp
constexpr int kPairsStage = 16;            // (gate, up) row pairs per ring stage
constexpr int kRing = 2;
constexpr int kDownTiles = 16;             // tiles whose down rows are resident at once
constexpr int kMaxTiles = 33;              // n * K + 1 <= 33
constexpr int kMaxHRows = 36;              // (tile, row) pairs: n * K + n <= 36
constexpr int kHdr = 1024;
constexpr int kTables = 4096;

struct Tables {                            // built after the selection, the same in every CTA
  int n_tiles;
  int n_hrows;
  int tile_e[kMaxTiles];                   // expert id (E = shared)
  int tile_mask[kMaxTiles];                // rows routed to it
  int tile_hrow0[kMaxTiles];               // first h / y row
  int tile_mode[kMaxTiles];                // 0 TMA, 1 absent, 2 plain loads (unaligned pointers)
  const unsigned char* w[3][kMaxTiles];
  int sel_idx[kMaxTok][kMaxTiles];         // [t][0..K]
  float sel_w[kMaxTok][kMaxTiles];
  int route_hrow[kMaxTok][kMaxTiles];      // [t][kk] -> h / y row of that route, -1 = absent; [t][K] = shared
  XTile xt;                                // the quantised input rows
  XTile hq;                                // the quantised h rows
};
static_assert(sizeof(Tables) <= kTables, "tables region");

struct StageDesc {
  int tile, pair0, np, mode;
};

struct Geom {
  int rows_per_cta;      // router rows per CTA
  int nr_max;            // output rows per CTA (down split)
  int sp_max;            // shared-expert pairs per CTA
  int rb_h, rb_f;        // bytes per gate/up row, per down row
  size_t off_prob, off_ptab, off_xh, off_rw, off_xt, off_sh, off_ring, off_dn, off_y, total;
  int stage_bytes, slot_bytes;
};
__host__ __device__ inline Geom geom(int n_max, int H, int FF, int E, int grid) {
  Geom g;
  g.rows_per_cta = (E + grid - 1) / grid;
  g.nr_max = (H + grid - 1) / grid;
  g.sp_max = (FF + grid - 1) / grid;
  g.rb_h = (H / kQK) * kW4;
  g.rb_f = (FF / kQK) * kW4;
  size_t p = kHdr + kTables;
  auto take = [&](size_t bytes) { const size_t at = p; p = (p + bytes + 127) & ~static_cast<size_t>(127); return at; };
  g.off_prob = take(static_cast<size_t>(kMaxTok) * E * 4);
  g.off_ptab = take(static_cast<size_t>(3) * E * 8);        // the layer's pointer table, read once per CTA
  // x rows as fp16 and the router rows; later the same bytes hold the quantised h rows
  const size_t a = static_cast<size_t>(kMaxTok) * H * 2 + 128 + static_cast<size_t>(g.rows_per_cta) * H * 4;
  const size_t b = xtile_bytes(kMaxHRows, FF / kQK);
  g.off_xh = take(a > b ? a : b);
  g.off_rw = g.off_xh + ((static_cast<size_t>(kMaxTok) * H * 2 + 127) & ~static_cast<size_t>(127));
  g.off_xt = take(xtile_bytes(kMaxTok, H / kQK));
  g.off_sh = take(static_cast<size_t>(2) * g.sp_max * g.rb_h);
  g.stage_bytes = 2 * kPairsStage * g.rb_h;
  g.off_ring = take(static_cast<size_t>(kRing) * g.stage_bytes);
  g.slot_bytes = g.nr_max * g.rb_f;
  g.off_dn = take(static_cast<size_t>(kDownTiles) * g.slot_bytes);
  g.off_y = take(static_cast<size_t>(kMaxHRows) * g.nr_max * 4);
  g.total = p;
  return g;
}

__device__ __forceinline__ void consumers_sync() {
  asm volatile("bar.sync 6, %0;" ::"n"(kConsumers) : "memory");
}
// CTA barrier of the consumers that also tells whether `ok` held in every one of them.
__device__ __forceinline__ bool consumers_all(bool ok) {
  int r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 6, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(ok ? 1 : 0), "n"(kConsumers)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Grid-wide barrier on a 64-bit arrival counter that only ever grows: the k-th barrier of the
// grid (over all launches on this workspace) completes when the counter reaches k * G. Waits are
// bounded: false when the others did not arrive in time.
// The grid barrier is driven by ONE thread per CTA that has no part in the work around it
// (the last consumer thread): at kernel start it reads the counter - some multiple of the
// grid size plus the arrivals of CTAs that are already further on, none of which can have
// passed the first barrier - so barrier k of this launch completes at base + k * grid. An
// arrival is a fence and a fire-and-forget add; nobody waits for the add's round trip.
__device__ __forceinline__ unsigned long long grid_base(const unsigned long long* ctr, unsigned grid) {
  return ld_acquire_u64(ctr) / grid * grid;
}
__device__ __forceinline__ void grid_arrive(unsigned long long* ctr) {
  __threadfence();
  asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(ctr) : "memory");
}
__device__ __forceinline__ bool grid_wait(const unsigned long long* ctr, unsigned long long target) {
  unsigned it = 0;
  while (ld_acquire_u64(ctr) < target && ++it < kSpinLimit) {
  }
  return it < kSpinLimit;
}

// Q8_K-quantise `rows` fp32 rows of h (global memory, FF values each) into a staged tile, a warp
// per 256-value block, four blocks' loads in flight per warp (arithmetic of stage_quantized_f32).
__device__ __forceinline__ void quantize_h_rows(const XTile& xt, int rows, const float* src, int FF, int warp, int lane) {
  const int jobs = rows * xt.nb;
  for (int j0 = warp; j0 < jobs; j0 += 4 * kWarps) {
    float4 a[4], b[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int job = min(j0 + u * kWarps, jobs - 1);
      const int t = job / xt.nb, blk = job - t * xt.nb;
      const float4* p = reinterpret_cast<const float4*>(src + static_cast<size_t>(t) * FF + blk * kQK) + lane * 2;
      a[u] = __ldcg(p);
      b[u] = __ldcg(p + 1);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int job = j0 + u * kWarps;
      if (job >= jobs) break;                    // warp-uniform
      const int t = job / xt.nb, blk = job - t * xt.nb;
      const float v[8] = {a[u].x, a[u].y, a[u].z, a[u].w, b[u].x, b[u].y, b[u].z, b[u].w};
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
      const int sum_next = __shfl_down_sync(0xFFFFFFFFu, sum, 4);
      if ((lane & 7) == 0)
        xt.put_sum_pair(t, blk, lane >> 3, (static_cast<uint32_t>(sum) & 0xFFFFu) | (static_cast<uint32_t>(sum_next) << 16));
      if (lane == 0) xt.d[t * xt.nb + blk] = d;
    }
  }
}

// The staged rows of a tile: row `base + (position of the t-th set bit of mask)` when by_bit
// (activation rows are indexed by token), `base + t` otherwise (h rows are stored per tile).
struct RowSet {
  int r0, r1, r2, r3, n;
  __device__ __forceinline__ int at(int t) const { return t == 0 ? r0 : (t == 1 ? r1 : (t == 2 ? r2 : r3)); }
};
__device__ __forceinline__ RowSet rows_of(int mask, int base, bool by_bit) {
  RowSet r;
  r.n = __popc(mask);
  r.r0 = base + (by_bit ? static_cast<int>(__fns(mask, 0, 1)) : 0);
  r.r1 = base + (by_bit ? static_cast<int>(__fns(mask, 0, 2)) : 1);
  r.r2 = base + (by_bit ? static_cast<int>(__fns(mask, 0, 3)) : 2);
  r.r3 = base + (by_bit ? static_cast<int>(__fns(mask, 0, 4)) : 3);
  return r;
}

// block_dot of q4k_common.cuh for one matrix and up to kMaxTok staged rows chosen by index.
// Deliberately NOT inlined and NOT unrolled over rows or nibble groups: every phase of this kernel
// runs once per CTA, so straight-line code is paid for in instruction fetch, not in issue slots
// (measured: the unrolled form spent 2.5 us per call site fetching ~12 KB of code). One compact
// loop serves the shared expert's gate / up, the routed gate / up and the down rows.
__device__ __noinline__ float4 block_dot_rows(const uint4* wblk, const XTile* xtp, int blk, RowSet rs) {
  const XTile& xt = *xtp;
  const uint4 hdr = wblk[0];
  const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x & 0xFFFFu)));
  const float dmin = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x >> 16)));
  const Scales6 s6 = unpack_scales6(hdr.y, hdr.z, hdr.w);
  float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
  for (int t = 0; t < rs.n; ++t) {
    const int r = rs.at(t);
    int isum = 0;
#pragma unroll 1
    for (int g = 0; g < 4; ++g) {
      const uint4 q0 = wblk[1 + 2 * g], q1 = wblk[2 + 2 * g];
      const uint32_t raw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      uint32_t lo[8], hi[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        lo[i] = raw[i] & 0x0F0F0F0Fu;
        hi[i] = (raw[i] >> 4) & 0x0F0F0F0Fu;
      }
      const uint32_t scw = (g & 2) ? s6.sc[1] : s6.sc[0];
      const int sc_lo = (scw >> (16 * (g & 1))) & 0xFF;
      const int sc_hi = (scw >> (16 * (g & 1) + 8)) & 0xFF;
      const uint4* xa = xt.codes(r, blk, 2 * g);
      const uint4 x0 = xa[0], x1 = xa[1], x2 = xa[2], x3 = xa[3];
      isum += sc_lo * dot8(lo, x0, x1) + sc_hi * dot8(hi, x2, x3);
    }
    const uint4 bs = xt.sums(r, blk);
    int msum = __dp2a_lo(static_cast<int>(bs.x), static_cast<int>(s6.mn[0]), 0);
    msum = __dp2a_hi(static_cast<int>(bs.y), static_cast<int>(s6.mn[0]), msum);
    msum = __dp2a_lo(static_cast<int>(bs.z), static_cast<int>(s6.mn[1]), msum);
    msum = __dp2a_hi(static_cast<int>(bs.w), static_cast<int>(s6.mn[1]), msum);
    const float v = xt.scale(r, blk) * (d * static_cast<float>(isum) - dmin * static_cast<float>(msum));
    if (t == 0) out.x = v;
    else if (t == 1) out.y = v;
    else if (t == 2) out.z = v;
    else out.w = v;
  }
  return out;
}

// Gate / up of `np` pairs staged at st (gate rows, then up rows) for the rows `mask` of one tile:
// thread = (pair, matrix, block lane); the lanes of a row add up with shuffles and the up row's
// lanes sit `lpr` lanes above the gate row's. SwiGLU, fp32 h rows [hrow0 + slot][FF] to global
// memory. One copy of this code serves the shared expert's stage and the ring stages.
__device__ __noinline__ void gate_up_stage(const unsigned char* st, int np, int mask, int hrow0, int pair0,
                                           const XTile* xt, float* hbuf, int FF, int nbh, int rb_h) {
  const int tid = threadIdx.x;
  const int lpr = next_pow2_cap32(nbh);
  const RowSet rs = rows_of(mask, 0, true);
  const int tasks = np * 2 * lpr;
#pragma unroll 1
  for (int base = 0; base < tasks; base += kConsumers) {        // uniform trip count
    const int q = base + tid;
    const int lr = q & (lpr - 1);
    const int rm = q / lpr;
    const int m = rm & 1, pair = rm >> 1;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q < tasks) {
      const unsigned char* row = st + static_cast<size_t>(m) * np * rb_h + static_cast<size_t>(pair) * rb_h;
#pragma unroll 1
      for (int blk = lr; blk < nbh; blk += lpr) {
        const float4 v = block_dot_rows(reinterpret_cast<const uint4*>(row + blk * kW4), xt, blk, rs);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    const float av[kMaxTok] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int t = 0; t < kMaxTok; ++t) {
      const float g = reduce_lanes(av[t], lpr);
      const float u = __shfl_down_sync(0xFFFFFFFFu, g, lpr);
      if (q < tasks && lr == 0 && m == 0 && t < rs.n)
        hbuf[static_cast<size_t>(hrow0 + t) * FF + pair0 + pair] = g / (1.f + expf(-g)) * u;
    }
  }
}

// One warp: Q8_K-quantise 256 fp16 values (eight per lane, `raw`) into block `blk` of row t of
// a staged tile (arithmetic of src/kernels/cuda/q4_k.cu:94-130 in the reference).
__device__ __forceinline__ void quantize_f16_to_tile(const XTile& xt, int t, int blk, const uint4 raw, int lane) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  float v[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = h2f(static_cast<uint16_t>(w[i] & 0xFFFFu));
    v[2 * i + 1] = h2f(static_cast<uint16_t>(w[i] >> 16));
  }
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
  const int sum_next = __shfl_down_sync(0xFFFFFFFFu, sum, 4);
  if ((lane & 7) == 0)
    xt.put_sum_pair(t, blk, lane >> 3, (static_cast<uint32_t>(sum) & 0xFFFFu) | (static_cast<uint32_t>(sum_next) << 16));
  if (lane == 0) xt.d[t * xt.nb + blk] = d;
}

// Producer: `bytes` (a multiple of 16) from a source that may be only 2-byte aligned.
__device__ __forceinline__ void copy_plain(unsigned char* dst, const unsigned char* src, int bytes, int lane) {
  for (int p = lane; p < bytes / 16; p += 32) rs::copy16_any(dst + p * 16, src + static_cast<size_t>(p) * 16);
}

__global__ void __launch_bounds__(kThreads, 1) token_layer_kernel(const LayerDev L) {
  extern __shared__ __align__(128) unsigned char smem[];
  const Geom G = geom(kMaxTok, L.H, L.FF, L.E, gridDim.x);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);              // [kRing]
  uint64_t* empty = full + kRing;                                  // [kRing]
  uint64_t* sh_full = empty + kRing;                               // shared expert's gate / up pairs
  uint64_t* shdn_full = sh_full + 1;                               // shared expert's down rows (slot 0)
  uint64_t* dn_full = shdn_full + 1;                               // routed tiles' down rows, one phase per round
  uint64_t* dn_empty = dn_full + 1;
  uint64_t* ready = dn_empty + 1;                                  // tables built
  StageDesc* desc = reinterpret_cast<StageDesc*>(smem + 128);      // [kRing]
  int* flag = reinterpret_cast<int*>(smem + 256);
  Tables& tb = *reinterpret_cast<Tables*>(smem + kHdr);
  float* prob = reinterpret_cast<float*>(smem + G.off_prob);
  const unsigned char** ptab = reinterpret_cast<const unsigned char**>(smem + G.off_ptab);   // [3][E]
  uint16_t* xh = reinterpret_cast<uint16_t*>(smem + G.off_xh);     // [n][H] fp16
  float* rw = reinterpret_cast<float*>(smem + G.off_rw);           // [rows_per_cta][H]
  unsigned char* sh_stage = smem + G.off_sh;
  unsigned char* ring = smem + G.off_ring;
  unsigned char* dn = smem + G.off_dn;
  float* ysm = reinterpret_cast<float*>(smem + G.off_y);           // [hrow][nr_max]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, grid = gridDim.x;
  const int n = L.n, H = L.H, FF = L.FF, E = L.E, K = L.K;
  const bool has_shared = L.sh[0] != nullptr;
  unsigned long long* gctr = reinterpret_cast<unsigned long long*>(L.cnt + 12);

  // this CTA's shares: shared-expert pairs [sp0, sp1), output rows [r0, r1)
  const int sp0 = static_cast<int>(static_cast<long long>(FF) * cta / grid);
  const int sp1 = static_cast<int>(static_cast<long long>(FF) * (cta + 1) / grid);
  const int r0 = static_cast<int>(static_cast<long long>(H) * cta / grid);
  const int r1 = static_cast<int>(static_cast<long long>(H) * (cta + 1) / grid);
  const int nr = r1 - r0;

  if (tid == 0) {
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kWarps);
    }
    mbar_init(sh_full, 1);
    mbar_init(shdn_full, 1);
    mbar_init(dn_full, 1);
    mbar_init(dn_empty, kWarps);
    mbar_init(ready, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  if (warp == kWarps) {
    // ---------------- producer warp ----------------
    const bool sh_aligned = ((reinterpret_cast<uintptr_t>(L.sh[0]) | reinterpret_cast<uintptr_t>(L.sh[1]) |
                              reinterpret_cast<uintptr_t>(L.sh[2])) & 15u) == 0;
    if (has_shared) {
      // the shared expert's weights are fixed: fetch this CTA's share before anything else
      const int np = sp1 - sp0;
      if (sh_aligned) {
        if (lane == 0) {
          if (np > 0) {
            mbar_expect_tx(sh_full, static_cast<uint32_t>(2 * np * G.rb_h));
            bulk_g2s(sh_stage, L.sh[0] + static_cast<size_t>(sp0) * G.rb_h, static_cast<uint32_t>(np * G.rb_h), sh_full);
            bulk_g2s(sh_stage + static_cast<size_t>(np) * G.rb_h, L.sh[1] + static_cast<size_t>(sp0) * G.rb_h,
                     static_cast<uint32_t>(np * G.rb_h), sh_full);
          } else {
            mbar_arrive_one(sh_full);
          }
          if (nr > 0) {
            mbar_expect_tx(shdn_full, static_cast<uint32_t>(nr * G.rb_f));
            bulk_g2s(dn, L.sh[2] + static_cast<size_t>(r0) * G.rb_f, static_cast<uint32_t>(nr * G.rb_f), shdn_full);
          } else {
            mbar_arrive_one(shdn_full);
          }
        }
      } else {
        copy_plain(sh_stage, L.sh[0] + static_cast<size_t>(sp0) * G.rb_h, np * G.rb_h, lane);
        copy_plain(sh_stage + static_cast<size_t>(np) * G.rb_h, L.sh[1] + static_cast<size_t>(sp0) * G.rb_h, np * G.rb_h, lane);
        copy_plain(dn, L.sh[2] + static_cast<size_t>(r0) * G.rb_f, nr * G.rb_f, lane);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_one(sh_full);
          mbar_arrive_one(shdn_full);
        }
      }
    }
    if (!mbar_wait(ready, 0)) {
      if (lane == 0) atomicExch(L.status, 7);
      return;
    }
    const int T = tb.n_tiles;
    const int t_first = has_shared ? 1 : 0;
    // routed gate / up pairs: a flat range of (tile, pair) per CTA
    const long long P = static_cast<long long>(T - t_first) * FF;
    const long long pa = P * cta / grid, pb = P * (cta + 1) / grid;
    long long pos = pa;
    int issued = 0;
    bool down_issued = false;
    int round = 0;
    const int rounds = (T + kDownTiles - 1) / kDownTiles;
    // down rows of the tiles of one round (tile 0 of round 0 is the shared expert's, fetched above)
    auto issue_down_round = [&](int rd) {
      const int j0 = rd * kDownTiles, j1 = min(T, j0 + kDownTiles);
      uint32_t bytes = 0;
      bool plain = false;
      for (int j = j0; j < j1; ++j) {
        if (j == 0 && has_shared) continue;
        if (tb.tile_mode[j] == 0) bytes += static_cast<uint32_t>(nr * G.rb_f);
        if (tb.tile_mode[j] == 2) plain = true;
      }
      if (plain) {
        for (int j = j0; j < j1; ++j)
          if (!(j == 0 && has_shared) && tb.tile_mode[j] == 2)
            copy_plain(dn + static_cast<size_t>(j - j0) * G.slot_bytes, tb.w[2][j] + static_cast<size_t>(r0) * G.rb_f,
                       nr * G.rb_f, lane);
        fence_proxy_async();
        __syncwarp();
      }
      if (lane == 0) {
        if (bytes > 0) {
          mbar_expect_tx(dn_full, bytes);
          for (int j = j0; j < j1; ++j)
            if (!(j == 0 && has_shared) && tb.tile_mode[j] == 0)
              bulk_g2s(dn + static_cast<size_t>(j - j0) * G.slot_bytes, tb.w[2][j] + static_cast<size_t>(r0) * G.rb_f,
                       static_cast<uint32_t>(nr * G.rb_f), dn_full);
        } else {
          mbar_arrive_one(dn_full);
        }
      }
    };
    while (pos < pb) {
      const int s = issued % kRing;
      const unsigned ph = (issued / kRing) & 1;
      if (issued == kRing && !down_issued) {        // the whole ring is in flight: now the down rows
        issue_down_round(0);
        down_issued = true;
        round = 1;
      }
      if (!mbar_wait(&empty[s], ph ^ 1u)) {
        if (lane == 0) atomicExch(L.status, 2);
        return;
      }
      const int tile = t_first + static_cast<int>(pos / FF);
      const int pair0 = static_cast<int>(pos - static_cast<long long>(tile - t_first) * FF);
      const int np = static_cast<int>(min(static_cast<long long>(kPairsStage), min(static_cast<long long>(FF - pair0), pb - pos)));
      const int mode = tb.tile_mode[tile];
      unsigned char* st = ring + static_cast<size_t>(s) * G.stage_bytes;
      if (lane == 0) {
        StageDesc d;
        d.tile = tile; d.pair0 = pair0; d.np = np; d.mode = mode;
        desc[s] = d;
      }
      if (mode == 2) {
        copy_plain(st, tb.w[0][tile] + static_cast<size_t>(pair0) * G.rb_h, np * G.rb_h, lane);
        copy_plain(st + static_cast<size_t>(np) * G.rb_h, tb.w[1][tile] + static_cast<size_t>(pair0) * G.rb_h, np * G.rb_h, lane);
        fence_proxy_async();
      }
      __syncwarp();
      if (lane == 0) {
        if (mode == 0) {
          mbar_expect_tx(&full[s], static_cast<uint32_t>(2 * np * G.rb_h));
          bulk_g2s(st, tb.w[0][tile] + static_cast<size_t>(pair0) * G.rb_h, static_cast<uint32_t>(np * G.rb_h), &full[s]);
          bulk_g2s(st + static_cast<size_t>(np) * G.rb_h, tb.w[1][tile] + static_cast<size_t>(pair0) * G.rb_h,
                   static_cast<uint32_t>(np * G.rb_h), &full[s]);
        } else {
          mbar_arrive_one(&full[s]);
        }
      }
      pos += np;
      ++issued;
    }
    if (!down_issued) {
      issue_down_round(0);
      round = 1;
    }
    for (; round < rounds; ++round) {               // later rounds reuse the region
      if (!mbar_wait(dn_empty, (round - 1) & 1)) {
        if (lane == 0) atomicExch(L.status, 2);
        return;
      }
      issue_down_round(round);
    }
    return;
  }

  // ---------------- consumers ----------------
  const bool bar_thread = tid == kConsumers - 1;
  unsigned long long bar_base = 0;
  if (bar_thread) bar_base = grid_base(gctr, grid);
  // router rows of this CTA's experts: fixed weights, on their way before the previous kernel is awaited
  if (warp < G.rows_per_cta) {
    const int e = cta + warp * grid;
    if (e < E) {
      const float* src = L.router_w + static_cast<size_t>(e) * H;
      float* dst = rw + static_cast<size_t>(warp) * H;
      if ((reinterpret_cast<uintptr_t>(L.router_w) & 15u) == 0) {
        for (int c = lane * 4; c < H; c += 128)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + c)), "l"(src + c) : "memory");
      } else {
        for (int c = lane; c < H; c += 32) dst[c] = __ldg(src + c);
      }
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  if (cta == 0 && tid == 0 && L.mail_n != nullptr) *L.mail_n = 0;

  // The layer's pointer table (3 x E pointers: after the selection the experts' addresses are then
  // one shared-memory read away) and the x rows: a warp fetches a 256-value block (16 bytes per
  // lane), keeps it as fp16 for the logits and quantises it from its registers; up to four blocks'
  // loads are in flight per warp.
  for (int i = tid; i < 3 * E; i += kConsumers) {
    const int m = i / E, e = i - m * E;
    ptab[i] = L.tab[static_cast<size_t>(m) * L.tab_stride + e];
  }
  const XTile xt = xtile_at(smem + G.off_xt, kMaxTok, L.nbh);
  if (tid == 0) {
    tb.xt = xt;
    tb.hq = xtile_at(smem + G.off_xh, kMaxHRows, L.nbf);
  }
  {
    const int jobs = n * L.nbh;
    for (int j0 = warp; j0 < jobs; j0 += 4 * kWarps) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int job = min(j0 + u * kWarps, jobs - 1);
        raw[u] = __ldcg(reinterpret_cast<const uint4*>(L.xn) + static_cast<size_t>(job) * 32 + lane);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int job = j0 + u * kWarps;
        if (job >= jobs) break;                  // warp-uniform
        reinterpret_cast<uint4*>(xh)[static_cast<size_t>(job) * 32 + lane] = raw[u];
        quantize_f16_to_tile(xt, job / L.nbh, job % L.nbh, raw[u], lane);
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  consumers_sync();                              // x rows (both forms), router rows and tables are in place
  // logits: one warp per expert row; lane l adds k = l, l + 32, ... in ascending order with FMA and
  // the lanes meet in a shuffle tree - the order of the reference's kernel (src/kernels/cuda/q4_k.cu:133-149).
  // Eight steps of loads are issued ahead of their FMAs.
  if (warp < G.rows_per_cta) {
    const int e = cta + warp * grid;
    if (e < E) {
      const float* wr = rw + static_cast<size_t>(warp) * H;
      float acc[kMaxTok] = {0.f, 0.f, 0.f, 0.f};
      int k = lane;
      for (; k + 7 * 32 < H; k += 8 * 32) {
        float wv[8];
        uint16_t xv[kMaxTok][8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          wv[j] = wr[k + 32 * j];
#pragma unroll
          for (int t = 0; t < kMaxTok; ++t) xv[t][j] = t < n ? xh[static_cast<size_t>(t) * H + k + 32 * j] : static_cast<uint16_t>(0);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int t = 0; t < kMaxTok; ++t)
            if (t < n) acc[t] = fmaf(wv[j], h2f(xv[t][j]), acc[t]);
      }
      for (; k < H; k += 32) {
        const float wv = wr[k];
#pragma unroll
        for (int t = 0; t < kMaxTok; ++t)
          if (t < n) acc[t] = fmaf(wv, h2f(xh[static_cast<size_t>(t) * H + k]), acc[t]);
      }
      const float b = L.bias != nullptr ? L.bias[e] : 0.f;
#pragma unroll
      for (int t = 0; t < kMaxTok; ++t) {
        float a = acc[t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a += __shfl_down_sync(0xFFFFFFFFu, a, off);
        if (lane == 0 && t < n) L.logits[static_cast<size_t>(t) * E + e] = a + b;
      }
    }
  }
  consumers_sync();
  if (bar_thread) grid_arrive(gctr);                       // arrive now; the wait comes after the shared expert's gate / up

  bool ok = true;
  // the shared expert does not depend on the routing: its gate / up share runs while the other
  // CTAs arrive at the barrier (tile 0: every row, h rows 0 .. n-1)
  if (has_shared && sp1 > sp0) {
    if (!mbar_wait(sh_full, 0)) ok = false;
    if (ok) gate_up_stage(sh_stage, sp1 - sp0, (1 << n) - 1, 0, sp0, &tb.xt, L.hbuf, FF, L.nbh, G.rb_h);
  }
  if (bar_thread) flag[0] = grid_wait(gctr, bar_base + grid) ? 1 : 0;
  consumers_sync();
  if (!flag[0]) {
    if (tid == 0) atomicExch(L.status, 5);
    return;
  }

  // ---- selection (every CTA, the same result) and the tile tables ----
  if (warp < n) {
    float* pr = prob + static_cast<size_t>(warp) * E;
    for (int i = lane; i < E; i += 32) pr[i] = __ldcg(L.logits + static_cast<size_t>(warp) * E + i);
    __syncwarp();
    router_select_warp(pr, E, K, tb.sel_idx[warp], tb.sel_w[warp], L.shared_w, true, lane);
  }
  consumers_sync();
  if (cta == 0 && tid < n * (K + 1)) {
    const int t = tid / (K + 1), kk = tid - t * (K + 1);
    if (kk < K) L.idx[static_cast<size_t>(t) * L.rstride + kk] = tb.sel_idx[t][kk];
    L.w[static_cast<size_t>(t) * L.rstride + kk] = tb.sel_w[t][kk];
  }
  const int t_first = has_shared ? 1 : 0;
  if (warp == 0) {
    // one lane per pick (n * K <= 32): picks of the same expert find each other with a match,
    // the lowest lane of a group founds the tile; tiles are numbered in pick order
    const int picks = n * K;
    const bool live = lane < picks;
    const int pt = live ? lane / K : 0, pk = live ? lane - pt * K : 0;
    const int e = live ? tb.sel_idx[pt][pk] : -1 - lane;             // dead lanes match nobody
    const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
    const bool leader = live && (__ffs(same) - 1 == lane);
    const unsigned leaders = __ballot_sync(0xFFFFFFFFu, leader);
    const int my_tile = t_first + __popc(leaders & ((1u << (__ffs(same) - 1)) - 1u));
    // rows of the tile: the token of every lane in the group
    int mask = 0;
    for (unsigned m = same; m != 0; m &= m - 1) mask |= 1 << ((__ffs(m) - 1) / K);
    if (has_shared && lane == 0) {
      tb.tile_e[0] = E;
      tb.tile_mask[0] = (1 << n) - 1;
      tb.w[0][0] = L.sh[0]; tb.w[1][0] = L.sh[1]; tb.w[2][0] = L.sh[2];
      tb.tile_mode[0] = ((reinterpret_cast<uintptr_t>(L.sh[0]) | reinterpret_cast<uintptr_t>(L.sh[1]) |
                          reinterpret_cast<uintptr_t>(L.sh[2])) & 15u) == 0 ? 0 : 2;
    }
    bool absent = false;
    if (leader) {
      const unsigned char *w0 = ptab[e], *w1 = ptab[E + e], *w2 = ptab[2 * E + e];
      absent = w0 == nullptr || w1 == nullptr || w2 == nullptr;
      const bool aligned = ((reinterpret_cast<uintptr_t>(w0) | reinterpret_cast<uintptr_t>(w1) |
                             reinterpret_cast<uintptr_t>(w2)) & 15u) == 0;
      tb.tile_e[my_tile] = e;
      tb.tile_mask[my_tile] = mask;
      tb.w[0][my_tile] = w0; tb.w[1][my_tile] = w1; tb.w[2][my_tile] = w2;
      tb.tile_mode[my_tile] = absent ? 1 : (aligned ? 0 : 2);
      if (absent && cta == 0 && L.mail != nullptr) {
        const int mi = atomicAdd(L.mail_n, 1);
        if (mi < E) L.mail[mi] = e;
      }
    }
    const int T = t_first + __popc(leaders);
    __syncwarp();
    // first h / y row of every tile: prefix sum of the tiles' row counts (lane j = tile j, T <= 33:
    // the last tile's start is the total minus its own rows)
    const int cnt = lane < T ? __popc(tb.tile_mask[lane]) : 0;
    int inc = cnt;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xFFFFFFFFu, inc, off);
      if (lane >= off) inc += v;
    }
    if (lane < T) tb.tile_hrow0[lane] = inc - cnt;
    const int total32 = __shfl_sync(0xFFFFFFFFu, inc, 31);
    if (lane == 0) {
      int hr = total32;
      if (T > 32) {
        tb.tile_hrow0[32] = hr;
        hr += __popc(tb.tile_mask[32]);
      }
      tb.n_tiles = T;
      tb.n_hrows = hr;
    }
    __syncwarp();
    if (live) {
      const bool gone = tb.tile_mode[my_tile] == 1;
      tb.route_hrow[pt][pk] = gone ? -1 : tb.tile_hrow0[my_tile] + __popc(mask & ((1 << pt) - 1));
    }
    if (lane < n) tb.route_hrow[lane][K] = has_shared ? lane : -1;
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      mbar_arrive_one(ready);                   // the producer may issue every weight copy now
    }
  }
  consumers_sync();
  const int T = tb.n_tiles;

  // ---- phase 3: gate / up of the routed tiles, SwiGLU ----
  {
    const long long P = static_cast<long long>(T - t_first) * FF;
    const long long pa = P * cta / grid, pb = P * (cta + 1) / grid;
    long long pos = pa;
    for (int i = 0; pos < pb && ok; ++i) {
      const int s = i % kRing;
      const unsigned ph = (i / kRing) & 1;
      if (!mbar_wait(&full[s], ph)) {
        ok = false;
        break;
      }
      const StageDesc d = desc[s];
      if (d.mode != 1)
        gate_up_stage(ring + static_cast<size_t>(s) * G.stage_bytes, d.np, tb.tile_mask[d.tile], tb.tile_hrow0[d.tile],
                      d.pair0, &tb.xt, L.hbuf, FF, L.nbh, G.rb_h);
      __syncwarp();
      if (lane == 0) mbar_arrive_one(&empty[s]);
      pos += d.np;
    }
  }
  ok = consumers_all(ok);                                   // (a wait that ran out in any thread ends the CTA's work)
  if (bar_thread) {
    grid_arrive(gctr);
    flag[1] = grid_wait(gctr, bar_base + 2ull * grid) ? 1 : 0;
  }
  consumers_sync();
  if (!flag[1] || !ok) {
    if (tid == 0) atomicExch(L.status, ok ? 5 : 3);
    return;
  }

  // ---- phase 4: quantise h (all rows, from L2), down rows of this CTA, combine in place ----
  const XTile hq = tb.hq;
  quantize_h_rows(hq, tb.n_hrows, L.hbuf, FF, warp, lane);
  consumers_sync();
  const int lpf = next_pow2_cap32(L.nbf);
  const int rounds = (T + kDownTiles - 1) / kDownTiles;
  for (int rd = 0; rd < rounds && ok; ++rd) {
    const int j0 = rd * kDownTiles, j1 = min(T, j0 + kDownTiles);
    if (rd == 0 && has_shared && !mbar_wait(shdn_full, 0)) ok = false;
    if (ok && !mbar_wait(dn_full, rd & 1)) ok = false;
    if (!ok) break;
    const int tasks = (j1 - j0) * nr * lpf;
#pragma unroll 1
    for (int base = 0; base < tasks; base += kConsumers) {
      const int q = base + tid;
      const int lr = q & (lpf - 1);
      const int jr = q / lpf;
      const int js = jr / max(nr, 1), r = jr - js * nr;
      const int tile = min(j0 + js, T - 1);
      const bool live = q < tasks && tb.tile_mode[tile] != 1;
      const int hrow0 = tb.tile_hrow0[tile];
      const RowSet rs = rows_of(live ? tb.tile_mask[tile] : 0, hrow0, false);   // h rows are stored per tile
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live) {
        const unsigned char* row = dn + static_cast<size_t>(js) * G.slot_bytes + static_cast<size_t>(r) * G.rb_f;
#pragma unroll 1
        for (int blk = lr; blk < L.nbf; blk += lpf) {
          const float4 v = block_dot_rows(reinterpret_cast<const uint4*>(row + blk * kW4), &tb.hq, blk, rs);
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
      }
      const float av[kMaxTok] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
      for (int t = 0; t < kMaxTok; ++t) {
        const float y = reduce_lanes(av[t], lpf);
        if (live && lr == 0 && t < rs.n) ysm[(hrow0 + t) * G.nr_max + r] = y;
      }
    }
    __syncwarp();
    if (lane == 0 && rd + 1 < rounds) mbar_arrive_one(dn_empty);
  }
  if (!consumers_all(ok)) {
    if (tid == 0) atomicExch(L.status, 3);
    return;
  }
  for (int i = tid; i < n * nr; i += kConsumers) {
    const int t = i / nr, rr = i - t * nr;
    const size_t o = static_cast<size_t>(t) * H + r0 + rr;
    float acc = (L.add_residual && L.x_f16 != nullptr) ? h2f(L.x_f16[o]) : 0.f;
    for (int kk = 0; kk <= K; ++kk) {
      const int hr = tb.route_hrow[t][kk];
      if (hr >= 0) acc += tb.sel_w[t][kk] * ysm[hr * G.nr_max + rr];
    }
    if (L.out_f32 != nullptr) L.out_f32[o] = acc;
    if (L.x_f16 != nullptr && L.add_residual) L.x_f16[o] = f2h(acc);
  }
}

}  // namespace tk
