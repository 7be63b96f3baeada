// expert_rows.cuh - the expert kernel for layers with many token rows (part of
// moe_layer.cu, which defines LayerDev and the plan before including this file).
//
// A persistent kernel, one CTA per SM, 16 consumer warps and 4 producer warps.
// Work is cut into groups: 128 (gate, up) row pairs of one tile (up to 16 token
// rows of one expert), or 256 rows of its down matrix. A group is streamed through
// a ring of shared-memory stages one super-block column at a time: a stage holds
// the 144-byte blocks of the group's 256 weight rows for one block index, plus
// that block of the tile's activation rows, re-laid for the dot engine. Every
// consumer warp owns sixteen of the rows for the whole group - eight gate rows
// and the eight up rows of the same indices, so SwiGLU needs no exchange - and
// keeps its sums in registers from the first column to the last: no partial sums
// in shared memory, no barrier between the warps; the only synchronisation is
// the full/empty mbarrier pair of each stage.
//
// Four weight warps fill a stage with 16-byte asynchronous copies (cp.async; a
// 144-byte piece per row is too small for a bulk copy to pay: one warp issues
// roughly one bulk copy per 60 cycles). A fifth producer warp copies the stage's
// block of the tile's activation rows, also asynchronously. The two roles walk
// the same list of stages independently, so the weight stream never waits for
// an activation row that is not ready yet.
//
// Gate/up groups write fp32 h. The last warp of a CTA to finish a group counts
// the CTA in at the group's 256-wide block of h (global counter); the CTA that
// completes the block quantises it for the tile's rows to Q8_K (padded 288-byte
// blocks, 16-byte copyable) and publishes it; the activation warp waits
// (bounded) for a tile's blocks before it copies them for a down group.
// Down groups write fp32 y; after a grid-wide barrier the CTAs add
// residual + sum_k w_k * y_k + shared expert (combine_rows).
#pragma once

#ifndef SGR_RS_PREFETCH
#define SGR_RS_PREFETCH 0
#endif

namespace rs {

constexpr int kTok = 16;                        // token rows per tile
constexpr int kConsumerWarps = 16;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kWeightWarps = 4;
constexpr int kWeightThreads = kWeightWarps * 32;
constexpr int kThreads = kConsumers + kWeightThreads + 64;      // + the activation warp and the finisher warp
constexpr int kStageCount = 5;
constexpr int kHalfRows = 128;                  // a stage is two halves of 128 rows
constexpr int kHalfBytes = kHalfRows * kW4;     // 18432
constexpr int kWBytes = 2 * kHalfBytes;
// activation part of a stage: codes [16][272] | int16 sums [16][8] | scales [16] at 16-byte steps
constexpr int kXCodes = kTok * kXqStride;
constexpr int kXBytes = kXCodes + kTok * 16 + kTok * 16;
constexpr int kStageBytes = (kWBytes + kXBytes + 127) & ~127;
constexpr int kPieces = kHalfBytes / 16 / kWeightThreads;       // 16-byte copies per thread and half: 9
constexpr int kHq = 288;                        // padded Q8_K block of h: d | 12 bytes | 256 codes | 8 sums
constexpr int kHdr = 1024;
constexpr size_t kSmem = kHdr + static_cast<size_t>(kStageCount) * kStageBytes;
constexpr int kGateUpPairs = 128;               // pairs per gate/up group
constexpr int kDownRows = 256;                  // rows per down group
constexpr int kCombineRows = 64;
constexpr int kFullArrivals = 2 * (kWeightThreads + 32);        // per producer thread: copies landed + plain stores done

static_assert(kPieces * kWeightThreads * 16 == kHalfBytes, "pieces must tile a half stage");
static_assert(kSmem <= 227 * 1024, "ring exceeds shared memory");

struct Desc {
  int kind;      // 0 gate/up, 1 down
  int mode;      // 0 weights streamed, 1 expert absent
  int tile, ntok;
  int hrow0;     // first h / y row of the tile
  int row0;      // first pair (gate/up) or first row (down) of the group
  int blk, nb;   // block column of this stage, columns per group
  int e, seq;    // expert id; running number of the group inside this CTA
  int pad[2];
};

// A finished gate/up group, handed from the consumers to the finisher warp.
struct Done {
  int tile, hb, hrow0, ntok;     // ntok == 0: absent expert, nothing to count
};
constexpr int kDoneSlots = 8;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// arrive on `bar` once every cp.async this thread has issued so far has landed
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void rs_consumers_sync() {
  asm volatile("bar.sync 5, %0;" ::"n"(kConsumers) : "memory");
}

// 16 bytes from a source that is only 2- or 4-byte aligned
__device__ __forceinline__ void copy16_any(unsigned char* dst, const unsigned char* src) {
  uint32_t v[4];
  if ((reinterpret_cast<uintptr_t>(src) & 3u) == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __ldg(reinterpret_cast<const uint32_t*>(src) + i);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint16_t* h = reinterpret_cast<const uint16_t*>(src) + 2 * i;
      v[i] = static_cast<uint32_t>(__ldg(h)) | (static_cast<uint32_t>(__ldg(h + 1)) << 16);
    }
  }
  *reinterpret_cast<uint4*>(dst) = make_uint4(v[0], v[1], v[2], v[3]);
}

// The list of stages of one CTA, walked identically by every role: gate/up groups
// [gu_lo, gu_lo + gu_cnt) with nbh columns each, then down groups with nbf columns.
struct Walk {
  int kind, gid, blk, nb, gpt, tile, gi, seq;
  int gu_end, dn_lo, nbf, gpt_dn;
  __device__ __forceinline__ void start(int gu_lo, int gu_cnt, int dn_lo_, int nbh, int nbf_, int gpt_gu, int gpt_dn_) {
    gu_end = gu_lo + gu_cnt; dn_lo = dn_lo_; nbf = nbf_; gpt_dn = gpt_dn_;
    seq = 0; blk = 0;
    if (gu_cnt > 0) { kind = 0; gid = gu_lo; nb = nbh; gpt = gpt_gu; }
    else { kind = 1; gid = dn_lo; nb = nbf; gpt = gpt_dn; }
    tile = gid / gpt; gi = gid - tile * gpt;
  }
  __device__ __forceinline__ void next() {
    if (++blk < nb) return;
    blk = 0; ++gid; ++seq;
    if (kind == 0 && gid == gu_end) { kind = 1; gid = dn_lo; nb = nbf; gpt = gpt_dn; }
    tile = gid / gpt; gi = gid - tile * gpt;
  }
};

// One warp: Q8_K-quantise block `hb` of the fp32 h rows [hrow0, hrow0 + ntok) into the
// padded rows of L.hq (arithmetic of src/kernels/cpu/q4_avx2.cpp:77-94 in the reference,
// the same as stage_quantized_f32). Two rows per pass keep two sets of loads in flight.
__device__ __forceinline__ void quantize_h_block(const LayerDev& L, int hrow0, int ntok, int hb, int lane) {
  const size_t hq_stride = static_cast<size_t>(L.nbf) * kHq;
  for (int t0 = 0; t0 < ntok; t0 += 2) {
    float4 a[2], b[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int t = min(t0 + u, ntok - 1);
      const float4* p = reinterpret_cast<const float4*>(L.hbuf + static_cast<size_t>(hrow0 + t) * L.FF + hb * kQK) + lane * 2;
      a[u] = __ldcg(p);
      b[u] = __ldcg(p + 1);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int t = t0 + u;
      if (t >= ntok) break;                      // warp-uniform
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
      const int sum_next = __shfl_down_sync(0xFFFFFFFFu, sum, 4);
      uint32_t* o32 = reinterpret_cast<uint32_t*>(L.hq + static_cast<size_t>(hrow0 + t) * hq_stride + hb * kHq);
      if (lane == 0) o32[0] = __float_as_uint(d);
      *reinterpret_cast<uint2*>(o32 + 4 + 2 * lane) =
          make_uint2((q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | (static_cast<uint32_t>(q[3] & 0xFF) << 24),
                     (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | (static_cast<uint32_t>(q[7] & 0xFF) << 24));
      if ((lane & 7) == 0)
        o32[68 + (lane >> 3)] = (static_cast<uint32_t>(sum) & 0xFFFFu) | (static_cast<uint32_t>(sum_next) << 16);
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) expert_rows_kernel(const LayerDev L) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = reinterpret_cast<uint64_t*>(smem + 64);
  int* flag = reinterpret_cast<int*>(smem + 128);
  unsigned* grp_cnt = reinterpret_cast<unsigned*>(smem + 256);      // [8] consumer warps done with a group
  Desc* desc = reinterpret_cast<Desc*>(smem + 384);
  Done* done_q = reinterpret_cast<Done*>(smem + 640);               // [kDoneSlots]
  volatile unsigned* done_tail = reinterpret_cast<volatile unsigned*>(smem + 136);   // groups handed over
  volatile unsigned* done_head = reinterpret_cast<volatile unsigned*>(smem + 140);   // groups taken by the finisher
  unsigned char* stages = smem + kHdr;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kStageCount; ++s) {
      mbar_init(&full[s], kFullArrivals);
      mbar_init(&empty[s], kConsumerWarps);
    }
    for (int i = 0; i < 8; ++i) grp_cnt[i] = 0u;
    *done_tail = 0u;
    *done_head = 0u;
    fence_barrier_init();
  }
  __syncthreads();
  pdl_wait();                       // plan, routing and quantised rows come from the route kernel
  pdl_launch_dependents();

  const int gpt_gu = L.FF / kGateUpPairs, gpt_dn = L.H / kDownRows;      // groups per tile
  // this CTA's run of gate/up groups and of down groups: equal-cost cuts made by the plan
  const int gu_lo = L.cta_lo[blockIdx.x], gu_cnt = L.cta_lo[blockIdx.x + 1] - gu_lo;
  const int dn_lo = L.cta_lo[kMaxGrid + 1 + blockIdx.x], dn_cnt = L.cta_lo[kMaxGrid + 2 + blockIdx.x] - dn_lo;
  const int n_stage = gu_cnt * L.nbh + dn_cnt * L.nbf;
  const int rb_h = L.nbh * kW4, rb_f = L.nbf * kW4;
  Walk wk;
  wk.start(gu_lo, gu_cnt, dn_lo, L.nbh, L.nbf, gpt_gu, gpt_dn);

  if (warp >= kConsumerWarps && warp < kConsumerWarps + kWeightWarps) {
    // ---------------- weight warps ----------------
    const int ptid = tid - kConsumers;
    int so_h[kPieces], so_f[kPieces];           // source offsets of this thread's pieces, per row pitch
#pragma unroll
    for (int j = 0; j < kPieces; ++j) {
      const int p = ptid + kWeightThreads * j;
      const int r = p / 9, c = (p - r * 9) * 16;
      so_h[j] = r * rb_h + c;
      so_f[j] = r * rb_f + c;
    }
    int cur_tile = -1, cur_gid = -1;
    const unsigned char *w0 = nullptr, *w1 = nullptr, *w2 = nullptr;
    bool absent = false, aligned = true;
    for (int q = 0; q < n_stage; ++q, wk.next()) {
      const int s = q % kStageCount;
      const unsigned ph = (q / kStageCount) & 1;
      if (wk.tile != cur_tile) {
        cur_tile = wk.tile;
        const int e = __ldcg(&L.rec[wk.tile].x);
        const bool shared = e == L.E;
        w0 = shared ? L.sh[0] : L.tab[e];
        w1 = shared ? L.sh[1] : L.tab[L.E + e];
        w2 = shared ? L.sh[2] : L.tab[2 * L.E + e];
        absent = w0 == nullptr || w1 == nullptr || w2 == nullptr;
        aligned = ((reinterpret_cast<uintptr_t>(w0) | reinterpret_cast<uintptr_t>(w1) |
                    reinterpret_cast<uintptr_t>(w2)) & 15u) == 0;
      }
      if (SGR_RS_PREFETCH != 0 && wk.gid != cur_gid && !absent && aligned) {
        // announce the group to L2 as long sequential reads
        if (wk.kind == 0) {
          const int bytes = kGateUpPairs * rb_h;
          const size_t at = static_cast<size_t>(wk.gi) * bytes;
          for (int o = ptid * 8192; o < 2 * bytes; o += kWeightThreads * 8192) {
            const int m = o >= bytes ? 1 : 0, oo = o - m * bytes;
            bulk_prefetch_l2((m ? w1 : w0) + at + oo, static_cast<uint32_t>(min(8192, bytes - oo)));
          }
        } else {
          const int bytes = kDownRows * rb_f;
          const size_t at = static_cast<size_t>(wk.gi) * bytes;
          for (int o = ptid * 8192; o < bytes; o += kWeightThreads * 8192)
            bulk_prefetch_l2(w2 + at + o, static_cast<uint32_t>(min(8192, bytes - o)));
        }
      }
      cur_gid = wk.gid;
      if (!mbar_wait(&empty[s], ph ^ 1u)) {
        if (lane == 0) atomicExch(L.status, 2);
        return;
      }
      if (!absent) {
        unsigned char* dst = stages + static_cast<size_t>(s) * kStageBytes + ptid * 16;
        const unsigned char *b0, *b1;
        if (wk.kind == 0) {
          b0 = w0 + static_cast<size_t>(wk.gi) * kGateUpPairs * rb_h + wk.blk * kW4;
          b1 = w1 + static_cast<size_t>(wk.gi) * kGateUpPairs * rb_h + wk.blk * kW4;
        } else {
          b0 = w2 + static_cast<size_t>(wk.gi) * kDownRows * rb_f + wk.blk * kW4;
          b1 = b0 + static_cast<size_t>(kHalfRows) * rb_f;
        }
        if (aligned) {
#pragma unroll
          for (int j = 0; j < kPieces; ++j) {
            const int so = wk.kind == 0 ? so_h[j] : so_f[j];
            cp_async16(dst + j * (kWeightThreads * 16), b0 + so);
            cp_async16(dst + j * (kWeightThreads * 16) + kHalfBytes, b1 + so);
          }
        } else {
#pragma unroll
          for (int j = 0; j < kPieces; ++j) {
            const int so = wk.kind == 0 ? so_h[j] : so_f[j];
            copy16_any(dst + j * (kWeightThreads * 16), b0 + so);
            copy16_any(dst + j * (kWeightThreads * 16) + kHalfBytes, b1 + so);
          }
        }
      }
      cp_async_arrive(&full[s]);
      mbar_arrive(&full[s]);
#ifdef SGR_PROFILE
      if (ptid == 0 && q < 120) {
        long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        (L.prof + 1024 * 16 + blockIdx.x * 512)[7 + 4 * q] = t;
      }
#endif
    }
    return;
  }

  if (warp == kConsumerWarps + kWeightWarps) {
    // ---------------- activation warp ----------------
    int cur_tile = -1, cur_kind = -1;
    int4 rc = make_int4(0, 0, 0, 0);
    bool absent = false;
    int myoff = 0;                              // lane t < 16: byte offset of token slot t's row
    for (int q = 0; q < n_stage; ++q, wk.next()) {
      const int s = q % kStageCount;
      const unsigned ph = (q / kStageCount) & 1;
      if (wk.tile != cur_tile || wk.kind != cur_kind) {
        if (wk.tile != cur_tile) {
          rc = __ldcg(L.rec + wk.tile);
          const bool shared = rc.x == L.E;
          const unsigned char* a0 = shared ? L.sh[0] : L.tab[rc.x];
          const unsigned char* a1 = shared ? L.sh[1] : L.tab[L.E + rc.x];
          const unsigned char* a2 = shared ? L.sh[2] : L.tab[2 * L.E + rc.x];
          absent = a0 == nullptr || a1 == nullptr || a2 == nullptr;
        }
        cur_tile = wk.tile;
        cur_kind = wk.kind;
        myoff = 0;
        if (wk.kind == 0) {
          if (lane < rc.y) {
            const int r = rc.x == L.E ? rc.w + lane : __ldcg(L.grows + rc.w + lane);
            myoff = r * L.nbh * kHq;
          }
        } else {
          if (lane < rc.y) myoff = (rc.z + lane) * L.nbf * kHq;
          if (!absent) {                        // the tile's h must be quantised and published
            unsigned it = 0;
            if (lane == 0)
              while (ld_acquire(L.ready + wk.tile) < static_cast<unsigned>(L.nbf) && ++it < kSpinLimit) __nanosleep(64);
            it = __shfl_sync(0xFFFFFFFFu, it, 0);
            if (it >= kSpinLimit) {
              if (lane == 0) atomicExch(L.status, 4);
              return;
            }
          }
        }
      }
      if (!mbar_wait(&empty[s], ph ^ 1u)) {
        if (lane == 0) atomicExch(L.status, 2);
        return;
      }
      unsigned char* xs = stages + static_cast<size_t>(s) * kStageBytes + kWBytes;
      if (!absent) {
        // 288-byte blocks (quantised inputs for gate/up, quantised h for down): 16-byte copies
        const unsigned char* xsrc = (wk.kind == 0 ? L.xq16 : L.hq) + wk.blk * kHq;
        const int total = rc.y * (kHq / 16);
        for (int base = 0; base < total; base += 32) {
          const int i = base + lane;
          const bool valid = i < total;
          const int t = valid ? i / (kHq / 16) : 0;
          const int c = i - t * (kHq / 16);
          const int off = __shfl_sync(0xFFFFFFFFu, myoff, t);
          if (valid) {
            unsigned char* dst = c == 0 ? xs + kXCodes + kTok * 16 + t * 16
                                        : (c <= 16 ? xs + t * kXqStride + (c - 1) * 16 : xs + kXCodes + t * 16);
            cp_async16(dst, xsrc + off + c * 16);
          }
        }
      }
      if (lane == 0) {
        Desc d;
        d.kind = wk.kind; d.mode = absent ? 1 : 0; d.tile = wk.tile; d.ntok = rc.y; d.hrow0 = rc.z;
        d.row0 = wk.gi * (wk.kind == 0 ? kGateUpPairs : kDownRows); d.blk = wk.blk; d.nb = wk.nb;
        d.e = rc.x; d.seq = wk.seq; d.pad[0] = d.pad[1] = 0;
        desc[s] = d;
      }
      cp_async_arrive(&full[s]);
      mbar_arrive(&full[s]);
    }
    return;
  }

  if (warp == kConsumerWarps + kWeightWarps + 1) {
    // ---------------- finisher warp ----------------
    // Takes the finished gate/up groups of this CTA in order: counts the CTA in at the
    // group's block of h, and if that completes the block, quantises it for the tile's
    // rows and publishes it. The consumers never wait for any of this.
    for (int g = 0; g < gu_cnt; ++g) {
      unsigned it = 0;
      if (lane == 0)
        while (*done_tail <= static_cast<unsigned>(g) && ++it < kSpinLimit) __nanosleep(100);
      it = __shfl_sync(0xFFFFFFFFu, it, 0);
      if (it >= kSpinLimit) {
        if (lane == 0) atomicExch(L.status, 6);
        return;
      }
      __threadfence_block();
      const Done r = done_q[g % kDoneSlots];
      __syncwarp();
      if (lane == 0) *done_head = static_cast<unsigned>(g) + 1u;     // the slot may be reused
      if (r.ntok == 0) continue;
      __threadfence();                         // cumulative: covers what the sixteen warps stored
      unsigned old = 0;
      if (lane == 0) old = atomicAdd(L.blk_cnt + r.tile * L.nbf + r.hb, 1u);
      old = __shfl_sync(0xFFFFFFFFu, old, 0);
      if (old == kQK / kGateUpPairs - 1) {
        __threadfence();
        quantize_h_block(L, r.hrow0, r.ntok, r.hb, lane);
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(L.ready + r.tile, 1u);
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  float acc[2][4];
  bool ok = true;
#ifdef SGR_PROFILE
  const int _pw = 0;
  long long* trace = L.prof + 1024 * 16 + blockIdx.x * 512;
  auto gtime = []() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
  if (tid == 0) { trace[0] = gtime(); trace[1] = n_stage; }
#endif
  PROF_T0();
  for (int q = 0; q < n_stage; ++q) {
    const int s = q % kStageCount;
    const unsigned ph = (q / kStageCount) & 1;
    PROF_ADD(2);
    if (!mbar_wait(&full[s], ph)) {
      if (lane == 0) atomicExch(L.status, 3);
      ok = false;
      break;
    }
    PROF_ADD(0);
    const Desc d = desc[s];
#ifdef SGR_PROFILE
    if (tid == 0 && q < 120) { trace[4 + 4 * q] = gtime(); trace[6 + 4 * q] = d.kind * 1000 + d.ntok * 10 + (d.blk == 0 ? 1 : 0); }
#endif
    unsigned char* st = stages + static_cast<size_t>(s) * kStageBytes;
    if (d.blk == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[0][j] = acc[1][j] = 0.f;
    }
#ifdef SGR_RS_NOCOMPUTE
    if (false) {
#else
    if (d.mode == 0) {
#endif
      XTile xt;
      xt.qs = reinterpret_cast<int8_t*>(st + kWBytes);
      xt.bs = reinterpret_cast<int16_t*>(st + kWBytes + kXCodes);
      xt.bl = nullptr;
      xt.d = reinterpret_cast<float*>(st + kWBytes + kXCodes + kTok * 16);
      xt.nb = 1;
      xt.tok_stride = kXqStride;
      xt.d_step = 4;
      // unit row u of this warp -> byte offset of its block in the stage
      auto row_at = [&](int u) {
        return d.kind == 0 ? ((u & 7) + 8 * warp) * kW4 + (u >> 3) * kHalfBytes : (16 * warp + u) * kW4;
      };
      if (d.ntok <= 2) {
        float a2[2] = {acc[0][0], acc[0][1]};
        half_block_dot<2>(reinterpret_cast<const uint4*>(st + row_at(lane >> 1)), lane & 1, xt, d.ntok, a2);
        acc[0][0] = a2[0];
        acc[0][1] = a2[1];
      } else {
        const unsigned char* a_ptr = st + row_at((lane & 7) + ((lane >> 3) & 1) * 8) + 16 + (lane >> 4) * 16;
        const unsigned char* h_lo = st + row_at(lane >> 2);
        const unsigned char* h_hi = st + row_at((lane >> 2) + 8);
        if (d.ntok <= 8) warp_mma_block<1>(a_ptr, h_lo, h_hi, xt, reinterpret_cast<float(&)[1][4]>(acc));
        else warp_mma_block<2>(a_ptr, h_lo, h_hi, xt, acc);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);       // this warp no longer reads the stage
#ifdef SGR_PROFILE
    if (tid == 0 && q < 120) trace[5 + 4 * q] = gtime();
    if (lane == 0 && warp == 0) {
      const int cls = d.ntok <= 2 ? 0 : (d.ntok <= 8 ? 1 : 2);
      atomicAdd(reinterpret_cast<unsigned long long*>(L.prof + blockIdx.x * 16 + 8 + cls), static_cast<unsigned long long>(clock64() - _pt));
      atomicAdd(reinterpret_cast<unsigned long long*>(L.prof + blockIdx.x * 16 + 11 + cls), 1ull);
    }
#endif
    PROF_ADD(1);
    if (d.blk != d.nb - 1) continue;

    // ---- the group is complete for this warp's rows ----
    const int gid = lane >> 2, tig = lane & 3;
    if (d.kind == 0) {
      if (d.mode == 1) {
        if (d.row0 == 0 && warp == 0 && lane == 0 && L.mail != nullptr && d.e != L.E) {
          const int mi = atomicAdd(L.mail_n, 1);
          if (mi < L.E) L.mail[mi] = d.e;
        }
      } else
      if (d.ntok <= 2) {
        const float u0 = __shfl_down_sync(0xFFFFFFFFu, acc[0][0], 16);
        const float u1 = __shfl_down_sync(0xFFFFFFFFu, acc[0][1], 16);
        if (lane < 16 && (lane & 1) == 0) {
          const int col = d.row0 + 8 * warp + (lane >> 1);
          const float g0 = acc[0][0], g1 = acc[0][1];
          L.hbuf[static_cast<size_t>(d.hrow0) * L.FF + col] = g0 / (1.f + expf(-g0)) * u0;
          if (d.ntok > 1) L.hbuf[static_cast<size_t>(d.hrow0 + 1) * L.FF + col] = g1 / (1.f + expf(-g1)) * u1;
        }
      } else {
        const int col = d.row0 + 8 * warp + gid;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const int t0 = 8 * n + 2 * tig;
          if (t0 < d.ntok) {
            const float g = acc[n][0], u = acc[n][2];
            L.hbuf[static_cast<size_t>(d.hrow0 + t0) * L.FF + col] = g / (1.f + expf(-g)) * u;
          }
          if (t0 + 1 < d.ntok) {
            const float g = acc[n][1], u = acc[n][3];
            L.hbuf[static_cast<size_t>(d.hrow0 + t0 + 1) * L.FF + col] = g / (1.f + expf(-g)) * u;
          }
        }
      }
      PROF_ADD(5);
      // Count the warp in at the CTA's counter of this group (shared memory); the last
      // warp hands the group to the finisher warp. Groups finish in order: a warp is at
      // most a ring's depth of stages ahead of the slowest one.
      __threadfence_block();
      __syncwarp();
      if (lane == 0) {
        if (atomicAdd(&grp_cnt[d.seq & 7], 1u) == kConsumerWarps - 1) {
          grp_cnt[d.seq & 7] = 0u;
          unsigned it = 0;                       // queue full: wait (bounded) for the finisher
          while (static_cast<unsigned>(d.seq) - *done_head >= static_cast<unsigned>(kDoneSlots) && ++it < kSpinLimit)
            __nanosleep(100);
          if (it >= kSpinLimit) atomicExch(L.status, 6);
          Done r;
          r.tile = d.tile; r.hb = d.row0 / kQK; r.hrow0 = d.hrow0; r.ntok = d.mode == 1 ? 0 : d.ntok;
          done_q[d.seq % kDoneSlots] = r;
          __threadfence_block();
          *done_tail = static_cast<unsigned>(d.seq) + 1u;
        }
      }
      PROF_ADD(6);
      PROF_ADD(7);
    } else {
      if (d.mode == 1) {
        for (int j = lane; j < 16 * d.ntok; j += 32)
          L.ybuf[static_cast<size_t>(d.hrow0 + j / 16) * L.H + d.row0 + 16 * warp + (j & 15)] = 0.f;
        continue;
      }
      if (d.ntok <= 2) {
        if ((lane & 1) == 0) {
          const int col = d.row0 + 16 * warp + (lane >> 1);
          L.ybuf[static_cast<size_t>(d.hrow0) * L.H + col] = acc[0][0];
          if (d.ntok > 1) L.ybuf[static_cast<size_t>(d.hrow0 + 1) * L.H + col] = acc[0][1];
        }
      } else {
        const int col = d.row0 + 16 * warp + gid;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const int t0 = 8 * n + 2 * tig;
          if (t0 < d.ntok) {
            L.ybuf[static_cast<size_t>(d.hrow0 + t0) * L.H + col] = acc[n][0];
            L.ybuf[static_cast<size_t>(d.hrow0 + t0) * L.H + col + 8] = acc[n][2];
          }
          if (t0 + 1 < d.ntok) {
            L.ybuf[static_cast<size_t>(d.hrow0 + t0 + 1) * L.H + col] = acc[n][1];
            L.ybuf[static_cast<size_t>(d.hrow0 + t0 + 1) * L.H + col + 8] = acc[n][3];
          }
        }
      }
      PROF_ADD(14);
    }
  }

  // ---- all y rows written everywhere: blend ------------------------------------------------
  PROF_ADD(2);
  __threadfence();
  rs_consumers_sync();
  if (tid == 0) {
    atomicAdd(&L.cnt[9], 1u);
    unsigned it = 0;
    while (ld_acquire(&L.cnt[9]) < gridDim.x && ++it < kSpinLimit) __nanosleep(32);
    flag[0] = (it < kSpinLimit && ok) ? 1 : 0;
  }
  rs_consumers_sync();
  PROF_ADD(3);
#ifdef SGR_PROFILE
  if (tid == 0) trace[2] = gtime();
#endif
  if (!flag[0]) {
    if (tid == 0) atomicExch(L.status, 5);
    return;
  }
  const int tgroups = (L.n + 15) / 16;
  const int chunks = (L.H + kCombineRows - 1) / kCombineRows;
  for (int job = blockIdx.x; job < chunks * tgroups; job += gridDim.x) {
    const int c = job / tgroups, tg = job - c * tgroups;
    combine_rows(L, c * kCombineRows, min(kCombineRows, L.H - c * kCombineRows), tg * 16, min(L.n, tg * 16 + 16),
                 tid, kConsumers);
  }
  PROF_ADD(4);
#ifdef SGR_PROFILE
  if (tid == 0) trace[3] = gtime();
#endif
}

}  // namespace rs
