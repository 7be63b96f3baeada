// expert_rows.cuh - the expert kernel for layers with many token rows (part of
// moe_layer.cu, which defines LayerDev and the plan before including this file).
//
// A persistent kernel, one CTA per SM: 16 consumer warps, a weight warp, three
// activation warps and a finisher warp.
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
// The weight part of a stage arrives by TMA: two tiled copies per stage (boxes of
// 144 bytes x 128 rows) through 2-D tensor maps over [rows][row bytes]. The maps
// are made on the host for a placeholder address; the weight warp patches a group's
// descriptors while the group before it streams: the expert's base addresses go into shared-memory copies
// (tensormap.replace), publishes them to a per-CTA ring of descriptors in global
// memory (tensormap.cp_fenceproxy) and acquires them before use. (16-byte cp.async
// copies reach the same HBM rate on their own, but every one of them passes through
// the load/store pipe that the consumers' shared-memory loads need; bulk copies of
// 144 bytes are issue-bound at roughly one per 60 cycles and warp.) Three more
// producer warps copy the stage's block of the tile's activation rows with
// cp.async. The two roles walk the same list of stages independently, so the
// weight stream never waits for an activation row that is not ready yet. Experts
// whose pointers are not 16-byte aligned cannot go through TMA: the weight warp
// copies them with plain loads.
//
// Gate/up groups write fp32 h. The last warp of a CTA to finish a group counts
// the CTA in at the group's 256-wide block of h (global counter); the CTA that
// completes the block quantises it for the tile's rows to Q8_K (padded 288-byte
// blocks, 16-byte copyable) and publishes it; the activation warp waits
// (bounded) for a tile's blocks before it copies them for a down group.
// Down groups write fp32 y; after a grid-wide barrier the CTAs add
// residual + sum_k w_k * y_k + shared expert (combine_rows).
#pragma once

namespace rs {

constexpr int kTok = 16;                        // token rows per tile
constexpr int kConsumerWarps = 16;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kXWarps = 3;                      // activation-row producers
constexpr int kXThreads = kXWarps * 32;
constexpr int kThreads = kConsumers + 32 + kXThreads + 32;      // consumers, weight warp, activation warps, finisher warp
constexpr int kStageCount = 5;
constexpr int kHalfRows = 128;                  // a stage is two halves of 128 rows
constexpr int kHalfBytes = kHalfRows * kW4;     // 18432
constexpr int kWBytes = 2 * kHalfBytes;
// activation part of a stage: codes [16][272] | int16 sums [16][8] | scales [16] at 16-byte steps
constexpr int kXCodes = kTok * kXqStride;
constexpr int kXBytes = kXCodes + kTok * 16 + kTok * 16;
constexpr int kStageBytes = (kWBytes + kXBytes + 127) & ~127;
constexpr int kHq = 288;                        // padded Q8_K block of h: d | 12 bytes | 256 codes | 8 sums
constexpr int kHdr = 4096;
// The plan of a layer, built by every CTA for itself when the routing was made by this call's own
// route kernel: row masks [E] | offsets [E + 1] | scan scratch | tile records | rows of the slots | slot
// of every route. One round trip for the routing and a few barriers per CTA, all CTAs at once, instead
// of one CTA planning in global memory while 147 wait (8 us per layer at 64 rows).
constexpr int kPlanExperts = 256, kPlanRoutes = 512;
constexpr int kPlanTiles = kPlanExperts + kPlanRoutes / kTok + 8;     // a tile per expert, per further 16 rows, shared expert's
constexpr int kPlanOffMask = 0, kPlanOffOff = kPlanExperts * 8, kPlanOffScan = kPlanOffOff + 1152;
constexpr int kPlanOffRec = kPlanOffScan + 512, kPlanOffRows = kPlanOffRec + kPlanTiles * 16;
constexpr int kPlanOffSlot = kPlanOffRows + kPlanRoutes * 4;
constexpr int kPlanBytes = (kPlanOffSlot + kPlanRoutes * 4 + 127) & ~127;
constexpr size_t kSmem = kHdr + kPlanBytes + static_cast<size_t>(kStageCount) * kStageBytes;
constexpr int kGateUpPairs = 128;               // pairs per gate/up group
constexpr int kDownRows = 256;                  // rows per down group
constexpr int kFullArrivals = 1 + kXThreads;      // weight warp: one arrival; activation warps: a thread's copies landed
constexpr int kMapRing = kStageCount + 1;        // descriptor slots per CTA: a slot is patched again only after every
                                                 // stage that could still reference it has been refilled (a tile has at
                                                 // least one stage, and at most kStageCount stages are in flight)

static_assert(kSmem <= 227 * 1024, "ring exceeds shared memory");
static_assert(kMapRing <= kTmapSlots, "the workspace holds kTmapSlots descriptor sets per CTA");

struct Desc {     // one 16-byte shared-memory load per stage and warp
  int flags;     // bit 0 kind (0 gate/up, 1 down), bit 1 expert absent, bits 2-7 token rows,
                 // bits 8-15 block column, bit 16 last column of the group, bit 17 end of this CTA's list,
                 // bits 20-31 group number in this CTA
  int tile;
  int hrow0;     // first h / y row of the tile
  int row0;      // first pair (gate/up) or first row (down) of the group
  __device__ __forceinline__ int kind() const { return flags & 1; }
  __device__ __forceinline__ int absent() const { return (flags >> 1) & 1; }
  __device__ __forceinline__ int ntok() const { return (flags >> 2) & 63; }
  __device__ __forceinline__ int blk() const { return (flags >> 8) & 255; }
  __device__ __forceinline__ int last() const { return (flags >> 16) & 1; }
  __device__ __forceinline__ int end() const { return (flags >> 17) & 1; }     // no more stages for this CTA
  __device__ __forceinline__ int seq() const { return (flags >> 20) & 4095; }
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
__device__ __forceinline__ void tmap_replace_addr(void* smem_map, const void* gaddr) {
  asm volatile("tensormap.replace.tile.global_address.shared::cta.b1024.b64 [%0], %1;" ::"r"(smem_u32(smem_map)), "l"(gaddr) : "memory");
}
// whole warp: copy the patched 128-byte descriptor to global memory for the TMA unit
__device__ __forceinline__ void tmap_publish(void* gmem_map, void* smem_map) {
  asm volatile("tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;"
               ::"l"(gmem_map), "r"(smem_u32(smem_map)) : "memory");
}
__device__ __forceinline__ void tmap_acquire(const void* gmem_map) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(gmem_map) : "memory");
}
// box (144 bytes x 128 rows) at byte column x, row y; dst 128-byte aligned, x a multiple of 16
__device__ __forceinline__ void tma_load_box(void* dst, const void* gmem_map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(dst)), "l"(gmem_map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
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

// Groups are handed out dynamically, in one global order: every gate/up group of the
// layer (tile-major), then every down group. A CTA starts with group blockIdx.x and takes
// further ones from a global counter; its weight warp draws the next number while it
// streams the current group and publishes the CTA's list in shared memory for the other
// roles. Equal finishing times need no cost model this way, and a tile's down groups are
// drawn long after its gate/up groups were (the whole gate/up list lies between).
struct Group {
  int kind, tile, gi, nb;        // 0 gate/up / 1 down, tile, group inside the tile, block columns
  bool valid;
};
struct Sched {
  int n_gu, total, nbh, nbf, gpt_gu, gpt_dn;
  __device__ __forceinline__ Group decode(int g) const {
    Group r;
    r.valid = g >= 0 && g < total;
    r.kind = g >= n_gu ? 1 : 0;
    const int local = r.kind ? g - n_gu : g;
    const int gpt = r.kind ? gpt_dn : gpt_gu;
    r.tile = r.valid ? local / gpt : 0;
    r.gi = local - r.tile * gpt;
    r.nb = r.kind ? nbf : nbh;
    return r;
  }
};
constexpr int kListSlots = 16;

// One entry of a CTA's group list, published by the weight warp one group ahead of its copies,
// with everything the other roles would otherwise fetch from global memory again.
struct GEntry {
  int id;          // global group number, -1 = end of this CTA's list
  int absent;      // bit 0: the expert's pointers are null; bit 1 (down groups): the tile's h was already published
                   // when the weight warp looked
  int4 rc;         // the tile's record: expert, token rows, first h / y row, first entry of grows
  int rows[kTok];  // gate/up groups: source row of the tile's token slot t in the quantised inputs
};
static_assert(sizeof(GEntry) * kListSlots + 2048 <= kHdr, "group list exceeds the header");

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

// Every thread of the CTA: the plan of build_plan (moe_layer.cu) in shared memory - same masks, same
// tile order (shared expert's tiles, tiles of more than half a tile's rows, the rest, each in expert
// order), same slots. CTA 0 also silences rows with ids outside [0, E) as moe_dispatch_scan does
// (moe.cu:385-398 of the reference) and leaves the counts in meta. Returns the number of tiles.
__device__ __forceinline__ int build_plan_shared(const LayerDev& L, unsigned char* ps, int tid) {
  unsigned long long* mask = reinterpret_cast<unsigned long long*>(ps + kPlanOffMask);
  int* off_s = reinterpret_cast<int*>(ps + kPlanOffOff);
  int* scan = reinterpret_cast<int*>(ps + kPlanOffScan);          // [3][40]: warp totals of rows, tiles, heavy tiles; [120]: bad ids
  int4* rec_s = reinterpret_cast<int4*>(ps + kPlanOffRec);
  int* rows_s = reinterpret_cast<int*>(ps + kPlanOffRows);
  int* slot_s = reinterpret_cast<int*>(ps + kPlanOffSlot);
  const int lane = tid & 31, wp = tid >> 5;
  const int total = L.n * L.K;
  // (the masks and the count of bad ids were cleared before the wait for the route kernel)
  int my_e = -1, my_r = 0;
  if (tid < total) {                            // kPlanRoutes <= kThreads: a route per thread
    my_r = tid / L.K;
    const int kk = tid - my_r * L.K;
    my_e = __ldcg(L.idx + static_cast<size_t>(my_r) * L.rstride + kk);
    if (my_e < 0 || my_e >= L.E) {
      if (blockIdx.x == 0) {
        for (int q = 0; q <= L.K; ++q) L.w[static_cast<size_t>(my_r) * L.rstride + q] = 0.f;
        atomicAdd(&scan[120], 1);
      }
      my_e = -1;
    } else if (my_e >= L.e_lo && my_e < L.e_hi) {
      atomicOr(&mask[my_e], 1ull << my_r);
    } else {
      my_e = -1;
    }
  }
  __syncthreads();
  auto is_heavy = [](int rows_in_tile) { return 2 * rows_in_tile > kTok; };
  int c = 0, t = 0, h = 0;
  if (tid < L.E) {
    c = __popcll(mask[tid]);
    t = (c + kTok - 1) / kTok;
    h = c / kTok + (is_heavy(c % kTok) ? 1 : 0);
  }
  int ic = c, it = t, ih = h;                   // inclusive scans inside the warps that hold experts
  if (tid < kPlanExperts) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int uc = __shfl_up_sync(0xFFFFFFFFu, ic, o), ut = __shfl_up_sync(0xFFFFFFFFu, it, o);
      const int uh = __shfl_up_sync(0xFFFFFFFFu, ih, o);
      if (lane >= o) { ic += uc; it += ut; ih += uh; }
    }
    if (lane == 31) { scan[wp] = ic; scan[40 + wp] = it; scan[80 + wp] = ih; }
  }
  __syncthreads();
  int rows_total = 0, tiles_total = 0, heavy_total = 0, pc = 0, pt = 0, phv = 0;
#pragma unroll
  for (int w = 0; w < kPlanExperts / 32; ++w) {
    if (w < wp) { pc += scan[w]; pt += scan[40 + w]; phv += scan[80 + w]; }
    rows_total += scan[w]; tiles_total += scan[40 + w]; heavy_total += scan[80 + w];
  }
  const int sh_tiles = (L.sh[0] != nullptr && L.sh_hi > L.sh_lo) ? (L.sh_hi - L.sh_lo + kTok - 1) / kTok : 0;
  if (tid < L.E) {
    const int ar = pc + ic - c;                 // exclusive prefixes of this expert
    int at_heavy = sh_tiles + (phv + ih - h), at_light = sh_tiles + heavy_total + ((pt + it - t) - (phv + ih - h));
    off_s[tid] = ar;
    for (int t0 = 0; t0 < c; t0 += kTok) {
      const int ct = min(kTok, c - t0);
      const int at = is_heavy(ct) ? at_heavy++ : at_light++;
      rec_s[at] = make_int4(tid, ct, ar + t0, ar + t0);
    }
  }
  if (tid == 0) off_s[L.E] = rows_total;
  if (tid < sh_tiles) {
    const int t0 = tid * kTok;
    rec_s[tid] = make_int4(L.E, min(kTok, L.sh_hi - L.sh_lo - t0), L.n_max * L.K + L.sh_lo + t0, L.sh_lo + t0);
  }
  __syncthreads();
  if (tid < total) {
    int pos = -1;
    if (my_e >= 0) {
      pos = off_s[my_e] + __popcll(mask[my_e] & ((1ull << my_r) - 1ull));
      rows_s[pos] = my_r;
    }
    slot_s[tid] = pos;
  }
  if (blockIdx.x == 0 && tid == 0) {
    L.meta[0] = rows_total;
    L.meta[1] = tiles_total + sh_tiles;
    L.meta[2] = scan[120];
    L.meta[3] = sh_tiles;
  }
  __syncthreads();
  return tiles_total + sh_tiles;
}

__global__ void __launch_bounds__(kThreads, 1) expert_rows_kernel(const LayerDev L) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = reinterpret_cast<uint64_t*>(smem + 64);      // a stage's activation part may be refilled
  uint64_t* wempty = reinterpret_cast<uint64_t*>(smem + 192);    // a stage's weight part may be refilled
  int* flag = reinterpret_cast<int*>(smem + 128);
  unsigned* grp_cnt = reinterpret_cast<unsigned*>(smem + 256);      // [8] consumer warps done with a group
  Desc* desc = reinterpret_cast<Desc*>(smem + 384);
  Done* done_q = reinterpret_cast<Done*>(smem + 640);               // [kDoneSlots]
  volatile unsigned* done_tail = reinterpret_cast<volatile unsigned*>(smem + 136);   // groups handed over
  volatile unsigned* done_head = reinterpret_cast<volatile unsigned*>(smem + 140);   // groups taken by the finisher
  unsigned char* plan_s = smem + kHdr;
  unsigned char* stages = smem + kHdr + kPlanBytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kStageCount; ++s) {
      mbar_init(&full[s], kFullArrivals);
      mbar_init(&empty[s], kConsumerWarps);
      mbar_init(&wempty[s], kConsumerWarps);
    }
    for (int i = 0; i < 8; ++i) grp_cnt[i] = 0u;
    *done_tail = 0u;
    *done_head = 0u;
    *reinterpret_cast<volatile unsigned*>(smem + 144) = 0u;
    fence_barrier_init();
  }
  if (L.plan_in_kernel) {           // shared memory of the plan that must start out clear
    for (int e = tid; e < kPlanExperts; e += kThreads) reinterpret_cast<unsigned long long*>(plan_s + kPlanOffMask)[e] = 0ull;
    if (tid == 0) reinterpret_cast<int*>(plan_s + kPlanOffScan)[120] = 0;
  }
  __syncthreads();
  pdl_wait();                       // routing and quantised rows (and, without a plan of its own, the plan) come from the route kernel
  pdl_launch_dependents();

  Sched sc;
  sc.gpt_gu = L.FF / kGateUpPairs; sc.gpt_dn = L.H / kDownRows;      // groups per tile
  sc.nbh = L.nbh; sc.nbf = L.nbf;
  // the plan: this CTA's own copy in shared memory, or the one a plan kernel left in the workspace
  const bool plan_own = L.plan_in_kernel != 0;
  if (plan_own && L.wait_flags != nullptr) {
    // owner side of an expert-parallel layer: the routing is in the records the home ranks store into
    // this rank's memory; every CTA waits (bounded) for their arrival words. A word that never comes
    // raises the status; the CTA then goes on with the records of an earlier step (valid memory).
    if (tid < L.wait_count) {
      const unsigned want = *L.wait_step * L.wait_mul + L.wait_add;
      unsigned it = 0, v;
      do {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(L.wait_flags + tid) : "memory");
      } while (static_cast<int>(v - want) < 0 && ++it < L.wait_limit && (__nanosleep(64), true));
      if (static_cast<int>(v - want) < 0) atomicExch(L.status, 8);
    }
    __syncthreads();
  }
  const int n_tiles = plan_own ? build_plan_shared(L, plan_s, tid) : L.meta[1];
  const int4* rec_p = plan_own ? reinterpret_cast<const int4*>(plan_s + kPlanOffRec) : L.rec;
  const int* rows_p = plan_own ? reinterpret_cast<const int*>(plan_s + kPlanOffRows) : L.grows;
  const int* slot_p = plan_own ? reinterpret_cast<const int*>(plan_s + kPlanOffSlot) : L.gslot;
  auto tile_rec = [&](int tile) { return plan_own ? rec_p[tile] : __ldcg(rec_p + tile); };
  sc.n_gu = n_tiles * sc.gpt_gu;
  sc.total = sc.n_gu + n_tiles * sc.gpt_dn;
  const int rb_h = L.nbh * kW4, rb_f = L.nbf * kW4;
  GEntry* glist = reinterpret_cast<GEntry*>(smem + 2048);                       // [kListSlots] this CTA's groups
  volatile unsigned* g_pub = reinterpret_cast<volatile unsigned*>(smem + 144);  // entries of glist published
  // a follower role's k-th group (bounded wait for the weight warp to publish it); an entry stays
  // valid for kListSlots further groups, far longer than any role can lag behind the ring
  auto follow = [&](int k, bool& ok) -> const GEntry* {
    unsigned it = 0;
    if (lane == 0)
      while (*g_pub <= static_cast<unsigned>(k) && ++it < kSpinLimit) __nanosleep(40);
    it = __shfl_sync(0xFFFFFFFFu, it, 0);
    ok = it < kSpinLimit;
    __threadfence_block();
    return glist + k % kListSlots;
  };

  if (warp == kConsumerWarps) {
    // ---------------- weight warp ----------------
    // Streams group k while it prepares group k + 1: the tile's record is requested between two
    // copies of group k, the expert's pointers (and the token slots' source rows) after its last copy,
    // and the descriptors are patched once the group's copies are all issued - so these global round
    // trips and the descriptor update overlap the stream. A group's number is drawn as late as that
    // allows: a number drawn is a group that no other CTA can take, and a gate/up group that waits
    // long for its CTA delays its tile's h, on which eight down groups elsewhere depend. So the next
    // number is drawn four stages before the current group ends - or, when the group it follows is a
    // short down group, as soon as that one's number is known.
    unsigned char* smaps = smem + 1024;                                 // three 128-byte descriptors being patched
    uint32_t* tmpl = reinterpret_cast<uint32_t*>(smem + 1408);          // the two host-made descriptors
    unsigned char* gmaps = L.tmaps + static_cast<size_t>(blockIdx.x) * kMapRing * 3 * 128;
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {             // constant indices only (see LayerDev)
        tmpl[i] = L.tmap_gu[i];
        tmpl[32 + i] = L.tmap_dn[i];
      }
    }
    __syncwarp();
    struct Prep {
      Group g;
      int id;
      int4 rc;
      const unsigned char *w0, *w1, *w2;
      const unsigned char* maps;
      int row;            // this lane's entry of GEntry::rows
      bool absent, aligned;
      unsigned ready;     // down groups: quantised blocks of the tile's h published so far
    };
    int map_seq = 0;
    auto load_ptrs = [&](Prep& p) {
      const bool shared = p.rc.x == L.E;
      p.w0 = shared ? L.sh[0] : L.tab[p.rc.x];
      p.w1 = shared ? L.sh[1] : L.tab[L.tab_stride + p.rc.x];
      p.w2 = shared ? L.sh[2] : L.tab[2 * L.tab_stride + p.rc.x];
      p.row = 0;
      if (p.g.kind == 0 && lane < p.rc.y)
        p.row = shared ? p.rc.w + lane : (plan_own ? rows_p[p.rc.w + lane] : __ldcg(rows_p + p.rc.w + lane));
      // a down group's activation rows are the tile's quantised h: seen complete here (acquire), the
      // activation warps need not look again (they run after this warp's publication of the entry)
      p.ready = p.g.kind == 1 ? ld_acquire(L.ready + p.g.tile) : 0u;
    };
    // descriptors of the matrices this group reads (gate and up, or down), in the next slot of the
    // CTA's ring: the ring keeps the descriptors of earlier groups intact while their copies fly
    auto patch = [&](Prep& p) {
      p.absent = p.w0 == nullptr || p.w1 == nullptr || p.w2 == nullptr;
      p.aligned = ((reinterpret_cast<uintptr_t>(p.w0) | reinterpret_cast<uintptr_t>(p.w1) |
                    reinterpret_cast<uintptr_t>(p.w2)) & 15u) == 0;
      p.maps = nullptr;
      if (p.absent || !p.aligned) return;
      unsigned char* slot = gmaps + static_cast<size_t>(map_seq % kMapRing) * 3 * 128;
      ++map_seq;
      uint32_t* m = reinterpret_cast<uint32_t*>(smaps);
      if (p.g.kind == 0) {
        m[lane] = tmpl[lane];
        m[32 + lane] = tmpl[lane];
        __syncwarp();
        if (lane == 0) {
          tmap_replace_addr(smaps, p.w0);
          tmap_replace_addr(smaps + 128, p.w1);
        }
        __syncwarp();
        tmap_publish(slot, smaps);
        tmap_publish(slot + 128, smaps + 128);
        if (lane == 0) {
          tmap_acquire(slot);
          tmap_acquire(slot + 128);
        }
      } else {
        m[64 + lane] = tmpl[32 + lane];
        __syncwarp();
        if (lane == 0) tmap_replace_addr(smaps + 256, p.w2);
        __syncwarp();
        tmap_publish(slot + 256, smaps + 256);
        if (lane == 0) tmap_acquire(slot + 256);
      }
      __syncwarp();
      p.maps = slot;
    };
    auto publish = [&](int k, const Prep& p) {
      GEntry* e = glist + k % kListSlots;
      if (lane < kTok) e->rows[lane] = p.row;
      if (lane == 0) {
        e->id = p.g.valid ? p.id : -1;
        e->absent = (p.absent ? 1 : 0) | (p.ready >= static_cast<unsigned>(L.nbf) ? 2 : 0);
        e->rc = p.rc;
      }
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        *g_pub = static_cast<unsigned>(k) + 1u;
      }
    };
    Prep cur;
    cur.id = blockIdx.x;                        // the first group is this CTA's own number
    cur.g = sc.decode(cur.id);
    cur.rc = make_int4(0, 0, 0, 0);
    cur.w0 = cur.w1 = cur.w2 = nullptr;
    cur.maps = nullptr;
    cur.row = 0;
    cur.absent = false;
    cur.aligned = true;
    cur.ready = 0u;
    int drawn = 0;                               // lane 0: the number last drawn
    bool id_ready = false;                       // ... which is that of the next group, not yet looked at
    if (cur.g.valid) {
      cur.rc = tile_rec(cur.g.tile);
      load_ptrs(cur);
      patch(cur);
    }
    publish(0, cur);
    int q = 0;
    for (int k = 0;; ++k) {
      const Group wk = cur.g;
      if (!wk.valid) {                           // end of the list: one last stage that only says so
        const int s = q % kStageCount;
        const unsigned ph = (q / kStageCount) & 1;
        if (!mbar_wait(&wempty[s], ph ^ 1u)) {
          if (lane == 0) atomicExch(L.status, 2);
          return;
        }
        if (lane == 0) {
          Desc d;
          d.flags = 1 << 17; d.tile = 0; d.hrow0 = 0; d.row0 = 0;
          desc[s] = d;
          mbar_arrive(&full[s]);
        }
        return;
      }
      Prep nx;
      nx.id = -1;
      nx.g = sc.decode(-1);
      nx.rc = make_int4(0, 0, 0, 0);
      nx.w0 = nx.w1 = nx.w2 = nullptr;
      nx.maps = nullptr;
      nx.row = 0;
      nx.absent = false;
      nx.aligned = true;
      nx.ready = 0u;
      const int draw_at = id_ready ? -1 : max(0, wk.nb - 4);                   // stage after which the number is drawn
      const int look_at = id_ready ? 0 : min(wk.nb - 1, draw_at + 1);          // ... and after which it is looked at
      const int4 rc = cur.rc;
      const bool absent = cur.absent, aligned = cur.aligned;
      const unsigned char* maps = cur.maps;
      for (int blk = 0; blk < wk.nb; ++blk, ++q) {
      const int s = q % kStageCount;
      const unsigned ph = (q / kStageCount) & 1;
      if (!mbar_wait(&wempty[s], ph ^ 1u)) {
        if (lane == 0) atomicExch(L.status, 2);
        return;
      }
      unsigned char* st = stages + static_cast<size_t>(s) * kStageBytes;
      if (lane == 0) {
        Desc d;
        d.flags = wk.kind | (absent ? 2 : 0) | (rc.y << 2) | (blk << 8) | (blk == wk.nb - 1 ? 1 << 16 : 0) |
                  ((k & 4095) << 20);
        d.tile = wk.tile; d.hrow0 = rc.z;
        d.row0 = wk.gi * (wk.kind == 0 ? kGateUpPairs : kDownRows);
        desc[s] = d;
      }
      if (!absent && aligned) {
        if (lane == 0) {
          mbar_expect_tx(&full[s], kWBytes);      // this lane's arrival, with the bytes to come
          if (wk.kind == 0) {
            tma_load_box(st, maps, blk * kW4, wk.gi * kGateUpPairs, &full[s]);
            tma_load_box(st + kHalfBytes, maps + 128, blk * kW4, wk.gi * kGateUpPairs, &full[s]);
          } else {
            tma_load_box(st, maps + 256, blk * kW4, wk.gi * kDownRows, &full[s]);
            tma_load_box(st + kHalfBytes, maps + 256, blk * kW4, wk.gi * kDownRows + kHalfRows, &full[s]);
          }
        }
      } else {
        if (!absent) {                           // sources without 16-byte alignment: plain loads
          const unsigned char *b0, *b1;
          int rb;
          if (wk.kind == 0) {
            rb = rb_h;
            b0 = cur.w0 + static_cast<size_t>(wk.gi) * kGateUpPairs * rb_h + blk * kW4;
            b1 = cur.w1 + static_cast<size_t>(wk.gi) * kGateUpPairs * rb_h + blk * kW4;
          } else {
            rb = rb_f;
            b0 = cur.w2 + static_cast<size_t>(wk.gi) * kDownRows * rb_f + blk * kW4;
            b1 = b0 + static_cast<size_t>(kHalfRows) * rb_f;
          }
          for (int p = lane; p < kHalfBytes / 16; p += 32) {
            const int r = p / 9, c = (p - r * 9) * 16;
            copy16_any(st + p * 16, b0 + static_cast<size_t>(r) * rb + c);
            copy16_any(st + kHalfBytes + p * 16, b1 + static_cast<size_t>(r) * rb + c);
          }
          fence_proxy_async();                   // the next fill of this stage may come from the TMA unit
        }
        __syncwarp();                            // every lane's part of the stage (and of its descriptor) is written
        if (lane == 0) mbar_arrive(&full[s]);
      }
      // the next group's number and global reads, requested between this group's copies
      if (blk == draw_at && lane == 0) drawn = static_cast<int>(atomicAdd(&L.cnt[10], 1u));
      if (blk == look_at) {
        nx.id = __shfl_sync(0xFFFFFFFFu, drawn, 0);
        nx.g = sc.decode(nx.id);
        id_ready = false;
        if (nx.g.valid) {
          nx.rc = tile_rec(nx.g.tile);
          if (nx.g.kind == 1) {                  // a short group: have the number after it at hand when it starts
            if (lane == 0) drawn = static_cast<int>(atomicAdd(&L.cnt[10], 1u));
            id_ready = true;
          }
        }
      }
      if (blk == wk.nb - 1 && nx.g.valid) load_ptrs(nx);
      }   // block columns of the group
      if (nx.g.valid) patch(nx);
      publish(k + 1, nx);
      cur = nx;
    }
  }

  if (warp > kConsumerWarps && warp <= kConsumerWarps + kXWarps) {
    // ---------------- activation warps ----------------
    const int xtid = tid - kConsumers - 32;
    int myoff = 0;                              // lane t < 16: byte offset of token slot t's row
    int q = 0;
    for (int k = 0;; ++k) {
      bool got;
      const GEntry* ge = follow(k, got);
      if (!got) {
        if (lane == 0) atomicExch(L.status, 7);
        return;
      }
      const Group wk = sc.decode(ge->id);
      const int4 rc = ge->rc;
      const bool absent = (ge->absent & 1) != 0;
      if (!wk.valid) {                           // end of the list: count in at the last stage and leave
        const int s = q % kStageCount;
        const unsigned ph = (q / kStageCount) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1u)) {
          if (lane == 0) atomicExch(L.status, 2);
          return;
        }
        cp_async_arrive(&full[s]);
        return;
      }
      myoff = 0;
      if (wk.kind == 0) {
        if (lane < rc.y) myoff = ge->rows[lane] * L.xq16_stride;
      } else {
        if (lane < rc.y) myoff = (rc.z + lane) * L.nbf * kHq;
        if (!absent && !(ge->absent & 2)) {     // the tile's h must be quantised and published
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
      for (int blk = 0; blk < wk.nb; ++blk, ++q) {
      const int s = q % kStageCount;
      const unsigned ph = (q / kStageCount) & 1;
      if (!mbar_wait(&empty[s], ph ^ 1u)) {
        if (lane == 0) atomicExch(L.status, 2);
        return;
      }
      unsigned char* xs = stages + static_cast<size_t>(s) * kStageBytes + kWBytes;
      if (!absent) {
        // 288-byte blocks (quantised inputs for gate/up, quantised h for down): 16-byte copies
        const unsigned char* xsrc = (wk.kind == 0 ? L.xq16 : L.hq) + blk * kHq;
        const int total = rc.y * (kHq / 16);
        for (int base = 0; base < total; base += kXThreads) {      // warp-uniform trip count
          const int i = base + xtid;
          const bool valid = i < total;
          const int t = valid ? i / (kHq / 16) : 0;
          const int c = i - t * (kHq / 16);
          const int off = __shfl_sync(0xFFFFFFFFu, myoff, t);
          if (valid) {
            // scale | codes (second half of the block 16 bytes further on: see XTile::mid_pad) | sums
            unsigned char* dst = c == 0 ? xs + kXCodes + kTok * 16 + t * 16
                                        : (c <= 16 ? xs + t * kXqStride + (c - 1) * 16 + (c > 8 ? 16 : 0)
                                                   : xs + kXCodes + t * 16);
            cp_async16(dst, xsrc + off + c * 16);
          }
        }
      }
      cp_async_arrive(&full[s]);
      }   // block columns of the group
    }
  }

  if (warp == kConsumerWarps + 1 + kXWarps) {
    // ---------------- finisher warp ----------------
    // Takes the finished gate/up groups of this CTA in order: counts the CTA in at the
    // group's block of h, and if that completes the block, quantises it for the tile's
    // rows and publishes it. The consumers never wait for any of this.
    for (int g = 0;; ++g) {
      bool got;
      const GEntry* ge = follow(g, got);
      if (!got) {
        if (lane == 0) atomicExch(L.status, 7);
        return;
      }
      const Group wk = sc.decode(ge->id);
      if (!wk.valid || wk.kind == 1) return;     // a CTA's gate/up groups all come before its down groups
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
  for (int q = 0;; ++q) {
    const int s = q % kStageCount;
    const unsigned ph = (q / kStageCount) & 1;
    if (!mbar_wait(&full[s], ph)) {
      if (lane == 0) atomicExch(L.status, 3);
      ok = false;
      break;
    }
    const Desc d = desc[s];
    if (d.end()) break;
    const int d_kind = d.kind(), d_mode = d.absent(), d_ntok = d.ntok(), d_blk = d.blk(), d_last = d.last(), d_seq = d.seq();
    unsigned char* st = stages + static_cast<size_t>(s) * kStageBytes;
    if (d_blk == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[0][j] = acc[1][j] = 0.f;
    }
    bool w_released = false;
    if (d_mode == 0) {
      XTile xt;
      xt.qs = reinterpret_cast<int8_t*>(st + kWBytes);
      xt.bs = reinterpret_cast<int16_t*>(st + kWBytes + kXCodes);
      xt.bl = nullptr;
      xt.d = reinterpret_cast<float*>(st + kWBytes + kXCodes + kTok * 16);
      xt.nb = 1;
      xt.tok_stride = kXqStride;
      xt.d_step = 4;
      xt.mid_pad = 16;
      // unit row u of this warp -> byte offset of its block in the stage
      auto row_at = [&](int u) {
        return d_kind == 0 ? ((u & 7) + 8 * warp) * kW4 + (u >> 3) * kHalfBytes : (16 * warp + u) * kW4;
      };
      if (d_ntok <= 2) {
        // the lane's half block goes to registers and the weight part of the stage back to the
        // weight warp before the arithmetic: its refill is the long round trip of the ring
        float a2[2] = {acc[0][0], acc[0][1]};
        uint4 hdr, wq[4];
        half_block_load(reinterpret_cast<const uint4*>(st + row_at(lane >> 1)), lane & 1, hdr, wq);
        __syncwarp();
        if (lane == 0) mbar_arrive(&wempty[s]);
        w_released = true;
        half_block_dot_regs<2>(hdr, wq, lane & 1, xt, d_ntok, a2);
        acc[0][0] = a2[0];
        acc[0][1] = a2[1];
      } else {
        const unsigned char* a_ptr = st + row_at((lane & 7) + ((lane >> 3) & 1) * 8) + 16 + (lane >> 4) * 16;
        const unsigned char* h_lo = st + row_at(lane >> 2);
        const unsigned char* h_hi = st + row_at((lane >> 2) + 8);
        auto loaded = [&]() {
          __syncwarp();
          if (lane == 0) mbar_arrive(&wempty[s]);
        };
        w_released = true;
        if (d_ntok <= 8) warp_mma_block<1>(a_ptr, h_lo, h_hi, xt, acc, loaded);
        else warp_mma_block<2>(a_ptr, h_lo, h_hi, xt, acc, loaded);
      }
    }
    __syncwarp();
    if (lane == 0) {                             // this warp no longer reads the stage
      if (!w_released) mbar_arrive(&wempty[s]);
      mbar_arrive(&empty[s]);
    }
    if (!d_last) continue;

    // ---- the group is complete for this warp's rows ----
    const int gid = lane >> 2, tig = lane & 3;
    if (d_kind == 0) {
      if (d_mode == 1) {
        if (d.row0 == 0 && warp == 0 && lane == 0 && L.mail != nullptr) {
          const int e = tile_rec(d.tile).x;
          if (e != L.E) {
            const int mi = atomicAdd(L.mail_n, 1);
            if (mi < L.E) L.mail[mi] = e;
          }
        }
      } else
      if (d_ntok <= 2) {
        const float u0 = __shfl_down_sync(0xFFFFFFFFu, acc[0][0], 16);
        const float u1 = __shfl_down_sync(0xFFFFFFFFu, acc[0][1], 16);
        if (lane < 16 && (lane & 1) == 0) {
          const int col = d.row0 + 8 * warp + (lane >> 1);
          const float g0 = acc[0][0], g1 = acc[0][1];
          L.hbuf[static_cast<size_t>(d.hrow0) * L.FF + col] = g0 / (1.f + expf(-g0)) * u0;
          if (d_ntok > 1) L.hbuf[static_cast<size_t>(d.hrow0 + 1) * L.FF + col] = g1 / (1.f + expf(-g1)) * u1;
        }
      } else {
        const int col = d.row0 + 8 * warp + gid;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const int t0 = 8 * n + 2 * tig;
          if (t0 < d_ntok) {
            const float g = acc[n][0], u = acc[n][2];
            L.hbuf[static_cast<size_t>(d.hrow0 + t0) * L.FF + col] = g / (1.f + expf(-g)) * u;
          }
          if (t0 + 1 < d_ntok) {
            const float g = acc[n][1], u = acc[n][3];
            L.hbuf[static_cast<size_t>(d.hrow0 + t0 + 1) * L.FF + col] = g / (1.f + expf(-g)) * u;
          }
        }
      }
      // Count the warp in at the CTA's counter of this group (shared memory); the last
      // warp hands the group to the finisher warp. Groups finish in order: a warp is at
      // most a ring's depth of stages ahead of the slowest one.
      __threadfence_block();
      __syncwarp();
      if (lane == 0) {
        if (atomicAdd(&grp_cnt[d_seq & 7], 1u) == kConsumerWarps - 1) {
          grp_cnt[d_seq & 7] = 0u;
          unsigned it = 0;                       // queue full: wait (bounded) for the finisher
          while (static_cast<unsigned>(d_seq) - *done_head >= static_cast<unsigned>(kDoneSlots) && ++it < kSpinLimit)
            __nanosleep(100);
          if (it >= kSpinLimit) atomicExch(L.status, 6);
          Done r;
          r.tile = d.tile; r.hb = d.row0 / kQK; r.hrow0 = d.hrow0; r.ntok = d_mode == 1 ? 0 : d_ntok;
          done_q[d_seq % kDoneSlots] = r;
          __threadfence_block();
          *done_tail = static_cast<unsigned>(d_seq) + 1u;
        }
      }
    } else {
      if (d_mode == 1) {
        for (int j = lane; j < 16 * d_ntok; j += 32)
          L.ybuf[static_cast<size_t>(d.hrow0 + j / 16) * L.H + d.row0 + 16 * warp + (j & 15)] = 0.f;
        continue;
      }
      if (d_ntok <= 2) {
        if ((lane & 1) == 0) {
          const int col = d.row0 + 16 * warp + (lane >> 1);
          L.ybuf[static_cast<size_t>(d.hrow0) * L.H + col] = acc[0][0];
          if (d_ntok > 1) L.ybuf[static_cast<size_t>(d.hrow0 + 1) * L.H + col] = acc[0][1];
        }
      } else {
        const int col = d.row0 + 16 * warp + gid;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const int t0 = 8 * n + 2 * tig;
          if (t0 < d_ntok) {
            L.ybuf[static_cast<size_t>(d.hrow0 + t0) * L.H + col] = acc[n][0];
            L.ybuf[static_cast<size_t>(d.hrow0 + t0) * L.H + col + 8] = acc[n][2];
          }
          if (t0 + 1 < d_ntok) {
            L.ybuf[static_cast<size_t>(d.hrow0 + t0 + 1) * L.H + col] = acc[n][1];
            L.ybuf[static_cast<size_t>(d.hrow0 + t0 + 1) * L.H + col + 8] = acc[n][3];
          }
        }
      }
    }
  }

  // ---- all y rows written everywhere: blend ------------------------------------------------
  __threadfence();
  rs_consumers_sync();
  if (tid == 0) {
    atomicAdd(&L.cnt[9], 1u);
    unsigned it = 0;
    while (ld_acquire(&L.cnt[9]) < gridDim.x && ++it < kSpinLimit) __nanosleep(32);
    flag[0] = (it < kSpinLimit && ok) ? 1 : 0;
  }
  rs_consumers_sync();
  if (!flag[0]) {
    if (tid == 0) atomicExch(L.status, 5);
    return;
  }
  combine_flat(L, blockIdx.x * kConsumers + tid, gridDim.x * kConsumers, slot_p, plan_own);
  if (L.ep_out != nullptr) {
    // Owner side of an expert-parallel layer: the rows went straight into the home ranks' buffers;
    // the last CTA to finish tells the home ranks.
    // (CTA barrier, then one thread's acquire-release count; its system-scope fence is cumulative)
    rs_consumers_sync();
    if (tid == 0) {
      if (atom_add_acq_rel(&L.cnt[11], 1u) == gridDim.x - 1) {
        L.cnt[11] = 0u;
        const unsigned v = *L.ep_step * L.ep_mul + L.ep_add;
        set_arrival_words(L.ep_flags, L.ep_world, v);
      }
    }
  }
}

}  // namespace rs
