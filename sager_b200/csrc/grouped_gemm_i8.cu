// grouped_gemm_i8.cu - the prefill MoE grouped GEMM on the 5th-generation tensor
// cores: tcgen05.mma kind::i8 with the accumulators in tensor memory.
//
// It replaces the reference's prefill expert math for chunks of many tokens
// (dequant_experts_q4_k_f16 + one cublasGemmEx per expert and matrix,
// src/kernels/cuda/tc_gemm.cu:124-152, 209-240, driven from
// src/core/session.cpp:2643-2760) but keeps the arithmetic of the reference's
// Q4_K x Q8_K path (gemv_grouped_tab_q4_k_q8_f16out_mtok, q4_k.cu:765-836): Q8_K
// activations, exact integer dots, fp32 scaling - so it is checked against that
// path, not against the fp16 one.
//
// The kernel is persistent: one CTA per SM takes work items (expert, tile of 128 weight rows)
// round-robin, so tensor memory, the barriers and the pipeline are set up once per SM and the
// roles run on into the next item without draining. Inside an item the CTA walks that expert's
// token rows in chunks of up to 64, two chunks per pass. The work of a pass is a list of jobs
// (super-block, chunk); job j uses accumulator set j & 1 in tensor memory and is
// finished by epilogue group j & 1, so with one chunk the two groups take alternate
// super-blocks and with two chunks each group owns a chunk. Four roles run as a
// pipeline over mbarriers:
//   * unpack warps (one thread per weight row): the 144-byte block becomes seventeen
//     int8 operand tiles per super-block. The 6-bit scale rides through the MMA: with
//     sc = 8a + b the products b*q and a*q (<= 105) are two u8 tiles per sub-block, so a
//     whole block accumulates exactly in int32 as D_b + 8*D_a; the eight min bytes are
//     one more tile. Double-buffered.
//   * stager warps: the activation codes of the job's chunk, copied asynchronously
//     into the B tiles (three buffers in flight), the sub-block sums split as
//     128*hi + lo into two more tiles (for the min term), the fp32 scales aside.
//   * one elected thread issues the 18 MMAs of a job (M=128, N=chunk, K=32,
//     tcgen05.mma kind::i8) and commits them to the barriers that release the
//     accumulators to the epilogue and the operand buffers to their producers.
//   * epilogue warps read their 32 lanes back (tcgen05.ld) and fold
//     xd*(d*(D_b + 8*D_a) - dmin*(mlo + 128*mhi)) into per-token fp32 registers while the
//     next job's MMAs run.
// Operand tiles use the canonical K-major layout without swizzle: 8 rows x 16 bytes
// per core matrix, the two K halves 128 bytes apart, 8-row groups 256 bytes apart.
// Every wait is bounded; on expiry the CTA raises the status word, frees its tensor
// memory and returns.
#include "api_util.cuh"
#include "q4k_common.cuh"

namespace sgr {
namespace {

constexpr int kGemmRows = 128;     // weight rows per CTA = MMA M
constexpr int kGemmTok = 64;       // token rows per chunk = max MMA N
constexpr int kTileA = kGemmRows * 32;            // bytes of one A tile (128 x 32 int8)
constexpr int kTileB = kGemmTok * 32;             // bytes of one B tile (64 x 32 int8)
constexpr int kATiles = 17;                       // 8 sub-blocks x {b*q, a*q} + the min tile
constexpr int kBTiles = 10;                       // 8 code tiles + 2 split-sum tiles
constexpr int kABufs = 2, kBBufs = 3, kDdRing = 4, kXdRing = 6;
constexpr int kTmemCols = 512;                    // two sets of four 64-column accumulators

constexpr int kEpiWarps = 8, kUnpackWarps = 4, kStageWarps = 3;
constexpr int kWarpUnpack0 = kEpiWarps, kWarpCtrl = kEpiWarps + kUnpackWarps, kWarpStage0 = kWarpCtrl + 1;
constexpr int kGemmThreads = (kEpiWarps + kUnpackWarps + 1 + kStageWarps) * 32;    // 512

// shared-memory map (bytes)
constexpr int kOffBar = 0;                                        // mbarriers, tmem base
constexpr int kOffA = 1024;
constexpr int kOffB = kOffA + kABufs * kATiles * kTileA;
constexpr int kOffXd = kOffB + kBBufs * kBTiles * kTileB;         // [kXdRing][64] fp32 activation scales
constexpr int kOffDd = kOffXd + kXdRing * kGemmTok * 4;           // [kDdRing][128] float2 (d, dmin)
constexpr int kOffRed = kOffDd + kDdRing * kGemmRows * 8;         // [128][32] floats: one-chunk passes, group 1 -> group 0
constexpr int kGemmSmem = kOffRed + kGemmRows * 32 * 4;
static_assert(kGemmSmem <= 227 * 1024, "shared memory");

enum { kBarAFull = 0, kBarAEmpty = 2, kBarBFull = 4, kBarBEmpty = 7, kBarAccFull = 10, kBarAccEmpty = 12, kBarCount = 14 };

__device__ __forceinline__ uint64_t umma_desc(const void* smem_tile) {
  // K-major, no swizzle: start >> 4 | LBO (128 B) >> 4 << 16 | SBO (256 B) >> 4 << 32 | version 1 << 46
  return static_cast<uint64_t>((smem_u32(smem_tile) & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(8) << 16) |
         (static_cast<uint64_t>(16) << 32) | (static_cast<uint64_t>(1) << 46);
}
// D format s32, A unsigned 8-bit, B signed 8-bit, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t umma_idesc_i8(int n) {
  return (2u << 4) | (0u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(kGemmRows >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// address of (row, 16-byte K half) inside a canonical tile
__device__ __forceinline__ unsigned char* tile_at(unsigned char* tile, int row, int khalf) {
  return tile + (row >> 3) * 256 + khalf * 128 + (row & 7) * 16;
}

// 16 bytes of a weight block: one 128-bit load when the expert's base is 16-byte
// aligned (the normal case), 32-bit or 16-bit loads otherwise (the pointer-table
// contract only promises the alignment of the block struct)
__device__ __forceinline__ uint4 load16(const unsigned char* p, int align) {
  if (align == 16) return __ldg(reinterpret_cast<const uint4*>(p));
  uint32_t v[4];
  if (align == 4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __ldg(reinterpret_cast<const uint32_t*>(p) + i);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint16_t* h = reinterpret_cast<const uint16_t*>(p) + 2 * i;
      v[i] = static_cast<uint32_t>(__ldg(h)) | (static_cast<uint32_t>(__ldg(h + 1)) << 16);
    }
  }
  return make_uint4(v[0], v[1], v[2], v[3]);
}

// The jobs of a CTA in the order every role walks them.
struct JobWalk {
  int m_e, nb;
  int pass, blk, ci, nc, j, abk;         // current pass, block column, chunk in pass, chunks in pass, job number, block number
  __device__ __forceinline__ void start(int m_e_, int nb_) {
    m_e = m_e_; nb = nb_; pass = 0; blk = 0; ci = 0; j = 0; abk = 0;
    nc = min(2, (m_e + kGemmTok - 1) / kGemmTok);
  }
  __device__ __forceinline__ bool done() const { return pass * 2 * kGemmTok >= m_e; }
  __device__ __forceinline__ int t0() const { return (2 * pass + ci) * kGemmTok; }
  __device__ __forceinline__ int nt() const { return min(kGemmTok, m_e - t0()); }
  __device__ __forceinline__ bool first_of_block() const { return ci == 0; }
  __device__ __forceinline__ bool last_of_block() const { return ci == nc - 1; }
  __device__ __forceinline__ void next() {
    ++j;
    if (++ci < nc) return;
    ci = 0; ++abk;
    if (++blk < nb) return;
    blk = 0; ++pass;
    nc = min(2, (m_e - pass * 2 * kGemmTok + kGemmTok - 1) / kGemmTok);
  }
};

// One work item: 128 weight rows of one expert against that expert's token rows.
struct Item {
  int e, row0, row_off, m_e;
  const unsigned char* w;
};

// grid: one CTA per SM (or per item when there are fewer); item i = expert i / tiles, row tile i % tiles.
// With single_w the kernel serves ONE matrix over single_rows token rows (a dense projection, the shared
// expert of a prefill chunk): item i = token pass i / tiles (128 rows each), row tile i % tiles.
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_i8_kernel(const unsigned char* const* __restrict__ w_tab, const int* __restrict__ off,
                       const unsigned char* __restrict__ xq, uint16_t* __restrict__ y, int n_rows,
                       int nb, int tiles, int n_items, const unsigned char* single_w, int single_rows,
                       int* status) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto item_at = [&](int it) {
    Item r;
    r.e = it / tiles;
    r.row0 = (it - r.e * tiles) * kGemmRows;
    if (single_w != nullptr) {                   // r.e is the token pass
      r.row_off = r.e * 2 * kGemmTok;
      r.m_e = min(2 * kGemmTok, single_rows - r.row_off);
      r.w = single_w;
      return r;
    }
    r.row_off = __ldg(off + r.e);
    r.m_e = __ldg(off + r.e + 1) - r.row_off;
    r.w = w_tab[r.e];
    return r;
  };
  // first item at or after `it` (in this CTA's stride) that has token rows; with `need_w` also weights
  auto next_item = [&](int it, bool need_w) {
    for (; it < n_items; it += gridDim.x) {
      const Item r = item_at(it);
      if (r.m_e > 0 && (!need_w || r.w != nullptr)) break;
    }
    return it;
  };
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBar + 128);
  int* fail = reinterpret_cast<int*>(smem + kOffBar + 136);
  unsigned char* a_base = smem + kOffA;
  unsigned char* b_base = smem + kOffB;
  float* xd_sm = reinterpret_cast<float*>(smem + kOffXd);
  float2* dd_sm = reinterpret_cast<float2*>(smem + kOffDd);
  float* red = reinterpret_cast<float*>(smem + kOffRed);

  if (tid == 0) {
    for (int i = 0; i < kABufs; ++i) { mbar_init(&bar[kBarAFull + i], kUnpackWarps * 32); mbar_init(&bar[kBarAEmpty + i], 1); }
    for (int i = 0; i < kBBufs; ++i) { mbar_init(&bar[kBarBFull + i], 32); mbar_init(&bar[kBarBEmpty + i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bar[kBarAccFull + i], 1); mbar_init(&bar[kBarAccEmpty + i], 4 * 32); }
    *fail = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  const size_t xrow_bytes = static_cast<size_t>(nb) * kX8;
  JobWalk jw;
  auto failed = [&]() { return *reinterpret_cast<volatile int*>(fail) != 0; };
  // a wait that gives up: flag the CTA, every role leaves its loop at its next wait
  auto wait = [&](int b, unsigned parity) {
    if (*reinterpret_cast<volatile int*>(fail)) return false;
    if (mbar_wait(&bar[b], parity)) return true;
    *reinterpret_cast<volatile int*>(fail) = 1;
    return false;
  };

  if (warp >= kWarpUnpack0 && warp < kWarpCtrl) {
    // ---------------- unpack: this thread's weight row -> operand tiles ----------------
    const int r = tid - kWarpUnpack0 * 32;
    auto row_ptr = [&](const Item& I) {
      const int row = min(I.row0 + r, n_rows - 1);         // ragged last tile: duplicate, never stored
      return I.w + static_cast<size_t>(row) * nb * kW4;
    };
    auto align_of = [](const unsigned char* w) {
      const uintptr_t wa = reinterpret_cast<uintptr_t>(w);
      return (wa & 15u) == 0 ? 16 : ((wa & 3u) == 0 ? 4 : 2);
    };
    // this thread's whole weight row of an item (nb blocks, contiguous) asked into L2: the loads that
    // follow an item later find it there instead of waiting for DRAM one block column at a time
    auto prefetch_row = [&](const unsigned char* p) {
      const unsigned char* end = p + static_cast<size_t>(nb) * kW4;
      for (const unsigned char* q = reinterpret_cast<const unsigned char*>(reinterpret_cast<uintptr_t>(p) & ~static_cast<uintptr_t>(127));
           q < end; q += 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(q));
    };
    int it = next_item(blockIdx.x, true);
    uint4 cur[9];
    if (it < n_items) {
      const Item I0 = item_at(it);
      const unsigned char* w0 = row_ptr(I0);
      const int a0 = align_of(I0.w);
      prefetch_row(w0);
#pragma unroll
      for (int i = 0; i < 9; ++i) cur[i] = load16(w0 + 16 * i, a0);
    }
    int abk_base = 0;
    while (it < n_items && !failed()) {
      const Item I = item_at(it);
      const unsigned char* wrow = row_ptr(I);
      const int walign = align_of(I.w);
      const int it_next = next_item(it + gridDim.x, true);
      const unsigned char* wrow_next = nullptr;
      int walign_next = 16;
      if (it_next < n_items) {
        const Item In = item_at(it_next);
        wrow_next = row_ptr(In);
        walign_next = align_of(In.w);
        prefetch_row(wrow_next);
      }
      jw.start(I.m_e, nb);
      int prev_abk = -1;
      bool gave_up = false;
      for (; !jw.done(); jw.next()) {
      if (jw.abk == prev_abk) continue;                     // one unpack per block column
      prev_abk = jw.abk;
      const int abk = abk_base + jw.abk;
      const int buf = abk % kABufs;
      const unsigned ph = (abk / kABufs) & 1;
      // the next block column in sequence is requested now: the next column of this row (column 0
      // again for the next pass), or the first column of the next item's row
      uint4 nxt[9];
      {
        const bool last_col = jw.blk + 1 == nb && (jw.pass + 1) * 2 * kGemmTok >= I.m_e;
        const unsigned char* wn = last_col ? wrow_next : wrow + static_cast<size_t>(jw.blk + 1 < nb ? jw.blk + 1 : 0) * kW4;
        const int an = last_col ? walign_next : walign;
        if (wn != nullptr) {
#pragma unroll
          for (int i = 0; i < 9; ++i) nxt[i] = load16(wn + 16 * i, an);
        } else {
#pragma unroll
          for (int i = 0; i < 9; ++i) nxt[i] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      if (!wait(kBarAEmpty + buf, ph ^ 1u)) { gave_up = true; break; }
      unsigned char* a_tiles = a_base + static_cast<size_t>(buf) * kATiles * kTileA;
      const uint4 hdr = cur[0];
      const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x & 0xFFFFu)));
      const float dmin = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x >> 16)));
      const Scales6 s6 = unpack_scales6(hdr.y, hdr.z, hdr.w);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint4 q0 = cur[1 + 2 * g], q1 = cur[2 + 2 * g];
        const uint32_t raw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint32_t sc_e = (s6.sc[g >> 1] >> (16 * (g & 1))) & 0xFFu;        // sub-block 2g
        const uint32_t sc_o = (s6.sc[g >> 1] >> (16 * (g & 1) + 8)) & 0xFFu;    // sub-block 2g+1
        const uint32_t be = sc_e & 7u, ae = sc_e >> 3, bo = sc_o & 7u, ao = sc_o >> 3;
        uint32_t tb_e[8], ta_e[8], tb_o[8], ta_o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t lo = raw[i] & 0x0F0F0F0Fu, hi = (raw[i] >> 4) & 0x0F0F0F0Fu;
          tb_e[i] = lo * be; ta_e[i] = lo * ae;            // bytes <= 105: no carry between bytes
          tb_o[i] = hi * bo; ta_o[i] = hi * ao;
        }
        unsigned char* t0p = a_tiles + (4 * g + 0) * kTileA;   // tile order: [sub-block][b part, a part]
        unsigned char* t1p = a_tiles + (4 * g + 1) * kTileA;
        unsigned char* t2p = a_tiles + (4 * g + 2) * kTileA;
        unsigned char* t3p = a_tiles + (4 * g + 3) * kTileA;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          *reinterpret_cast<uint4*>(tile_at(t0p, r, h)) = make_uint4(tb_e[4 * h], tb_e[4 * h + 1], tb_e[4 * h + 2], tb_e[4 * h + 3]);
          *reinterpret_cast<uint4*>(tile_at(t1p, r, h)) = make_uint4(ta_e[4 * h], ta_e[4 * h + 1], ta_e[4 * h + 2], ta_e[4 * h + 3]);
          *reinterpret_cast<uint4*>(tile_at(t2p, r, h)) = make_uint4(tb_o[4 * h], tb_o[4 * h + 1], tb_o[4 * h + 2], tb_o[4 * h + 3]);
          *reinterpret_cast<uint4*>(tile_at(t3p, r, h)) = make_uint4(ta_o[4 * h], ta_o[4 * h + 1], ta_o[4 * h + 2], ta_o[4 * h + 3]);
        }
      }
      {  // min tile: the eight min bytes at k = 0..7, zeros elsewhere
        unsigned char* t_mn = a_tiles + 16 * kTileA;
        *reinterpret_cast<uint4*>(tile_at(t_mn, r, 0)) = make_uint4(s6.mn[0], s6.mn[1], 0u, 0u);
        *reinterpret_cast<uint4*>(tile_at(t_mn, r, 1)) = make_uint4(0u, 0u, 0u, 0u);
      }
      dd_sm[(abk % kDdRing) * kGemmRows + r] = make_float2(d, dmin);
      fence_proxy_async();                                 // operand tiles -> visible to the tensor core
      mbar_arrive_cta(&bar[kBarAFull + buf]);
#pragma unroll
      for (int i = 0; i < 9; ++i) cur[i] = nxt[i];
      }   // block columns of the item
      if (gave_up) break;
      abk_base += jw.abk;
      it = it_next;
    }
  } else if (warp >= kWarpStage0) {
    // ---------------- stagers: activation codes, split sums and scales of a job's chunk ----------------
    // Each of the three stager warps takes every third job; a lane owns token rows `lane` and
    // `lane + 32` of the chunk. The 256 codes of a packed Q8_K block start 4 bytes into the
    // 276-byte block, so their 16-byte pieces are not aligned: the lane reads the 17 aligned
    // pieces that cover them and picks each operand piece out of two neighbours by whole words.
    const int sg = warp - kWarpStage0;
    int j_base = 0;
    bool ok = true;
    for (int it = next_item(blockIdx.x, true); it < n_items && !failed(); it = next_item(it + gridDim.x, true)) {
    const Item I = item_at(it);
    const int row_off = I.row_off;
    jw.start(I.m_e, nb);
    for (; !jw.done(); jw.next()) {
      const int j = j_base + jw.j, buf = j % kBBufs;
      if (j % kStageWarps != sg) continue;
      const unsigned ph = (j / kBBufs) & 1;
      const int t0 = jw.t0(), nt = jw.nt();
      unsigned char* b_tiles = b_base + static_cast<size_t>(buf) * kBTiles * kTileB;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        const int s = lane + 32 * half;                    // token row of the chunk
        uint4 wv[17];
        uint32_t pf[5] = {0u, 0u, 0u, 0u, 0u};             // scale, four words of sub-block sums
        int sh = 0;
        if (s < nt) {                                       // requested before the buffer is known to be free
          const unsigned char* xb = xq + static_cast<size_t>(row_off + t0 + s) * xrow_bytes + static_cast<size_t>(jw.blk) * kX8;
          const uintptr_t cs = reinterpret_cast<uintptr_t>(xb) + 4;
          sh = static_cast<int>(cs & 15u) >> 2;
          const uint4* a0 = reinterpret_cast<const uint4*>(cs & ~static_cast<uintptr_t>(15));
#pragma unroll
          for (int i = 0; i < 17; ++i) wv[i] = __ldg(a0 + i);
          pf[0] = __ldg(reinterpret_cast<const uint32_t*>(xb));
          const uint32_t* bs = reinterpret_cast<const uint32_t*>(xb + 260);       // 8 x int16
          pf[1] = __ldg(bs); pf[2] = __ldg(bs + 1); pf[3] = __ldg(bs + 2); pf[4] = __ldg(bs + 3);
        }
        if (half == 0) {
          ok = __all_sync(0xFFFFFFFFu, wait(kBarBEmpty + buf, ph ^ 1u));
          if (!ok) break;
        }
        if (s < nt) {
          auto put = [&](int c, uint32_t a, uint32_t b, uint32_t cc, uint32_t d) {
            *reinterpret_cast<uint4*>(tile_at(b_tiles + (c >> 1) * kTileB, s, c & 1)) = make_uint4(a, b, cc, d);
          };
          if (sh == 0) {
#pragma unroll
            for (int c = 0; c < 16; ++c) put(c, wv[c].x, wv[c].y, wv[c].z, wv[c].w);
          } else if (sh == 1) {
#pragma unroll
            for (int c = 0; c < 16; ++c) put(c, wv[c].y, wv[c].z, wv[c].w, wv[c + 1].x);
          } else if (sh == 2) {
#pragma unroll
            for (int c = 0; c < 16; ++c) put(c, wv[c].z, wv[c].w, wv[c + 1].x, wv[c + 1].y);
          } else {
#pragma unroll
            for (int c = 0; c < 16; ++c) put(c, wv[c].w, wv[c + 1].x, wv[c + 1].y, wv[c + 1].z);
          }
        }
        {                                                   // sums split as bsum = 128*hi + lo; rows beyond nt: zero scale
          uint32_t lo01 = 0, lo23 = 0, hi01 = 0, hi23 = 0;
          float xd = 0.f;
          if (s < nt) {
            xd = __uint_as_float(pf[0]);
            lo01 = __byte_perm(pf[1] & 0x007F007Fu, pf[2] & 0x007F007Fu, 0x6420);
            lo23 = __byte_perm(pf[3] & 0x007F007Fu, pf[4] & 0x007F007Fu, 0x6420);
            hi01 = __byte_perm((pf[1] >> 7) & 0x00FF00FFu, (pf[2] >> 7) & 0x00FF00FFu, 0x6420);
            hi23 = __byte_perm((pf[3] >> 7) & 0x00FF00FFu, (pf[4] >> 7) & 0x00FF00FFu, 0x6420);
          }
          xd_sm[(j % kXdRing) * kGemmTok + s] = xd;
          *reinterpret_cast<uint4*>(tile_at(b_tiles + 8 * kTileB, s, 0)) = make_uint4(lo01, lo23, 0u, 0u);
          *reinterpret_cast<uint4*>(tile_at(b_tiles + 8 * kTileB, s, 1)) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(tile_at(b_tiles + 9 * kTileB, s, 0)) = make_uint4(hi01, hi23, 0u, 0u);
          *reinterpret_cast<uint4*>(tile_at(b_tiles + 9 * kTileB, s, 1)) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      if (!ok) break;
      fence_proxy_async();
      mbar_arrive_cta(&bar[kBarBFull + buf]);
    }
    if (!ok) break;
    j_base += jw.j;
    }   // items
  } else if (warp == kWarpCtrl) {
    // ---------------- MMA issue: one elected thread ----------------
    if (lane == 0) {
      int j_base = 0, abk_base = 0;
      unsigned use[2] = {0u, 0u};                           // jobs issued so far into each accumulator set
      bool ok = true;
      for (int it = next_item(blockIdx.x, true); it < n_items && ok; it = next_item(it + gridDim.x, true)) {
      const Item I = item_at(it);
      jw.start(I.m_e, nb);
      for (; !jw.done(); jw.next()) {
        const int j = j_base + jw.j, abk = abk_base + jw.abk;
        const int abuf = abk % kABufs, bbuf = j % kBBufs, set = jw.j & 1;
        ok = false;
        if (jw.first_of_block() && !wait(kBarAFull + abuf, (abk / kABufs) & 1)) break;
        if (!wait(kBarBFull + bbuf, (j / kBBufs) & 1)) break;
        if (!wait(kBarAccEmpty + set, (use[set] & 1u) ^ 1u)) break;
        ok = true;
        ++use[set];
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // descriptors of consecutive tiles differ by the tile size in the address field
        const uint64_t da0 = umma_desc(a_base + static_cast<size_t>(abuf) * kATiles * kTileA);
        const uint64_t db0 = umma_desc(b_base + static_cast<size_t>(bbuf) * kBTiles * kTileB);
        constexpr uint64_t kStepA = kTileA >> 4, kStepB = kTileB >> 4;
        const int n_mma = (jw.nt() + 15) & ~15;             // MMA N: multiple of 16
        const uint32_t idesc = umma_idesc_i8(n_mma);
        const uint32_t acc = tmem + set * 4 * kGemmTok;
        // D0 = sum (b*q) x, D1 = sum (a*q) x, D2 = min x sums_lo, D3 = min x sums_hi
#pragma unroll
        for (int sb = 0; sb < 8; ++sb) {
          umma_i8(acc + 0 * kGemmTok, da0 + (2 * sb) * kStepA, db0 + sb * kStepB, idesc, sb > 0);
          umma_i8(acc + 1 * kGemmTok, da0 + (2 * sb + 1) * kStepA, db0 + sb * kStepB, idesc, sb > 0);
        }
        umma_i8(acc + 2 * kGemmTok, da0 + 16 * kStepA, db0 + 8 * kStepB, idesc, 0u);
        umma_i8(acc + 3 * kGemmTok, da0 + 16 * kStepA, db0 + 9 * kStepB, idesc, 0u);
        umma_commit(&bar[kBarAccFull + set]);               // accumulators ready for the epilogue
        umma_commit(&bar[kBarBEmpty + bbuf]);               // B tiles free
        if (jw.last_of_block()) umma_commit(&bar[kBarAEmpty + abuf]);   // A tiles free
      }
      j_base += jw.j;
      abk_base += jw.abk;
      }   // items
    }
  } else {
    // ---------------- epilogue: two groups of four warps; this thread's row, the job's tokens ----------------
    const int grp = warp >> 2;
    const int row = (warp & 3) * 32 + lane;                // accumulator lane = weight row in the tile
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float acc[kGemmTok];
#pragma unroll
    for (int t = 0; t < kGemmTok; ++t) acc[t] = 0.f;
    bool ok = true;
    int j_base = 0, abk_base = 0;
    unsigned use = 0u;                                     // jobs this group has finished (the phase of its accumulator set)
    for (int it = next_item(blockIdx.x, false); it < n_items; it = next_item(it + gridDim.x, false)) {
    const Item I = item_at(it);
    const int row0 = I.row0, row_off = I.row_off, m_e = I.m_e;
    if (I.w == nullptr) {                                    // absent expert: zero rows
      for (int i = tid; i < m_e * kGemmRows; i += kEpiWarps * 32) {
        const int t = i / kGemmRows, r = row0 + (i % kGemmRows);
        if (r < n_rows) y[static_cast<size_t>(row_off + t) * n_rows + r] = 0;
      }
      continue;
    }
    jw.start(m_e, nb);
    int pass_t0 = 0, pass_nc = jw.nc, pass_nt0 = 0, pass_nt1 = 0, cur_pass = 0;
    auto flush = [&]() {
      // end of a pass: one chunk -> group 1 hands its sums to group 0 through shared memory
      // (two halves of 32 tokens); two chunks -> each group stores its own chunk
      const bool valid = row0 + row < n_rows && ok && !failed();
      if (pass_nc == 1) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (grp == 1) {
#pragma unroll
            for (int t = 0; t < 32; ++t) red[t * kGemmRows + row] = acc[32 * half + t];
          }
          asm volatile("bar.sync 1, 256;" ::: "memory");
          if (grp == 0) {
#pragma unroll
            for (int t = 0; t < 32; ++t) acc[32 * half + t] += red[t * kGemmRows + row];
          }
          asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        if (grp == 0 && valid) {
#pragma unroll
          for (int t = 0; t < kGemmTok; ++t)
            if (t < pass_nt0) y[static_cast<size_t>(row_off + pass_t0 + t) * n_rows + row0 + row] = f2h(acc[t]);
        }
      } else if (valid) {
        const int nt = grp == 0 ? pass_nt0 : pass_nt1;
        const int t0 = pass_t0 + grp * kGemmTok;
#pragma unroll
        for (int t = 0; t < kGemmTok; ++t)
          if (t < nt) y[static_cast<size_t>(row_off + t0 + t) * n_rows + row0 + row] = f2h(acc[t]);
      }
#pragma unroll
      for (int t = 0; t < kGemmTok; ++t) acc[t] = 0.f;
    };
    pass_nt0 = min(kGemmTok, m_e);
    pass_nt1 = min(kGemmTok, max(0, m_e - kGemmTok));
    for (; !jw.done(); jw.next()) {
      if (jw.pass != cur_pass) {                            // both groups see the pass change at the same job
        flush();
        cur_pass = jw.pass;
        pass_t0 = cur_pass * 2 * kGemmTok;
        pass_nc = jw.nc;
        pass_nt0 = min(kGemmTok, m_e - pass_t0);
        pass_nt1 = min(kGemmTok, max(0, m_e - pass_t0 - kGemmTok));
      }
      if ((jw.j & 1) != grp || !ok) continue;              // (a group that gave up still walks the list: the
                                                            //  barriers of the pass ends need both groups)
      const int j = j_base + jw.j, abk = abk_base + jw.abk;
      if (!__all_sync(0xFFFFFFFFu, wait(kBarAccFull + grp, use & 1u))) { ok = false; continue; }
      ++use;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float2 dd = dd_sm[(abk % kDdRing) * kGemmRows + row];
      const float* xd = xd_sm + (j % kXdRing) * kGemmTok;
      const int n_mma = (jw.nt() + 15) & ~15;
      const uint32_t accp = tmem + lane_base + grp * 4 * kGemmTok;
#pragma unroll
      for (int c0 = 0; c0 < kGemmTok; c0 += 16) {
        if (c0 < n_mma) {
          int vb[16], va[16], mlo[16], mhi[16];
          tmem_ld16(accp + 0 * kGemmTok + c0, vb);
          tmem_ld16(accp + 1 * kGemmTok + c0, va);
          tmem_ld16(accp + 2 * kGemmTok + c0, mlo);
          tmem_ld16(accp + 3 * kGemmTok + c0, mhi);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            const int isum = vb[q] + 8 * va[q];
            const int msum = mlo[q] + 128 * mhi[q];
            acc[c0 + q] += xd[c0 + q] * (dd.x * static_cast<float>(isum) - dd.y * static_cast<float>(msum));
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive_cta(&bar[kBarAccEmpty + grp]);
    }
    flush();
    j_base += jw.j;
    abk_base += jw.abk;
    }   // items
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && *fail && status != nullptr) atomicExch(status, 6);
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

}  // namespace
}  // namespace sgr

using namespace sgr;

// y[t][r] = W[r][:] . xq[t][:] for one matrix and n_tok token rows on the same tensor-core kernel
// (the shared expert of a prefill chunk: one "expert" that every row visits).
int sgr::gemm_i8_dense(const void* w, const void* xq, uint16_t* y, int n_tok, int n_rows, int k, cudaStream_t stream) {
  if (n_tok <= 0 || n_rows <= 0) return kOk;
  if (!w || !xq || !y || k <= 0 || k % kQK != 0) return kErrArg;
  if (reinterpret_cast<uintptr_t>(xq) & 15u) return kErrAlign;
  auto kern = grouped_gemm_i8_kernel;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem) != cudaSuccess)
    return kErrLaunch;
  int* status = status_word();
  if (status == nullptr) return kErrLaunch;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return kErrLaunch;
  const int tiles = (n_rows + kGemmRows - 1) / kGemmRows;
  const long long n_items = static_cast<long long>(tiles) * ((n_tok + 2 * kGemmTok - 1) / (2 * kGemmTok));
  if (n_items > 0x7FFFFFFF) return kErrUnsupported;
  kern<<<static_cast<unsigned>(n_items < sms ? n_items : sms), kGemmThreads, kGemmSmem, stream>>>(
      nullptr, nullptr, static_cast<const unsigned char*>(xq), y, n_rows, k / kQK, tiles, static_cast<int>(n_items),
      static_cast<const unsigned char*>(w), n_tok, status);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// y[off[e] + t][r] = W_e[r][:] . xq[off[e] + t][:] for every expert e and its rows
// t < off[e+1] - off[e]; fp16 out, row length n_rows. w_tab[e] == null: zero rows.
SGR_API int sgr_moe_grouped_gemm_i8(const void* const* w_tab, const int* off, const void* xq,
                                    uint16_t* y, int n_rows, int k, int n_expert, void* stream) {
  if (n_expert <= 0 || n_rows <= 0) return kOk;
  if (!w_tab || !off || !xq || !y || k <= 0 || k % kQK != 0) return kErrArg;
  if (reinterpret_cast<uintptr_t>(xq) & 15u) return kErrAlign;   // rows are read in aligned 16-byte pieces
  if (n_expert > 65535) return kErrUnsupported;
  auto kern = grouped_gemm_i8_kernel;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem) != cudaSuccess)
    return kErrLaunch;
  int* status = status_word();
  if (status == nullptr) return kErrLaunch;       // the kernel reports an expired wait through it
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return kErrLaunch;
  const int tiles = (n_rows + kGemmRows - 1) / kGemmRows;
  const long long n_items = static_cast<long long>(tiles) * n_expert;
  if (n_items > 0x7FFFFFFF) return kErrUnsupported;
  kern<<<static_cast<unsigned>(n_items < sms ? n_items : sms), kGemmThreads, kGemmSmem, as_stream(stream)>>>(
      reinterpret_cast<const unsigned char* const*>(w_tab), off, static_cast<const unsigned char*>(xq), y,
      n_rows, k / kQK, tiles, static_cast<int>(n_items), nullptr, 0, status);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}

