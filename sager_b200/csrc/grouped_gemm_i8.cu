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
// A CTA owns 128 weight rows of one expert and walks that expert's token rows in
// chunks of up to 64. For every super-block (256 weights):
//   * each thread (= one weight row) unpacks its 144-byte block and writes two
//     int8 operand tiles per 32-weight sub-block: the product sc*q (< 1024) split
//     as 128*hi + lo, so that the 6-bit scale rides through the MMA and the whole
//     block accumulates exactly in int32 (|sum| <= 256*127*127);
//   * the activation codes of the chunk are laid out as the B operand; the min
//     term sum_s mn[s]*bsum[s] is one more pair of MMAs (min bytes as A, the
//     sub-block sums split the same way as B);
//   * one elected thread issues the 18 MMAs (M=128, N=chunk, K=32) into four
//     accumulators in tensor memory and commits them to an mbarrier;
//   * the four warps read their 32 lanes back (tcgen05.ld) and fold
//     xd*(d*(128*hi+lo) - dmin*(128*mhi+mlo)) into per-token fp32 registers.
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
constexpr int kTmemCols = 256;                    // four accumulators of 64 columns

// shared-memory map (bytes)
constexpr int kOffBar = 0;                        // mbarrier + tmem base
constexpr int kOffA = 1024;                       // 8 sub-blocks x {lo, hi} + min tile = 17 A tiles
constexpr int kOffB = kOffA + 17 * kTileA;        // 8 code tiles + 2 sum tiles = 10 B tiles
constexpr int kOffXd = kOffB + 10 * kTileB;       // fp32 activation scales of the chunk
constexpr int kGemmSmem = kOffXd + kGemmTok * 4;

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

// sc * q for four weights (one per byte of `q4`, each 0..15), split as 128*hi + lo
__device__ __forceinline__ void scale_split(uint32_t q4, uint32_t sc, uint32_t& lo, uint32_t& hi) {
  const uint32_t pe = (q4 & 0x00FF00FFu) * sc;            // two 16-bit products, each <= 945
  const uint32_t po = ((q4 >> 8) & 0x00FF00FFu) * sc;
  lo = (pe & 0x007F007Fu) | ((po & 0x007F007Fu) << 8);
  hi = ((pe >> 7) & 0x000F000Fu) | (((po >> 7) & 0x000F000Fu) << 8);
}

// grid (ceil(n_rows / 128), n_expert), 128 threads
__global__ void __launch_bounds__(kGemmRows, 2)
grouped_gemm_i8_kernel(const unsigned char* const* __restrict__ w_tab, const int* __restrict__ off,
                       const unsigned char* __restrict__ xq, uint16_t* __restrict__ y, int n_rows,
                       int nb, int* status) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int e = blockIdx.y;
  const int row_off = off[e];
  const int m_e = off[e + 1] - row_off;
  if (m_e <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row0 = blockIdx.x * kGemmRows;
  const int row = min(row0 + tid, n_rows - 1);            // ragged last tile: duplicate, never store
  const unsigned char* w = w_tab[e];
  if (w == nullptr) {                                      // absent expert: zero rows
    for (int i = tid; i < m_e * kGemmRows; i += kGemmRows) {
      const int t = i / kGemmRows, r = row0 + (i % kGemmRows);
      if (r < n_rows) y[static_cast<size_t>(row_off + t) * n_rows + r] = 0;
    }
    return;
  }
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBar + 16);
  unsigned char* a_tiles = smem + kOffA;
  unsigned char* b_tiles = smem + kOffB;
  float* xd_sm = reinterpret_cast<float*>(smem + kOffXd);

  if (tid == 0) {
    mbar_init(bar, 1);
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
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const size_t xrow_bytes = static_cast<size_t>(nb) * kX8;
  const unsigned char* wrow = w + static_cast<size_t>(row) * nb * kW4;
  const uintptr_t wa = reinterpret_cast<uintptr_t>(w);
  const int walign = (wa & 15u) == 0 ? 16 : ((wa & 3u) == 0 ? 4 : 2);
  unsigned phase = 0;
  bool ok = true;

  for (int t0 = 0; t0 < m_e && ok; t0 += kGemmTok) {
    const int nt = min(kGemmTok, m_e - t0);
    const int n_mma = (nt + 15) & ~15;                     // MMA N: multiple of 16
    const uint32_t idesc = umma_idesc_i8(n_mma);
    float acc[kGemmTok];
#pragma unroll
    for (int t = 0; t < kGemmTok; ++t) acc[t] = 0.f;

    for (int blk = 0; blk < nb && ok; ++blk) {
      // ---- A: this thread's weight block -> 16 scaled operand tiles + the min tile ----
      const unsigned char* wb = wrow + static_cast<size_t>(blk) * kW4;
      const uint4 hdr = load16(wb, walign);
      const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x & 0xFFFFu)));
      const float dmin = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x >> 16)));
      const Scales6 s6 = unpack_scales6(hdr.y, hdr.z, hdr.w);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint4 q0 = load16(wb + 16 + 32 * g, walign), q1 = load16(wb + 32 + 32 * g, walign);
        const uint32_t raw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint32_t sc_e = (s6.sc[g >> 1] >> (16 * (g & 1))) & 0xFFu;        // sub-block 2g
        const uint32_t sc_o = (s6.sc[g >> 1] >> (16 * (g & 1) + 8)) & 0xFFu;    // sub-block 2g+1
        uint32_t lo_e[8], hi_e[8], lo_o[8], hi_o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          scale_split(raw[i] & 0x0F0F0F0Fu, sc_e, lo_e[i], hi_e[i]);
          scale_split((raw[i] >> 4) & 0x0F0F0F0Fu, sc_o, lo_o[i], hi_o[i]);
        }
        unsigned char* t_lo_e = a_tiles + (4 * g + 0) * kTileA;   // tile order: [sub-block][lo, hi]
        unsigned char* t_hi_e = a_tiles + (4 * g + 1) * kTileA;
        unsigned char* t_lo_o = a_tiles + (4 * g + 2) * kTileA;
        unsigned char* t_hi_o = a_tiles + (4 * g + 3) * kTileA;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          *reinterpret_cast<uint4*>(tile_at(t_lo_e, tid, h)) = make_uint4(lo_e[4 * h], lo_e[4 * h + 1], lo_e[4 * h + 2], lo_e[4 * h + 3]);
          *reinterpret_cast<uint4*>(tile_at(t_hi_e, tid, h)) = make_uint4(hi_e[4 * h], hi_e[4 * h + 1], hi_e[4 * h + 2], hi_e[4 * h + 3]);
          *reinterpret_cast<uint4*>(tile_at(t_lo_o, tid, h)) = make_uint4(lo_o[4 * h], lo_o[4 * h + 1], lo_o[4 * h + 2], lo_o[4 * h + 3]);
          *reinterpret_cast<uint4*>(tile_at(t_hi_o, tid, h)) = make_uint4(hi_o[4 * h], hi_o[4 * h + 1], hi_o[4 * h + 2], hi_o[4 * h + 3]);
        }
      }
      {  // min tile: the eight min bytes at k = 0..7, zeros elsewhere
        unsigned char* t_mn = a_tiles + 16 * kTileA;
        *reinterpret_cast<uint4*>(tile_at(t_mn, tid, 0)) = make_uint4(s6.mn[0], s6.mn[1], 0u, 0u);
        *reinterpret_cast<uint4*>(tile_at(t_mn, tid, 1)) = make_uint4(0u, 0u, 0u, 0u);
      }
      // ---- B: activation codes, split sub-block sums and scales of the chunk ----
      for (int i = tid; i < n_mma * 16; i += kGemmRows) {
        const int t = i >> 4, c = i & 15;                  // token slot, 16-byte chunk of the block
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (t < nt) {
          const uint32_t* src = reinterpret_cast<const uint32_t*>(
              xq + static_cast<size_t>(row_off + t0 + t) * xrow_bytes + static_cast<size_t>(blk) * kX8 + 4 + c * 16);
          v = make_uint4(__ldg(src), __ldg(src + 1), __ldg(src + 2), __ldg(src + 3));
        }
        *reinterpret_cast<uint4*>(tile_at(b_tiles + (c >> 1) * kTileB, t, c & 1)) = v;
      }
      for (int t = tid; t < n_mma; t += kGemmRows) {
        uint32_t lo01 = 0, lo23 = 0, hi01 = 0, hi23 = 0;
        float xd = 0.f;
        if (t < nt) {
          const unsigned char* xb = xq + static_cast<size_t>(row_off + t0 + t) * xrow_bytes + static_cast<size_t>(blk) * kX8;
          xd = __uint_as_float(__ldg(reinterpret_cast<const uint32_t*>(xb)));
          const uint32_t* bs = reinterpret_cast<const uint32_t*>(xb + 260);       // 8 x int16
          uint32_t lo[8], hi[8];
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const uint32_t v = __ldg(bs + p);
            const int s0 = static_cast<int16_t>(v & 0xFFFFu), s1 = static_cast<int16_t>(v >> 16);
            lo[2 * p] = s0 & 127; lo[2 * p + 1] = s1 & 127;
            hi[2 * p] = (s0 >> 7) & 0xFF; hi[2 * p + 1] = (s1 >> 7) & 0xFF;
          }
          lo01 = lo[0] | (lo[1] << 8) | (lo[2] << 16) | (lo[3] << 24);
          lo23 = lo[4] | (lo[5] << 8) | (lo[6] << 16) | (lo[7] << 24);
          hi01 = hi[0] | (hi[1] << 8) | (hi[2] << 16) | (hi[3] << 24);
          hi23 = hi[4] | (hi[5] << 8) | (hi[6] << 16) | (hi[7] << 24);
        }
        xd_sm[t] = xd;
        *reinterpret_cast<uint4*>(tile_at(b_tiles + 8 * kTileB, t, 0)) = make_uint4(lo01, lo23, 0u, 0u);
        *reinterpret_cast<uint4*>(tile_at(b_tiles + 8 * kTileB, t, 1)) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(tile_at(b_tiles + 9 * kTileB, t, 0)) = make_uint4(hi01, hi23, 0u, 0u);
        *reinterpret_cast<uint4*>(tile_at(b_tiles + 9 * kTileB, t, 1)) = make_uint4(0u, 0u, 0u, 0u);
      }
      fence_proxy_async();                                 // operand tiles -> visible to the tensor core
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncthreads();
      // ---- MMAs: D0 = sum lo, D1 = sum hi, D2 = min x sums_lo, D3 = min x sums_hi ----
      if (tid == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          const uint64_t db = umma_desc(b_tiles + s * kTileB);
          umma_i8(tmem + 0 * kGemmTok, umma_desc(a_tiles + (2 * s) * kTileA), db, idesc, s > 0);
          umma_i8(tmem + 1 * kGemmTok, umma_desc(a_tiles + (2 * s + 1) * kTileA), db, idesc, s > 0);
        }
        const uint64_t dmn = umma_desc(a_tiles + 16 * kTileA);
        umma_i8(tmem + 2 * kGemmTok, dmn, umma_desc(b_tiles + 8 * kTileB), idesc, 0u);
        umma_i8(tmem + 3 * kGemmTok, dmn, umma_desc(b_tiles + 9 * kTileB), idesc, 0u);
        umma_commit(bar);
      }
      ok = __syncthreads_and(mbar_wait(bar, phase)) != 0;
      phase ^= 1u;
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // ---- epilogue: this thread's row, all tokens of the chunk ----
#pragma unroll
      for (int c0 = 0; c0 < kGemmTok; c0 += 16) {
        if (c0 < n_mma) {
          int lo[16], hi[16], mlo[16], mhi[16];
          tmem_ld16(tmem + lane_base + 0 * kGemmTok + c0, lo);
          tmem_ld16(tmem + lane_base + 1 * kGemmTok + c0, hi);
          tmem_ld16(tmem + lane_base + 2 * kGemmTok + c0, mlo);
          tmem_ld16(tmem + lane_base + 3 * kGemmTok + c0, mhi);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int isum = lo[j] + 128 * hi[j];
            const int msum = mlo[j] + 128 * mhi[j];
            acc[c0 + j] += xd_sm[c0 + j] * (d * static_cast<float>(isum) - dmin * static_cast<float>(msum));
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncthreads();                                     // accumulators and tiles free for the next block
    }
    if (ok && row0 + tid < n_rows) {
#pragma unroll
      for (int t = 0; t < kGemmTok; ++t)
        if (t < nt) y[static_cast<size_t>(row_off + t0 + t) * n_rows + row0 + tid] = f2h(acc[t]);
    }
  }
  if (!ok && tid == 0 && status != nullptr) atomicExch(status, 6);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

}  // namespace
}  // namespace sgr

using namespace sgr;

// y[off[e] + t][r] = W_e[r][:] . xq[off[e] + t][:] for every expert e and its rows
// t < off[e+1] - off[e]; fp16 out, row length n_rows. w_tab[e] == null: zero rows.
SGR_API int sgr_moe_grouped_gemm_i8(const void* const* w_tab, const int* off, const void* xq,
                                    uint16_t* y, int n_rows, int k, int n_expert, void* stream) {
  if (n_expert <= 0 || n_rows <= 0) return kOk;
  if (!w_tab || !off || !xq || !y || k <= 0 || k % kQK != 0) return kErrArg;
  if (reinterpret_cast<uintptr_t>(xq) & 3u) return kErrAlign;
  if (n_expert > 65535) return kErrUnsupported;
  auto kern = grouped_gemm_i8_kernel;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem) != cudaSuccess)
    return kErrLaunch;
  kern<<<dim3((n_rows + kGemmRows - 1) / kGemmRows, n_expert), kGemmRows, kGemmSmem, as_stream(stream)>>>(
      reinterpret_cast<const unsigned char* const*>(w_tab), off, static_cast<const unsigned char*>(xq), y,
      n_rows, k / kQK, status_word());
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}
