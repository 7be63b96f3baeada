// tile.cuh - the one tile routine behind every Q4_K x Q8_K GEMV / small-batch
// GEMM entry point.
//
// A CTA of 128 threads owns `nrows` consecutive rows of one matrix (or of a
// gate/up pair) and a list of activation rows. Weight rows arrive in shared
// memory by TMA bulk copies (16-byte aligned sources; anything else is copied
// with plain loads), one copy per row onto a padded row stride so that shared
// loads of eight different rows never collide on a bank. Activation rows are
// re-laid for 16-byte shared loads. Many such CTAs are resident per SM, so all
// weight bytes of a decode-sized launch are in flight at once - the kernels are
// HBM-bound and that is what keeps the memory system full.
//
// Two compute paths share the staging:
//   TT <= 4  : dp4a. Each thread owns one (row, super-block) pair per pass,
//              `lpr` adjacent lanes share a row and are summed with shuffles.
//   TT == 8  : int8 tensor-core MMA (mma.sync m16n8k32, u8 nibbles x s8 codes,
//              int32 accumulators) over 16-row x 8-token fragments; the per
//              sub-block scales are applied to the int32 partial sums and the
//              min term is a second MMA against the replicated min bytes.
// Both paths compute the same integers, so they agree to fp32 rounding.
#pragma once

#include "q4k_common.cuh"

namespace sgr {

constexpr int kTileThreads = 128;

// rows of one matrix a CTA takes for rows of nb super-blocks
__host__ __device__ constexpr int tile_rows(int nb) { return kTileThreads / next_pow2_cap32(nb); }

// Shared-memory row stride. A row of nb blocks is 36*nb words: for nb a multiple of
// four that is 0 or 16 (mod 32) and eight rows would pile onto one or two bank
// groups, so those rows are padded by 16 bytes (stride 4 mod 8 words, conflict
// free, one bulk copy per row). Other nb keep the packed stride and a single bulk
// copy (conflict free for odd nb, two-way at worst for nb = 2 mod 4).
__host__ __device__ constexpr int tile_wstride(int nb) { return nb * kW4 + ((nb & 3) ? 0 : 16); }

// dynamic shared memory of a tile CTA (the last term is the cross-warp reduction
// scratch of the MMA path)
__host__ __device__ constexpr size_t tile_smem(int nmat, int nb, int tt) {
  return 16 + static_cast<size_t>(nmat) * tile_rows(nb) * tile_wstride(nb) + xtile_bytes(tt, nb) +
         (tt == 8 ? static_cast<size_t>(nmat) * 4 * 128 * 4 : 0);
}

// Cooperative copy for sources that are not 16-byte aligned (the pointer-table
// contract only promises the alignment of the block struct, 2 bytes).
__device__ __forceinline__ void copy_unaligned(unsigned char* dst, const unsigned char* src,
                                               int bytes, int tid, int nthr) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(src);
  if ((a & 3u) == 0) {
    for (int i = tid; i < bytes / 4; i += nthr)
      reinterpret_cast<uint32_t*>(dst)[i] = reinterpret_cast<const uint32_t*>(src)[i];
  } else if ((a & 1u) == 0) {
    for (int i = tid; i < bytes / 2; i += nthr)
      reinterpret_cast<uint16_t*>(dst)[i] = reinterpret_cast<const uint16_t*>(src)[i];
  } else {
    for (int i = tid; i < bytes; i += nthr) dst[i] = src[i];
  }
}

// Shared-memory view of a tile CTA.
struct TileSmem {
  uint64_t* bar;
  unsigned char* w;     // NMAT x tile_rows x wstride
  unsigned char* x;     // XTile storage
  float* red;           // MMA path: [NMAT][4 warps][128] partial sums
  int wstride;
  int mat_stride;
};
__device__ __forceinline__ TileSmem tile_smem_view(unsigned char* smem, int nmat, int nb, int tt) {
  TileSmem s;
  s.wstride = tile_wstride(nb);
  s.mat_stride = tile_rows(nb) * s.wstride;
  s.bar = reinterpret_cast<uint64_t*>(smem);
  s.w = smem + 16;
  s.x = s.w + static_cast<size_t>(nmat) * s.mat_stride;
  s.red = reinterpret_cast<float*>(s.x + xtile_bytes(tt, nb));
  return s;
}

// Start the weight copies of a tile (call from all threads, before any wait).
// Returns true when the copies go through the mbarrier (TMA), false when they
// were done synchronously with plain loads (caller still needs a __syncthreads).
template <int NMAT>
__device__ __forceinline__ bool tile_load_weights(const TileSmem& s,
                                                  const unsigned char* const (&wsrc)[NMAT],
                                                  int nrows, int nb) {
  const int tid = threadIdx.x;
  const uint32_t row_bytes = static_cast<uint32_t>(nb) * kW4;
  bool aligned = true;
#pragma unroll
  for (int m = 0; m < NMAT; ++m) aligned = aligned && ((reinterpret_cast<uintptr_t>(wsrc[m]) & 15u) == 0);
  if (aligned) {
    if (tid == 0) {
      mbar_init(s.bar, 1);
      fence_barrier_init();
      fence_proxy_async();                         // make the init visible to the copy engine
      mbar_expect_tx(s.bar, row_bytes * nrows * NMAT);
    }
    __syncthreads();
    if (s.wstride == static_cast<int>(row_bytes)) {
      if (tid < NMAT) bulk_g2s(s.w + tid * s.mat_stride, wsrc[tid], row_bytes * nrows, s.bar);
    } else {
      for (int i = tid; i < nrows * NMAT; i += kTileThreads) {
        const int m = i / nrows, r = i - m * nrows;
        bulk_g2s(s.w + m * s.mat_stride + r * s.wstride, wsrc[m] + static_cast<size_t>(r) * row_bytes,
                 row_bytes, s.bar);
      }
    }
    return true;
  }
  for (int i = 0; i < nrows * NMAT; ++i) {
    const int m = i / nrows, r = i - m * nrows;
    copy_unaligned(s.w + m * s.mat_stride + r * s.wstride, wsrc[m] + static_cast<size_t>(r) * row_bytes,
                   static_cast<int>(row_bytes), tid, kTileThreads);
  }
  return false;
}

// ---- dp4a path ------------------------------------------------------------------------
// emit(row, slot, v) is called once per (row, token slot) with v[m] = the dot of
// that row of matrix m with that token.
template <int NMAT, int TT, typename Emit>
__device__ __forceinline__ void tile_compute_dp4a(const TileSmem& s, const XTile& xt, int nrows,
                                                  int nb, int t0, int nt, Emit emit) {
  const int lpr = next_pow2_cap32(nb);
  const int rp = kTileThreads / lpr;               // rows per pass (== tile_rows(nb))
  const int lr = threadIdx.x & (lpr - 1);
  for (int r0 = 0; r0 < nrows; r0 += rp) {          // uniform trip count: shuffles stay converged
    const int r = r0 + threadIdx.x / lpr;
    float acc[NMAT][TT];
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int t = 0; t < TT; ++t) acc[m][t] = 0.f;
    if (r < nrows) {
      for (int blk = lr; blk < nb; blk += lpr) {
        const uint4* wb[NMAT];
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
          wb[m] = reinterpret_cast<const uint4*>(s.w + m * s.mat_stride + r * s.wstride + blk * kW4);
        block_dot<NMAT, TT>(wb, xt, blk, nt, acc);
      }
    }
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int t = 0; t < TT; ++t) acc[m][t] = reduce_lanes(acc[m][t], lpr);
    if (r < nrows && lr == 0) {
#pragma unroll
      for (int t = 0; t < TT; ++t)
        if (t < nt) {
          float v[NMAT];
#pragma unroll
          for (int m = 0; m < NMAT; ++m) v[m] = acc[m][t];
          emit(r, t0 + t, v);
        }
    }
  }
}

// ---- tensor-core path --------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}
// D(16x8, s32) = A(16x32, u8) * B(32x8, s8) + C
__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1, const int (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%12,%13};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]),
        "r"(c[2]), "r"(c[3]));
}

// One warp, rows [r0, r0+16) of every matrix, blocks blk0, blk0+bstep, ... < nb,
// NT groups of eight staged tokens. Fragment ownership (PTX m16n8k32): lane =
// 4*gid + tig holds results for rows r0+gid and r0+gid+8, tokens 8*n + 2*tig and
// 8*n + 2*tig + 1: acc[m][n][0] = (gid, 2tig), [1] = (gid, 2tig+1),
// [2] = (gid+8, 2tig), [3] = (gid+8, 2tig+1).
template <int NMAT, int NT>
__device__ __forceinline__ void warp_mma_rows(const unsigned char* w, int wstride, int mat_stride,
                                              const XTile& xt, int r0, int nrows, int nb, int blk0,
                                              int bstep, float (&acc)[NMAT][NT][4]) {
  const int lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  // ldmatrix row addresses. A: matrices 0..3 = (rows 0-7, k 0-15), (rows 8-15, k 0-15),
  // (rows 0-7, k 16-31), (rows 8-15, k 16-31). B: (tokens, k 0-15 / 16-31) of sub-block
  // 2g, then of sub-block 2g+1.
  const int a_row = min(r0 + (lane & 7) + ((lane >> 3) & 1) * 8, nrows - 1);   // clamp ragged tiles
  const int a_koff = (lane >> 4) * 16;
  const int b_tok = lane & 7;
  const int b_off = (lane >> 3) * 16;          // 0,16 -> sub-block 2g; 32,48 -> sub-block 2g+1
  const int row_lo = min(r0 + gid, nrows - 1), row_hi = min(r0 + gid + 8, nrows - 1);
#pragma unroll
  for (int m = 0; m < NMAT; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[m][n][j] = 0.f;

  for (int blk = blk0; blk < nb; blk += bstep) {
    int isum[NMAT][NT][4], msum[NMAT][NT][4];
    Scales6 s_lo[NMAT], s_hi[NMAT];
    float d_lo[NMAT], d_hi[NMAT], m_lo[NMAT], m_hi[NMAT];
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
      const unsigned char* wm = w + m * mat_stride + blk * kW4;
      const uint4 h0 = *reinterpret_cast<const uint4*>(wm + row_lo * wstride);
      const uint4 h1 = *reinterpret_cast<const uint4*>(wm + row_hi * wstride);
      // d enters as d/16 (exact): the integer sums below carry a factor 16
      d_lo[m] = 0.0625f * __half2float(__ushort_as_half(static_cast<uint16_t>(h0.x & 0xFFFFu)));
      m_lo[m] = __half2float(__ushort_as_half(static_cast<uint16_t>(h0.x >> 16)));
      d_hi[m] = 0.0625f * __half2float(__ushort_as_half(static_cast<uint16_t>(h1.x & 0xFFFFu)));
      m_hi[m] = __half2float(__ushort_as_half(static_cast<uint16_t>(h1.x >> 16)));
      s_lo[m] = unpack_scales6(h0.y, h0.z, h0.w);
      s_hi[m] = unpack_scales6(h1.y, h1.z, h1.w);
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) { isum[m][n][j] = 0; msum[m][n][j] = 0; }
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t b[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) ldmatrix_x4(b[n], xt.code_ptr(8 * n + b_tok, blk, 2 * g) + b_off);
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        uint32_t raw[4];
        ldmatrix_x4(raw, w + m * mat_stride + a_row * wstride + blk * kW4 + 16 + g * 32 + a_koff);
        // The high nibbles stay where they are: 16*q still fits u8, so the odd
        // sub-block's dots come out 16-fold. The even sub-block's scale is taken
        // 16-fold instead and the common factor leaves with the final fp32 multiply.
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          lo[j] = raw[j] & 0x0F0F0F0Fu;
          hi[j] = raw[j] & 0xF0F0F0F0u;
        }
        const int sh = 16 * (g & 1);
        const int sc0_lo = ((s_lo[m].sc[g >> 1] >> sh) & 0xFF) << 4, sc1_lo = (s_lo[m].sc[g >> 1] >> (sh + 8)) & 0xFF;
        const int sc0_hi = ((s_hi[m].sc[g >> 1] >> sh) & 0xFF) << 4, sc1_hi = (s_hi[m].sc[g >> 1] >> (sh + 8)) & 0xFF;
        const int zero[4] = {0, 0, 0, 0};
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          int c0[4], c1[4];
          mma_u8s8(c0, lo, b[n][0], b[n][1], zero);        // sub-block 2g
          mma_u8s8(c1, hi, b[n][2], b[n][3], zero);        // sub-block 2g+1
          isum[m][n][0] += sc0_lo * c0[0] + sc1_lo * c1[0];
          isum[m][n][1] += sc0_lo * c0[1] + sc1_lo * c1[1];
          isum[m][n][2] += sc0_hi * c0[2] + sc1_hi * c1[2];
          isum[m][n][3] += sc0_hi * c0[3] + sc1_hi * c1[3];
        }
      }
    }
    // Min term sum_s mn[s]*bsum[s] as one tiny contraction per block: the eight min
    // bytes of a row are k = 0..7 of an A fragment, the sub-block sums split as
    // bsum = 128*hi + lo are two B fragments (lo in 0..127 and hi in -32..31 fit s8).
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      uint32_t blo = 0u, bhi = 0u;
      if (tig < 2) {
        const int8_t* sp = xt.split_sums(8 * n + gid, blk);
        blo = *reinterpret_cast<const uint32_t*>(sp + 4 * tig);
        bhi = *reinterpret_cast<const uint32_t*>(sp + 8 + 4 * tig);
      }
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        const uint32_t a_lo = tig == 0 ? s_lo[m].mn[0] : (tig == 1 ? s_lo[m].mn[1] : 0u);
        const uint32_t a_hi = tig == 0 ? s_hi[m].mn[0] : (tig == 1 ? s_hi[m].mn[1] : 0u);
        const uint32_t ma[4] = {a_lo, a_hi, 0u, 0u};
        const int zero[4] = {0, 0, 0, 0};
        int dl[4], dh[4];
        mma_u8s8(dl, ma, blo, 0u, zero);
        mma_u8s8(dh, ma, bhi, 0u, zero);
#pragma unroll
        for (int j = 0; j < 4; ++j) msum[m][n][j] = dl[j] + 128 * dh[j];
      }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const float xd0 = xt.scale(8 * n + 2 * tig, blk), xd1 = xt.scale(8 * n + 2 * tig + 1, blk);
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        acc[m][n][0] += xd0 * (d_lo[m] * static_cast<float>(isum[m][n][0]) - m_lo[m] * static_cast<float>(msum[m][n][0]));
        acc[m][n][1] += xd1 * (d_lo[m] * static_cast<float>(isum[m][n][1]) - m_lo[m] * static_cast<float>(msum[m][n][1]));
        acc[m][n][2] += xd0 * (d_hi[m] * static_cast<float>(isum[m][n][2]) - m_hi[m] * static_cast<float>(msum[m][n][2]));
        acc[m][n][3] += xd1 * (d_hi[m] * static_cast<float>(isum[m][n][3]) - m_hi[m] * static_cast<float>(msum[m][n][3]));
      }
    }
  }
}

// One super-block of sixteen weight rows that need not be adjacent: `a_ptr` is this
// lane's ldmatrix row address (start of the row's block + 16 + 16 * (lane >> 4)),
// `h_lo` / `h_hi` the blocks of the rows whose results this lane owns (fragment
// rows gid and gid + 8). Activations: block 0 of a tile staged with nb == 1 (codes, int16
// sums and scales; the split sums of the staged layout are not used).
// Accumulates into acc (same ownership as warp_mma_rows).
// `loaded()` runs once the weight bytes are in registers: from then on only the activations are read.
template <int NT, int NACC, typename Loaded>
__device__ __forceinline__ void warp_mma_block(const unsigned char* a_ptr, const unsigned char* h_lo,
                                               const unsigned char* h_hi, const XTile& xt,
                                               float (&acc)[NACC][4], Loaded loaded) {
  static_assert(NT <= NACC, "accumulator rows");
  const int lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int b_tok = lane & 7;
  const int b_off = (lane >> 3) * 16;
  const uint4 h0 = *reinterpret_cast<const uint4*>(h_lo);
  const uint4 h1 = *reinterpret_cast<const uint4*>(h_hi);
  const float d_lo = 0.0625f * __half2float(__ushort_as_half(static_cast<uint16_t>(h0.x & 0xFFFFu)));
  const float m_lo = __half2float(__ushort_as_half(static_cast<uint16_t>(h0.x >> 16)));
  const float d_hi = 0.0625f * __half2float(__ushort_as_half(static_cast<uint16_t>(h1.x & 0xFFFFu)));
  const float m_hi = __half2float(__ushort_as_half(static_cast<uint16_t>(h1.x >> 16)));
  const Scales6 s_lo = unpack_scales6(h0.y, h0.z, h0.w);
  const Scales6 s_hi = unpack_scales6(h1.y, h1.z, h1.w);
  uint32_t raw[4][4];
#pragma unroll
  for (int g = 0; g < 4; ++g) ldmatrix_x4(raw[g], a_ptr + g * 32);
  loaded();
  int isum[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) isum[n][j] = 0;
  const int zero[4] = {0, 0, 0, 0};
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint32_t b[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) ldmatrix_x4(b[n], xt.code_ptr(8 * n + b_tok, 0, 2 * g) + b_off);
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo[j] = raw[g][j] & 0x0F0F0F0Fu;
      hi[j] = raw[g][j] & 0xF0F0F0F0u;            // 16 * q: see warp_mma_rows
    }
    const int sh = 16 * (g & 1);
    const int sc0_lo = ((s_lo.sc[g >> 1] >> sh) & 0xFF) << 4, sc1_lo = (s_lo.sc[g >> 1] >> (sh + 8)) & 0xFF;
    const int sc0_hi = ((s_hi.sc[g >> 1] >> sh) & 0xFF) << 4, sc1_hi = (s_hi.sc[g >> 1] >> (sh + 8)) & 0xFF;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      int c0[4], c1[4];
      mma_u8s8(c0, lo, b[n][0], b[n][1], zero);
      mma_u8s8(c1, hi, b[n][2], b[n][3], zero);
      isum[n][0] += sc0_lo * c0[0] + sc1_lo * c1[0];
      isum[n][1] += sc0_lo * c0[1] + sc1_lo * c1[1];
      isum[n][2] += sc0_hi * c0[2] + sc1_hi * c1[2];
      isum[n][3] += sc0_hi * c0[3] + sc1_hi * c1[3];
    }
  }
  const uint32_t a_lo = tig == 0 ? s_lo.mn[0] : (tig == 1 ? s_lo.mn[1] : 0u);
  const uint32_t a_hi = tig == 0 ? s_hi.mn[0] : (tig == 1 ? s_hi.mn[1] : 0u);
  const uint32_t ma[4] = {a_lo, a_hi, 0u, 0u};
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    // sub-block sums 4*tig .. 4*tig+3 of token 8n+gid, split as bsum = 128*hi + lo
    // (lo in 0..127, hi in -32..31) straight from the int16 sums
    uint32_t blo = 0u, bhi = 0u;
    if (tig < 2) {
      const uint2 sv = *reinterpret_cast<const uint2*>(xt.bs + static_cast<size_t>(8 * n + gid) * 8 + 4 * tig);
      blo = __byte_perm(sv.x & 0x007F007Fu, sv.y & 0x007F007Fu, 0x6420);
      bhi = __byte_perm((sv.x >> 7) & 0x00FF00FFu, (sv.y >> 7) & 0x00FF00FFu, 0x6420);
    }
    int dl[4], dh[4];
    mma_u8s8(dl, ma, blo, 0u, zero);
    mma_u8s8(dh, ma, bhi, 0u, zero);
    const float xd0 = xt.scale(8 * n + 2 * tig, 0), xd1 = xt.scale(8 * n + 2 * tig + 1, 0);
    acc[n][0] += xd0 * (d_lo * static_cast<float>(isum[n][0]) - m_lo * static_cast<float>(dl[0] + 128 * dh[0]));
    acc[n][1] += xd1 * (d_lo * static_cast<float>(isum[n][1]) - m_lo * static_cast<float>(dl[1] + 128 * dh[1]));
    acc[n][2] += xd0 * (d_hi * static_cast<float>(isum[n][2]) - m_hi * static_cast<float>(dl[2] + 128 * dh[2]));
    acc[n][3] += xd1 * (d_hi * static_cast<float>(isum[n][3]) - m_hi * static_cast<float>(dl[3] + 128 * dh[3]));
  }
}

// Half a super-block (sub-blocks 4*half .. 4*half+3) of one weight row against up to
// TT staged tokens (block 0 of a tile staged with nb == 1), for a pair of adjacent
// lanes that share the row: the integer sums of the two halves are added across
// the pair before the one fp32 rounding, so the result equals block_dot's.
template <int TT>
__device__ __forceinline__ void half_block_dot_regs(const uint4 hdr, const uint4 (&wq)[4], int half, const XTile& xt,
                                                    int nt, float (&acc)[TT]) {
  const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x & 0xFFFFu)));
  const float dmin = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x >> 16)));
  const Scales6 s6 = unpack_scales6(hdr.y, hdr.z, hdr.w);
  const uint32_t scw = half ? s6.sc[1] : s6.sc[0];
  const uint32_t mnw = half ? s6.mn[1] : s6.mn[0];
  int isum[TT];
#pragma unroll
  for (int t = 0; t < TT; ++t) isum[t] = 0;
#pragma unroll
  for (int gg = 0; gg < 2; ++gg) {
    const int g = 2 * half + gg;
    const uint4 q0 = wq[2 * gg], q1 = wq[2 * gg + 1];
    const uint32_t raw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo[i] = raw[i] & 0x0F0F0F0Fu;
      hi[i] = (raw[i] >> 4) & 0x0F0F0F0Fu;
    }
    const int sc_lo = (scw >> (16 * gg)) & 0xFF, sc_hi = (scw >> (16 * gg + 8)) & 0xFF;
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      if (t < nt) {
        const uint4* xa = xt.codes(t, 0, 2 * g);
        const uint4 x0 = xa[0], x1 = xa[1], x2 = xa[2], x3 = xa[3];
        isum[t] += sc_lo * dot8(lo, x0, x1) + sc_hi * dot8(hi, x2, x3);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    if (t < nt) {                               // nt is warp-uniform: the shuffles stay converged
      const uint4 bs = xt.sums(t, 0);
      int msum = __dp2a_lo(static_cast<int>(half ? bs.z : bs.x), static_cast<int>(mnw), 0);
      msum = __dp2a_hi(static_cast<int>(half ? bs.w : bs.y), static_cast<int>(mnw), msum);
      const int is = isum[t] + __shfl_xor_sync(0xFFFFFFFFu, isum[t], 1);
      const int ms = msum + __shfl_xor_sync(0xFFFFFFFFu, msum, 1);
      acc[t] += xt.scale(t, 0) * (d * static_cast<float>(is) - dmin * static_cast<float>(ms));
    }
  }
}

// The same from shared memory: the lane's half of the block is read first, so a caller that wants
// to hand the weight bytes back before the arithmetic can use the two steps separately.
__device__ __forceinline__ void half_block_load(const uint4* wrow, int half, uint4& hdr, uint4 (&wq)[4]) {
  hdr = wrow[0];
#pragma unroll
  for (int i = 0; i < 4; ++i) wq[i] = wrow[1 + 4 * half + i];
}
template <int TT>
__device__ __forceinline__ void half_block_dot(const uint4* wrow, int half, const XTile& xt, int nt,
                                               float (&acc)[TT]) {
  uint4 hdr, wq[4];
  half_block_load(wrow, half, hdr, wq);
  half_block_dot_regs<TT>(hdr, wq, half, xt, nt, acc);
}

// Four warps cover the tile: with at least four 16-row groups each warp takes
// groups w, w+4, ...; with fewer, the warps of a group split the super-blocks and
// their partial sums meet in shared memory (fixed order, so results are
// reproducible).
template <int NMAT, typename Emit>
__device__ __forceinline__ void tile_compute_mma(const TileSmem& s, const XTile& xt, int nrows,
                                                 int nb, int t0, int nt, Emit emit) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int groups = (nrows + 15) / 16;
  auto emit_frag = [&](int r0, const float (&a)[NMAT][1][4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = r0 + gid + (j >> 1) * 8, t = 2 * tig + (j & 1);
      if (r < nrows && t < nt) {
        float v[NMAT];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) v[m] = a[m][0][j];
        emit(r, t0 + t, v);
      }
    }
  };
  if (groups >= 4) {
    for (int grp = warp; grp < groups; grp += 4) {
      float acc[NMAT][1][4];
      warp_mma_rows<NMAT, 1>(s.w, s.wstride, s.mat_stride, xt, grp * 16, nrows, nb, 0, 1, acc);
      emit_frag(grp * 16, acc);
    }
    return;
  }
  // groups in {1, 2, 3}: wpg warps per group split the blocks
  const int wpg = groups == 1 ? 4 : (groups == 2 ? 2 : 1);
  const int grp = warp / wpg, part = warp - grp * wpg;
  float acc[NMAT][1][4];
  const bool active = grp < groups;
  if (active)
    warp_mma_rows<NMAT, 1>(s.w, s.wstride, s.mat_stride, xt, grp * 16, nrows, nb, part, wpg, acc);
  if (wpg == 1) {
    if (active) emit_frag(grp * 16, acc);
    if (groups == 3 && warp == 3) { /* idle warp */ }
    return;
  }
  if (active) {
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) s.red[(m * 4 + warp) * 128 + j * 32 + lane] = acc[m][0][j];
  }
  __syncthreads();
  if (active && part == 0) {
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = acc[m][0][j];
        for (int p = 1; p < wpg; ++p) v += s.red[(m * 4 + warp + p) * 128 + j * 32 + lane];
        acc[m][0][j] = v;
      }
    emit_frag(grp * 16, acc);
  }
}

template <int NMAT, int TT, typename Emit>
__device__ __forceinline__ void tile_compute(const TileSmem& s, const XTile& xt, int nrows, int nb,
                                             int t0, int nt, Emit emit) {
  if constexpr (TT == 8) tile_compute_mma<NMAT>(s, xt, nrows, nb, t0, nt, emit);
  else tile_compute_dp4a<NMAT, TT>(s, xt, nrows, nb, t0, nt, emit);
}

// Whole tile: load weights once, then walk the token list in sub-tiles of TT.
//   before_x()          runs after the weight copies were issued and before any
//                       activation is read (the place for a dependent-launch wait)
//   stage(xt, t0, nt)   fills the tile with token slots t0 .. t0+nt-1 (all threads)
//   emit(row, slot, v)  once per (row, token slot), v[m] per matrix
template <int NMAT, int TT, typename BeforeX, typename Stage, typename Emit>
__device__ __forceinline__ void tile_run_staged(unsigned char* smem,
                                                const unsigned char* const (&wsrc)[NMAT],
                                                int nrows, int nb, int ntok, BeforeX before_x,
                                                Stage stage, Emit emit, int* status) {
  const TileSmem s = tile_smem_view(smem, NMAT, nb, TT);
  const XTile xt = xtile_at(s.x, TT, nb);
  const bool tma = tile_load_weights<NMAT>(s, wsrc, nrows, nb);
  before_x();
  bool ok = true;
  for (int t0 = 0; t0 < ntok; t0 += TT) {
    const int nt = min(TT, ntok - t0);
    if (t0 > 0) __syncthreads();                    // previous sub-tile fully consumed
    stage(xt, t0, nt);
    __syncthreads();                                // x staged (and plain-copied weights visible)
    if (t0 == 0 && tma) ok = __syncthreads_and(mbar_wait(s.bar, 0)) != 0;
    if (!ok) break;                                 // uniform: every thread saw the same vote
    tile_compute<NMAT, TT>(s, xt, nrows, nb, t0, nt, emit);
  }
  if (!ok && threadIdx.x == 0 && status != nullptr) atomicExch(status, 1);
}

// Same, with the activations taken from packed Q8_K rows in global memory:
//   xrow(t) -> pointer to the row of token slot t (0 <= t < ntok)
template <int NMAT, int TT, typename XRow, typename Emit>
__device__ __forceinline__ void tile_run(unsigned char* smem,
                                         const unsigned char* const (&wsrc)[NMAT], int nrows,
                                         int nb, int ntok, XRow xrow, Emit emit, int* status) {
  tile_run_staged<NMAT, TT>(
      smem, wsrc, nrows, nb, ntok, [] {},
      [&](const XTile& xt, int t0, int nt) {
        xtile_stage(xt, nt, [&](int t) { return xrow(t0 + t); }, threadIdx.x, kTileThreads);
      },
      emit, status);
}

}  // namespace sgr
