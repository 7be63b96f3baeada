// tile.cuh - the one tile routine behind every Q4_K x Q8_K GEMV / small-batch
// GEMM entry point.
//
// A CTA of 128 threads owns `nrows` consecutive rows of one matrix (or of a
// gate/up pair) and a list of activation rows. The weight rows are one
// contiguous byte range, so a single TMA bulk copy per matrix brings them into
// shared memory (16-byte aligned sources; anything else is copied with plain
// loads). Activation rows are re-laid for 16-byte shared loads. Each thread
// then owns one (row, super-block) pair per pass: `lpr` adjacent lanes share a
// row and are summed with shuffles. Many such CTAs are resident per SM, so all
// weight bytes of a decode-sized launch are in flight at once - the kernels are
// HBM-bound and that is what keeps the memory system full.
#pragma once

#include "q4k_common.cuh"

namespace sgr {

constexpr int kTileThreads = 128;

// rows of one matrix a CTA takes for rows of nb super-blocks
__host__ __device__ constexpr int tile_rows(int nb) { return kTileThreads / next_pow2_cap32(nb); }

// dynamic shared memory of a tile CTA
__host__ __device__ constexpr size_t tile_smem(int nmat, int nb, int tt) {
  return 16 + static_cast<size_t>(nmat) * tile_rows(nb) * nb * kW4 + xtile_bytes(tt, nb);
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
  unsigned char* w;     // NMAT x rows x nb x 144
  unsigned char* x;     // XTile storage
};
__device__ __forceinline__ TileSmem tile_smem_view(unsigned char* smem, int nmat, int nb) {
  TileSmem s;
  s.bar = reinterpret_cast<uint64_t*>(smem);
  s.w = smem + 16;
  s.x = s.w + static_cast<size_t>(nmat) * tile_rows(nb) * nb * kW4;
  return s;
}

// Start the weight copies of a tile (call from all threads, before any wait).
// Returns true when the copy went through the mbarrier (TMA), false when it was
// done synchronously with plain loads (caller still needs a __syncthreads).
template <int NMAT>
__device__ __forceinline__ bool tile_load_weights(const TileSmem& s,
                                                  const unsigned char* const (&wsrc)[NMAT],
                                                  int nrows, int nb, int* status) {
  const int tid = threadIdx.x;
  const uint32_t bytes = static_cast<uint32_t>(nrows) * nb * kW4;
  const size_t mat_stride = static_cast<size_t>(tile_rows(nb)) * nb * kW4;
  bool aligned = true;
#pragma unroll
  for (int m = 0; m < NMAT; ++m) aligned = aligned && ((reinterpret_cast<uintptr_t>(wsrc[m]) & 15u) == 0);
  if (aligned) {
    if (tid == 0) {
      mbar_init(s.bar, 1);
      fence_barrier_init();
      fence_proxy_async();                         // make the init visible to the copy engine
      mbar_expect_tx(s.bar, bytes * NMAT);
#pragma unroll
      for (int m = 0; m < NMAT; ++m) bulk_g2s(s.w + m * mat_stride, wsrc[m], bytes, s.bar);
    }
    return true;
  }
#pragma unroll
  for (int m = 0; m < NMAT; ++m)
    copy_unaligned(s.w + m * mat_stride, wsrc[m], static_cast<int>(bytes), tid, kTileThreads);
  (void)status;
  return false;
}

// Compute one token sub-tile. `emit(row, res)` is called by the first lane of
// every row group with res[m][t] = dot of row `row` of matrix m with token t.
template <int NMAT, int TT, typename Emit>
__device__ __forceinline__ void tile_compute(const TileSmem& s, const XTile& xt, int nrows, int nb,
                                             int nt, Emit emit) {
  const int lpr = next_pow2_cap32(nb);
  const int rp = kTileThreads / lpr;               // rows per pass (== tile_rows(nb))
  const int lr = threadIdx.x & (lpr - 1);
  const size_t mat_stride = static_cast<size_t>(tile_rows(nb)) * nb * kW4;
  for (int r0 = 0; r0 < nrows; r0 += rp) {          // uniform trip count: shuffles stay converged
    const int r = r0 + threadIdx.x / lpr;
    float acc[NMAT][TT];
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int t = 0; t < TT; ++t) acc[m][t] = 0.f;
    if (r < nrows) {
      for (int blk = lr; blk < nb; blk += lpr) {
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          const uint4* wb = reinterpret_cast<const uint4*>(
              s.w + m * mat_stride + (static_cast<size_t>(r) * nb + blk) * kW4);
          block_dot<TT>(wb, xt, blk, nt, acc[m]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int t = 0; t < TT; ++t) acc[m][t] = reduce_lanes(acc[m][t], lpr);
    if (r < nrows && lr == 0) emit(r, acc);
  }
}

// Whole tile: load weights once, then walk the token list in sub-tiles of TT.
//   before_x()            runs after the weight copies were issued and before any
//                         activation is read (the place for a dependent-launch wait)
//   stage(xt, t0, nt)     fills the tile with token slots t0 .. t0+nt-1 (all threads)
//   emit(row, t0, nt, res) with res[m][i] for token slot t0 + i
template <int NMAT, int TT, typename BeforeX, typename Stage, typename Emit>
__device__ __forceinline__ void tile_run_staged(unsigned char* smem,
                                                const unsigned char* const (&wsrc)[NMAT],
                                                int nrows, int nb, int ntok, BeforeX before_x,
                                                Stage stage, Emit emit, int* status) {
  const TileSmem s = tile_smem_view(smem, NMAT, nb);
  const XTile xt = xtile_at(s.x, TT, nb);
  const bool tma = tile_load_weights<NMAT>(s, wsrc, nrows, nb, status);
  before_x();
  bool ok = true;
  for (int t0 = 0; t0 < ntok; t0 += TT) {
    const int nt = min(TT, ntok - t0);
    if (t0 > 0) __syncthreads();                    // previous sub-tile fully consumed
    stage(xt, t0, nt);
    __syncthreads();                                // x staged; mbarrier init visible
    if (t0 == 0 && tma) ok = __syncthreads_and(mbar_wait(s.bar, 0)) != 0;
    if (!ok) break;                                 // uniform: every thread saw the same vote
    tile_compute<NMAT, TT>(s, xt, nrows, nb, nt,
                           [&](int r, float (&res)[NMAT][TT]) { emit(r, t0, nt, res); });
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
