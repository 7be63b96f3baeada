// q4k_common.cuh - block formats and the per-block dot engine shared by every
// Q4_K x Q8_K kernel of the library (sm_100a only).
//
// Formats follow the reference's include/sager/kernels/q4_k.hpp:45-63:
//   Q4_K super-block, 144 B / 256 weights: fp16 d, fp16 dmin, 12 B of packed
//   6-bit scales and mins, 128 B of nibbles (four 32-byte groups; group g's low
//   nibbles are sub-block 2g, its high nibbles sub-block 2g+1).
//   Q8_K activation block, 276 B packed / 256 values: fp32 d, 256 int8 codes,
//   8 int16 sub-block sums.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sgr {

constexpr int kQK = 256;          // weights per super-block
constexpr int kW4 = 144;          // bytes per Q4_K super-block
constexpr int kX8 = 276;          // bytes per Q8_K block (packed)
constexpr int kXqStride = 272;    // staged int8 codes per block, padded: 68 words -> the
                                  // 8 lanes of a row hit 8 distinct 4-bank groups

// Error codes returned by the C entry points.
enum : int {
  kOk = 0,
  kErrArg = 1,        // null pointer, non-positive size, k % 256 != 0
  kErrAlign = 2,      // a pointer that must be 4-byte (activations) or 2-byte aligned is not
  kErrUnsupported = 3,
  kErrLaunch = 4,     // the CUDA runtime refused the launch
  kErrGeometry = 5,   // a fused entry point was given a shape it was not built for
  kErrStaticLimit = 6,  // the allocation-free entry point: shape exceeds the built-in scratch
};

__device__ __forceinline__ float h2f(uint16_t h) {
  return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ uint16_t f2h(float f) {
  return __half_as_ushort(__float2half(f));   // round to nearest even
}

// ---- mbarrier + bulk copy (TMA without a tensor map, one CTA per copy) --------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (each poll itself blocks for a
// hardware-defined slice) and reports failure, so a lost copy can never hang
// the GPU; callers raise the status word and skip the tile.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (int it = 0; it < (1 << 22); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
__device__ __forceinline__ void mbar_arrive_one(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// global -> shared bulk copy; src and dst 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// Programmatic dependent launch: wait for the previous kernel in the stream
// (no-op when the launch carried no programmatic attribute).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- staged activations -------------------------------------------------------
// One tile of up to TT Q8_K rows re-laid for 16-byte shared loads:
//   qs   [TT][tok_stride]   int8 codes, 272 bytes per block (256 used)
//   bs   [TT][nb][8]        int16 sub-block sums (one uint4 per block)
//   bl   [TT][nb][16]       the same sums split as bsum = 128*hi + lo: eight lo bytes
//                           (0..127) then eight hi bytes (-32..31), for the MMA path
//   d    [TT][nb]           fp32 scales
// Blocks are 68 words apart and token rows tok_stride/4 = 4 (mod 8) words apart,
// so eight lanes that read the same 16 bytes of eight different blocks - or of
// eight different tokens - touch eight distinct 4-bank groups.
__host__ __device__ constexpr int xtile_tok_stride(int nb) {
  return nb * kXqStride + ((nb & 1) ? 0 : 16);
}

struct XTile {
  int8_t* qs;
  int16_t* bs;
  int8_t* bl;
  float* d;
  int nb;
  int tok_stride;
  int d_step;          // floats between the scales of consecutive token rows (nb when packed)
  int mid_pad;         // bytes between the codes of sub-blocks 3 and 4 of a block (0, or 16 when the
                       // block's own padding sits in the middle: lanes that read sub-blocks s and
                       // s + 4 of one row at once then hit different banks)
  __device__ __forceinline__ const int8_t* code_ptr(int t, int blk, int sb) const {
    return qs + static_cast<size_t>(t) * tok_stride + blk * kXqStride + sb * 32 + (sb >> 2) * mid_pad;
  }
  __device__ __forceinline__ const uint4* codes(int t, int blk, int sb) const {
    return reinterpret_cast<const uint4*>(code_ptr(t, blk, sb));
  }
  __device__ __forceinline__ uint4 sums(int t, int blk) const {
    return *reinterpret_cast<const uint4*>(bs + (static_cast<size_t>(t) * nb + blk) * 8);
  }
  __device__ __forceinline__ float scale(int t, int blk) const { return d[t * d_step + blk]; }
  __device__ __forceinline__ const int8_t* split_sums(int t, int blk) const {
    return bl + (static_cast<size_t>(t) * nb + blk) * 16;
  }
  // store sub-block sums 2p and 2p+1 (packed in v as two int16) in both forms
  __device__ __forceinline__ void put_sum_pair(int t, int blk, int p, uint32_t v) const {
    reinterpret_cast<uint32_t*>(bs + (static_cast<size_t>(t) * nb + blk) * 8)[p] = v;
    const int s0 = static_cast<int16_t>(v & 0xFFFFu), s1 = static_cast<int16_t>(v >> 16);
    int8_t* q = bl + (static_cast<size_t>(t) * nb + blk) * 16;
    reinterpret_cast<uint16_t*>(q)[p] = static_cast<uint16_t>((s0 & 127) | ((s1 & 127) << 8));
    reinterpret_cast<uint16_t*>(q + 8)[p] = static_cast<uint16_t>(((s0 >> 7) & 0xFF) | (((s1 >> 7) & 0xFF) << 8));
  }
};

__host__ __device__ constexpr size_t xtile_bytes(int tt, int nb) {
  return static_cast<size_t>(tt) * (xtile_tok_stride(nb) + nb * (16 + 16 + 4));
}

__device__ __forceinline__ XTile xtile_at(unsigned char* base, int tt, int nb) {
  XTile x;
  x.nb = nb;
  x.d_step = nb;
  x.mid_pad = 0;
  x.tok_stride = xtile_tok_stride(nb);
  x.qs = reinterpret_cast<int8_t*>(base);
  x.bs = reinterpret_cast<int16_t*>(base + static_cast<size_t>(tt) * x.tok_stride);
  x.bl = reinterpret_cast<int8_t*>(base + static_cast<size_t>(tt) * (x.tok_stride + nb * 16));
  x.d = reinterpret_cast<float*>(base + static_cast<size_t>(tt) * (x.tok_stride + nb * 32));
  return x;
}

// Copy `nt` packed Q8_K rows (4-byte aligned, 276*nb bytes each) into the tile.
// row_of(t) gives the source row pointer of tile slot t.
template <typename RowOf>
__device__ __forceinline__ void xtile_stage(const XTile& xt, int nt, RowOf row_of, int tid,
                                            int nthr) {
  const int words_per_blk = kX8 / 4;   // 69: [0]=d, [1..64]=codes, [65..68]=bsums
  const int total = nt * xt.nb * words_per_blk;
  for (int i = tid; i < total; i += nthr) {
    const int t = i / (xt.nb * words_per_blk);
    const int r = i - t * (xt.nb * words_per_blk);
    const int blk = r / words_per_blk;
    const int w = r - blk * words_per_blk;
    const uint32_t v = reinterpret_cast<const uint32_t*>(row_of(t))[blk * words_per_blk + w];
    if (w == 0) {
      xt.d[t * xt.nb + blk] = __uint_as_float(v);
    } else if (w <= 64) {
      reinterpret_cast<uint32_t*>(xt.qs + static_cast<size_t>(t) * xt.tok_stride + blk * kXqStride)[w - 1] = v;
    } else {
      xt.put_sum_pair(t, blk, w - 65, v);
    }
  }
}

// ---- the dot engine -------------------------------------------------------------
// 16 six-bit values of one block, packed one per byte:
//   sc[0] = scales 0..3, sc[1] = scales 4..7, mn[0] = mins 0..3, mn[1] = mins 4..7
// (bit layout: get_scale_min_k4, q4_k.hpp:110-118 of the reference).
struct Scales6 {
  uint32_t sc[2];
  uint32_t mn[2];
};
__device__ __forceinline__ Scales6 unpack_scales6(uint32_t w0, uint32_t w1, uint32_t w2) {
  Scales6 s;
  s.sc[0] = w0 & 0x3F3F3F3Fu;
  s.mn[0] = w1 & 0x3F3F3F3Fu;
  s.sc[1] = (w2 & 0x0F0F0F0Fu) | ((w0 >> 2) & 0x30303030u);
  s.mn[1] = ((w2 >> 4) & 0x0F0F0F0Fu) | ((w1 >> 2) & 0x30303030u);
  return s;
}

__device__ __forceinline__ int dot8(const uint32_t (&w)[8], const uint4& a, const uint4& b) {
  int acc = __dp4a(static_cast<int>(w[0]), static_cast<int>(a.x), 0);
  acc = __dp4a(static_cast<int>(w[1]), static_cast<int>(a.y), acc);
  acc = __dp4a(static_cast<int>(w[2]), static_cast<int>(a.z), acc);
  acc = __dp4a(static_cast<int>(w[3]), static_cast<int>(a.w), acc);
  acc = __dp4a(static_cast<int>(w[4]), static_cast<int>(b.x), acc);
  acc = __dp4a(static_cast<int>(w[5]), static_cast<int>(b.y), acc);
  acc = __dp4a(static_cast<int>(w[6]), static_cast<int>(b.z), acc);
  acc = __dp4a(static_cast<int>(w[7]), static_cast<int>(b.w), acc);
  return acc;
}

// The same block position `blk` of NMAT weight rows (blocks in shared memory,
// 16-byte aligned) against `nt` staged activation rows; the activation codes are
// loaded once and used for every matrix. For every token the eight sub-block dots
// are integers (exact); they are combined as
//     acc += xd * ( d * sum_s sc[s]*dot[s]  -  dmin * sum_s mn[s]*bsum[s] )
// with both inner sums held in int32 (|.| <= 8*63*60960 < 2^25), so only the last
// line rounds. The reference rounds sd = d*sc first and sums eight fp32 terms
// (q4_k.cu:57-91, q4_avx2.cpp:124-145); the two agree to fp32 rounding.
// If dots_out != nullptr the raw sub-block dots of matrix 0, token 0 are stored.
template <int NMAT, int TT>
__device__ __forceinline__ void block_dot(const uint4* const (&wblk)[NMAT], const XTile& xt,
                                          int blk, int nt, float (&acc)[NMAT][TT],
                                          int* dots_out = nullptr) {
  float d[NMAT], dmin[NMAT];
  Scales6 s6[NMAT];
  int isum[NMAT][TT];
#pragma unroll
  for (int m = 0; m < NMAT; ++m) {
    const uint4 hdr = wblk[m][0];
    d[m] = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x & 0xFFFFu)));
    dmin[m] = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x >> 16)));
    s6[m] = unpack_scales6(hdr.y, hdr.z, hdr.w);
#pragma unroll
    for (int t = 0; t < TT; ++t) isum[m][t] = 0;
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint32_t lo[NMAT][8], hi[NMAT][8];
    int sc_lo[NMAT], sc_hi[NMAT];
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
      const uint4 q0 = wblk[m][1 + 2 * g];
      const uint4 q1 = wblk[m][2 + 2 * g];
      const uint32_t raw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        lo[m][i] = raw[i] & 0x0F0F0F0Fu;
        hi[m][i] = (raw[i] >> 4) & 0x0F0F0F0Fu;
      }
      sc_lo[m] = (s6[m].sc[g >> 1] >> (16 * (g & 1))) & 0xFF;       // scale of sub-block 2g
      sc_hi[m] = (s6[m].sc[g >> 1] >> (16 * (g & 1) + 8)) & 0xFF;   // scale of sub-block 2g+1
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      if (t < nt) {
        const uint4* xa = xt.codes(t, blk, 2 * g);
        const uint4 x0 = xa[0], x1 = xa[1], x2 = xa[2], x3 = xa[3];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          const int dl = dot8(lo[m], x0, x1);
          const int dh = dot8(hi[m], x2, x3);
          isum[m][t] += sc_lo[m] * dl + sc_hi[m] * dh;
          if (dots_out != nullptr && t == 0 && m == 0) {
            dots_out[2 * g] = dl;
            dots_out[2 * g + 1] = dh;
          }
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    if (t < nt) {
      const uint4 bs = xt.sums(t, blk);
      const float xd = xt.scale(t, blk);
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        // bs.x = bsum0 | bsum1<<16 ... ; mn[0] bytes = mins 0..3
        int msum = __dp2a_lo(static_cast<int>(bs.x), static_cast<int>(s6[m].mn[0]), 0);
        msum = __dp2a_hi(static_cast<int>(bs.y), static_cast<int>(s6[m].mn[0]), msum);
        msum = __dp2a_lo(static_cast<int>(bs.z), static_cast<int>(s6[m].mn[1]), msum);
        msum = __dp2a_hi(static_cast<int>(bs.w), static_cast<int>(s6[m].mn[1]), msum);
        acc[m][t] += xd * (d[m] * static_cast<float>(isum[m][t]) - dmin[m] * static_cast<float>(msum));
      }
    }
  }
}

// Sum over the `lpr` (power of two, <= 32) adjacent lanes that share a row.
__device__ __forceinline__ float reduce_lanes(float v, int lpr) {
  for (int off = lpr >> 1; off > 0; off >>= 1) v += __shfl_down_sync(0xFFFFFFFFu, v, off, 32);
  return v;
}

__host__ __device__ constexpr int next_pow2_cap32(int v) {
  int p = 1;
  while (p < v && p < 32) p <<= 1;
  return p;
}

}  // namespace sgr
