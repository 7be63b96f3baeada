// tc_gemm.cu - the fp16 tensor-core family of the reference's prefill path
// (include/sager/kernels/cuda_ops.hpp:104-152; src/kernels/cuda/tc_gemm.cu): Q4_K
// weights dequantised to fp16, then  y[t][row] = sum_k x[t][k] * w[row][k]  with
// fp32 accumulation. The reference hands the GEMM to a library; here it is one
// tcgen05 kernel:
//
//   * warp 0 moves operand tiles (128 rows x 64 halfs) global -> shared with TMA
//     through two tensor maps encoded by the launcher and passed as kernel
//     parameters, a four-stage ring of (weights, activations) tile pairs;
//   * warp 1 owns tensor memory and issues tcgen05.mma kind::f16 (M 128, N up to
//     128, K 16 per instruction, fp32 accumulators in 128 TMEM columns);
//   * warps 2-5 read the accumulators back (tcgen05.ld) and store fp16 or fp32
//     rows, 32 consecutive weight rows of one token per warp store.
//
// Two operand layouts are built: 128-byte swizzled tiles (one 2-D box per tile) and
// unswizzled 8x16-byte core matrices (a 3-D box whose innermost extent is one core
// matrix row). Every wait is bounded; an expired wait raises the status word and the
// CTA still releases its tensor memory.
#include <cuda.h>

#include <atomic>
#include <cstring>

#include "api_util.cuh"
#include "q4k_common.cuh"

namespace sgr {
namespace {

constexpr int kBM = 128;            // weight rows per CTA (MMA M)
constexpr int kBN = 128;            // token rows per CTA (max MMA N)
constexpr int kBK = 64;             // halfs per stage and operand row: 128 bytes
constexpr int kTcStages = 4;
constexpr int kTileBytes = kBM * kBK * 2;                 // 16 KB, both operands
constexpr int kTcThreads = 192;
constexpr int kTcSmem = 1024 /*alignment slack*/ + 1024 /*barriers*/ + kTcStages * 2 * kTileBytes;
constexpr int kTcCols = 128;

enum { kLayoutSwizzled = 0, kLayoutCore = 1 };

// Shared-memory operand descriptors (K-major).
//   swizzled: rows of 128 bytes, eight-row groups 1024 bytes apart, 128-byte swizzle
//   core:     8x16-byte core matrices; K-adjacent ones a whole column of the tile apart
//             (tile rows x 16 bytes), eight-row groups 128 bytes apart
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, int layout, int tile_rows) {
  const uint64_t start = (saddr & 0x3FFFFu) >> 4;
  if (layout == kLayoutSwizzled)
    return start | (static_cast<uint64_t>(1) << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
           (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
  return start | (static_cast<uint64_t>(tile_rows) << 16) /* tile_rows * 16 bytes >> 4 */ |
         (static_cast<uint64_t>(128 >> 4) << 32) | (static_cast<uint64_t>(1) << 46);
}
// D fp32, A and B fp16, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t tc_idesc(int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_tma_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

struct TcArgs {
  void* y;
  int n_rows, k, n_tokens;
  int layout;
  int bn;                 // token rows per CTA: 128, or 64 when that is what fills the machine
  int* status;
};

template <bool F32OUT>
__global__ void __launch_bounds__(kTcThreads) tc_gemm_kernel(const __grid_constant__ CUtensorMap map_w,
                                                             const __grid_constant__ CUtensorMap map_x,
                                                             const TcArgs a) {
  extern __shared__ unsigned char tc_smem_raw[];
  const uint32_t base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = tc_smem_raw + (base - smem_u32(tc_smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);          // full[S], empty[S], acc
  uint64_t* full = bars;
  uint64_t* empty = bars + kTcStages;
  uint64_t* acc_full = bars + 2 * kTcStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kTcStages + 1);
  int* fail = reinterpret_cast<int*>(tmem_slot + 1);
  const uint32_t tiles = base + 1024;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * kBM, tok0 = blockIdx.y * a.bn;
  const int ntok = min(a.bn, a.n_tokens - tok0);
  const uint32_t b_bytes = static_cast<uint32_t>(a.bn) * kBK * 2;
  const int n_mma = max(16, (ntok + 15) & ~15);
  const int nkb = a.k / kBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kTcStages; ++i) {
      mbar_init(full + i, 1);
      mbar_init(empty + i, 1);
    }
    mbar_init(acc_full, 1);
    *fail = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTcCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % kTcStages;
        if (kb >= kTcStages && !mbar_wait(empty + s, ((kb / kTcStages) - 1) & 1)) {
          atomicExch(fail, 1);
          break;
        }
        mbar_expect_tx(full + s, kTileBytes + b_bytes);
        const uint32_t ta = tiles + s * 2 * kTileBytes, tb = ta + kTileBytes;
        if (a.layout == kLayoutSwizzled) {
          tc_tma_2d(ta, &map_w, kb * kBK, row0, full + s);
          tc_tma_2d(tb, &map_x, kb * kBK, tok0, full + s);
        } else {
          tc_tma_3d(ta, &map_w, 0, row0, kb * (kBK / 8), full + s);
          tc_tma_3d(tb, &map_x, 0, tok0, kb * (kBK / 8), full + s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = tc_idesc(n_mma);
      // bytes between K = 16 slices of a tile
      const int kstep_a = a.layout == kLayoutSwizzled ? 32 : 2 * kBM * 16;
      const int kstep_b = a.layout == kLayoutSwizzled ? 32 : 2 * a.bn * 16;
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % kTcStages;
        ok = mbar_wait(full + s, (kb / kTcStages) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t ta = tiles + s * 2 * kTileBytes, tb = ta + kTileBytes;
#pragma unroll
        for (int j = 0; j < kBK / 16; ++j)
          tc_mma(tmem, tc_desc(ta + j * kstep_a, a.layout, kBM), tc_desc(tb + j * kstep_b, a.layout, a.bn), idesc,
                 (kb | j) != 0);
        tc_commit(empty + s);
      }
      if (!ok) atomicExch(fail, 1);
      tc_commit(acc_full);             // arrives when everything issued so far has finished
    }
  } else {
    const int quarter = warp & 3;      // the TMEM lanes this warp may read
    const bool ok = mbar_wait(acc_full, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!ok && lane == 0) atomicExch(fail, 1);
    const int row = row0 + quarter * 32 + lane;
    if (__all_sync(0xFFFFFFFFu, ok && *reinterpret_cast<volatile int*>(fail) == 0)) {
      for (int c = 0; c < ntok; c += 16) {
        uint32_t v[16];
        tc_ld16(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < a.n_rows) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (c + i < ntok) {
              const size_t o = static_cast<size_t>(tok0 + c + i) * a.n_rows + row;
              if constexpr (F32OUT) reinterpret_cast<float*>(a.y)[o] = __uint_as_float(v[i]);
              else reinterpret_cast<uint16_t*>(a.y)[o] = f2h(__uint_as_float(v[i]));
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTcCols) : "memory");
  }
  if (threadIdx.x == 0 && *fail != 0 && a.status != nullptr) atomicExch(a.status, 1);
}

// ---- dequantisation ----------------------------------------------------------------------
// Lane l of a warp owns weights 8l .. 8l+7 of one super-block: sub-block l/4, its
// (l%4)-th octet. The warp's 32 stores are one contiguous 512-byte run.
// value = fp16( fma(d*sc, q, -(dmin*m)) ): one rounding to fp32, one to fp16
// (src/kernels/cuda/tc_gemm.cu:58-95 of the reference).
__device__ __forceinline__ uint4 dequant_octet(const unsigned char* blk, int lane) {
  const uint32_t dm = __ldg(reinterpret_cast<const uint32_t*>(blk));
  const Scales6 s6 = unpack_scales6(__ldg(reinterpret_cast<const uint32_t*>(blk + 4)),
                                    __ldg(reinterpret_cast<const uint32_t*>(blk + 8)),
                                    __ldg(reinterpret_cast<const uint32_t*>(blk + 12)));
  const int sb = lane >> 2, q = lane & 3;
  const float sd = h2f(static_cast<uint16_t>(dm & 0xFFFFu)) *
                   static_cast<float>(((sb < 4 ? s6.sc[0] : s6.sc[1]) >> (8 * (sb & 3))) & 0xFFu);
  const float sm = h2f(static_cast<uint16_t>(dm >> 16)) *
                   static_cast<float>(((sb < 4 ? s6.mn[0] : s6.mn[1]) >> (8 * (sb & 3))) & 0xFFu);
  const uint32_t* qp = reinterpret_cast<const uint32_t*>(blk + 16 + (sb >> 1) * 32 + q * 8);
  const uint2 w = make_uint2(__ldg(qp), __ldg(qp + 1));
  const int shift = (sb & 1) * 4;
  auto half_of = [&](uint32_t word, int byte) -> uint32_t {
    const uint32_t nib = (word >> (8 * byte + shift)) & 0xFu;
    return f2h(__fmaf_rn(sd, static_cast<float>(nib), -sm));
  };
  uint4 o;
  o.x = half_of(w.x, 0) | (half_of(w.x, 1) << 16);
  o.y = half_of(w.x, 2) | (half_of(w.x, 3) << 16);
  o.z = half_of(w.y, 0) | (half_of(w.y, 1) << 16);
  o.w = half_of(w.y, 2) | (half_of(w.y, 3) << 16);
  return o;
}

__global__ void __launch_bounds__(256) dequant_rows_kernel(const unsigned char* __restrict__ w,
                                                           uint4* __restrict__ out, long long n_blocks) {
  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long b = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); b < n_blocks;
       b += warps)
    out[b * 32 + lane] = dequant_octet(w + b * kW4, lane);
}

// The routed experts of one layer into a ring of fp16 slots
// (src/kernels/cuda/tc_gemm.cu:124-152 of the reference): slot e % ring holds
// rows_per rows of k halfs starting at element dst_row0; with two tables the first
// half of the rows comes from tab_a[e], the second from tab_b[e]. Experts without
// routed rows (off[e+1] <= off[e]) and null table entries are skipped.
__global__ void __launch_bounds__(256) dequant_experts_kernel(const unsigned char* const* __restrict__ tab_a,
                                                              const unsigned char* const* __restrict__ tab_b,
                                                              const int* __restrict__ off, uint16_t* slots,
                                                              long long dst_row0, int rows_per, int nb, int ring,
                                                              long long slot_elems) {
  const int e = blockIdx.y;
  if (off[e + 1] <= off[e]) return;
  const int lane = threadIdx.x & 31;
  const int half_rows = rows_per >> 1;
  const long long blocks = static_cast<long long>(rows_per) * nb;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  uint16_t* dst = slots + static_cast<long long>(e & (ring - 1)) * slot_elems + dst_row0;
  for (long long b = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); b < blocks;
       b += warps) {
    int r = static_cast<int>(b / nb);
    const int blk = static_cast<int>(b - static_cast<long long>(r) * nb);
    const unsigned char* src = tab_a[e];
    if (tab_b != nullptr && r >= half_rows) {
      src = tab_b[e];
      r -= half_rows;
    }
    if (src == nullptr) continue;
    reinterpret_cast<uint4*>(dst)[b * 32 + lane] =
        dequant_octet(src + (static_cast<long long>(r) * nb + blk) * kW4, lane);
  }
}

__global__ void __launch_bounds__(256) cast_f32_f16_kernel(const float4* __restrict__ src, uint2* __restrict__ dst,
                                                           long long n4) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = __ldg(src + i);
    dst[i] = make_uint2(f2h(v.x) | (static_cast<uint32_t>(f2h(v.y)) << 16),
                        f2h(v.z) | (static_cast<uint32_t>(f2h(v.w)) << 16));
  }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn tc_encoder() {
  static std::atomic<EncodeFn> cached{nullptr};
  EncodeFn f = cached.load(std::memory_order_acquire);
  if (f != nullptr) return f;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      fn == nullptr || qres != cudaDriverEntryPointSuccess)
    return nullptr;
  f = reinterpret_cast<EncodeFn>(fn);
  cached.store(f, std::memory_order_release);
  return f;
}

std::atomic<int> g_tc_layout{kLayoutSwizzled};

// A [rows][k] fp16 matrix as operand tiles of 128 rows x 64 halfs.
bool operand_map(CUtensorMap* tm, const void* base, int rows, int k, int layout, int tile_rows) {
  EncodeFn enc = tc_encoder();
  if (enc == nullptr) return false;
  if (layout == kLayoutSwizzled) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(tile_rows)};
    const cuuint32_t estr[2] = {1u, 1u};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  // (8 halfs, rows, k / 8): the box lands as [k-chunk][row][16 bytes]
  const cuuint64_t dims[3] = {8, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(k / 8)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(k) * 2, 16};
  const cuuint32_t box[3] = {8, static_cast<cuuint32_t>(tile_rows), kBK / 8};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool F32OUT>
int launch_tc_gemm(const void* w16, const void* x16, void* y, int n_rows, int k, int n_tokens, cudaStream_t s) {
  if (n_rows <= 0 || n_tokens <= 0) return kOk;
  if (!w16 || !x16 || !y || k <= 0) return kErrArg;
  if (k % kBK != 0) return kErrUnsupported;
  if ((reinterpret_cast<uintptr_t>(w16) | reinterpret_cast<uintptr_t>(x16)) & 15u) return kErrAlign;
  if (reinterpret_cast<uintptr_t>(y) & (F32OUT ? 3u : 1u)) return kErrAlign;
  const int layout = g_tc_layout.load(std::memory_order_relaxed);
  // 128 x 128 tiles when they fill the machine, else 128 x 64 for twice the CTAs
  const int row_tiles = (n_rows + kBM - 1) / kBM;
  const int bn = row_tiles * ((n_tokens + kBN - 1) / kBN) >= 148 ? kBN : 64;
  CUtensorMap mw, mx;
  if (!operand_map(&mw, w16, n_rows, k, layout, kBM) || !operand_map(&mx, x16, n_tokens, k, layout, bn))
    return kErrUnsupported;
  auto kern = tc_gemm_kernel<F32OUT>;
  // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem) != cudaSuccess)
    return kErrLaunch;
  TcArgs a{y, n_rows, k, n_tokens, layout, bn, status_word()};
  kern<<<dim3(row_tiles, (n_tokens + bn - 1) / bn), kTcThreads, kTcSmem, s>>>(mw, mx, a);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}

int grid_for(long long warps_needed, int warps_per_cta) {
  const long long ctas = (warps_needed + warps_per_cta - 1) / warps_per_cta;
  return static_cast<int>(ctas < 1 ? 1 : (ctas > 148 * 16 ? 148 * 16 : ctas));
}

int launch_dequant(const void* w, void* out16, long long n_blocks, cudaStream_t s) {
  if (n_blocks <= 0) return kOk;
  dequant_rows_kernel<<<grid_for(n_blocks, 8), 256, 0, s>>>(static_cast<const unsigned char*>(w),
                                                           static_cast<uint4*>(out16), n_blocks);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}

}  // namespace
}  // namespace sgr

using namespace sgr;

SGR_API void* sgr_tc_handle(void) { return reinterpret_cast<void*>(tc_encoder()); }

SGR_API size_t sgr_tc_scratch_elems(int max_rows, int max_k) {
  return static_cast<size_t>(max_rows > 0 ? max_rows : 1) * static_cast<size_t>(max_k > 0 ? max_k : 1);
}

SGR_API int sgr_tc_set_operand_layout(int layout) {
  if (layout != kLayoutSwizzled && layout != kLayoutCore) return kErrArg;
  g_tc_layout.store(layout, std::memory_order_relaxed);
  return kOk;
}

SGR_API int sgr_tc_gemm_f16_raw(const void* w16, const void* x16, void* y16, int n_rows, int k, int n_tokens,
                                void* stream) {
  return launch_tc_gemm<false>(w16, x16, y16, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_tc_gemm_f16_f32out_raw(const void* w16, const void* x16, float* y32, int n_rows, int k,
                                       int n_tokens, void* stream) {
  return launch_tc_gemm<true>(w16, x16, y32, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_dequant_q4_k_f16(const void* w, uint16_t* out16, int n_rows, int k, void* stream) {
  if (n_rows <= 0) return kOk;
  if (!w || !out16 || k <= 0 || k % kQK != 0) return kErrArg;
  if ((reinterpret_cast<uintptr_t>(w) & 3u) || (reinterpret_cast<uintptr_t>(out16) & 15u)) return kErrAlign;
  return launch_dequant(w, out16, static_cast<long long>(n_rows) * (k / kQK), as_stream(stream));
}

SGR_API int sgr_tc_gemm_q4_k_f16(const void* w, const uint16_t* x, uint16_t* y, uint16_t* scratch, int n_rows,
                                 int k, int n_tokens, void* stream) {
  if (n_rows <= 0 || n_tokens <= 0) return kOk;
  if (!w || !x || !y || !scratch) return kErrArg;
  // the reference's own refusals (callers then take the GEMV path): k a power of two
  // >= 256, weights 16-byte aligned
  if (k < kQK || (k & (k - 1)) != 0) return kErrUnsupported;
  if (reinterpret_cast<uintptr_t>(w) & 15u) return kErrAlign;
  if (reinterpret_cast<uintptr_t>(scratch) & 15u) return kErrAlign;
  const int rc = launch_dequant(w, scratch, static_cast<long long>(n_rows) * (k / kQK), as_stream(stream));
  if (rc != kOk) return rc;
  return launch_tc_gemm<false>(scratch, x, y, n_rows, k, n_tokens, as_stream(stream));
}

SGR_API int sgr_dequant_experts_q4_k_f16(const void* const* tab_a, const void* const* tab_b, const int* off,
                                         void* slots, long long dst_row0, int rows_sl2, int k, int n_experts,
                                         int ring, long long slot_elems, void* stream) {
  if (n_experts <= 0) return kOk;
  if (!tab_a || !off || !slots || k <= 0 || k % kQK != 0 || rows_sl2 < 1 || rows_sl2 > 24 || ring <= 0 ||
      (ring & (ring - 1)) != 0)
    return kErrArg;
  if ((reinterpret_cast<uintptr_t>(slots) & 15u) || (dst_row0 & 7) || (slot_elems & 7)) return kErrAlign;
  const int rows_per = 1 << rows_sl2;
  const int nb = k / kQK;
  const long long blocks = static_cast<long long>(rows_per) * nb;
  int gx = grid_for(blocks, 8);
  if (gx > 64) gx = 64;                                     // x n_experts CTAs; grid-stride inside
  dequant_experts_kernel<<<dim3(gx, n_experts), 256, 0, as_stream(stream)>>>(
      reinterpret_cast<const unsigned char* const*>(tab_a), reinterpret_cast<const unsigned char* const*>(tab_b),
      off, static_cast<uint16_t*>(slots), dst_row0, rows_per, nb, ring, slot_elems);
  return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch;
}

SGR_API int sgr_tc_router_f32(const float* w_f32, const uint16_t* x, float* y, uint16_t* scratch, int n_rows,
                              int k, int n_tokens, void* stream) {
  if (n_rows <= 0 || n_tokens <= 0) return kOk;
  if (!w_f32 || !x || !y || !scratch || k <= 0) return kErrArg;
  if (k % kBK != 0) return kErrUnsupported;
  if ((reinterpret_cast<uintptr_t>(w_f32) & 15u) || (reinterpret_cast<uintptr_t>(scratch) & 15u)) return kErrAlign;
  const long long n4 = static_cast<long long>(n_rows) * k / 4;
  cast_f32_f16_kernel<<<grid_for((n4 + 31) / 32, 8), 256, 0, as_stream(stream)>>>(
      reinterpret_cast<const float4*>(w_f32), reinterpret_cast<uint2*>(scratch), n4);
  if (cudaPeekAtLastError() != cudaSuccess) return kErrLaunch;
  return launch_tc_gemm<true>(scratch, x, y, n_rows, k, n_tokens, as_stream(stream));
}
