// moe_ops.cu - the device-side plan, row movement, SwiGLU and combine kernels of
// the MoE half (src/kernels/cuda/moe.cu and src/kernels/cuda/norm_rotary.cu:
// 133-183 of the reference). All of them move or blend fp16 rows; they are
// written around 16-byte accesses (8 halves) with a scalar path for odd sizes.
#include <algorithm>

#include "api_util.cuh"
#include "q4k_common.cuh"

namespace sgr {
namespace {

__device__ __forceinline__ bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// ---- dispatch plan (moe.cu:366-434) ---------------------------------------------
// One CTA. hist -> exclusive prefixes off/toff -> grouped slots. Up to
// kStableMax routes the slots inside an expert are filled in ascending
// (row, kk) order (each expert's thread walks the id list in shared memory),
// which makes the plan reproducible; larger plans use atomics like the
// reference, whose consumers are all position-keyed.
constexpr int kScanThreads = 1024;
constexpr int kStableMax = 4096;

__global__ void __launch_bounds__(kScanThreads)
dispatch_scan_kernel(const int* __restrict__ idx, float* __restrict__ weight, int* __restrict__ gslot,
                     int* __restrict__ grows, int* __restrict__ off, int* __restrict__ toff,
                     int* __restrict__ meta, int* __restrict__ mail_n, int n_rows, int k,
                     int n_expert, int tok_per) {
  extern __shared__ int sm_i[];
  int* hist = sm_i;                    // [n_expert]
  int* fill = sm_i + n_expert;         // [n_expert]
  int* ids = sm_i + 2 * n_expert;      // [total] when the stable path is taken
  __shared__ int bad_sh;
  const int tid = threadIdx.x;
  const int total = n_rows * k;
  const bool stable = total <= kStableMax;
  if (tid == 0) bad_sh = 0;
  for (int e = tid; e < n_expert; e += kScanThreads) hist[e] = 0;
  __syncthreads();

  for (int i = tid; i < total; i += kScanThreads) {
    const int r = i / k, kk = i - r * k;
    const int e = idx[static_cast<size_t>(r) * (k + 1) + kk];
    const bool valid = e >= 0 && e < n_expert;
    if (stable) ids[i] = valid ? e : -1;
    if (!valid) {
      // a corrupt id silences the whole row, shared-expert slot included
      float* wr = weight + static_cast<size_t>(r) * (k + 1);
      for (int q = 0; q <= k; ++q) wr[q] = 0.f;
      atomicAdd(&bad_sh, 1);
    } else {
      atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();

  // exclusive prefixes of rows and of tiles over the experts: kScanThreads experts per round, scans
  // inside the warps, the warps' totals and the running totals through shared memory
  {
    __shared__ int wsum[2][kScanThreads / 32];
    __shared__ int carry[2];
    const int lane = tid & 31, wp = tid >> 5;
    if (tid == 0) carry[0] = carry[1] = 0;
    __syncthreads();
    for (int base = 0; base < n_expert; base += kScanThreads) {
      const int e = base + tid;
      const int c = e < n_expert ? hist[e] : 0;
      const int t = (c + tok_per - 1) / tok_per;
      int ic = c, it = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int uc = __shfl_up_sync(0xFFFFFFFFu, ic, o), ut = __shfl_up_sync(0xFFFFFFFFu, it, o);
        if (lane >= o) { ic += uc; it += ut; }
      }
      if (lane == 31) { wsum[0][wp] = ic; wsum[1][wp] = it; }
      __syncthreads();
      int pc = carry[0], pt = carry[1];
      for (int w = 0; w < wp; ++w) { pc += wsum[0][w]; pt += wsum[1][w]; }
      if (e < n_expert) {
        off[e] = pc + ic - c;
        toff[e] = pt + it - t;
        fill[e] = pc + ic - c;
      }
      __syncthreads();
      if (tid == kScanThreads - 1) { carry[0] = pc + ic; carry[1] = pt + it; }
      __syncthreads();
    }
    if (tid == 0) {
      off[n_expert] = carry[0];
      toff[n_expert] = carry[1];
      meta[0] = carry[0];
      meta[1] = carry[1];
      meta[2] = bad_sh;
      if (mail_n != nullptr) *mail_n = 0;
    }
  }
  __syncthreads();

  if (stable) {
    for (int i = tid; i < total; i += kScanThreads)
      if (ids[i] < 0) gslot[i] = -1;
    for (int e = tid; e < n_expert; e += kScanThreads) {
      if (hist[e] == 0) continue;
      int pos = fill[e];
      for (int i = 0; i < total; ++i) {
        if (ids[i] == e) {
          gslot[i] = pos;
          grows[pos] = i / k;
          ++pos;
        }
      }
    }
  } else {
    for (int i = tid; i < total; i += kScanThreads) {
      const int r = i / k, kk = i - r * k;
      const int e = idx[static_cast<size_t>(r) * (k + 1) + kk];
      if (e < 0 || e >= n_expert) { gslot[i] = -1; continue; }
      const int pos = atomicAdd(&fill[e], 1);
      gslot[i] = pos;
      grows[pos] = r;
    }
  }
}

// ---- row movement ------------------------------------------------------------------
// dst row r <- src row src_rows[r]; rows of `row_bytes` bytes (multiple of 4).
// grid.x = rows (bounded by *meta when meta != nullptr), grid.y = chunks of a row.
__global__ void gather_rows_kernel(unsigned char* __restrict__ dst,
                                   const unsigned char* __restrict__ src,
                                   const int* __restrict__ src_rows, const int* __restrict__ meta,
                                   int row_bytes) {
  const int r = blockIdx.x;
  if (meta != nullptr && r >= *meta) return;
  const unsigned char* s = src + static_cast<size_t>(src_rows[r]) * row_bytes;
  unsigned char* d = dst + static_cast<size_t>(r) * row_bytes;
  if (aligned16(s) && aligned16(d) && (row_bytes & 15) == 0) {
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < row_bytes / 16; i += gridDim.y * blockDim.x)
      reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
  } else if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 3u) == 0) {
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < row_bytes / 4; i += gridDim.y * blockDim.x)
      reinterpret_cast<uint32_t*>(d)[i] = reinterpret_cast<const uint32_t*>(s)[i];
  } else {
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < row_bytes / 2; i += gridDim.y * blockDim.x)
      reinterpret_cast<uint16_t*>(d)[i] = reinterpret_cast<const uint16_t*>(s)[i];
  }
}

// dst[dst_rows[i]] = src[i] (fp16 rows of `hidden`); grid.x = rows
__global__ void scatter_rows_kernel(uint16_t* __restrict__ dst, const uint16_t* __restrict__ src,
                                    const int* __restrict__ dst_rows, int hidden) {
  const int i = blockIdx.x;
  const uint16_t* s = src + static_cast<size_t>(i) * hidden;
  uint16_t* d = dst + static_cast<size_t>(dst_rows[i]) * hidden;
  if (aligned16(s) && aligned16(d) && (hidden & 7) == 0) {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < hidden / 8; j += gridDim.y * blockDim.x)
      reinterpret_cast<uint4*>(d)[j] = reinterpret_cast<const uint4*>(s)[j];
  } else {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < hidden; j += gridDim.y * blockDim.x)
      d[j] = s[j];
  }
}

// expert_y[row][kk][:] = grouped_out[gslot[row*n_used + kk]][:] (slab has n_used+1 slots
// per row; gslot < 0: slot left as is); grid (rows, chunks, n_used)
__global__ void scatter_routed_kernel(uint16_t* __restrict__ expert_y,
                                      const uint16_t* __restrict__ grouped_out,
                                      const int* __restrict__ gslot, int n_used, int hidden) {
  const int row = blockIdx.x, kk = blockIdx.z;
  const int gs = gslot[static_cast<size_t>(row) * n_used + kk];
  if (gs < 0) return;
  const uint16_t* s = grouped_out + static_cast<size_t>(gs) * hidden;
  uint16_t* d = expert_y + (static_cast<size_t>(row) * (n_used + 1) + kk) * hidden;
  if (aligned16(s) && aligned16(d) && (hidden & 7) == 0) {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < hidden / 8; j += gridDim.y * blockDim.x)
      reinterpret_cast<uint4*>(d)[j] = reinterpret_cast<const uint4*>(s)[j];
  } else {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < hidden; j += gridDim.y * blockDim.x)
      d[j] = s[j];
  }
}

// expert_out[k][:] = fp16(miss_y[slot_of_k[k]][:]) for slot >= 0; grid (k_rows, chunks)
__global__ void scatter_miss_kernel(uint16_t* __restrict__ expert_out,
                                    const int* __restrict__ slot_of_k,
                                    const float* __restrict__ miss_y, int hidden) {
  const int k = blockIdx.x;
  const int slot = slot_of_k[k];
  if (slot < 0) return;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x)
    expert_out[static_cast<size_t>(k) * hidden + i] = f2h(miss_y[static_cast<size_t>(slot) * hidden + i]);
}

// dst[dst_flat[i] + j] = fp16(src[i][j]); dst_flat holds element offsets; grid (n_list, chunks)
__global__ void scatter_rows_generic_kernel(uint16_t* __restrict__ dst, const float* __restrict__ src,
                                            const int* __restrict__ dst_flat, int hidden) {
  const int i = blockIdx.x;
  const size_t base = static_cast<size_t>(dst_flat[i]);
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < hidden; j += gridDim.y * blockDim.x)
    dst[base + j] = f2h(src[static_cast<size_t>(i) * hidden + j]);
}

// ---- SwiGLU and gates (norm_rotary.cu:133-183) ------------------------------------
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + expf(-g)) * u; }

__global__ void silu_mul_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ g,
                                const uint16_t* __restrict__ u, long long total,
                                const int* __restrict__ d_rows, int n_ff) {
  if (d_rows != nullptr) total = min(total, static_cast<long long>(*d_rows) * n_ff);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (aligned16(out) && aligned16(g) && aligned16(u)) {
    const long long n8 = total / 8;
    for (long long i = t0; i < n8; i += stride) {
      const uint4 gv = reinterpret_cast<const uint4*>(g)[i];
      const uint4 uv = reinterpret_cast<const uint4*>(u)[i];
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t ow[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint16_t lo = f2h(silu_mul(h2f(gw[j] & 0xFFFF), h2f(uw[j] & 0xFFFF)));
        const uint16_t hi = f2h(silu_mul(h2f(gw[j] >> 16), h2f(uw[j] >> 16)));
        ow[j] = lo | (static_cast<uint32_t>(hi) << 16);
      }
      reinterpret_cast<uint4*>(out)[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    for (long long i = n8 * 8 + t0; i < total; i += stride) out[i] = f2h(silu_mul(h2f(g[i]), h2f(u[i])));
  } else {
    for (long long i = t0; i < total; i += stride) out[i] = f2h(silu_mul(h2f(g[i]), h2f(u[i])));
  }
}

// out[row][i] *= sigmoid(g[row]); grid (rows, chunks)
__global__ void sigmoid_gate_scalar_kernel(uint16_t* __restrict__ out, const float* __restrict__ g,
                                           int hidden) {
  const int row = blockIdx.x;
  const float sig = 1.f / (1.f + expf(-g[row]));
  uint16_t* p = out + static_cast<size_t>(row) * hidden;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x)
    p[i] = f2h(h2f(p[i]) * sig);
}

// ---- combine (moe.cu:88-100, 265-280, 503-518) --------------------------------------
// out[row][i] = f16( f32(out[row][i]) + sum_kk w[kk] * f32(y[row][kk][i]) ), kk ascending.
// idx != nullptr: single-row form, slots with idx[kk] < 0 are skipped and the slab has
// `slots` rows; idx == nullptr: batched positional form with `slots` = n_used + 1.
__global__ void combine_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ expert_y,
                               const int* __restrict__ idx, const float* __restrict__ weight,
                               int slots, int hidden) {
  extern __shared__ float wsm[];       // [slots] weights of this row, then [slots] skip flags
  int* skip_sm = reinterpret_cast<int*>(wsm + slots);
  const int row = blockIdx.x;
  for (int kk = threadIdx.x; kk < slots; kk += blockDim.x) {
    wsm[kk] = weight[static_cast<size_t>(row) * slots + kk];
    skip_sm[kk] = (idx != nullptr && idx[kk] < 0) ? 1 : 0;   // slot not delivered (yet)
  }
  __syncthreads();
  uint16_t* o = out + static_cast<size_t>(row) * hidden;
  const uint16_t* y = expert_y + static_cast<size_t>(row) * slots * hidden;
  if (aligned16(o) && aligned16(y) && (hidden & 7) == 0) {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < hidden / 8; j += gridDim.y * blockDim.x) {
      const uint4 rv = reinterpret_cast<const uint4*>(o)[j];
      const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
      float acc[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) { acc[2 * q] = h2f(rw[q] & 0xFFFF); acc[2 * q + 1] = h2f(rw[q] >> 16); }
      for (int kk = 0; kk < slots; ++kk) {
        const float w = wsm[kk];
        if (skip_sm[kk]) continue;
        const uint4 yv = reinterpret_cast<const uint4*>(y + static_cast<size_t>(kk) * hidden)[j];
        const uint32_t yw[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[2 * q] += w * h2f(yw[q] & 0xFFFF);
          acc[2 * q + 1] += w * h2f(yw[q] >> 16);
        }
      }
      uint32_t ow[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) ow[q] = f2h(acc[2 * q]) | (static_cast<uint32_t>(f2h(acc[2 * q + 1])) << 16);
      reinterpret_cast<uint4*>(o)[j] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
  } else {
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x) {
      float acc = h2f(o[i]);
      for (int kk = 0; kk < slots; ++kk) {
        const float w = wsm[kk];
        if (skip_sm[kk]) continue;
        acc += w * h2f(y[static_cast<size_t>(kk) * hidden + i]);
      }
      o[i] = f2h(acc);
    }
  }
}

// Late add of patched slots, one after another inside each thread so that the
// read-modify-write of a row never races (moe.cu:497-518).
__global__ void combine_add_slots_kernel(uint16_t* __restrict__ out,
                                         const uint16_t* __restrict__ expert_y,
                                         const float* __restrict__ weight, const int* __restrict__ rk,
                                         int n_used, int hidden, int n_list) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) {
    for (int li = 0; li < n_list; ++li) {
      const size_t slot = static_cast<size_t>(rk[li]);
      const size_t row = slot / (n_used + 1);
      const float acc = h2f(out[row * hidden + i]) + weight[slot] * h2f(expert_y[slot * hidden + i]);
      out[row * hidden + i] = f2h(acc);
    }
  }
}

// chunks of a row (grid.y) for kernels that put rows in grid.x: `units` work items per row,
// `threads` per CTA; few rows get more chunks so a single-row call still spreads out
inline int row_chunks(int units, int threads, int rows) {
  const int full = (units + threads - 1) / threads;
  return rows >= 64 ? 1 : (full < 1 ? 1 : (full > 64 ? 64 : full));
}
inline int ok_or_launch() { return cudaPeekAtLastError() == cudaSuccess ? kOk : kErrLaunch; }

}  // namespace
}  // namespace sgr

using namespace sgr;

SGR_API int sgr_moe_dispatch_scan(const int* idx, float* weight, int* gslot, int* grows, int* off,
                                  int* toff, int* meta, int* mail, int* mail_n, int n_rows, int k,
                                  int n_expert, int tok_per, void* stream) {
  (void)mail;
  if (!idx || !weight || !gslot || !grows || !off || !toff || !meta || n_rows < 0 || k <= 0 ||
      n_expert <= 0 || tok_per <= 0)
    return kErrArg;
  const long long total = static_cast<long long>(n_rows) * k;
  const size_t smem = (2 * static_cast<size_t>(n_expert) + (total <= kStableMax ? total : 0)) * sizeof(int);
  if (smem > 48 * 1024) return kErrUnsupported;
  dispatch_scan_kernel<<<1, kScanThreads, smem, as_stream(stream)>>>(
      idx, weight, gslot, grows, off, toff, meta, mail_n, n_rows, k, n_expert, tok_per);
  return ok_or_launch();
}

SGR_API int sgr_gather_rows_q8(void* dst, const void* src, const int* src_rows, int n_rows,
                               int row_blocks, void* stream) {
  if (n_rows <= 0 || row_blocks <= 0) return kOk;
  if (!dst || !src || !src_rows) return kErrArg;
  if ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 3u) return kErrAlign;
  const int row_bytes = row_blocks * kX8;
  gather_rows_kernel<<<dim3(n_rows, row_chunks(row_bytes / 16, 128, n_rows)), 128, 0, as_stream(stream)>>>(
      static_cast<unsigned char*>(dst), static_cast<const unsigned char*>(src), src_rows, nullptr,
      row_bytes);
  return ok_or_launch();
}

SGR_API int sgr_gather_rows_q8_n(void* dst, const void* src, const int* src_rows, const int* meta,
                                 int r_max, int row_blocks, void* stream) {
  if (r_max <= 0 || row_blocks <= 0) return kOk;
  if (!dst || !src || !src_rows || !meta) return kErrArg;
  if ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 3u) return kErrAlign;
  gather_rows_kernel<<<dim3(r_max, row_chunks(row_blocks * kX8 / 16, 128, r_max)), 128, 0,
                       as_stream(stream)>>>(static_cast<unsigned char*>(dst),
                                            static_cast<const unsigned char*>(src), src_rows, meta,
                                            row_blocks * kX8);
  return ok_or_launch();
}

SGR_API int sgr_gather_rows_f16_n(uint16_t* dst, const uint16_t* src, const int* src_rows,
                                  const int* meta, int r_max, int hidden, void* stream) {
  if (r_max <= 0 || hidden <= 0) return kOk;
  if (!dst || !src || !src_rows || !meta) return kErrArg;
  gather_rows_kernel<<<dim3(r_max, row_chunks(hidden / 8, 128, r_max)), 128, 0, as_stream(stream)>>>(
      reinterpret_cast<unsigned char*>(dst), reinterpret_cast<const unsigned char*>(src), src_rows,
      meta, hidden * 2);
  return ok_or_launch();
}

SGR_API int sgr_scatter_rows_f16(uint16_t* dst, const uint16_t* src, const int* dst_rows, int n_rows,
                                 int hidden, void* stream) {
  if (n_rows <= 0 || hidden <= 0) return kOk;
  if (!dst || !src || !dst_rows) return kErrArg;
  scatter_rows_kernel<<<dim3(n_rows, row_chunks(hidden / 8, 128, n_rows)), 128, 0, as_stream(stream)>>>(dst, src, dst_rows, hidden);
  return ok_or_launch();
}

SGR_API int sgr_scatter_routed_f16(uint16_t* expert_y, const uint16_t* grouped_out, const int* gslot,
                                   int n_rows, int n_used, int hidden, void* stream) {
  if (n_rows <= 0 || n_used <= 0 || hidden <= 0) return kOk;
  if (!expert_y || !grouped_out || !gslot) return kErrArg;
  if (n_used > 65535) return kErrUnsupported;
  scatter_routed_kernel<<<dim3(n_rows, row_chunks(hidden / 8, 128, n_rows), n_used), 128, 0,
                          as_stream(stream)>>>(
      expert_y, grouped_out, gslot, n_used, hidden);
  return ok_or_launch();
}

SGR_API int sgr_scatter_miss_f32(uint16_t* expert_out, const int* d_slot_of_k, const float* miss_y,
                                 int k_rows, int hidden, void* stream) {
  if (k_rows <= 0 || hidden <= 0) return kOk;
  if (!expert_out || !d_slot_of_k || !miss_y) return kErrArg;
  scatter_miss_kernel<<<dim3(k_rows, row_chunks(hidden, 256, k_rows)), 256, 0, as_stream(stream)>>>(
      expert_out, d_slot_of_k, miss_y, hidden);
  return ok_or_launch();
}

SGR_API int sgr_scatter_rows_generic_f16(uint16_t* dst, const float* src, const int* dst_flat,
                                         int n_list, int hidden, void* stream) {
  if (n_list <= 0 || hidden <= 0) return kOk;
  if (!dst || !src || !dst_flat) return kErrArg;
  scatter_rows_generic_kernel<<<dim3(n_list, row_chunks(hidden, 256, n_list)), 256, 0, as_stream(stream)>>>(
      dst, src, dst_flat, hidden);
  return ok_or_launch();
}

SGR_API int sgr_silu_mul_f16(uint16_t* out, const uint16_t* g, const uint16_t* u, int rows, int n_ff,
                             void* stream) {
  const long long total = static_cast<long long>(rows) * n_ff;
  if (total <= 0) return kOk;
  if (!out || !g || !u) return kErrArg;
  const int blocks = static_cast<int>(std::min<long long>((total / 8 + 255) / 256 + 1, 148 * 8));
  silu_mul_kernel<<<blocks, 256, 0, as_stream(stream)>>>(out, g, u, total, nullptr, n_ff);
  return ok_or_launch();
}

SGR_API int sgr_silu_mul_f16_n(uint16_t* out, const uint16_t* g, const uint16_t* u, const int* d_rows,
                               int rows_max, int n_ff, void* stream) {
  const long long total = static_cast<long long>(rows_max) * n_ff;
  if (total <= 0) return kOk;
  if (!out || !g || !u || !d_rows) return kErrArg;
  const int blocks = static_cast<int>(std::min<long long>((total / 8 + 255) / 256 + 1, 148 * 8));
  silu_mul_kernel<<<blocks, 256, 0, as_stream(stream)>>>(out, g, u, total, d_rows, n_ff);
  return ok_or_launch();
}

SGR_API int sgr_sigmoid_gate_scalar_f16(uint16_t* out, const float* g, int n, void* stream) {
  if (n <= 0) return kOk;
  if (!out || !g) return kErrArg;
  sigmoid_gate_scalar_kernel<<<dim3(1, row_chunks(n, 256, 1)), 256, 0, as_stream(stream)>>>(out, g, n);
  return ok_or_launch();
}

SGR_API int sgr_sigmoid_gate_scalar_batched_f16(uint16_t* out, const float* g, int n_rows, int hidden,
                                                void* stream) {
  if (n_rows <= 0 || hidden <= 0) return kOk;
  if (!out || !g) return kErrArg;
  sigmoid_gate_scalar_kernel<<<dim3(n_rows, row_chunks(hidden, 256, n_rows)), 256, 0, as_stream(stream)>>>(
      out, g, hidden);
  return ok_or_launch();
}

SGR_API int sgr_moe_combine_f16(uint16_t* out, const uint16_t* expert_out, const int* idx,
                                const float* weight, int n_expert_used, int hidden, void* stream) {
  if (n_expert_used <= 0 || hidden <= 0) return kOk;
  if (!out || !expert_out || !idx || !weight) return kErrArg;
  combine_kernel<<<dim3(1, row_chunks(hidden / 8, 64, 1)), 64, n_expert_used * 8,
                   as_stream(stream)>>>(out, expert_out, idx, weight, n_expert_used, hidden);
  return ok_or_launch();
}

SGR_API int sgr_moe_combine_batched_f16(uint16_t* out, const uint16_t* expert_y, const float* weight,
                                        int n_used, int hidden, int n_rows, void* stream) {
  if (n_rows <= 0 || hidden <= 0) return kOk;
  if (!out || !expert_y || !weight || n_used < 0) return kErrArg;
  combine_kernel<<<dim3(n_rows, row_chunks(hidden / 8, 64, n_rows)), 64, (n_used + 1) * 8,
                   as_stream(stream)>>>(out, expert_y, nullptr, weight, n_used + 1, hidden);
  return ok_or_launch();
}

SGR_API int sgr_moe_combine_add_slots_f16(uint16_t* out, const uint16_t* expert_y,
                                          const float* weight, const int* rk, int n_used, int hidden,
                                          int n_list, void* stream) {
  if (n_list <= 0 || hidden <= 0) return kOk;
  if (!out || !expert_y || !weight || !rk) return kErrArg;
  combine_add_slots_kernel<<<(hidden + 255) / 256, 256, 0, as_stream(stream)>>>(
      out, expert_y, weight, rk, n_used, hidden, n_list);
  return ok_or_launch();
}
