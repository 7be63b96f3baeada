// ref_wrap.cpp - extern "C" handles on the reference's OWN CPU code.
//
// TEST INFRASTRUCTURE ONLY. This translation unit contains no arithmetic: it
// forwards to the reference's functions, which the Makefile compiles from the
// reference tree where it lies (src/kernels/q4_k.cpp, src/kernels/cpu/
// q4_avx2.cpp, src/kernels/cpu/pool.cpp). The result, oracle/_ref/
// libsager_ref.so, pins the C restatement in sager_oracle.c and serves as the
// timed CPU baseline (the reference's AVX2 expert pool).
#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <vector>

#include "sager/core/expert_source.hpp"
#include "sager/kernels/cpu_ops.hpp"
#include "sager/kernels/q4_k.hpp"

using namespace sager;  // NOLINT

extern "C" {

int ref_have_avx2() { return cpu::have_avx2() ? 1 : 0; }

float ref_half_to_float(uint16_t h) { return q4k::half_to_float(h); }
uint16_t ref_float_to_half(float f) { return q4k::float_to_half(f); }

void ref_get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  q4k::get_scale_min_k4(j, q, d, m);
}
void ref_set_scale_min_k4(int j, uint8_t* q, uint8_t d, uint8_t m) {
  q4k::set_scale_min_k4(j, q, d, m);
}

void ref_dequant_row(const void* blocks, float* out, int n) {
  q4k::dequant_row(static_cast<const q4k::BlockQ4K*>(blocks), out, n);
}

void ref_quantize_row_q4k(const float* x, void* out, int n) {
  const std::vector<q4k::BlockQ4K> v = q4k::quantize_row(x, n);
  std::memcpy(out, v.data(), v.size() * sizeof(q4k::BlockQ4K));
}

void ref_quantize_row_q8k(const float* x, void* out, int n) {
  q4k::quantize_row_q8_K(x, static_cast<q4k::BlockQ8K*>(out), n);
}

void ref_quantize_row_q8k_avx2(const float* x, void* out, int n) {
  cpu::quantize_row_q8_k_avx2(x, static_cast<q4k::BlockQ8K*>(out), n);
}

float ref_vec_dot_ref(const void* w, const void* xq, int n) {
  return q4k::vec_dot_ref(static_cast<const q4k::BlockQ4K*>(w),
                          static_cast<const q4k::BlockQ8K*>(xq), n);
}

void ref_gemv_q4k_q8k_avx2(const void* w, const void* xq, float* y, int n_rows, int k) {
  cpu::gemv_q4_k_q8_avx2(static_cast<const q4k::BlockQ4K*>(w),
                         static_cast<const q4k::BlockQ8K*>(xq), y, n_rows, k);
}

void ref_gemv_q4k_q8k_scalar(const void* w, const void* xq, float* y, int n_rows, int k) {
  cpu::gemv_q4_k_q8_scalar(static_cast<const q4k::BlockQ4K*>(w),
                           static_cast<const q4k::BlockQ8K*>(xq), y, n_rows, k);
}

void ref_expert_ffn_q4(const void* wg, const void* wu, const void* wd, const float* x,
                       float* y, float* scratch, int hidden, int n_ff) {
  cpu::expert_ffn_q4(static_cast<const q4k::BlockQ4K*>(wg),
                     static_cast<const q4k::BlockQ4K*>(wu),
                     static_cast<const q4k::BlockQ4K*>(wd), x, y, scratch, hidden, n_ff);
}

int ref_validate_pool_geometry(int h0, int f0, int e0, int b0, int h1, int f1, int e1, int b1) {
  return static_cast<int>(validate_pool_geometry(PoolGeometry{h0, f0, e0, b0},
                                                 PoolGeometry{h1, f1, e1, b1}));
}

// ---- the reference's CPU expert pool (make_cpu_pool / submit / wait_done) ----
struct RefPool {
  std::unique_ptr<CpuPool> pool;
};

void* ref_pool_create(int workers, int hidden, int n_ff, int n_expert) {
  auto* p = new RefPool;
  p->pool = make_cpu_pool();
  const PoolGeometry geo{hidden, n_ff, n_expert, static_cast<int>(q4k::kBlockBytes)};
  if (p->pool->start(workers, geo) != Status::kOk) {
    delete p;
    return nullptr;
  }
  return p;
}

void ref_pool_destroy(void* h) {
  auto* p = static_cast<RefPool*>(h);
  if (!p) return;
  p->pool->stop();
  delete p;
}

// One submit() of n_jobs MissJobs followed by wait_done(): job j runs the
// expert whose three matrices are w3[3j..3j+2] on x + j*hidden into
// y + j*hidden. Returns the number of jobs the pool accepted. The pool's job
// ring only grows, so callers always wait before the next submit.
int ref_pool_run(void* h, const void* const* w3, const float* x, float* y, int n_jobs,
                 int hidden, int n_ff) {
  auto* p = static_cast<RefPool*>(h);
  std::vector<MissJob> jobs(static_cast<size_t>(n_jobs));
  for (int j = 0; j < n_jobs; ++j) {
    MissJob& mj = jobs[static_cast<size_t>(j)];
    mj.layer = 0;
    mj.expert = j;
    mj.w_gate = static_cast<const q4k::BlockQ4K*>(w3[3 * j]);
    mj.w_up = static_cast<const q4k::BlockQ4K*>(w3[3 * j + 1]);
    mj.w_out = static_cast<const q4k::BlockQ4K*>(w3[3 * j + 2]);
    mj.x = x + static_cast<size_t>(j) * hidden;
    mj.y = y + static_cast<size_t>(j) * hidden;
    mj.hidden = hidden;
    mj.n_ff = n_ff;
  }
  const int accepted = p->pool->submit(std::move(jobs));
  p->pool->wait_done(nullptr);
  return accepted;
}

}  // extern "C"
