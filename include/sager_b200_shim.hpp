// sager_b200_shim.hpp - turns the C ABI of libsager_b200.so back into the C++
// launchers the reference's session loop calls (namespace sager::cuda,
// include/sager/kernels/cuda_ops.hpp of the reference): same names, same
// parameter lists, same void return. Compile ONE translation unit of the host
// program with SAGER_B200_SHIM_IMPLEMENTATION defined to get the definitions,
// drop the reference's own q4_k.cu / moe.cu / mmq.cu / norm_rotary.cu objects for
// these symbols from the link, and link libsager_b200.so instead.
//
// A non-zero code from the library (argument validation) is kept in
// sager::cuda::b200_last_error() - the reference's launchers return void and
// report through cudaGetLastError, which a separately linked runtime cannot see.
#pragma once

#include <cstdint>

#include "sager_b200.h"

#ifndef __CUDA_RUNTIME_H__
struct CUstream_st;
typedef CUstream_st* cudaStream_t;
#endif

namespace sager::q4k {
struct BlockQ4K;   // 144-byte super-block, include/sager/kernels/q4_k.hpp:46-52
struct BlockQ8K;   // 276-byte activation block, include/sager/kernels/q4_k.hpp:58-62
}  // namespace sager::q4k

namespace sager::cuda {

int b200_last_error();

void quantize_q8_k(const uint16_t* x_f16, q4k::BlockQ8K* out, int n, cudaStream_t stream);
void quantize_q8_k_n(const uint16_t* x_f16, q4k::BlockQ8K* out, const int* d_rows, int row_mult, int n_max, cudaStream_t stream);
void gemv_q4_k_q8(const q4k::BlockQ4K* w, const q4k::BlockQ8K* x_q8, float* y, int n_rows, int k, cudaStream_t stream);
void gemv_q4_k_q8_f16out(const q4k::BlockQ4K* w, const q4k::BlockQ8K* x_q8, uint16_t* y, int n_rows, int k, cudaStream_t stream);
void gemv_ptrs_q4_k_q8_f16out(const q4k::BlockQ4K* const* ptrs, const q4k::BlockQ8K* x_q8, uint16_t* y, int n_ptrs, int rows_per, int k, cudaStream_t stream);
void gemv_q4_k_q8_f16out_batched(const q4k::BlockQ4K* w, const q4k::BlockQ8K* x_q8, uint16_t* y, int n_rows, int k, int n_tokens, cudaStream_t stream);
void gemv_q4_k_q8_batched(const q4k::BlockQ4K* w, const q4k::BlockQ8K* x_q8, float* y, int n_rows, int k, int n_tokens, cudaStream_t stream);
void gemv_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* w, const q4k::BlockQ8K* xq, uint16_t* y, int n_rows, int k, int n_tokens, cudaStream_t stream);
void mmq_q4_k_q8_f16out(const q4k::BlockQ4K* w, const q4k::BlockQ8K* xq, uint16_t* y, int n_rows, int k, int n_tokens, cudaStream_t stream);
void mmq2_q4_k_q8_f16out(const q4k::BlockQ4K* wg, const q4k::BlockQ4K* wu, const q4k::BlockQ8K* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int n_tokens, cudaStream_t stream);
void gemv2_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* wg, const q4k::BlockQ4K* wu, const q4k::BlockQ8K* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int n_tokens, cudaStream_t stream);
void gemv_grouped2_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* const* wg, const q4k::BlockQ4K* const* wu, const int* off, const int* m, const int* tile_base, const int* job_of_tile, int n_tiles, const q4k::BlockQ8K* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int tok_per, cudaStream_t stream);
void gemv_grouped_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* const* w, const int* off, const int* m, const int* tile_base, const int* job_of_tile, int n_tiles, const q4k::BlockQ8K* xq, uint16_t* y, int n_rows, int k, int tok_per, cudaStream_t stream);
void gemv_grouped2_tab_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* const* wg_tab, const q4k::BlockQ4K* const* wu_tab, const int* off, const int* toff, const int* meta, int* mail, int* mail_n, int tiles_max, const q4k::BlockQ8K* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int n_expert, int tok_per, cudaStream_t stream);
void gemv_grouped_tab_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* const* w_tab, const int* off, const int* toff, const int* meta, int tiles_max, const q4k::BlockQ8K* xq, uint16_t* y, int n_rows, int k, int n_expert, int tok_per, cudaStream_t stream);
void gemv_f32_out_f16x(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k, cudaStream_t stream);
void gemv_f32_out_f16x_batched(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k, int n_tokens, cudaStream_t stream);
void gemv_f32_out_f16x_mtok(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k, int n_tokens, cudaStream_t stream);
void router_topk(const float* logits, int* idx, float* weight, int n_expert, int n_expert_used, float shared_w, cudaStream_t stream);
void router_topk_batched(const float* logits, int* idx, float* weight, int n_expert, int n_expert_used, int idx_stride, int n_rows, float shared_w, cudaStream_t stream);
void router_topk_fused(const float* w_f32, const uint16_t* x_f16, int* idx, float* weight, int n_expert, int n_expert_used, int hidden, cudaStream_t stream);
void moe_dispatch_scan(const int* idx, float* weight, int* gslot, int* grows, int* off, int* toff, int* meta, int* mail, int* mail_n, int n_rows, int k, int n_expert, int tok_per, cudaStream_t stream);
void gather_rows_q8(q4k::BlockQ8K* dst, const q4k::BlockQ8K* src, const int* src_rows, int n_rows, int row_blocks, cudaStream_t stream);
void gather_rows_q8_n(q4k::BlockQ8K* dst, const q4k::BlockQ8K* src, const int* src_rows, const int* meta, int r_max, int row_blocks, cudaStream_t stream);
void gather_rows_f16_n(uint16_t* dst, const uint16_t* src, const int* src_rows, const int* meta, int r_max, int hidden, cudaStream_t stream);
void scatter_rows_f16(uint16_t* dst, const uint16_t* src, const int* dst_rows, int n_rows, int hidden, cudaStream_t stream);
void scatter_routed_f16(uint16_t* expert_y, const uint16_t* grouped_out, const int* gslot, int n_rows, int n_used, int hidden, cudaStream_t stream);
void scatter_miss_f32(uint16_t* expert_out, const int* d_slot_of_k, const float* miss_y, int k_rows, int hidden, cudaStream_t stream);
void scatter_rows_generic_f16(uint16_t* dst, const float* src, const int* dst_flat, int n_list, int hidden, cudaStream_t stream);
void silu_mul_f16(uint16_t* out, const uint16_t* g, const uint16_t* u, int rows, int n_ff, cudaStream_t stream);
void silu_mul_f16_n(uint16_t* out, const uint16_t* g, const uint16_t* u, const int* d_rows, int rows_max, int n_ff, cudaStream_t stream);
void sigmoid_gate_scalar_f16(uint16_t* out, const float* g, int n, cudaStream_t stream);
void sigmoid_gate_scalar_batched_f16(uint16_t* out, const float* g, int n_rows, int hidden, cudaStream_t stream);
void moe_combine_f16(uint16_t* out, const uint16_t* expert_out, const int* idx, const float* weight, int n_expert_used, int hidden, cudaStream_t stream);
void moe_combine_batched_f16(uint16_t* out, const uint16_t* expert_y, const float* weight, int n_used, int hidden, int n_rows, cudaStream_t stream);
void moe_combine_add_slots_f16(uint16_t* out, const uint16_t* expert_y, const float* weight, const int* rk, int n_used, int hidden, int n_list, cudaStream_t stream);
void gemv_q6_k_q8(const void* w_q6, const q4k::BlockQ8K* x_q8, float* y, int n_rows, int k, cudaStream_t stream);
void gemv_q6_k_q8_smx(const void* w_q6, const q4k::BlockQ8K* x_q8, float* y, int n_rows, int k, cudaStream_t stream);
void topk_select_f32_2p(const float* logits, float* seg_v, int* seg_i, int seg_slots, float* out_v, int* out_i, int n, int k, cudaStream_t stream);
void rmsnorm_quant_f16(uint16_t* out, const uint16_t* x, const uint16_t* w, q4k::BlockQ8K* xq, int n, float eps, int n_rows, cudaStream_t stream);
void gemv2m_q4_k_q8_f16out(const q4k::BlockQ4K* w1, const q4k::BlockQ4K* w2, const q4k::BlockQ8K* xq, uint16_t* y1, uint16_t* y2, int rows1, int rows2, int k, int slot, cudaStream_t stream);
void gemv3m_q4_k_q8_f16out(const q4k::BlockQ4K* w1, const q4k::BlockQ4K* w2, const q4k::BlockQ4K* w3, const q4k::BlockQ8K* xq, uint16_t* y1, uint16_t* y2, uint16_t* y3, int rows1, int rows2, int rows3, int k, int slot, cudaStream_t stream);
void gemv_q4_k_q8_f16out_resadd(const q4k::BlockQ4K* w, const q4k::BlockQ8K* xq, uint16_t* y, uint16_t* res_inout, int n_rows, int k, cudaStream_t stream);
bool tc_gemm_q4_k_f16(const q4k::BlockQ4K* w, const uint16_t* x, uint16_t* y, uint16_t* scratch, int n_rows, int k, int n_tokens, cudaStream_t stream);
void* tc_handle();
size_t tc_scratch_elems(int max_rows, int max_k);
bool tc_gemm_f16_raw(const void* w16, const void* x16, void* y16, int n_rows, int k, int n_tokens, cudaStream_t stream);
void dequant_experts_q4_k_f16(const q4k::BlockQ4K* const* tab_a, const q4k::BlockQ4K* const* tab_b, const int* off, void* slots, long long dst_row0, int rows_sl2, int k, int n_experts, int ring, long long slot_elems, cudaStream_t stream);
bool tc_gemm_f16_f32out_raw(const void* w16, const void* x16, float* y32, int n_rows, int k, int n_tokens, cudaStream_t stream);
void tc_router_f32(const float* w_f32, const uint16_t* x, float* y, uint16_t* scratch, int n_rows, int k, int n_tokens, cudaStream_t stream);

#ifdef SAGER_B200_SHIM_IMPLEMENTATION
namespace b200_detail {
inline int& slot() { static thread_local int e = 0; return e; }
inline void note(int rc) { if (rc != 0) slot() = rc; }
}  // namespace b200_detail
int b200_last_error() { const int e = b200_detail::slot(); b200_detail::slot() = 0; return e; }

void quantize_q8_k(const uint16_t* x_f16, q4k::BlockQ8K* out, int n, cudaStream_t stream) {
  b200_detail::note(sgr_quantize_q8_k(x_f16, out, n, stream));
}
void quantize_q8_k_n(const uint16_t* x_f16, q4k::BlockQ8K* out, const int* d_rows, int row_mult, int n_max, cudaStream_t stream) {
  b200_detail::note(sgr_quantize_q8_k_n(x_f16, out, d_rows, row_mult, n_max, stream));
}
void gemv_q4_k_q8(const q4k::BlockQ4K* w, const q4k::BlockQ8K* x_q8, float* y, int n_rows, int k, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_q4_k_q8(w, x_q8, y, n_rows, k, stream));
}
void gemv_q4_k_q8_f16out(const q4k::BlockQ4K* w, const q4k::BlockQ8K* x_q8, uint16_t* y, int n_rows, int k, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_q4_k_q8_f16out(w, x_q8, y, n_rows, k, stream));
}
void gemv_ptrs_q4_k_q8_f16out(const q4k::BlockQ4K* const* ptrs, const q4k::BlockQ8K* x_q8, uint16_t* y, int n_ptrs, int rows_per, int k, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_ptrs_q4_k_q8_f16out(reinterpret_cast<const void* const*>(ptrs), x_q8, y, n_ptrs, rows_per, k, stream));
}
void gemv_q4_k_q8_f16out_batched(const q4k::BlockQ4K* w, const q4k::BlockQ8K* x_q8, uint16_t* y, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_q4_k_q8_f16out_batched(w, x_q8, y, n_rows, k, n_tokens, stream));
}
void gemv_q4_k_q8_batched(const q4k::BlockQ4K* w, const q4k::BlockQ8K* x_q8, float* y, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_q4_k_q8_batched(w, x_q8, y, n_rows, k, n_tokens, stream));
}
void gemv_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* w, const q4k::BlockQ8K* xq, uint16_t* y, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_q4_k_q8_f16out_mtok(w, xq, y, n_rows, k, n_tokens, stream));
}
void mmq_q4_k_q8_f16out(const q4k::BlockQ4K* w, const q4k::BlockQ8K* xq, uint16_t* y, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  b200_detail::note(sgr_mmq_q4_k_q8_f16out(w, xq, y, n_rows, k, n_tokens, stream));
}
void mmq2_q4_k_q8_f16out(const q4k::BlockQ4K* wg, const q4k::BlockQ4K* wu, const q4k::BlockQ8K* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  b200_detail::note(sgr_mmq2_q4_k_q8_f16out(wg, wu, xq, yg, yu, n_rows, k, n_tokens, stream));
}
void gemv2_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* wg, const q4k::BlockQ4K* wu, const q4k::BlockQ8K* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  b200_detail::note(sgr_gemv2_q4_k_q8_f16out_mtok(wg, wu, xq, yg, yu, n_rows, k, n_tokens, stream));
}
void gemv_grouped2_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* const* wg, const q4k::BlockQ4K* const* wu, const int* off, const int* m, const int* tile_base, const int* job_of_tile, int n_tiles, const q4k::BlockQ8K* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int tok_per, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_grouped2_q4_k_q8_f16out_mtok(reinterpret_cast<const void* const*>(wg), reinterpret_cast<const void* const*>(wu), off, m, tile_base, job_of_tile, n_tiles, xq, yg, yu, n_rows, k, tok_per, stream));
}
void gemv_grouped_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* const* w, const int* off, const int* m, const int* tile_base, const int* job_of_tile, int n_tiles, const q4k::BlockQ8K* xq, uint16_t* y, int n_rows, int k, int tok_per, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_grouped_q4_k_q8_f16out_mtok(reinterpret_cast<const void* const*>(w), off, m, tile_base, job_of_tile, n_tiles, xq, y, n_rows, k, tok_per, stream));
}
void gemv_grouped2_tab_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* const* wg_tab, const q4k::BlockQ4K* const* wu_tab, const int* off, const int* toff, const int* meta, int* mail, int* mail_n, int tiles_max, const q4k::BlockQ8K* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int n_expert, int tok_per, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_grouped2_tab_q4_k_q8_f16out_mtok(reinterpret_cast<const void* const*>(wg_tab), reinterpret_cast<const void* const*>(wu_tab), off, toff, meta, mail, mail_n, tiles_max, xq, yg, yu, n_rows, k, n_expert, tok_per, stream));
}
void gemv_grouped_tab_q4_k_q8_f16out_mtok(const q4k::BlockQ4K* const* w_tab, const int* off, const int* toff, const int* meta, int tiles_max, const q4k::BlockQ8K* xq, uint16_t* y, int n_rows, int k, int n_expert, int tok_per, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_grouped_tab_q4_k_q8_f16out_mtok(reinterpret_cast<const void* const*>(w_tab), off, toff, meta, tiles_max, xq, y, n_rows, k, n_expert, tok_per, stream));
}
void gemv_f32_out_f16x(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_f32_out_f16x(w_f32, x_f16, y, n_rows, k, stream));
}
void gemv_f32_out_f16x_batched(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_f32_out_f16x_batched(w_f32, x_f16, y, n_rows, k, n_tokens, stream));
}
void gemv_f32_out_f16x_mtok(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_f32_out_f16x_mtok(w_f32, x_f16, y, n_rows, k, n_tokens, stream));
}
void router_topk(const float* logits, int* idx, float* weight, int n_expert, int n_expert_used, float shared_w, cudaStream_t stream) {
  b200_detail::note(sgr_router_topk(logits, idx, weight, n_expert, n_expert_used, shared_w, stream));
}
void router_topk_batched(const float* logits, int* idx, float* weight, int n_expert, int n_expert_used, int idx_stride, int n_rows, float shared_w, cudaStream_t stream) {
  b200_detail::note(sgr_router_topk_batched(logits, idx, weight, n_expert, n_expert_used, idx_stride, n_rows, shared_w, stream));
}
void router_topk_fused(const float* w_f32, const uint16_t* x_f16, int* idx, float* weight, int n_expert, int n_expert_used, int hidden, cudaStream_t stream) {
  b200_detail::note(sgr_router_topk_fused(w_f32, x_f16, idx, weight, n_expert, n_expert_used, hidden, stream));
}
void moe_dispatch_scan(const int* idx, float* weight, int* gslot, int* grows, int* off, int* toff, int* meta, int* mail, int* mail_n, int n_rows, int k, int n_expert, int tok_per, cudaStream_t stream) {
  b200_detail::note(sgr_moe_dispatch_scan(idx, weight, gslot, grows, off, toff, meta, mail, mail_n, n_rows, k, n_expert, tok_per, stream));
}
void gather_rows_q8(q4k::BlockQ8K* dst, const q4k::BlockQ8K* src, const int* src_rows, int n_rows, int row_blocks, cudaStream_t stream) {
  b200_detail::note(sgr_gather_rows_q8(dst, src, src_rows, n_rows, row_blocks, stream));
}
void gather_rows_q8_n(q4k::BlockQ8K* dst, const q4k::BlockQ8K* src, const int* src_rows, const int* meta, int r_max, int row_blocks, cudaStream_t stream) {
  b200_detail::note(sgr_gather_rows_q8_n(dst, src, src_rows, meta, r_max, row_blocks, stream));
}
void gather_rows_f16_n(uint16_t* dst, const uint16_t* src, const int* src_rows, const int* meta, int r_max, int hidden, cudaStream_t stream) {
  b200_detail::note(sgr_gather_rows_f16_n(dst, src, src_rows, meta, r_max, hidden, stream));
}
void scatter_rows_f16(uint16_t* dst, const uint16_t* src, const int* dst_rows, int n_rows, int hidden, cudaStream_t stream) {
  b200_detail::note(sgr_scatter_rows_f16(dst, src, dst_rows, n_rows, hidden, stream));
}
void scatter_routed_f16(uint16_t* expert_y, const uint16_t* grouped_out, const int* gslot, int n_rows, int n_used, int hidden, cudaStream_t stream) {
  b200_detail::note(sgr_scatter_routed_f16(expert_y, grouped_out, gslot, n_rows, n_used, hidden, stream));
}
void scatter_miss_f32(uint16_t* expert_out, const int* d_slot_of_k, const float* miss_y, int k_rows, int hidden, cudaStream_t stream) {
  b200_detail::note(sgr_scatter_miss_f32(expert_out, d_slot_of_k, miss_y, k_rows, hidden, stream));
}
void scatter_rows_generic_f16(uint16_t* dst, const float* src, const int* dst_flat, int n_list, int hidden, cudaStream_t stream) {
  b200_detail::note(sgr_scatter_rows_generic_f16(dst, src, dst_flat, n_list, hidden, stream));
}
void silu_mul_f16(uint16_t* out, const uint16_t* g, const uint16_t* u, int rows, int n_ff, cudaStream_t stream) {
  b200_detail::note(sgr_silu_mul_f16(out, g, u, rows, n_ff, stream));
}
void silu_mul_f16_n(uint16_t* out, const uint16_t* g, const uint16_t* u, const int* d_rows, int rows_max, int n_ff, cudaStream_t stream) {
  b200_detail::note(sgr_silu_mul_f16_n(out, g, u, d_rows, rows_max, n_ff, stream));
}
void sigmoid_gate_scalar_f16(uint16_t* out, const float* g, int n, cudaStream_t stream) {
  b200_detail::note(sgr_sigmoid_gate_scalar_f16(out, g, n, stream));
}
void sigmoid_gate_scalar_batched_f16(uint16_t* out, const float* g, int n_rows, int hidden, cudaStream_t stream) {
  b200_detail::note(sgr_sigmoid_gate_scalar_batched_f16(out, g, n_rows, hidden, stream));
}
void moe_combine_f16(uint16_t* out, const uint16_t* expert_out, const int* idx, const float* weight, int n_expert_used, int hidden, cudaStream_t stream) {
  b200_detail::note(sgr_moe_combine_f16(out, expert_out, idx, weight, n_expert_used, hidden, stream));
}
void moe_combine_batched_f16(uint16_t* out, const uint16_t* expert_y, const float* weight, int n_used, int hidden, int n_rows, cudaStream_t stream) {
  b200_detail::note(sgr_moe_combine_batched_f16(out, expert_y, weight, n_used, hidden, n_rows, stream));
}
void moe_combine_add_slots_f16(uint16_t* out, const uint16_t* expert_y, const float* weight, const int* rk, int n_used, int hidden, int n_list, cudaStream_t stream) {
  b200_detail::note(sgr_moe_combine_add_slots_f16(out, expert_y, weight, rk, n_used, hidden, n_list, stream));
}
void gemv_q6_k_q8(const void* w_q6, const q4k::BlockQ8K* x_q8, float* y, int n_rows, int k, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_q6_k_q8(w_q6, x_q8, y, n_rows, k, stream));
}
void gemv_q6_k_q8_smx(const void* w_q6, const q4k::BlockQ8K* x_q8, float* y, int n_rows, int k, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_q6_k_q8_smx(w_q6, x_q8, y, n_rows, k, stream));
}
void topk_select_f32_2p(const float* logits, float* seg_v, int* seg_i, int seg_slots, float* out_v, int* out_i, int n, int k, cudaStream_t stream) {
  b200_detail::note(sgr_topk_select_f32_2p(logits, seg_v, seg_i, seg_slots, out_v, out_i, n, k, stream));
}
void rmsnorm_quant_f16(uint16_t* out, const uint16_t* x, const uint16_t* w, q4k::BlockQ8K* xq, int n, float eps, int n_rows, cudaStream_t stream) {
  b200_detail::note(sgr_rmsnorm_quant_f16(out, x, w, xq, n, eps, n_rows, stream));
}
void gemv2m_q4_k_q8_f16out(const q4k::BlockQ4K* w1, const q4k::BlockQ4K* w2, const q4k::BlockQ8K* xq, uint16_t* y1, uint16_t* y2, int rows1, int rows2, int k, int slot, cudaStream_t stream) {
  b200_detail::note(sgr_gemv2m_q4_k_q8_f16out(w1, w2, xq, y1, y2, rows1, rows2, k, slot, stream));
}
void gemv3m_q4_k_q8_f16out(const q4k::BlockQ4K* w1, const q4k::BlockQ4K* w2, const q4k::BlockQ4K* w3, const q4k::BlockQ8K* xq, uint16_t* y1, uint16_t* y2, uint16_t* y3, int rows1, int rows2, int rows3, int k, int slot, cudaStream_t stream) {
  b200_detail::note(sgr_gemv3m_q4_k_q8_f16out(w1, w2, w3, xq, y1, y2, y3, rows1, rows2, rows3, k, slot, stream));
}
void gemv_q4_k_q8_f16out_resadd(const q4k::BlockQ4K* w, const q4k::BlockQ8K* xq, uint16_t* y, uint16_t* res_inout, int n_rows, int k, cudaStream_t stream) {
  b200_detail::note(sgr_gemv_q4_k_q8_f16out_resadd(w, xq, y, res_inout, n_rows, k, stream));
}
bool tc_gemm_q4_k_f16(const q4k::BlockQ4K* w, const uint16_t* x, uint16_t* y, uint16_t* scratch, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  return sgr_tc_gemm_q4_k_f16(w, x, y, scratch, n_rows, k, n_tokens, stream) == 0;
}
void* tc_handle() { return sgr_tc_handle(); }
size_t tc_scratch_elems(int max_rows, int max_k) { return sgr_tc_scratch_elems(max_rows, max_k); }
bool tc_gemm_f16_raw(const void* w16, const void* x16, void* y16, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  return sgr_tc_gemm_f16_raw(w16, x16, y16, n_rows, k, n_tokens, stream) == 0;
}
void dequant_experts_q4_k_f16(const q4k::BlockQ4K* const* tab_a, const q4k::BlockQ4K* const* tab_b, const int* off, void* slots, long long dst_row0, int rows_sl2, int k, int n_experts, int ring, long long slot_elems, cudaStream_t stream) {
  b200_detail::note(sgr_dequant_experts_q4_k_f16(reinterpret_cast<const void* const*>(tab_a), reinterpret_cast<const void* const*>(tab_b), off, slots, dst_row0, rows_sl2, k, n_experts, ring, slot_elems, stream));
}
bool tc_gemm_f16_f32out_raw(const void* w16, const void* x16, float* y32, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  return sgr_tc_gemm_f16_f32out_raw(w16, x16, y32, n_rows, k, n_tokens, stream) == 0;
}
void tc_router_f32(const float* w_f32, const uint16_t* x, float* y, uint16_t* scratch, int n_rows, int k, int n_tokens, cudaStream_t stream) {
  b200_detail::note(sgr_tc_router_f32(w_f32, x, y, scratch, n_rows, k, n_tokens, stream));
}
#endif  // SAGER_B200_SHIM_IMPLEMENTATION

}  // namespace sager::cuda
