// ref_cuda_wrap.cpp - TEST INFRASTRUCTURE, not part of the product.
//
// Puts the reference's own CUDA launchers (namespace sager::cuda,
// include/sager/kernels/cuda_ops.hpp of the reference) behind the C names of
// include/sager_b200.h, so that a test or the benchmark can load the reference's
// kernels and this library's side by side with one set of prototypes and run the
// same launch sequence on either. Built by oracle/Makefile (target refcuda) together
// with the reference's src/kernels/cuda/{q4_k,mmq,moe,norm_rotary,sampling}.cu, compiled
// where they lie for sm_100a, into oracle/_ref/libsager_ref_cuda.so. The cuBLAS
// family (tc_*) is left out. Every forward returns 0: the reference's launchers
// are void.
#include <stdint.h>

#include "sager/kernels/cuda_ops.hpp"

using namespace sager;

#define SGR_REF_API extern "C" __attribute__((visibility("default")))

SGR_REF_API int sgr_ref_cuda_marker(void) { return 1; }

SGR_REF_API int sgr_quantize_q8_k(const uint16_t* x_f16, void* out_q8, long long n, void* stream) {
  sager::cuda::quantize_q8_k((const uint16_t*)x_f16, (q4k::BlockQ8K*)out_q8, (int)n, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_quantize_q8_k_n(const uint16_t* x_f16, void* out_q8, const int* d_rows, int row_mult, int n_max, void* stream) {
  sager::cuda::quantize_q8_k_n((const uint16_t*)x_f16, (q4k::BlockQ8K*)out_q8, (const int*)d_rows, (int)row_mult, (int)n_max, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_q4_k_q8(const void* w, const void* x_q8, float* y, int n_rows, int k, void* stream) {
  sager::cuda::gemv_q4_k_q8((const q4k::BlockQ4K*)w, (const q4k::BlockQ8K*)x_q8, (float*)y, (int)n_rows, (int)k, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_q4_k_q8_f16out(const void* w, const void* x_q8, uint16_t* y, int n_rows, int k, void* stream) {
  sager::cuda::gemv_q4_k_q8_f16out((const q4k::BlockQ4K*)w, (const q4k::BlockQ8K*)x_q8, (uint16_t*)y, (int)n_rows, (int)k, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_ptrs_q4_k_q8_f16out(const void* const* ptrs, const void* x_q8, uint16_t* y, int n_ptrs, int rows_per, int k, void* stream) {
  sager::cuda::gemv_ptrs_q4_k_q8_f16out((const q4k::BlockQ4K* const*)ptrs, (const q4k::BlockQ8K*)x_q8, (uint16_t*)y, (int)n_ptrs, (int)rows_per, (int)k, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_q4_k_q8_f16out_batched(const void* w, const void* x_q8, uint16_t* y, int n_rows, int k, int n_tokens, void* stream) {
  sager::cuda::gemv_q4_k_q8_f16out_batched((const q4k::BlockQ4K*)w, (const q4k::BlockQ8K*)x_q8, (uint16_t*)y, (int)n_rows, (int)k, (int)n_tokens, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_q4_k_q8_batched(const void* w, const void* x_q8, float* y, int n_rows, int k, int n_tokens, void* stream) {
  sager::cuda::gemv_q4_k_q8_batched((const q4k::BlockQ4K*)w, (const q4k::BlockQ8K*)x_q8, (float*)y, (int)n_rows, (int)k, (int)n_tokens, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_q4_k_q8_f16out_mtok(const void* w, const void* xq, uint16_t* y, int n_rows, int k, int n_tokens, void* stream) {
  sager::cuda::gemv_q4_k_q8_f16out_mtok((const q4k::BlockQ4K*)w, (const q4k::BlockQ8K*)xq, (uint16_t*)y, (int)n_rows, (int)k, (int)n_tokens, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_mmq_q4_k_q8_f16out(const void* w, const void* xq, uint16_t* y, int n_rows, int k, int n_tokens, void* stream) {
  sager::cuda::mmq_q4_k_q8_f16out((const q4k::BlockQ4K*)w, (const q4k::BlockQ8K*)xq, (uint16_t*)y, (int)n_rows, (int)k, (int)n_tokens, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_mmq2_q4_k_q8_f16out(const void* wg, const void* wu, const void* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int n_tokens, void* stream) {
  sager::cuda::mmq2_q4_k_q8_f16out((const q4k::BlockQ4K*)wg, (const q4k::BlockQ4K*)wu, (const q4k::BlockQ8K*)xq, (uint16_t*)yg, (uint16_t*)yu, (int)n_rows, (int)k, (int)n_tokens, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv2_q4_k_q8_f16out_mtok(const void* wg, const void* wu, const void* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int n_tokens, void* stream) {
  sager::cuda::gemv2_q4_k_q8_f16out_mtok((const q4k::BlockQ4K*)wg, (const q4k::BlockQ4K*)wu, (const q4k::BlockQ8K*)xq, (uint16_t*)yg, (uint16_t*)yu, (int)n_rows, (int)k, (int)n_tokens, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_grouped2_q4_k_q8_f16out_mtok(const void* const* wg, const void* const* wu, const int* off, const int* m, const int* tile_base, const int* job_of_tile, int n_tiles, const void* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int tok_per, void* stream) {
  sager::cuda::gemv_grouped2_q4_k_q8_f16out_mtok((const q4k::BlockQ4K* const*)wg, (const q4k::BlockQ4K* const*)wu, (const int*)off, (const int*)m, (const int*)tile_base, (const int*)job_of_tile, (int)n_tiles, (const q4k::BlockQ8K*)xq, (uint16_t*)yg, (uint16_t*)yu, (int)n_rows, (int)k, (int)tok_per, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_grouped_q4_k_q8_f16out_mtok(const void* const* w, const int* off, const int* m, const int* tile_base, const int* job_of_tile, int n_tiles, const void* xq, uint16_t* y, int n_rows, int k, int tok_per, void* stream) {
  sager::cuda::gemv_grouped_q4_k_q8_f16out_mtok((const q4k::BlockQ4K* const*)w, (const int*)off, (const int*)m, (const int*)tile_base, (const int*)job_of_tile, (int)n_tiles, (const q4k::BlockQ8K*)xq, (uint16_t*)y, (int)n_rows, (int)k, (int)tok_per, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_grouped2_tab_q4_k_q8_f16out_mtok(const void* const* wg_tab, const void* const* wu_tab, const int* off, const int* toff, const int* meta, int* mail, int* mail_n, int tiles_max, const void* xq, uint16_t* yg, uint16_t* yu, int n_rows, int k, int n_expert, int tok_per, void* stream) {
  sager::cuda::gemv_grouped2_tab_q4_k_q8_f16out_mtok((const q4k::BlockQ4K* const*)wg_tab, (const q4k::BlockQ4K* const*)wu_tab, (const int*)off, (const int*)toff, (const int*)meta, (int*)mail, (int*)mail_n, (int)tiles_max, (const q4k::BlockQ8K*)xq, (uint16_t*)yg, (uint16_t*)yu, (int)n_rows, (int)k, (int)n_expert, (int)tok_per, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_grouped_tab_q4_k_q8_f16out_mtok(const void* const* w_tab, const int* off, const int* toff, const int* meta, int tiles_max, const void* xq, uint16_t* y, int n_rows, int k, int n_expert, int tok_per, void* stream) {
  sager::cuda::gemv_grouped_tab_q4_k_q8_f16out_mtok((const q4k::BlockQ4K* const*)w_tab, (const int*)off, (const int*)toff, (const int*)meta, (int)tiles_max, (const q4k::BlockQ8K*)xq, (uint16_t*)y, (int)n_rows, (int)k, (int)n_expert, (int)tok_per, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_f32_out_f16x(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k, void* stream) {
  sager::cuda::gemv_f32_out_f16x((const float*)w_f32, (const uint16_t*)x_f16, (float*)y, (int)n_rows, (int)k, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_f32_out_f16x_batched(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k, int n_tokens, void* stream) {
  sager::cuda::gemv_f32_out_f16x_batched((const float*)w_f32, (const uint16_t*)x_f16, (float*)y, (int)n_rows, (int)k, (int)n_tokens, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_f32_out_f16x_mtok(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k, int n_tokens, void* stream) {
  sager::cuda::gemv_f32_out_f16x_mtok((const float*)w_f32, (const uint16_t*)x_f16, (float*)y, (int)n_rows, (int)k, (int)n_tokens, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_router_topk(const float* logits, int* idx, float* weight, int n_expert, int n_expert_used, float shared_w, void* stream) {
  sager::cuda::router_topk((const float*)logits, (int*)idx, (float*)weight, (int)n_expert, (int)n_expert_used, (float)shared_w, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_router_topk_batched(const float* logits, int* idx, float* weight, int n_expert, int n_expert_used, int idx_stride, int n_rows, float shared_w, void* stream) {
  sager::cuda::router_topk_batched((const float*)logits, (int*)idx, (float*)weight, (int)n_expert, (int)n_expert_used, (int)idx_stride, (int)n_rows, (float)shared_w, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_router_topk_fused(const float* w_f32, const uint16_t* x_f16, int* idx, float* weight, int n_expert, int n_expert_used, int hidden, void* stream) {
  sager::cuda::router_topk_fused((const float*)w_f32, (const uint16_t*)x_f16, (int*)idx, (float*)weight, (int)n_expert, (int)n_expert_used, (int)hidden, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_moe_dispatch_scan(const int* idx, float* weight, int* gslot, int* grows, int* off, int* toff, int* meta, int* mail, int* mail_n, int n_rows, int k, int n_expert, int tok_per, void* stream) {
  sager::cuda::moe_dispatch_scan((const int*)idx, (float*)weight, (int*)gslot, (int*)grows, (int*)off, (int*)toff, (int*)meta, (int*)mail, (int*)mail_n, (int)n_rows, (int)k, (int)n_expert, (int)tok_per, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gather_rows_q8(void* dst, const void* src, const int* src_rows, int n_rows, int row_blocks, void* stream) {
  sager::cuda::gather_rows_q8((q4k::BlockQ8K*)dst, (const q4k::BlockQ8K*)src, (const int*)src_rows, (int)n_rows, (int)row_blocks, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gather_rows_q8_n(void* dst, const void* src, const int* src_rows, const int* meta, int r_max, int row_blocks, void* stream) {
  sager::cuda::gather_rows_q8_n((q4k::BlockQ8K*)dst, (const q4k::BlockQ8K*)src, (const int*)src_rows, (const int*)meta, (int)r_max, (int)row_blocks, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gather_rows_f16_n(uint16_t* dst, const uint16_t* src, const int* src_rows, const int* meta, int r_max, int hidden, void* stream) {
  sager::cuda::gather_rows_f16_n((uint16_t*)dst, (const uint16_t*)src, (const int*)src_rows, (const int*)meta, (int)r_max, (int)hidden, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_scatter_rows_f16(uint16_t* dst, const uint16_t* src, const int* dst_rows, int n_rows, int hidden, void* stream) {
  sager::cuda::scatter_rows_f16((uint16_t*)dst, (const uint16_t*)src, (const int*)dst_rows, (int)n_rows, (int)hidden, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_scatter_routed_f16(uint16_t* expert_y, const uint16_t* grouped_out, const int* gslot, int n_rows, int n_used, int hidden, void* stream) {
  sager::cuda::scatter_routed_f16((uint16_t*)expert_y, (const uint16_t*)grouped_out, (const int*)gslot, (int)n_rows, (int)n_used, (int)hidden, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_scatter_miss_f32(uint16_t* expert_out, const int* d_slot_of_k, const float* miss_y, int k_rows, int hidden, void* stream) {
  sager::cuda::scatter_miss_f32((uint16_t*)expert_out, (const int*)d_slot_of_k, (const float*)miss_y, (int)k_rows, (int)hidden, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_scatter_rows_generic_f16(uint16_t* dst, const float* src, const int* dst_flat, int n_list, int hidden, void* stream) {
  sager::cuda::scatter_rows_generic_f16((uint16_t*)dst, (const float*)src, (const int*)dst_flat, (int)n_list, (int)hidden, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_silu_mul_f16(uint16_t* out, const uint16_t* g, const uint16_t* u, int rows, int n_ff, void* stream) {
  sager::cuda::silu_mul_f16((uint16_t*)out, (const uint16_t*)g, (const uint16_t*)u, (int)rows, (int)n_ff, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_silu_mul_f16_n(uint16_t* out, const uint16_t* g, const uint16_t* u, const int* d_rows, int rows_max, int n_ff, void* stream) {
  sager::cuda::silu_mul_f16_n((uint16_t*)out, (const uint16_t*)g, (const uint16_t*)u, (const int*)d_rows, (int)rows_max, (int)n_ff, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_sigmoid_gate_scalar_f16(uint16_t* out, const float* g, int n, void* stream) {
  sager::cuda::sigmoid_gate_scalar_f16((uint16_t*)out, (const float*)g, (int)n, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_sigmoid_gate_scalar_batched_f16(uint16_t* out, const float* g, int n_rows, int hidden, void* stream) {
  sager::cuda::sigmoid_gate_scalar_batched_f16((uint16_t*)out, (const float*)g, (int)n_rows, (int)hidden, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_moe_combine_f16(uint16_t* out, const uint16_t* expert_out, const int* idx, const float* weight, int n_expert_used, int hidden, void* stream) {
  sager::cuda::moe_combine_f16((uint16_t*)out, (const uint16_t*)expert_out, (const int*)idx, (const float*)weight, (int)n_expert_used, (int)hidden, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_moe_combine_batched_f16(uint16_t* out, const uint16_t* expert_y, const float* weight, int n_used, int hidden, int n_rows, void* stream) {
  sager::cuda::moe_combine_batched_f16((uint16_t*)out, (const uint16_t*)expert_y, (const float*)weight, (int)n_used, (int)hidden, (int)n_rows, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_moe_combine_add_slots_f16(uint16_t* out, const uint16_t* expert_y, const float* weight, const int* rk, int n_used, int hidden, int n_list, void* stream) {
  sager::cuda::moe_combine_add_slots_f16((uint16_t*)out, (const uint16_t*)expert_y, (const float*)weight, (const int*)rk, (int)n_used, (int)hidden, (int)n_list, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_q6_k_q8(const void* w_q6, const void* x_q8, float* y, int n_rows, int k, void* stream) {
  sager::cuda::gemv_q6_k_q8((const void*)w_q6, (const q4k::BlockQ8K*)x_q8, (float*)y, (int)n_rows, (int)k, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_q6_k_q8_smx(const void* w_q6, const void* x_q8, float* y, int n_rows, int k, void* stream) {
  sager::cuda::gemv_q6_k_q8_smx((const void*)w_q6, (const q4k::BlockQ8K*)x_q8, (float*)y, (int)n_rows, (int)k, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_topk_select_f32_2p(const float* logits, float* seg_v, int* seg_i, int seg_slots, float* out_v, int* out_i, int n, int k, void* stream) {
  sager::cuda::topk_select_f32_2p((const float*)logits, (float*)seg_v, (int*)seg_i, (int)seg_slots, (float*)out_v, (int*)out_i, (int)n, (int)k, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_rmsnorm_quant_f16(uint16_t* out, const uint16_t* x, const uint16_t* w, void* xq, int n, float eps, int n_rows, void* stream) {
  sager::cuda::rmsnorm_quant_f16((uint16_t*)out, (const uint16_t*)x, (const uint16_t*)w, (q4k::BlockQ8K*)xq, (int)n, (float)eps, (int)n_rows, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv2m_q4_k_q8_f16out(const void* w1, const void* w2, const void* xq, uint16_t* y1, uint16_t* y2, int rows1, int rows2, int k, int slot, void* stream) {
  sager::cuda::gemv2m_q4_k_q8_f16out((const q4k::BlockQ4K*)w1, (const q4k::BlockQ4K*)w2, (const q4k::BlockQ8K*)xq, (uint16_t*)y1, (uint16_t*)y2, (int)rows1, (int)rows2, (int)k, (int)slot, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv3m_q4_k_q8_f16out(const void* w1, const void* w2, const void* w3, const void* xq, uint16_t* y1, uint16_t* y2, uint16_t* y3, int rows1, int rows2, int rows3, int k, int slot, void* stream) {
  sager::cuda::gemv3m_q4_k_q8_f16out((const q4k::BlockQ4K*)w1, (const q4k::BlockQ4K*)w2, (const q4k::BlockQ4K*)w3, (const q4k::BlockQ8K*)xq, (uint16_t*)y1, (uint16_t*)y2, (uint16_t*)y3, (int)rows1, (int)rows2, (int)rows3, (int)k, (int)slot, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_gemv_q4_k_q8_f16out_resadd(const void* w, const void* x_q8, uint16_t* y, uint16_t* res_inout, int n_rows, int k, void* stream) {
  sager::cuda::gemv_q4_k_q8_f16out_resadd((const q4k::BlockQ4K*)w, (const q4k::BlockQ8K*)x_q8, (uint16_t*)y, (uint16_t*)res_inout, (int)n_rows, (int)k, (cudaStream_t)stream);
  return 0;
}


// Reference-only pieces that the fused launchers are specified against (the two-kernel sequences
// they replace): the unfused RMS norm and the fp16 add. No counterpart in include/sager_b200.h.
SGR_REF_API int sgr_ref_rmsnorm_batched_f16(uint16_t* out, const uint16_t* x, const uint16_t* w, int n, float eps, int n_rows, void* stream) {
  sager::cuda::rmsnorm_batched_f16(out, x, w, n, eps, n_rows, (cudaStream_t)stream);
  return 0;
}

SGR_REF_API int sgr_ref_add_f16(uint16_t* in_out, const uint16_t* residual, int n, void* stream) {
  sager::cuda::add_f16(in_out, residual, n, (cudaStream_t)stream);
  return 0;
}
