/*
 * sager_b200.h - C ABI of libsager_b200.so: the B200 (sm_100a) implementation of
 * SAGER's Q4_K mixture-of-experts hot path.
 *
 * Every function replaces one launcher of the reference's device interface
 * (include/sager/kernels/cuda_ops.hpp, namespace sager::cuda); the citation
 * beside each declaration names it. Parameter lists are the reference's, with
 * three mechanical changes that make them C: block types become `const void*`
 * (Q4_K super-blocks of 144 bytes, Q8_K activation blocks of 276 bytes, layouts
 * as in include/sager/kernels/q4_k.hpp:45-63), `cudaStream_t` becomes `void*`,
 * and the return type is `int` instead of `void` (0 = launched; otherwise one
 * of the SGR_E* codes - argument validation only, nothing is synchronised).
 * include/sager_b200_shim.hpp turns these back into the C++ signatures.
 *
 * Conventions kept from the reference (cuda_ops.hpp:1-14): all calls are
 * stream-ordered and never synchronise; all buffers are caller-owned device
 * pointers; per-step values (row counts, tile counts, residency) are read from
 * fixed-address device memory, so every call is legal inside stream capture -
 * with one exception: the first call of the library on a device looks up the
 * address of its status word (cudaGetSymbolAddress) and must be made outside
 * capture; until that has happened the entry points that need the word return
 * SGR_ELAUNCH inside a capture.
 * fp16 values travel as uint16_t. A null pointer-table entry means "expert
 * not resident": its output rows are written as zero and, for the gate/up
 * call, the expert id is posted to the mailbox.
 */
#ifndef SAGER_B200_H_
#define SAGER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SGR_OK 0
#define SGR_EARG 1         /* null pointer, non-positive size, k not a multiple of 256 */
#define SGR_EALIGN 2       /* activation blocks must be 4-byte aligned, fp16 rows 2-byte */
#define SGR_EUNSUPPORTED 3 /* shape outside what the kernels were built for */
#define SGR_ELAUNCH 4      /* the CUDA runtime refused the launch */
#define SGR_EGEOMETRY 5    /* fused entry point: geometry mismatch (refused, never misindexed) */
#define SGR_ESTATICLIMIT 6 /* sgr_moe_layer_decode_static: the shape needs more scratch than the
                              library's built-in array holds (sgr_moe_layer_static_limit bytes) */

int sgr_abi_version(void);
/* Device status word of the current device: non-zero after a bounded device-side
 * wait gave up. Synchronises; diagnostics only. clear != 0 resets it. */
int sgr_status(int clear);

/* ---- activation quantiser ------------------------------------------------------ */
/* cuda_ops.hpp:272  quantize_q8_k(x_f16, out, n, stream) */
int sgr_quantize_q8_k(const uint16_t* x_f16, void* out_q8, long long n, void* stream);
/* cuda_ops.hpp:235  quantize_q8_k_n(x_f16, out, d_rows, row_mult, n_max, stream) */
int sgr_quantize_q8_k_n(const uint16_t* x_f16, void* out_q8, const int* d_rows, int row_mult,
                        int n_max, void* stream);

/* cuda_ops.hpp:149  rmsnorm_quant_f16: out = f16(x * rsqrt(mean(x^2) + eps) * w) per row of n values and the
 * Q8_K blocks of out, in one launch; bit-identical to the norm followed by the quantiser. n % 256 == 0
 * (the reference's fallback for other n is its unfused norm kernel, which this library does not hold:
 * SGR_EUNSUPPORTED). */
int sgr_rmsnorm_quant_f16(uint16_t* out, const uint16_t* x, const uint16_t* w, void* xq, int n, float eps,
                          int n_rows, void* stream);

/* ---- Q4_K x Q8_K GEMV family --------------------------------------------------- */
/* cuda_ops.hpp:41   gemv_q4_k_q8 (fp32 out) */
int sgr_gemv_q4_k_q8(const void* w, const void* x_q8, float* y, int n_rows, int k, void* stream);
/* cuda_ops.hpp:53   gemv_q4_k_q8_f16out */
int sgr_gemv_q4_k_q8_f16out(const void* w, const void* x_q8, uint16_t* y, int n_rows, int k,
                            void* stream);
/* cuda_ops.hpp:60   gemv_ptrs_q4_k_q8_f16out: y[e*rows_per + r]; every pointer reads
 * the same activation row, exactly as the reference kernel does. */
int sgr_gemv_ptrs_q4_k_q8_f16out(const void* const* ptrs, const void* x_q8, uint16_t* y,
                                 int n_ptrs, int rows_per, int k, void* stream);
/* cuda_ops.hpp:67   gemv_q4_k_q8_f16out_batched: y[tok*n_rows + row] */
int sgr_gemv_q4_k_q8_f16out_batched(const void* w, const void* x_q8, uint16_t* y, int n_rows,
                                    int k, int n_tokens, void* stream);
/* cuda_ops.hpp:72   gemv_q4_k_q8_batched (fp32 out) */
int sgr_gemv_q4_k_q8_batched(const void* w, const void* x_q8, float* y, int n_rows, int k,
                             int n_tokens, void* stream);
/* cuda_ops.hpp:88   gemv_q4_k_q8_f16out_mtok */
int sgr_gemv_q4_k_q8_f16out_mtok(const void* w, const void* xq, uint16_t* y, int n_rows, int k,
                                 int n_tokens, void* stream);
/* cuda_ops.hpp:95   mmq_q4_k_q8_f16out */
int sgr_mmq_q4_k_q8_f16out(const void* w, const void* xq, uint16_t* y, int n_rows, int k,
                           int n_tokens, void* stream);
/* cuda_ops.hpp:100  mmq2_q4_k_q8_f16out (gate + up in one launch) */
int sgr_mmq2_q4_k_q8_f16out(const void* wg, const void* wu, const void* xq, uint16_t* yg,
                            uint16_t* yu, int n_rows, int k, int n_tokens, void* stream);
/* cuda_ops.hpp:186  gemv2_q4_k_q8_f16out_mtok */
int sgr_gemv2_q4_k_q8_f16out_mtok(const void* wg, const void* wu, const void* xq, uint16_t* yg,
                                  uint16_t* yu, int n_rows, int k, int n_tokens, void* stream);
/* cuda_ops.hpp:195  gemv_grouped2_q4_k_q8_f16out_mtok (host plan) */
int sgr_gemv_grouped2_q4_k_q8_f16out_mtok(const void* const* wg, const void* const* wu,
                                          const int* off, const int* m, const int* tile_base,
                                          const int* job_of_tile, int n_tiles, const void* xq,
                                          uint16_t* yg, uint16_t* yu, int n_rows, int k,
                                          int tok_per, void* stream);
/* cuda_ops.hpp:203  gemv_grouped_q4_k_q8_f16out_mtok (host plan, down projection) */
int sgr_gemv_grouped_q4_k_q8_f16out_mtok(const void* const* w, const int* off, const int* m,
                                         const int* tile_base, const int* job_of_tile,
                                         int n_tiles, const void* xq, uint16_t* y, int n_rows,
                                         int k, int tok_per, void* stream);
/* cuda_ops.hpp:240  gemv_grouped2_tab_q4_k_q8_f16out_mtok (device plan + pointer table) */
int sgr_gemv_grouped2_tab_q4_k_q8_f16out_mtok(const void* const* wg_tab,
                                              const void* const* wu_tab, const int* off,
                                              const int* toff, const int* meta, int* mail,
                                              int* mail_n, int tiles_max, const void* xq,
                                              uint16_t* yg, uint16_t* yu, int n_rows, int k,
                                              int n_expert, int tok_per, void* stream);
/* cuda_ops.hpp:247  gemv_grouped_tab_q4_k_q8_f16out_mtok (device plan, down projection) */
int sgr_gemv_grouped_tab_q4_k_q8_f16out_mtok(const void* const* w_tab, const int* off,
                                             const int* toff, const int* meta, int tiles_max,
                                             const void* xq, uint16_t* y, int n_rows, int k,
                                             int n_expert, int tok_per, void* stream);
/* cuda_ops.hpp:169  gemv_q4_k_q8_f16out_resadd: y as gemv_q4_k_q8_f16out, then
 * res_inout[i] = f16(f32(res_inout[i]) + f32(y[i])); one token row. */
int sgr_gemv_q4_k_q8_f16out_resadd(const void* w, const void* x_q8, uint16_t* y, uint16_t* res_inout,
                                   int n_rows, int k, void* stream);
/* cuda_ops.hpp:156  gemv2m_q4_k_q8_f16out: two projections of one token row in one launch
 * (`slot` is accepted and ignored: there is no per-layer parameter block to key). */
int sgr_gemv2m_q4_k_q8_f16out(const void* w1, const void* w2, const void* xq, uint16_t* y1, uint16_t* y2,
                              int rows1, int rows2, int k, int slot, void* stream);
/* cuda_ops.hpp:160  gemv3m_q4_k_q8_f16out: three projections. */
int sgr_gemv3m_q4_k_q8_f16out(const void* w1, const void* w2, const void* w3, const void* xq, uint16_t* y1,
                              uint16_t* y2, uint16_t* y3, int rows1, int rows2, int rows3, int k, int slot,
                              void* stream);
/* Parity probe, no counterpart launcher: the raw int32 sub-block dots of one
 * activation row, out[(row*nb + blk)*8 + s] - the unit src/kernels/cuda/q4_k.cu:38-53
 * and src/kernels/cpu/q4_avx2.cpp:99-119 both compute. */
int sgr_q4k_subblock_dots(const void* w, const void* x_q8, int* out, int n_rows, int k,
                          void* stream);

/* ---- LM head on Q6_K weights and the candidate selection after it -------------------- */
/* cuda_ops.hpp:48   gemv_q6_k_q8: y[row] = W6[row] . x, W6 in raw block_q6_K bytes (210 per 256 weights) */
int sgr_gemv_q6_k_q8(const void* w_q6, const void* x_q8, float* y, int n_rows, int k, void* stream);
/* cuda_ops.hpp:181  gemv_q6_k_q8_smx: the same (bit-identical to sgr_gemv_q6_k_q8) */
int sgr_gemv_q6_k_q8_smx(const void* w_q6, const void* x_q8, float* y, int n_rows, int k, void* stream);
/* cuda_ops.hpp:436  topk_select_f32_2p: the k <= 64 largest logits in descending order, ties by lower
 * index; seg_v / seg_i: scratch of at least ceil(n / 2048) * k slots (SGR_EUNSUPPORTED when smaller).
 * The logits are left as they are. */
int sgr_topk_select_f32_2p(const float* logits, float* seg_v, int* seg_i, int seg_slots, float* out_v,
                           int* out_i, int n, int k, void* stream);

/* ---- router --------------------------------------------------------------------- */
/* cuda_ops.hpp:277  gemv_f32_out_f16x */
int sgr_gemv_f32_out_f16x(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows, int k,
                          void* stream);
/* cuda_ops.hpp:77   gemv_f32_out_f16x_batched */
int sgr_gemv_f32_out_f16x_batched(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows,
                                  int k, int n_tokens, void* stream);
/* cuda_ops.hpp:262  gemv_f32_out_f16x_mtok */
int sgr_gemv_f32_out_f16x_mtok(const float* w_f32, const uint16_t* x_f16, float* y, int n_rows,
                               int k, int n_tokens, void* stream);
/* cuda_ops.hpp:351  router_topk */
int sgr_router_topk(const float* logits, int* idx, float* weight, int n_expert,
                    int n_expert_used, float shared_w, void* stream);
/* cuda_ops.hpp:358  router_topk_batched */
int sgr_router_topk_batched(const float* logits, int* idx, float* weight, int n_expert,
                            int n_expert_used, int idx_stride, int n_rows, float shared_w,
                            void* stream);
/* cuda_ops.hpp:175  router_topk_fused (does not write slot K) */
int sgr_router_topk_fused(const float* w_f32, const uint16_t* x_f16, int* idx, float* weight,
                          int n_expert, int n_expert_used, int hidden, void* stream);

/* ---- plan, row movement, SwiGLU, combine ------------------------------------------ */
/* cuda_ops.hpp:219  moe_dispatch_scan */
int sgr_moe_dispatch_scan(const int* idx, float* weight, int* gslot, int* grows, int* off,
                          int* toff, int* meta, int* mail, int* mail_n, int n_rows, int k,
                          int n_expert, int tok_per, void* stream);
/* cuda_ops.hpp:364  gather_rows_q8 */
int sgr_gather_rows_q8(void* dst, const void* src, const int* src_rows, int n_rows,
                       int row_blocks, void* stream);
/* cuda_ops.hpp:226  gather_rows_q8_n */
int sgr_gather_rows_q8_n(void* dst, const void* src, const int* src_rows, const int* meta,
                         int r_max, int row_blocks, void* stream);
/* cuda_ops.hpp:229  gather_rows_f16_n */
int sgr_gather_rows_f16_n(uint16_t* dst, const uint16_t* src, const int* src_rows,
                          const int* meta, int r_max, int hidden, void* stream);
/* cuda_ops.hpp:408  scatter_rows_f16 */
int sgr_scatter_rows_f16(uint16_t* dst, const uint16_t* src, const int* dst_rows, int n_rows,
                         int hidden, void* stream);
/* cuda_ops.hpp:372  scatter_routed_f16 */
int sgr_scatter_routed_f16(uint16_t* expert_y, const uint16_t* grouped_out, const int* gslot,
                           int n_rows, int n_used, int hidden, void* stream);
/* cuda_ops.hpp:403  scatter_miss_f32 */
int sgr_scatter_miss_f32(uint16_t* expert_out, const int* d_slot_of_k, const float* miss_y,
                         int k_rows, int hidden, void* stream);
/* cuda_ops.hpp:391  scatter_rows_generic_f16 */
int sgr_scatter_rows_generic_f16(uint16_t* dst, const float* src, const int* dst_flat,
                                 int n_list, int hidden, void* stream);
/* cuda_ops.hpp:305  silu_mul_f16 */
int sgr_silu_mul_f16(uint16_t* out, const uint16_t* g, const uint16_t* u, int rows, int n_ff,
                     void* stream);
/* cuda_ops.hpp:232  silu_mul_f16_n */
int sgr_silu_mul_f16_n(uint16_t* out, const uint16_t* g, const uint16_t* u, const int* d_rows,
                       int rows_max, int n_ff, void* stream);
/* cuda_ops.hpp:315  sigmoid_gate_scalar_f16 */
int sgr_sigmoid_gate_scalar_f16(uint16_t* out, const float* g, int n, void* stream);
/* cuda_ops.hpp:384  sigmoid_gate_scalar_batched_f16 */
int sgr_sigmoid_gate_scalar_batched_f16(uint16_t* out, const float* g, int n_rows, int hidden,
                                        void* stream);
/* cuda_ops.hpp:397  moe_combine_f16 */
int sgr_moe_combine_f16(uint16_t* out, const uint16_t* expert_out, const int* idx,
                        const float* weight, int n_expert_used, int hidden, void* stream);
/* cuda_ops.hpp:379  moe_combine_batched_f16 */
int sgr_moe_combine_batched_f16(uint16_t* out, const uint16_t* expert_y, const float* weight,
                                int n_used, int hidden, int n_rows, void* stream);
/* cuda_ops.hpp:255  moe_combine_add_slots_f16 */
int sgr_moe_combine_add_slots_f16(uint16_t* out, const uint16_t* expert_y, const float* weight,
                                  const int* rk, int n_used, int hidden, int n_list,
                                  void* stream);

/* ---- one MoE layer of a decode step, fused ------------------------------------------
 * Replaces the launch sequence of Session::moe_dispatch_device for n <= 64 token rows
 * (src/core/session.cpp:2482-3030 of the reference; the launchers it strings together
 * are listed at the top of csrc/moe_layer.cu) with two dependent launches. Same
 * contracts: xn fp16 rows, router [E][H] fp32, [3][E] pointer table (gate, up, down;
 * null = expert absent: zero contribution, id posted to mail[]), route_idx / route_w
 * rows of stride K+1 with slot K = shared_w, residual stream x_f16 updated in place.
 * Intermediate g, u, h, y stay fp32 (the arithmetic of the CPU expert FFN,
 * src/kernels/cpu/q4_avx2.cpp:175-196).
 *
 * Expert parallelism: only routes to experts in [expert_lo, expert_hi) are computed
 * (expert_hi == 0 means n_expert) and the shared expert only for rows
 * [shared_lo, shared_hi) (shared_hi == 0 means n). With routing_given != 0 the router
 * is skipped: route_idx / route_w and xq_in (packed Q8_K rows) are inputs. With
 * no_residual != 0 out_f32 receives the weighted expert sum alone.
 *
 * The workspace (size from sgr_moe_layer_workspace_bytes, 256-byte aligned) must be
 * cleared once with sgr_moe_layer_workspace_init before its first use; one layer call
 * may be in flight per workspace. */
typedef struct sgr_moe_layer {
  int n;                 /* token rows this call, 1..n_max */
  int n_max;             /* rows the workspace was sized for, <= 64 */
  int hidden, n_ff, n_expert, n_used;
  int expert_lo, expert_hi;
  int shared_lo, shared_hi;
  int routing_given;
  int no_residual;
  float shared_w;        /* written to route_w[row][K] by the router */
  const uint16_t* xn;    /* [n][hidden] fp16, 16-byte aligned */
  const void* xq_in;     /* optional [n][hidden/256] Q8_K blocks: skip the quantiser */
  const float* router_w; /* [n_expert][hidden] */
  const float* router_bias; /* optional [n_expert], added to the logits */
  const void* const* w_tab; /* [3][n_expert] device pointers to Q4_K matrices (slices tab_stride apart) */
  const void* shared_gate;  /* shared expert matrices, or all NULL */
  const void* shared_up;
  const void* shared_down;
  uint16_t* x_f16;       /* optional [n][hidden]: residual in, residual + MoE out (4-byte aligned) */
  float* out_f32;        /* optional [n][hidden] fp32 copy of the result (8-byte aligned) */
  int* route_idx;        /* [n][n_used+1] */
  float* route_w;        /* [n][n_used+1] */
  int* mail;             /* optional [n_expert] absent-expert mailbox */
  int* mail_n;           /* [1], reset by every call */
  void* workspace;
  size_t workspace_bytes;
  /* row strides for records that travel between ranks; 0 = packed */
  int route_stride;      /* elements between rows of route_idx / route_w (default n_used+1) */
  int xq_stride;         /* bytes between Q8_K rows of xq_in / xq_out (default hidden/256*276) */
  void* xq_out;          /* optional: the router's Q8_K rows are written here, not to the workspace */
  /* expert parallelism over peer memory: with routing_given, the plan first waits (bounded) until
   * each of the wait_count words at wait_flags is >= *wait_step * wait_mul + wait_add - the arrival
   * flags that sgr_ep_push sets on this rank. wait_flags == NULL: no wait. */
  const unsigned* wait_flags;
  const unsigned* wait_step;
  int wait_count, wait_mul, wait_add;
  /* records between ranks may carry the Q8_K rows in 288-byte blocks (d | 12 bytes | 256 codes |
   * 8 sums, 16-byte aligned) instead of packed 276-byte ones: set for both the route stage that
   * writes them (xq_out) and the owner that reads them (xq_in, routing_given, >= 4 rows). */
  int xq_padded;
  /* pointers between the gate, up and down slices of w_tab; 0 = n_expert (a packed [3][E] table).
   * The reference's decode table is [3][Lm][E] (src/core/session.cpp:3596-3598): pass
   * w_tab = table + layer * E and tab_stride = Lm * E to use it in place. */
  long long tab_stride;
  /* Expert parallelism with both exchanges done by the layer's own kernels over peer memory (all
   * NULL / 0: off). ep_flags[p] is this rank's address of an arrival word of rank p, set to
   * *ep_step * ep_mul + ep_add by the kernel's last CTA (an acq_rel count of the CTAs that stored, one
   * system-scope fence, then the words as relaxed stores) once the data are there.
   *   home side (stages 1 | 8 with xq_out = the record block of ep_rec_bytes per row): after the
   *     selection the records are stored into ep_dst[p] (this rank's slot in rank p's receive
   *     buffer) for every p < ep_world, then the owners' words are set;
   *   owner side (routing_given): row t of the result is stored to
   *     ep_out[t / ep_home_rows] + (t % ep_home_rows) * hidden (this rank's slot in the home rank's
   *     return buffer) instead of out_f32, then the home ranks' words are set.
   * ep_out[p] 8-byte aligned. Plain stores to peer memory only: no multicast, no library kernel
   * touches a peer's memory. */
  void* const* ep_dst;
  unsigned* const* ep_flags;
  float* const* ep_out;
  const unsigned* ep_step;
  int ep_world, ep_rec_bytes, ep_home_rows, ep_mul, ep_add;
  /* Expert parallelism, one launch less on the owner side: the route stage of this (home) call also
   * re-arms the counters of a second workspace - that of the owner call which follows it on the same
   * stream, made for rearm_n_max rows and otherwise this call's geometry - and clears that call's
   * mailbox count. The owner call may then be issued as stages 2 | 4 | 128: no plan launch, every CTA of
   * its expert kernel waits for the arrival words and plans for itself. NULL / 0: off. */
  void* rearm_workspace;
  int* rearm_mail_n;
  int rearm_n_max;
} sgr_moe_layer;

size_t sgr_moe_layer_workspace_bytes(int n_max, int hidden, int n_ff, int n_expert, int n_used);
int sgr_moe_layer_workspace_init(void* workspace, size_t bytes, void* stream);
int sgr_moe_layer_decode(const sgr_moe_layer* args, void* stream);
/* The same layer, only the launches named in `stages` (1 = route/plan, 2 or 4 or 6 =
 * the expert kernel, 1|8 = route without building the plan), on a workspace that still
 * holds what the earlier stage of a previous call left there. For measuring one kernel
 * at a time and for the home side of an expert-parallel layer. */
int sgr_moe_layer_decode_stages(const sgr_moe_layer* args, int stages, void* stream);

/* Prefill grouped GEMM on int8 tensor cores (tcgen05, accumulators in tensor memory).
 * Replaces dequant_experts_q4_k_f16 + tc_gemm_f16_raw (cuda_ops.hpp:125-131, one cuBLAS GEMM per
 * expert and matrix) with the contract of gemv_grouped_tab_q4_k_q8_f16out_mtok (cuda_ops.hpp:247):
 * xq is the expert-major slab of Q8_K rows, off[n_expert+1] the row prefix of the device plan,
 * y[off[e]+t][r] = W_e[r] . xq[off[e]+t] in fp16; a null table entry gives zero rows. The integer
 * arithmetic is that of the Q4_K x Q8_K path (exact sub-block dots), not of the fp16 GEMM. */
int sgr_moe_grouped_gemm_i8(const void* const* w_tab, const int* off, const void* xq, uint16_t* y,
                            int n_rows, int k, int n_expert, void* stream);

/* ---- one MoE layer over a prefill chunk, behind one call -----------------------------------
 * The launch sequence of Session::moe_dispatch_device for a chunk of n token rows
 * (src/core/session.cpp:2482-3030 of the reference) on the session's own scratch buffers
 * (src/core/session.cpp:207-257; shapes below with R = n_max * n_used): quantise, router logits,
 * top-k, device plan, gather, gate / up, SwiGLU, requantise, down, scatter, shared expert,
 * combine into x_f16. The routed projections run on sgr_moe_grouped_gemm_i8; every other step is
 * the library's launcher of the same name. Stream-ordered, allocates nothing. */
typedef struct sgr_moe_prefill {
  int n, n_max;             /* token rows of this chunk / rows the buffers were sized for */
  int hidden, n_ff, n_expert, n_used;
  int tok_per;              /* rows per tile of the device plan (0 = 16) */
  float shared_w;           /* weight of the shared expert (slot K of route_w), 1.0 in the reference */
  const uint16_t* xn;       /* [n][hidden] fp16 layer input */
  const float* router_w;    /* [n_expert][hidden]; unused when logits_in is given */
  const float* logits_in;   /* optional [n][n_expert]: skip the router GEMV */
  const void* const* w_tab; /* gate / up / down slices of n_expert pointers, tab_stride apart */
  long long tab_stride;     /* 0 = n_expert */
  const void* shared_gate;  /* shared expert matrices, or all NULL */
  const void* shared_up;
  const void* shared_down;
  const float* shared_gate_w; /* optional [hidden] scalar gate of the shared expert (needs sgate) */
  uint16_t* x_f16;          /* [n][hidden] residual stream, combined in place */
  void* xq;                 /* [n_max][hidden/256] Q8_K blocks */
  float* logits;            /* [n_max][n_expert] */
  int* route_idx;           /* [n_max][n_used+1] */
  float* route_w;           /* [n_max][n_used+1] */
  int* gslot;               /* [R] */
  int* grows;               /* [R] */
  int* off;                 /* [n_expert+1] */
  int* toff;                /* [n_expert+1] */
  int* meta;                /* [4] */
  int* mail;                /* [n_expert] */
  int* mail_n;              /* [1] */
  void* xqg;                /* [R][hidden/256] Q8_K blocks, 16-byte aligned */
  uint16_t* g;              /* [R][n_ff] */
  uint16_t* u;              /* [R][n_ff] */
  void* hq;                 /* [R][n_ff/256] Q8_K blocks, 16-byte aligned */
  uint16_t* y_grouped;      /* [R][hidden] */
  uint16_t* expert_y;       /* [n_max][n_used+1][hidden] combine slab: used only when x_f16, y_grouped or sh_y is
                               not 16-byte aligned - otherwise the combine reads the grouped rows in place */
  uint16_t* sh_g;           /* [n_max][n_ff] */
  uint16_t* sh_u;           /* [n_max][n_ff] */
  void* sh_q;               /* [n_max][n_ff/256] Q8_K blocks */
  uint16_t* sh_y;           /* [n_max][hidden] */
  float* sgate;             /* [n_max], only with shared_gate_w */
} sgr_moe_prefill;
int sgr_moe_layer_prefill(const sgr_moe_prefill* args, void* stream);

/* ---- the fp16 tensor-core family of the prefill path (cuda_ops.hpp:104-152) ----------------
 * The reference dequantises Q4_K to fp16 and calls a library GEMM; here the GEMM is the
 * library's own tcgen05 kernel (kind::f16, fp32 accumulation in tensor memory, TMA operand
 * tiles). Layout contract of all of them: y[t * n_rows + row] = sum_k x[t * k + kk] * w[row * k + kk].
 * Where the reference returns bool, 0 means "ran" and a non-zero code means "not run, take the
 * GEMV path" (SGR_EUNSUPPORTED / SGR_EALIGN for the reference's own refusals). w16, x16 and the
 * scratch must be 16-byte aligned and k a multiple of 64. */
/* tc_handle (cuda_ops.hpp:112): non-null when the tensor-core path can run on this driver. */
void* sgr_tc_handle(void);
/* tc_scratch_elems (cuda_ops.hpp:113). */
size_t sgr_tc_scratch_elems(int max_rows, int max_k);
/* tc_gemm_q4_k_f16 (cuda_ops.hpp:109-111): dequantise w into scratch, then the GEMM. */
int sgr_tc_gemm_q4_k_f16(const void* w, const uint16_t* x, uint16_t* y, uint16_t* scratch, int n_rows,
                         int k, int n_tokens, void* stream);
/* tc_gemm_f16_raw (cuda_ops.hpp:125-126). */
int sgr_tc_gemm_f16_raw(const void* w16, const void* x16, void* y16, int n_rows, int k, int n_tokens,
                        void* stream);
/* tc_gemm_f16_f32out_raw (cuda_ops.hpp:137-139). */
int sgr_tc_gemm_f16_f32out_raw(const void* w16, const void* x16, float* y32, int n_rows, int k,
                               int n_tokens, void* stream);
/* dequant_experts_q4_k_f16 (cuda_ops.hpp:127-131): routed experts into a ring of fp16 slots; slot
 * e % ring, rows_per = 1 << rows_sl2 rows of k halfs from element dst_row0; with tab_b the second
 * half of the rows reads tab_b[e]; experts with no routed rows or a null entry are skipped. */
int sgr_dequant_experts_q4_k_f16(const void* const* tab_a, const void* const* tab_b, const int* off,
                                 void* slots, long long dst_row0, int rows_sl2, int k, int n_experts,
                                 int ring, long long slot_elems, void* stream);
/* The dense dequantisation tc_gemm_q4_k_f16 starts with, on its own: out16[row * k + i]. */
int sgr_dequant_q4_k_f16(const void* w, uint16_t* out16, int n_rows, int k, void* stream);
/* tc_router_f32 (cuda_ops.hpp:143-145): router weights cast to fp16 in scratch, fp32 logits. */
int sgr_tc_router_f32(const float* w_f32, const uint16_t* x, float* y, uint16_t* scratch, int n_rows,
                      int k, int n_tokens, void* stream);

/* Expert parallelism, last step on the home rank (no counterpart in the reference, which is
 * single-GPU): x[i] = f16(f32(x[i]) + sum_p parts[p*part_stride + i]), p ascending. */
int sgr_ep_reduce_add_f16(uint16_t* x_f16, const float* parts, int n_parts, long long part_stride,
                          long long count, void* stream);

/* Expert parallelism over peer memory (NVLink), for buffers every rank has mapped (symmetric
 * memory; no counterpart in the reference). One kernel copies `bytes` from src + p * src_stride
 * into dst[p] for every peer p < world with plain 16-byte stores (dst[p] and flags[p] are this
 * rank's addresses of peer p's buffer and arrival word; src_stride 0 sends the same bytes to
 * everyone), fences at system scope and then sets every flags[p] to *step * mul + add. `scratch`
 * is one zeroed device word per call site. src, dst[p] 16-byte aligned, bytes % 16 == 0. */
int sgr_ep_push(const void* src, long long src_stride, long long bytes, void* const* dst,
                unsigned* const* flags, int world, const unsigned* step, int mul, int add,
                unsigned* scratch, void* stream);
/* sgr_ep_reduce_add_f16 that first waits (bounded) until each of the n_parts words at `flags` is
 * >= *step * mul + add. */
int sgr_ep_reduce_add_f16_wait(uint16_t* x_f16, const float* parts, int n_parts, long long part_stride,
                               long long count, const unsigned* flags, const unsigned* step, int mul,
                               int add, void* stream);
/* How long a kernel that waits for a peer's arrival words (the plan of an owner-side layer with
 * wait_flags, sgr_ep_reduce_add_f16_wait) polls before it gives up: `polls` loads, 64 ns apart, per
 * word (default 1 << 22, several seconds). A kernel whose wait runs out sets the status word to 8 and
 * returns with the context intact - the plan then reads the records of an earlier step, the home
 * reduction leaves x_f16 as it was - so a rank that stopped posting turns into an error code that the
 * host reads with sgr_status, not into a hang. Applies to launches made after the call. */
int sgr_ep_set_wait_limit(int polls);
/* *step += 1 (one thread), in stream order: the end of a step. */
int sgr_ep_step_advance(unsigned* step, void* stream);

/* ---- host side: model container and expert pool (no GPU involved) ---------------------------
 * A GGUF v3 reader over a read-only mapping (include/sager/core/gguf.hpp, src/core/gguf.cpp of the
 * reference: header, typed key/value metadata, tensor directory, data section at the file's
 * alignment) and the builder of the expert pool that the pointer tables point into
 * (Weights::load_expert_pool, src/core/weights.cpp:730-862): expert (layer, e) at
 * (layer * n_expert + e) * sgr_expert_bytes(), its gate, up and down Q4_K matrices back to back,
 * cut from blk.<L>.ffn_{gate,up,down}_exps; a Q6_K down tensor is dequantised and requantised to
 * Q4_K row by row with the reference's quantiser (src/kernels/q4_k.cpp:68-174), byte for byte. */
typedef struct sgr_gguf_tensor_info {
  int type;                 /* ggml type id: 0 F32, 1 F16, 8 Q8_0, 12 Q4_K, 14 Q6_K, 30 BF16 */
  int n_dims;
  long long dims[4];        /* dims[0] is the fastest-varying */
  long long offset;         /* from the start of the data section */
  long long nbytes;         /* 0 for a type whose size the reader does not know */
  long long row_bytes;      /* bytes of one row of dims[0] elements */
  const void* data;         /* inside the mapping: valid until sgr_gguf_close */
} sgr_gguf_tensor_info;
int sgr_gguf_open(const char* path, void** handle);   /* SGR_EARG: not a GGUF file / truncated; SGR_EUNSUPPORTED: not v3 */
void sgr_gguf_close(void* handle);
long long sgr_gguf_count(const void* handle, int what);   /* 0 tensors, 1 key/value pairs, 2 alignment, 3 data offset */
int sgr_gguf_kv_type(const void* handle, const char* key);   /* GGUF value type id, -1 = no such key */
long long sgr_gguf_kv_int(const void* handle, const char* key, long long dflt);
double sgr_gguf_kv_double(const void* handle, const char* key, double dflt);
long long sgr_gguf_kv_str(const void* handle, const char* key, char* buf, long long cap);   /* length, -1 = absent */
long long sgr_gguf_kv_array(const void* handle, const char* key, int* elem_type, const void** data);   /* count, -1 */
int sgr_gguf_tensor(const void* handle, const char* name, sgr_gguf_tensor_info* out);
long long sgr_gguf_tensor_name(const void* handle, long long index, char* buf, long long cap);
/* q4k::quantize_row (src/kernels/q4_k.cpp:68-174) and dequant_row_q6 (src/core/weights.cpp:171-209) on the host */
int sgr_quantize_row_q4_k(const float* x, int n, void* out_blocks);
int sgr_dequant_row_q6_k(const void* src, float* out, int cols);
size_t sgr_expert_bytes(int hidden, int n_ff);
int sgr_expert_pool_fill(const void* handle, void* pool, size_t pool_bytes, int first_block, int n_layer,
                         int n_expert, int hidden, int n_ff, int n_threads);

/* ---- residency: where the experts live on the device, and the tables the kernels read --------
 * HotTier::rebuild (src/core/layer.cpp:21-109), the arena half of ExpertPump
 * (src/core/expert_pump.cpp:130-216) and Session::build_decode_table
 * (src/core/session.cpp:3569-3627) behind one handle. All memory is the caller's: the host pool
 * (expert (l, e) at (l * E + e) * sgr_expert_bytes), a device slab of slab_experts experts, a device
 * arena of arena_slots experts, the device table of 3 * L * E pointers laid out [3][L][E] - the
 * table sgr_moe_layer / sgr_moe_prefill take with tab_stride = L * E. With host_only != 0 the
 * "device" pointers are host memory and no CUDA call is made (the policy can be tested without a GPU).
 * Single producer: one thread drives a handle, as the session thread does in the reference. */
int sgr_residency_create(int n_layers, int n_experts, int hidden, int n_ff, long long slab_experts,
                         int arena_slots, void** out);
void sgr_residency_destroy(void* handle);
int sgr_residency_bind(void* handle, const void* host_pool, void* dev_slab, void* dev_arena, void* dev_table,
                       void* copy_stream, int host_only);
int sgr_residency_set_resident(void* handle, int layer, int expert, int on);
int sgr_residency_rebuild(void* handle, void* stream, int* resident);
/* arena slot (>= 0), -1 = no slot can be had right now: fall back for this expert, -2 = in the slab */
int sgr_residency_submit(void* handle, int layer, int expert, unsigned long long step);
int sgr_residency_wait(void* handle, int slot, void* stream);
int sgr_residency_clear_arena(void* handle);
int sgr_residency_build_decode_table(void* handle, void* stream, int* total_absent);
long long sgr_residency_stat(const void* handle, int what);
int sgr_residency_where(const void* handle, int layer, int expert);
const void* const* sgr_residency_host_table(const void* handle, int which);

/* No counterpart in the reference. sgr_moe_layer_decode for callers that cannot
 * allocate device memory - an engine whose whole VRAM budget was handed out at
 * start-up (KV cache, expert slab) and that treats any later cudaMalloc as a bug,
 * a host binding with no way to own CUDA buffers, code that only ever runs inside a
 * captured region. The scratch is a file-scope device array inside the library,
 * sgr_moe_layer_static_limit() bytes (2 MiB: at hidden 2048, expert FFN 512, 256 experts,
 * top-8 that is up to n_max = 16 token rows; n_max = 8 needs 1.3 MB); `workspace` / `workspace_bytes` of the
 * argument block are ignored, inputs and outputs are still the caller's. A shape
 * whose scratch would not fit returns SGR_ESTATICLIMIT and launches nothing. The first
 * call on each device looks up the array's device address and must be made outside
 * stream capture. Every call on a device uses the same array: calls that overlap on
 * the GPU race. */
size_t sgr_moe_layer_static_limit(void);
int sgr_moe_layer_decode_static(const sgr_moe_layer* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SAGER_B200_H_ */
