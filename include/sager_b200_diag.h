/*
 * sager_b200_diag.h - entry points of libsager_b200.so that serve tests and
 * measurements only. None of them replaces a launcher of the reference
 * (include/sager/kernels/cuda_ops.hpp) and a caller of the library never needs them.
 */
#ifndef SAGER_B200_DIAG_H_
#define SAGER_B200_DIAG_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Operand tile layout of the fp16 tensor-core GEMM kernel behind the sgr_tc_* entries: 0 = 128-byte
 * swizzled tiles (default), 1 = unswizzled core matrices. Same results either way; process-global. */
int sgr_tc_set_operand_layout(int layout);

/* Byte offset of a region inside the workspace of sgr_moe_layer_decode (same geometry arguments as
 * sgr_moe_layer_workspace_bytes), so that a test can read the intermediate rows a finished call
 * left there. which: 0 = fp32 h rows [n_max*K + n_max][n_ff] (routed rows in grouped order, then
 * the shared expert's), 1 = fp32 y rows [..][hidden], 2 = gslot [n_max*K] (route -> grouped row,
 * -1 = not computed), 3 = grows, 4 = plan records, 5 = meta. -1 for a refused geometry. */
long long sgr_moe_layer_workspace_offset(int n_max, int hidden, int n_ff, int n_expert, int n_used,
                                         int which);

/* Residency handle in host-only mode: mark an arena slot as "its copy is still in flight" (what an
 * unfinished event says on the device), so that the rule "an in-flight slot is never evicted" can be
 * exercised without a GPU. */
int sgr_residency_test_set_inflight(void* handle, int slot, int on);

#ifdef __cplusplus
}
#endif
#endif /* SAGER_B200_DIAG_H_ */
