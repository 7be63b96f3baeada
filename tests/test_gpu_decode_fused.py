"""The decode-fusion neighbours of the MoE half (include/sager/kernels/cuda_ops.hpp:147-171 of the
reference, "all bit-identical to what they replace"): rmsnorm_quant_f16, which produces the MoE
input rows; gemv_q4_k_q8_f16out_resadd; gemv2m / gemv3m. Each is held (a) to that contract inside
this library - bit-identical to the unfused launchers it stands for - and (b) to the reference's own
CUDA kernels compiled for sm_100a, where those are built."""
import numpy as np
import pytest
import torch

from oracle import ref_cuda
from oracle.oracle import rmsnorm_quant_f16 as rmsnorm_quant_cpu
from sager_b200 import lib, ops
from tests.util import DEV, f16_ulp_diff, make_q4k, make_x16

pytestmark = pytest.mark.gpu

needs_ref = pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libsager_ref_cuda.so not built")


def _norm_inputs(rows, n, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, n, generator=g) * 1.7).half()
    w = (1.0 + 0.1 * torch.randn(n, generator=g)).half()
    return x, w


@pytest.mark.parametrize("rows,n", [(1, 2048), (4, 2048), (64, 2048), (3, 512), (2, 4096), (5, 256)])
def test_rmsnorm_quant_blocks_are_those_of_its_own_output(oracle, rows, n):
    x, w = _norm_inputs(rows, n, 10 + rows)
    xd, wd = x.to(DEV), w.to(DEV)
    out = torch.zeros(rows, n, dtype=torch.float16, device=DEV)
    xq = torch.zeros(rows, n // 256 * 276, dtype=torch.uint8, device=DEV)
    ops.rmsnorm_quant_f16(out, xd, wd, xq, n, 1e-6, rows)
    torch.cuda.synchronize()
    out_np = out.cpu().numpy()
    # the quantised rows are exactly the Q8_K blocks of the fp16 rows written beside them
    assert np.array_equal(xq.cpu().numpy(), oracle.quantize_q8k_f16(out_np))
    xq2 = torch.zeros_like(xq)
    ops.quantize_q8_k(out, xq2, rows * n)
    torch.cuda.synchronize()
    assert torch.equal(xq, xq2)
    # and the rows are the RMS norm: against the CPU restatement of the kernel's own order
    want, _ = rmsnorm_quant_cpu(oracle, x.numpy(), w.numpy(), 1e-6)
    assert f16_ulp_diff(out_np, want) <= 1
    assert (out_np.view(np.uint16) != want.view(np.uint16)).mean() < 0.01
    ref64 = (x.double() * torch.rsqrt((x.double() ** 2).mean(dim=1, keepdim=True) + 1e-6) * w.double()).numpy()
    assert np.abs(out_np.astype(np.float64) - ref64).max() <= 2e-3 * np.abs(ref64).max()


@needs_ref
@pytest.mark.parametrize("rows,n", [(1, 2048), (4, 2048), (64, 2048), (3, 512), (2, 4096)])
def test_rmsnorm_quant_is_bit_identical_to_the_reference_kernels(rows, n):
    ref = ref_cuda.reference_launchers()
    x, w = _norm_inputs(rows, n, 40 + rows)
    xd, wd = x.to(DEV), w.to(DEV)
    res = []
    for o in (ops, ref):
        out = torch.zeros(rows, n, dtype=torch.float16, device=DEV)
        xq = torch.zeros(rows, n // 256 * 276, dtype=torch.uint8, device=DEV)
        o.rmsnorm_quant_f16(out, xd, wd, xq, n, 1e-6, rows)
        torch.cuda.synchronize()
        res.append((out, xq))
    assert torch.equal(res[0][0], res[1][0])                 # fp16 rows: bit-identical
    assert torch.equal(res[0][1], res[1][1])                 # Q8_K blocks: bit-identical
    # and to the two-kernel sequence it replaces in the reference
    import ctypes as C
    out2 = torch.zeros(rows, n, dtype=torch.float16, device=DEV)
    xq2 = torch.zeros_like(res[0][1])
    sp = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ref.cdll.sgr_ref_rmsnorm_batched_f16.argtypes = [C.c_void_p] * 3 + [C.c_int, C.c_float, C.c_int, C.c_void_p]
    ref.cdll.sgr_ref_rmsnorm_batched_f16(out2.data_ptr(), xd.data_ptr(), wd.data_ptr(), n, 1e-6, rows, sp)
    ref.quantize_q8_k(out2, xq2, rows * n)
    torch.cuda.synchronize()
    assert torch.equal(res[0][0], out2) and torch.equal(res[0][1], xq2)


@pytest.mark.parametrize("rows,k", [(2048, 4096), (2048, 512), (512, 2048), (4096, 2048)])
def test_resadd_equals_the_gemv_followed_by_the_add(rows, k):
    _, w = make_q4k(rows, k, 3)
    _, x = make_x16(1, k, 4)
    xq = torch.zeros(1, k // 256 * 276, dtype=torch.uint8, device=DEV)
    ops.quantize_q8_k(x, xq, k)
    _, res0 = make_x16(1, rows, 5)
    y1 = torch.zeros(rows, dtype=torch.float16, device=DEV)
    ops.gemv_q4_k_q8_f16out(w, xq, y1, rows, k)
    want_res = (res0.reshape(-1).float() + y1.float()).half()
    y2 = torch.zeros(rows, dtype=torch.float16, device=DEV)
    res = res0.reshape(-1).clone()
    ops.gemv_q4_k_q8_f16out_resadd(w, xq, y2, res, rows, k)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and torch.equal(res, want_res)
    if ref_cuda.available():
        ref = ref_cuda.reference_launchers()
        y3 = torch.zeros(rows, dtype=torch.float16, device=DEV)
        res3 = res0.reshape(-1).clone()
        ref.gemv_q4_k_q8_f16out_resadd(w, xq, y3, res3, rows, k)
        torch.cuda.synchronize()
        # the same exact integer dots summed in another fp32 order: at most one fp16 step apart
        assert f16_ulp_diff(y2.cpu().numpy(), y3.cpu().numpy()) <= 1
        assert np.abs(res.float().cpu().numpy() - res3.float().cpu().numpy()).max() <= 2.0 ** -8 * 4


@pytest.mark.parametrize("nm,rows,k", [(3, (4096, 512, 512), 2048), (2, (8192, 64), 2048), (3, (40, 8, 24), 512),
                                      (2, (2048, 2048), 4096)])
def test_multi_matrix_gemv_equals_the_separate_gemvs(nm, rows, k):
    ws = [make_q4k(r, k, 20 + i)[1] for i, r in enumerate(rows)]
    _, x = make_x16(1, k, 9)
    xq = torch.zeros(1, k // 256 * 276, dtype=torch.uint8, device=DEV)
    ops.quantize_q8_k(x, xq, k)
    sep = []
    for w, r in zip(ws, rows):
        y = torch.zeros(r, dtype=torch.float16, device=DEV)
        ops.gemv_q4_k_q8_f16out(w, xq, y, r, k)
        sep.append(y)
    ys = [torch.full((r,), 7.0, dtype=torch.float16, device=DEV) for r in rows]
    if nm == 2:
        ops.gemv2m_q4_k_q8_f16out(ws[0], ws[1], xq, ys[0], ys[1], rows[0], rows[1], k, 0)
    else:
        ops.gemv3m_q4_k_q8_f16out(ws[0], ws[1], ws[2], xq, ys[0], ys[1], ys[2], rows[0], rows[1], rows[2], k, 0)
    torch.cuda.synchronize()
    for a, b in zip(sep, ys):
        assert torch.equal(a, b)
    if ref_cuda.available():
        ref = ref_cuda.reference_launchers()
        yr = [torch.zeros(r, dtype=torch.float16, device=DEV) for r in rows]
        if nm == 2:
            ref.gemv2m_q4_k_q8_f16out(ws[0], ws[1], xq, yr[0], yr[1], rows[0], rows[1], k, 0)
        else:
            ref.gemv3m_q4_k_q8_f16out(ws[0], ws[1], ws[2], xq, yr[0], yr[1], yr[2], rows[0], rows[1], rows[2], k, 0)
        torch.cuda.synchronize()
        for a, b in zip(ys, yr):
            assert f16_ulp_diff(a.cpu().numpy(), b.cpu().numpy()) <= 1
    assert lib().raw("sgr_status")(0) == 0
