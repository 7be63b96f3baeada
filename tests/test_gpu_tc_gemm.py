"""The fp16 tensor-core family (dequantise Q4_K, then a real GEMM) against plain
torch fp32 arithmetic on the same fp16 inputs, through the C ABI. The reference
holds this path to cos > 0.99 / relRMSE < 0.10 against its dp4a path
(tests/test_cuda_q4.cu:185-202); here the GEMM itself is held to fp32 accumulation
error and the dequantisation to the bit."""
import ctypes as C

import numpy as np
import pytest
import torch

from sager_b200 import ops
from sager_b200.capi import lib
from tests.util import DEV, make_q4k, make_x16, rel

pytestmark = pytest.mark.gpu


def dequant_numpy(blocks_u8, rows, k):
    """fp16( fma(d*sc, q, -(dmin*m)) ) per weight, ggml Q4_K order (q4_k.hpp:46-52,110-118)."""
    nb = k // 256
    b = blocks_u8.reshape(rows * nb, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)[:, 0]
    sc = b[:, 4:16].astype(np.int32)
    s6 = np.zeros((b.shape[0], 8), np.int32)
    m6 = np.zeros((b.shape[0], 8), np.int32)
    for j in range(8):
        if j < 4:
            s6[:, j] = sc[:, j] & 63
            m6[:, j] = sc[:, j + 4] & 63
        else:
            s6[:, j] = (sc[:, j + 4] & 0xF) | ((sc[:, j - 4] >> 6) << 4)
            m6[:, j] = (sc[:, j + 4] >> 4) | ((sc[:, j] >> 6) << 4)
    sd = (d[:, None] * s6.astype(np.float32)).astype(np.float32)          # one fp32 rounding each
    sm = (dmin[:, None] * m6.astype(np.float32)).astype(np.float32)
    qs = b[:, 16:144].reshape(-1, 4, 32)
    out = np.zeros((b.shape[0], 8, 32), np.float16)
    for sb in range(8):
        nib = (qs[:, sb >> 1, :] >> (4 * (sb & 1))) & 0xF
        v = sd[:, sb, None].astype(np.float64) * nib - sm[:, sb, None].astype(np.float64)   # exact
        out[:, sb, :] = v.astype(np.float32).astype(np.float16)
    return out.reshape(rows, k)


@pytest.fixture(params=[0, 1], ids=["swizzled", "core"])
def layout(request):
    assert lib().raw("sgr_tc_set_operand_layout")(request.param) == 0
    yield request.param
    lib().raw("sgr_tc_set_operand_layout")(0)


def test_handle_and_scratch():
    assert lib().raw("sgr_tc_handle")()
    assert lib().raw("sgr_tc_scratch_elems")(12288, 2048) == 12288 * 2048
    assert lib().raw("sgr_tc_scratch_elems")(0, 0) == 1


@pytest.mark.parametrize("rows,k", [(512, 2048), (2048, 512), (24, 256)])
def test_dense_dequant_is_bit_exact(rows, k, oracle):
    w_np, w_dev = make_q4k(rows, k, 5)
    out = torch.zeros(rows, k, dtype=torch.float16, device=DEV)
    ops.dequant_q4_k_f16(w_dev, out, rows, k)
    want = dequant_numpy(w_np, rows, k)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    # and against the reference's fp32 dequantisation (q4_k.cpp), one fp16 rounding away
    ref32 = oracle.dequant(w_np.reshape(-1), rows * k).reshape(rows, k)
    assert np.abs(out.cpu().numpy().astype(np.float32) - ref32).max() <= np.abs(ref32).max() * 1e-3


def test_expert_dequant_ring_and_skips():
    E, F, H, ring = 6, 64, 512, 4
    ws = [make_q4k(F, H, 10 + e) for e in range(E)]
    us = [make_q4k(F, H, 30 + e) for e in range(E)]
    ds = [make_q4k(H, F * 4, 50 + e) for e in range(E)]          # down: H rows of k = 256
    tab_a = torch.tensor([w[1].data_ptr() for w in ws], dtype=torch.int64, device=DEV)
    tab_b = torch.tensor([u[1].data_ptr() for u in us], dtype=torch.int64, device=DEV)
    tab_a[2] = 0                                                  # absent expert
    off = torch.tensor([0, 3, 3, 5, 9, 9, 12], dtype=torch.int32, device=DEV)   # experts 1 and 4 idle
    rows_sl2 = 7                                                  # 128 rows per slot: 64 gate + 64 up
    slot_elems = 128 * H + 512 * 256
    slots = torch.full((ring, slot_elems), 7.0, dtype=torch.float16, device=DEV)
    # only the last four experts fit the ring (e % 4): run the sub-table [2, 6)
    ops.dequant_experts_q4_k_f16(tab_a[2:], tab_b[2:], off[2:], slots, 0, rows_sl2, H, 4, ring, slot_elems)
    got = slots.cpu().numpy()
    for e_sub, e in enumerate(range(2, 6)):
        region = got[e_sub & 3, :128 * H].reshape(128, H)
        if e in (2, 4):
            if e == 4:
                assert (region == 7.0).all()                      # no routed rows: untouched
            else:
                assert (region[:64] == 7.0).all()                 # null gate entry skipped ...
                assert np.array_equal(region[64:].view(np.uint16),   # ... the up half is written
                                      dequant_numpy(us[e][0], F, H).view(np.uint16))
            continue
        assert np.array_equal(region[:64].view(np.uint16), dequant_numpy(ws[e][0], F, H).view(np.uint16))
        assert np.array_equal(region[64:].view(np.uint16), dequant_numpy(us[e][0], F, H).view(np.uint16))
    # down mode: one table, region after the gate/up rows
    tab_d = torch.tensor([d[1].data_ptr() for d in ds], dtype=torch.int64, device=DEV)
    ops.dequant_experts_q4_k_f16(tab_d[2:], None, off[2:], slots, 128 * H, 9, 256, 4, ring, slot_elems)
    got = slots.cpu().numpy()
    for e_sub, e in enumerate(range(2, 6)):
        region = got[e_sub & 3, 128 * H:].reshape(512, 256)
        if e == 4:
            assert (region == 7.0).all()
        else:
            assert np.array_equal(region.view(np.uint16), dequant_numpy(ds[e][0], H, 256).view(np.uint16))


def gemm_want(w16, x16):
    return x16.float() @ w16.float().t()


@pytest.mark.parametrize("rows,k,tok", [(512, 2048, 64), (2048, 512, 200), (100, 64, 5), (128, 256, 128),
                                        (384, 1024, 129)])
def test_raw_gemm_matches_fp32_matmul(rows, k, tok, layout):
    g = torch.Generator(device=DEV).manual_seed(rows + tok)
    w16 = (torch.randn(rows, k, generator=g, device=DEV) * 0.05).half()
    x16 = torch.randn(tok, k, generator=g, device=DEV).half()
    want = gemm_want(w16, x16)
    y32 = torch.full((tok, rows), float("nan"), dtype=torch.float32, device=DEV)
    assert lib().raw("sgr_tc_gemm_f16_f32out_raw")(w16.data_ptr(), x16.data_ptr(), y32.data_ptr(), rows, k, tok,
                                                   ops.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert lib().raw("sgr_status")(0) == 0
    assert rel(y32.cpu().numpy(), want.cpu().numpy()) < 1e-5           # fp32 accumulation, another order
    y16 = torch.full((tok, rows), float("nan"), dtype=torch.float16, device=DEV)
    ops.tc_gemm_f16_raw(w16, x16, y16, rows, k, tok)
    # the same fp32 sums rounded once to fp16
    assert np.array_equal(y16.cpu().numpy().view(np.uint16), y32.half().cpu().numpy().view(np.uint16))


def test_q4k_gemm_and_router(layout):
    rows, k, tok = 512, 2048, 96
    w_np, w_dev = make_q4k(rows, k, 3)
    x_np, x_dev = make_x16(tok, k, 4)
    scratch = torch.empty(lib().raw("sgr_tc_scratch_elems")(rows, k), dtype=torch.float16, device=DEV)
    y = torch.zeros(tok, rows, dtype=torch.float16, device=DEV)
    ops.tc_gemm_q4_k_f16(w_dev, x_dev, y, scratch, rows, k, tok)
    w16 = torch.from_numpy(dequant_numpy(w_np, rows, k)).to(DEV)
    want = gemm_want(w16, x_dev)
    assert np.array_equal(scratch.cpu().numpy().view(np.uint16).reshape(rows, k), w16.cpu().numpy().view(np.uint16))
    assert rel(y.float().cpu().numpy(), want.cpu().numpy()) < 1e-3      # fp16 storage
    # router: fp32 weights cast to fp16 once, fp32 logits
    E = 256
    g = torch.Generator(device=DEV).manual_seed(9)
    wr = torch.randn(E, k, generator=g, device=DEV) * 0.02
    logits = torch.zeros(tok, E, dtype=torch.float32, device=DEV)
    rs = torch.empty(E * k, dtype=torch.float16, device=DEV)
    ops.tc_router_f32(wr, x_dev, logits, rs, E, k, tok)
    want_l = gemm_want(wr.half(), x_dev)
    assert rel(logits.cpu().numpy(), want_l.cpu().numpy()) < 1e-5
    # against the exact fp32 router the difference is the fp16 rounding of the weights
    assert rel(logits.cpu().numpy(), (x_dev.float() @ wr.t()).cpu().numpy()) < 2e-3


def test_refusals_launch_nothing():
    t = torch.zeros(4096, dtype=torch.float16, device=DEV)
    p = t.data_ptr()
    raw = lib().raw
    assert raw("sgr_tc_gemm_f16_raw")(p, p, p, 8, 100, 4, None) == 3            # k % 64
    assert raw("sgr_tc_gemm_f16_raw")(p + 2, p, p, 8, 64, 4, None) == 2         # operand alignment
    assert raw("sgr_tc_gemm_q4_k_f16")(p, p, p, p, 8, 768, 4, None) == 3        # k not a power of two
    assert raw("sgr_tc_gemm_q4_k_f16")(p + 4, p, p, p, 8, 512, 4, None) == 2    # weights not 16-byte aligned
    assert raw("sgr_tc_gemm_f16_raw")(p, p, p, 0, 64, 4, None) == 0             # empty
