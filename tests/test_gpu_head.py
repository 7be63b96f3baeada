"""LM head on Q6_K weights and the two-phase top-k after it (gemv_q6_k_q8, gemv_q6_k_q8_smx,
topk_select_f32_2p of the reference: src/kernels/cuda/q4_k.cu:1564-1658, src/kernels/cuda/mmq.cu:890-986,
src/kernels/cuda/sampling.cu:162-289). The GEMV is held to the oracle's exact-integer restatement and
to the reference's own kernels to fp32 rounding; the selection is index work and must be exact."""
import numpy as np
import pytest
import torch

from oracle import ref_cuda
from oracle.oracle import dequant_q6k, gemv_q6k_q8k, make_q6k, topk_select
from sager_b200 import lib, ops
from tests.util import DEV, GEMV_TOL, make_x16, rel

pytestmark = pytest.mark.gpu


def _q8(x_dev, k):
    xq = torch.zeros(1, k // 256 * 276, dtype=torch.uint8, device=DEV)
    ops.quantize_q8_k(x_dev, xq, k)
    return xq


@pytest.mark.parametrize("rows,k", [(1000, 2048), (37, 512), (151936, 2048), (4096, 4096)])
def test_q6k_head_gemv(oracle, rows, k):
    rng = np.random.default_rng(rows + k)
    w_np = make_q6k(rng, rows, k)
    w = torch.from_numpy(w_np).to(DEV)
    _, x = make_x16(1, k, 3)
    xq = _q8(x, k)
    y = torch.zeros(rows, dtype=torch.float32, device=DEV)
    y2 = torch.zeros(rows, dtype=torch.float32, device=DEV)
    ops.gemv_q6_k_q8(w, xq, y, rows, k)
    ops.gemv_q6_k_q8_smx(w, xq, y2, rows, k)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)                                      # the two entry points agree to the bit
    check = slice(0, rows) if rows <= 4096 else rng.choice(rows, 3000, replace=False)
    want = gemv_q6k_q8k(w_np[check], xq.cpu().numpy()[0], k)
    assert rel(y.cpu().numpy()[check], want) <= GEMV_TOL
    # and the integer dot is the dot of the dequantised weights with the dequantised activations
    if rows <= 1000:
        xb = xq.cpu().numpy()[0].reshape(-1, 276)
        xdq = (xb[:, :4].copy().view(np.float32) * xb[:, 4:260].copy().view(np.int8).astype(np.float32)).reshape(-1)
        full = dequant_q6k(w_np, k).astype(np.float64) @ xdq.astype(np.float64)
        assert rel(want, full) <= 1e-5
    if ref_cuda.available():
        ref = ref_cuda.reference_launchers()
        yr = torch.zeros(rows, dtype=torch.float32, device=DEV)
        ref.gemv_q6_k_q8(w, xq, yr, rows, k)
        torch.cuda.synchronize()
        assert rel(y.cpu().numpy(), yr.cpu().numpy()) <= GEMV_TOL
    assert lib().raw("sgr_status")(0) == 0


def test_q6k_head_gemv_unaligned_base_takes_the_plain_path(oracle):
    rows, k = 600, 2048
    rng = np.random.default_rng(9)
    w_np = make_q6k(rng, rows, k)
    big = torch.zeros(w_np.size + 16, dtype=torch.uint8, device=DEV)
    w = big[2:2 + w_np.size]
    w.copy_(torch.from_numpy(w_np.reshape(-1)))
    _, x = make_x16(1, k, 4)
    xq = _q8(x, k)
    y = torch.zeros(rows, dtype=torch.float32, device=DEV)
    ops.gemv_q6_k_q8(w, xq, y, rows, k)
    torch.cuda.synchronize()
    assert rel(y.cpu().numpy(), gemv_q6k_q8k(w_np, xq.cpu().numpy()[0], k)) <= GEMV_TOL


def _run_topk(o, logits, k):
    n = logits.numel()
    nseg = (n + 2047) // 2048
    seg_v = torch.zeros(nseg * 64, dtype=torch.float32, device=DEV)
    seg_i = torch.zeros(nseg * 64, dtype=torch.int32, device=DEV)
    out_v = torch.zeros(64, dtype=torch.float32, device=DEV)
    out_i = torch.zeros(64, dtype=torch.int32, device=DEV)
    o.topk_select_f32_2p(logits, seg_v, seg_i, nseg * 64, out_v, out_i, n, k)
    torch.cuda.synchronize()
    kk = min(k, 64)
    return out_v.cpu().numpy()[:kk], out_i.cpu().numpy()[:kk]


@pytest.mark.parametrize("n,k", [(151936, 32), (248320, 64), (2048, 8), (5000, 1), (100, 64), (40, 64)])
def test_two_phase_topk_is_exact(n, k):
    rng = np.random.default_rng(n + k)
    x = rng.standard_normal(n).astype(np.float32)
    # ties (also across segment borders), both zeros, values that never qualify
    x[rng.integers(0, n, size=max(4, n // 50))] = np.float32(2.5)
    if n > 4100:
        x[[2047, 2048, 4095, 4096]] = np.float32(7.25)
    x[rng.integers(0, n, size=3)] = np.float32(-0.0)
    x[rng.integers(0, n, size=3)] = np.nan
    x[rng.integers(0, n, size=2)] = -np.inf
    x[rng.integers(0, n, size=2)] = np.float32(-3.4e38)
    logits = torch.from_numpy(x).to(DEV)
    before = logits.clone()
    got_v, got_i = _run_topk(ops, logits, k)
    want_v, want_i = topk_select(x, k)
    assert np.array_equal(got_i, want_i)
    assert np.array_equal(got_v, want_v)
    assert torch.equal(logits.view(torch.int32), before.view(torch.int32))     # the logits are left alone
    if ref_cuda.available():
        ref_v, ref_i = _run_topk(ref_cuda.reference_launchers(), before.clone(), k)
        nv = int((want_i >= 0).sum())              # entries past the last qualifying value are padding
        assert np.array_equal(got_i[:nv], ref_i[:nv]) and np.array_equal(got_v[:nv], ref_v[:nv])


def test_topk_with_fewer_candidates_than_k_and_small_scratch():
    x = np.full(300, -np.inf, dtype=np.float32)
    x[[5, 17, 250]] = [1.0, 3.0, 1.0]
    logits = torch.from_numpy(x).to(DEV)
    v, i = _run_topk(ops, logits, 8)
    assert i.tolist() == [17, 5, 250, -1, -1, -1, -1, -1]
    assert v[:3].tolist() == [3.0, 1.0, 1.0] and np.all(v[3:] == np.float32(-3.4e38))
    # a scratch smaller than ceil(n / 2048) * k is refused before anything is launched
    from sager_b200.capi import SagerError
    big = torch.zeros(10000, dtype=torch.float32, device=DEV)
    sv = torch.zeros(64, dtype=torch.float32, device=DEV)
    si = torch.zeros(64, dtype=torch.int32, device=DEV)
    with pytest.raises(SagerError) as e:
        ops.topk_select_f32_2p(big, sv, si, 64, sv, si, 10000, 32)
    assert e.value.code == 3
