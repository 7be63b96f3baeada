"""GPU parity: router logits and softmax/top-k selection through the C ABI. The
reference has no test for these kernels; the oracle restates them
(src/kernels/cuda/q4_k.cu:133-149, moe.cu:25-85, mmq.cu:420-510) and the bars
are: logits bit-exact (same FMA order), indices exact in value and order,
weights within 1e-6."""
import numpy as np
import pytest
import torch

from sager_b200 import ops
from tests.util import DEV, dev, make_x16

pytestmark = pytest.mark.gpu

E, K, H = 256, 8, 2048


def router_w(seed, e=E, h=H):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(e, h, generator=g) * 0.02).float()
    return w.numpy(), w.to(DEV)


@pytest.mark.parametrize("n_tok", [1, 4, 11, 64])
def test_logits_bit_exact(oracle, n_tok):
    w_np, w_dev = router_w(1)
    x_np, x_dev = make_x16(n_tok, H, 2)
    want = np.stack([oracle.router_logits(w_np, x_np[t]) for t in range(n_tok)])
    for name in ("gemv_f32_out_f16x_batched", "gemv_f32_out_f16x_mtok"):
        y = torch.zeros(n_tok, E, dtype=torch.float32, device=DEV)
        getattr(ops, name)(w_dev, x_dev, y, E, H, n_tok)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32)), name
    if n_tok == 1:
        y = torch.zeros(E, dtype=torch.float32, device=DEV)
        ops.gemv_f32_out_f16x(w_dev, x_dev, y, E, H)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want[0].view(np.uint32))


def test_logits_odd_shapes(oracle):
    w_np, w_dev = router_w(3, e=13, h=736)       # rows not a multiple of the CTA, k % 256 != 0
    x_np, x_dev = make_x16(3, 736, 4)
    y = torch.zeros(3, 13, dtype=torch.float32, device=DEV)
    ops.gemv_f32_out_f16x_batched(w_dev, x_dev, y, 13, 736, 3)
    want = np.stack([oracle.router_logits(w_np, x_np[t]) for t in range(3)])
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("seed", range(8))
def test_topk_selection_exact(oracle, seed):
    rng = np.random.default_rng(seed)
    n = 33
    logits = (rng.standard_normal((n, E)) * 0.9).astype(np.float32)
    idx = torch.full((n, K + 1), -5, dtype=torch.int32, device=DEV)
    w = torch.full((n, K + 1), -5.0, dtype=torch.float32, device=DEV)
    ops.router_topk_batched(dev(logits), idx, w, E, K, K + 1, n, 1.0)
    idx_np, w_np = idx.cpu().numpy(), w.cpu().numpy()
    for r in range(n):
        oi, ow = oracle.router_topk(logits[r], K, shared_w=1.0)
        assert np.array_equal(idx_np[r, :K], oi[:K])          # same experts, same order
        assert np.abs(w_np[r, :K] - ow[:K]).max() <= 1e-6
        assert w_np[r, K] == 1.0 and idx_np[r, K] == -5        # slot K: weight only
    # single-row launcher, shared_w = 0
    i1 = torch.zeros(K + 1, dtype=torch.int32, device=DEV)
    w1 = torch.full((K + 1,), 3.0, dtype=torch.float32, device=DEV)
    ops.router_topk(dev(logits[0]), i1, w1, E, K, 0.0)
    assert np.array_equal(i1.cpu().numpy()[:K], idx_np[0, :K]) and w1[K].item() == 0.0


def test_topk_ties_nan_and_degenerate_rows(oracle):
    rows = np.zeros((5, 16), dtype=np.float32)
    rows[1, [3, 9, 12]] = 2.0                       # three-way tie -> ascending index
    rows[2, :] = np.nan                             # nothing valid -> kk % E, weight -1
    rows[3, 5] = np.inf                             # inf - inf = nan inside the softmax
    rows[4] = np.linspace(-3, 3, 16)
    rows[4, 7] = np.nan                             # one NaN is simply never picked
    k = 4
    idx = torch.zeros(5, k + 1, dtype=torch.int32, device=DEV)
    w = torch.zeros(5, k + 1, dtype=torch.float32, device=DEV)
    ops.router_topk_batched(dev(rows), idx, w, 16, k, k + 1, 5, 0.5)
    for r in range(5):
        oi, ow = oracle.router_topk(rows[r], k, shared_w=0.5)
        assert np.array_equal(idx.cpu().numpy()[r, :k], oi[:k]), r
        got = w.cpu().numpy()[r]
        assert np.allclose(got[:k], ow[:k], atol=1e-6, equal_nan=True), r
        assert got[k] == 0.5
    assert idx.cpu().numpy()[0, :k].tolist() == [0, 1, 2, 3]
    assert idx.cpu().numpy()[1, :3].tolist() == [3, 9, 12]


@pytest.mark.parametrize("seed", range(4))
def test_fused_router_matches_two_step_path(oracle, seed):
    w_np, w_dev = router_w(10 + seed)
    x_np, x_dev = make_x16(1, H, 20 + seed)
    idx = torch.full((K + 1,), -5, dtype=torch.int32, device=DEV)
    wt = torch.full((K + 1,), -5.0, dtype=torch.float32, device=DEV)
    ops.router_topk_fused(w_dev, x_dev, idx, wt, E, K, H)
    logits = oracle.router_logits(w_np, x_np[0])
    oi, ow = oracle.router_topk(logits, K, write_shared=False)
    assert np.array_equal(idx.cpu().numpy()[:K], oi[:K])
    assert np.abs(wt.cpu().numpy()[:K] - ow[:K]).max() <= 1e-6
    assert wt[K].item() == -5.0                     # the fused kernel leaves slot K alone
    # and bit-identical to the library's own two-launch path
    lg = torch.zeros(E, dtype=torch.float32, device=DEV)
    ops.gemv_f32_out_f16x(w_dev, x_dev, lg, E, H)
    i2 = torch.zeros(K + 1, dtype=torch.int32, device=DEV)
    w2 = torch.zeros(K + 1, dtype=torch.float32, device=DEV)
    ops.router_topk(lg, i2, w2, E, K, 1.0)
    assert torch.equal(i2[:K], idx[:K]) and torch.equal(w2[:K], wt[:K])
