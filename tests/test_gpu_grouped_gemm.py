"""GPU parity of the tcgen05 int8 grouped GEMM (sgr_moe_grouped_gemm_i8) against the
oracle's Q4_K x Q8_K row dot and against the library's own device-plan grouped GEMV,
which implements the reference's batched Q4_K path (q4_k.cu:765-836). Same integers
on every path, so fp16 outputs agree to one fp16 step."""
import numpy as np
import pytest
import torch

from sager_b200 import ops
from tests.util import DEV, dev, f16_close, f16_ulp_diff, make_q4k, make_x16

pytestmark = pytest.mark.gpu


def quantize_dev(x16_dev):
    n, k = x16_dev.shape
    out = torch.zeros(n, k // 256 * 276, dtype=torch.uint8, device=DEV)
    ops.quantize_q8_k(x16_dev, out, n * k)
    return out


def run_case(oracle, n_rows, k, counts, absent=(), seed=0, check_rows=6):
    E = len(counts)
    mats = [make_q4k(n_rows, k, 900 + seed * 50 + e) for e in range(E)]
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    R = int(off[-1])
    x_np, x_dev = make_x16(max(R, 1), k, 33 + seed)
    xq = quantize_dev(x_dev)
    tab = ops.ptr_table([None if e in absent else mats[e][1] for e in range(E)], DEV)
    y = torch.full((max(R, 1), n_rows), 9.0, dtype=torch.float16, device=DEV)
    ops.moe_grouped_gemm_i8(tab, dev(off), xq, y, n_rows, k, E)
    torch.cuda.synchronize()
    y_np = y.cpu().numpy()
    xq_np = xq.cpu().numpy()
    rng = np.random.default_rng(seed)
    for e in range(E):
        lo, hi = off[e], off[e + 1]
        if e in absent:
            assert np.all(y_np[lo:hi] == 0)
            continue
        for r in ([lo, hi - 1] + rng.integers(lo, hi, check_rows).tolist() if hi > lo else []):
            want = oracle.gemv(mats[e][0], xq_np[r], n_rows, k)
            assert f16_close(y_np[r], want), (e, r)
    return mats, off, xq, y


def test_small_shapes(oracle):
    run_case(oracle, 128, 256, [5, 0, 17, 1], seed=1)
    run_case(oracle, 200, 512, [3, 64, 65], seed=2)          # ragged row tile, chunk boundary
    from sager_b200 import lib
    assert lib().raw("sgr_status")(0) == 0


@pytest.mark.parametrize("n_rows,k", [(512, 2048), (2048, 512)])
def test_expert_shapes_match_device_plan_gemv(oracle, n_rows, k):
    counts = [64, 1, 0, 130, 16, 7]
    mats, off, xq, y = run_case(oracle, n_rows, k, counts, absent=(4,), seed=3)
    # the same plan through the dp4a/MMA grouped kernel of the decode path
    E, tok_per = len(counts), 16
    toff = np.concatenate([[0], np.cumsum([(c + tok_per - 1) // tok_per for c in counts])]).astype(np.int32)
    meta = np.int32([off[-1], toff[-1], 0, 0])
    tab = ops.ptr_table([None if e == 4 else mats[e][1] for e in range(E)], DEV)
    y2 = torch.zeros_like(y)
    ops.gemv_grouped_tab_q4_k_q8_f16out_mtok(tab, dev(off), dev(toff), dev(meta), int(toff[-1]), xq, y2,
                                             n_rows, k, E, tok_per)
    torch.cuda.synchronize()
    assert f16_ulp_diff(y.cpu().numpy(), y2.cpu().numpy()) <= 1 or \
        f16_close(y.cpu().numpy(), y2.float().cpu().numpy())


def test_prefill_sized_plan(oracle):
    """2048 token rows, top-8 of 256 experts with uniform logits: 16384 routed rows, about 64
    per expert - the prefill configuration. Spot-checked against the oracle."""
    rng = np.random.default_rng(4)
    picks = np.argsort(rng.random((2048, 256)), axis=1)[:, :8]
    counts = np.bincount(picks.reshape(-1), minlength=256).tolist()
    # one weight matrix shared by all experts keeps the test light; the kernel cannot tell
    n_rows, k = 512, 2048
    w_np, w_dev = make_q4k(n_rows, k, 77)
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    R = int(off[-1])
    x_np, x_dev = make_x16(R, k, 5)
    xq = quantize_dev(x_dev)
    tab = ops.ptr_table([w_dev] * 256, DEV)
    y = torch.zeros(R, n_rows, dtype=torch.float16, device=DEV)
    ops.moe_grouped_gemm_i8(tab, dev(off), xq, y, n_rows, k, 256)
    torch.cuda.synchronize()
    xq_np = xq.cpu().numpy()
    for r in rng.integers(0, R, 12).tolist():
        assert f16_close(y[r].cpu().numpy(), oracle.gemv(w_np, xq_np[r], n_rows, k))


def test_prefill_layer_against_oracle(oracle):
    """The whole prefill call sequence (router, plan, gather, three tensor-core grouped GEMMs,
    SwiGLU, requantisation, scatter, shared expert, combine). The launchers keep the reference's
    fp16 staging (g, u, h, y and the combine slab are fp16: their signatures say so), so the check
    is made twice: against the oracle's restatement of that staged device path (a few fp16 steps)
    and against the fp32 CPU layer. The second gap is not a kernel property: rounding h to fp16
    before it is requantised moves Q8 codes, so the staged path and the fp32 path differ at the
    level of the Q8 grid (measured 3.6e-3 of the largest output here, with weights 2.5x the
    benchmark's scale); it is asserted below 1e-2 and printed. The fused decode layer, which keeps
    fp32 intermediates, meets the 1e-3 bound at 1e-7."""
    from sager_b200 import synth
    from sager_b200.layer import PrefillLayer
    from tests.test_gpu_moe_layer import oracle_layer
    H, F, E, K, n = 512, 256, 16, 4, 300
    w = synth.MoeWeights(H, F, E, DEV, seed=61, std=0.05)
    x16 = synth.normal_fp16((n, H), 62, DEV)
    layer = PrefillLayer(n, H, F, E, K, DEV)
    x = x16.clone()
    layer.run(n, x16, x, w, w.table())
    torch.cuda.synchronize()
    x_np = x16.cpu().numpy()
    got = x.cpu().numpy()
    want = oracle_layer(oracle, w, x_np, x_np.astype(np.float32), K)
    assert np.array_equal(layer.idx.cpu().numpy()[:n, :K], want["idx"][:, :K])
    assert int(layer.meta[0].item()) == n * K
    gap = np.abs(got.astype(np.float32) - want["out"]).max() / np.abs(want["out"]).max()
    print(f"prefill layer (fp16 staging) vs fp32 CPU layer: max relative error {gap:.2e}")
    assert gap < 1e-2
    # the staged device path, restated with the oracle's pieces, for a few rows
    mats = {e: [w.matrix(e, m).cpu().numpy() for m in range(3)] for e in range(E + 1)}
    for r in (0, 17, 299):
        xq = oracle.quantize_q8k_f16(x_np[r][None])[0]
        slab = np.zeros((K + 1, H), dtype=np.float16)
        for kk in range(K + 1):
            e = int(want["idx"][r, kk]) if kk < K else E
            g16 = oracle.gemv(mats[e][0], xq, F, H).astype(np.float16)
            u16 = oracle.gemv(mats[e][1], xq, F, H).astype(np.float16)
            h16 = oracle.silu_mul_f16(g16, u16).view(np.float16)
            hq = oracle.quantize_q8k_f16(h16[None])[0]
            slab[kk] = oracle.gemv(mats[e][2], hq, H, F).astype(np.float16)
        ref = oracle.combine_batched_f16(x_np[r][None], slab[None], want["w"][r][None], K, H, 1)
        # one Q8 code of h may flip where the device's expf differs by an ulp: allow a few fp16 steps
        assert f16_ulp_diff(got[r], ref.view(np.float16).reshape(H)) <= 4
