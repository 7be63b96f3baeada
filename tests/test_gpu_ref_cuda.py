"""This library's launchers against the reference's own CUDA launchers compiled for
sm_100a (oracle/_ref/libsager_ref_cuda.so; skipped when it was not built), on the same
device buffers: piece by piece, then the whole device MoE path in the reference's
launch sequence, then the fused layer."""
import numpy as np
import pytest
import torch

from oracle import ref_cuda
from sager_b200 import synth
from sager_b200.layer import MoeLayerRunner
from tests.test_gpu_moe_layer import oracle_layer
from tests.util import DEV, f16_ulp_diff, make_q4k, make_x16, rel

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libsager_ref_cuda.so not built")]


@pytest.fixture(scope="module")
def both():
    return ref_cuda.reference_launchers(), ref_cuda.library_launchers()


def test_quantiser_router_and_topk_match_the_reference_kernels(both):
    ref, mine = both
    n, H, E, K = 37, 2048, 256, 8
    _, x = make_x16(n, H, 21)
    g = torch.Generator(device=DEV).manual_seed(3)
    router = torch.randn(E, H, generator=g, device=DEV) * 0.02
    out = {}
    for name, o in (("ref", ref), ("mine", mine)):
        xq = torch.zeros(n, H // 256 * 276, dtype=torch.uint8, device=DEV)
        logits = torch.zeros(n, E, dtype=torch.float32, device=DEV)
        idx = torch.zeros(n, K + 1, dtype=torch.int32, device=DEV)
        w = torch.zeros(n, K + 1, dtype=torch.float32, device=DEV)
        o.quantize_q8_k(x, xq, n * H)
        o.gemv_f32_out_f16x_mtok(router, x, logits, E, H, n)
        o.router_topk_batched(logits, idx, w, E, K, K + 1, n, 1.0)
        torch.cuda.synchronize()
        out[name] = [t.cpu().numpy() for t in (xq, logits, idx, w)]
    assert np.array_equal(out["ref"][0], out["mine"][0])                       # Q8_K blocks: bit-exact
    assert np.array_equal(out["ref"][1].view(np.uint32), out["mine"][1].view(np.uint32))   # logits: bit-exact
    assert np.array_equal(out["ref"][2][:, :K], out["mine"][2][:, :K])         # experts and their order
    assert np.abs(out["ref"][3] - out["mine"][3]).max() <= 1e-6


def test_dense_gemv_family_matches_the_reference_kernels(both):
    ref, mine = both
    rows, k, tok = 512, 2048, 4
    _, w = make_q4k(rows, k, 8)
    _, x = make_x16(tok, k, 9)
    xq = torch.zeros(tok, k // 256 * 276, dtype=torch.uint8, device=DEV)
    mine.quantize_q8_k(x, xq, tok * k)
    res = {}
    for name, o in (("ref", ref), ("mine", mine)):
        y1 = torch.zeros(rows, dtype=torch.float32, device=DEV)
        o.gemv_q4_k_q8(w, xq, y1, rows, k)
        yb = torch.zeros(tok, rows, dtype=torch.float32, device=DEV)
        o.gemv_q4_k_q8_batched(w, xq, yb, rows, k, tok)
        ym = torch.zeros(tok, rows, dtype=torch.float16, device=DEV)
        o.gemv_q4_k_q8_f16out_mtok(w, xq, ym, rows, k, tok)
        torch.cuda.synchronize()
        res[name] = (y1.cpu().numpy(), yb.cpu().numpy(), ym.cpu().numpy())
    assert rel(res["mine"][0], res["ref"][0]) < 2e-6          # same exact integer dots, another fp32 order
    assert rel(res["mine"][1], res["ref"][1]) < 2e-6
    assert f16_ulp_diff(res["mine"][2], res["ref"][2]) <= 1


@pytest.mark.parametrize("n,hidden,n_ff,E,K", [(64, 2048, 512, 256, 8), (9, 512, 256, 16, 4)])
def test_device_moe_path_and_fused_layer_against_the_reference_sequence(both, oracle, n, hidden, n_ff, E, K):
    """The reference's device MoE sequence on its own kernels against (a) the same sequence on this
    library's launchers and (b) the fused layer. Measured on the MoE half's own output (zero
    residual), where nothing masks a difference, and on top of a residual stream, the layer output
    as the session sees it. Both are held to the stated 1e-3 of the largest output."""
    ref, mine = both
    w = synth.MoeWeights(hidden, n_ff, E, DEV, seed=5, std=0.02 if hidden == 2048 else 0.05)
    xn = synth.normal_fp16((n, hidden), 6, DEV)
    table, shared = w.table(), w.shared_ptrs()
    zero = torch.zeros(n, hidden, dtype=torch.float16, device=DEV)
    resid = synth.normal_fp16((n, hidden), 7, DEV)
    res = {}
    for name, o in (("ref", ref), ("mine", mine)):
        path = ref_cuda.DeviceMoePath(o, n, hidden, n_ff, E, K, DEV)
        y, x = zero.clone(), resid.clone()
        path.run(n, xn, y, w.router, table, shared)
        path.run(n, xn, x, w.router, table, shared)
        torch.cuda.synchronize()
        res[name] = (y.cpu().numpy(), path.idx.cpu().numpy(), path.off.cpu().numpy(), path.meta.cpu().numpy(),
                     x.cpu().numpy())
    assert np.array_equal(res["ref"][1][:, :K], res["mine"][1][:, :K])
    assert np.array_equal(res["ref"][2], res["mine"][2])                       # expert-major plan
    assert np.array_equal(res["ref"][3][:2], res["mine"][3][:2])
    # (a) launch for launch the same arithmetic up to the fp32 summation order inside a GEMV;
    # g, u, y pass through fp16 and h through Q8, so single elements may move by an fp16 step
    want = res["ref"][0].astype(np.float32)
    err_seq = rel(res["mine"][0].astype(np.float32), want)
    err_seq_x = rel(res["mine"][4].astype(np.float32), res["ref"][4].astype(np.float32))
    print(f"n={n} H={hidden}: the reference's device sequence on this library's launchers vs on the reference's own "
          f"kernels: MoE output {err_seq:.2e}, with a residual stream {err_seq_x:.2e}")
    assert max(err_seq, err_seq_x) <= 1e-3, (err_seq, err_seq_x)
    # (b) The fused layer keeps g, u, h, y in fp32, as the reference's CPU path does
    # (src/kernels/cpu/q4_avx2.cpp:175-196), where the reference's device sequence rounds each of
    # them to fp16. The reference's two implementations are themselves a few 1e-3 apart for that
    # reason (h is requantised to Q8_K from differently rounded values), so no single result can be
    # within 1e-3 of both. The fused layer is held to the CPU path (the stated 1e-3; 1e-7 typical), and
    # must be no further from the reference's CUDA path than the reference's own CPU path is.
    runner = MoeLayerRunner(n, hidden, n_ff, E, K, DEV)
    y = zero.clone()
    out32 = torch.zeros(n, hidden, dtype=torch.float32, device=DEV)
    runner.run(runner.args(n, xn, w.router, table, shared, x_f16=y, out_f32=out32))
    torch.cuda.synchronize()
    assert np.array_equal(runner.route_idx.cpu().numpy()[:n, :K], res["ref"][1][:, :K])
    x_np = xn.cpu().numpy()
    cpu = oracle_layer(oracle, w, x_np, np.zeros((n, hidden), dtype=np.float32), K, n_threads=16)["out"]
    d_fused_cpu = rel(out32.cpu().numpy(), cpu)
    d_fused_cuda = rel(y.cpu().numpy().astype(np.float32), want)
    d_cpu_cuda = rel(cpu, want)
    print(f"  fused layer vs the reference's CPU path {d_fused_cpu:.2e}; vs its CUDA sequence {d_fused_cuda:.2e}; "
          f"the reference's CPU path vs its own CUDA sequence {d_cpu_cuda:.2e}")
    assert d_fused_cpu <= 1e-3, d_fused_cpu
    assert d_fused_cuda <= d_cpu_cuda * 1.05 + 5e-4, (d_fused_cuda, d_cpu_cuda)
