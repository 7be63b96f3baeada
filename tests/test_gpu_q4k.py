"""GPU parity: Q8_K quantiser and the Q4_K x Q8_K GEMV family, through the C ABI,
against the CPU oracle and the reference-written golden vectors. Modelled on the
reference's tests/test_cuda_q4.cu (K=2048, ROWS=512, TOK=5) with its bars
tightened: Q8 blocks and integer dots bit-exact, fp32 within GEMV_TOL."""
import numpy as np
import pytest
import torch

from sager_b200 import ops
from tests.util import DEV, GEMV_TOL, dev, f16_close, make_q4k, make_x16, rel

pytestmark = pytest.mark.gpu


def quantize_dev(x16_dev):
    n, k = x16_dev.shape
    out = torch.zeros(n, k // 256 * 276, dtype=torch.uint8, device=DEV)
    ops.quantize_q8_k(x16_dev, out, n * k)
    return out


def test_quantize_q8_k_bit_exact(oracle, golden):
    x_np, x_dev = make_x16(5, 2048, 1234, std=0.6)
    got = quantize_dev(x_dev).cpu().numpy()
    assert np.array_equal(got, oracle.quantize_q8k_f16(x_np))
    # reference-written vectors, including all-zero, spike, +-amax tie and tiny rows
    gx = golden["gemv_x"].astype(np.float16)
    assert np.array_equal(quantize_dev(dev(gx)).cpu().numpy(), golden["gemv_xq"])
    ex = golden["q8_edge_x"].astype(np.float16)
    assert np.array_equal(quantize_dev(dev(ex)).cpu().numpy(), golden["q8_edge_q"])


def test_quantize_q8_k_unaligned_input(oracle):
    x_np, x_dev = make_x16(1, 1024 + 8, 7)
    view = x_dev.reshape(-1)[3:3 + 1024]                 # 6-byte offset: scalar load path
    out = torch.zeros(4 * 276, dtype=torch.uint8, device=DEV)
    ops.quantize_q8_k(view, out, 1024)
    want = oracle.quantize_q8k_f16(x_np.reshape(-1)[3:3 + 1024].reshape(1, 1024))
    assert np.array_equal(out.cpu().numpy(), want.reshape(-1))


def test_quantize_q8_k_n_reads_row_count_on_device(oracle):
    x_np, x_dev = make_x16(16, 512, 11)
    out = torch.full((16, 2 * 276), 0xAB, dtype=torch.uint8, device=DEV)
    rows = torch.tensor([5], dtype=torch.int32, device=DEV)
    ops.quantize_q8_k_n(x_dev, out, rows, 512, 16 * 2)
    got = out.cpu().numpy()
    assert np.array_equal(got[:5], oracle.quantize_q8k_f16(x_np[:5]))
    assert np.all(got[5:] == 0xAB)                        # rows past the device count untouched


@pytest.mark.parametrize("rows,k", [(512, 2048), (2048, 512), (24, 256), (40, 768), (8, 4096)])
def test_subblock_int_dots_bit_exact(oracle, rows, k):
    w_np, w_dev = make_q4k(rows, k, 3)
    x_np, x_dev = make_x16(1, k, 4)
    xq = quantize_dev(x_dev)
    out = torch.zeros(rows, k // 256, 8, dtype=torch.int32, device=DEV)
    ops.q4k_subblock_dots(w_dev, xq, out, rows, k)
    assert np.array_equal(out.cpu().numpy(), oracle.subblock_dots(w_np, xq.cpu().numpy(), rows, k))


def test_gemv_golden_vectors(golden):
    wq, xq = golden["gemv_wq"], golden["gemv_xq"]
    rows = wq.shape[0]
    for t in range(2):
        y = torch.zeros(rows, dtype=torch.float32, device=DEV)
        ops.gemv_q4_k_q8(dev(wq), dev(xq[t]), y, rows, 2048)
        assert rel(y.cpu().numpy(), golden["gemv_y_avx2"][t]) < GEMV_TOL


# the five shapes of the dense GEMV sweep: q/o projections, expert gate-up/down, LM head
SWEEP = [(4096, 2048), (2048, 4096), (512, 2048), (2048, 512), (151936, 2048)]


@pytest.mark.parametrize("rows,k", SWEEP)
@pytest.mark.parametrize("batch", [1, 4])
def test_gemv_sweep_vs_oracle(oracle, rows, k, batch):
    w_np, w_dev = make_q4k(rows, k, 100 + rows % 97)
    x_np, x_dev = make_x16(batch, k, 200 + k)
    xq = quantize_dev(x_dev)
    xq_np = xq.cpu().numpy()
    assert np.array_equal(xq_np, oracle.quantize_q8k_f16(x_np))
    want = np.stack([oracle.gemv(w_np, xq_np[t], rows, k) for t in range(batch)])
    y = torch.zeros(batch, rows, dtype=torch.float32, device=DEV)
    if batch == 1:
        ops.gemv_q4_k_q8(w_dev, xq, y, rows, k)
    else:
        ops.gemv_q4_k_q8_batched(w_dev, xq, y, rows, k, batch)
    assert rel(y.cpu().numpy(), want) < GEMV_TOL
    y16 = torch.zeros(batch, rows, dtype=torch.float16, device=DEV)
    if batch == 1:
        ops.gemv_q4_k_q8_f16out(w_dev, xq, y16, rows, k)
    else:
        ops.gemv_q4_k_q8_f16out_batched(w_dev, xq, y16, rows, k, batch)
    # the fp16 store rounds the same fp32 value: at most one fp16 step from the oracle's
    assert f16_close(y16.cpu().numpy(), want)


@pytest.mark.parametrize("rows,k,batch", [(40005, 2048, 3), (160001, 512, 2), (20003, 4096, 1)])
def test_large_dense_gemv_persistent_kernel(oracle, rows, k, batch):
    """Matrices of several stages per SM take the persistent streaming kernel; ragged last
    stage, every supported row length (2, 8, 16 super-blocks) and token count."""
    w_np, w_dev = make_q4k(rows, k, 41)
    x_np, x_dev = make_x16(batch, k, 42)
    xq = quantize_dev(x_dev)
    xq_np = xq.cpu().numpy()
    want = np.stack([oracle.gemv(w_np, xq_np[t], rows, k) for t in range(batch)])
    y = torch.full((batch, rows), float("nan"), dtype=torch.float32, device=DEV)
    if batch == 1:
        ops.gemv_q4_k_q8(w_dev, xq, y, rows, k)
    else:
        ops.gemv_q4_k_q8_batched(w_dev, xq, y, rows, k, batch)
    assert rel(y.cpu().numpy(), want) < GEMV_TOL
    y16 = torch.full((batch, rows), float("nan"), dtype=torch.float16, device=DEV)
    ops.gemv_q4_k_q8_f16out_mtok(w_dev, xq, y16, rows, k, batch)
    assert f16_close(y16.cpu().numpy(), want)


@pytest.mark.parametrize("tok", [2, 4, 5, 19])
def test_multi_token_variants_agree(oracle, tok):
    rows, k = 512, 2048
    w_np, w_dev = make_q4k(rows, k, 1)
    w2_np, w2_dev = make_q4k(rows, k, 2)
    x_np, x_dev = make_x16(tok, k, 1234, std=0.6)
    xq = quantize_dev(x_dev)
    xq_np = xq.cpu().numpy()
    want = np.stack([oracle.gemv(w_np, xq_np[t], rows, k) for t in range(tok)])
    want2 = np.stack([oracle.gemv(w2_np, xq_np[t], rows, k) for t in range(tok)])
    outs = {}
    for name in ("gemv_q4_k_q8_f16out_batched", "gemv_q4_k_q8_f16out_mtok", "mmq_q4_k_q8_f16out"):
        y = torch.zeros(tok, rows, dtype=torch.float16, device=DEV)
        getattr(ops, name)(w_dev, xq, y, rows, k, tok)
        outs[name] = y.cpu().numpy()
        assert rel(outs[name].astype(np.float32), want) < 1e-3      # fp16 storage
        assert f16_close(outs[name], want)
    # the reference promises bit-identical outputs between these three launchers
    assert np.array_equal(outs["gemv_q4_k_q8_f16out_batched"].view(np.uint16),
                          outs["gemv_q4_k_q8_f16out_mtok"].view(np.uint16))
    assert np.array_equal(outs["mmq_q4_k_q8_f16out"].view(np.uint16),
                          outs["gemv_q4_k_q8_f16out_mtok"].view(np.uint16))
    for name in ("gemv2_q4_k_q8_f16out_mtok", "mmq2_q4_k_q8_f16out"):
        yg = torch.zeros(tok, rows, dtype=torch.float16, device=DEV)
        yu = torch.zeros(tok, rows, dtype=torch.float16, device=DEV)
        getattr(ops, name)(w_dev, w2_dev, xq, yg, yu, rows, k, tok)
        assert np.array_equal(yg.cpu().numpy().view(np.uint16), outs["mmq_q4_k_q8_f16out"].view(np.uint16))
        assert f16_close(yu.cpu().numpy(), want2)


def test_ragged_rows_and_many_tokens(oracle):
    rows, k, tok = 37, 512, 19            # rows not a multiple of the tile, tokens > one tile
    w_np, w_dev = make_q4k(rows, k, 5)
    x_np, x_dev = make_x16(tok, k, 6)
    xq = quantize_dev(x_dev)
    xq_np = xq.cpu().numpy()
    want = np.stack([oracle.gemv(w_np, xq_np[t], rows, k) for t in range(tok)])
    y = torch.full((tok, rows + 3), 7.0, dtype=torch.float32, device=DEV)
    yv = torch.zeros(tok, rows, dtype=torch.float32, device=DEV)
    ops.gemv_q4_k_q8_batched(w_dev, xq, yv, rows, k, tok)
    assert rel(yv.cpu().numpy(), want) < GEMV_TOL
    assert torch.all(y == 7.0)


def test_unaligned_weight_pointers_take_the_plain_copy_path(oracle):
    rows, k = 64, 2048
    w_np, _ = make_q4k(rows, k, 9)
    x_np, x_dev = make_x16(1, k, 10)
    xq = quantize_dev(x_dev)
    want = oracle.gemv(w_np, xq.cpu().numpy()[0], rows, k)
    for shift in (4, 2, 8):
        buf = torch.zeros(w_np.size + 64, dtype=torch.uint8, device=DEV)
        buf[shift:shift + w_np.size] = dev(w_np.reshape(-1))
        y = torch.zeros(rows, dtype=torch.float32, device=DEV)
        ops.gemv_q4_k_q8(buf[shift:], xq, y, rows, k)
        assert rel(y.cpu().numpy(), want) < GEMV_TOL


def test_pointer_table_gemv(oracle):
    """n_hit experts in one launch: y[e*rows_per + r]; every expert reads the one
    activation row it is given (the reference kernel's behaviour)."""
    for rows_per, k in ((512, 2048), (2048, 512)):
        mats = [make_q4k(rows_per, k, 30 + e) for e in range(5)]
        x_np, x_dev = make_x16(1, k, 12)
        xq = quantize_dev(x_dev)
        tab = ops.ptr_table([m[1] for m in mats], DEV)
        y = torch.zeros(5 * rows_per, dtype=torch.float16, device=DEV)
        ops.gemv_ptrs_q4_k_q8_f16out(tab, xq, y, 5, rows_per, k)
        want = np.concatenate([oracle.gemv(m[0], xq.cpu().numpy()[0], rows_per, k) for m in mats])
        assert f16_close(y.cpu().numpy(), want)


def _host_plan(m_per_job, tok_per):
    off = np.concatenate([[0], np.cumsum(m_per_job)[:-1]]).astype(np.int32)
    tiles = [(m + tok_per - 1) // tok_per for m in m_per_job]
    tile_base = np.concatenate([[0], np.cumsum(tiles)[:-1]]).astype(np.int32)
    job_of_tile = np.concatenate([[j] * t for j, t in enumerate(tiles)]).astype(np.int32)
    return off, np.asarray(m_per_job, dtype=np.int32), tile_base, job_of_tile


@pytest.mark.parametrize("tok_per", [1, 4, 16])
def test_grouped_host_plan(oracle, tok_per):
    n_ff, hidden = 512, 2048
    m_per_job = [1, 3, 7, 2, 17]
    jobs = len(m_per_job)
    gates = [make_q4k(n_ff, hidden, 40 + j) for j in range(jobs)]
    ups = [make_q4k(n_ff, hidden, 50 + j) for j in range(jobs)]
    downs = [make_q4k(hidden, n_ff, 60 + j) for j in range(jobs)]
    R = sum(m_per_job)
    x_np, x_dev = make_x16(R, hidden, 13)
    xq = quantize_dev(x_dev)
    xq_np = xq.cpu().numpy()
    off, m, tile_base, job_of_tile = _host_plan(m_per_job, tok_per)
    yg = torch.zeros(R, n_ff, dtype=torch.float16, device=DEV)
    yu = torch.zeros(R, n_ff, dtype=torch.float16, device=DEV)
    ops.gemv_grouped2_q4_k_q8_f16out_mtok(
        ops.ptr_table([g[1] for g in gates], DEV), ops.ptr_table([u[1] for u in ups], DEV),
        dev(off), dev(m), dev(tile_base), dev(job_of_tile), len(job_of_tile), xq, yg, yu, n_ff,
        hidden, tok_per)
    h_np, h_dev = make_x16(R, n_ff, 14)
    hq = quantize_dev(h_dev)
    hq_np = hq.cpu().numpy()
    yd = torch.zeros(R, hidden, dtype=torch.float16, device=DEV)
    ops.gemv_grouped_q4_k_q8_f16out_mtok(
        ops.ptr_table([d[1] for d in downs], DEV), dev(off), dev(m), dev(tile_base),
        dev(job_of_tile), len(job_of_tile), hq, yd, hidden, n_ff, tok_per)
    for j in range(jobs):
        for t in range(m_per_job[j]):
            r = off[j] + t
            assert f16_close(yg[r].cpu().numpy(), oracle.gemv(gates[j][0], xq_np[r], n_ff, hidden))
            assert f16_close(yu[r].cpu().numpy(), oracle.gemv(ups[j][0], xq_np[r], n_ff, hidden))
            assert f16_close(yd[r].cpu().numpy(), oracle.gemv(downs[j][0], hq_np[r], hidden, n_ff))


@pytest.mark.parametrize("tok_per", [1, 4])
def test_grouped_device_plan_with_absent_experts(oracle, tok_per):
    """Device plan + pointer table: null entries give zero rows and one mail per
    tile from the gate/up launch (the reference's mailbox contract)."""
    n_ff, hidden, E, K, n = 256, 512, 12, 3, 9
    rng = np.random.default_rng(77)
    idx = np.zeros((n, K + 1), dtype=np.int32)
    for r in range(n):
        idx[r, :K] = rng.choice(E, K, replace=False)
    w = rng.random((n, K + 1)).astype(np.float32)
    plan = oracle.dispatch_scan(idx, w, n, K, E, tok_per)
    absent = {int(idx[0, 0]), int(idx[3, 1])}
    mats = {e: [make_q4k(n_ff, hidden, 300 + e), make_q4k(n_ff, hidden, 400 + e),
                make_q4k(hidden, n_ff, 500 + e)] for e in range(E)}
    tabs = [ops.ptr_table([None if e in absent else mats[e][mi][1] for e in range(E)], DEV)
            for mi in range(3)]
    R = int(plan["meta"][0])
    x_np, x_dev = make_x16(n, hidden, 15)
    xq_rows = quantize_dev(x_dev)
    xqg = torch.zeros(R, hidden // 256 * 276, dtype=torch.uint8, device=DEV)
    ops.gather_rows_q8(xqg, xq_rows, dev(plan["grows"][:R]), R, hidden // 256)
    xqg_np = xqg.cpu().numpy()
    assert np.array_equal(xqg_np, xq_rows.cpu().numpy()[plan["grows"][:R]])
    mail = torch.full((E,), -1, dtype=torch.int32, device=DEV)
    mail_n = torch.zeros(1, dtype=torch.int32, device=DEV)
    yg = torch.full((R, n_ff), 9.0, dtype=torch.float16, device=DEV)
    yu = torch.full((R, n_ff), 9.0, dtype=torch.float16, device=DEV)
    tiles_max = int(plan["meta"][1]) + 5                   # grid may over-provision
    d_off, d_toff, d_meta = dev(plan["off"]), dev(plan["toff"]), dev(plan["meta"])
    ops.gemv_grouped2_tab_q4_k_q8_f16out_mtok(tabs[0], tabs[1], d_off, d_toff, d_meta, mail, mail_n,
                                              tiles_max, xqg, yg, yu, n_ff, hidden, E, tok_per)
    h_np, h_dev = make_x16(R, n_ff, 16)
    hq = quantize_dev(h_dev)
    yd = torch.full((R, hidden), 9.0, dtype=torch.float16, device=DEV)
    ops.gemv_grouped_tab_q4_k_q8_f16out_mtok(tabs[2], d_off, d_toff, d_meta, tiles_max, hq, yd,
                                             hidden, n_ff, E, tok_per)
    hq_np = hq.cpu().numpy()
    mails_expected = []
    for e in range(E):
        lo, hi = plan["off"][e], plan["off"][e + 1]
        if e in absent:
            assert torch.all(yg[lo:hi] == 0) and torch.all(yu[lo:hi] == 0) and torch.all(yd[lo:hi] == 0)
            mails_expected += [e] * int(plan["toff"][e + 1] - plan["toff"][e])
            continue
        for r in range(lo, hi):
            assert f16_close(yg[r].cpu().numpy(), oracle.gemv(mats[e][0][0], xqg_np[r], n_ff, hidden))
            assert f16_close(yu[r].cpu().numpy(), oracle.gemv(mats[e][1][0], xqg_np[r], n_ff, hidden))
            assert f16_close(yd[r].cpu().numpy(), oracle.gemv(mats[e][2][0], hq_np[r], hidden, n_ff))
    n_mail = int(mail_n.item())
    assert sorted(mail.cpu().numpy()[:n_mail].tolist()) == sorted(mails_expected)
