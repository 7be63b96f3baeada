"""GPU parity: dispatch plan, row movement, SwiGLU, gates and combine through the
C ABI, against the oracle's restatement of src/kernels/cuda/moe.cu and
norm_rotary.cu:133-183 of the reference. Integer outputs and row copies are
bit-exact; fp16 blends may differ by one fp16 step (device expf / FMA)."""
import numpy as np
import pytest
import torch

from sager_b200 import ops
from tests.util import DEV, dev, f16_ulp_diff, make_x16

pytestmark = pytest.mark.gpu


def run_scan(idx, w, n, k, e, tok):
    d_w = dev(w.copy())
    out = dict(gslot=torch.full((max(1, n * k),), -9, dtype=torch.int32, device=DEV),
               grows=torch.full((max(1, n * k),), -9, dtype=torch.int32, device=DEV),
               off=torch.zeros(e + 1, dtype=torch.int32, device=DEV),
               toff=torch.zeros(e + 1, dtype=torch.int32, device=DEV),
               meta=torch.full((4,), 7, dtype=torch.int32, device=DEV),
               mail_n=torch.full((1,), 5, dtype=torch.int32, device=DEV))
    ops.moe_dispatch_scan(dev(idx), d_w, out["gslot"], out["grows"], out["off"], out["toff"],
                          out["meta"], None, out["mail_n"], n, k, e, tok)
    res = {kk: v.cpu().numpy() for kk, v in out.items()}
    res["weight"] = d_w.cpu().numpy()
    return res


@pytest.mark.parametrize("n,k,e,tok", [(1, 8, 256, 16), (4, 8, 256, 16), (64, 8, 256, 4), (7, 3, 10, 4)])
def test_dispatch_scan_matches_oracle(oracle, n, k, e, tok):
    rng = np.random.default_rng(n * 31 + e)
    idx = np.zeros((n, k + 1), dtype=np.int32)
    for r in range(n):
        idx[r, :k] = rng.choice(e, k, replace=False)
    if n >= 4:
        idx[2, 1] = e + 3                 # corrupt ids: row silenced, route dropped
        idx[3, 0] = -1
    w = rng.random((n, k + 1)).astype(np.float32)
    got = run_scan(idx, w, n, k, e, tok)
    want = oracle.dispatch_scan(idx, w, n, k, e, tok)
    for key in ("off", "toff", "weight"):
        assert np.array_equal(got[key], want[key]), key
    assert np.array_equal(got["meta"][:3], want["meta"][:3])
    R = want["meta"][0]
    assert np.array_equal(got["gslot"][:n * k], want["gslot"])      # stable order below 4096 routes
    assert np.array_equal(got["grows"][:R], want["grows"][:R])
    assert got["mail_n"][0] == 0                                      # the scan resets the mailbox


def test_dispatch_scan_large_plan_properties():
    n, k, e, tok = 2048, 8, 256, 16       # prefill-sized: atomic fill, order inside an expert free
    rng = np.random.default_rng(5)
    idx = np.zeros((n, k + 1), dtype=np.int32)
    idx[:, :k] = np.argsort(rng.random((n, e)), axis=1)[:, :k]
    w = np.ones((n, k + 1), dtype=np.float32)
    got = run_scan(idx, w, n, k, e, tok)
    hist = np.bincount(idx[:, :k].reshape(-1), minlength=e)
    assert np.array_equal(np.diff(got["off"]), hist)
    assert np.array_equal(np.diff(got["toff"]), (hist + tok - 1) // tok)
    assert got["meta"][:3].tolist() == [n * k, int(((hist + tok - 1) // tok).sum()), 0]
    gs = got["gslot"].reshape(n, k)
    assert np.array_equal(np.sort(gs.reshape(-1)), np.arange(n * k))  # a permutation
    ex_of_slot = np.searchsorted(got["off"], gs, side="right") - 1
    assert np.array_equal(ex_of_slot, idx[:, :k])
    assert np.array_equal(got["grows"][gs.reshape(-1)], np.repeat(np.arange(n), k))


def test_gathers_and_scatters_are_exact_copies():
    rng = np.random.default_rng(9)
    n, hidden, k = 6, 2048, 3
    x_np, x_dev = make_x16(n, hidden, 1)
    rows = rng.integers(0, n, 11).astype(np.int32)
    meta = torch.tensor([8, 0, 0, 0], dtype=torch.int32, device=DEV)
    dst = torch.zeros(11, hidden, dtype=torch.float16, device=DEV)
    ops.gather_rows_f16_n(dst, x_dev, dev(rows), meta, 11, hidden)
    assert np.array_equal(dst.cpu().numpy()[:8].view(np.uint16), x_np[rows[:8]].view(np.uint16))
    assert torch.all(dst[8:] == 0)
    q = torch.from_numpy(rng.integers(0, 256, (n, 2 * 276), dtype=np.uint8)).to(DEV)   # k=512 rows: 552 B
    dq = torch.zeros(11, 2 * 276, dtype=torch.uint8, device=DEV)
    ops.gather_rows_q8_n(dq, q, dev(rows), meta, 11, 2)
    assert np.array_equal(dq.cpu().numpy()[:8], q.cpu().numpy()[rows[:8]]) and torch.all(dq[8:] == 0)
    ops.gather_rows_q8(dq, q, dev(rows), 11, 2)
    assert np.array_equal(dq.cpu().numpy(), q.cpu().numpy()[rows])
    # scatter_rows: dst[dst_rows[i]] = src[i]
    perm = rng.permutation(n).astype(np.int32)
    out = torch.zeros(n, hidden, dtype=torch.float16, device=DEV)
    ops.scatter_rows_f16(out, x_dev, dev(perm), n, hidden)
    assert np.array_equal(out.cpu().numpy()[perm].view(np.uint16), x_np.view(np.uint16))
    # scatter_routed: slab [n][k+1][hidden], gslot < 0 leaves the slot alone
    g_np, g_dev = make_x16(n * k, hidden, 2)
    gslot = rng.permutation(n * k).astype(np.int32)
    gslot[4] = -1
    slab = torch.full((n, k + 1, hidden), 3.0, dtype=torch.float16, device=DEV)
    ops.scatter_routed_f16(slab, g_dev, dev(gslot), n, k, hidden)
    s = slab.cpu().numpy()
    for r in range(n):
        for kk in range(k):
            gsl = gslot[r * k + kk]
            if gsl < 0:
                assert np.all(s[r, kk] == 3.0)
            else:
                assert np.array_equal(s[r, kk].view(np.uint16), g_np[gsl].view(np.uint16))
        assert np.all(s[r, k] == 3.0)
    # fp32 -> fp16 scatters
    m = rng.standard_normal((2, hidden)).astype(np.float32)
    eo = torch.full((k, hidden), 1.0, dtype=torch.float16, device=DEV)
    ops.scatter_miss_f32(eo, dev(np.int32([-1, 1, 0])), dev(m), k, hidden)
    e = eo.cpu().numpy()
    assert np.all(e[0] == 1.0) and np.array_equal(e[1], m[1].astype(np.float16)) and np.array_equal(e[2], m[0].astype(np.float16))
    flat = np.int32([hidden * 5, 0])
    dd = torch.zeros(8 * hidden, dtype=torch.float16, device=DEV)
    ops.scatter_rows_generic_f16(dd, dev(m), dev(flat), 2, hidden)
    d2 = dd.cpu().numpy()
    assert np.array_equal(d2[hidden * 5:hidden * 6], m[0].astype(np.float16)) and np.array_equal(d2[:hidden], m[1].astype(np.float16))


def test_silu_mul_and_gates(oracle):
    g_np, g_dev = make_x16(9, 512, 3, std=2.0)
    u_np, u_dev = make_x16(9, 512, 4)
    out = torch.zeros(9, 512, dtype=torch.float16, device=DEV)
    ops.silu_mul_f16(out, g_dev, u_dev, 9, 512)
    want = oracle.silu_mul_f16(g_np, u_np)
    assert f16_ulp_diff(out.cpu().numpy(), want) <= 1
    out2 = torch.full((9, 512), 5.0, dtype=torch.float16, device=DEV)
    ops.silu_mul_f16_n(out2, g_dev, u_dev, torch.tensor([4], dtype=torch.int32, device=DEV), 9, 512)
    assert torch.equal(out2[:4], out[:4]) and torch.all(out2[4:] == 5.0)
    # in place, as the reference's session calls it (out == g)
    gg = g_dev.clone()
    ops.silu_mul_f16(gg, gg, u_dev, 9, 512)
    assert torch.equal(gg, out)
    gate = np.float32([0.3, -1.2, 4.0])
    y_np, y_dev = make_x16(3, 2048, 5)
    yb = y_dev.clone()
    ops.sigmoid_gate_scalar_batched_f16(yb, dev(gate), 3, 2048)
    want = (y_np.astype(np.float32) * (1.0 / (1.0 + np.exp(-gate)))[:, None].astype(np.float32)).astype(np.float16)
    assert f16_ulp_diff(yb.cpu().numpy(), want) <= 1
    y1 = y_dev[0].clone()
    ops.sigmoid_gate_scalar_f16(y1, dev(gate[:1]), 2048)
    assert torch.equal(y1, yb[0])


def test_combine_variants(oracle):
    rng = np.random.default_rng(12)
    n, K, hidden = 5, 8, 2048
    res_np, res_dev = make_x16(n, hidden, 6)
    y_np, y_dev = make_x16(n * (K + 1), hidden, 7, std=0.3)
    w = rng.random((n, K + 1)).astype(np.float32)
    out = res_dev.clone()
    ops.moe_combine_batched_f16(out, y_dev, dev(w), K, hidden, n)
    want = oracle.combine_batched_f16(res_np, y_np, w, K, hidden, n)
    assert f16_ulp_diff(out.cpu().numpy(), want.view(np.float16).reshape(n, hidden)) <= 1
    # single row with idx: negative ids are skipped; called with K+1 slots like the session does
    idx = rng.integers(0, 256, K + 1).astype(np.int32)
    idx[2] = -1
    o1 = res_dev[0].clone()
    ops.moe_combine_f16(o1, y_dev[:K + 1], dev(idx), dev(w[0]), K + 1, hidden)
    want1 = oracle.combine_f16(res_np[0], y_np[:K + 1], idx, w[0], K + 1, hidden)
    assert f16_ulp_diff(o1.cpu().numpy(), want1.view(np.float16)) <= 1
    # late add of patched slots, applied one after another
    rk = np.int32([0 * (K + 1) + 3, 0 * (K + 1) + 5, 2 * (K + 1) + 1])
    o2 = res_dev.clone()
    ops.moe_combine_add_slots_f16(o2, y_dev, dev(w.reshape(-1)), dev(rk), K, hidden, 3)
    ref = res_np.astype(np.float32).copy()
    for s in rk:
        r = s // (K + 1)
        ref[r] = (ref[r] + w.reshape(-1)[s] * y_np[s].astype(np.float32)).astype(np.float16).astype(np.float32)
    assert f16_ulp_diff(o2.cpu().numpy(), ref.astype(np.float16)) <= 1
    assert torch.equal(o2[1], res_dev[1])
