"""CPU checks that pin oracle/sager_oracle.c.

Three anchors: (1) the golden vectors the reference's own CPU code wrote
(tests/golden/ref_cpu_golden.npz), (2) the reference build itself when
oracle/_ref is present, (3) the invariants the reference's host test checks
(tests/test_q4_host.cpp in the reference tree).
"""
import numpy as np
import pytest

FP32_TOL = 1e-5   # fp32 order / FMA-contraction differences, relative to max |ref|


def rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


# ---- golden vectors -------------------------------------------------------------
def test_golden_q8_quantiser_bit_exact(oracle, golden):
    assert np.array_equal(oracle.quantize_q8k(golden["gemv_x"]), golden["gemv_xq"])
    assert np.array_equal(oracle.quantize_q8k(golden["q8_edge_x"]), golden["q8_edge_q"])
    x16 = golden["gemv_x"].astype(np.float16)
    assert np.array_equal(oracle.quantize_q8k_f16(x16), golden["gemv_xq"])


def test_golden_dequant_and_dots(oracle, golden):
    wq, xq = golden["gemv_wq"], golden["gemv_xq"]
    rows, k = wq.shape[0], 2048
    assert np.array_equal(oracle.dequant(wq[0], k), golden["gemv_dequant_row0"])
    for t in range(2):
        y = oracle.gemv(wq, xq[t], rows, k)
        assert rel(y, golden["gemv_y_avx2"][t]) < FP32_TOL
        assert rel(y, golden["gemv_y_scalar"][t]) < FP32_TOL
        assert rel(oracle.gemv(wq, xq[t], rows, k, lane_order=True), golden["gemv_y_avx2"][t]) < FP32_TOL
    vd = np.array([oracle.vec_dot_ref(wq[r], xq[0], k) for r in range(rows)], dtype=np.float32)
    assert rel(vd, golden["gemv_vec_dot_ref"]) < FP32_TOL


def test_golden_int_dots_reproduce_reference_rows(oracle, golden):
    """Rebuild y from the oracle's int32 sub-block dots in float64: the integer
    part is what must be exact, so the fp64 recombination has to land on the
    reference's fp32 result to fp32 rounding."""
    wq, xq = golden["gemv_wq"], golden["gemv_xq"][0]
    rows, k = wq.shape[0], 2048
    dots = oracle.subblock_dots(wq, xq, rows, k)
    blocks = wq.reshape(rows, k // 256, 144)
    xb = xq.reshape(k // 256, 276)
    xd = xb[:, :4].copy().view(np.float32)[:, 0].astype(np.float64)
    bsums = xb[:, 260:].copy().view(np.int16).reshape(-1, 8).astype(np.float64)
    y = np.zeros(rows)
    for r in range(rows):
        for b in range(k // 256):
            d = float(blocks[r, b, 0:2].copy().view(np.float16)[0])
            dmin = float(blocks[r, b, 2:4].copy().view(np.float16)[0])
            sc = blocks[r, b, 4:16]
            for s in range(8):
                if s < 4:
                    d6, m6 = sc[s] & 63, sc[s + 4] & 63
                else:
                    d6 = (sc[s + 4] & 0xF) | ((sc[s - 4] >> 6) << 4)
                    m6 = (sc[s + 4] >> 4) | ((sc[s] >> 6) << 4)
                y[r] += xd[b] * (d * d6 * dots[r, b, s] - dmin * m6 * bsums[b, s])
    assert rel(y.astype(np.float32), golden["gemv_y_avx2"][0]) < FP32_TOL


def test_golden_expert_ffn(oracle, golden):
    y = oracle.expert_ffn(golden["ffn_wg"], golden["ffn_wu"], golden["ffn_wd"], golden["ffn_x"],
                          512, 256)
    assert rel(y, golden["ffn_y"]) < 1e-4   # one Q8(h) code may flip on an fp32 ulp


def test_golden_q4k_quantiser_close(oracle, golden):
    """The weight quantiser is a generator, not part of the timed path. Its
    error search compares fp32 sums, so a build with FMA contraction (the
    reference's) and one without (the oracle's) may pick a neighbouring
    (scale, min) pair on near ties: require >= 98 % identical bytes."""
    got = oracle.quantize_q4k(golden["gemv_w_f32"])
    want = golden["gemv_wq"][:4]
    assert (got == want).mean() > 0.98
    assert np.array_equal(got[:, :4].reshape(4, -1)[:, :4], want[:, :4])  # d, dmin of block 0


# ---- the reference build, when present ----------------------------------------------
def test_ref_full_size_expert_ffn(oracle, reference):
    """H=2048 / FFX=512, the geometry of the reference's own equivalence
    harness (tests/q4_equiv_test.cpp), same input distributions."""
    rng = np.random.default_rng(20260718)
    H, F = 2048, 512
    x = (rng.uniform(-1, 1, H) * 0.5).astype(np.float32)
    wg = reference.quantize_q4k((rng.uniform(-1, 1, (F, H)) * 0.05).astype(np.float32))
    wu = reference.quantize_q4k((rng.uniform(-1, 1, (F, H)) * 0.05).astype(np.float32))
    wd = reference.quantize_q4k((rng.uniform(-1, 1, (H, F)) * 0.05).astype(np.float32))
    y_ref = reference.expert_ffn(wg, wu, wd, x, H, F)
    y = oracle.expert_ffn(wg, wu, wd, x, H, F)
    assert rel(y, y_ref) < 1e-4
    xq = reference.quantize_q8k_avx2(x[None])
    assert np.array_equal(oracle.quantize_q8k(x[None]), xq)
    g_ref = reference.gemv(wg, xq[0], F, H)
    assert rel(oracle.gemv(wg, xq[0], F, H), g_ref) < FP32_TOL
    assert np.array_equal(reference.gemv(wg, xq[0], F, H, scalar=True), g_ref) or \
        rel(reference.gemv(wg, xq[0], F, H, scalar=True), g_ref) < 1e-4


def test_ref_fp16_tables(oracle, reference):
    for h in range(0, 65536, 7):
        a, b = oracle.lib.orc_half_to_float(h), reference.lib.ref_half_to_float(h)
        assert a == b or (a != a and b != b)
    rng = np.random.default_rng(3)
    for v in (rng.standard_normal(2000) * np.exp(rng.uniform(-12, 12, 2000))).astype(np.float32):
        assert oracle.lib.orc_float_to_half_trunc(float(v)) == reference.lib.ref_float_to_half(float(v))


def test_ref_pool_matches_direct_ffn(reference, golden):
    pool = reference.pool(2, 512, 256, 4)
    try:
        w3 = [golden["ffn_wg"], golden["ffn_wu"], golden["ffn_wd"]] * 3
        x = np.stack([golden["ffn_x"], golden["ffn_x"] * 0.5, -golden["ffn_x"]]).astype(np.float32)
        y = pool.run(w3, x)
        assert np.array_equal(y[0], golden["ffn_y"])
        assert np.array_equal(y[2], reference.expert_ffn(*w3[:3], x[2], 512, 256))
    finally:
        pool.close()
    # C4: a wrong geometry is refused (tests/test_q4_host.cpp:162-169)
    assert reference.lib.ref_validate_pool_geometry(2048, 768, 128, 144, 2048, 768, 128, 144) == 0
    assert reference.lib.ref_validate_pool_geometry(2048, 768, 128, 144, 2048, 4096, 128, 144) == 4


# ---- invariants of the reference's host test ------------------------------------------
def test_fp16_round_to_nearest_even_matches_numpy(oracle):
    rng = np.random.default_rng(11)
    vals = (rng.standard_normal(4000) * np.exp(rng.uniform(-14, 12, 4000))).astype(np.float32)
    vals = np.concatenate([vals, np.float32([0, -0.0, 65504, 65520, 65519.99, 6e-8, 2.98e-8, 1e-10])])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.lib.orc_float_to_half_rn(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)


def test_scale_pack_roundtrip(oracle):
    import ctypes as C
    rng = np.random.default_rng(7)
    for _ in range(1000):
        d = rng.integers(0, 64, 8).astype(np.uint8)
        m = rng.integers(0, 64, 8).astype(np.uint8)
        q = np.zeros(12, dtype=np.uint8)
        for j in range(8):
            oracle.lib.orc_set_scale_min_k4(j, q.ctypes.data, int(d[j]), int(m[j]))
        for j in range(8):
            gd, gm = C.c_uint8(), C.c_uint8()
            oracle.lib.orc_get_scale_min_k4(j, q.ctypes.data, C.addressof(gd), C.addressof(gm))
            assert gd.value == d[j] and gm.value == m[j]


def test_quant_dequant_error_budget(oracle):
    rng = np.random.default_rng(42)
    x = rng.standard_normal((1, 4096)).astype(np.float32)
    y = oracle.dequant(oracle.quantize_q4k(x), 4096)
    assert np.sqrt(((y - x[0]) ** 2).mean()) / np.sqrt((x[0] ** 2).mean()) < 0.10


def test_q8_scale_and_clamp(oracle):
    rng = np.random.default_rng(99)
    x = (rng.standard_normal((1, 1024)) * 3).astype(np.float32)
    q = oracle.quantize_q8k(x).reshape(4, 276)
    for b in range(4):
        d = q[b, :4].copy().view(np.float32)[0]
        assert abs(d - np.abs(x[0, b * 256:(b + 1) * 256]).max() / 127.0) < 1e-6
        codes = q[b, 4:260].view(np.int8)
        assert np.abs(codes.astype(int)).max() <= 127
        assert np.array_equal(codes.reshape(8, 32).astype(int).sum(1),
                              q[b, 260:].copy().view(np.int16).astype(int))


# ---- router / plan restatements (no reference test covers them: checked against numpy) ----
def test_router_topk_matches_numpy(oracle):
    rng = np.random.default_rng(5)
    for _ in range(50):
        logits = rng.standard_normal(256).astype(np.float32)
        idx, w = oracle.router_topk(logits, 8, shared_w=1.0)
        order = np.lexsort((np.arange(256), -logits))[:8]   # descending, ties -> lower index
        assert np.array_equal(idx[:8], order)
        p = np.exp(logits[order] - logits.max())
        assert np.allclose(w[:8], p / p.sum(), atol=1e-6)
        assert w[8] == 1.0


def test_router_topk_ties_nan_degenerate(oracle):
    logits = np.zeros(16, dtype=np.float32)
    idx, w = oracle.router_topk(logits, 4, shared_w=0.0)
    assert idx[:4].tolist() == [0, 1, 2, 3] and np.allclose(w[:4], 0.25) and w[4] == 0.0
    logits = np.array([1, np.nan, 3, 3, 2], dtype=np.float32)
    idx, _ = oracle.router_topk(logits, 3)
    assert idx[:3].tolist() == [0, 1, 2]     # NaN poisons max/z: every prob is NaN -> kk % E
    idx, w = oracle.router_topk(np.float32([0, 5, 5, 1]), 2, write_shared=False)
    assert idx[:2].tolist() == [1, 2] and w[2] == -7.0   # fused variant leaves slot K alone


def test_dispatch_scan_plan(oracle):
    rng = np.random.default_rng(8)
    n, k, e, tok = 7, 3, 10, 4
    idx = np.zeros((n, k + 1), dtype=np.int32)
    for r in range(n):
        idx[r, :k] = rng.choice(e, k, replace=False)
    idx[2, 1] = 99          # out of range: the row's weights are zeroed, the route dropped
    idx[5, 0] = -1
    w = rng.random((n, k + 1)).astype(np.float32)
    p = oracle.dispatch_scan(idx, w, n, k, e, tok)
    hist = np.bincount(idx[:, :k][(idx[:, :k] >= 0) & (idx[:, :k] < e)], minlength=e)
    assert np.array_equal(np.diff(p["off"]), hist)
    assert np.array_equal(np.diff(p["toff"]), (hist + tok - 1) // tok)
    assert p["meta"][:3].tolist() == [hist.sum(), ((hist + tok - 1) // tok).sum(), 2]
    assert np.all(p["weight"][2] == 0) and np.all(p["weight"][5] == 0)
    assert np.array_equal(p["weight"][0], w[0])
    assert p["gslot"][2 * k + 1] == -1 and p["gslot"][5 * k] == -1
    for r in range(n):
        for kk in range(k):
            g = p["gslot"][r * k + kk]
            if g >= 0:
                ex = idx[r, kk]
                assert p["off"][ex] <= g < p["off"][ex + 1] and p["grows"][g] == r


def test_moe_layer_is_sum_of_ffns(oracle, golden):
    rng = np.random.default_rng(21)
    H, F, E, K = 512, 256, 4, 2
    ex = (golden["ffn_wg"], golden["ffn_wu"], golden["ffn_wd"])
    experts = [ex, None, ex, ex]       # expert 1 absent -> contributes zero
    router = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    x16 = rng.standard_normal((3, H)).astype(np.float16)
    res = rng.standard_normal((3, H)).astype(np.float32)
    r = oracle.moe_layer(x16, router, experts, ex, res, K, F, shared_w=1.0, n_threads=2)
    for t in range(3):
        y = oracle.expert_ffn(*ex, x16[t].astype(np.float32), H, F)
        wsum = sum(r["w"][t, kk] for kk in range(K) if r["idx"][t, kk] != 1)
        assert rel(r["out"][t], res[t] + (wsum + 1.0) * y) < 1e-5
        assert np.array_equal(r["logits"][t], oracle.router_logits(router, x16[t]))


def test_rmsnorm_quant_restatement(oracle):
    """The CPU restatement of the fused norm + quantiser: the rows are the RMS norm (against a
    float64 evaluation, to the fp16 store) and the blocks are the Q8_K blocks of those rows."""
    from oracle.oracle import rmsnorm_quant_f16
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((3, 2048)) * 1.7).astype(np.float16)
    w = (1.0 + 0.1 * rng.standard_normal(2048)).astype(np.float16)
    out, xq = rmsnorm_quant_f16(oracle, x, w, 1e-6)
    xd = x.astype(np.float64)
    want = xd / np.sqrt((xd ** 2).mean(axis=1, keepdims=True) + 1e-6) * w.astype(np.float64)
    assert np.abs(out.astype(np.float64) - want).max() <= 2.0 ** -10 * np.abs(want).max() * 1.01
    assert np.array_equal(xq, oracle.quantize_q8k_f16(out))
    assert xq.shape == (3, 8 * 276)


def test_q6k_restatements_agree_with_each_other():
    """The integer-dot restatement of the Q6_K head GEMV against the dequantise-then-dot form
    (src/core/weights.cpp:168-209 of the reference), and the top-k rule on hand-made cases."""
    from oracle.oracle import dequant_q6k, gemv_q6k_q8k, make_q6k, topk_select
    from oracle.oracle import Oracle
    o = Oracle()
    rng = np.random.default_rng(2)
    k = 512
    w6 = make_q6k(rng, 9, k)
    x = rng.standard_normal(k).astype(np.float32)
    xq = o.quantize_q8k(x[None])[0]
    xb = xq.reshape(-1, 276)
    xdq = (xb[:, :4].copy().view(np.float32) * xb[:, 4:260].copy().view(np.int8).astype(np.float32)).reshape(-1)
    a = gemv_q6k_q8k(w6, xq, k)
    b = dequant_q6k(w6, k).astype(np.float64) @ xdq.astype(np.float64)
    assert np.abs(a - b).max() <= 1e-5 * np.abs(b).max()
    v, i = topk_select(np.float32([1, 5, 5, np.nan, -np.inf, 2, 5]), 5)
    assert i.tolist() == [1, 2, 6, 5, 0] and v.tolist() == [5, 5, 5, 2, 1]
    v, i = topk_select(np.float32([np.nan, -3.4e38]), 3)
    assert i.tolist() == [-1, -1, -1]
