"""GPU parity of the fused MoE layer (sgr_moe_layer_decode) against the oracle's
whole-layer restatement: router as the device computes it, every selected and
the shared expert through the CPU expert FFN, weighted sum in slot order.
Bars: selected experts exact in value and order, routing weights within 1e-6,
fp32 layer output within 1e-3 max relative error (the stated bound; the measured
figure is asserted an order of magnitude tighter)."""
import numpy as np
import pytest
import torch

from sager_b200 import lib, ops, synth
from sager_b200.layer import MoeLayerRunner, MoeStack
from tests.util import DEV, LAYER_TOL, dev, f16_close, rel

pytestmark = pytest.mark.gpu


def oracle_layer(oracle, w, x16_np, resid_np, k, absent=(), bias=None, n_threads=8, use_shared=True,
                 blob_np=None):
    """Run the oracle on the experts the routing needs only (the rest stay None). blob_np: a host
    copy of w.blob to slice the matrices from (saves one device copy per matrix)."""
    E = w.n_expert
    if blob_np is not None:
        o3 = [0, w.gu_bytes, 2 * w.gu_bytes, w.expert_bytes]
        mat = lambda e, m: blob_np[w.slot(e), o3[m]:o3[m + 1]]
    else:
        mat = lambda e, m: w.matrix(e, m).cpu().numpy()
    logits = np.stack([oracle.router_logits(w.router.cpu().numpy(), x16_np[t]) for t in range(x16_np.shape[0])])
    if bias is not None:
        logits = logits + bias[None, :]
    need = set()
    for t in range(x16_np.shape[0]):
        need |= set(oracle.router_topk(logits[t], k)[0][:k].tolist())
    experts = [None] * E
    for e in need:
        if e in absent:
            continue
        experts[e] = tuple(mat(e, m) for m in range(3))
    shared = tuple(mat(E, m) for m in range(3)) if use_shared else None
    router = w.router.cpu().numpy()
    if bias is not None:
        # the oracle computes logits itself: fold the bias in by routing on biased logits
        res = _oracle_with_logits(oracle, x16_np, logits, experts, shared, resid_np, k, w.n_ff, n_threads)
    else:
        res = oracle.moe_layer(x16_np, router, experts, shared, resid_np, k, w.n_ff, shared_w=1.0,
                               n_threads=n_threads)
    return res


def _oracle_with_logits(oracle, x16_np, logits, experts, shared, resid_np, k, n_ff, n_threads):
    n, H = x16_np.shape
    out = np.zeros((n, H), dtype=np.float32)
    idx = np.zeros((n, k + 1), dtype=np.int32)
    wts = np.zeros((n, k + 1), dtype=np.float32)
    jobs_w, jobs_x, slots = [], [], []
    for t in range(n):
        i, wv = oracle.router_topk(logits[t], k, shared_w=1.0)
        idx[t], wts[t] = i, wv
        idx[t, k] = -1
        for kk in range(k + 1):
            ex = experts[i[kk]] if kk < k else shared
            if ex is None:
                continue
            jobs_w += list(ex)
            jobs_x.append(x16_np[t].astype(np.float32))
            slots.append((t, kk))
    ys = oracle.expert_ffn_batch(jobs_w, np.stack(jobs_x), H, n_ff, n_threads)
    acc = resid_np.astype(np.float32).copy()
    per = {s: y for s, y in zip(slots, ys)}
    for t in range(n):
        for kk in range(k + 1):
            if (t, kk) in per:
                acc[t] = acc[t] + wts[t, kk] * per[(t, kk)]
    return dict(out=acc, idx=idx, w=wts, logits=logits)


def run_layer(w, n, k, x16_dev, n_max=None, absent=(), bias=None, use_shared=True, kernel=None):
    runner = MoeLayerRunner(n_max or n, w.hidden, w.n_ff, w.n_expert, k, DEV)
    x = x16_dev.clone()
    out32 = torch.zeros(n, w.hidden, dtype=torch.float32, device=DEV)
    a = runner.args(n, x16_dev, w.router, w.table(absent), w.shared_ptrs() if use_shared else None,
                    x_f16=x, out_f32=out32, bias=None if bias is None else dev(bias))
    runner.run(a, kernel=kernel)
    torch.cuda.synchronize()
    assert lib().raw("sgr_status")(0) == 0, "a bounded device-side wait gave up"
    return runner, x, out32


def check(oracle, w, n, k, seed, absent=(), bias=None, use_shared=True, n_max=None, tol=1e-4, kernel=None):
    x16 = synth.normal_fp16((n, w.hidden), seed, DEV)
    x_np = x16.cpu().numpy()
    runner, x_out, out32 = run_layer(w, n, k, x16, n_max=n_max, absent=absent, bias=bias,
                                     use_shared=use_shared, kernel=kernel)
    want = oracle_layer(oracle, w, x_np, x_np.astype(np.float32), k, absent=absent, bias=bias,
                        use_shared=use_shared)
    idx = runner.route_idx.cpu().numpy()[:n]
    wt = runner.route_w.cpu().numpy()[:n]
    assert np.array_equal(idx[:, :k], want["idx"][:, :k])
    assert np.abs(wt[:, :k] - want["w"][:, :k]).max() <= 1e-6
    assert np.all(wt[:, k] == 1.0)
    err = rel(out32.cpu().numpy(), want["out"])
    assert err < LAYER_TOL and err < tol, err
    assert f16_close(x_out.cpu().numpy(), want["out"], tol=tol)
    return runner, want, err


@pytest.fixture(scope="module")
def small_w():
    return synth.MoeWeights(512, 256, 16, DEV, seed=11, std=0.05)


@pytest.fixture(scope="module")
def full_w():
    # the benchmark geometry: hidden 2048, expert FFN 512, 256 experts + shared
    return synth.MoeWeights(2048, 512, 256, DEV, seed=20260718)


@pytest.mark.parametrize("kernel", ["items", "rows", None])
@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 17, 64])
def test_small_layer_all_row_counts(oracle, small_w, n, kernel):
    check(oracle, small_w, n, 4, seed=100 + n, n_max=64, kernel=kernel)


@pytest.mark.parametrize("kernel", ["items", "rows"])
def test_small_layer_without_shared_expert_and_with_bias(oracle, small_w, kernel):
    check(oracle, small_w, 3, 4, seed=7, use_shared=False, kernel=kernel)
    bias = synth.zipf_bias(16, seed=3, alpha=0.5)
    check(oracle, small_w, 9, 4, seed=8, bias=bias, kernel=kernel)
    # hot experts: full tiles of 16 rows and ragged ones. (The seed matters: h is requantised
    # to Q8_K between the projections, and when an h value sits on a rounding boundary the two
    # summation orders can pick different codes - one token row then moves by ~1e-3 of the
    # largest output on this 512-wide layer. This seed has no such value.)
    check(oracle, small_w, 40, 4, seed=12, bias=bias * 4, kernel=kernel)


@pytest.mark.parametrize("kernel", ["items", "rows"])
def test_absent_experts_contribute_zero_and_are_mailed(oracle, small_w, kernel):
    n, k = 6, 4
    x16 = synth.normal_fp16((n, 512), 55, DEV)
    r0, _, _ = run_layer(small_w, n, k, x16)
    used = sorted(set(r0.route_idx.cpu().numpy()[:n, :k].reshape(-1).tolist()))
    absent = (used[0], used[-1])
    runner, want, _ = check(oracle, small_w, n, k, seed=55, absent=absent, kernel=kernel)
    n_mail = int(runner.mail_n.item())
    mails = runner.mail.cpu().numpy()[:n_mail].tolist()
    assert sorted(set(mails)) == sorted(absent)


@pytest.mark.parametrize("kernel", ["items", "rows"])
@pytest.mark.parametrize("shift", [2, 4])
def test_weight_pointers_with_only_block_alignment(oracle, small_w, kernel, shift):
    """The pointer table only promises the alignment of the block struct (2 bytes): the
    same weights at addresses 2 and 4 bytes off a 16-byte boundary must give the same layer."""
    import copy
    w = copy.copy(small_w)
    big = torch.empty(small_w.blob.numel() + 16, dtype=torch.uint8, device=DEV)
    w.blob = big[shift:shift + small_w.blob.numel()].view(small_w.blob.shape)
    w.blob.copy_(small_w.blob)
    assert w.blob.data_ptr() % 16 == shift
    check(oracle, w, 21, 4, seed=77, kernel=kernel)


@pytest.mark.parametrize("kernel", ["items", "rows", None])
@pytest.mark.parametrize("n", [1, 2, 4, 64])
def test_benchmark_geometry(oracle, full_w, n, kernel):
    bias = synth.zipf_bias(256, seed=5, alpha=0.6) if n == 64 else None
    _, _, err = check(oracle, full_w, n, 8, seed=20260718 + n, bias=bias, n_max=64, kernel=kernel)
    print(f"n={n}: max relative error of the fp32 layer output = {err:.3e}")


def test_expert_ranges_partition_the_layer(full_w):
    """Expert parallelism on one device: two owner-side calls over disjoint expert
    ranges with the routing given, summed, reproduce the single call exactly up to
    fp32 addition order."""
    n, k = 16, 8
    w = full_w
    x16 = synth.normal_fp16((n, w.hidden), 77, DEV)
    runner, x_full, out_full = run_layer(w, n, k, x16, n_max=64)
    nb = w.hidden // 256
    xq = torch.zeros(n, nb * 276, dtype=torch.uint8, device=DEV)
    ops.quantize_q8_k(x16, xq, n * w.hidden)
    parts = []
    for lo, hi, sh in ((0, 128, (0, n)), (128, 256, None)):
        r = MoeLayerRunner(64, w.hidden, w.n_ff, w.n_expert, k, DEV, expert_lo=lo, expert_hi=hi)
        out = torch.zeros(n, w.hidden, dtype=torch.float32, device=DEV)
        a = r.args(n, None, None, w.table(), w.shared_ptrs() if sh else None, out_f32=out, xq_in=xq,
                   routing_given=True, no_residual=True, route_idx=runner.route_idx.clone(),
                   route_w=runner.route_w.clone())
        r.run(a)
        parts.append(out)
    torch.cuda.synchronize()
    total = x16.float() + parts[0] + parts[1]
    assert rel(total.cpu().numpy(), out_full.cpu().numpy()) < 1e-6


def test_stack_graph_replay_is_deterministic(oracle):
    layers = [synth.MoeWeights(512, 256, 16, DEV, seed=200 + i, std=0.05) for i in range(3)]
    n, k = 4, 4
    x0 = synth.normal_fp16((n, 512), 9, DEV)
    st = MoeStack(layers, 8, k, DEV)
    st.x[:n] = x0
    st.step_eager(n)
    torch.cuda.synchronize()
    eager = st.x[:n].clone()
    idx_eager = st.idx.clone()
    st.x[:n] = x0
    st.capture(n)
    outs = []
    for _ in range(3):
        st.x[:n] = x0
        st.replay()
        torch.cuda.synchronize()
        outs.append(st.x[:n].clone())
    assert all(torch.equal(o, eager) for o in outs)
    assert torch.equal(st.idx, idx_eager)
    # and the chain matches the oracle layer by layer (fp16 residual stream between layers)
    x_np = x0.cpu().numpy()
    for li, w in enumerate(layers):
        want = oracle_layer(oracle, w, x_np, x_np.astype(np.float32), k)
        assert np.array_equal(st.idx[li].cpu().numpy()[:n, :k], want["idx"][:, :k])
        x_np = want["out"].astype(np.float16)
    assert f16_close(eager.cpu().numpy(), x_np.astype(np.float32), tol=2e-3)
    from sager_b200 import lib
    assert lib().raw("sgr_status")(0) == 0


@pytest.mark.parametrize("padded", [False, True])
@pytest.mark.parametrize("world,tokens", [(4, 16), (4, 64), (8, 64)])
def test_expert_parallel_record_path_on_one_device(full_w, padded, world, tokens):
    """The expert-parallel layer with its exchanges done by hand on one device: each
    emulated rank routes its home rows straight into dispatch records (strided Q8_K
    rows, ids, weights), every rank's owner call runs its expert range over all
    records, partial sums are added at home. Must reproduce the single call."""
    import ctypes as C
    from sager_b200 import lib
    from sager_b200.ep import record_layout
    from sager_b200.ops import stream_ptr
    w, k = full_w, 8
    n_home = tokens // world
    x16 = synth.normal_fp16((tokens, w.hidden), 91, DEV)
    _, x_full, out_full = run_layer(w, tokens, k, x16, n_max=64)
    rec, idx_off, w_off = record_layout(w.hidden, k, padded)      # padded: Q8 rows in 288-byte blocks, read in place
    records = torch.zeros(world, n_home, rec, dtype=torch.uint8, device=DEV)
    for r in range(world):                                    # home side of every rank
        home = MoeLayerRunner(n_home, w.hidden, w.n_ff, w.n_expert, k, DEV)
        a = home.args(n_home, x16[r * n_home:(r + 1) * n_home].contiguous(), w.router, w.table(), None,
                      x_f16=torch.zeros(n_home, w.hidden, dtype=torch.float16, device=DEV))
        base = records[r].data_ptr()
        a.xq_out, a.xq_stride = C.c_void_p(base), rec
        a.route_idx, a.route_w = C.c_void_p(base + idx_off), C.c_void_p(base + w_off)
        a.route_stride = rec // 4
        a.xq_padded = int(padded)
        lib().call("sgr_moe_layer_decode_stages", C.byref(a), 1 | 8, stream_ptr())
    torch.cuda.synchronize()
    total = x16.float().clone()
    per = w.n_expert // world
    for r in range(world):                                    # owner side of every rank
        owner = MoeLayerRunner(64, w.hidden, w.n_ff, w.n_expert, k, DEV, expert_lo=r * per,
                               expert_hi=(r + 1) * per)
        part = torch.zeros(tokens, w.hidden, dtype=torch.float32, device=DEV)
        b = owner.args(tokens, None, None, w.table(), w.shared_ptrs(), out_f32=part, xq_in=records,
                       routing_given=True, no_residual=True, shared_lo=r * n_home,
                       shared_hi=(r + 1) * n_home)
        b.xq_stride, b.route_stride = rec, rec // 4
        b.xq_padded = int(padded)
        b.route_idx = C.c_void_p(records.data_ptr() + idx_off)
        b.route_w = C.c_void_p(records.data_ptr() + w_off)
        lib().call("sgr_moe_layer_decode_stages", C.byref(b), 7, stream_ptr())
        torch.cuda.synchronize()
        total += part
    assert rel(total.cpu().numpy(), out_full.cpu().numpy()) < 1e-6
    # and the home-side reduction kernel
    xh = x16[:n_home].clone()
    parts = torch.randn(world, n_home, w.hidden, device=DEV)
    lib().call("sgr_ep_reduce_add_f16", C.c_void_p(xh.data_ptr()), C.c_void_p(parts.data_ptr()), world,
               n_home * w.hidden, n_home * w.hidden, stream_ptr())
    want = x16[:n_home].float()
    for p_ in range(world):
        want = want + parts[p_]
    assert torch.equal(xh, want.half())


def test_route_only_stage_repeats_on_one_workspace(full_w):
    """The home side of expert parallelism calls the route stage without the plan once per layer on
    one workspace: the second call must route its own rows (its per-tile counters start at zero
    again), not leave the first call's routing in place."""
    import ctypes as C
    from sager_b200.ops import stream_ptr
    w, k, n = full_w, 8, 32
    runner = MoeLayerRunner(n, w.hidden, w.n_ff, w.n_expert, k, DEV)
    picks = []
    for seed in (301, 302):
        x16 = synth.normal_fp16((n, w.hidden), seed, DEV)
        a = runner.args(n, x16, w.router, w.table(), None,
                        x_f16=torch.zeros(n, w.hidden, dtype=torch.float16, device=DEV))
        lib().call("sgr_moe_layer_decode_stages", C.byref(a), 1 | 8, stream_ptr())
        torch.cuda.synchronize()
        idx = runner.route_idx.cpu().numpy()[:n, :k].copy()
        want = (x16.float() @ w.router.t()).topk(k, dim=1).indices.cpu().numpy()
        assert np.array_equal(np.sort(idx, axis=1), np.sort(want, axis=1)), seed
        picks.append(idx)
    assert not np.array_equal(picks[0], picks[1])


def test_peer_memory_entry_points_with_one_rank():
    """sgr_ep_push / the waits / sgr_ep_step_advance with this device as its own only peer: the
    bytes arrive, the arrival word takes step * mul + add, a wait on a word that is already set
    returns, and the step counter advances in stream order."""
    import ctypes as C
    from sager_b200.ops import stream_ptr
    L, sp = lib(), stream_ptr()
    src = torch.arange(4096, dtype=torch.int32, device=DEV)
    dst = torch.zeros(2, 4096, dtype=torch.int32, device=DEV)
    flags = torch.zeros(2, dtype=torch.int32, device=DEV)
    step = torch.full((1,), 3, dtype=torch.int32, device=DEV)
    scratch = torch.zeros(1, dtype=torch.int32, device=DEV)
    dptr = torch.tensor([dst[0].data_ptr(), dst[1].data_ptr()], dtype=torch.int64, device=DEV)
    fptr = torch.tensor([flags.data_ptr(), flags.data_ptr() + 4], dtype=torch.int64, device=DEV)
    p = lambda t: C.c_void_p(t.data_ptr())
    L.call("sgr_ep_push", p(src), 0, src.numel() * 4, p(dptr), p(fptr), 2, p(step), 5, 2, p(scratch), sp)
    torch.cuda.synchronize()
    assert torch.equal(dst[0], src) and torch.equal(dst[1], src)
    assert flags.tolist() == [17, 17] and int(scratch.item()) == 0
    x = torch.ones(1024, dtype=torch.float16, device=DEV)
    parts = torch.full((2, 1024), 0.5, dtype=torch.float32, device=DEV)
    L.call("sgr_ep_reduce_add_f16_wait", p(x), p(parts), 2, 1024, 1024, p(flags), p(step), 5, 2, sp)
    L.call("sgr_ep_step_advance", p(step), sp)
    torch.cuda.synchronize()
    assert torch.all(x == 2.0) and int(step.item()) == 4
    assert lib().raw("sgr_status")(0) == 0


# ---- seed sweep at the benchmark geometry ---------------------------------------------------------
def _h_code_flips(oracle, w, blob_np, runner, x16_np, idx_row, t, k):
    """For token row t of a finished call: the Q8_K codes of h (the SwiGLU output that is
    requantised between the projections) as the device's fp32 h rows give them, against the codes
    the CPU path's h gives. -> (codes compared, codes that differ)."""
    H, F, E, n_max = w.hidden, w.n_ff, w.n_expert, runner.n_max
    off = lambda which: lib().raw("sgr_moe_layer_workspace_offset")(n_max, H, F, E, k, which)
    rows = n_max * k + n_max
    ws = runner.ws
    hbuf = ws[off(0):off(0) + rows * F * 4].view(torch.float32).view(rows, F)
    gslot = ws[off(2):off(2) + n_max * k * 4].view(torch.int32).cpu().numpy()
    o3 = [0, w.gu_bytes, 2 * w.gu_bytes]
    xq = oracle.quantize_q8k(x16_np[t].astype(np.float32)[None])[0]
    total = flips = 0
    for kk in range(k + 1):
        e = int(idx_row[kk]) if kk < k else E
        row = int(gslot[t * k + kk]) if kk < k else n_max * k + t
        g = oracle.gemv(blob_np[w.slot(e), o3[0]:o3[1]], xq, F, H)
        u = oracle.gemv(blob_np[w.slot(e), o3[1]:o3[2]], xq, F, H)
        h_cpu = (g / (np.float32(1) + np.exp(-g, dtype=np.float32)) * u).astype(np.float32)
        h_dev = hbuf[row].cpu().numpy()
        qa = oracle.quantize_q8k(h_cpu[None])[0].reshape(-1, 276)[:, 4:260]
        qb = oracle.quantize_q8k(h_dev[None])[0].reshape(-1, 276)[:, 4:260]
        total += qa.size
        flips += int((qa != qb).sum())
    return total, flips


@pytest.mark.parametrize("kernel", ["items", "rows", None])
def test_benchmark_geometry_seed_sweep(oracle, kernel):
    """32 seeded cases (4 weight sets x 8 input sets) x 1, 4 and 64 token rows, none of them picked:
    every case must meet the stated bound of 1e-3 against the CPU expert path, and the distribution
    is printed. Where a case is far from the typical 1e-7, the cause is counted, not assumed: h is
    requantised to Q8_K between the projections, and a value that sits on a rounding boundary can
    take another code on the device (other fp32 summation order, expf) than on the CPU."""
    k = 8
    errs = {1: [], 4: [], 64: []}
    worst = (0.0, None)
    for wi, wseed in enumerate((20260718, 11, 12, 13)):
        w = synth.MoeWeights(2048, 512, 256, DEV, seed=wseed)
        blob_np = w.blob.cpu().numpy()
        for xi in range(8):
            for n in (1, 4, 64):
                seed = 5000 + 100 * wi + 10 * xi + n
                bias = synth.zipf_bias(256, seed=seed, alpha=0.6) if n == 64 else None
                x16 = synth.normal_fp16((n, w.hidden), seed, DEV)
                x_np = x16.cpu().numpy()
                runner, _, out32 = run_layer(w, n, k, x16, n_max=64, bias=bias, kernel=kernel)
                want = oracle_layer(oracle, w, x_np, x_np.astype(np.float32), k, bias=bias, blob_np=blob_np,
                                    n_threads=16)
                idx = runner.route_idx.cpu().numpy()[:n]
                assert np.array_equal(idx[:, :k], want["idx"][:, :k]), (wseed, xi, n)
                got = out32.cpu().numpy()
                err = rel(got, want["out"])
                errs[n].append(err)
                if err > worst[0]:
                    t = int(np.abs(got - want["out"]).max(axis=1).argmax())
                    worst = (err, (wseed, xi, n, t) + _h_code_flips(oracle, w, blob_np, runner, x_np, idx[t], t, k))
        del w
    for n, v in errs.items():
        print(f"{kernel} kernel, {n:2d} rows: {len(v)} cases, max relative error median {np.median(v):.2e}, "
              f"max {np.max(v):.2e}")
    wseed, xi, n, t, total, flips = worst[1]
    print(f"worst case (weights {wseed}, inputs {xi}, {n} rows, row {t}): {worst[0]:.2e}; "
          f"{flips} of {total} Q8_K codes of h differ from the CPU path's")
    assert max(max(v) for v in errs.values()) <= LAYER_TOL


def test_strided_pointer_table_is_used_in_place(small_w):
    """The reference's decode table is [3][Lm][E] (src/core/session.cpp:3596-3598): a layer's
    gate / up / down slices are Lm * E pointers apart. tab_stride takes them where they are."""
    k, Lm, li = 4, 3, 2
    E = small_w.n_expert
    for kernel, n in (("items", 9), ("rows", 9), (None, 3)):
        x16 = synth.normal_fp16((n, small_w.hidden), 431, DEV)
        _, _, want = run_layer(small_w, n, k, x16, n_max=16, kernel=kernel)
        big = torch.zeros(3, Lm, E, dtype=torch.int64, device=DEV)
        big[:, li, :] = small_w.table()
        runner = MoeLayerRunner(16, small_w.hidden, small_w.n_ff, E, k, DEV)
        out32 = torch.zeros(n, small_w.hidden, dtype=torch.float32, device=DEV)
        a = runner.args(n, x16, small_w.router, big[0, li], small_w.shared_ptrs(), x_f16=x16.clone(), out_f32=out32)
        a.tab_stride = Lm * E
        runner.run(a, kernel=kernel)
        torch.cuda.synchronize()
        assert torch.equal(out32, want)
    assert lib().raw("sgr_status")(0) == 0


@pytest.mark.parametrize("hidden,n_ff", [(256, 2048), (2048, 256)])
def test_rows_kernel_with_one_block_column_per_group(oracle, hidden, n_ff):
    """hidden == 256 (gate / up groups) or n_ff == 256 (down groups) makes a group a single stage, so
    a CTA that draws several groups changes tile with every stage: more tiles than descriptor
    slots pass through a CTA while earlier copies are still in flight. 64 rows x top-8 over 64
    experts are about 70 tiles and several hundred single-stage groups, a handful per CTA."""
    E, k, n = 64, 8, 64
    w = synth.MoeWeights(hidden, n_ff, E, DEV, seed=77, std=0.05)
    for seed in (1, 2):
        check(oracle, w, n, k, seed=900 + seed, n_max=64, kernel="rows", tol=1e-3)


# ---- the single persistent launch for up to three token rows (kernel=None; four rows covered too,
# whichever path the library picks there) --------------------------------------------------------
@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_token_kernel_variants(oracle, small_w, n):
    """Without the shared expert, with a router bias, with absent experts (zero contribution, id
    mailed once), and with weight pointers that are only 2- or 4-byte aligned."""
    import copy
    k = 4
    check(oracle, small_w, n, k, seed=600 + n, use_shared=False)
    bias = synth.zipf_bias(16, seed=3, alpha=2.0)
    check(oracle, small_w, n, k, seed=610 + n, bias=bias)
    x16 = synth.normal_fp16((n, 512), 620 + n, DEV)
    r0, _, _ = run_layer(small_w, n, k, x16)
    used = sorted(set(r0.route_idx.cpu().numpy()[:n, :k].reshape(-1).tolist()))
    absent = (used[0], used[-1])
    runner, _, _ = check(oracle, small_w, n, k, seed=620 + n, absent=absent)
    n_mail = int(runner.mail_n.item())
    assert sorted(runner.mail.cpu().numpy()[:n_mail].tolist()) == sorted(absent)
    for shift in (2, 4):
        w = copy.copy(small_w)
        big = torch.empty(small_w.blob.numel() + 16, dtype=torch.uint8, device=DEV)
        w.blob = big[shift:shift + small_w.blob.numel()].view(small_w.blob.shape)
        w.blob.copy_(small_w.blob)
        check(oracle, w, n, k, seed=630 + n)


def test_token_kernel_agrees_with_the_two_launch_path(full_w):
    """Same routing bit for bit and the same layer to fp32 rounding as route + expert kernel, over
    repeated calls on one workspace (the grid barrier's counter carries over from call to call)."""
    k = 8
    for n in (1, 2, 3, 4):
        runner = MoeLayerRunner(4, full_w.hidden, full_w.n_ff, full_w.n_expert, k, DEV)
        for rep in range(3):
            x16 = synth.normal_fp16((n, full_w.hidden), 700 + 10 * n + rep, DEV)
            res = []
            for kernel in (None, "two_launch"):
                out32 = torch.zeros(n, full_w.hidden, dtype=torch.float32, device=DEV)
                x = x16.clone()
                a = runner.args(n, x16, full_w.router, full_w.table(), full_w.shared_ptrs(), x_f16=x, out_f32=out32)
                runner.run(a, kernel=kernel)
                torch.cuda.synchronize()
                res.append((out32.clone(), x.clone(), runner.route_idx.clone(), runner.route_w.clone()))
            assert torch.equal(res[0][2][:n], res[1][2][:n])
            assert torch.equal(res[0][3][:n], res[1][3][:n])
            assert rel(res[0][0].cpu().numpy(), res[1][0].cpu().numpy()) < 1e-5
    assert lib().raw("sgr_status")(0) == 0


@pytest.mark.parametrize("own_plan", [False, True])
@pytest.mark.parametrize("tokens", [8, 64])
def test_fused_exchange_entry_points_with_one_rank(full_w, tokens, own_plan):
    """The expert-parallel layer with the exchanges done by its own kernels, this device being its
    own only peer: the route kernel stores the records into the 'owner's' receive slot and sets the
    arrival word, the owner call waits for it and stores its rows into the 'home rank's' return
    slot, the home reduction waits for that word. Must reproduce the single call."""
    import ctypes as C
    from sager_b200.ep import record_layout
    from sager_b200.ops import stream_ptr
    w, k, H = full_w, 8, full_w.hidden
    x16 = synth.normal_fp16((tokens, H), 191, DEV)
    _, x_full, _ = run_layer(w, tokens, k, x16, n_max=64)
    rec, idx_off, w_off = record_layout(H, k, True)
    send = torch.zeros(tokens, rec, dtype=torch.uint8, device=DEV)
    recv = torch.zeros(tokens, rec, dtype=torch.uint8, device=DEV)
    back = torch.zeros(1, tokens, H, dtype=torch.float32, device=DEV)
    flags = torch.zeros(2, dtype=torch.int32, device=DEV)
    step = torch.full((1,), 5, dtype=torch.int32, device=DEV)
    p64 = lambda *addr: torch.tensor(list(addr), dtype=torch.int64, device=DEV)
    dst_recv, dst_back = p64(recv.data_ptr()), p64(back.data_ptr())
    fl_d, fl_r = p64(flags.data_ptr()), p64(flags.data_ptr() + 4)
    ptr = lambda t, off=0: C.c_void_p(t.data_ptr() + off)
    L, sp = lib(), stream_ptr()
    home = MoeLayerRunner(tokens, H, w.n_ff, w.n_expert, k, DEV)
    x = x16.clone()
    tab = w.table()                               # kept alive: the calls hold its device address only
    a = home.args(tokens, x16, w.router, tab, None, x_f16=x)
    a.xq_out, a.xq_stride, a.xq_padded = ptr(send), rec, 1
    a.route_idx, a.route_w, a.route_stride = ptr(send, idx_off), ptr(send, w_off), rec // 4
    a.ep_dst, a.ep_flags, a.ep_step = ptr(dst_recv), ptr(fl_d), ptr(step)
    a.ep_world, a.ep_rec_bytes, a.ep_mul, a.ep_add = 1, rec, 3, 2
    owner = MoeLayerRunner(64, H, w.n_ff, w.n_expert, k, DEV)
    if own_plan:
        # the owner call plans inside its expert kernel (stage bit 7, no plan launch); the home call's
        # route stage re-arms the owner workspace's counters
        a.rearm_workspace, a.rearm_mail_n, a.rearm_n_max = ptr(owner.ws), ptr(owner.mail_n), 64
    L.call("sgr_moe_layer_decode_stages", C.byref(a), 1 | 8, sp)
    b = owner.args(tokens, None, None, tab, w.shared_ptrs(), xq_in=recv, routing_given=True, no_residual=True)
    b.xq_stride, b.route_stride, b.xq_padded = rec, rec // 4, 1
    b.route_idx, b.route_w = ptr(recv, idx_off), ptr(recv, w_off)
    b.wait_flags, b.wait_step, b.wait_count, b.wait_mul, b.wait_add = ptr(flags), ptr(step), 1, 3, 2
    b.ep_out, b.ep_flags, b.ep_step = ptr(dst_back), ptr(fl_r), ptr(step)
    b.ep_world, b.ep_home_rows, b.ep_mul, b.ep_add = 1, tokens, 3, 2
    def issue():
        L.call("sgr_moe_layer_decode_stages", C.byref(a), 1 | 8, sp)
        L.call("sgr_moe_layer_decode_stages", C.byref(b), (6 | 16 | 128) if own_plan else (7 | 16), sp)
        L.call("sgr_ep_reduce_add_f16_wait", ptr(x), ptr(back), 1, tokens * H, tokens * H, ptr(flags, 4), ptr(step), 3, 2, sp)
    L.call("sgr_moe_layer_decode_stages", C.byref(b), (6 | 16 | 128) if own_plan else (7 | 16), sp)
    L.call("sgr_ep_reduce_add_f16_wait", ptr(x), ptr(back), 1, tokens * H, tokens * H, ptr(flags, 4), ptr(step), 3, 2, sp)
    torch.cuda.synchronize()
    assert flags.tolist() == [17, 17]
    if own_plan:                                  # a second layer on the same workspaces: the re-armed counters hold
        x_once = x.clone()
        x.copy_(x16)
        step.fill_(6)
        issue()
        torch.cuda.synchronize()
        assert flags.tolist() == [20, 20]
        assert torch.equal(x, x_once)
    assert torch.equal(recv, send)
    assert rel(x.float().cpu().numpy(), x_full.float().cpu().numpy()) <= 2.0 ** -10      # fp16 store after another add order
    assert lib().raw("sgr_status")(0) == 0
