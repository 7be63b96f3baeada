"""GPU check of sgr_moe_layer_decode_static, the entry point for callers that
cannot allocate device memory (an engine that handed out all of its VRAM at
start-up, a binding that cannot own CUDA buffers): the library's built-in
scratch array stands in for the caller's workspace. Called through the C ABI,
two calls in a row on different inputs, and compared with sgr_moe_layer_decode
on a caller-allocated workspace; the second call also proves that nothing left
in the shared array by the first one leaks into the result. This file sorts
last on purpose, so a run that stops at the first failure has run every other
test before it."""
import ctypes as C

import numpy as np
import pytest
import torch

from sager_b200 import lib, synth
from sager_b200.layer import MoeLayerRunner
from sager_b200.ops import stream_ptr
from tests.util import DEV, LAYER_TOL, rel

pytestmark = pytest.mark.gpu


def _run_both(w, runner, n, k, seed):
    x16 = synth.normal_fp16((n, w.hidden), seed, DEV)
    outs = []
    for name in ("sgr_moe_layer_decode", "sgr_moe_layer_decode_static"):
        x = x16.clone()
        out32 = torch.zeros(n, w.hidden, dtype=torch.float32, device=DEV)
        idx = torch.full((runner.n_max, k + 1), -3, dtype=torch.int32, device=DEV)
        wts = torch.zeros(runner.n_max, k + 1, dtype=torch.float32, device=DEV)
        a = runner.args(n, x16, w.router, w.table(), w.shared_ptrs(), x_f16=x, out_f32=out32,
                        route_idx=idx, route_w=wts)
        if name.endswith("_static"):
            a.workspace, a.workspace_bytes = None, 0          # ignored by the static entry point
        lib().call(name, C.byref(a), stream_ptr())
        torch.cuda.synchronize()
        outs.append((out32.cpu().numpy(), x.cpu().numpy(), idx.cpu().numpy()[:n, :k], wts.cpu().numpy()[:n]))
    return outs


def test_static_scratch_entry_point_matches_workspace_entry_point():
    hidden, n_ff, n_expert, k = 512, 256, 16, 4
    w = synth.MoeWeights(hidden, n_ff, n_expert, DEV, seed=31, std=0.05)
    runner = MoeLayerRunner(8, hidden, n_ff, n_expert, k, DEV)
    for n, seed in ((3, 41), (8, 42)):                 # two calls in a row, second with more rows
        (o_ws, x_ws, i_ws, w_ws), (o_st, x_st, i_st, w_st) = _run_both(w, runner, n, k, seed)
        assert np.array_equal(i_ws, i_st)
        assert np.abs(w_ws - w_st).max() <= 1e-6
        assert rel(o_st, o_ws) < LAYER_TOL and rel(o_st, o_ws) <= 1e-6
        assert np.array_equal(x_ws.view(np.uint16), x_st.view(np.uint16))
    assert lib().raw("sgr_status")(0) == 0


@pytest.mark.parametrize("n", [1, 4, 8])
def test_static_scratch_at_the_decode_geometry_against_the_oracle(oracle, n):
    """The use the entry point is documented for - hidden 2048, expert FFN 512, 256 experts, top-8, a
    handful of token rows - against the CPU expert path, two calls in a row. At n = 4 and 8 a call
    on a workspace runs the row-streaming expert kernel; the static call must make the same choice
    (the whole layout fits the array) and give the same result."""
    from tests.test_gpu_moe_layer import oracle_layer
    hidden, n_ff, n_expert, k = 2048, 512, 256, 8
    w = synth.MoeWeights(hidden, n_ff, n_expert, DEV, seed=20260718)
    runner = MoeLayerRunner(8, hidden, n_ff, n_expert, k, DEV)
    assert lib().raw("sgr_moe_layer_workspace_bytes")(8, hidden, n_ff, n_expert, k) <= \
        lib().raw("sgr_moe_layer_static_limit")()
    blob_np = w.blob.cpu().numpy()
    for seed in (61 + n, 71 + n):
        (o_ws, x_ws, i_ws, w_ws), (o_st, x_st, i_st, w_st) = _run_both(w, runner, n, k, seed)
        x_np = synth.normal_fp16((n, hidden), seed, DEV).cpu().numpy()
        want = oracle_layer(oracle, w, x_np, x_np.astype(np.float32), k, blob_np=blob_np)
        assert np.array_equal(i_st, want["idx"][:, :k]) and np.array_equal(i_st, i_ws)
        err = rel(o_st, want["out"])
        print(f"static entry, {n} rows: max relative error vs the CPU path {err:.2e}")
        assert err <= LAYER_TOL
        assert np.array_equal(o_st, o_ws)              # same kernels, same arithmetic as the workspace call
    assert lib().raw("sgr_status")(0) == 0


def test_static_scratch_refuses_shapes_beyond_its_limit():
    limit = lib().raw("sgr_moe_layer_static_limit")()
    assert limit == 2 << 20
    assert lib().raw("sgr_moe_layer_workspace_bytes")(24, 2048, 512, 256, 8) > limit     # 24 rows: refused too
    need = lib().raw("sgr_moe_layer_workspace_bytes")(64, 2048, 512, 256, 8)
    assert need > limit
    w = synth.MoeWeights(2048, 512, 4, DEV, seed=5)        # few experts: cheap to make
    k, n = 2, 4
    x16 = synth.normal_fp16((n, 2048), 6, DEV)
    out32 = torch.full((n, 2048), 7.0, dtype=torch.float32, device=DEV)
    idx = torch.zeros(64, k + 1, dtype=torch.int32, device=DEV)
    wts = torch.zeros(64, k + 1, dtype=torch.float32, device=DEV)
    from sager_b200.capi import MoeLayerArgs
    a = MoeLayerArgs()
    a.n, a.n_max, a.hidden, a.n_ff, a.n_expert, a.n_used = n, 64, 2048, 512, 256, 8
    a.xn = C.c_void_p(x16.data_ptr())
    a.router_w = C.c_void_p(w.router.data_ptr())
    a.w_tab = C.c_void_p(w.table().data_ptr())
    a.out_f32 = C.c_void_p(out32.data_ptr())
    a.route_idx, a.route_w = C.c_void_p(idx.data_ptr()), C.c_void_p(wts.data_ptr())
    rc = lib().raw("sgr_moe_layer_decode_static")(C.byref(a), stream_ptr())
    torch.cuda.synchronize()
    assert rc == 6                                          # SGR_ESTATICLIMIT, nothing launched
    assert torch.all(out32 == 7.0)
