"""Bounded device-side waits that run out. The expert-parallel kernels wait for arrival words that
a peer rank sets over NVLink; when a peer never posts, the wait must end with an error status that
the host can read, the context must stay usable and the next call must be clean. The failure is
made on the host (a word that nothing sets) with a short poll limit; no GPU fault, trap or hang is
involved. Reference analogue: every wait of the expert pump is bounded
(tests/test_expert_pump.cpp:162-180, "lookup times out instead of hanging")."""
import ctypes as C

import pytest
import torch

from sager_b200 import lib, ops, synth
from sager_b200.layer import MoeLayerRunner
from sager_b200.ops import stream_ptr
from tests.util import DEV

pytestmark = pytest.mark.gpu

SHORT = 2000            # polls, 64 ns apart: well under a millisecond
DEFAULT = 1 << 22


def _p(t):
    return C.c_void_p(t.data_ptr())


@pytest.fixture
def short_waits():
    L = lib()
    assert L.raw("sgr_status")(1) in (0, 8)
    L.call("sgr_ep_set_wait_limit", SHORT)
    yield L
    L.call("sgr_ep_set_wait_limit", DEFAULT)
    L.raw("sgr_status")(1)


def test_home_reduction_gives_up_when_an_owner_never_posts(short_waits):
    L, sp = short_waits, stream_ptr()
    x = torch.ones(4096, dtype=torch.float16, device=DEV)
    parts = torch.full((2, 4096), 0.5, dtype=torch.float32, device=DEV)
    flags = torch.zeros(2, dtype=torch.int32, device=DEV)
    flags[0] = 7                                     # owner 0 posted step 1 of (mul 5, add 2); owner 1 never does
    step = torch.ones(1, dtype=torch.int32, device=DEV)
    L.call("sgr_ep_reduce_add_f16_wait", _p(x), _p(parts), 2, 4096, 4096, _p(flags), _p(step), 5, 2, sp)
    torch.cuda.synchronize()                         # returns: the kernel gave up instead of spinning
    assert L.raw("sgr_status")(0) == 8
    assert torch.all(x == 1.0)                       # nothing was added from the part that never arrived
    assert L.raw("sgr_status")(1) == 8               # read and clear
    flags[1] = 7
    L.call("sgr_ep_reduce_add_f16_wait", _p(x), _p(parts), 2, 4096, 4096, _p(flags), _p(step), 5, 2, sp)
    torch.cuda.synchronize()
    assert L.raw("sgr_status")(0) == 0 and torch.all(x == 2.0)


def test_owner_plan_gives_up_when_a_home_rank_never_dispatches(short_waits):
    L, sp = short_waits, stream_ptr()
    hidden, n_ff, E, k, n = 512, 256, 16, 4, 8
    w = synth.MoeWeights(hidden, n_ff, E, DEV, seed=3, std=0.05)
    x16 = synth.normal_fp16((n, hidden), 4, DEV)
    home = MoeLayerRunner(n, hidden, n_ff, E, k, DEV)
    out_ref = torch.zeros(n, hidden, dtype=torch.float32, device=DEV)
    home.run(home.args(n, x16, w.router, w.table(), w.shared_ptrs(), out_f32=out_ref, no_residual=True))
    xq = torch.zeros(n, hidden // 256 * 276, dtype=torch.uint8, device=DEV)
    ops.quantize_q8_k(x16, xq, n * hidden)
    owner = MoeLayerRunner(n, hidden, n_ff, E, k, DEV)
    out = torch.zeros(n, hidden, dtype=torch.float32, device=DEV)
    flags = torch.zeros(2, dtype=torch.int32, device=DEV)
    step = torch.ones(1, dtype=torch.int32, device=DEV)
    a = owner.args(n, None, None, w.table(), w.shared_ptrs(), out_f32=out, xq_in=xq, routing_given=True,
                   no_residual=True, route_idx=home.route_idx, route_w=home.route_w)
    a.wait_flags, a.wait_step = _p(flags), _p(step)
    a.wait_count, a.wait_mul, a.wait_add = 2, 1, 0
    owner.run(a)                                     # both words stay 0 < 1: the plan's wait runs out
    torch.cuda.synchronize()
    assert L.raw("sgr_status")(1) == 8
    flags.fill_(1)                                   # the records "arrive": the same call is clean and right
    owner.run(a)
    torch.cuda.synchronize()
    assert L.raw("sgr_status")(0) == 0
    assert torch.allclose(out, out_ref, rtol=0, atol=1e-6 * float(out_ref.abs().max()))
