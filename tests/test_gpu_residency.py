"""The residency handle on the device: experts copied from a pinned host pool into a device slab and
arena, the [3][L][E] decode table uploaded, and the fused layer reading that table in place
(tab_stride = L * E) - against the same layer on a table built directly from the weights. Absent
experts go through the arena (submit, wait on the compute stream, table rebuilt) as the session's
miss path does (src/core/session.cpp:1880-1900 of the reference)."""
import numpy as np
import pytest
import torch

from sager_b200 import lib, synth
from sager_b200.layer import MoeLayerRunner
from sager_b200.residency import Residency
from tests.util import DEV

pytestmark = pytest.mark.gpu


def test_layers_run_from_the_residency_table():
    H, F, E, K, Lm = 512, 256, 16, 4, 3
    layers = [synth.MoeWeights(H, F, E, DEV, seed=40 + l, std=0.05) for l in range(Lm)]
    eb = layers[0].expert_bytes
    pool = torch.empty(Lm * E * eb, dtype=torch.uint8).pin_memory()
    for l, w in enumerate(layers):
        pool[l * E * eb:(l + 1) * E * eb] = w.blob[:E].reshape(-1).cpu()
    r = Residency(Lm, E, H, F, slab_experts=Lm * E - 4, arena_slots=3)
    assert r.expert_bytes == eb
    slab = torch.zeros((Lm * E - 4) * eb, dtype=torch.uint8, device=DEV)
    arena = torch.zeros(3 * eb, dtype=torch.uint8, device=DEV)
    table = torch.zeros(3, Lm, E, dtype=torch.int64, device=DEV)
    copy_stream = torch.cuda.Stream()
    r.bind(pool, slab, arena, table, copy_stream=copy_stream.cuda_stream)
    missing = {(0, 2), (1, 5), (1, 9), (2, 0)}
    for l in range(Lm):
        for e in range(E):
            if (l, e) not in missing:
                r.set_resident(l, e)
    cur = torch.cuda.current_stream().cuda_stream
    assert r.rebuild(cur) == Lm * E - 4
    assert r.build_decode_table(cur) == 4 and [r.absent(l) for l in range(Lm)] == [1, 2, 1]
    n = 6
    x16 = synth.normal_fp16((n, H), 77, DEV)

    def run(l, tab, stride, mail=False):
        runner = MoeLayerRunner(8, H, F, E, K, DEV)
        out = torch.zeros(n, H, dtype=torch.float32, device=DEV)
        a = runner.args(n, x16, layers[l].router, tab, layers[l].shared_ptrs(), out_f32=out)
        a.tab_stride = stride
        runner.run(a)
        torch.cuda.synchronize()
        nm = int(runner.mail_n.item())
        return out, sorted(set(runner.mail.cpu().numpy()[:nm].tolist()))

    for l in range(Lm):
        absent = tuple(e for (ll, e) in missing if ll == l)
        want, _ = run(l, layers[l].table(absent), 0)
        got, mailed = run(l, table[0, l], Lm * E)
        assert torch.equal(got, want)
        routed = set(mailed)
        assert routed <= set(absent)                   # only absent experts are mailed, and only if routed to
    # the miss path: bring the absent experts of layer 1 into the arena, wait, rebuild the table
    for e in (5, 9):
        slot = r.submit(1, e, step=1)
        assert slot >= 0
        r.wait(slot, cur)
    assert r.build_decode_table(cur) == 2
    full, _ = run(1, layers[1].table(), 0)
    got, mailed = run(1, table[0, 1], Lm * E)
    assert torch.equal(got, full) and mailed == []
    assert lib().raw("sgr_status")(0) == 0
    r.close()
