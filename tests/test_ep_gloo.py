"""CPU (gloo, world size 2) check of the expert-parallel exchange logic: token
records out by all-to-all, partial sums back by all-to-all, residual add at home.
The expert arithmetic on each rank is the oracle's (this is test code), so the
result can be compared with the oracle's single-rank layer."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.oracle import Oracle
    from sager_b200.ep import EpExchange
    g = dict(np.load(os.path.join(ROOT, "tests", "golden", "ref_cpu_golden.npz")))
    o = Oracle()
    H, F, E, K, tokens = 512, 256, 4, 2, 4
    n_home = tokens // world
    rng = np.random.default_rng(77)                       # same data on every rank
    router = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    x16 = rng.standard_normal((tokens, H)).astype(np.float16)
    ex_w = (g["ffn_wg"], g["ffn_wu"], g["ffn_wd"])
    experts = [ex_w] * E
    ex = EpExchange(world, rank, n_home, H, K, "cpu")
    # home: quantise + route into the records of slot 0
    h0 = rank * n_home
    send = ex.send.numpy()
    for t in range(n_home):
        row = x16[h0 + t]
        send[0, t, :ex.idx_off] = o.quantize_q8k_f16(row[None])[0]
        idx, w = o.router_topk(o.router_logits(router, row), K, shared_w=1.0)
        send[0, t, ex.idx_off:ex.idx_off + (K + 1) * 4] = idx.view(np.uint8)
        send[0, t, ex.w_off:ex.w_off + (K + 1) * 4] = w.view(np.uint8)
    ex.dispatch()
    recv = ex.recv.numpy().reshape(tokens, ex.rec)
    # owner: local experts over every received row; shared expert only for the home rows
    lo, hi = rank * (E // world), (rank + 1) * (E // world)
    part = ex.part.numpy().reshape(tokens, H)
    part[:] = 0
    for t in range(tokens):
        idx = recv[t, ex.idx_off:ex.idx_off + (K + 1) * 4].copy().view(np.int32)
        w = recv[t, ex.w_off:ex.w_off + (K + 1) * 4].copy().view(np.float32)
        xf = x16[t].astype(np.float32)                      # the oracle's FFN re-quantises from fp32
        assert np.array_equal(recv[t, :ex.idx_off], o.quantize_q8k_f16(x16[t][None])[0])
        for kk in range(K):
            if lo <= idx[kk] < hi:
                part[t] += w[kk] * o.expert_ffn(*experts[idx[kk]], xf, H, F)
        if h0 <= t < h0 + n_home:
            part[t] += w[K] * o.expert_ffn(*ex_w, xf, H, F)
    ex.combine()
    back = ex.back.numpy()
    out = x16[h0:h0 + n_home].astype(np.float32)
    for p in range(world):
        out = out + back[p]
    np.save(os.path.join(out_dir, f"out{rank}.npy"), out)
    dist.destroy_process_group()


def test_two_rank_exchange_reproduces_single_rank_layer(tmp_path, oracle, golden):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    H, F, E, K, tokens = 512, 256, 4, 2, 4
    rng = np.random.default_rng(77)
    router = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    x16 = rng.standard_normal((tokens, H)).astype(np.float16)
    ex_w = (golden["ffn_wg"], golden["ffn_wu"], golden["ffn_wd"])
    want = oracle.moe_layer(x16, router, [ex_w] * E, ex_w, x16.astype(np.float32), K, F)["out"]
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-6


def _silent_peer_worker(rank, world, port, out_dir):
    """Rank 1 joins the group and then never posts its side of the dispatch; rank 0 must get an
    error within its time limit instead of waiting for ever."""
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sager_b200.ep import EpExchange, ExchangeTimeout
    ex = EpExchange(world, rank, 2, 512, 2, "cpu", timeout_s=2.0)
    dist.barrier()
    if rank == 1:
        time.sleep(8.0)                       # alive, but takes no part in the exchange
        os._exit(0)
    t0 = time.time()
    try:
        ex.dispatch()
        result = "completed"
    except ExchangeTimeout as exc:
        result = f"timeout after {time.time() - t0:.1f} s: {exc}"
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(result)
    os._exit(0)                               # the group is aborted: no orderly shutdown to wait for


def test_a_rank_that_never_posts_becomes_an_error_not_a_hang(tmp_path):
    world = 2
    ctx = mp.spawn(_silent_peer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=False)
    import time
    deadline = time.time() + 60
    while not ctx.join(timeout=1.0):
        assert time.time() < deadline, "the ranks are still running: the wait was not bounded"
    text = (tmp_path / "rank0.txt").read_text()
    assert text.startswith("timeout after"), text
    assert float(text.split()[2]) < 6.0
