"""Seeded synthetic inputs for the MoE path (weights, router, activations).

The reference's benchmarks run a private checkpoint; everything here is
synthetic and stands for nothing external. Shapes and distributions follow the
benchmark configurations: activations N(0,1) rounded to fp16, router
[E][H] fp32 N(0,0.02), expert matrices N(0,0.02) quantised to Q4_K, optional
Zipf(s=1.1) bias on the router logits.

`quantize_q4k` is a vectorised torch quantiser that emits valid Q4_K bytes
(layout of include/sager/kernels/q4_k.hpp:45-52 in the reference): per
sub-block the scale and min are anchored on the sub-block's range instead of
searched, which is enough for inputs whose only job is to be consumed
identically by the CUDA kernels and the CPU oracle.
"""
from __future__ import annotations

import math

import numpy as np
import torch

QK_K = 256
Q4K_BYTES = 144
Q8K_BYTES = 276


def quantize_q4k(w: torch.Tensor) -> torch.Tensor:
    """fp32 [rows, k] -> uint8 [rows, k/256*144] on w's device."""
    rows, k = w.shape
    assert k % QK_K == 0
    nb = rows * k // QK_K
    x = w.reshape(nb, 8, 32).float()
    mn = x.amin(dim=2)
    mx = x.amax(dim=2)
    rng = (mx - mn)
    d = (rng.amax(dim=1, keepdim=True) / 63.0).clamp_min(1e-30)
    d16 = d.half()
    df = d16.float().clamp_min(6e-8)                       # what the kernels will read back
    sc = torch.clamp(torch.round(rng / 15.0 / df), 1, 63)   # [nb, 8]
    mi = torch.clamp(torch.round(-mn / df), 0, 63)
    q = torch.clamp(torch.round((x + (df * mi).unsqueeze(2)) / (df * sc).unsqueeze(2)), 0, 15)
    q = q.to(torch.uint8)
    qs = (q[:, 0::2, :] & 0xF) | (q[:, 1::2, :] << 4)       # [nb, 4, 32]: low = even sub-block
    sc = sc.to(torch.uint8)
    mi = mi.to(torch.uint8)
    scales = torch.zeros(nb, 12, dtype=torch.uint8, device=w.device)
    scales[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    scales[:, 4:8] = (mi[:, 0:4] & 63) | ((mi[:, 4:8] >> 4) << 6)
    scales[:, 8:12] = (sc[:, 4:8] & 0xF) | ((mi[:, 4:8] & 0xF) << 4)
    out = torch.empty(nb, Q4K_BYTES, dtype=torch.uint8, device=w.device)
    d_bytes = d16.view(torch.uint8).reshape(nb, 2)
    out[:, 0:2] = d_bytes
    out[:, 2:4] = d_bytes                                    # dmin = d
    out[:, 4:16] = scales
    out[:, 16:] = qs.reshape(nb, 128)
    return out.reshape(rows, k // QK_K * Q4K_BYTES)


def normal_fp16(shape, seed, device, std=1.0) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).half().to(device)


class MoeWeights:
    """One layer's weights: router [E][H] fp32 and a blob of E+1 experts, each
    [gate | up | down] contiguous (expert E is the always-on shared expert)."""

    def __init__(self, hidden, n_ff, n_expert, device, seed, std=0.02, distinct=None,
                 expert_range=None):
        """expert_range=(lo, hi): keep only the routed experts lo..hi-1 (and the shared
        expert) - one rank's shard under expert parallelism. The bytes of an expert
        are the same whichever shard holds it."""
        self.hidden, self.n_ff, self.n_expert = hidden, n_ff, n_expert
        self.lo, self.hi = (0, n_expert) if expert_range is None else expert_range
        self.gu_bytes = n_ff * (hidden // QK_K) * Q4K_BYTES
        self.dn_bytes = hidden * (n_ff // QK_K) * Q4K_BYTES
        self.expert_bytes = 2 * self.gu_bytes + self.dn_bytes
        g = torch.Generator(device=device).manual_seed(seed)
        self.router = (torch.randn(n_expert, hidden, generator=g, device=device) * std).float()
        n_all = n_expert + 1
        n_make = n_all if distinct is None else min(distinct, n_all)
        # blob slot of expert e: e - lo for local routed experts, (hi - lo) for the shared one
        self.n_slots = self.hi - self.lo + 1
        self.blob = torch.empty(self.n_slots, self.expert_bytes, dtype=torch.uint8, device=device)
        step = 32
        for e0 in range(0, n_make, step):
            e1 = min(n_make, e0 + step)
            wg = torch.randn((e1 - e0) * 2 * n_ff, hidden, generator=g, device=device) * std
            wd = torch.randn((e1 - e0) * hidden, n_ff, generator=g, device=device) * std
            keep = [e for e in range(e0, e1) if self.slot(e) is not None]
            if not keep:
                continue                      # same generator stream, another rank's experts
            qg = quantize_q4k(wg).reshape(e1 - e0, 2 * self.gu_bytes)
            qd = quantize_q4k(wd).reshape(e1 - e0, self.dn_bytes)
            for e in keep:
                self.blob[self.slot(e), :2 * self.gu_bytes] = qg[e - e0]
                self.blob[self.slot(e), 2 * self.gu_bytes:] = qd[e - e0]
        # remaining experts reuse the made ones' bytes at their own addresses
        # (distinct HBM lines; the arithmetic cost is the same)
        for e in range(n_make, n_all):
            if self.slot(e) is not None and self.slot(e % n_make) is not None:
                self.blob[self.slot(e)] = self.blob[self.slot(e % n_make)]

    def slot(self, e):
        if e == self.n_expert:
            return self.hi - self.lo
        return e - self.lo if self.lo <= e < self.hi else None

    def matrix(self, e, m):
        """uint8 view of matrix m (0 gate, 1 up, 2 down) of expert e."""
        o = [0, self.gu_bytes, 2 * self.gu_bytes, self.expert_bytes]
        return self.blob[self.slot(e), o[m]:o[m + 1]]

    def table(self, absent=()):
        """int64 [3][E] device pointer table; experts outside this shard and `absent`
        ones get null entries."""
        # Callers hand the table to the library by its device address only, so the tensor must outlive
        # every launch that reads it: tables are kept with the weights (one per set of absent experts).
        key = tuple(sorted(absent))
        cache = self.__dict__.setdefault("_tables", {})
        if key in cache:
            return cache[key]
        base = self.blob.data_ptr()
        t = torch.zeros(3, self.n_expert, dtype=torch.int64)
        o = [0, self.gu_bytes, 2 * self.gu_bytes]
        for m in range(3):
            t[m, self.lo:self.hi] = base + torch.arange(self.hi - self.lo, dtype=torch.int64) * self.expert_bytes + o[m]
        for e in absent:
            t[:, e] = 0
        cache[key] = t.to(self.blob.device)
        return cache[key]

    def shared_ptrs(self):
        base = self.blob.data_ptr() + (self.hi - self.lo) * self.expert_bytes
        return [base, base + self.gu_bytes, base + 2 * self.gu_bytes]


def zipf_bias(n_expert, seed, alpha, s=1.1) -> np.ndarray:
    """bias[e] = alpha * ln(rank(e)^-s) for a seeded random ranking of the experts."""
    rng = np.random.default_rng(seed)
    rank = rng.permutation(n_expert) + 1
    return (alpha * (-s) * np.log(rank)).astype(np.float32)


def hot_share(idx: np.ndarray, n_expert, frac=0.2) -> float:
    """Share of routed picks that go to the `frac` most-picked experts."""
    cnt = np.bincount(idx.reshape(-1), minlength=n_expert)
    top = np.sort(cnt)[::-1][: max(1, int(math.ceil(frac * n_expert)))]
    return float(top.sum() / max(1, cnt.sum()))
