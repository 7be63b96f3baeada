"""TEST INFRASTRUCTURE, not part of the product: the reference's own CUDA launchers
(oracle/_ref/libsager_ref_cuda.so, built by oracle/Makefile from the reference's
src/kernels/cuda/{q4_k,mmq,moe,norm_rotary,sampling}.cu for sm_100a) on torch tensors, and the
launch sequence of the reference's device MoE path written over a launcher set, so
that the same sequence runs on the reference's kernels and on this library's.

Only tests/ and bench.py's reference legs import this.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libsager_ref_cuda.so")


def available() -> bool:
    return os.path.exists(LIB_PATH)


class Launchers:
    """`<obj>.<name>(...)` calls `sgr_<name>` of a shared library that exports the C
    names of include/sager_b200.h, tensors passed as device pointers, torch's current
    stream appended - the calling convention of sager_b200.ops."""

    def __init__(self, path: str, protos: dict):
        self.cdll = C.CDLL(path)
        self.names = set()
        for name, (res, args) in protos.items():
            try:
                fn = getattr(self.cdll, name)
            except AttributeError:
                continue
            fn.restype, fn.argtypes = res, args
            self.names.add(name)

    @staticmethod
    def _conv(a):
        if a is None:
            return None
        if isinstance(a, torch.Tensor):
            return C.c_void_p(a.data_ptr())
        if isinstance(a, int) and a > 0x7FFFFFFF:
            return C.c_void_p(a)
        return a

    def __getattr__(self, name):
        if name.startswith("_") or "sgr_" + name not in self.names:
            raise AttributeError(name)
        fn = getattr(self.cdll, "sgr_" + name)

        def call(*args):
            rc = fn(*[self._conv(a) for a in args], C.c_void_p(torch.cuda.current_stream().cuda_stream))
            if rc != 0:
                raise RuntimeError(f"{name} returned {rc}")
        return call


def reference_launchers() -> Launchers:
    from sager_b200.capi import parse_header
    return Launchers(LIB_PATH, parse_header())


def library_launchers() -> Launchers:
    from sager_b200.capi import LIB_PATH as mine, parse_header
    return Launchers(mine, parse_header())


class DeviceMoePath:
    """The MoE half of a layer as `Session::moe_dispatch_device` launches it for a
    batch of token rows on the dp4a path (src/core/session.cpp:2482-3030 with
    SAGER_MOE_TC=0; buffers of src/core/session.cpp:207-257): quantise, router GEMV,
    batched top-k, device plan, gather, grouped gate/up GEMV, SwiGLU, requantise,
    grouped down GEMV, scatter, shared expert, combine - 15 launches."""

    def __init__(self, o: Launchers, n_max, hidden, n_ff, n_expert, n_used, device, tok_per=None):
        self.o = o
        if tok_per is None:          # the session's tile choice (src/core/session.cpp:2579-2584)
            hb = hidden // 256
            t = (49152 - 16 * hb * 144 - 512) // (hb * 276)
            tok_per = 4 if t < 4 else (16 if t > 16 else t)
        self.n_max, self.H, self.F, self.E, self.K, self.tok_per = n_max, hidden, n_ff, n_expert, n_used, tok_per
        d, u8, f16, i32, f32 = device, torch.uint8, torch.float16, torch.int32, torch.float32
        R = n_max * n_used
        self.R = R
        self.tiles_max = min(R // tok_per + n_expert + 16, R)       # src/core/session.cpp:2785-2786
        self.xq = torch.empty(n_max, hidden // 256 * 276, dtype=u8, device=d)
        self.logits = torch.empty(n_max, n_expert, dtype=f32, device=d)
        self.idx = torch.zeros(n_max, n_used + 1, dtype=i32, device=d)
        self.w = torch.zeros(n_max, n_used + 1, dtype=f32, device=d)
        self.gslot = torch.zeros(R, dtype=i32, device=d)
        self.grows = torch.zeros(R, dtype=i32, device=d)
        self.off = torch.zeros(n_expert + 1, dtype=i32, device=d)
        self.toff = torch.zeros(n_expert + 1, dtype=i32, device=d)
        self.meta = torch.zeros(4, dtype=i32, device=d)
        self.mail = torch.zeros(n_expert, dtype=i32, device=d)
        self.mail_n = torch.zeros(1, dtype=i32, device=d)
        self.xqg = torch.empty(R, hidden // 256 * 276, dtype=u8, device=d)
        self.g = torch.empty(R, n_ff, dtype=f16, device=d)
        self.u = torch.empty(R, n_ff, dtype=f16, device=d)
        self.hq = torch.empty(R, n_ff // 256 * 276, dtype=u8, device=d)
        self.yg = torch.empty(R, hidden, dtype=f16, device=d)
        self.expert_y = torch.zeros(n_max, n_used + 1, hidden, dtype=f16, device=d)
        self.sh_g = torch.empty(n_max, n_ff, dtype=f16, device=d)
        self.sh_u = torch.empty(n_max, n_ff, dtype=f16, device=d)
        self.sh_q = torch.empty(n_max, n_ff // 256 * 276, dtype=u8, device=d)
        self.sh_y = torch.empty(n_max, hidden, dtype=f16, device=d)

    def run(self, n, xn, x, router, table, shared_ptrs, bias=None, logits=None):
        """xn [n][H] fp16 layer input, x [n][H] fp16 residual (combined in place);
        table = the [3][E] pointer-table slices, shared_ptrs = (gate, up, down); bias [E]
        fp32 is added to the logits (the benchmark's routing skew; one more launch); `logits`
        replaces the router GEMV."""
        o, H, F, E, K = self.o, self.H, self.F, self.E, self.K
        o.quantize_q8_k(xn, self.xq, n * H)
        if logits is None:
            o.gemv_f32_out_f16x_mtok(router, xn, self.logits, E, H, n)
        else:                        # the prefill benchmark draws the logits directly
            self.logits[:n].copy_(logits)
        if bias is not None:
            self.logits[:n].add_(bias)
        o.router_topk_batched(self.logits, self.idx, self.w, E, K, K + 1, n, 1.0)
        o.moe_dispatch_scan(self.idx, self.w, self.gslot, self.grows, self.off, self.toff, self.meta,
                            self.mail, self.mail_n, n, K, E, self.tok_per)
        o.gather_rows_q8_n(self.xqg, self.xq, self.grows, self.meta, n * K, H // 256)
        o.gemv_grouped2_tab_q4_k_q8_f16out_mtok(table[0], table[1], self.off, self.toff, self.meta, self.mail,
                                                self.mail_n, self.tiles_max, self.xqg, self.g, self.u,
                                                F, H, E, self.tok_per)
        o.silu_mul_f16_n(self.g, self.g, self.u, self.meta, n * K, F)
        o.quantize_q8_k_n(self.g, self.hq, self.meta, F, n * K * (F // 256))
        o.gemv_grouped_tab_q4_k_q8_f16out_mtok(table[2], self.off, self.toff, self.meta, self.tiles_max,
                                               self.hq, self.yg, H, F, E, self.tok_per)
        o.scatter_routed_f16(self.expert_y, self.yg, self.gslot, n, K, H)
        sg, su, sd = shared_ptrs
        o.gemv2_q4_k_q8_f16out_mtok(sg, su, self.xq, self.sh_g, self.sh_u, F, H, n)
        o.silu_mul_f16(self.sh_g, self.sh_g, self.sh_u, n, F)
        o.quantize_q8_k(self.sh_g, self.sh_q, n * F)
        o.gemv_q4_k_q8_f16out_mtok(sd, self.sh_q, self.sh_y, H, F, n)
        # slot K of the combine slab = the shared expert's rows (one strided device copy)
        self.expert_y[:n, K, :].copy_(self.sh_y[:n])
        o.moe_combine_batched_f16(x, self.expert_y, self.w, K, H, n)

    launches = 15
