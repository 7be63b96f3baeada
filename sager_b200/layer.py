"""Host-side driver of the fused MoE layer (the part of the reference's
`Session` that owns the MoE scratch buffers and walks the layers,
src/core/session.cpp:207-257 and 2482-3030), on torch device memory.

`MoeLayerRunner` owns the workspace and the routing buffers of one stream of
decode steps and issues `sgr_moe_layer_decode` per layer; `MoeStack` holds the
weights of several layers and replays a whole step from a CUDA graph.
All arithmetic happens in the library.
"""
from __future__ import annotations

import ctypes as C

import torch

from .capi import MoeLayerArgs, MoePrefillArgs, lib
from .ops import stream_ptr


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


# None = the library's choice (one persistent launch for up to three rows, else route + the expert kernel
# picked by row count); "two_launch" = route + expert kernel by row count; "rows" / "items" force one of them
KERNEL_BITS = {None: 0, "rows": 16, "items": 32, "two_launch": 64}


class MoeLayerRunner:
    def __init__(self, n_max, hidden, n_ff, n_expert, n_used, device, expert_lo=0, expert_hi=0):
        self.n_max, self.hidden, self.n_ff = n_max, hidden, n_ff
        self.n_expert, self.n_used = n_expert, n_used
        self.expert_lo, self.expert_hi = expert_lo, expert_hi
        self.device = device
        L = lib()
        nbytes = L.raw("sgr_moe_layer_workspace_bytes")(n_max, hidden, n_ff, n_expert, n_used)
        if nbytes == 0:
            raise ValueError("geometry refused by sgr_moe_layer_workspace_bytes")
        self.ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        assert self.ws.data_ptr() % 256 == 0
        with torch.cuda.device(device):
            L.call("sgr_moe_layer_workspace_init", _p(self.ws), nbytes, stream_ptr())
        self.route_idx = torch.zeros(n_max, n_used + 1, dtype=torch.int32, device=device)
        self.route_w = torch.zeros(n_max, n_used + 1, dtype=torch.float32, device=device)
        self.mail = torch.zeros(n_expert, dtype=torch.int32, device=device)
        self.mail_n = torch.zeros(1, dtype=torch.int32, device=device)

    def args(self, n, xn, router_w, w_tab, shared_ptrs, x_f16=None, out_f32=None, bias=None,
             shared_w=1.0, xq_in=None, routing_given=False, no_residual=False, shared_lo=0,
             shared_hi=0, route_idx=None, route_w=None):
        a = MoeLayerArgs()
        a.n, a.n_max = n, self.n_max
        a.hidden, a.n_ff, a.n_expert, a.n_used = self.hidden, self.n_ff, self.n_expert, self.n_used
        a.expert_lo, a.expert_hi = self.expert_lo, self.expert_hi
        a.shared_lo, a.shared_hi = shared_lo, shared_hi
        a.routing_given, a.no_residual = int(routing_given), int(no_residual)
        a.shared_w = shared_w
        a.xn, a.xq_in = _p(xn), _p(xq_in)
        a.router_w, a.router_bias = _p(router_w), _p(bias)
        a.w_tab = _p(w_tab)
        sh = shared_ptrs or [None, None, None]
        a.shared_gate, a.shared_up, a.shared_down = sh[0], sh[1], sh[2]
        a.x_f16, a.out_f32 = _p(x_f16), _p(out_f32)
        a.route_idx = _p(self.route_idx if route_idx is None else route_idx)
        a.route_w = _p(self.route_w if route_w is None else route_w)
        a.mail, a.mail_n = _p(self.mail), _p(self.mail_n)
        a.workspace, a.workspace_bytes = _p(self.ws), self.ws.numel()
        return a

    def run(self, a: MoeLayerArgs, kernel=None):
        """kernel: None = the library's choice by row count, "rows" / "items" force the
        row-streaming or the item expert kernel."""
        lib().call("sgr_moe_layer_decode_stages", C.byref(a), 7 | KERNEL_BITS[kernel], stream_ptr())


class MoeStack:
    """L layers of weights and a graph-replayed decode step over them.

    The residual stream x [n][H] fp16 passes through the MoE half of every layer in
    turn: layer l reads its input rows from `inputs[l]` (or from x itself when no
    inputs are given) and adds its output to x. With `per_layer_ws` every layer
    keeps its own workspace, so that after a step each layer's plan and staged
    activations are still there and single stages can be re-launched (timing)."""

    def __init__(self, layers, n_max, n_used, device, biases=None, inputs=None,
                 per_layer_ws=False, kernel=None, chain=False):
        self.layers = layers
        self.kernel_bits = KERNEL_BITS[kernel]
        w0 = layers[0]
        self.device = device
        n_ws = len(layers) if per_layer_ws else 1
        self.runners = [MoeLayerRunner(n_max, w0.hidden, w0.n_ff, w0.n_expert, n_used, device)
                        for _ in range(n_ws)]
        self.runner = self.runners[0]
        self.tables = [w.table() for w in layers]
        self.biases = biases
        self.inputs = inputs
        self.n_used = n_used
        self.graph = None
        self.x = torch.zeros(n_max, w0.hidden, dtype=torch.float16, device=device)
        # per-layer routing records, so a finished step can be inspected
        self.idx = torch.zeros(len(layers), n_max, n_used + 1, dtype=torch.int32, device=device)
        self.w = torch.zeros(len(layers), n_max, n_used + 1, dtype=torch.float32, device=device)
        # one persistent launch per layer for up to three rows, else route + experts
        self.launches_per_step = (1 if (kernel is None and n_max <= 3) else 2) * len(layers)
        # chain: layer l's input rows are RMSNorm(x) computed on the device by rmsnorm_quant_f16 (the
        # producer of the MoE half's rows in the reference's decode layer, src/core/session.cpp:1020-1032),
        # so every layer depends on the residual its predecessor wrote
        self.chain = chain
        if chain:
            g = torch.Generator().manual_seed(77)
            self.norm_w = (1.0 + 0.1 * torch.randn(len(layers), w0.hidden, generator=g)).half().to(device)
            self.xn = torch.zeros(n_max, w0.hidden, dtype=torch.float16, device=device)
            self.xq = torch.zeros(n_max, w0.hidden // 256 * 276, dtype=torch.uint8, device=device)
            self.launches_per_step += len(layers)

    def layer_args(self, li, n):
        w = self.layers[li]
        r = self.runners[li % len(self.runners)]
        xn = self.xn if self.chain else self.x if self.inputs is None else self.inputs[li]
        return r, r.args(n, xn, w.router, self.tables[li], w.shared_ptrs(), x_f16=self.x,
                         bias=None if self.biases is None else self.biases[li],
                         route_idx=self.idx[li], route_w=self.w[li])

    def _issue(self, n, stages=7):
        for li in range(len(self.layers)):
            r, a = self.layer_args(li, n)
            if self.chain and (stages & 1):
                lib().call("sgr_rmsnorm_quant_f16", _p(self.xn), _p(self.x), _p(self.norm_w[li]), _p(self.xq),
                           self.layers[0].hidden, 1e-6, n, stream_ptr())
            lib().call("sgr_moe_layer_decode_stages", C.byref(a), stages | self.kernel_bits, stream_ptr())

    def step_eager(self, n):
        self._issue(n)

    def stage_only(self, n, stages):
        """Re-launch one stage of every layer back to back (needs per_layer_ws and a
        finished step)."""
        assert len(self.runners) == len(self.layers)
        self._issue(n, stages)

    def capture_stage(self, n, stages):
        """A graph of one stage of every layer back to back (needs per_layer_ws and a
        finished step, whose plans the workspaces still hold)."""
        assert len(self.runners) == len(self.layers)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._issue(n, stages)
        return g

    def capture(self, n):
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._issue(n)                     # warm-up outside capture (sets func attributes)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._issue(n)
        return self.graph

    def replay(self):
        self.graph.replay()


class PrefillLayer:
    """One MoE layer over a chunk of many token rows, as the reference's
    `Session::moe_dispatch_device` drives it for prefill (src/core/session.cpp:2482-3030),
    call for call through the library's launchers - with the expert math on the int8
    tensor-core grouped GEMM instead of the reference's fp16 cuBLAS path. Buffers follow
    the session's scratch (src/core/session.cpp:207-257)."""

    TOK_PER = 16

    def __init__(self, n_max, hidden, n_ff, n_expert, n_used, device):
        from . import ops
        self.ops = ops
        self.n_max, self.H, self.F, self.E, self.K = n_max, hidden, n_ff, n_expert, n_used
        d, u8, f16, i32, f32 = device, torch.uint8, torch.float16, torch.int32, torch.float32
        R = n_max * n_used
        self.R = R
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

    def args(self, n, xn, x, weights, table, logits=None, shared=True):
        """The argument block of sgr_moe_layer_prefill over this object's buffers; `table` is
        the [3][E] pointer table (any slice stride: a [3][Lm][E] table is passed as the layer's
        slice of matrix 0 with tab_stride = Lm * E)."""
        a = MoePrefillArgs()
        a.n, a.n_max = n, self.n_max
        a.hidden, a.n_ff, a.n_expert, a.n_used = self.H, self.F, self.E, self.K
        a.tok_per, a.shared_w = self.TOK_PER, 1.0
        a.xn, a.router_w, a.logits_in = _p(xn), _p(weights.router), _p(logits)
        a.w_tab, a.tab_stride = _p(table), table.stride(0) if table.dim() == 2 else 0
        if shared:
            a.shared_gate, a.shared_up, a.shared_down = weights.shared_ptrs()
        a.x_f16, a.xq, a.logits = _p(x), _p(self.xq), _p(self.logits)
        a.route_idx, a.route_w, a.gslot, a.grows = _p(self.idx), _p(self.w), _p(self.gslot), _p(self.grows)
        a.off, a.toff, a.meta, a.mail, a.mail_n = _p(self.off), _p(self.toff), _p(self.meta), _p(self.mail), _p(self.mail_n)
        a.xqg, a.g, a.u, a.hq, a.y_grouped = _p(self.xqg), _p(self.g), _p(self.u), _p(self.hq), _p(self.yg)
        a.expert_y = _p(self.expert_y)
        a.sh_g, a.sh_u, a.sh_q, a.sh_y = _p(self.sh_g), _p(self.sh_u), _p(self.sh_q), _p(self.sh_y)
        return a

    def run(self, n, xn, x, weights, table, logits=None, shared=True, experts_only=False):
        """x [n][H] fp16 residual, combined in place: one call of sgr_moe_layer_prefill.
        `logits` replaces the router GEMV (the prefill benchmark draws them directly).
        experts_only re-issues the routed expert stage alone (gate, up, SwiGLU, requantise,
        down) on the plan a full call left behind (timing)."""
        o, H, F, E, K = self.ops, self.H, self.F, self.E, self.K
        if not experts_only:
            a = self.args(n, xn, x, weights, table, logits=logits, shared=shared)
            lib().call("sgr_moe_layer_prefill", C.byref(a), stream_ptr())
            return
        o.moe_grouped_gemm_i8(table[0], self.off, self.xqg, self.g, F, H, E)
        o.moe_grouped_gemm_i8(table[1], self.off, self.xqg, self.u, F, H, E)
        o.silu_mul_f16_n(self.g, self.g, self.u, self.meta, n * K, F)
        o.quantize_q8_k_n(self.g, self.hq, self.meta, F, n * K * (F // 256))
        o.moe_grouped_gemm_i8(table[2], self.off, self.hq, self.yg, H, F, E)
