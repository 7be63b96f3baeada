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

from .capi import MoeLayerArgs, lib
from .ops import stream_ptr


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


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

    def run(self, a: MoeLayerArgs):
        lib().call("sgr_moe_layer_decode", C.byref(a), stream_ptr())


class MoeStack:
    """L layers of weights and a graph-replayed decode step over them.

    The residual stream x [n][H] fp16 passes through the MoE half of every layer in
    turn: layer l reads its input rows from `inputs[l]` (or from x itself when no
    inputs are given) and adds its output to x. With `per_layer_ws` every layer
    keeps its own workspace, so that after a step each layer's plan and staged
    activations are still there and single stages can be re-launched (timing)."""

    def __init__(self, layers, n_max, n_used, device, biases=None, inputs=None,
                 per_layer_ws=False):
        self.layers = layers
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
        self.launches_per_step = 2 * len(layers)     # route + experts

    def layer_args(self, li, n):
        w = self.layers[li]
        r = self.runners[li % len(self.runners)]
        xn = self.x if self.inputs is None else self.inputs[li]
        return r, r.args(n, xn, w.router, self.tables[li], w.shared_ptrs(), x_f16=self.x,
                         bias=None if self.biases is None else self.biases[li],
                         route_idx=self.idx[li], route_w=self.w[li])

    def _issue(self, n, stages=7):
        for li in range(len(self.layers)):
            r, a = self.layer_args(li, n)
            lib().call("sgr_moe_layer_decode_stages", C.byref(a), stages, stream_ptr())

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
