"""Expert parallelism over the ranks of one node.

Every rank is home to `tokens / world` token rows and owns a contiguous range of
`E / world` experts of every layer (router and shared expert are replicated).
One layer is: route at home -> all-to-all dispatch of fixed-size token records
(Q8_K row, top-k ids, weights) -> owner-side partial layer over all received
rows (only the local experts; shared expert only for the home rows) ->
all-to-all return of the fp32 partial sums -> residual add at home. Both
exchanges are NCCL all-to-alls with fixed capacity (every rank's slot holds all
of its home rows), so the step is static and can be captured in a CUDA graph.
The reference has no multi-GPU path; the layer arithmetic is that of the
single-GPU fused layer.
"""
from __future__ import annotations

import ctypes as C
import json
import os

import numpy as np
import torch
import torch.distributed as dist

Q8K_BYTES = 276


def record_layout(hidden: int, k: int, padded: bool = False):
    """Byte layout of one dispatched token record: Q8_K row (packed 276-byte blocks, or
    288-byte blocks when `padded`), k+1 ids, k+1 weights, padded to 16 bytes.
    -> (record_bytes, idx_offset, w_offset)."""
    xq = hidden // 256 * (288 if padded else Q8K_BYTES)
    idx_off = xq
    w_off = xq + (k + 1) * 4
    rec = (w_off + (k + 1) * 4 + 15) // 16 * 16
    return rec, idx_off, w_off


class ExchangeTimeout(RuntimeError):
    """A peer did not take part in an exchange within the time limit. The process group has
    been aborted (its communicators are gone): the caller re-forms the group or stops."""


def abort_group(group=None):
    """Tear an NCCL group's communicators down without waiting for the peers (ncclCommAbort): no
    collective of this rank stays enqueued behind the one that will never complete. After it the
    group is unusable. gloo has no such call - its shutdown would itself wait for the pending
    operation - so a gloo group is left as it is and the caller just stops using it."""
    try:
        if dist.get_backend(group) != "nccl":
            return
        fn = getattr(dist.distributed_c10d, "_abort_process_group", None)
        if fn is not None:
            fn(group)
        else:
            dist.destroy_process_group(group)
    except Exception:                        # already gone, or nothing to abort
        pass


def guarded_wait(work, timeout_s, what, group=None):
    """Host-side bounded wait for one asynchronous collective. On expiry - or when the backend
    reports an asynchronous error (a peer died: ncclCommGetAsyncError through the watchdog) -
    the group is aborted and ExchangeTimeout raised, so a rank that never posts becomes an
    error on the other ranks and not a hang."""
    import time
    deadline = time.monotonic() + timeout_s
    try:
        while not work.is_completed():        # non-blocking: an event query (NCCL) / a flag (gloo)
            if time.monotonic() > deadline:
                abort_group(group)
                raise ExchangeTimeout(f"{what}: no completion within {timeout_s} s")
            time.sleep(0.0005)
        work.wait()                           # completed: surfaces an error the backend recorded
    except ExchangeTimeout:
        raise
    except RuntimeError as exc:
        abort_group(group)
        raise ExchangeTimeout(f"{what}: {str(exc).splitlines()[0][:200]}") from exc


class EpExchange:
    """The two fixed-capacity all-to-alls of a layer, on whatever device the buffers
    live (NCCL on GPUs; gloo on CPU in the host-logic tests). With timeout_s the
    collectives are issued asynchronously and waited for on the host with that limit
    (eager steps only: inside a captured graph there is no host wait, and the limit
    that applies is the process group's own, enforced by its watchdog)."""

    def __init__(self, world, rank, n_home, hidden, k, device, padded=False, timeout_s=None):
        self.world, self.rank, self.n_home, self.hidden, self.k = world, rank, n_home, hidden, k
        self.padded = padded
        self.timeout_s = timeout_s
        self.rec, self.idx_off, self.w_off = record_layout(hidden, k, padded)
        self.send = torch.zeros(world, n_home, self.rec, dtype=torch.uint8, device=device)
        self.recv = torch.zeros(world, n_home, self.rec, dtype=torch.uint8, device=device)
        self.part = torch.zeros(world, n_home, hidden, dtype=torch.float32, device=device)
        self.back = torch.zeros(world, n_home, hidden, dtype=torch.float32, device=device)

    def dispatch(self):
        """send[0] holds this rank's home records; afterwards recv[p] holds rank p's."""
        if self.world > 1:
            self.send[1:] = self.send[0]
        self._all_to_all(self.recv, self.send, "dispatch all-to-all")

    def combine(self):
        """part[p] holds this rank's partial sums for rank p's home rows; afterwards
        back[p] holds rank p's partial sums for this rank's home rows."""
        self._all_to_all(self.back, self.part, "return all-to-all")

    def _all_to_all(self, dst, src, what):
        if self.timeout_s is None:
            dist.all_to_all_single(dst.view(-1), src.view(-1))
            return
        work = dist.all_to_all_single(dst.view(-1), src.view(-1), async_op=True)
        guarded_wait(work, self.timeout_s, f"rank {self.rank}: {what}")


class PeerExchange:
    """The same two exchanges as stores into peer memory over NVLink: `recv`, `back` and the
    arrival words live in one symmetric-memory buffer that every rank has mapped; a rank's
    kernels write its records / partial sums straight into the owners' / home ranks' slots
    (sgr_ep_push) and the consumer kernels wait for the arrival words (bounded). No library
    collective touches the data path."""

    def __init__(self, world, rank, n_home, hidden, k, device, padded=False):
        import torch.distributed._symmetric_memory as symm
        self.world, self.rank, self.n_home, self.hidden, self.k = world, rank, n_home, hidden, k
        self.padded = padded
        self.rec, self.idx_off, self.w_off = record_layout(hidden, k, padded)
        slot_r, slot_b = n_home * self.rec, n_home * hidden * 4
        off_recv, off_back = 0, world * slot_r
        off_flag_d = off_back + world * slot_b
        off_flag_r = off_flag_d + 256
        total = off_flag_r + 256
        assert slot_r % 16 == 0 and slot_b % 16 == 0 and world <= 64
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        hdl = symm.rendezvous(self.buf, dist.group.WORLD.group_name)
        base = [int(p) for p in hdl.buffer_ptrs]
        u8, f32, i32 = torch.uint8, torch.float32, torch.int32
        self.recv = self.buf[off_recv:off_recv + world * slot_r].view(world, n_home, self.rec)
        self.back = self.buf[off_back:off_back + world * slot_b].view(f32).view(world, n_home, hidden)
        self.flag_d = self.buf[off_flag_d:off_flag_d + 4 * world].view(i32)      # set by the dispatching peers
        self.flag_r = self.buf[off_flag_r:off_flag_r + 4 * world].view(i32)      # set by the returning owners
        self.send = torch.zeros(n_home, self.rec, dtype=u8, device=device)
        self.part = torch.zeros(world, n_home, hidden, dtype=f32, device=device)
        i64 = torch.int64
        # this rank's addresses of its slot in every peer's buffer
        self.dst_recv = torch.tensor([base[p] + off_recv + rank * slot_r for p in range(world)], dtype=i64, device=device)
        self.dst_back = torch.tensor([base[p] + off_back + rank * slot_b for p in range(world)], dtype=i64, device=device)
        self.dst_flag_d = torch.tensor([base[p] + off_flag_d + rank * 4 for p in range(world)], dtype=i64, device=device)
        self.dst_flag_r = torch.tensor([base[p] + off_flag_r + rank * 4 for p in range(world)], dtype=i64, device=device)
        self.step = torch.zeros(1, dtype=i32, device=device)
        self.scratch = torch.zeros(2, dtype=i32, device=device)
        self.slot_r, self.slot_b = slot_r, slot_b
        dist.barrier()
        torch.cuda.synchronize()


class EpStack:
    def __init__(self, layers, tokens, n_used, device, rank, world, biases, inputs, x0, peer=None):
        from .layer import MoeLayerRunner
        w0 = layers[0]
        self.layers, self.device, self.rank, self.world = layers, device, rank, world
        self.tokens, self.k = tokens, n_used
        self.n_home = tokens // world
        lo, hi = w0.lo, w0.hi
        # records carry the Q8 rows in 288-byte blocks when the owner runs the row-streaming kernel,
        # which then reads them in place
        self.padded = device != "cpu" and tokens >= 16
        # peer-memory exchange when the ranks can map each other's memory, NCCL all-to-alls otherwise.
        # SGR_EP_EXCHANGE: "fused" (default: the layer's kernels store into peer memory themselves),
        # "push" (separate copy kernels between the layer's launches), "nccl" (two all-to-alls per layer)
        mode = os.environ.get("SGR_EP_EXCHANGE", "fused")
        self.fused = mode == "fused"
        if peer is None:
            peer = world > 1 and device != "cpu" and mode in ("fused", "push", "peer")
        self.peer = None
        if peer:
            try:
                self.peer = PeerExchange(world, rank, self.n_home, w0.hidden, n_used, device, padded=self.padded)
            except Exception as e:                      # no symmetric memory on this system
                if rank == 0:
                    print(f"peer-memory exchange unavailable ({type(e).__name__}: {e}); using NCCL all-to-alls",
                          file=__import__("sys").stderr)
                self.peer = None
        # every rank must take the same path
        if world > 1 and device != "cpu":
            ok = torch.tensor([1 if self.peer is not None else 0], device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                self.peer = None
        self.ex = (EpExchange(world, rank, self.n_home, w0.hidden, n_used, device, padded=self.padded)
                   if self.peer is None else None)
        self.home = MoeLayerRunner(self.n_home, w0.hidden, w0.n_ff, w0.n_expert, n_used, device)
        self.owner = MoeLayerRunner(tokens, w0.hidden, w0.n_ff, w0.n_expert, n_used, device,
                                    expert_lo=lo, expert_hi=hi)
        self.tables = [w.table() for w in layers]
        self.biases = biases
        h0 = rank * self.n_home
        self.inputs = [x[h0:h0 + self.n_home].contiguous() for x in inputs]
        self.x0 = x0[h0:h0 + self.n_home].contiguous()
        self.x = self.x0.clone()
        self.graph = None
        # route, (push,) plan, experts, (push,) reduce
        own_plan = self.padded and layers[0].n_expert <= 256 and tokens * n_used <= 512     # see issue_layer_fused
        self.launches_per_step = (((3 if own_plan else 4) if self.fused else 6) if self.peer is not None else 4) * len(layers)
        self.n_layers = len(layers)

    def _ptr(self, t, off=0):
        return C.c_void_p(t.data_ptr() + off)

    def issue_layer_peer(self, li):
        """One layer with the exchanges as stores into peer memory."""
        from .capi import lib
        from .ops import stream_ptr
        w, px = self.layers[li], self.peer
        L, sp = lib(), stream_ptr()
        mul, add = self.n_layers, li + 1               # arrival value of this layer in this step
        a = self.home.args(self.n_home, self.inputs[li], w.router, self.tables[li], None, x_f16=self.x,
                           bias=None if self.biases is None else self.biases[li])
        a.xq_out = self._ptr(px.send)
        a.xq_stride = px.rec
        a.route_idx = self._ptr(px.send, px.idx_off)
        a.route_w = self._ptr(px.send, px.w_off)
        a.route_stride = px.rec // 4
        a.xq_padded = int(self.padded)
        L.call("sgr_moe_layer_decode_stages", C.byref(a), 1 | 8, sp)
        L.call("sgr_ep_push", self._ptr(px.send), 0, px.slot_r, self._ptr(px.dst_recv), self._ptr(px.dst_flag_d),
               self.world, self._ptr(px.step), mul, add, self._ptr(px.scratch), sp)
        h0 = self.rank * self.n_home
        b = self.owner.args(self.tokens, None, None, self.tables[li], w.shared_ptrs(), out_f32=px.part,
                            xq_in=px.recv, routing_given=True, no_residual=True, shared_lo=h0,
                            shared_hi=h0 + self.n_home)
        b.xq_stride = px.rec
        b.route_idx = self._ptr(px.recv, px.idx_off)
        b.route_w = self._ptr(px.recv, px.w_off)
        b.route_stride = px.rec // 4
        b.wait_flags, b.wait_step = self._ptr(px.flag_d), self._ptr(px.step)
        b.wait_count, b.wait_mul, b.wait_add = self.world, mul, add
        b.xq_padded = int(self.padded)
        L.call("sgr_moe_layer_decode_stages", C.byref(b), 7, sp)
        L.call("sgr_ep_push", self._ptr(px.part), px.slot_b, px.slot_b, self._ptr(px.dst_back), self._ptr(px.dst_flag_r),
               self.world, self._ptr(px.step), mul, add, self._ptr(px.scratch, 4), sp)
        n = self.n_home * w.hidden
        L.call("sgr_ep_reduce_add_f16_wait", self._ptr(self.x), self._ptr(px.back), self.world, n, n,
               self._ptr(px.flag_r), self._ptr(px.step), mul, add, sp)

    def issue_layer_fused(self, li):
        """One layer with both exchanges done by the layer's own kernels: the route kernel stores the
        records into the owners' receive slots, the expert kernel stores its rows into the home
        ranks' return slots. Four launches: route, plan (waits for the records), experts, home
        reduction (waits for the rows)."""
        from .capi import lib
        from .ops import stream_ptr
        w, px = self.layers[li], self.peer
        L, sp = lib(), stream_ptr()
        mul, add = self.n_layers, li + 1               # arrival value of this layer in this step
        a = self.home.args(self.n_home, self.inputs[li], w.router, self.tables[li], None, x_f16=self.x,
                           bias=None if self.biases is None else self.biases[li])
        a.xq_out = self._ptr(px.send)
        a.xq_stride = px.rec
        a.route_idx = self._ptr(px.send, px.idx_off)
        a.route_w = self._ptr(px.send, px.w_off)
        a.route_stride = px.rec // 4
        a.xq_padded = int(self.padded)
        a.ep_dst, a.ep_flags, a.ep_step = self._ptr(px.dst_recv), self._ptr(px.dst_flag_d), self._ptr(px.step)
        a.ep_world, a.ep_rec_bytes, a.ep_mul, a.ep_add = self.world, px.rec, mul, add
        # the owner call below plans inside its expert kernel (no plan launch) when the records carry
        # padded blocks and the plan fits shared memory; this call's route stage re-arms its counters
        own_plan = self.padded and w.n_expert <= 256 and self.tokens * self.home.n_used <= 512
        if own_plan:
            a.rearm_workspace, a.rearm_mail_n = self._ptr(self.owner.ws), self._ptr(self.owner.mail_n)
            a.rearm_n_max = self.owner.n_max
        L.call("sgr_moe_layer_decode_stages", C.byref(a), 1 | 8, sp)
        h0 = self.rank * self.n_home
        b = self.owner.args(self.tokens, None, None, self.tables[li], w.shared_ptrs(), out_f32=None,
                            xq_in=px.recv, routing_given=True, no_residual=True, shared_lo=h0,
                            shared_hi=h0 + self.n_home)
        b.xq_stride = px.rec
        b.route_idx = self._ptr(px.recv, px.idx_off)
        b.route_w = self._ptr(px.recv, px.w_off)
        b.route_stride = px.rec // 4
        b.wait_flags, b.wait_step = self._ptr(px.flag_d), self._ptr(px.step)
        b.wait_count, b.wait_mul, b.wait_add = self.world, mul, add
        b.xq_padded = int(self.padded)
        b.ep_out, b.ep_flags, b.ep_step = self._ptr(px.dst_back), self._ptr(px.dst_flag_r), self._ptr(px.step)
        b.ep_world, b.ep_home_rows, b.ep_mul, b.ep_add = self.world, self.n_home, mul, add
        L.call("sgr_moe_layer_decode_stages", C.byref(b), (6 | 128) if own_plan else 7, sp)
        n = self.n_home * w.hidden
        L.call("sgr_ep_reduce_add_f16_wait", self._ptr(self.x), self._ptr(px.back), self.world, n, n,
               self._ptr(px.flag_r), self._ptr(px.step), mul, add, sp)

    def issue_layer(self, li):
        if self.peer is not None:
            return self.issue_layer_fused(li) if self.fused else self.issue_layer_peer(li)
        from .capi import lib
        from .ops import stream_ptr
        w, ex = self.layers[li], self.ex
        # 1. home: quantise + route straight into the dispatch record slot 0
        a = self.home.args(self.n_home, self.inputs[li], w.router, self.tables[li], None, x_f16=self.x,
                           bias=None if self.biases is None else self.biases[li])
        a.xq_out = self._ptr(ex.send)
        a.xq_stride = ex.rec
        a.route_idx = self._ptr(ex.send, ex.idx_off)
        a.route_w = self._ptr(ex.send, ex.w_off)
        a.route_stride = ex.rec // 4
        a.xq_padded = int(self.padded)
        lib().call("sgr_moe_layer_decode_stages", C.byref(a), 1 | 8, stream_ptr())
        ex.dispatch()
        # 2. owner: the local experts over every received row, weighted, no residual
        h0 = self.rank * self.n_home
        b = self.owner.args(self.tokens, None, None, self.tables[li], w.shared_ptrs(), out_f32=ex.part,
                            xq_in=ex.recv, routing_given=True, no_residual=True, shared_lo=h0,
                            shared_hi=h0 + self.n_home)
        b.xq_stride = ex.rec
        b.route_idx = self._ptr(ex.recv, ex.idx_off)
        b.route_w = self._ptr(ex.recv, ex.w_off)
        b.route_stride = ex.rec // 4
        b.xq_padded = int(self.padded)
        lib().call("sgr_moe_layer_decode_stages", C.byref(b), 7, stream_ptr())
        ex.combine()
        # 3. home: residual += sum over owner ranks
        n = self.n_home * w.hidden
        lib().call("sgr_ep_reduce_add_f16", self._ptr(self.x), self._ptr(ex.back), self.world, n, n,
                   stream_ptr())

    def step_eager(self):
        for li in range(len(self.layers)):
            self.issue_layer(li)
        if self.peer is not None:
            from .capi import lib
            from .ops import stream_ptr
            lib().call("sgr_ep_step_advance", self._ptr(self.peer.step), stream_ptr())

    def capture(self):
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.step_eager()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step_eager()

    def replay(self):
        self.graph.replay()


def run_ep_bench(args, rank, world, device):
    """N > 1 leg of bench.py: returns the JSON line (rank 0 prints it)."""
    import bench
    from . import synth
    from .capi import lib
    E, K, H, FF = bench.E, bench.K, bench.H, bench.FF
    layers_n, tokens = args.layers, args.tokens     # (`bench` imported here is a second copy of the script's module)
    assert E % world == 0 and tokens % world == 0
    lo, hi = rank * (E // world), (rank + 1) * (E // world)
    ws = [synth.MoeWeights(H, FF, E, device, seed=bench.SEED + li, expert_range=(lo, hi))
          for li in range(layers_n)]
    inputs = [synth.normal_fp16((tokens, H), bench.SEED + 500 + li, device) for li in range(layers_n)]
    x0 = synth.normal_fp16((tokens, H), bench.SEED + 499, device)
    alpha = bench.calibrate_alpha(inputs[0], ws[0].router, device)
    biases = [torch.from_numpy(synth.zipf_bias(E, bench.SEED + 900 + li, alpha)).to(device)
              for li in range(layers_n)]
    st = EpStack(ws, tokens, K, device, rank, world, biases, inputs, x0)
    st.capture()

    def step():
        st.x.copy_(st.x0, non_blocking=True)
        st.replay()

    def timed(fn, iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(args.warmup):
        step()
    # parity inside the line: a step of a sub-stack (the first 2 layers; with --check the whole
    # stack that --layers gives) against the single-GPU fused layers on rank 0
    n_chk = layers_n if getattr(args, "check", False) else min(2, layers_n)
    if n_chk == layers_n:
        chk = st
    else:
        chk = EpStack(ws[:n_chk], tokens, K, device, rank, world, biases[:n_chk], inputs[:n_chk], x0)
        chk.capture()
    chk.x.copy_(chk.x0)
    chk.replay()
    torch.cuda.synchronize()
    parts = [torch.empty_like(chk.x) for _ in range(world)]
    dist.all_gather(parts, chk.x)
    check = None
    if rank == 0:
        from .layer import MoeStack
        full = [synth.MoeWeights(H, FF, E, device, seed=bench.SEED + li) for li in range(n_chk)]
        ref = MoeStack(full, tokens, K, device, biases=biases[:n_chk], inputs=inputs[:n_chk])
        ref.x.copy_(x0)
        ref.step_eager(tokens)
        torch.cuda.synchronize()
        got = torch.cat(parts).float()
        want = ref.x.float()
        check = float((got - want).abs().max() / want.abs().max())
        del full, ref
    if chk is not st:
        del chk
    nvlink = nvlink_bytes(ws, inputs, biases, tokens, world, K, H, st)
    sampler = bench.ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    ms_step = timed(step, args.steps)

    h_in = torch.empty(layers_n + 1, st.n_home, H, dtype=torch.float16).pin_memory()
    h_in[0].copy_(st.x0.cpu())
    for li in range(layers_n):
        h_in[li + 1].copy_(st.inputs[li].cpu())
    d_in = torch.empty_like(h_in, device=device)
    h_out = torch.empty(st.n_home, H, dtype=torch.float16).pin_memory()

    def e2e_step():
        d_in.copy_(h_in, non_blocking=True)
        st.x.copy_(d_in[0], non_blocking=True)
        for li in range(layers_n):
            st.inputs[li].copy_(d_in[li + 1], non_blocking=True)
        st.replay()
        h_out.copy_(st.x, non_blocking=True)

    for _ in range(3):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    clocks = sampler.stop()
    status = lib().raw("sgr_status")(0)
    line = {
        "metric": "q4k_moe_decode_tokens_per_s", "value": tokens / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 dots, fp32 accumulate", "data": "synthetic",
        "config": dict(bench.workload_config(world), layers=layers_n, tokens=tokens, zipf_alpha=alpha,
                       exchange=(("records and partial sums stored into peer memory over NVLink by the layer's own "
                                  "kernels (route and expert kernel), arrival words, 3 launches per layer (route, experts with their own plan, home reduction)") if st.fused else
                                 ("records and partial sums stored into peer memory over NVLink by copy kernels "
                                  "between the layer's launches, arrival words, 6 launches per layer")) if st.peer is not None
                       else "2 NCCL all-to-alls per layer, fixed capacity, captured in the step graph"),
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": int(h_in.numel() * 2) * world,
                "d2h_bytes_per_step": int(h_out.numel() * 2) * world},
        "gpu_launches": st.launches_per_step * args.steps, "clocks": clocks,
        "roofline": {"kernel": "expert_rows_kernel", "bound": "hbm", "achieved": None, "peak": bench.load_peaks()[0],
                     "unit": "GB/s", "frac": None, "traffic": None,
                     "note": "per-kernel timing is taken at N=1; at N>1 the step is exchange-latency bound"},
    }
    if status != 0:
        line["device_status"] = "a bounded device-side wait gave up"
    if check is not None:
        line["check_max_rel_err_vs_single_gpu"] = check
        line["check_layers"] = n_chk
    line["nvlink_bytes_per_layer"] = nvlink
    return line


def nvlink_bytes(ws, inputs, biases, tokens, world, k, hidden, st):
    """Bytes that cross NVLink per layer, whole job (mean over the layers), counted from the
    routing: algorithmic = one Q8_K row (hidden/256 * 276 B) per (token, owner rank other than its
    home that holds at least one of its top-k) and one fp32 row back per such pair; moved = what
    the exchange kernels store into other ranks' memory (every record to every other rank, every
    rank's partial rows back)."""
    n_exp = ws[0].n_expert
    per = n_exp // world
    n_home = tokens // world
    pairs = []
    for li in range(len(ws)):
        lg = inputs[li].float() @ ws[li].router.t()
        if biases is not None:
            lg = lg + biases[li]
        owner = lg.topk(k, dim=1).indices // per                       # [tokens][k] owner rank of each pick
        home = torch.arange(tokens, device=lg.device) // n_home
        hit = torch.zeros(tokens, world, dtype=torch.bool, device=lg.device)
        hit.scatter_(1, owner, True)
        hit[torch.arange(tokens), home] = False
        pairs.append(int(hit.sum().item()))
    p = float(np.mean(pairs))
    rec = st.peer.rec if st.peer is not None else st.ex.rec
    return {"dispatch_algorithmic": p * (hidden // 256 * Q8K_BYTES), "return_algorithmic": p * hidden * 4,
            "dispatch_moved": float(tokens * (world - 1) * rec), "return_moved": float(tokens * (world - 1) * hidden * 4),
            "remote_token_owner_pairs": p}
