#!/usr/bin/env python3
"""Decode-throughput benchmark of the Q4_K MoE expert path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (one "step" = one decode step of the MoE halves of a 40-layer stack):
64 concurrent token rows, hidden 2048, 256 routed experts (FFN 512, top-8) plus
one shared expert per layer, Q4_K weights drawn from N(0, 0.02), fp16 inputs
drawn from N(0, 1), router logits skewed with a Zipf(s=1.1) bias so that about
20 % of the experts take about 70 % of the routed picks. With N > 1 the experts
of every layer are sharded contiguously over the ranks (expert parallelism) and
token rows travel by all-to-all. Everything is synthetic and seeded.

Prints one JSON line (rank 0). `value` is tokens/s with the inputs resident in
HBM, `e2e` the same through host buffers, `roofline` describes the dominant
kernel (the expert kernel: gate/up/down projections of all routed experts), `cpu_baseline` the reference's CPU expert pool on
this machine's cores over a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, FF, E, K, LAYERS, TOKENS = 2048, 512, 256, 8, 40, 64
SEED = 20260718 + 1000 * 4
MAT_BYTES = 589_824           # one 512x2048 or 2048x512 Q4_K matrix
EXPERT_BYTES = 3 * MAT_BYTES
ROUTER_BYTES = E * H * 4
HOT_TARGET = 0.70


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()          # the exact process started above
        self.t.join(timeout=2)
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------
def build_workload(device, rank, world, layers, tokens):
    """Seeded weights (this rank's expert shard only when world > 1), inputs, biases."""
    import torch
    from sager_b200 import synth
    ws = []
    for li in range(layers):
        ws.append(synth.MoeWeights(H, FF, E, device, seed=SEED + li))
    inputs = [synth.normal_fp16((tokens, H), SEED + 500 + li, device) for li in range(layers)]
    x0 = synth.normal_fp16((tokens, H), SEED + 499, device)
    alpha = calibrate_alpha(inputs[0], ws[0].router, device)
    biases = [torch.from_numpy(synth.zipf_bias(E, SEED + 900 + li, alpha)).to(device)
              for li in range(layers)]
    return ws, inputs, x0, biases, alpha


def calibrate_alpha(x0_rows, router, device):
    """Zipf bias strength: one alpha for the stack, found by bisection on layer 0 so that
    the top 20 % of the experts take ~70 % of the routed picks."""
    import torch
    from sager_b200 import synth
    ranks0 = synth.zipf_bias(E, SEED + 900, 1.0)

    def share(alpha):
        lg = x0_rows.float() @ router.t() + torch.from_numpy(ranks0 * alpha).to(device)
        idx = lg.topk(K, dim=1).indices.cpu().numpy()
        return synth.hot_share(idx, E)

    lo, hi = 0.0, 4.0
    for _ in range(24):
        mid = 0.5 * (lo + hi)
        if share(mid) < HOT_TARGET:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


def cpu_pool_sample(ws0, xn0, bias0, budget_s=12.0, layers=None, max_steps=20):
    """Time the reference's CPU expert pool (oracle/_ref: src/kernels/cpu/pool.cpp:74-134 running
    src/kernels/cpu/q4_avx2.cpp:175-196 per job) - or, without it, the C port - on the workload's
    expert FFNs. The routing of layer 0 (router + top-8 with the stack's Zipf bias, by the C
    restatement on one thread; the reference itself never routes on the CPU) is computed once and
    timed apart. A step submits, for each of `layers` layers, one pool job per (token row, routed
    expert) and per (token row, shared expert) - layer 0's jobs every time, 453 MB of expert
    weights, more than the host's last-level cache - and waits for them; the weighted sum is done
    on the host. `layers` is cut down (and the step time scaled up, which the result says) only
    when a full step would not fit the time budget."""
    from oracle import oracle as orc
    o = orc.Oracle() if os.path.exists(os.path.join(orc.HERE, "libsager_oracle.so")) else None
    if o is None:
        orc.build(ref_root=os.devnull)
        o = orc.Oracle()
    layers = LAYERS if layers is None else layers
    cores = os.cpu_count() or 1
    x16 = xn0.cpu().numpy()
    router = ws0.router.cpu().numpy()
    bias = bias0.cpu().numpy()
    n = x16.shape[0]
    blob = ws0.blob.cpu().numpy()
    gu = ws0.gu_bytes
    base = blob.ctypes.data

    def ptrs(e):
        b = base + e * ws0.expert_bytes
        return [b, b + gu, b + 2 * gu]

    try:
        ref = orc.Reference()
        pool = ref.pool(cores, H, FF, E)
        kind = "reference"
    except (FileNotFoundError, OSError, RuntimeError):
        ref, pool, kind = None, None, "port"

    t0 = time.perf_counter()
    idx = np.zeros((n, K + 1), dtype=np.int32)
    wts = np.zeros((n, K + 1), dtype=np.float32)
    for t in range(n):
        lg = o.router_logits(router, x16[t]) + bias
        idx[t], wts[t] = o.router_topk(lg, K, shared_w=1.0)
    router_s = time.perf_counter() - t0
    xf = x16.astype(np.float32)
    w3, xs = [], []
    for t in range(n):
        for kk in range(K + 1):
            w3 += ptrs(int(idx[t, kk]) if kk < K else E)
            xs.append(xf[t])
    xs = np.stack(xs)
    n_ffn = xs.shape[0]

    def run_jobs(p, w3_, xs_):
        return p.run(w3_, xs_) if p is not None else _port_batch(o, w3_, xs_, cores)

    def one_layer():
        t1 = time.perf_counter()
        ys = run_jobs(pool, w3, xs).reshape(n, K + 1, H)
        out = xf.copy()
        for kk in range(K + 1):
            out += wts[:, kk:kk + 1] * ys[:, kk]
        return time.perf_counter() - t1

    one_layer()                                   # warm-up (page in the weights)
    t_probe = one_layer()
    per_step = max(1, min(layers, int(budget_s / 3.0 / max(t_probe, 1e-4))))    # layers actually run per step
    steps_t = []
    t_start = time.perf_counter()
    while (time.perf_counter() - t_start < budget_s and len(steps_t) < max_steps) or not steps_t:
        t_step = 0.0
        for _ in range(per_step):
            t_step += one_layer()
        steps_t.append(t_step * layers / per_step)
    # one worker, on a slice of the same jobs
    one_worker_ms = None
    if ref is not None:
        m = min(n_ffn, 36)
        p1 = ref.pool(1, H, FF, E)
        p1.run(w3[:3 * m], xs[:m])
        t1 = time.perf_counter()
        p1.run(w3[:3 * m], xs[:m])
        one_worker_ms = (time.perf_counter() - t1) * 1e3 / m
        p1.close()
    if pool is not None:
        pool.close()
    t_step = float(np.median(steps_t))
    del blob
    return {"t_step_s": t_step, "steps_list": steps_t, "cores": cores, "kind": kind, "steps_timed": len(steps_t),
            "layers_per_step_run": per_step, "layers": layers, "ffn_per_layer": n_ffn,
            "ms_per_ffn": t_step * 1e3 / (layers * n_ffn),
            "effective_gbs": layers * n_ffn * EXPERT_BYTES / t_step / 1e9,
            "one_worker_ms_per_ffn": one_worker_ms,
            "router_ms_per_layer_not_in_value": router_s * 1e3}


def cpu_baseline_entry(res, n):
    scaled = "" if res["layers_per_step_run"] == res["layers"] else \
        f" ({res['layers_per_step_run']} layers run per step, time scaled to {res['layers']})"
    return {"value": n / res["t_step_s"], "unit": "tokens/s", "cores": res["cores"], "kind": res["kind"],
            "sample": f"{res['steps_timed']} steps of {res['layers']} layers x {res['ffn_per_layer']} expert FFNs "
                      f"({n} token rows x (top-{K} + shared), layer 0's routing and weights every layer) through the "
                      f"reference's CPU pool on all host cores{scaled}; the router (C restatement, one thread, "
                      f"{res['router_ms_per_layer_not_in_value']:.0f} ms per layer) is not in the value: the reference never "
                      "routes on the CPU",
            "ms_per_step": res["t_step_s"] * 1e3, "ms_per_ffn": res["ms_per_ffn"],
            "effective_gbs": res["effective_gbs"], "one_worker_ms_per_ffn": res["one_worker_ms_per_ffn"],
            "router_ms_per_layer": res["router_ms_per_layer_not_in_value"]}


def ref_cuda_decode(ws, inputs, x0, biases, n, device, steps, ours_x):
    """The same decode step on the reference's own CUDA kernels (compiled for sm_100a into
    oracle/_ref/libsager_ref_cuda.so) in the reference's launch sequence for its device MoE
    path (src/core/session.cpp:2482-3030, dp4a branch), captured in a CUDA graph like the
    reference's step graph. None when that library was not built."""
    import torch
    from oracle import ref_cuda
    if not ref_cuda.available():
        return None
    path = ref_cuda.DeviceMoePath(ref_cuda.reference_launchers(), n, H, FF, E, K, device)
    x = x0.clone()
    tables = [w.table() for w in ws]

    def issue():
        for li, w in enumerate(ws):
            path.run(n, inputs[li], x, w.router, tables[li], w.shared_ptrs(), bias=biases[li])

    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        issue()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    diff = float((x.float() - ours_x.float()).abs().max() / ours_x.float().abs().max())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        issue()
    for _ in range(3):
        x.copy_(x0, non_blocking=True)
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        x.copy_(x0, non_blocking=True)
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"value": n / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "kind": "the reference's CUDA kernels built for sm_100a, its device MoE launch sequence "
                    "(dp4a branch), one CUDA graph per step",
            "launches_per_step": (path.launches + 2) * len(ws),
            "max_rel_diff_vs_this_library_after_one_step": diff}


def _port_batch(o, w3_ptrs, xs, cores):
    """expert_ffn_batch on raw addresses (the C port takes void* either way)."""
    import ctypes as C
    n_jobs = xs.shape[0]
    y = np.zeros((n_jobs, H), dtype=np.float32)
    arr = (C.c_void_p * len(w3_ptrs))(*w3_ptrs)
    o.lib.orc_expert_ffn_batch(arr, xs.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p),
                               n_jobs, H, FF, cores)
    return y


def run_reference_arm(args):
    """The reference's own CPU implementation of the path on this machine's cores: each step
    runs the expert FFNs of the 40-layer, 64-row step through the reference's CpuPool (see
    cpu_pool_sample), with the same calibrated routing skew as the GPU arm."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    device = "cuda:0" if torch.cuda.is_available() else "cpu"
    from sager_b200 import synth
    w0 = synth.MoeWeights(H, FF, E, device, seed=SEED)
    xn0 = synth.normal_fp16((TOKENS, H), SEED + 500, device)
    alpha = calibrate_alpha(xn0, w0.router, device)
    bias0 = torch.from_numpy(synth.zipf_bias(E, SEED + 900, alpha)).to(device)
    total = args.steps + args.warmup
    res = cpu_pool_sample(w0, xn0, bias0, budget_s=max(10.0, min(150.0, 6.0 * total)), max_steps=total)
    timed = res["steps_list"][args.warmup:] or res["steps_list"]      # the first W steps are warm-up
    res["t_step_s"], res["steps_timed"] = float(np.median(timed)), len(timed)
    value = TOKENS / res["t_step_s"]
    cb = cpu_baseline_entry(res, TOKENS)
    line = {
        "impl": "reference", "metric": "q4k_moe_decode_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": res["steps_timed"], "warmup": args.warmup,
        "ms_per_step": res["t_step_s"] * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 dots, fp32 accumulate", "data": "synthetic",
        "config": dict(workload_config(args.gpus), zipf_alpha=alpha),
        "cpu_baseline": cb,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(n_gpus):
    return {"workload": "expert-parallel decode: 40 MoE layers x 256 Q4_K experts (top-8 + shared), "
                        "64 token rows, Zipf-skewed routing",
            "hidden": H, "expert_ffn": FF, "experts": E, "top_k": K, "layers": LAYERS,
            "tokens": TOKENS, "experts_per_gpu": E // n_gpus,
            "parallelism": f"ep{n_gpus}" if n_gpus > 1 else "single",
            "l2": "per-step weight traffic (>5 GB) far exceeds the 126 MB L2; no flush needed"}


# ---------------------------------------------------------------------------------------
def prefill_measure(args, device, sampler=None):
    """Prefill chunk of one MoE layer: 2048 token rows, top-8 of 256 experts, router logits
    drawn uniformly (about 64 rows per expert), expert math on the int8 tensor-core grouped
    GEMM. A step = quantise, top-k, plan, gather, gate/up/down grouped GEMMs, SwiGLU,
    requantise, scatter, shared expert, combine. The 453 MB of expert weights exceed L2."""
    import torch
    from sager_b200 import lib, synth
    from sager_b200.layer import PrefillLayer
    n = args.prefill_tokens
    w = synth.MoeWeights(H, FF, E, device, seed=SEED + 3000)
    table = w.table()
    xn = synth.normal_fp16((n, H), SEED + 3001, device)
    x0 = synth.normal_fp16((n, H), SEED + 3002, device)
    x = x0.clone()
    gen = torch.Generator(device=device)
    gen.manual_seed(SEED + 3003)
    logits = torch.rand(n, E, generator=gen, device=device, dtype=torch.float32)
    layer = PrefillLayer(n, H, FF, E, K, device)

    def step():
        x.copy_(x0, non_blocking=True)
        layer.run(n, xn, x, w, table, logits=logits)

    def timed(fn, reps):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    own_sampler = sampler is None
    if own_sampler:
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
    ms_step = timed(step, args.steps)
    # the routed expert stage alone: gate, up, SwiGLU, requantise, down (plan and gathered rows still in place)
    ms_gemm = timed(lambda: layer.run(n, xn, x, w, table, experts_only=True), args.steps)
    h_xn, h_x = xn.cpu().pin_memory(), x0.cpu().pin_memory()
    h_lg = logits.cpu().pin_memory()
    h_out = torch.empty(n, H, dtype=torch.float16).pin_memory()

    def e2e_step():
        xn.copy_(h_xn, non_blocking=True)
        x.copy_(h_x, non_blocking=True)
        logits.copy_(h_lg, non_blocking=True)
        layer.run(n, xn, x, w, table, logits=logits)
        h_out.copy_(x, non_blocking=True)

    ms_e2e = timed(e2e_step, args.steps)
    clocks = sampler.stop() if own_sampler else None
    off = layer.off.cpu().numpy()
    rows = np.diff(off)
    routed = int(rows.sum())
    used = int((rows > 0).sum())
    ops = 2.0 * routed * 3 * FF * H                       # int8 multiply-adds x 2, algorithmic
    gemm_bytes = used * EXPERT_BYTES
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0}
    i8_peak = 2.0 * float(peaks["bf16_tflops"])           # dense int8 = twice the bf16 rate
    tops = ops / (ms_gemm * 1e-3) / 1e12
    gbs = gemm_bytes / (ms_gemm * 1e-3) / 1e9
    line = {
        "metric": "q4k_moe_prefill_tokens_per_s", "value": n / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 tensor-core dots (tcgen05), fp32 scaling", "data": "synthetic",
        "config": {"workload": f"prefill MoE layer: {n} token rows, top-{K} of {E} Q4_K experts + shared, "
                               "uniform router logits", "hidden": H, "expert_ffn": FF,
                   "rows_per_expert_mean": float(rows.mean()), "rows_per_expert_max": int(rows.max()),
                   "l2": "453 MB of expert weights per step exceed the 126 MB L2; no flush needed"},
        "e2e": {"value": n / (ms_e2e * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": int(h_xn.numel() * 2 + h_x.numel() * 2 + h_lg.numel() * 4),
                "d2h_bytes_per_step": int(h_out.numel() * 2)},
        "gpu_launches": 15 * args.steps, "clocks": clocks,
        "roofline": {"kernel": "grouped_gemm_i8_kernel (gate, up, down launches; the timed region also holds the SwiGLU and requantise launches between them)", "bound": "tensor",
                     "achieved": tops, "peak": i8_peak, "unit": "TOP/s", "frac": tops / i8_peak,
                     "peak_source": "2 x measured cuBLAS bf16 burst rate (dense int8 runs at twice bf16)",
                     "traffic": None, "ms_expert_stage": ms_gemm,
                     "hbm": {"achieved": gbs, "peak": float(peaks["hbm_gbs"]), "unit": "GB/s",
                             "frac": gbs / float(peaks["hbm_gbs"]), "bytes": gemm_bytes}},
    }
    if lib().raw("sgr_status")(0) != 0:
        line["device_status"] = "a bounded device-side wait gave up"
    if not args.no_gpu_baseline:
        # the same chunk on the reference's own CUDA kernels in its device MoE sequence (dp4a branch)
        try:
            from oracle import ref_cuda
            if ref_cuda.available():
                path = ref_cuda.DeviceMoePath(ref_cuda.reference_launchers(), n, H, FF, E, K, device)
                xr = x0.clone()

                def ref_step():
                    xr.copy_(x0, non_blocking=True)
                    path.run(n, xn, xr, w.router, table, w.shared_ptrs(), logits=logits)
                ms_ref = timed(ref_step, max(2, min(args.steps, 5)))
                step()
                torch.cuda.synchronize()
                line["gpu_baseline"] = {
                    "value": n / (ms_ref * 1e-3), "unit": "tokens/s", "ms_per_step": ms_ref,
                    "kind": "the reference's CUDA kernels built for sm_100a, its device MoE launch sequence "
                            "(dp4a branch), eager launches",
                    "max_rel_diff_vs_this_library": float((xr.float() - x.float()).abs().max() /
                                                          x.float().abs().max())}
        except Exception as exc:
            line["gpu_baseline"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    return line


def run_prefill_bench(args, device):
    print(json.dumps(prefill_measure(args, device)))


def prefill_config_leg(args, device):
    """config[3] inside the default line: the prefill chunk, compact."""
    line = prefill_measure(args, device, sampler=False)
    r = line["roofline"]
    out = {"workload": line["config"]["workload"], "tokens_per_s": line["value"], "ms_per_step": line["ms_per_step"],
           "e2e_tokens_per_s": line["e2e"]["value"], "ms_expert_stage": r["ms_expert_stage"],
           "tensor_frac_of_int8_peak": r["frac"], "tops": r["achieved"], "hbm_frac": r["hbm"]["frac"], "hbm_gbs": r["hbm"]["achieved"],
           "binding": "hbm (227 op/B at ~64 rows per expert is below the int8 ridge of ~500 op/B)"}
    if "gpu_baseline" in line:
        out["gpu_baseline"] = line["gpu_baseline"]
    return out


def gemv_measure(args, device, shapes=None, sampler=None):
    """Dense Q4_K x Q8_K GEMV sweep (config[1]): the five shapes at batch 1 and 4, weights drawn
    from N(0, 0.02), activations from N(0, 1) and Q8-quantised by the library. Each shape is timed
    over enough distinct weight copies to exceed L2 (the small matrices would otherwise be served
    from it), CUDA events around the loop; GB/s counts the weight bytes only."""
    import torch
    from sager_b200 import lib, ops, synth
    peak, kind = load_peaks()
    shapes = shapes or [(4096, 2048), (2048, 4096), (512, 2048), (2048, 512), (151936, 2048)]
    q6_only = args.shape == "q6head"             # profiling captures: only the Q6_K head and its top-k
    if q6_only:
        shapes = []
    elif args.shape:
        shapes = [tuple(int(v) for v in args.shape.split(","))]
    rows_out = []
    ref = None
    if not args.no_gpu_baseline:
        from oracle import ref_cuda
        if ref_cuda.available():
            ref = ref_cuda.reference_launchers()      # the reference's own kernels, timed on the same buffers
    own_sampler = sampler is None
    if own_sampler:
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
    for rows, k in shapes:
        wbytes = rows * (k // 256) * 144
        copies = max(1, min(512, (192 << 20) // wbytes + 1))       # > 126 MB L2 in flight per sweep
        g = torch.Generator(device=device).manual_seed(SEED + rows)
        w1 = synth.quantize_q4k(torch.randn(min(rows, 4096), k, generator=g, device=device) * 0.02).reshape(-1)
        w = torch.empty(copies, wbytes, dtype=torch.uint8, device=device)
        for c in range(copies):
            for r0 in range(0, wbytes, w1.numel()):
                n = min(w1.numel(), wbytes - r0)
                w[c, r0:r0 + n] = w1[:n]
        for batch in (1, 4):
            x = synth.normal_fp16((batch, k), SEED + k + batch, device)
            xq = torch.empty(batch, k // 256 * 276, dtype=torch.uint8, device=device)
            ops.quantize_q8_k(x, xq, batch * k)
            y = torch.zeros(batch, rows, dtype=torch.float32, device=device)
            def timed(o):
                def sweep():
                    for c in range(copies):
                        if batch == 1:
                            o.gemv_q4_k_q8(w[c], xq, y, rows, k)
                        else:
                            o.gemv_q4_k_q8_batched(w[c], xq, y, rows, k, batch)
                sweep()                                   # sets function attributes outside capture
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()                # launches back to back, no host time between them
                with torch.cuda.graph(graph):
                    sweep()
                for _ in range(max(args.warmup, 3)):
                    graph.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.steps):
                    graph.replay()
                e1.record()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1) * 1e3 / (args.steps * copies)
            us = timed(ops)
            row = {"rows": rows, "k": k, "batch": batch, "us": us, "gbs": wbytes / us / 1e3,
                   "frac": wbytes / us / 1e3 / peak, "weight_copies": copies}
            if ref is not None:
                ref_us = timed(ref)
                row["reference_cuda_us"] = ref_us
                row["reference_cuda_gbs"] = wbytes / ref_us / 1e3
            rows_out.append(row)
    q6 = q6_head_measure(args, device, ops, ref, peak) if (q6_only or not args.shape) else None
    clocks = sampler.stop() if own_sampler else None
    if q6_only:
        return {"metric": "q6k_head_hbm_gbs", "value": q6["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": q6["us"] * 1e-3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "int8 dots, fp32 accumulate", "data": "synthetic",
                "config": {"workload": "Q6_K LM head 151936 x 2048 at batch 1 and the two-phase top-k of its logits",
                           "l2": "two weight copies of 255 MB alternate"},
                "e2e": None, "gpu_launches": args.steps * 18, "clocks": clocks,
                "roofline": {"kernel": "gemv_q6_stream_kernel (head.cu)", "bound": "hbm", "achieved": q6["gbs"],
                             "peak": peak, "unit": "GB/s", "frac": q6["frac"],
                             "peak_source": f"{kind} copy bandwidth (burst)", "traffic": None},
                "q6k_head": q6}
    head = max((r for r in rows_out if r["batch"] == 1), key=lambda r: r["rows"] * r["k"])
    line = {
        "metric": "q4k_gemv_hbm_gbs", "value": head["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": head["us"] * 1e-3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 dots, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "dense Q4_K GEMV sweep at batch 1 and 4; value = LM head 2048->151936 at batch 1",
                   "l2": "every launch of a sweep reads a different weight copy, > 126 MB between reuses"},
        "e2e": None, "gpu_launches": args.steps * sum(r["weight_copies"] for r in rows_out), "clocks": clocks,
        "roofline": {"kernel": "gemv_stream_kernel (gemv.cu)", "bound": "hbm", "achieved": head["gbs"], "peak": peak,
                     "unit": "GB/s", "frac": head["frac"], "peak_source": f"{kind} copy bandwidth (burst)",
                     "traffic": None},
        "sweep": rows_out,
    }
    if q6 is not None:
        line["q6k_head"] = q6
    if lib().raw("sgr_status")(0) != 0:
        line["device_status"] = "a bounded device-side wait gave up"
    return line


def q6_head_measure(args, device, ops, ref, peak):
    """The LM head as the checkpoint stores it (Q6_K, 210-byte blocks) and the two-phase top-k over
    its logits: 151936 x 2048 = 255 MB per launch, twice the L2, two weight copies alternating.
    Random 6-bit codes and sub-block scales with a small block scale; time does not depend on
    the values."""
    import torch
    rows, k, topk = 151936, 2048, 40
    nblk = rows * (k // 256)
    g = torch.Generator(device=device).manual_seed(SEED + 6)
    w = torch.randint(0, 256, (2, nblk, 210), dtype=torch.uint8, device=device, generator=g)
    w[:, :, 208:210] = torch.tensor([0.01], dtype=torch.float16).view(torch.uint8).to(device)
    from sager_b200 import synth
    x = synth.normal_fp16((1, k), SEED + 66, device)
    xq = torch.empty(1, k // 256 * 276, dtype=torch.uint8, device=device)
    ops.quantize_q8_k(x, xq, k)
    y = torch.zeros(rows, dtype=torch.float32, device=device)
    slots = (rows + 2047) // 2048 * topk
    seg_v = torch.zeros(slots, dtype=torch.float32, device=device)
    seg_i = torch.zeros(slots, dtype=torch.int32, device=device)
    out_v = torch.zeros(64, dtype=torch.float32, device=device)
    out_i = torch.zeros(64, dtype=torch.int32, device=device)

    def timed(fn, per_replay):
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (args.steps * per_replay)

    def head(o):
        return lambda: [o.gemv_q6_k_q8(w[c], xq, y, rows, k) for c in range(2)]

    def select(o):
        return lambda: [o.topk_select_f32_2p(y, seg_v, seg_i, slots, out_v, out_i, rows, topk) for _ in range(8)]

    wbytes = nblk * 210
    us = timed(head(ops), 2)
    out = {"rows": rows, "k": k, "us": us, "gbs": wbytes / us / 1e3, "frac": wbytes / us / 1e3 / peak,
           "topk": topk, "topk_us": timed(select(ops), 8)}
    if ref is not None:
        out["reference_cuda_us"] = timed(head(ref), 2)
        out["reference_cuda_topk_us"] = timed(select(ref), 8)
    return out


def run_gemv_bench(args, device):
    print(json.dumps(gemv_measure(args, device)))


def gemv_config_leg(args, device):
    """config[1] inside the default line: all five shapes at batch 1 and 4, with the reference's own
    CUDA kernels timed on the same buffers."""
    line = gemv_measure(args, device, sampler=False)
    keys = ("rows", "k", "batch", "us", "gbs", "frac", "reference_cuda_us")
    return {"workload": line["config"]["workload"], "lm_head_gbs": line["value"], "lm_head_frac": line["roofline"]["frac"],
            "sweep": [{k: r[k] for k in keys if k in r} for r in line["sweep"]],
            "q6k_head": line.get("q6k_head")}


def run_tc_bench(args, device):
    """The fp16 tensor-core GEMM behind the tc_* entries on the prefill shapes: one projection
    over a whole 2048-row chunk and over the 64 rows one expert gets (the reference issues one
    GEMM per expert and matrix). Operands beyond L2 by rotating over copies."""
    import torch
    from sager_b200 import lib, ops
    peak_bw, kind = load_peaks()
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    peak_tf = float(peaks.get("bf16_tflops", 1590.0))
    out = []
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    tc_shapes = [(512, 2048, 2048), (2048, 512, 2048), (512, 2048, 64), (2048, 512, 64)]
    if args.shape:
        tc_shapes = [tuple(int(v) for v in args.shape.split(","))]
    for rows, k, tok in tc_shapes:
        copies = max(2, min(128, (192 << 20) // (rows * k * 2) + 1))
        g = torch.Generator(device=device).manual_seed(SEED + rows + tok)
        w = (torch.randn(copies, rows, k, generator=g, device=device) * 0.02).half()
        x = torch.randn(tok, k, generator=g, device=device).half()
        y = torch.zeros(tok, rows, dtype=torch.float16, device=device)

        def timed(sweep):
            sweep()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                sweep()
            for _ in range(max(args.warmup, 3)):
                graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / (args.steps * copies)

        us = timed(lambda: [ops.tc_gemm_f16_raw(w[c], x, y, rows, k, tok) for c in range(copies)])
        # what the reference calls at this point (cublasGemmEx, fp16 operands, fp32 accumulate,
        # src/kernels/cuda/tc_gemm.cu:193-199), reached through torch: a baseline, not on any product path
        y_lib = torch.zeros(tok, rows, dtype=torch.float16, device=device)
        lib_us = timed(lambda: [torch.mm(x, w[c].t(), out=y_lib) for c in range(copies)])
        flops = 2.0 * rows * k * tok
        nbytes = 2.0 * (rows * k + tok * k + tok * rows)
        out.append({"rows": rows, "k": k, "tokens": tok, "us": us, "tflops": flops / us / 1e6,
                    "tensor_frac": flops / us / 1e6 / peak_tf, "gbs": nbytes / us / 1e3,
                    "hbm_frac": nbytes / us / 1e3 / peak_bw, "weight_copies": copies,
                    "library_gemm_us": lib_us})
    clocks = sampler.stop()
    head = out[0]
    line = {
        "metric": "tc_gemm_f16_tflops", "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": head["us"] * 1e-3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp16 operands, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "tc_gemm_f16_raw on the prefill projection shapes; value = 512x2048 weights, 2048 rows",
                   "l2": "every launch reads another weight copy"},
        "e2e": None, "gpu_launches": args.steps * sum(r["weight_copies"] for r in out), "clocks": clocks,
        "roofline": {"kernel": "tc_gemm_kernel", "bound": "tensor", "achieved": head["tflops"], "peak": peak_tf,
                     "unit": "TFLOP/s", "frac": head["tensor_frac"],
                     "peak_source": "measured bf16 GEMM (burst)" if peaks else "fallback", "traffic": None},
        "shapes": out,
    }
    if lib().raw("sgr_status")(0) != 0:
        line["device_status"] = "a bounded device-side wait gave up"
    print(json.dumps(line))


def main():
    global LAYERS, TOKENS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true",
                    help="decode: skip the `configs` block (1 and 4 token rows, GEMV sweep points, prefill chunk)")
    ap.add_argument("--no-gpu-baseline", action="store_true",
                    help="skip the leg that times the reference's own CUDA kernels on this GPU")
    ap.add_argument("--layers", type=int, default=LAYERS, help="shrink the stack (profiling captures)")
    ap.add_argument("--tokens", type=int, default=TOKENS, help="token rows per step, 1..64")
    ap.add_argument("--check", action="store_true",
                    help="N > 1: compare one step with the single-GPU layer stack on rank 0 (use with a small --layers)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "gemv", "tc"],
                    help="decode: the 40-layer stack (default); prefill: one layer over a 2048-row chunk; "
                         "gemv: the dense GEMV sweep; tc: the fp16 tensor-core GEMM of the tc_* entries")
    ap.add_argument("--kernel", default=None, choices=["rows", "items", "two_launch"],
                    help="decode: force the row-streaming or the item expert kernel (default: the library's choice)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--chain", action="store_true",
                    help="decode: every layer's input rows are rmsnorm_quant_f16 of the residual its predecessor "
                         "wrote (one more launch per layer) instead of pre-drawn matrices")
    ap.add_argument("--shape", default=None, help="gemv workload: only this ROWS,K shape, or q6head; tc workload: ROWS,K,TOKENS (profiling captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    LAYERS, TOKENS = args.layers, args.tokens

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from sager_b200 import lib
    from sager_b200.layer import MoeStack

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    lib()                                              # fails loudly when the .so is missing
    device = f"cuda:{local_rank}"
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(device))

    if args.workload == "prefill":
        if world == 1:
            run_prefill_bench(args, device)
        return
    if args.workload == "gemv":
        if world == 1:
            run_gemv_bench(args, device)
        return
    if args.workload == "tc":
        if world == 1:
            run_tc_bench(args, device)
        return
    if world > 1:
        from sager_b200.ep import run_ep_bench
        line = run_ep_bench(args, rank, world, device)
        if rank == 0:
            print(json.dumps(line))
        dist.destroy_process_group()
        return

    ws, inputs, x0, biases, alpha = build_workload(device, rank, world, LAYERS, TOKENS)
    n = TOKENS
    sampler = ClockSampler(local_rank)
    sampler.start()                      # runs across every timed region of this process
    main_leg = decode_leg(ws, inputs, x0, biases, n, args, device, e2e=True, chain=args.chain)
    ms_step, value, e2e, roofline = main_leg["ms_step"], main_leg["value"], main_leg["e2e"], main_leg["roofline"]

    line = {
        "metric": "q4k_moe_decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 dots, fp32 accumulate",
        "data": "synthetic",
        "config": dict(workload_config(1), layers=LAYERS, tokens=n, zipf_alpha=alpha, hot20_share=main_leg["hot"],
                       distinct_experts_per_layer=main_leg["uniq_mean"]),
        "e2e": e2e, "gpu_launches": main_leg["launches_per_step"] * args.steps,
        "roofline": roofline,
    }
    if not args.no_configs and n == 64 and LAYERS == 40:
        # the other configurations of the benchmark, measured in the same run (a few seconds each)
        cfgs = {}
        for name, tok, use_bias in (("tokens1", 1, False), ("tokens4", 4, True)):
            try:
                leg = decode_leg(ws, inputs, x0, biases if use_bias else None, tok, args, device, e2e=False)
                cfgs[name] = {
                    "workload": ("one token row through the 40-layer stack (the single-token layer x 40)" if tok == 1 else
                                 "verify window: 4 token rows through the 40-layer stack, Zipf-skewed routing"),
                    "tokens_per_s": leg["value"], "ms_per_step": leg["ms_step"], "us_per_layer": leg["ms_step"] * 1e3 / LAYERS,
                    "distinct_experts_per_layer": leg["uniq_mean"],
                    "step_frac_of_hbm_peak": leg["roofline"]["step"]["frac"],
                    "expert_kernel": leg["roofline"]["kernel"], "expert_kernel_frac": leg["roofline"]["frac"],
                    "expert_kernel_us": leg["roofline"]["us_per_launch"],
                    "stage_ms_per_step": leg["roofline"]["stage_ms_per_step"]}
            except Exception as exc:
                cfgs[name] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
        try:
            # the same step with a true dependency between layers (input rows = RMSNorm of the residual)
            leg = decode_leg(ws, inputs, x0, biases, n, args, device, e2e=False, chain=True)
            cfgs["chained"] = {
                "workload": "the headline step with every layer's input computed from its predecessor's residual "
                            "by rmsnorm_quant_f16 (3 launches per layer)",
                "tokens_per_s": leg["value"], "ms_per_step": leg["ms_step"],
                "distinct_experts_per_layer": leg["uniq_mean"]}
            del leg
        except Exception as exc:
            cfgs["chained"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
        for name, fn in (("gemv", gemv_config_leg), ("prefill", prefill_config_leg)):
            try:
                cfgs[name] = fn(args, device)
            except Exception as exc:
                cfgs[name] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
        line["configs"] = cfgs
    line["clocks"] = sampler.stop()
    if lib().raw("sgr_status")(0) != 0:
        line["device_status"] = "a bounded device-side wait gave up"
    if not args.no_cpu_baseline:
        res = cpu_pool_sample(ws[0], inputs[0], biases[0])
        line["cpu_baseline"] = cpu_baseline_entry(res, n)
    if not args.no_gpu_baseline:
        stack = main_leg["stack"]
        stack.x.copy_(x0[:n])
        stack.replay()
        torch.cuda.synchronize()
        try:
            gpu_ref = ref_cuda_decode(ws, inputs, x0, biases, n, device, max(3, min(args.steps, 10)), stack.x)
        except Exception as exc:                      # a baseline, never a reason to lose the line
            gpu_ref = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
        if gpu_ref is not None:
            line["gpu_baseline"] = gpu_ref
    print(json.dumps(line))


def decode_leg(ws, inputs, x0, biases, n, args, device, e2e, chain=False):
    """One decode measurement over the layer stack with n token rows: graph-replayed steps with
    the inputs resident (value), optionally the same through host buffers (e2e), and each stage of
    all layers back to back (the roofline of the expert kernel)."""
    import torch
    from sager_b200 import synth
    from sager_b200.layer import MoeStack
    layers = len(ws)
    stack = MoeStack(ws, n, K, device, biases=biases, inputs=inputs, per_layer_ws=True, kernel=args.kernel,
                     chain=chain)
    stack.x.copy_(x0[:n])
    stack.capture(n)

    def step():
        stack.x.copy_(x0[:n], non_blocking=True)
        stack.replay()

    def timed(fn, reps):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    for _ in range(args.warmup):
        step()
    ms_step = timed(step, args.steps)
    out = {"stack": stack, "ms_step": ms_step, "value": n / (ms_step * 1e-3),
           "launches_per_step": stack.launches_per_step, "e2e": None}

    if e2e:
        # host buffers in, host buffer out: the 40 layer inputs and the residual rows come from
        # pinned host memory every step, the result goes back
        h_in = torch.empty(layers + 1, n, H, dtype=torch.float16).pin_memory()
        h_in[0].copy_(x0[:n].cpu())
        for li in range(layers):
            h_in[li + 1].copy_(inputs[li][:n].cpu())
        d_in = torch.empty(layers + 1, n, H, dtype=torch.float16, device=device)
        h_out = torch.empty(n, H, dtype=torch.float16).pin_memory()

        def e2e_step():
            d_in.copy_(h_in, non_blocking=True)
            stack.x.copy_(d_in[0], non_blocking=True)
            for li in range(layers):
                inputs[li][:n].copy_(d_in[li + 1], non_blocking=True)     # the graph reads inputs[l] in place
            stack.replay()
            h_out.copy_(stack.x, non_blocking=True)

        for _ in range(3):
            e2e_step()
        ms_e2e = timed(e2e_step, args.steps)
        out["e2e"] = {"value": n / (ms_e2e * 1e-3), "unit": "tokens/s",
                      "h2d_bytes_per_step": int(h_in.numel() * 2), "d2h_bytes_per_step": int(h_out.numel() * 2)}

    # ---- roofline of the dominant kernel: the expert kernel of every layer, back to back ----
    idx = stack.idx.cpu().numpy()[:, :n, :K]
    uniq = [len(np.unique(idx[li])) for li in range(layers)]
    ex_bytes = sum((u + 1) * EXPERT_BYTES for u in uniq)
    step_bytes = sum((u + 1) * EXPERT_BYTES + ROUTER_BYTES for u in uniq)
    peak, peak_kind = load_peaks()
    if args.kernel is None and n <= 3:
        # one persistent launch per layer does everything (router, selection, experts, combine): the
        # launch is the layer, timed inside the step; its algorithmic bytes include the router matrix
        gbs = step_bytes / (ms_step * 1e-3) / 1e9
        out["roofline"] = {"kernel": "token_layer_kernel", "bound": "hbm", "achieved": gbs, "peak": peak,
                           "unit": "GB/s", "frac": gbs / peak, "peak_source": f"{peak_kind} copy bandwidth (burst)",
                           "frac_of_nominal_8tbs": gbs / 8000.0,
                           "traffic": traffic_per_launch("token_layer_kernel", step_bytes / layers)[0],
                           "traffic_source": traffic_per_launch("token_layer_kernel", step_bytes / layers)[1],
                           "bytes_per_launch": step_bytes / layers, "us_per_launch": ms_step * 1e3 / layers,
                           "stage_ms_per_step": {"layer": ms_step},
                           "step": {"algorithmic_bytes": step_bytes, "gbs": gbs, "frac": gbs / peak}}
    else:
        stage_ms = {}
        for name, mask in (("route", 1), ("experts", 6)):
            g = stack.capture_stage(n, mask)          # that stage of all layers, back to back
            g.replay()
            stage_ms[name] = timed(g.replay, 5)
        ex_gbs = ex_bytes / (stage_ms["experts"] * 1e-3) / 1e9
        use_rows = args.kernel == "rows" or (args.kernel in (None, "two_launch") and n >= 4)
        kernel = "expert_rows_kernel" if use_rows else "expert_stream_kernel"
        traffic, traffic_source = traffic_per_launch(kernel, ex_bytes / layers)
        out["roofline"] = {"kernel": kernel, "bound": "hbm", "achieved": ex_gbs, "peak": peak,
                           "unit": "GB/s", "frac": ex_gbs / peak, "peak_source": f"{peak_kind} copy bandwidth (burst)",
                           "frac_of_nominal_8tbs": ex_gbs / 8000.0,
                           "traffic": traffic, "traffic_source": traffic_source,
                           "bytes_per_launch": ex_bytes / layers, "us_per_launch": stage_ms["experts"] * 1e3 / layers,
                           "stage_ms_per_step": stage_ms,
                           "step": {"algorithmic_bytes": step_bytes, "gbs": step_bytes / (ms_step * 1e-3) / 1e9,
                                    "frac": step_bytes / (ms_step * 1e-3) / 1e9 / peak}}
    out["uniq_mean"] = float(np.mean(uniq))
    out["hot"] = float(np.mean([synth.hot_share(idx[li], E) for li in range(layers)]))
    return out


def traffic_per_launch(kernel, algorithmic_bytes):
    """DRAM bytes per launch of `kernel` from the ncu capture recorded in profiles/traffic.json
    (dram__bytes_read.sum + dram__bytes_write.sum of a smaller case of the same kernel), scaled to
    this run's launch by the algorithmic bytes; (None, reason) when no capture of it is recorded."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        rec = json.load(open(path))[kernel]
        scale = (rec["dram_read_bytes"] + rec["dram_write_bytes"]) / rec["algorithmic_bytes"]
        return scale * algorithmic_bytes, f"profiles/traffic.json: {rec['source']}; scaled by algorithmic bytes"
    except (OSError, KeyError, ValueError):
        return None, "no ncu capture of this kernel is recorded in profiles/traffic.json"


if __name__ == "__main__":
    main()
