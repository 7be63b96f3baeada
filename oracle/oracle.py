"""ctypes access to the parity checkers (test infrastructure, not product code).

``Oracle()`` loads ``oracle/libsager_oracle.so`` (the C restatement in
``sager_oracle.c``); ``Reference()`` loads ``oracle/_ref/libsager_ref.so`` (the
reference's own CPU sources compiled by ``oracle/Makefile``) and raises
``FileNotFoundError`` when that build is not present. Only tests, the smoke
check and the CPU-baseline legs of the benchmark may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
Q4K_BYTES = 144
Q8K_BYTES = 276
QK_K = 256

_vp = C.c_void_p
_i = C.c_int
_f = C.c_float


def reference_root() -> str:
    """Where the reference's source tree lies: $SAGER_REFERENCE, else a directory named
    `reference` beside this repository."""
    return os.environ.get("SAGER_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root: str | None = None) -> None:
    """Compile the C restatement and, when the reference tree is present, the
    reference's own CPU sources."""
    ref_root = ref_root or reference_root()
    subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
    if os.path.isdir(ref_root):
        subprocess.check_call(["make", "-s", "-C", HERE, "ref", f"REF={ref_root}"],
                              stderr=subprocess.DEVNULL)
        subprocess.check_call(["make", "-s", "-C", HERE, "refcuda", f"REF={ref_root}"],
                              stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "array must be C-contiguous"
    return a.ctypes.data_as(_vp)


def _u8(a):
    return np.ascontiguousarray(a).view(np.uint8).reshape(-1)


class _Lib:
    def __init__(self, path, sigs):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        for name, (res, args) in sigs.items():
            fn = getattr(self.lib, name)
            fn.restype = res
            fn.argtypes = args


_ORC_SIGS = {
    "orc_half_to_float": (_f, [C.c_uint16]),
    "orc_float_to_half_rn": (C.c_uint16, [_f]),
    "orc_float_to_half_trunc": (C.c_uint16, [_f]),
    "orc_get_scale_min_k4": (None, [_i, _vp, _vp, _vp]),
    "orc_set_scale_min_k4": (None, [_i, _vp, C.c_uint8, C.c_uint8]),
    "orc_dequant_row": (None, [_vp, _vp, _i]),
    "orc_quantize_row_q8k": (None, [_vp, _vp, _i]),
    "orc_quantize_row_q8k_f16": (None, [_vp, _vp, _i]),
    "orc_quantize_row_q4k": (None, [_vp, _vp, _i]),
    "orc_subblock_dots": (None, [_vp, _vp, _vp, _i, _i]),
    "orc_vec_dot_ref": (_f, [_vp, _vp, _i]),
    "orc_gemv_q4k_q8k": (None, [_vp, _vp, _vp, _i, _i]),
    "orc_gemv_q4k_q8k_lane_order": (None, [_vp, _vp, _vp, _i, _i]),
    "orc_expert_ffn_q4": (None, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "orc_router_logits": (None, [_vp, _vp, _vp, _i, _i]),
    "orc_router_topk": (None, [_vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "orc_dispatch_scan": (None, [_vp] * 7 + [_i] * 4),
    "orc_silu_mul_f16": (None, [_vp, _vp, _vp, _i]),
    "orc_combine_f16": (None, [_vp, _vp, _vp, _vp, _i, _i]),
    "orc_combine_batched_f16": (None, [_vp, _vp, _vp, _i, _i, _i]),
    "orc_moe_layer": (None, [_vp] * 9 + [_i] * 5 + [_f, _i]),
    "orc_expert_ffn_batch": (None, [_vp, _vp, _vp, _i, _i, _i, _i]),
}

_REF_SIGS = {
    "ref_have_avx2": (_i, []),
    "ref_half_to_float": (_f, [C.c_uint16]),
    "ref_float_to_half": (C.c_uint16, [_f]),
    "ref_get_scale_min_k4": (None, [_i, _vp, _vp, _vp]),
    "ref_set_scale_min_k4": (None, [_i, _vp, C.c_uint8, C.c_uint8]),
    "ref_dequant_row": (None, [_vp, _vp, _i]),
    "ref_quantize_row_q4k": (None, [_vp, _vp, _i]),
    "ref_quantize_row_q8k": (None, [_vp, _vp, _i]),
    "ref_quantize_row_q8k_avx2": (None, [_vp, _vp, _i]),
    "ref_vec_dot_ref": (_f, [_vp, _vp, _i]),
    "ref_gemv_q4k_q8k_avx2": (None, [_vp, _vp, _vp, _i, _i]),
    "ref_gemv_q4k_q8k_scalar": (None, [_vp, _vp, _vp, _i, _i]),
    "ref_expert_ffn_q4": (None, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "ref_validate_pool_geometry": (_i, [_i] * 8),
    "ref_pool_create": (_vp, [_i, _i, _i, _i]),
    "ref_pool_destroy": (None, [_vp]),
    "ref_pool_run": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
}


def _ptr_array(arrays):
    """A C array of void* from numpy arrays / ints / None (kept alive by caller)."""
    out = (_vp * len(arrays))()
    for j, a in enumerate(arrays):
        if a is None:
            out[j] = None
        elif isinstance(a, (int, np.integer)):
            out[j] = int(a)
        else:
            out[j] = a.ctypes.data
    return out


class _Common:
    """Array-level helpers shared by the restatement and the reference build;
    ``p`` is the symbol prefix."""

    p = ""

    def _fn(self, name):
        return getattr(self.lib, self.p + name)

    def quantize_q4k(self, w: np.ndarray) -> np.ndarray:
        """fp32 [rows, k] (k % 256 == 0) -> uint8 [rows, k/256*144]."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        rows, k = w.shape
        out = np.zeros((rows, k // QK_K * Q4K_BYTES), dtype=np.uint8)
        self._fn("quantize_row_q4k")(_ptr(w), _ptr(out), rows * k)
        return out

    def quantize_q8k(self, x: np.ndarray) -> np.ndarray:
        """fp32 [rows, k] -> uint8 [rows, k/256*276]."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, k = x.shape
        out = np.zeros((rows, k // QK_K * Q8K_BYTES), dtype=np.uint8)
        self._fn("quantize_row_q8k")(_ptr(x), _ptr(out), rows * k)
        return out

    def dequant(self, blocks: np.ndarray, n: int) -> np.ndarray:
        out = np.zeros(n, dtype=np.float32)
        self._fn("dequant_row")(_ptr(_u8(blocks)), _ptr(out), n)
        return out

    def vec_dot_ref(self, w, xq, n):
        return float(self._fn("vec_dot_ref")(_ptr(_u8(w)), _ptr(_u8(xq)), n))

    def expert_ffn(self, wg, wu, wd, x, hidden, n_ff):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.zeros(hidden, dtype=np.float32)
        scratch = np.zeros(2 * n_ff, dtype=np.float32)
        self._fn("expert_ffn_q4")(_ptr(_u8(wg)), _ptr(_u8(wu)), _ptr(_u8(wd)), _ptr(x), _ptr(y),
                                  _ptr(scratch), hidden, n_ff)
        return y


class Oracle(_Common, _Lib):
    p = "orc_"

    def __init__(self):
        _Lib.__init__(self, os.path.join(HERE, "libsager_oracle.so"), _ORC_SIGS)

    def half_to_float(self, h):
        h = np.asarray(h, dtype=np.uint16)
        return h.view(np.float16).astype(np.float32)

    def quantize_q8k_f16(self, x16: np.ndarray) -> np.ndarray:
        x16 = np.ascontiguousarray(x16).view(np.uint16)
        rows, k = x16.shape
        out = np.zeros((rows, k // QK_K * Q8K_BYTES), dtype=np.uint8)
        self.lib.orc_quantize_row_q8k_f16(_ptr(x16), _ptr(out), rows * k)
        return out

    def subblock_dots(self, w, xq, n_rows, k) -> np.ndarray:
        out = np.zeros((n_rows, k // QK_K, 8), dtype=np.int32)
        self.lib.orc_subblock_dots(_ptr(_u8(w)), _ptr(_u8(xq)), _ptr(out), n_rows, k)
        return out

    def gemv(self, w, xq, n_rows, k, lane_order=False) -> np.ndarray:
        y = np.zeros(n_rows, dtype=np.float32)
        fn = self.lib.orc_gemv_q4k_q8k_lane_order if lane_order else self.lib.orc_gemv_q4k_q8k
        fn(_ptr(_u8(w)), _ptr(_u8(xq)), _ptr(y), n_rows, k)
        return y

    def router_logits(self, w, x16) -> np.ndarray:
        w = np.ascontiguousarray(w, dtype=np.float32)
        x16 = np.ascontiguousarray(x16).view(np.uint16)
        y = np.zeros(w.shape[0], dtype=np.float32)
        self.lib.orc_router_logits(_ptr(w), _ptr(x16), _ptr(y), w.shape[0], w.shape[1])
        return y

    def router_topk(self, logits, k, shared_w=1.0, write_shared=True):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        e = logits.shape[0]
        idx = np.full(k + 1, -7, dtype=np.int32)
        w = np.full(k + 1, -7.0, dtype=np.float32)
        prob = np.zeros(e, dtype=np.float32)
        self.lib.orc_router_topk(_ptr(logits), _ptr(idx), _ptr(w), e, k, shared_w,
                                 1 if write_shared else 0, _ptr(prob))
        return idx, w

    def dispatch_scan(self, idx, weight, n_rows, k, n_expert, tok_per):
        """idx int32 [n_rows, k+1]; weight float32 [n_rows, k+1] (mutated copy returned)."""
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        weight = np.array(weight, dtype=np.float32, copy=True)
        gslot = np.full(n_rows * k, -9, dtype=np.int32)
        grows = np.full(n_rows * k, -9, dtype=np.int32)
        off = np.zeros(n_expert + 1, dtype=np.int32)
        toff = np.zeros(n_expert + 1, dtype=np.int32)
        meta = np.zeros(4, dtype=np.int32)
        self.lib.orc_dispatch_scan(_ptr(idx), _ptr(weight), _ptr(gslot), _ptr(grows), _ptr(off),
                                   _ptr(toff), _ptr(meta), n_rows, k, n_expert, tok_per)
        return dict(weight=weight, gslot=gslot, grows=grows, off=off, toff=toff, meta=meta)

    def silu_mul_f16(self, g16, u16):
        g16 = np.ascontiguousarray(g16).view(np.uint16)
        u16 = np.ascontiguousarray(u16).view(np.uint16)
        out = np.zeros_like(g16)
        self.lib.orc_silu_mul_f16(_ptr(out), _ptr(g16), _ptr(u16), g16.size)
        return out

    def combine_f16(self, out16, expert_out16, idx, weight, k, hidden):
        out = np.array(np.ascontiguousarray(out16).view(np.uint16), copy=True)
        self.lib.orc_combine_f16(_ptr(out), _ptr(np.ascontiguousarray(expert_out16).view(np.uint16)),
                                 _ptr(np.ascontiguousarray(idx, dtype=np.int32)),
                                 _ptr(np.ascontiguousarray(weight, dtype=np.float32)), k, hidden)
        return out

    def combine_batched_f16(self, out16, expert_y16, weight, n_used, hidden, n_rows):
        out = np.array(np.ascontiguousarray(out16).view(np.uint16), copy=True)
        self.lib.orc_combine_batched_f16(
            _ptr(out), _ptr(np.ascontiguousarray(expert_y16).view(np.uint16)),
            _ptr(np.ascontiguousarray(weight, dtype=np.float32)), n_used, hidden, n_rows)
        return out

    def moe_layer(self, x16, router_w, experts, shared, resid, k, n_ff, shared_w=1.0,
                  n_threads=1):
        """experts: list of E entries, each None (absent) or (gate, up, down) uint8 arrays.
        shared: None or (gate, up, down). Returns dict(out, idx, w, logits)."""
        x16 = np.ascontiguousarray(x16).view(np.uint16)
        n, hidden = x16.shape
        router_w = np.ascontiguousarray(router_w, dtype=np.float32)
        n_expert = router_w.shape[0]
        keep = []
        tab = []
        for m in range(3):
            for e in range(n_expert):
                if experts[e] is None:
                    tab.append(None)
                else:
                    a = _u8(experts[e][m])
                    keep.append(a)
                    tab.append(a)
        tab_c = _ptr_array(tab)
        sh_c = None
        if shared is not None:
            sh = [_u8(a) for a in shared]
            keep.extend(sh)
            sh_c = _ptr_array(sh)
        out = np.zeros((n, hidden), dtype=np.float32)
        idx = np.zeros((n, k + 1), dtype=np.int32)
        w = np.zeros((n, k + 1), dtype=np.float32)
        logits = np.zeros((n, n_expert), dtype=np.float32)
        res = None if resid is None else np.ascontiguousarray(resid, dtype=np.float32)
        self.lib.orc_moe_layer(_ptr(x16), _ptr(router_w), tab_c, sh_c, _ptr(res), _ptr(out),
                               _ptr(idx), _ptr(w), _ptr(logits), n, hidden, n_ff, n_expert, k,
                               shared_w, n_threads)
        return dict(out=out, idx=idx, w=w, logits=logits)

    def expert_ffn_batch(self, w3, x, hidden, n_ff, n_threads):
        """w3: flat list of 3*n_jobs uint8 arrays; x fp32 [n_jobs, hidden]."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        n_jobs = x.shape[0]
        y = np.zeros((n_jobs, hidden), dtype=np.float32)
        w3c = _ptr_array([_u8(a) for a in w3])
        self.lib.orc_expert_ffn_batch(w3c, _ptr(x), _ptr(y), n_jobs, hidden, n_ff, n_threads)
        return y


def rmsnorm_quant_f16(oracle, x16: np.ndarray, w16: np.ndarray, eps: float):
    """CPU restatement of the fused RMS norm + Q8_K quantiser of the reference
    (src/kernels/cuda/mmq.cu:533-641): x16 [rows][n] fp16, w16 [n] fp16 ->
    (out fp16 [rows][n], Q8_K blocks uint8 [rows][n/256*276]). The summation order of the
    kernel is followed step for step (that is what fixes the bits): with b = min(1024,
    n rounded up to 32) threads, thread t adds x[t]^2, x[t+b]^2, ... with FMA (the square of
    an fp16 value is exact in fp32, so the FMA equals an fp32 add of the exact square), a warp
    folds with shfl_down 16, 8, 4, 2, 1 (only lane 0's value is used), thread 0 adds the warp
    sums in order; scale = rsqrt(sum / n + eps); out = f16((x * scale) * w). The device's rsqrtf is
    an approximation within 2 ulp of the correctly rounded value used here, so `out` can differ
    from the device's by one fp16 step in a few places; the Q8_K blocks are exactly those of `out`."""
    rows, n = x16.shape
    b = min(1024, (n + 31) // 32 * 32)
    xf = x16.astype(np.float32)
    wf = w16.astype(np.float32)
    out = np.zeros((rows, n), dtype=np.float16)
    f32 = np.float32
    for r in range(rows):
        acc = np.zeros(b, dtype=np.float32)
        for i0 in range(0, n, b):
            seg = xf[r, i0:i0 + b]
            acc[:seg.size] = acc[:seg.size] + seg * seg
        lanes = acc.reshape(b // 32, 32).copy()
        for off in (16, 8, 4, 2, 1):                 # lane l += lane l + off (lanes >= 32 - off keep theirs)
            shifted = np.zeros_like(lanes)
            shifted[:, :32 - off] = lanes[:, off:]
            shifted[:, 32 - off:] = lanes[:, 32 - off:]     # shfl_down past the end returns the lane's own value
            lanes = (lanes + shifted).astype(np.float32)
        s = f32(0)
        for wsum in lanes[:, 0]:
            s = f32(s + wsum)
        scale = f32(1) / np.sqrt(f32(f32(s / f32(n)) + f32(eps)), dtype=np.float32)
        out[r] = ((xf[r] * scale).astype(np.float32) * wf).astype(np.float32).astype(np.float16)
    return out, oracle.quantize_q8k_f16(out)


Q6K_BYTES = 210


def make_q6k(rng: np.random.Generator, rows: int, k: int, d_scale: float = 1e-3) -> np.ndarray:
    """Seeded raw Q6_K rows [rows][k/256*210]: random 6-bit codes and int8 sub-group scales, fp16 block
    scale around d_scale. Any byte pattern is a valid block; both sides consume the same bytes."""
    nb = k // QK_K
    blk = np.zeros((rows, nb, Q6K_BYTES), dtype=np.uint8)
    blk[:, :, :192] = rng.integers(0, 256, size=(rows, nb, 192), dtype=np.uint8)
    blk[:, :, 192:208] = rng.integers(-64, 64, size=(rows, nb, 16)).astype(np.int8).view(np.uint8)
    d = (d_scale * (0.5 + rng.random((rows, nb)))).astype(np.float16)
    blk[:, :, 208:210] = d.view(np.uint8).reshape(rows, nb, 2)
    return blk.reshape(rows, nb * Q6K_BYTES)


def dequant_q6k(w6: np.ndarray, k: int) -> np.ndarray:
    """Raw Q6_K rows -> fp32 [rows][k], the host dequantiser of the reference restated
    (src/core/weights.cpp:168-209): ql[128] | qh[64] | sc int8[16] | d fp16 per 256 weights; in each
    128-weight half, weight l + 32*j (l < 32, j < 4) is ((ql[l + 32*(j&1)] >> 4*(j>>1)) & 15) |
    (((qh[l] >> 2*j) & 3) << 4), minus 32, times d * sc[8*half + l/16 + 2*j]."""
    rows = w6.shape[0]
    nb = k // QK_K
    b = w6.reshape(rows, nb, Q6K_BYTES)
    ql = b[:, :, :128].reshape(rows, nb, 2, 64).astype(np.int32)
    qh = b[:, :, 128:192].reshape(rows, nb, 2, 32).astype(np.int32)
    sc = b[:, :, 192:208].view(np.int8).reshape(rows, nb, 2, 8).astype(np.float32)
    d = b[:, :, 208:210].copy().view(np.float16).reshape(rows, nb).astype(np.float32)
    out = np.zeros((rows, nb, 2, 128), dtype=np.float32)
    for j in range(4):
        lo = (ql[:, :, :, 32 * (j & 1):32 * (j & 1) + 32] >> (4 * (j >> 1))) & 15
        hi = (qh >> (2 * j)) & 3
        q = (lo | (hi << 4)) - 32                                   # [rows][nb][2][32]
        scale = np.repeat(sc[:, :, :, 2 * j:2 * j + 2], 16, axis=3)  # l/16 picks one of two scales
        out[:, :, :, 32 * j:32 * j + 32] = d[:, :, None, None] * scale * q
    return out.reshape(rows, k)


def gemv_q6k_q8k(w6: np.ndarray, xq: np.ndarray, k: int) -> np.ndarray:
    """y[row] = W6[row] . x on Q8_K activations, the arithmetic of the reference's head kernel
    (src/kernels/cuda/q4_k.cu:1578-1658): per 16-weight sub-group t of a block the exact integer
    sums isum = sum q*x and xsum = sum x, term = xd * d * sc[t] * (isum - 32 * xsum), terms added in
    fp32 (here in float64, compared to fp32 rounding)."""
    rows = w6.shape[0]
    nb = k // QK_K
    b = w6.reshape(rows, nb, Q6K_BYTES)
    ql = b[:, :, :128].reshape(rows, nb, 2, 64).astype(np.int64)
    qh = b[:, :, 128:192].reshape(rows, nb, 2, 32).astype(np.int64)
    sc = b[:, :, 192:208].view(np.int8).reshape(rows, nb, 16).astype(np.float64)
    d = b[:, :, 208:210].copy().view(np.float16).reshape(rows, nb).astype(np.float64)
    xb = np.ascontiguousarray(xq).view(np.uint8).reshape(nb, Q8K_BYTES)
    xd = xb[:, :4].copy().view(np.float32).reshape(nb).astype(np.float64)
    xc = xb[:, 4:260].copy().view(np.int8).reshape(nb, 2, 4, 2, 16).astype(np.int64)   # [blk][half][qslot][is][j]
    y = np.zeros(rows, dtype=np.float64)
    for t in range(16):
        n_half, qslot, is_ = t >> 3, (t & 7) >> 1, t & 1
        lo = (ql[:, :, n_half, (qslot & 1) * 32 + is_ * 16:(qslot & 1) * 32 + is_ * 16 + 16] >> (4 if qslot & 2 else 0)) & 15
        hi = (qh[:, :, n_half, is_ * 16:is_ * 16 + 16] >> (2 * qslot)) & 3
        q = lo | (hi << 4)                                           # [rows][nb][16], 0..63
        x = xc[:, n_half, qslot, is_, :]                              # [nb][16]
        isum = (q * x[None]).sum(axis=2)
        xsum = x.sum(axis=1)
        y += (xd[None] * d * sc[:, :, t] * (isum - 32 * xsum[None])).sum(axis=1)
    return y


def topk_select(logits: np.ndarray, k: int):
    """The selection rule of the reference's top-k kernels (src/kernels/cuda/sampling.cu:109-153,
    173-289): k <= 64 largest values in descending order, equal values by ascending index; values
    that are not greater than -3.4e38 (and NaN) never qualify, missing entries are (-3.4e38, -1)."""
    k = min(k, 64)
    none = np.float32(-3.4e38)
    v = np.asarray(logits, dtype=np.float32)
    ok = v > none                                  # False for NaN, -inf and the sentinel
    idx = np.nonzero(ok)[0]
    order = idx[np.lexsort((idx, -v[idx].astype(np.float64)))][:k]
    out_v = np.full(k, none, dtype=np.float32)
    out_i = np.full(k, -1, dtype=np.int32)
    out_v[:order.size] = v[order]
    out_i[:order.size] = order
    return out_v, out_i


class Reference(_Common, _Lib):
    p = "ref_"

    def __init__(self):
        _Lib.__init__(self, os.path.join(HERE, "_ref", "libsager_ref.so"), _REF_SIGS)

    def quantize_q8k_avx2(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, k = x.shape
        out = np.zeros((rows, k // QK_K * Q8K_BYTES), dtype=np.uint8)
        self.lib.ref_quantize_row_q8k_avx2(_ptr(x), _ptr(out), rows * k)
        return out

    def gemv(self, w, xq, n_rows, k, scalar=False):
        y = np.zeros(n_rows, dtype=np.float32)
        fn = self.lib.ref_gemv_q4k_q8k_scalar if scalar else self.lib.ref_gemv_q4k_q8k_avx2
        fn(_ptr(_u8(w)), _ptr(_u8(xq)), _ptr(y), n_rows, k)
        return y

    class Pool:
        """The reference's CpuPool (make_cpu_pool -> start -> submit -> wait_done)."""

        def __init__(self, ref, workers, hidden, n_ff, n_expert):
            self.ref = ref
            self.hidden, self.n_ff = hidden, n_ff
            self.h = ref.lib.ref_pool_create(workers, hidden, n_ff, n_expert)
            if not self.h:
                raise RuntimeError("reference pool refused to start")

        def run(self, w3, x):
            x = np.ascontiguousarray(x, dtype=np.float32)
            n_jobs = x.shape[0]
            y = np.zeros((n_jobs, self.hidden), dtype=np.float32)
            keep = [a if isinstance(a, (int, np.integer)) else _u8(a) for a in w3]
            w3c = _ptr_array(keep)
            got = self.ref.lib.ref_pool_run(self.h, w3c, _ptr(x), _ptr(y), n_jobs, self.hidden,
                                            self.n_ff)
            if got != n_jobs:
                raise RuntimeError(f"reference pool accepted {got} of {n_jobs} jobs")
            return y

        def close(self):
            if self.h:
                self.ref.lib.ref_pool_destroy(self.h)
                self.h = None

    def pool(self, workers, hidden, n_ff, n_expert):
        return Reference.Pool(self, workers, hidden, n_ff, n_expert)
