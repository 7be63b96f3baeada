"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from sager_b200 import synth

DEV = "cuda:0"

# fp32 outputs: the kernels sum the same exact integer dots as the oracle in a
# different order, so they agree to fp32 rounding. The north-star bound for layer
# outputs is 1e-3 max relative error; single GEMVs are held to a much tighter one.
GEMV_TOL = 2e-5
LAYER_TOL = 1e-3


def rel(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV)


def make_q4k(rows, k, seed, std=0.02):
    """uint8 [rows, k/256*144] Q4_K weights, numpy (CPU) and torch (GPU) copies."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    q = torch.empty(rows, k // 256 * 144, dtype=torch.uint8, device=DEV)
    step = max(1, (1 << 24) // k)                 # bound the fp32 temporaries
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        q[r0:r1] = synth.quantize_q4k(torch.randn(r1 - r0, k, generator=g, device=DEV) * std)
    return q.cpu().numpy(), q


def make_x16(n, k, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(n, k, generator=g) * std).half()
    return x.numpy(), x.to(DEV)


def f16_ulp_diff(a_u16, b_u16):
    """Max distance in fp16 representable steps between two uint16 bit patterns."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return int(np.abs(key(np.asarray(a_u16).view(np.uint16)) - key(np.asarray(b_u16).view(np.uint16))).max())


def f16_close(got_f16, want_f32, tol=GEMV_TOL):
    """fp16 outputs of an fp32 computation: within one fp16 step of the oracle's fp32
    value, plus the fp32 tolerance relative to the largest output (values near zero
    come from cancellation and carry the absolute error of the large terms)."""
    got = np.asarray(got_f16).view(np.float16).astype(np.float64).reshape(-1)
    want = np.asarray(want_f32, dtype=np.float64).reshape(-1)
    step = np.spacing(np.abs(want).astype(np.float16)).astype(np.float64)
    bound = step + tol * np.abs(want).max()
    return bool(np.all(np.abs(got - want) <= bound))
