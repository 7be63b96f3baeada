"""Writes tests/golden/ref_cpu_golden.npz from the reference's own CPU code.

Run in a container that has the reference tree (it needs oracle/_ref/
libsager_ref.so, built by `make -C oracle ref`):

    python tests/golden/make_golden.py

Every array below is an input drawn from a seeded numpy generator or an output
of a reference function called through oracle/ref_wrap.cpp:
  q4k::quantize_row, q4k::quantize_row_q8_K, q4k::dequant_row, q4k::vec_dot_ref,
  cpu::gemv_q4_k_q8_avx2 / _scalar, cpu::expert_ffn_q4.
The file pins oracle/sager_oracle.c (tests/test_oracle.py) and the CUDA
kernels (tests/test_gpu_*.py) where the reference tree is not available.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.oracle import Reference  # noqa: E402

SEED = 20260718


def main():
    ref = Reference()
    rng = np.random.default_rng(SEED)
    out = {}

    # GEMV case: 48 rows x k=2048, two activation rows (fp16-representable).
    rows, k = 48, 2048
    w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((2, k)).astype(np.float16).astype(np.float32)
    wq = ref.quantize_q4k(w)
    xq = ref.quantize_q8k(x)
    out["gemv_w_f32"] = w[:4].copy()            # first rows only: quantiser spot check
    out["gemv_wq"] = wq
    out["gemv_x"] = x
    out["gemv_xq"] = xq
    out["gemv_y_avx2"] = np.stack([ref.gemv(wq, xq[t], rows, k) for t in range(2)])
    out["gemv_y_scalar"] = np.stack([ref.gemv(wq, xq[t], rows, k, scalar=True) for t in range(2)])
    out["gemv_vec_dot_ref"] = np.array(
        [ref.vec_dot_ref(wq[r], xq[0], k) for r in range(rows)], dtype=np.float32)
    out["gemv_dequant_row0"] = ref.dequant(wq[0], k)

    # Expert FFN case: H=512, FFX=256 (two super-blocks per gate/up row).
    hdim, ffx = 512, 256
    xg = (rng.standard_normal(hdim)).astype(np.float16).astype(np.float32)
    wg = ref.quantize_q4k((rng.standard_normal((ffx, hdim)) * 0.05).astype(np.float32))
    wu = ref.quantize_q4k((rng.standard_normal((ffx, hdim)) * 0.05).astype(np.float32))
    wd = ref.quantize_q4k((rng.standard_normal((hdim, ffx)) * 0.05).astype(np.float32))
    out["ffn_x"] = xg
    out["ffn_wg"], out["ffn_wu"], out["ffn_wd"] = wg, wu, wd
    out["ffn_y"] = ref.expert_ffn(wg, wu, wd, xg, hdim, ffx)

    # Q8_K edge rows: zeros, a single spike, +-amax ties, tiny values.
    e = np.zeros((4, 256), dtype=np.float32)
    e[1, 17] = 3.0
    e[2, :] = np.where(np.arange(256) % 2 == 0, 1.5, -1.5)
    e[3, :] = (rng.standard_normal(256) * 1e-6).astype(np.float16).astype(np.float32)
    out["q8_edge_x"] = e
    out["q8_edge_q"] = ref.quantize_q8k(e)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cpu_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
