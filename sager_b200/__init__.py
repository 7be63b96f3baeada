"""sager_b200 - B200 (sm_100a) implementation of SAGER's Q4_K MoE expert hot path.

The product is `libsager_b200.so` (CUDA kernels behind a C ABI, declared in
`include/sager_b200.h`). This package is the thin host side used by tests and
benchmarks: `capi` binds the library, `ops` mirrors the reference's launcher
names on torch device tensors, `layer` drives one MoE layer the way the
reference's session does, `synth` makes seeded synthetic inputs.
"""
from .capi import SagerError, lib  # noqa: F401

__all__ = ["lib", "SagerError"]
