"""The reference's launcher names on torch device tensors.

`ops.<name>(...)` calls `sgr_<name>` of the C ABI with the same argument order
as `sager::cuda::<name>` (include/sager/kernels/cuda_ops.hpp of the reference);
tensors are passed as raw device pointers and the trailing stream argument is
torch's current stream. Nothing here computes: a missing library raises.
"""
from __future__ import annotations

import ctypes as C

import torch

from .capi import lib


def _conv(a):
    if a is None:
        return None
    if isinstance(a, torch.Tensor):
        return C.c_void_p(a.data_ptr())
    if isinstance(a, int) and a > 0x7FFFFFFF:
        return C.c_void_p(a)                 # a raw device address
    return a


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def call(name: str, *args):
    lib().call("sgr_" + name, *[_conv(a) for a in args], stream_ptr())


def __getattr__(name):
    if name.startswith("_"):
        raise AttributeError(name)
    protos = lib().protos
    if "sgr_" + name not in protos:
        raise AttributeError(f"no entry point sgr_{name}")

    def fn(*args):
        call(name, *args)

    fn.__name__ = name
    return fn


def ptr_table(tensors, device):
    """int64 device tensor of data pointers (0 for None)."""
    return torch.tensor([0 if t is None else t.data_ptr() for t in tensors], dtype=torch.int64,
                        device=device)
