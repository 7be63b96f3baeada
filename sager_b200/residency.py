"""Host-side mirror of the reference's residency plumbing - `HotTier::rebuild`
(src/core/layer.cpp:21-109), the arena of `ExpertPump` (src/core/expert_pump.cpp:130-216) and
`Session::build_decode_table` (src/core/session.cpp:3569-3627) - over the library's residency
handle. All buffers are the caller's; with `host_only` they are numpy arrays and no GPU is touched."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .capi import SagerError, lib


def _addr(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return C.c_void_p(a.ctypes.data)
    return C.c_void_p(a.data_ptr())            # a torch tensor


class Residency:
    def __init__(self, n_layers, n_experts, hidden, n_ff, slab_experts, arena_slots):
        self.L, self.E = n_layers, n_experts
        self.expert_bytes = lib().raw("sgr_expert_bytes")(hidden, n_ff)
        self._h = C.c_void_p()
        rc = lib().raw("sgr_residency_create")(n_layers, n_experts, hidden, n_ff, slab_experts, arena_slots,
                                               C.byref(self._h))
        if rc != 0:
            raise SagerError("sgr_residency_create", rc)
        self._keep = None

    def close(self):
        if self._h:
            lib().raw("sgr_residency_destroy")(self._h)
            self._h = C.c_void_p()

    def bind(self, host_pool, slab, arena, table, copy_stream=None, host_only=False):
        """host_pool: every expert at (l * E + e) * expert_bytes; slab / arena / table: device buffers
        (torch tensors) or, with host_only, numpy arrays. `table` holds 3 * L * E pointers, [3][L][E]."""
        self._keep = (host_pool, slab, arena, table)
        lib().call("sgr_residency_bind", self._h, _addr(host_pool), _addr(slab), _addr(arena), _addr(table),
                   C.c_void_p(copy_stream) if copy_stream else None, int(host_only))

    def set_resident(self, layer, expert, on=True):
        lib().call("sgr_residency_set_resident", self._h, layer, expert, int(on))

    def rebuild(self, stream=None) -> int:
        n = C.c_int()
        lib().call("sgr_residency_rebuild", self._h, C.c_void_p(stream) if stream else None, C.byref(n))
        return n.value

    def submit(self, layer, expert, step) -> int:
        return lib().raw("sgr_residency_submit")(self._h, layer, expert, step)

    def wait(self, slot, stream):
        lib().call("sgr_residency_wait", self._h, slot, C.c_void_p(stream) if stream else None)

    def clear_arena(self):
        lib().call("sgr_residency_clear_arena", self._h)

    def build_decode_table(self, stream=None) -> int:
        n = C.c_int()
        lib().call("sgr_residency_build_decode_table", self._h, C.c_void_p(stream) if stream else None, C.byref(n))
        return n.value

    def stat(self, what) -> int:
        return lib().raw("sgr_residency_stat")(self._h, what)

    def absent(self, layer) -> int:
        return self.stat(8 + layer)

    def where(self, layer, expert) -> int:
        return lib().raw("sgr_residency_where")(self._h, layer, expert)

    def host_table(self, which=0) -> np.ndarray:
        """which 0: the decode table [3][L][E]; 1: the hot tier's tables [L][3][E] (addresses as uint64)."""
        p = lib().raw("sgr_residency_host_table")(self._h, which)
        buf = (C.c_uint64 * (3 * self.L * self.E)).from_address(p)
        a = np.frombuffer(buf, dtype=np.uint64).copy()
        return a.reshape(3, self.L, self.E) if which == 0 else a.reshape(self.L, 3, self.E)
