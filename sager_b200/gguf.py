"""Host-side mirror of the reference's container reader and expert-pool loader
(`gguf::File`, include/sager/core/gguf.hpp, and `Weights::load_expert_pool`,
src/core/weights.cpp:730-862) over the library's C entry points. Nothing here parses
or quantises: the library does."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .capi import SagerError, lib

TYPE_NAMES = {0: "F32", 1: "F16", 8: "Q8_0", 12: "Q4_K", 14: "Q6_K", 30: "BF16"}
_ELEM_DTYPES = {0: np.uint8, 1: np.int8, 2: np.uint16, 3: np.int16, 4: np.uint32, 5: np.int32, 6: np.float32,
                7: np.bool_, 10: np.uint64, 11: np.int64, 12: np.float64}


class TensorInfo(C.Structure):
    """struct sgr_gguf_tensor_info of include/sager_b200.h."""
    _fields_ = [("type", C.c_int), ("n_dims", C.c_int), ("dims", C.c_longlong * 4), ("offset", C.c_longlong),
                ("nbytes", C.c_longlong), ("row_bytes", C.c_longlong), ("data", C.c_void_p)]


class File:
    """A GGUF v3 file mapped read-only; tensor data are views into the mapping and stay valid
    until close()."""

    def __init__(self, path: str):
        self._h = C.c_void_p()
        rc = lib().raw("sgr_gguf_open")(path.encode(), C.byref(self._h))
        if rc != 0:
            raise SagerError("sgr_gguf_open", rc)

    def close(self):
        if self._h:
            lib().raw("sgr_gguf_close")(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def n_tensors(self):
        return lib().raw("sgr_gguf_count")(self._h, 0)

    @property
    def n_kv(self):
        return lib().raw("sgr_gguf_count")(self._h, 1)

    @property
    def alignment(self):
        return lib().raw("sgr_gguf_count")(self._h, 2)

    @property
    def data_offset(self):
        return lib().raw("sgr_gguf_count")(self._h, 3)

    def kv_type(self, key):
        return lib().raw("sgr_gguf_kv_type")(self._h, key.encode())

    def kv_int(self, key, dflt=0):
        return lib().raw("sgr_gguf_kv_int")(self._h, key.encode(), dflt)

    def kv_double(self, key, dflt=0.0):
        return lib().raw("sgr_gguf_kv_double")(self._h, key.encode(), dflt)

    def kv_str(self, key, dflt=""):
        n = lib().raw("sgr_gguf_kv_str")(self._h, key.encode(), None, 0)
        if n < 0:
            return dflt
        buf = C.create_string_buffer(n + 1)
        lib().raw("sgr_gguf_kv_str")(self._h, key.encode(), buf, n + 1)
        return buf.raw[:n].decode()

    def kv_array(self, key):
        """numpy view of a numeric array value, list of str for a string array, None if absent."""
        et, data = C.c_int(), C.c_void_p()
        n = lib().raw("sgr_gguf_kv_array")(self._h, key.encode(), C.byref(et), C.byref(data))
        if n < 0:
            return None
        if et.value == 8:
            out, p = [], data.value
            for _ in range(n):
                ln = C.c_uint64.from_address(p).value
                out.append(C.string_at(p + 8, ln).decode())
                p += 8 + ln
            return out
        dt = np.dtype(_ELEM_DTYPES[et.value])
        buf = (C.c_uint8 * (n * dt.itemsize)).from_address(data.value)
        return np.frombuffer(buf, dtype=dt, count=n)

    def tensor(self, name):
        info = TensorInfo()
        if lib().raw("sgr_gguf_tensor")(self._h, name.encode(), C.byref(info)) != 0:
            return None
        return info

    def tensor_bytes(self, name) -> np.ndarray:
        """uint8 view of a tensor's data inside the mapping."""
        t = self.tensor(name)
        if t is None:
            raise KeyError(name)
        buf = (C.c_uint8 * t.nbytes).from_address(t.data)
        return np.frombuffer(buf, dtype=np.uint8, count=t.nbytes)

    def tensor_names(self):
        out = []
        for i in range(self.n_tensors):
            n = lib().raw("sgr_gguf_tensor_name")(self._h, i, None, 0)
            buf = C.create_string_buffer(n + 1)
            lib().raw("sgr_gguf_tensor_name")(self._h, i, buf, n + 1)
            out.append(buf.raw[:n].decode())
        return out

    def fill_expert_pool(self, pool: np.ndarray, first_block, n_layer, n_expert, hidden, n_ff, n_threads=0):
        """pool: writable uint8 array of at least n_layer * n_expert * expert_bytes(hidden, n_ff) bytes
        (pinned host memory, a file mapping, ...). Expert (l, e) lands at (l * n_expert + e) * expert_bytes."""
        assert pool.dtype == np.uint8 and pool.flags["C_CONTIGUOUS"] and pool.flags["WRITEABLE"]
        lib().call("sgr_expert_pool_fill", self._h, C.c_void_p(pool.ctypes.data), pool.nbytes, first_block, n_layer,
                   n_expert, hidden, n_ff, n_threads)


def expert_bytes(hidden, n_ff) -> int:
    return lib().raw("sgr_expert_bytes")(hidden, n_ff)


def quantize_row_q4_k(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(x.size // 256 * 144, dtype=np.uint8)
    lib().call("sgr_quantize_row_q4_k", C.c_void_p(x.ctypes.data), x.size, C.c_void_p(out.ctypes.data))
    return out


def dequant_row_q6_k(row: np.ndarray, cols: int) -> np.ndarray:
    row = np.ascontiguousarray(row, dtype=np.uint8)
    out = np.zeros(cols, dtype=np.float32)
    lib().call("sgr_dequant_row_q6_k", C.c_void_p(row.ctypes.data), C.c_void_p(out.ctypes.data), cols)
    return out
