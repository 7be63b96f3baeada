"""ctypes binding of libsager_b200.so.

The prototypes are read from include/sager_b200.h, so the header is the single
statement of the ABI: a symbol the header declares and the library lacks is an
error at load time. There is no fallback: if the library is missing or was
built for another toolkit, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
HEADER = os.path.join(ROOT, "include", "sager_b200.h")
DIAG_HEADER = os.path.join(ROOT, "include", "sager_b200_diag.h")
LIB_PATH = os.path.join(HERE, "libsager_b200.so")

ERRORS = {1: "SGR_EARG", 2: "SGR_EALIGN", 3: "SGR_EUNSUPPORTED", 4: "SGR_ELAUNCH", 5: "SGR_EGEOMETRY",
          6: "SGR_ESTATICLIMIT"}

_SCALARS = {"int": C.c_int, "float": C.c_float, "double": C.c_double, "long long": C.c_longlong, "size_t": C.c_size_t,
            "unsigned long long": C.c_ulonglong}


class SagerError(RuntimeError):
    def __init__(self, fn, code):
        super().__init__(f"{fn} returned {code} ({ERRORS.get(code, 'unknown')})")
        self.code = code


def parse_header(path: str = HEADER):
    """-> {name: (restype, [argtypes])} for every `int sgr_*(...)` in the header."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    protos = {}
    for m in re.finditer(r"\b(const void\* const\*|int|long long|double|void\s*\*|void|size_t)\s*(sgr_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = "".join(m.group(1).split()), m.group(2), m.group(3).strip()
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = " ".join(a.split())
                if "*" in a:
                    argtypes.append(C.c_void_p)
                else:
                    base = a.rsplit(" ", 1)[0].replace("const ", "").strip()
                    argtypes.append(_SCALARS[base])
        protos[name] = ({"int": C.c_int, "longlong": C.c_longlong, "double": C.c_double, "size_t": C.c_size_t, "void": None,
                        "void*": C.c_void_p, "constvoid*const*": C.c_void_p}[ret], argtypes)
    return protos


class Lib:
    def __init__(self, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} is missing: build it with `python -m sager_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        self.path = path
        self.cdll = C.CDLL(path)
        self.protos = dict(parse_header(), **parse_header(DIAG_HEADER))
        missing = []
        for name, (res, args) in self.protos.items():
            try:
                fn = getattr(self.cdll, name)
            except AttributeError:
                missing.append(name)
                continue
            fn.restype = res
            fn.argtypes = args
        if missing:
            raise RuntimeError(f"{path} lacks symbols declared in the header: {missing}")

    def call(self, name, *args):
        """Call an int-returning entry point; raise SagerError on a non-zero return."""
        rc = getattr(self.cdll, name)(*args)
        if rc != 0:
            raise SagerError(name, rc)

    def raw(self, name):
        return getattr(self.cdll, name)


class MoeLayerArgs(C.Structure):
    """struct sgr_moe_layer of include/sager_b200.h (field order is the ABI)."""
    _fields_ = [
        ("n", C.c_int), ("n_max", C.c_int),
        ("hidden", C.c_int), ("n_ff", C.c_int), ("n_expert", C.c_int), ("n_used", C.c_int),
        ("expert_lo", C.c_int), ("expert_hi", C.c_int),
        ("shared_lo", C.c_int), ("shared_hi", C.c_int),
        ("routing_given", C.c_int), ("no_residual", C.c_int),
        ("shared_w", C.c_float),
        ("xn", C.c_void_p), ("xq_in", C.c_void_p),
        ("router_w", C.c_void_p), ("router_bias", C.c_void_p),
        ("w_tab", C.c_void_p),
        ("shared_gate", C.c_void_p), ("shared_up", C.c_void_p), ("shared_down", C.c_void_p),
        ("x_f16", C.c_void_p), ("out_f32", C.c_void_p),
        ("route_idx", C.c_void_p), ("route_w", C.c_void_p),
        ("mail", C.c_void_p), ("mail_n", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("route_stride", C.c_int), ("xq_stride", C.c_int), ("xq_out", C.c_void_p),
        ("wait_flags", C.c_void_p), ("wait_step", C.c_void_p),
        ("wait_count", C.c_int), ("wait_mul", C.c_int), ("wait_add", C.c_int),
        ("xq_padded", C.c_int),
        ("tab_stride", C.c_longlong),
        ("ep_dst", C.c_void_p), ("ep_flags", C.c_void_p), ("ep_out", C.c_void_p), ("ep_step", C.c_void_p),
        ("ep_world", C.c_int), ("ep_rec_bytes", C.c_int), ("ep_home_rows", C.c_int), ("ep_mul", C.c_int),
        ("ep_add", C.c_int),
        ("rearm_workspace", C.c_void_p), ("rearm_mail_n", C.c_void_p), ("rearm_n_max", C.c_int),
    ]


class MoePrefillArgs(C.Structure):
    """struct sgr_moe_prefill of include/sager_b200.h."""
    _fields_ = [
        ("n", C.c_int), ("n_max", C.c_int),
        ("hidden", C.c_int), ("n_ff", C.c_int), ("n_expert", C.c_int), ("n_used", C.c_int),
        ("tok_per", C.c_int), ("shared_w", C.c_float),
        ("xn", C.c_void_p), ("router_w", C.c_void_p), ("logits_in", C.c_void_p),
        ("w_tab", C.c_void_p), ("tab_stride", C.c_longlong),
        ("shared_gate", C.c_void_p), ("shared_up", C.c_void_p), ("shared_down", C.c_void_p),
        ("shared_gate_w", C.c_void_p),
        ("x_f16", C.c_void_p), ("xq", C.c_void_p), ("logits", C.c_void_p),
        ("route_idx", C.c_void_p), ("route_w", C.c_void_p), ("gslot", C.c_void_p), ("grows", C.c_void_p),
        ("off", C.c_void_p), ("toff", C.c_void_p), ("meta", C.c_void_p), ("mail", C.c_void_p),
        ("mail_n", C.c_void_p), ("xqg", C.c_void_p), ("g", C.c_void_p), ("u", C.c_void_p),
        ("hq", C.c_void_p), ("y_grouped", C.c_void_p), ("expert_y", C.c_void_p),
        ("sh_g", C.c_void_p), ("sh_u", C.c_void_p), ("sh_q", C.c_void_p), ("sh_y", C.c_void_p),
        ("sgate", C.c_void_p),
    ]


_LIB = None


def lib() -> Lib:
    global _LIB
    if _LIB is None:
        _LIB = Lib()
    return _LIB
