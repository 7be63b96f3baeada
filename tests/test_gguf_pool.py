"""CPU tests of the host side: the GGUF v3 reader and the expert-pool builder. The files are
written here with numpy in the layout of the specification the reference implements
(include/sager/core/gguf.hpp:7-12); the Q4_K requantisation of a Q6_K down tensor is held, byte
for byte, to the reference's own quantiser (src/kernels/q4_k.cpp:68-174, compiled into
oracle/_ref) and the Q6_K dequantiser to the numpy restatement of src/core/weights.cpp:168-209."""
import struct

import numpy as np
import pytest

from oracle.oracle import dequant_q6k, make_q6k
from sager_b200 import gguf as sg
from sager_b200.capi import SagerError


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, kv, tensors, alignment=32, version=3):
    """kv: list of (key, type_id, python value); tensors: list of (name, dims, type_id, bytes)."""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kv)))
    fmt = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}
    for key, t, v in kv:
        out += _s(key.encode()) + struct.pack("<I", t)
        if t in fmt:
            out += struct.pack(fmt[t], v)
        elif t == 8:
            out += _s(v.encode())
        else:                                        # array: (elem_type, list)
            et, items = v
            out += struct.pack("<IQ", et, len(items))
            for it in items:
                out += _s(it.encode()) if et == 8 else struct.pack(fmt[et], it)
    off = 0
    offsets = []
    for name, dims, t, data in tensors:
        offsets.append(off)
        out += _s(name.encode()) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", t, off)
        off = (off + len(data) + alignment - 1) // alignment * alignment
    out += b"\0" * ((-len(out)) % alignment)
    start = len(out)
    for (name, dims, t, data), o in zip(tensors, offsets):
        out += b"\0" * (start + o - len(out)) + bytes(data)
    with open(path, "wb") as f:
        f.write(out)


def test_reader_parses_header_kv_and_tensor_directory(tmp_path):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((3, 8)).astype(np.float32)
    q = rng.integers(0, 256, size=2 * 144 * 5, dtype=np.uint8)
    kv = [("general.architecture", 8, "qwen3moe"), ("general.alignment", 4, 64), ("sage.block_count", 4, 40),
          ("sage.rope.freq_base", 6, 1e6), ("flag", 7, 1), ("neg", 5, -7), ("big", 10, 1 << 40), ("pi", 12, 3.14159),
          ("ints", 9, (5, [1, -2, 3])), ("names", 9, (8, ["a", "bcd", ""]))]
    tensors = [("token_embd.weight", [8, 3], 0, a.tobytes()), ("blk.0.w", [512, 5], 12, q.tobytes())]
    p = str(tmp_path / "m.gguf")
    write_gguf(p, kv, tensors, alignment=64)
    with sg.File(p) as f:
        assert (f.n_tensors, f.n_kv, f.alignment) == (2, 10, 64) and f.data_offset % 64 == 0
        assert f.kv_str("general.architecture") == "qwen3moe" and f.kv_str("missing", "x") == "x"
        assert f.kv_int("sage.block_count") == 40 and f.kv_int("neg") == -7 and f.kv_int("big") == 1 << 40
        assert f.kv_int("flag") == 1 and f.kv_int("nope", 9) == 9 and f.kv_type("nope") == -1
        assert abs(f.kv_double("sage.rope.freq_base") - 1e6) < 1 and abs(f.kv_double("pi") - 3.14159) < 1e-12
        assert f.kv_array("ints").tolist() == [1, -2, 3] and f.kv_array("names") == ["a", "bcd", ""]
        assert f.tensor_names() == ["token_embd.weight", "blk.0.w"]
        t = f.tensor("blk.0.w")
        assert (t.type, t.n_dims, list(t.dims)[:2], t.nbytes, t.row_bytes) == (12, 2, [512, 5], q.size, 288)
        assert np.array_equal(f.tensor_bytes("blk.0.w"), q)
        assert np.array_equal(f.tensor_bytes("token_embd.weight").view(np.float32).reshape(3, 8), a)
        assert f.tensor("absent") is None


def test_reader_refuses_what_is_not_a_v3_file(tmp_path):
    p = str(tmp_path / "bad.gguf")
    open(p, "wb").write(b"GGML" + b"\0" * 64)
    with pytest.raises(SagerError):
        sg.File(p)
    write_gguf(p, [], [], version=2)
    with pytest.raises(SagerError) as e:
        sg.File(p)
    assert e.value.code == 3                                   # not version 3
    write_gguf(p, [], [("t", [4096, 4096], 0, b"\0" * 64)])     # tensor data beyond the end of the file
    with pytest.raises(SagerError):
        sg.File(p)
    with pytest.raises(SagerError):
        sg.File(str(tmp_path / "does_not_exist.gguf"))


def test_q6k_dequant_and_q4k_quantiser_match_their_references(reference):
    rng = np.random.default_rng(4)
    cols = 512
    w6 = make_q6k(rng, 6, cols, d_scale=2e-3)
    want = dequant_q6k(w6, cols)
    for r in range(6):
        assert np.array_equal(sg.dequant_row_q6_k(w6[r], cols), want[r])
    # the quantiser: byte for byte the reference's own q4k::quantize_row, on gaussian rows, on
    # dequantised Q6_K rows (what the pool builder feeds it) and on degenerate sub-blocks
    rows = [rng.standard_normal(2048).astype(np.float32) * 0.02 for _ in range(24)]
    rows += [want[r] for r in range(6)]
    flat = np.zeros(512, dtype=np.float32)
    flat[256:288] = 0.5
    rows.append(flat)
    total = same = 0
    for x in rows:
        got = sg.quantize_row_q4_k(x)
        ref = reference.quantize_q4k(x[None])[0]
        total += got.size
        same += int((got == ref).sum())
    assert same == total, f"{total - same} of {total} bytes differ from the reference's quantiser"


def test_expert_pool_layout_and_q6k_down_requantisation(tmp_path, reference):
    H, F, E, L = 512, 256, 3, 2
    rng = np.random.default_rng(8)
    gu = F * (H // 256) * 144
    dn = H * (F // 256) * 144
    kv = [("general.architecture", 8, "test")]
    tensors, keep = [], {}
    for l in range(L):
        g = rng.integers(0, 256, size=E * gu, dtype=np.uint8)
        u = rng.integers(0, 256, size=E * gu, dtype=np.uint8)
        keep[(l, "g")], keep[(l, "u")] = g, u
        tensors.append((f"blk.{l + 3}.ffn_gate_exps.weight", [H, F, E], 12, g.tobytes()))
        tensors.append((f"blk.{l + 3}.ffn_up_exps.weight", [H, F, E], 12, u.tobytes()))
        if l == 0:                                    # layer 0: down stored as Q4_K, copied
            d = rng.integers(0, 256, size=E * dn, dtype=np.uint8)
            keep[(l, "d")] = d
            tensors.append((f"blk.{l + 3}.ffn_down_exps.weight", [F, H, E], 12, d.tobytes()))
        else:                                         # layer 1: down stored as Q6_K, requantised
            d6 = make_q6k(rng, E * H, F, d_scale=2e-3)
            keep[(l, "d6")] = d6
            tensors.append((f"blk.{l + 3}.ffn_down_exps.weight", [F, H, E], 14, d6.tobytes()))
    p = str(tmp_path / "moe.gguf")
    write_gguf(p, kv, tensors)
    eb = sg.expert_bytes(H, F)
    assert eb == 2 * gu + dn
    pool = np.zeros(L * E * eb, dtype=np.uint8)
    with sg.File(p) as f:
        f.fill_expert_pool(pool, first_block=3, n_layer=L, n_expert=E, hidden=H, n_ff=F, n_threads=3)
        with pytest.raises(SagerError) as e:          # geometry that the tensors do not have
            f.fill_expert_pool(np.zeros(L * (E + 1) * eb, dtype=np.uint8), 3, L, E + 1, H, F)
        assert e.value.code == 5
        with pytest.raises(SagerError):               # a block range without expert tensors
            f.fill_expert_pool(pool, 0, L, E, H, F)
    for l in range(L):
        for e in range(E):
            blob = pool[(l * E + e) * eb:(l * E + e + 1) * eb]
            assert np.array_equal(blob[:gu], keep[(l, "g")][e * gu:(e + 1) * gu])
            assert np.array_equal(blob[gu:2 * gu], keep[(l, "u")][e * gu:(e + 1) * gu])
            if l == 0:
                assert np.array_equal(blob[2 * gu:], keep[(l, "d")][e * dn:(e + 1) * dn])
            else:
                rows6 = keep[(l, "d6")][e * H:(e + 1) * H]
                want = reference.quantize_q4k(dequant_q6k(rows6, F))      # the reference's requantisation
                assert np.array_equal(blob[2 * gu:].reshape(H, -1), want)
