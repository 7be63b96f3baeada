"""CPU checks of the C boundary: the library builds for sm_100a, loads without a
GPU and exports every symbol the header declares; the shim header compiles."""
import os
import subprocess

from sager_b200 import build as sbuild
from sager_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_builds_and_exports_header_symbols():
    path = sbuild.build()
    assert os.path.exists(path)
    lib = capi.Lib(path)            # raises if a declared symbol is missing
    assert len(lib.protos) >= 39
    assert lib.raw("sgr_abi_version")() == 4
    out = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True).stdout
    exported = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    assert set(lib.protos) <= exported


def test_argument_validation_needs_no_gpu():
    lib = capi.lib()
    # null pointers and bad sizes are refused before any CUDA call
    assert lib.raw("sgr_gemv_q4_k_q8")(None, None, None, 8, 2048, None) == 1
    assert lib.raw("sgr_gemv_q4_k_q8")(16, 16, 16, 8, 2000, None) == 1      # k % 256 != 0
    assert lib.raw("sgr_gemv_q4_k_q8")(16, 18, 16, 8, 2048, None) == 2      # x_q8 not 4-byte aligned
    assert lib.raw("sgr_quantize_q8_k")(16, 16, 100, None) == 1
    assert lib.raw("sgr_router_topk_batched")(16, 16, 16, 256, 8, 8, 1, 1.0, None) == 1  # stride < K+1
    assert lib.raw("sgr_gemv_q4_k_q8")(16, 16, 16, 0, 2048, None) == 0      # empty: nothing to do
    # the tensor-core family refuses what the reference refuses, before any CUDA call
    assert lib.raw("sgr_tc_gemm_f16_raw")(16, 16, 16, 8, 100, 4, None) == 3          # k % 64 != 0
    assert lib.raw("sgr_tc_gemm_f16_raw")(18, 16, 16, 8, 64, 4, None) == 2           # operand not 16-byte aligned
    assert lib.raw("sgr_tc_gemm_q4_k_f16")(16, 16, 16, 16, 8, 768, 4, None) == 3     # k not a power of two
    assert lib.raw("sgr_tc_scratch_elems")(512, 2048) == 512 * 2048


def test_shim_header_compiles_against_c_abi():
    shim = os.path.join(ROOT, "include", "sager_b200_shim.hpp")
    if not os.path.exists(shim):
        import pytest
        pytest.skip("shim header not written yet")
    src = '#include "sager_b200_shim.hpp"\nint main() { return 0; }\n'
    res = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"),
                          "-x", "c++", "-"], input=src, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_shim_defines_exactly_the_reference_launchers(tmp_path):
    """Link check against the reference's own header: a translation unit that only
    sees include/sager/kernels/cuda_ops.hpp takes the address of every launcher the
    shim claims to provide; it links only if the shim defines those exact
    signatures. Needs the reference tree and the CUDA headers."""
    import pytest
    from oracle.oracle import reference_root
    import shutil
    ref_inc = os.path.join(reference_root(), "include")
    nvcc = shutil.which("nvcc")
    cuda_home = os.environ.get("CUDA_HOME") or (os.path.dirname(os.path.dirname(os.path.realpath(nvcc))) if nvcc else "")
    cuda_inc = os.path.join(cuda_home, "include")
    if not (os.path.isdir(ref_inc) and os.path.isdir(cuda_inc)):
        pytest.skip("reference tree or CUDA headers not present")
    import re
    shim = open(os.path.join(ROOT, "include", "sager_b200_shim.hpp")).read()
    body = shim.split("int b200_last_error();", 1)[1].split("#ifdef SAGER_B200_SHIM_IMPLEMENTATION", 1)[0]
    # every launcher the shim declares, whatever it returns (void, bool, void*, size_t)
    names = re.findall(r"^(?:void|bool|void\*|size_t) (\w+)\(", body, flags=re.M)
    assert len(names) >= 41 and {"tc_gemm_q4_k_f16", "tc_handle", "tc_scratch_elems", "tc_gemm_f16_raw",
                                 "tc_gemm_f16_f32out_raw"} <= set(names)
    user = tmp_path / "user.cpp"
    user.write_text('#include "sager/kernels/cuda_ops.hpp"\n'
                    "const void* volatile sink[] = {\n" +
                    "".join(f"  reinterpret_cast<const void*>(&sager::cuda::{n}),\n" for n in names) +
                    "};\nint main() { return sink[0] != nullptr ? 0 : 1; }\n")
    impl = tmp_path / "impl.cpp"
    impl.write_text('#include "sager/kernels/cuda_ops.hpp"\n#define SAGER_B200_SHIM_IMPLEMENTATION\n'
                    '#include "sager_b200_shim.hpp"\n')
    lib = sbuild.build()
    exe = tmp_path / "a.out"
    cmd = ["g++", "-std=c++20", "-I", ref_inc, "-I", cuda_inc, "-I", os.path.join(ROOT, "include"),
           str(user), str(impl), lib, f"-Wl,-rpath,{os.path.dirname(lib)}", "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
