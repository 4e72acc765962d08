"""CPU-only checks of the boundary: the shared library loads, exports every symbol the header
declares, and refuses to compute without a GPU (there is no CPU fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200llama.h")).read()
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_python_mirror_agree(pkg):
    assert declared_symbols() == sorted(pkg.api.EXPORTS)


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.api.lib()
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_desc_struct_layout(pkg):
    # 16 int32/float fields + 128 bytes of NCCL id, no padding
    assert ctypes.sizeof(pkg.api.ModelDesc) == 16 * 4 + 128


def test_no_cpu_fallback(pkg):
    if pkg.api.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.B200Error, match="no CUDA device"):
        pkg.api.dequant(8, np.zeros(34, np.uint8), 1)
    with pytest.raises(pkg.B200Error, match="no CUDA device"):
        pkg.Engine.create(dict(pkg.synth.SHAPES["tiny"], eps=1e-5))


def test_create_rejects_bad_dims(pkg):
    bad = dict(pkg.synth.SHAPES["tiny"], eps=1e-5, hidden=250)
    with pytest.raises(pkg.B200Error):
        pkg.Engine.create(bad)


def test_create_rejects_head_sizes_the_kernels_do_not_map(pkg):
    """The attention kernels map lanes to positions assuming a power-of-two head size: 48, 80, 96 and 112 are refused
    (the check runs before any device is touched)."""
    for hd in (48, 80, 96, 112, 256):
        bad = dict(pkg.synth.SHAPES["tiny"], eps=1e-5, hidden=hd * 4 * 4, n_heads=16, n_kv_heads=4)
        assert bad["hidden"] % 256 == 0
        with pytest.raises(pkg.B200Error, match="head_dim must be 16, 32, 64 or 128"):
            pkg.Engine.create(bad)


def test_header_compiles_as_c_and_cpp(tmp_path):
    """The boundary header is plain C: it must go through a C11 and a C++17 compiler on its own."""
    import subprocess
    inc = os.path.join(ROOT, "include")
    (tmp_path / "c.c").write_text('#include "b200llama.h"\nint main(void) { return B200_KV_I8 == 1 ? 0 : 1; }\n')
    (tmp_path / "cpp.cpp").write_text('#include "b200llama.h"\nint main() { b200_model_desc d{}; return d.tp_size; }\n')
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-I", inc, str(tmp_path / "c.c")], check=True)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-I", inc, str(tmp_path / "cpp.cpp")], check=True)


def test_reference_side_adapter_compiles_and_links(pkg, tmp_path):
    """The adapter of INTEGRATION.md (TinyLlamaModel / KVCache members forwarded to the C ABI) compiles with g++,
    links against libb200llama.so alone and, run without a model file, reports the library's error instead of crashing."""
    import subprocess
    pkg.api.lib()
    so_dir = os.path.join(ROOT, "tinyllama.cpp_b200", "csrc")
    exe = str(tmp_path / "adapter_check")
    subprocess.run(["g++", "-std=c++17", "-Wall", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "abi", "adapter_check.cpp"),
                    "-o", exe, "-L", so_dir, "-lb200llama", f"-Wl,-rpath,{so_dir}"], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert "init failed as expected" in r.stdout, (r.stdout, r.stderr)
    assert r.returncode in (0, 1)  # 0 without a GPU, 1 with one (the model file does not exist either way)


def test_product_never_touches_oracle():
    """Nothing under the package or the C ABI may reference the oracle folder."""
    for root, _, files in os.walk(os.path.join(ROOT, "tinyllama.cpp_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", ".inc")):
                text = open(os.path.join(root, f), errors="replace").read()
                assert "oracle" not in text.lower(), os.path.join(root, f)
