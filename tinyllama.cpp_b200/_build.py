"""Builds the package's native libraries in-tree (next to their sources).

libb200llama.so  CUDA kernels + C ABI, compiled for sm_100a only (nvcc cross-compiles without a GPU)
libb200synth.so  host-only synthetic GGUF writer (g++ / OpenMP)
"""
import os
import shutil
import subprocess

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
LIB_ENGINE = os.path.join(CSRC, "libb200llama.so")
LIB_SYNTH = os.path.join(CSRC, "libb200synth.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources(exts):
    out = []
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith(exts)]
    out.append(os.path.join(os.path.dirname(CSRC), "..", "include", "b200llama.h"))
    return out


def build_engine(force=False, verbose=False):
    srcs = _sources((".cu", ".cuh", ".cpp", ".h", ".inc"))
    if not force and _newer(LIB_ENGINE, srcs):
        return LIB_ENGINE
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
          ["-o", LIB_ENGINE, os.path.join(CSRC, "engine.cu"), os.path.join(CSRC, "gguf.cpp"), "-ldl"]
    subprocess.run(cmd, check=True, cwd=CSRC)
    return LIB_ENGINE


def build_synth(force=False):
    src = os.path.join(CSRC, "synth.cpp")
    if not force and _newer(LIB_SYNTH, [src]):
        return LIB_SYNTH
    subprocess.run(["g++", "-O2", "-fopenmp", "-fPIC", "-shared", "-o", LIB_SYNTH, src], check=True, cwd=CSRC)
    return LIB_SYNTH


def build_all(force=False):
    return build_engine(force), build_synth(force)
