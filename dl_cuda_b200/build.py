"""Builds libdlcuda_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

One object per .cu file under csrc/, rebuilt only when the source or a header
is newer, linked into dl_cuda_b200/libdlcuda_b200.so.  Run as
``python -m dl_cuda_b200.build`` or through ``build()``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libdlcuda_b200.so"

NVCC_FLAGS = [
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built (there is no CPU fallback)")
    return exe


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every CUDA source and link the shared library; returns its path."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "dlcuda_b200.h"]

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), file=sys.stderr)
            res = subprocess.run(cmd, capture_output=True, text=True)
            if verbose:
                sys.stderr.write(res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))

    if force or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(LIB_PATH), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr}")
    return LIB_PATH


CPP_TEST_SRC = PKG_DIR.parent / "tests" / "cpp" / "layer_api_test.cu"
CPP_TEST_BIN = PKG_DIR.parent / "tests" / "cpp" / "layer_api_test"


CPP_MODELS_SRC = PKG_DIR.parent / "tests" / "cpp" / "layer_models.cu"
CPP_MODELS_LIB = PKG_DIR.parent / "tests" / "cpp" / "libnative_models.so"


def build_cpp_tests() -> Path:
    """Compile the C++ test programs that drive the layer classes of src/*.cuh against the library:
    the known-answer binary and the shared library of small models (tests/cpp/layer_models.cu)."""
    build()
    common = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2",
              f"-I{PKG_DIR / 'src'}", f"-I{PKG_DIR.parent / 'include'}"]
    link = [f"-L{PKG_DIR}", "-ldlcuda_b200", "-Xlinker", "-rpath,$ORIGIN/../../dl_cuda_b200", "-lcurand"]
    headers = sorted((PKG_DIR / "src").glob("*.cuh"))
    jobs = [(CPP_TEST_SRC, CPP_TEST_BIN, []),
            (CPP_MODELS_SRC, CPP_MODELS_LIB, ["-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden"])]
    for src, out, extra in jobs:
        if _stale(out, [src, LIB_PATH] + headers):
            cmd = [_nvcc(), *common, *extra, str(src), "-o", str(out), *link]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stderr}")
    return CPP_TEST_BIN


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
    print(build_cpp_tests())
