"""In-tree build of the native code (no setuptools, no JIT cache).

Two shared objects are produced next to this file:

* ``libw4a16_b200.so`` -- the CUDA kernels behind a plain C ABI (``include/w4a16_b200.h``),
  compiled by nvcc for ``sm_100a`` only; it does not link against torch.
* ``_C.so`` -- the torch operator shim (``csrc/int4_linear.cpp``) that registers
  ``torch.ops.w4a16.linear`` / ``dequantize`` and forwards to the C ABI.

``python nibble_b200/_build.py`` builds both; nothing is rebuilt while the outputs are newer than
every source.
"""
from __future__ import annotations

import concurrent.futures
import os
import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
OBJ = PKG / "build"
CORE_LIB = PKG / "libw4a16_b200.so"
CHECKED_LIB = PKG / "libw4a16_b200_checked.so"
TORCH_LIB = PKG / "_C.so"

CUDA_SOURCES = ["capi.cu", "linear_mma.cu", "linear_generic.cu", "dequantize.cu", "linear_static_scratch.cu", "linear_tcgen05.cu", "quantize.cu", "decode_ops.cu", "decode_persistent.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++20", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = pathlib.Path(cuda_home) / "bin" / "nvcc"
    if candidate.exists():
        return str(candidate)
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def _newest(paths) -> float:
    return max(p.stat().st_mtime for p in paths)


def _sources_mtime() -> float:
    files = list(CSRC.glob("*")) + list(INCLUDE.glob("*.h")) + [pathlib.Path(__file__)]
    return _newest(files)


def _run(cmd: list[str], log: pathlib.Path | None = None) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def build_core(force: bool = False) -> pathlib.Path:
    """Compile the CUDA sources and link ``libw4a16_b200.so``."""
    if not force and CORE_LIB.exists() and CORE_LIB.stat().st_mtime >= _sources_mtime():
        return CORE_LIB
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(name: str) -> pathlib.Path:
        obj = OBJ / (name + ".o")
        _run([nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(CSRC / name), "-o", str(obj)],
             log=OBJ / (name + ".ptxas.log"))
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(CUDA_SOURCES)) as pool:
        objects = list(pool.map(compile_one, CUDA_SOURCES))
    _run([nvcc, "-shared", "-o", str(CORE_LIB), *map(str, objects)])
    return CORE_LIB


def build_checked(force: bool = False) -> pathlib.Path:
    """``libw4a16_b200_checked.so``: the core library with the streaming kernel compiled with
    ``-DW4A16_BOUNDS_CHECK`` (every index compared with its extent; see ``w4a16_bounds_check_status``).  Only
    ``linear_mma.cu`` is compiled again; the other objects are those of the ordinary build."""
    build_core(force)
    if not force and CHECKED_LIB.exists() and CHECKED_LIB.stat().st_mtime >= max(_sources_mtime(), CORE_LIB.stat().st_mtime):
        return CHECKED_LIB
    nvcc = _nvcc()
    checked = OBJ / "linear_mma.cu.checked.o"
    _run([nvcc, *NVCC_FLAGS, "-DW4A16_BOUNDS_CHECK", "-I", str(INCLUDE), "-c", str(CSRC / "linear_mma.cu"), "-o", str(checked)],
         log=OBJ / "linear_mma.cu.checked.ptxas.log")
    objects = [checked if name == "linear_mma.cu" else OBJ / (name + ".o") for name in CUDA_SOURCES]
    _run([nvcc, "-shared", "-o", str(CHECKED_LIB), *map(str, objects)])
    return CHECKED_LIB


def build_torch_shim(force: bool = False) -> pathlib.Path:
    """Compile ``csrc/int4_linear.cpp`` against the installed torch and link it to the core library."""
    build_core(force)
    if (not force and TORCH_LIB.exists()
            and TORCH_LIB.stat().st_mtime >= max(_sources_mtime(), CORE_LIB.stat().st_mtime)):
        return TORCH_LIB
    import torch
    from torch.utils import cpp_extension

    includes = []
    for path in cpp_extension.include_paths("cuda"):
        includes += ["-isystem", path]
    torch_lib_dir = pathlib.Path(torch.__file__).resolve().parent / "lib"
    cmd = [
        os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        "-DTORCH_EXTENSION_NAME=_C",
        *includes, "-I", str(INCLUDE),
        str(CSRC / "int4_linear.cpp"), "-o", str(TORCH_LIB),
        f"-L{torch_lib_dir}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
        f"-L{PKG}", "-l:libw4a16_b200.so",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib_dir}",
    ]
    _run(cmd)
    return TORCH_LIB


def build_all(force: bool = False) -> None:
    build_core(force)
    build_torch_shim(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", CORE_LIB, "and", TORCH_LIB)
    if "--bounds-check" in sys.argv:
        print("built", build_checked(force="--force" in sys.argv))
