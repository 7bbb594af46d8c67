"""Builds ``lib/libpsi_cuda.so`` (the C-ABI library) from ``csrc/`` with nvcc for sm_100a, and beside it
``lib/libpsi_cuda_checked.so``, the same sources with ``-DPSI_CUDA_CHECKED=1``: every kernel bounds-checks the page
IDs and table indices it reads (see ``csrc/device_common.cuh``).

Run as ``python psi-dec_b200/build.py`` or call :func:`build_library`.  A library is rebuilt only when a source or
header is newer than it.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "libpsi_cuda.so"
LIB_CHECKED = PKG / "lib" / "libpsi_cuda_checked.so"
SOURCES = ["api_common.cu", "api_context.cu", "api_arena.cu", "api_snapshot.cu", "api_policy.cu", "api_gqa.cu", "api_exchange.cu", "api_host_step.cu", "kv_pages.cu", "prep.cu", "attend_generic.cu", "attend_staged.cu", "attend_mma.cu", "attend_chunk.cu", "attend_chunk_umma.cu", "tma_map.cu", "attend_static.cu", "exchange.cu", "probe.cu", "host_logic.cpp", "snapshot.cpp"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libpsi_cuda.so")
    return found


def _stale(lib: Path) -> bool:
    if not lib.exists():
        return True
    built = lib.stat().st_mtime
    deps = list(CSRC.glob("*")) + [ROOT / "include" / "psi_cuda.h", Path(__file__)]
    return any(p.stat().st_mtime > built for p in deps)


def build_library(force: bool = False, verbose: bool = False, checked: bool = False) -> Path:
    lib = LIB_CHECKED if checked else LIB
    if not force and not _stale(lib):
        return lib
    lib.parent.mkdir(parents=True, exist_ok=True)
    obj_dir = PKG / ("build_checked" if checked else "build")
    obj_dir.mkdir(exist_ok=True)
    host_cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else (shutil.which("g++") or "g++")
    common = [_nvcc(), "-ccbin", host_cxx, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3",
              "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", f"-I{ROOT / 'include'}", f"-I{CSRC}"]
    if checked:
        common += ["-DPSI_CUDA_CHECKED=1"]
    if verbose:
        common += ["-Xptxas", "-v"]
    # extra -D flags from the environment, e.g. PSI_CUDA_DEFINES="NDEBUG"
    common += [f"-D{name}" for name in os.environ.get("PSI_CUDA_DEFINES", "").split() if name]
    procs = []
    objects = []
    for src in SOURCES:
        obj = obj_dir / (src + ".o")
        objects.append(str(obj))
        cmd = common + (["-x", "cu"] if src.endswith(".cpp") else []) + ["-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(out)
        if proc.returncode != 0:
            failed.append(src)
    if failed:
        raise RuntimeError(f"nvcc failed for {failed}")
    link = [_nvcc(), "-ccbin", host_cxx, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(lib)] + objects
    subprocess.run(link, check=True)
    return lib


def build_all(force: bool = False, verbose: bool = False):
    return build_library(force, verbose), build_library(force, verbose, checked=True)


if __name__ == "__main__":
    print(*build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
