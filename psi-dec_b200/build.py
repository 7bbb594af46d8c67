"""Builds ``lib/libpsi_cuda.so`` (the C-ABI library) from ``csrc/`` with nvcc for sm_100a.

Run as ``python psi-dec_b200/build.py`` or call :func:`build_library`.  The library is rebuilt only when a source or
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
SOURCES = ["api_common.cu", "api_context.cu", "api_arena.cu", "api_snapshot.cu", "api_policy.cu", "api_gqa.cu", "api_exchange.cu", "api_host_step.cu", "kv_pages.cu", "prep.cu", "attend_generic.cu", "attend_mma.cu", "attend_chunk.cu", "attend_chunk_umma.cu", "attend_static.cu", "exchange.cu", "probe.cu", "host_logic.cpp", "snapshot.cpp"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libpsi_cuda.so")
    return found


def _stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*")) + [ROOT / "include" / "psi_cuda.h", Path(__file__)]
    return any(p.stat().st_mtime > built for p in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    LIB.parent.mkdir(parents=True, exist_ok=True)
    obj_dir = PKG / "build"
    obj_dir.mkdir(exist_ok=True)
    host_cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else (shutil.which("g++") or "g++")
    common = [_nvcc(), "-ccbin", host_cxx, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3",
              "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", f"-I{ROOT / 'include'}", f"-I{CSRC}"]
    if verbose:
        common += ["-Xptxas", "-v"]
    # extra -D flags for tracing builds, e.g. PSI_CUDA_DEFINES="PSI_UMMA_TRACE"
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
    link = [_nvcc(), "-ccbin", host_cxx, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB)] + objects
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
