"""The C++ host-side mirror (include/psi_cuda.hpp) as a C++ compiler sees it: tests/cpp_host/host_mirror_check.cpp is
compiled as C++17 against the two public headers and linked against the built library.  Without a GPU it runs the
host-only types against the vectors of the reference's own tests; with one it runs the CPU-scale configuration end to
end through the mirrored component types and the result is checked against the CPU oracle."""
import shutil
import subprocess
from pathlib import Path

import numpy as np
import pytest

import hostapi as H
from test_c_abi import check_cpu_scale_step

pkg = H.pkg
ROOT = Path(__file__).resolve().parent.parent
SOURCE = ROOT / "tests" / "cpp_host" / "host_mirror_check.cpp"


def _cuda_include():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return Path(nvcc).resolve().parent.parent / "include"


@pytest.fixture(scope="module")
def mirror_check(tmp_path_factory):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no C++ compiler")
    lib_dir = pkg.library_path().parent
    cuda = _cuda_include()
    exe = tmp_path_factory.mktemp("cpp_host") / "host_mirror_check"
    cmd = [gxx, "-std=c++17", "-Wall", "-Wextra", "-Werror", f"-I{ROOT / 'include'}", f"-isystem{cuda}", str(SOURCE),
           "-o", str(exe), f"-L{lib_dir}", "-lpsi_cuda", f"-L{cuda.parent / 'lib64'}", "-lcudart",
           f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{cuda.parent / 'lib64'}"]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    return exe


def test_host_only_types_reproduce_the_reference_vectors_from_cpp(mirror_check):
    done = subprocess.run([str(mirror_check), "host"], capture_output=True, text=True)
    assert done.returncode == 0 and "host ok" in done.stdout, done.stdout + done.stderr


@pytest.mark.gpu
def test_cpp_program_runs_the_cpu_scale_configuration_through_the_mirrored_types(mirror_check, tmp_path):
    out_file = tmp_path / "step.bin"
    done = subprocess.run([str(mirror_check), "step", str(out_file)], capture_output=True, text=True)
    assert done.returncode == 0 and "step ok" in done.stdout, done.stdout + done.stderr
    check_cpu_scale_step(np.fromfile(out_file, dtype=np.uint16))
