"""The C-ABI library loads without a GPU and exports every function the public header declares (no GPU)."""
import ctypes as C
import re
from pathlib import Path

import __graft_entry__ as entry

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "psi_cuda.h").read_text()
    return sorted(set(re.findall(r"PSI_API\s+int32_t\s+(psi_\w+)\s*\(", text)))


def test_header_declares_and_library_exports_every_entry_point():
    entry.build()
    lib = entry.load_package().library()
    names = declared_functions()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # the bounds-checked build is the same library with device-side checks compiled in: same exports
    checked = C.CDLL(str(entry.load_package().library_path().with_name("libpsi_cuda_checked.so")))
    missing = [n for n in names if not hasattr(checked, n)]
    assert not missing, missing


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        return
    pkg = entry.load_package()
    try:
        pkg.Context(0)
    except pkg.PsiError as err:
        assert err.status == 5 and "no CPU fallback" in err.message
    else:
        raise AssertionError("context creation must fail without a CUDA device")


def test_product_does_not_reference_the_oracle():
    for path in (ROOT / "psi-dec_b200").rglob("*"):
        if path.suffix in {".py", ".cu", ".cuh", ".cpp", ".hpp", ".h"}:
            assert "oracle" not in path.read_text().lower(), path
