"""The C ABI as a C compiler sees it: tests/c_abi/abi_check.c includes only include/psi_cuda.h, is compiled as C11 and
linked against the built library.  Its struct layouts are held against the ctypes mirror (psi-dec_b200/binding.py)
and against the #[repr(C)] blocks a Rust binding would carry; with a GPU it runs the CPU-scale
configuration end to end from C and the result is checked against the CPU oracle."""
import ctypes as C
import re
import shutil
import subprocess
from pathlib import Path

import numpy as np
import pytest

import hostapi as H
from oracle import psi_oracle as O

pkg = H.pkg
ROOT = Path(__file__).resolve().parent.parent
SOURCE = ROOT / "tests" / "c_abi" / "abi_check.c"


@pytest.fixture(scope="module")
def abi_check(tmp_path_factory):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    lib_dir = pkg.library_path().parent
    exe = tmp_path_factory.mktemp("c_abi") / "abi_check"
    cmd = [gcc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", f"-I{ROOT / 'include'}", str(SOURCE), "-o", str(exe),
           f"-L{lib_dir}", "-lpsi_cuda", f"-Wl,-rpath,{lib_dir}"]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    return exe


def _layout(exe):
    out = subprocess.run([str(exe), "layout"], capture_output=True, text=True, check=True).stdout
    sizes, fields, enums = {}, {}, {}
    for line in out.splitlines():
        m = re.match(r"(\w+) sizeof (\d+)$", line)
        if m:
            sizes[m.group(1)] = int(m.group(2))
            continue
        m = re.match(r"(\w+)\.(\w+) offset (\d+) size (\d+)$", line)
        if m:
            fields.setdefault(m.group(1), []).append((m.group(2), int(m.group(3)), int(m.group(4))))
            continue
        if line.startswith(("enum ", "define ")):
            words = line.split()[1:]
            enums.update({words[i]: int(words[i + 1]) for i in range(0, len(words), 2)})
    return sizes, fields, enums


def test_header_compiles_as_c11_and_matches_the_ctypes_mirror(abi_check):
    from psi_dec_b200 import binding as B
    sizes, fields, enums = _layout(abi_check)
    mirrors = {"psi_page_table_layout": B.GQAPageTableLayout, "psi_replay_shape": B.GQAReplayShape,
               "psi_split_kv_variant": B.GQASplitKVVariant, "psi_norm_rope_config": B.NormRopeConfig,
               "psi_gqa_config": B.GQAConfig, "psi_u32_range": B._U32Range, "psi_hibernation_plan": B._HibernationPlan,
               "psi_kv_exchange": B.KvExchange}
    assert set(mirrors) == set(sizes), "every struct of the header has a mirror and the other way round"
    for name, mirror in mirrors.items():
        assert C.sizeof(mirror) == sizes[name], name
        assert len(mirror._fields_) == len(fields[name]), name
        for (c_name, offset, size), (py_name, py_type) in zip(fields[name], mirror._fields_):
            descriptor = getattr(mirror, py_name)
            assert (descriptor.offset, descriptor.size) == (offset, size), (name, c_name, py_name)
    assert enums["PSI_ERR_PAGE_ID"] == 6 and enums["PSI_DTYPE_F16"] == B.F16
    assert enums["PSI_KERNEL_MMA_SYNC"] == B.KERNEL_MMA_SYNC and enums["PSI_CAPACITY_CALLER_TOKENS"] == B.CAPACITY_CALLER_TOKENS
    assert enums["PSI_MD_CU_KV_SPLITS"] == B.MD_CU_KV_SPLITS
    assert enums["PSI_SNAPSHOT_DSPARK_GQA_REQUEST_PAGE_TABLE"] == B.SNAPSHOT_DSPARK_GQA_REQUEST_PAGE_TABLE


_RUST_SIZES = {"u32": (4, 4), "i32": (4, 4), "f32": (4, 4), "u64": (8, 8), "usize": (8, 8)}


def _rust_struct_layout(body, known):
    """(size, [(field, offset, size)]) of a #[repr(C)] struct body under the C layout rules on a 64-bit target."""
    offset, align_max, out = 0, 1, []
    for name, ty in re.findall(r"pub\s+(\w+)\s*:\s*([^,}]+)", body):
        ty = ty.strip()
        if ty.startswith("*"):
            size, align = 8, 8
        elif ty in _RUST_SIZES:
            size, align = _RUST_SIZES[ty]
        else:
            size, align = known[ty]
        offset = (offset + align - 1) // align * align
        out.append((name, offset, size))
        offset += size
        align_max = max(align_max, align)
    return (offset + align_max - 1) // align_max * align_max, align_max, out


def test_rust_repr_c_blocks_of_the_integration_notes_match_the_header(abi_check):
    sizes, fields, _ = _layout(abi_check)
    text = (ROOT / "INTEGRATION.md").read_text()
    known, seen = {}, 0
    for name, body in re.findall(r"pub struct (psi_\w+)\s*\{([^}]*)\}", text):
        if "_p: [u8; 0]" in body:
            continue                                    # opaque handles
        size, align, layout = _rust_struct_layout(body, known)
        known[name] = (size, align)
        assert name in sizes, f"{name} is in INTEGRATION.md but not in the header"
        assert size == sizes[name], name
        assert layout == fields[name], name
        seen += 1
    assert seen >= 5


@pytest.mark.gpu
def test_c_program_runs_the_cpu_scale_configuration_end_to_end(abi_check, tmp_path):
    out_file = tmp_path / "step.bin"
    done = subprocess.run([str(abi_check), "step", str(out_file)], capture_output=True, text=True)
    assert done.returncode == 0 and "step ok" in done.stdout, done.stdout + done.stderr
    check_cpu_scale_step(np.fromfile(out_file, dtype=np.uint16))


def check_cpu_scale_step(raw):
    """`raw` = q | k | v | arena after the step | out (f16 bits) of the CPU-scale configuration as the C and C++ callers
    write it: the inputs are regenerated here, the arena and the output are held against the CPU oracle."""
    hq, hkv, d, p, pages, context = 4, 1, 128, 16, 64, 256
    page_elems = 2 * hkv * p * d
    q, k, v, arena, out = np.split(raw, np.cumsum([hq * d, hkv * d, hkv * d, pages * page_elems]))
    # the program's inputs, regenerated: the same LCG, the same truncating float -> half conversion
    state = 0x4C8F17D2
    values = np.empty(pages * page_elems + hq * d + 2 * hkv * d, dtype=np.float32)
    for i in range(values.size):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        values[i] = np.float32(state >> 8) / np.float32(16777216.0) * np.float32(2.0) - np.float32(1.0)
    bits = values.view(np.uint32)
    exponent = ((bits >> 23) & 0xFF).astype(np.int64) - 127 + 15
    half = np.where(exponent <= 0, (bits >> 16) & 0x8000,
                    ((bits >> 16) & 0x8000) | (np.clip(exponent, 0, 30).astype(np.uint32) << 10) | ((bits & 0x7FFFFF) >> 13))
    half = half.astype(np.uint16)
    arena0, q0, k0, v0 = np.split(half, np.cumsum([pages * page_elems, hq * d, hkv * d]))
    assert np.array_equal(q, q0) and np.array_equal(k, k0) and np.array_equal(v, v0)
    table = ((np.arange(pages, dtype=np.uint32) * 37 + 11) % pages).astype(np.uint32)
    layout = O.Layout(1, 1, pages, 1)
    expected_arena = arena0.copy()
    O.kv_page_write(expected_arena, k0.reshape(1, hkv, d), v0.reshape(1, hkv, d), [0], [context], table, 1, 0, layout, hkv, d,
                    page_elems * 2)
    assert np.array_equal(arena, expected_arena), "the appended K/V rows are not where the oracle puts them"
    expected = O.paged_attention(expected_arena, O.F16, q0.reshape(1, hq, d), [0], [context], table, 0, layout, hq, hkv, d,
                                 page_elems * 2, 1.0 / np.sqrt(d))
    diff = np.abs(O.decode(out.reshape(1, hq, d), O.F16) - expected)
    assert diff.max() <= 2e-2 and diff.mean() <= 2e-3, (diff.max(), diff.mean())
