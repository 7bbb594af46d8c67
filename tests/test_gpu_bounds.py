"""Bounds checks on page IDs: on the host where IDs enter the table (both builds of the library), and in every kernel
before an address is formed (the checked build, libpsi_cuda_checked.so, driven by tests/checked_build_worker.py in a
process of its own).

The reference checks IDs on the way into the table (crates/inference-executor-metal/src/state/gqa.rs:97-102) and table
indices with debug assertions (crates/inference-executor-metal/src/attn/gqa/request_page_table.rs:75,115); its shaders
trust the table, and so does the production build here.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

import workloads as W

pkg = W.pkg
pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


class Small:
    """One request slot over a 16-page buffer of which the arena object declares only the first 8 pages."""

    def __init__(self, dtype=pkg.BF16, kernel_mode=pkg.KERNEL_AUTO, head_dim=128, tokens_per_page=16):
        import torch
        self.torch = torch
        tdtype = {pkg.F32: torch.float32, pkg.BF16: torch.bfloat16}[dtype]
        esz = 4 if dtype == pkg.F32 else 2
        self.hq, self.hkv, self.d, self.p = 4, 2, head_dim, tokens_per_page
        self.page_bytes = 2 * self.hkv * self.p * self.d * esz
        self.buffer = torch.randn((16, self.page_bytes // esz), device="cuda:0", dtype=torch.float32).to(tdtype)
        self.ctx = pkg.Context(0, stream=torch.cuda.current_stream().cuda_stream)
        self.pages = pkg.PageArena(self.ctx, 8, self.page_bytes, device_ptr=self.buffer)      # declared: 8 pages
        self.layout = pkg.GQAPageTableLayout(1, 1, 4, 1)
        self.table = pkg.GQARequestPageTable(self.ctx, self.layout)
        cfg = pkg.GQAConfig(self.hq, self.hkv, self.d, 0.1, self.page_bytes, dtype, self.layout, 4, pkg.PLAN_BALANCED,
                            kernel_mode, 0)
        self.gqa = pkg.GQA(self.ctx, cfg)
        self.q = torch.randn((1, self.hq, self.d), device="cuda:0", dtype=torch.float32).to(tdtype)
        self.k = torch.randn((1, self.hkv, self.d), device="cuda:0", dtype=torch.float32).to(tdtype)
        self.v = torch.randn((1, self.hkv, self.d), device="cuda:0", dtype=torch.float32).to(tdtype)
        self.out = torch.zeros_like(self.q)

    def close(self):
        self.ctx.sync()
        self.gqa.close()
        self.table.close()
        self.pages.close()
        self.ctx.close()


def test_table_refuses_page_ids_beyond_its_declared_bound():
    s = Small()
    s.table.write_row(0, 0, [3, 12, 1, 0])                 # no bound declared: accepted, as the reference's table does
    with pytest.raises(pkg.PsiError, match="already holds a page ID outside the declared bound"):
        s.table.set_page_bound(8)
    s.table.write_row(0, 0, [3, 7, 1, 0])
    s.table.set_page_bound(8)
    with pytest.raises(pkg.PsiError, match="outside the cache-page buffer"):
        s.table.write_row(0, 0, [3, 12, 1, 0])
    with pytest.raises(pkg.PsiError, match="outside the cache-page buffer"):
        s.table.write_page_ids(0, 0, 1, [8])
    assert s.table.read_page_ids(0, 0, 1) == [7]            # the refused writes changed nothing
    s.table.set_page_bound(0)                               # bound withdrawn
    s.table.write_page_ids(0, 0, 1, [12])
    s.close()


def test_every_kernel_of_the_checked_build_skips_and_reports_an_out_of_range_page_id():
    worker = ROOT / "tests" / "checked_build_worker.py"
    done = subprocess.run([sys.executable, str(worker)], capture_output=True, text=True, timeout=900,
                          env={**os.environ, "PSI_CUDA_LIBRARY": "checked"})
    assert done.returncode == 0 and "checked build ok" in done.stdout, done.stdout[-3000:] + done.stderr[-3000:]


def test_snapshot_load_refuses_ids_beyond_the_declared_bound(tmp_path):
    s = Small()
    s.table.write_row(0, 0, [3, 12, 1, 0])
    plan = pkg.ExecutorHibernationPlan.all()
    files = [pkg.SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE]
    writer = pkg.StateSnapshotWriter(tmp_path / "snap", files, plan)
    writer.write_table(files[0], s.table)
    writer.commit()
    s.table.write_row(0, 0, [4, 5, 6, 7])
    s.table.set_page_bound(8)
    reader = pkg.StateSnapshotReader(tmp_path / "snap", files, plan)
    with pytest.raises(pkg.PsiError, match="outside the cache-page buffer"):
        reader.read_table(files[0], s.table)
    reader.close()
    assert [s.table.read_page_ids(0, 0, b)[0] for b in range(4)] == [4, 5, 6, 7]   # the refused load changed nothing
    s.table.write_page_ids(0, 0, 0, [1])                                          # and the host mirror is intact too
    assert [s.table.read_page_ids(0, 0, b)[0] for b in range(4)] == [1, 5, 6, 7]
    s.close()
