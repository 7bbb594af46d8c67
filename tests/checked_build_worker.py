"""Worker of tests/test_gpu_bounds.py: runs in a process of its own with PSI_CUDA_LIBRARY=checked, so that the package
loads the bounds-checked build of the library (libpsi_cuda_checked.so), and drives every kernel through a page table
that holds an out-of-range page ID.

The arena object declares 8 pages over a buffer that really holds 16 and the bad ID is 12: the access a check must skip
would have stayed inside the buffer anyway, so no run can touch memory it does not own.
"""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import torch

import __graft_entry__ as entry

pkg = entry.load_package()
PSI_ERR_PAGE_ID = 6


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



def kernels_skip_an_out_of_range_page_id_and_report_it(dtype, kernel_mode):
    import torch
    s = Small(dtype=dtype, kernel_mode=kernel_mode)
    s.table.write_row(0, 0, [3, 12, 1, 0])                  # logical page 1 -> physical 12, beyond the declared 8
    before = s.buffer.clone()

    # append of token 20 (logical page 1): the write is skipped, nothing in the buffer changes
    s.gqa.prepare([0], [20], [0, 1])
    s.gqa.kv_page_write(s.pages, s.table, 0, s.k, s.v)
    assert s.gqa.device_status() == PSI_ERR_PAGE_ID
    assert torch.equal(s.buffer.view(torch.uint8), before.view(torch.uint8))
    assert s.gqa.device_status() == 0                       # cleared by the read

    # attention over tokens 0..20 reads logical page 1: flagged (the read went to page 0 instead)
    s.gqa.attend(s.pages, s.table, 0, s.q, s.out)
    assert s.gqa.device_status() == PSI_ERR_PAGE_ID

    # the fused step both reads and writes through the bad entry
    s.gqa.append_attend(s.pages, s.table, 0, s.k, s.v, s.q, s.out)
    assert s.gqa.device_status() == PSI_ERR_PAGE_ID
    assert torch.equal(s.buffer.view(torch.uint8), before.view(torch.uint8))

    # gather of tokens 16..24 leaves its outputs untouched
    k_out = torch.full((8, s.hkv, s.d), 7.0, device="cuda:0", dtype=s.buffer.dtype)
    v_out = torch.full_like(k_out, 7.0)
    s.gqa.page_gather(s.pages, s.table, 0, 0, 16, 24, k_out, v_out)
    assert s.gqa.device_status() == PSI_ERR_PAGE_ID
    assert bool((k_out == 7.0).all()) and bool((v_out == 7.0).all())

    # with the entry repaired the same calls run clean
    s.table.write_row(0, 0, [3, 5, 1, 0])
    s.gqa.append_attend(s.pages, s.table, 0, s.k, s.v, s.q, s.out)
    assert s.gqa.device_status() == 0
    assert not torch.equal(s.buffer.view(torch.uint8), before.view(torch.uint8))
    s.close()



def chunk_kernels_report_an_out_of_range_page_id():
    # a long query run (96 tokens of one request = 12 query tiles of 8 tokens at G = 2) goes to the chunk kernels
    import torch
    for kernel_mode in (pkg.KERNEL_AUTO, pkg.KERNEL_MMA_SYNC):
        s = Small(kernel_mode=kernel_mode, head_dim=128)
        layout = pkg.GQAPageTableLayout(1, 1, 8, 1)
        table = pkg.GQARequestPageTable(s.ctx, layout)
        cfg = pkg.GQAConfig(s.hq, s.hkv, s.d, 0.1, s.page_bytes, pkg.BF16, layout, 96, pkg.PLAN_BALANCED, kernel_mode, 0)
        gqa = pkg.GQA(s.ctx, cfg)
        table.write_row(0, 0, [3, 12, 1, 0, 2, 4, 6, 7])    # 8 logical pages = 128 tokens; logical page 1 is bad
        q = torch.randn((96, s.hq, s.d), device="cuda:0", dtype=torch.float32).to(torch.bfloat16)
        out = torch.zeros_like(q)
        gqa.prepare([0], [32], [0, 96])                     # 96 query tokens at positions 32..127
        assert gqa.plan_stats()["chunk_ctas"] > 0
        gqa.attend(s.pages, table, 0, q, out)
        assert gqa.device_status() == PSI_ERR_PAGE_ID
        table.write_row(0, 0, [3, 5, 1, 0, 2, 4, 6, 7])
        gqa.attend(s.pages, table, 0, q, out)
        assert gqa.device_status() == 0
        s.ctx.sync()
        gqa.close()
        table.close()
        s.close()



def main():
    assert pkg.library_path().name == "libpsi_cuda_checked.so", pkg.library_path()
    for dtype, kernel_mode in ((pkg.BF16, pkg.KERNEL_AUTO), (pkg.BF16, pkg.KERNEL_GENERIC), (pkg.F32, pkg.KERNEL_AUTO)):
        kernels_skip_an_out_of_range_page_id_and_report_it(dtype, kernel_mode)
    chunk_kernels_report_an_out_of_range_page_id()
    print("checked build ok")


if __name__ == "__main__":
    main()
