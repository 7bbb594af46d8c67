"""Hibernation of the device page arena and request page table through snapshot directories, then attention on the
restored state (crates/inference-executor-metal/src/model/state_snapshot.rs, page_arena.rs release / allocate)."""
import numpy as np
import pytest

import checks
import gpuharness as G

pkg = G.pkg
pytestmark = pytest.mark.gpu
FILES = [pkg.SNAPSHOT_PAGE_ARENA, pkg.SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE]


def _rig(seed):
    import torch
    hq, hkv, d, p = 8, 2, 128, 16
    rig = G.Rig(pkg.BF16, hq, hkv, d, p, 1.0 / np.sqrt(d), (6, 2, 5, 2), 16, num_pages=40)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    rig.arena.copy_(torch.randn(rig.arena.shape, device="cuda", generator=gen).to(torch.bfloat16))
    rng = np.random.default_rng(seed)
    ids = rng.permutation(40).astype(np.uint32)
    for slot in range(6):
        for layer in range(2):
            rig.set_pages(slot, layer, ids[(slot * 3 + layer * 17) % 30:][:10])
    return rig


def _attend(rig, layer):
    import torch
    q = torch.randn((4, rig.hq, rig.d), device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)).to(torch.bfloat16)
    out = torch.empty_like(q)
    rig.gqa.prepare([0, 2, 5], [37, 90, 140], [0, 1, 3, 4])  # one, two and one query tokens
    rig.gqa.attend(rig.pages, rig.table, layer, q, out)
    rig.ctx.sync()
    return out


def test_full_snapshot_restores_arena_and_table(tmp_path):
    import torch
    src = _rig(1)
    path = tmp_path / "full"
    writer = pkg.StateSnapshotWriter(path, FILES, pkg.ExecutorHibernationPlan.all())
    writer.write_pages(pkg.SNAPSHOT_PAGE_ARENA, src.pages)
    writer.write_table(pkg.SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE, src.table)
    writer.commit()
    assert (path / "page-arena").stat().st_size == src.num_pages * src.page_bytes
    assert (path / "main-gqa-request-page-table").stat().st_size == 6 * 2 * 5 * 2 * 4
    assert (path / "page-arena").read_bytes() == checks.to_numpy_bits(src.arena).tobytes()

    dst = _rig(2)  # different contents and table
    reader = pkg.StateSnapshotReader(path, FILES, pkg.ExecutorHibernationPlan.all())
    reader.read_pages(pkg.SNAPSHOT_PAGE_ARENA, dst.pages)
    reader.read_table(pkg.SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE, dst.table)
    reader.finish()
    assert torch.equal(dst.arena.view(torch.int16), src.arena.view(torch.int16))
    for slot in range(6):
        for layer in range(2):
            for block in range(5):
                assert dst.table.read_page_ids(slot, layer, block) == src.table.read_page_ids(slot, layer, block)
    # the restored state serves attention exactly like the original
    out_src = _attend(src, 1)
    out_dst = _attend(dst, 1)
    assert torch.equal(out_src.view(torch.int16), out_dst.view(torch.int16))
    src.close()
    dst.close()


def test_selected_snapshot_touches_only_the_planned_pages_and_slots(tmp_path):
    import torch
    src = _rig(3)
    plan = pkg.ExecutorHibernationPlan.selected([(1, 3), (5, 6)], [(0, 4), (10, 11), (30, 40)])
    path = tmp_path / "selected"
    writer = pkg.StateSnapshotWriter(path, FILES, plan)
    writer.write_pages(pkg.SNAPSHOT_PAGE_ARENA, src.pages)
    writer.write_table(pkg.SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE, src.table)
    writer.commit()
    assert (path / "page-arena").stat().st_size == 15 * src.page_bytes
    assert (path / "main-gqa-request-page-table").stat().st_size == 3 * 2 * 5 * 2 * 4

    dst = _rig(4)
    before = dst.arena.clone()
    before_rows = {(s, l, b): dst.table.read_page_ids(s, l, b) for s in range(6) for l in range(2) for b in range(5)}
    reader = pkg.StateSnapshotReader(path, FILES, plan)
    reader.read_pages(pkg.SNAPSHOT_PAGE_ARENA, dst.pages)
    reader.read_table(pkg.SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE, dst.table)
    reader.finish()
    planned_pages = set(range(0, 4)) | {10} | set(range(30, 40))
    for page in range(40):
        want = src.arena[page] if page in planned_pages else before[page]
        assert torch.equal(dst.arena[page].view(torch.int16), want.view(torch.int16)), page
    for (s, l, b), old in before_rows.items():
        want = src.table.read_page_ids(s, l, b) if s in (1, 2, 5) else old
        assert dst.table.read_page_ids(s, l, b) == want
    with pytest.raises(pkg.PsiError, match="plan does not match"):
        pkg.StateSnapshotReader(path, FILES, pkg.ExecutorHibernationPlan.all())
    src.close()
    dst.close()
