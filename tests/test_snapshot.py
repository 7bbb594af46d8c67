"""Hibernation snapshot directories through the C ABI, after the reference's own tests
(crates/inference-executor-metal/src/model/state_snapshot.rs:883-1380); host buffers only, no GPU."""
import struct

import numpy as np
import pytest

import hostapi as H

pkg = H.pkg
PAGE_ARENA, GQA_TABLE = pkg.SNAPSHOT_PAGE_ARENA, pkg.SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE
GDN_TABLE = pkg.SNAPSHOT_MAIN_GDN_REQUEST_STATE_TABLE
Plan = pkg.ExecutorHibernationPlan
U32_MAX = 0xFFFFFFFF


def manifest_bytes(plan, files):
    """Independent restatement of the manifest layout: magic, u32 version, u8 plan tag (+ two u32-counted lists of
    (u32, u32) ranges), u32-counted list of (u8 file, u8 kind, u64 payload bytes); little endian."""
    out = b"PSISTATE" + struct.pack("<I", 3)
    if plan.is_selected:
        out += b"\x01"
        for ranges in (plan.request_slot_ranges, plan.page_id_ranges):
            out += struct.pack("<I", len(ranges)) + b"".join(struct.pack("<II", b, e) for b, e in ranges)
    else:
        out += b"\x00"
    out += struct.pack("<I", len(files))
    for file, kind, payload in files:
        out += struct.pack("<BBQ", file, kind, payload)
    return out


def test_directory_snapshot_unload_load(tmp_path):
    source = (np.arange(4096) % 251).astype(np.uint8)
    restored = np.zeros_like(source)
    metadata = struct.pack("<I4I", 4, 3, 5, 8, 13)
    path = tmp_path / "nested" / "unload-load"
    writer = pkg.StateSnapshotWriter(path, [PAGE_ARENA, GDN_TABLE], Plan.all())
    writer.write_full_buffer(PAGE_ARENA, source)
    writer.write_metadata(GDN_TABLE, metadata)
    writer.commit()
    writer.close()
    assert sorted(p.name for p in path.iterdir()) == ["main-gdn-request-state-table", "manifest", "page-arena"]
    assert (path / "manifest").read_bytes() == manifest_bytes(Plan.all(), [(0, 0, 4096), (2, 1, len(metadata))])
    assert not [p for p in path.parent.iterdir() if p.name.startswith(".")]  # the temporary directory is gone

    reader = pkg.StateSnapshotReader(path, [PAGE_ARENA, GDN_TABLE], Plan.all())
    reader.read_full_buffer(PAGE_ARENA, restored)
    assert reader.read_metadata(GDN_TABLE) == metadata
    reader.finish()
    assert np.array_equal(restored, source)


def test_selected_buffer_entries_unload_load(tmp_path):
    source = np.arange(10, 18, dtype=np.uint32)
    restored = np.full(8, U32_MAX, dtype=np.uint32)
    entry_ranges = [(1, 3), (5, 6)]
    plan = Plan.selected([(3, 4)], entry_ranges)
    path = tmp_path / "selected-buffer-entries"
    writer = pkg.StateSnapshotWriter(path, [PAGE_ARENA], plan)
    writer.write_selected_buffer(PAGE_ARENA, source, entry_ranges, 4)
    writer.commit()
    assert (path / "page-arena").stat().st_size == 12
    assert (path / "manifest").read_bytes() == manifest_bytes(plan, [(0, 0, 12)])
    reader = pkg.StateSnapshotReader(path, [PAGE_ARENA], plan)
    reader.read_selected_buffer(PAGE_ARENA, restored, entry_ranges, 4)
    reader.finish()
    assert restored.tolist() == [U32_MAX, 11, 12, U32_MAX, U32_MAX, 15, U32_MAX, U32_MAX]


def test_selected_buffer_entries_reject_bad_ranges(tmp_path):
    source = np.arange(8, dtype=np.uint32)
    for ranges in ([(1, 3), (3, 4)], [(2, 2)], [(4, 6), (1, 2)]):
        writer = pkg.StateSnapshotWriter(tmp_path / "bad", [PAGE_ARENA], Plan.selected([], []))
        with pytest.raises(pkg.PsiError, match="nonempty, sorted, disjoint, and nonadjacent"):
            writer.write_selected_buffer(PAGE_ARENA, source, ranges, 4)
        writer.close()
    writer = pkg.StateSnapshotWriter(tmp_path / "bad", [PAGE_ARENA], Plan.selected([], []))
    with pytest.raises(pkg.PsiError, match="out of bounds"):
        writer.write_selected_buffer(PAGE_ARENA, source, [(7, 9)], 4)
    writer.close()
    assert not list(tmp_path.iterdir())  # abandoned writers leave nothing behind


def test_empty_selected_buffer_unload_load(tmp_path):
    source = np.arange(8, dtype=np.uint32)
    plan = Plan.selected([], [])
    path = tmp_path / "empty-selected"
    writer = pkg.StateSnapshotWriter(path, [PAGE_ARENA], plan)
    writer.write_selected_buffer(PAGE_ARENA, source, [], 4)
    writer.commit()
    assert (path / "page-arena").stat().st_size == 0
    restored = np.full(8, 7, dtype=np.uint32)
    reader = pkg.StateSnapshotReader(path, [PAGE_ARENA], plan)
    reader.read_selected_buffer(PAGE_ARENA, restored, [], 4)
    reader.finish()
    assert restored.tolist() == [7] * 8


def _write(path, plan, payload=None):
    writer = pkg.StateSnapshotWriter(path, [PAGE_ARENA], plan)
    payload = np.arange(16, dtype=np.uint8) if payload is None else payload
    if plan.is_selected:
        writer.write_selected_buffer(PAGE_ARENA, payload, plan.page_id_ranges, 1)
    else:
        writer.write_full_buffer(PAGE_ARENA, payload)
    writer.commit()
    writer.close()


def test_reader_rejects_mismatched_plan_and_file_sets(tmp_path):
    path = tmp_path / "snap"
    _write(path, Plan.selected([(0, 2)], [(1, 3)]))
    with pytest.raises(pkg.PsiError, match="plan does not match"):
        pkg.StateSnapshotReader(path, [PAGE_ARENA], Plan.all())
    with pytest.raises(pkg.PsiError, match="plan does not match"):
        pkg.StateSnapshotReader(path, [PAGE_ARENA], Plan.selected([(0, 2)], [(1, 4)]))
    with pytest.raises(pkg.PsiError, match="file is missing: file=MainGQARequestPageTable"):
        pkg.StateSnapshotReader(path, [PAGE_ARENA, GQA_TABLE], Plan.selected([(0, 2)], [(1, 3)]))
    with pytest.raises(pkg.PsiError, match="file is missing: file=MainGQARequestPageTable"):  # missing is reported first
        pkg.StateSnapshotReader(path, [GQA_TABLE], Plan.selected([(0, 2)], [(1, 3)]))
    with pytest.raises(pkg.PsiError, match="contains duplicates"):
        pkg.StateSnapshotReader(path, [PAGE_ARENA, PAGE_ARENA], Plan.all())
    with pytest.raises(pkg.PsiError, match="must not be empty"):
        pkg.StateSnapshotReader(path, [], Plan.all())
    with pytest.raises(pkg.PsiError, match="request slot ranges must be nonempty, sorted"):
        pkg.StateSnapshotReader(path, [PAGE_ARENA], Plan.selected([(2, 2)], []))
    reader = pkg.StateSnapshotReader(path, [PAGE_ARENA], Plan.selected([(0, 2)], [(1, 3)]))
    with pytest.raises(pkg.PsiError, match="was not read: file=PageArena"):
        reader.finish()
    target = np.zeros(16, dtype=np.uint8)
    with pytest.raises(pkg.PsiError, match="length mismatch: file=PageArena expected=16 actual=2"):
        reader.read_full_buffer(PAGE_ARENA, target)
    reader.read_selected_buffer(PAGE_ARENA, target, [(1, 3)], 1)
    with pytest.raises(pkg.PsiError, match="read twice"):
        reader.read_selected_buffer(PAGE_ARENA, target, [(1, 3)], 1)
    with pytest.raises(pkg.PsiError, match="file is missing: file=MainGQARequestPageTable"):
        reader.read_full_buffer(GQA_TABLE, target)
    reader.finish()
    assert target.tolist() == [0, 1, 2] + [0] * 13


def test_reader_rejects_damaged_directories(tmp_path):
    plan = Plan.all()
    path = tmp_path / "snap"
    _write(path, plan)
    good = (path / "manifest").read_bytes()
    assert good == manifest_bytes(plan, [(0, 0, 16)])

    def reopen(match):
        with pytest.raises(pkg.PsiError, match=match):
            pkg.StateSnapshotReader(path, [PAGE_ARENA], plan)

    (path / "manifest").write_bytes(good + b"\x00")
    reopen("trailing bytes")
    (path / "manifest").write_bytes(good[:-3])
    reopen("unable to decode model state manifest")
    (path / "manifest").write_bytes(b"PSISTATX" + good[8:])
    reopen("magic mismatch")
    (path / "manifest").write_bytes(good[:8] + struct.pack("<I", 2) + good[12:])
    reopen("version mismatch: expected=3 actual=2")
    (path / "manifest").write_bytes(manifest_bytes(plan, []))
    reopen("must contain at least one file")
    (path / "manifest").write_bytes(manifest_bytes(plan, [(1, 0, 4), (0, 0, 16)]))
    reopen("unique and sorted")
    (path / "manifest").write_bytes(manifest_bytes(plan, [(0, 1, 16)]))
    reopen("kind does not match")
    (path / "manifest").write_bytes(manifest_bytes(Plan.selected([(1, 2), (2, 3)], []), [(0, 0, 16)]))
    reopen("request slot ranges must be nonempty, sorted")
    (path / "manifest").write_bytes(manifest_bytes(plan, [(0, 0, 17)]))
    reopen("length mismatch: file=PageArena expected=17 actual=16")
    (path / "manifest").write_bytes(good)
    (path / "stray").write_bytes(b"x")
    reopen("unexpected file")
    (path / "stray").unlink()
    (path / "page-arena").unlink()
    reopen("file is missing")
    (path / "page-arena").mkdir()
    reopen("must be a regular file")
    (path / "page-arena").rmdir()
    (path / "page-arena").write_bytes(bytes(16))
    pkg.StateSnapshotReader(path, [PAGE_ARENA], plan).close()
    with pytest.raises(pkg.PsiError, match="must be a directory"):
        pkg.StateSnapshotReader(path / "manifest", [PAGE_ARENA], plan)
    with pytest.raises(pkg.PsiError, match="unable to inspect model state snapshot"):
        pkg.StateSnapshotReader(tmp_path / "absent", [PAGE_ARENA], plan)


def test_writer_contracts(tmp_path):
    data = np.arange(16, dtype=np.uint8)
    path = tmp_path / "snap"
    _write(path, Plan.all())
    with pytest.raises(pkg.PsiError, match="destination already exists"):
        pkg.StateSnapshotWriter(path, [PAGE_ARENA], Plan.all())
    writer = pkg.StateSnapshotWriter(tmp_path / "second", [PAGE_ARENA, GDN_TABLE], Plan.all())
    with pytest.raises(pkg.PsiError, match="does not contain metadata: file=PageArena"):
        writer.write_metadata(PAGE_ARENA, b"abc")
    with pytest.raises(pkg.PsiError, match="does not contain a buffer: file=MainGDNRequestStateTable"):
        writer.write_full_buffer(GDN_TABLE, data)
    with pytest.raises(pkg.PsiError, match="metadata must not be empty"):
        writer.write_metadata(GDN_TABLE, b"")
    with pytest.raises(pkg.PsiError, match="buffer must not be empty"):
        writer.write_full_buffer(PAGE_ARENA, data[:0])
    writer.write_full_buffer(PAGE_ARENA, data)
    with pytest.raises(pkg.PsiError, match="written twice: file=PageArena"):
        writer.write_full_buffer(PAGE_ARENA, data)
    with pytest.raises(pkg.PsiError, match="file is missing: file=MainGDNRequestStateTable"):
        writer.commit()
    writer.close()
    assert sorted(p.name for p in tmp_path.iterdir()) == ["snap"]
    writer = pkg.StateSnapshotWriter(tmp_path / "third", [PAGE_ARENA], Plan.all())
    writer.write_full_buffer(PAGE_ARENA, data)
    writer.write_full_buffer(GQA_TABLE, data)
    with pytest.raises(pkg.PsiError, match="unexpected file: file=MainGQARequestPageTable"):
        writer.commit()
    writer.close()
    with pytest.raises(pkg.PsiError, match="page ID ranges must be nonempty, sorted"):
        pkg.StateSnapshotWriter(tmp_path / "fourth", [PAGE_ARENA], Plan.selected([], [(3, 5), (5, 6)]))


def test_manifest_bytes_match_the_committed_fixture(tmp_path):
    # tests/golden/snapshot_manifest_selected.hex is the byte-for-byte manifest of a two-file Selected snapshot, one
    # annotated field per line, kept so that a Rust-side test can decode it with the reference's own manifest type;
    # here: the library still writes exactly those bytes, and they are what the independent restatement above gives.
    import importlib.util
    from pathlib import Path
    golden = Path(__file__).resolve().parent / "golden"
    spec = importlib.util.spec_from_file_location("make_manifest_fixture", golden / "make_manifest_fixture.py")
    maker = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(maker)
    raw = maker.write_snapshot(tmp_path / "snapshot")
    stored = b"".join(bytes.fromhex(line.split("|")[0]) for line in
                      (golden / "snapshot_manifest_selected.hex").read_text().splitlines() if not line.startswith("#"))
    assert raw == stored
    plan = Plan.selected(maker.REQUEST_SLOT_RANGES, maker.PAGE_ID_RANGES)
    assert raw == manifest_bytes(plan, [(0, 0, 3 * 16), (2, 1, len(maker.METADATA))])
