"""Writes tests/golden/snapshot_manifest_selected.hex: the manifest of a two-file hibernation snapshot under a Selected
plan, as the library writes it, one annotated field per line.

The manifest is the one part of the snapshot format whose byte encoding comes from a third-party crate (wincode 0.6.1,
configured in crates/inference-executor-metal/src/model/state_snapshot.rs:46-47 as fixed-width native-endian integers,
u32 sequence lengths and u8 enum tags); the reference's tests hold no manifest bytes.  This file is what a Rust-side
test can decode with the reference's own `StateSnapshotManifest` to settle, in one assertion, whether the two writers
agree.  tests/test_snapshot.py checks that the library still writes exactly these bytes.

    python tests/golden/make_manifest_fixture.py
"""
import struct
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import hostapi as H  # noqa: E402

pkg = H.pkg
REQUEST_SLOT_RANGES = [(1, 3)]
PAGE_ID_RANGES = [(0, 2), (5, 6)]
METADATA = struct.pack("<I4I", 4, 3, 5, 8, 13)


def write_snapshot(directory):
    """page-arena (8 entries of 16 bytes, entries 0..2 and 5 selected) + main-gdn-request-state-table (metadata)."""
    plan = pkg.ExecutorHibernationPlan.selected(REQUEST_SLOT_RANGES, PAGE_ID_RANGES)
    files = [pkg.SNAPSHOT_PAGE_ARENA, pkg.SNAPSHOT_MAIN_GDN_REQUEST_STATE_TABLE]
    writer = pkg.StateSnapshotWriter(directory, files, plan)
    writer.write_selected_buffer(pkg.SNAPSHOT_PAGE_ARENA, np.arange(128, dtype=np.uint8), PAGE_ID_RANGES, 16)
    writer.write_metadata(pkg.SNAPSHOT_MAIN_GDN_REQUEST_STATE_TABLE, METADATA)
    writer.commit()
    writer.close()
    return (Path(directory) / "manifest").read_bytes()


def annotate(raw):
    """(hex, meaning) per field, walking the layout documented in INTEGRATION.md."""
    at = 0

    def take(n, meaning):
        nonlocal at
        part = raw[at:at + n]
        at += n
        return part.hex(" "), meaning

    rows = [take(8, 'magic "PSISTATE"'), take(4, "version: u32 = 3")]
    tag = raw[at]
    rows.append(take(1, "plan tag: u8, 0 = All, 1 = Selected"))
    if tag == 1:
        for name in ("request_slot_ranges", "page_id_ranges"):
            count = struct.unpack_from("<I", raw, at)[0]
            rows.append(take(4, f"{name}: u32 count = {count}"))
            for i in range(count):
                begin, end = struct.unpack_from("<II", raw, at)
                rows.append(take(8, f"  range {i}: u32 start = {begin}, u32 end = {end}"))
    count = struct.unpack_from("<I", raw, at)[0]
    rows.append(take(4, f"files: u32 count = {count}"))
    for i in range(count):
        file, kind, payload = struct.unpack_from("<BBQ", raw, at)
        rows.append(take(10, f"  entry {i}: u8 file = {file}, u8 kind = {kind} (0 buffer, 1 metadata), u64 payload_bytes = {payload}"))
    assert at == len(raw)
    return rows


def main():
    with tempfile.TemporaryDirectory() as tmp:
        raw = write_snapshot(Path(tmp) / "snapshot")
    lines = ["# manifest of a two-file Selected snapshot; `hex bytes | meaning`; integers little endian (native on x86-64 / aarch64)"]
    lines += [f"{hexed} | {meaning}" for hexed, meaning in annotate(raw)]
    (Path(__file__).resolve().parent / "snapshot_manifest_selected.hex").write_text("\n".join(lines) + "\n")
    print(f"{len(raw)} bytes")


if __name__ == "__main__":
    main()
