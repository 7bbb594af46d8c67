"""Test-side entry to the synthetic workloads: re-exports the package's generator and adds the smoke check."""
from __future__ import annotations

import __graft_entry__ as entry

pkg = entry.load_package()
from psi_dec_b200 import workloads as W  # noqa: E402

config = W.config
Spec = W.Spec
Session = W.Session


def smoke_check():
    from oracle import harness
    harness.smoke_check()
