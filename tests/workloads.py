"""Test-side entry to the synthetic workloads: re-exports the package's generator and adds the smoke check."""
from __future__ import annotations

import __graft_entry__ as entry

pkg = entry.load_package()
from psi_dec_b200 import workloads as W  # noqa: E402

config = W.config
Spec = W.Spec
Session = W.Session


def smoke_check():
    """Configuration 1 (batch 1, 4/1 heads, D128, fp16, 256+1 tokens in 16-token pages) on cuda:0: append one token,
    attend over 257, compare page contents bit-exactly and the output within tolerance against the CPU oracle."""
    import numpy as np
    import checks
    s = Session(config(1))
    before = checks.to_numpy_bits(s.arena)
    s.step()
    s.ctx.sync()
    expected = checks.expected_arena_after_append(s, before)
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), expected), "append differs from the oracle"
    max_abs, mean_abs = checks.assert_attention_close(s)
    stats = s.gqa.plan_stats()
    launches = s.ctx.launch_count
    s.close()
    print(f"smoke ok: max_abs={max_abs:.3e} mean_abs={mean_abs:.3e} plan={stats} launches={launches}")
