"""The allocation-free attention entry point against the ordinary one (collected last on purpose).

psi_gqa_attend_static serves hosts that cannot allocate device memory while running: it keeps its plan, counters and
partial outputs in a fixed array inside the library.  Its output must equal psi_gqa_attend's on the same inputs, on
two calls in a row (the second call meets the first call's leftovers in the shared scratch), and a step that does not
fit the fixed scratch must be refused with a message.
"""
import numpy as np
import pytest

import workloads as W

pkg = W.pkg
pytestmark = pytest.mark.gpu


def _static_config(s, kernel_mode=pkg.KERNEL_AUTO):
    spec = s.spec
    return pkg.GQAConfig(spec.num_q_heads, spec.num_kv_heads, spec.head_dim, spec.scale, spec.page_bytes, spec.dtype,
                         s.layout, spec.num_tokens, pkg.PLAN_BALANCED, kernel_mode, 0)


@pytest.mark.parametrize("index,scale_down,kernel_mode", [
    (4, 64, pkg.KERNEL_AUTO),      # few long sequences: every unit is cut across CTAs, so partial slots are exercised
    (2, 8, pkg.KERNEL_AUTO),       # ragged decode batch
    (3, 16, pkg.KERNEL_GENERIC),   # two query tokens per sequence through the generic kernel and its reduce pass
])
def test_static_attention_matches_the_allocating_entry_point_twice(index, scale_down, kernel_mode):
    import torch
    s = W.Session(W.config(index, scale_down=scale_down), kernel_mode=kernel_mode)
    s.append()
    s.attend()
    s.ctx.sync()
    reference = s.out.float().cpu().numpy()
    for call in range(2):
        out = torch.full_like(s.out, float("nan"))
        pkg.attend_static(0, s.stream.cuda_stream, _static_config(s, kernel_mode), s.arena, s.table.page_ids_buffer(),
                          *s.spec.batch(), s.spec.layer, s.q, out)
        torch.cuda.synchronize()
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all(), f"call {call}: output rows were not written"
        diff = np.abs(got - reference)
        assert diff.max() <= 2e-2 and diff.mean() <= 2e-3, (call, diff.max(), diff.mean())
    s.close()


def test_static_attention_refuses_a_step_beyond_its_scratch():
    import torch
    spec = W.Spec("too-many-units", pkg.BF16, 8, 8, 64, 16, [40] * 80, 1, seed=7)   # 80 tiles x 8 KV heads = 640 items
    s = W.Session(spec)
    out = torch.zeros_like(s.out)
    with pytest.raises(pkg.PsiError, match="work items; the static scratch holds 512") as err:
        pkg.attend_static(0, s.stream.cuda_stream, _static_config(s), s.arena, s.table.page_ids_buffer(),
                          *spec.batch(), 0, s.q, out)
    assert err.value.status == 1
    big = pkg.GQAConfig(8, 8, 512, 0.1, 2 * 8 * 16 * 512 * 2, pkg.BF16, s.layout, 1, 0, 0, 0)
    with pytest.raises(pkg.PsiError, match="head_dim exceeds the static scratch"):
        pkg.attend_static(0, s.stream.cuda_stream, big, s.arena, s.table.page_ids_buffer(), [0], [0], [0, 1], 0, s.q, out)
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0   # nothing was enqueued
    s.close()
