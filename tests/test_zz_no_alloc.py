"""The allocation-free attention entry point against the ordinary one (collected last on purpose).

psi_gqa_attend_static serves hosts that cannot allocate device memory while running: it keeps its plan, counters and
partial outputs in a fixed array inside the library.  Its output must equal psi_gqa_attend's on the same inputs, on
two calls in a row (the second call meets the first call's leftovers in the shared scratch), and a step that does not
fit the fixed scratch must be refused with a message.
"""
import numpy as np
import pytest

import checks
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


def test_static_attention_matches_the_oracle_and_allocates_nothing():
    # D=256 bf16 through the tensor-core kernel, checked against the CPU oracle itself (not only against the other
    # entry point), and the property the entry point exists for: the device's free memory does not move while it runs.
    import torch
    s = W.Session(W.config(2, scale_down=4))
    s.append()
    s.ctx.sync()
    out = torch.full_like(s.out, float("nan"))
    args = (0, s.stream.cuda_stream, _static_config(s), s.arena, s.table.page_ids_buffer(), *s.spec.batch(), s.spec.layer,
            s.q, out)
    pkg.attend_static(*args)                       # first call on the device: resolves the scratch address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(8):
        pkg.attend_static(*args)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    s.out.copy_(out)
    checks.assert_attention_close(s)
    s.close()


def test_static_attention_at_the_limits_of_its_scratch():
    # 64 CTAs (PSI_STATIC_MAX_CTAS) with every unit cut across CTAs, and a step just under PSI_STATIC_MAX_ITEMS items.
    import torch
    long_spec = W.Spec("static-64-ctas", pkg.BF16, 16, 2, 256, 16, [6000, 7000, 8000, 9000], 1, seed=21)
    many_spec = W.Spec("static-many-items", pkg.BF16, 8, 8, 64, 16, [40] * 56, 1, seed=22)  # 448 units + up to 63 cuts
    for spec in (long_spec, many_spec):
        s = W.Session(spec)
        s.append()
        s.ctx.sync()
        out = torch.full_like(s.out, float("nan"))
        pkg.attend_static(0, s.stream.cuda_stream, _static_config(s), s.arena, s.table.page_ids_buffer(), *spec.batch(),
                          0, s.q, out)
        torch.cuda.synchronize()
        s.out.copy_(out)
        checks.assert_attention_close(s)
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
    with pytest.raises(pkg.PsiError, match="unknown kernel mode"):
        pkg.attend_static(0, s.stream.cuda_stream, _static_config(s, kernel_mode=9), s.arena, s.table.page_ids_buffer(),
                          *spec.batch(), 0, s.q, out)
    f32 = W.Session(W.Spec("f32", pkg.F32, 4, 2, 64, 16, [40], 1, seed=8))
    for mode in (pkg.KERNEL_MMA, pkg.KERNEL_MMA_SYNC):   # refused as psi_gqa_create refuses them, not silently replaced
        with pytest.raises(pkg.PsiError, match="does not support this profile"):
            pkg.attend_static(0, f32.stream.cuda_stream, _static_config(f32, kernel_mode=mode), f32.arena,
                              f32.table.page_ids_buffer(), *f32.spec.batch(), 0, f32.q, f32.out)
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0   # nothing was enqueued
    f32.close()
    s.close()


def test_static_attention_refuses_a_capturing_stream():
    # The plan is uploaded from host memory that is gone when the call returns; a captured call would replay it.
    import torch
    s = W.Session(W.config(2, scale_down=8))
    out = torch.zeros_like(s.out)
    args = (s.arena, s.table.page_ids_buffer(), *s.spec.batch(), s.spec.layer, s.q, out)
    side = pkg.Context(0)                                                # a context with a stream of its own
    pkg.attend_static(0, side.stream, _static_config(s), *args)           # set-up call, outside any capture
    torch.cuda.synchronize()
    side.capture_begin()
    try:
        with pytest.raises(pkg.PsiError, match="cannot be recorded into a stream capture"):
            pkg.attend_static(0, side.stream, _static_config(s), *args)
    finally:
        graph = side.capture_end()
    assert graph.kernel_count() == 0
    graph.close()
    side.close()
    s.close()


def test_static_attention_leaves_the_callers_device_current():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = W.Session(W.config(2, scale_down=8))          # lives on cuda:0
    out = torch.zeros_like(s.out)
    torch.cuda.set_device(1)
    try:
        pkg.attend_static(0, s.stream.cuda_stream, _static_config(s), s.arena, s.table.page_ids_buffer(), *s.spec.batch(),
                          s.spec.layer, s.q, out)
        assert torch.cuda.current_device() == 1
    finally:
        torch.cuda.set_device(0)
    torch.cuda.synchronize()
    s.close()
