"""Pins the CPU oracle against the known-answer and golden vectors of the reference's own tests (no GPU)."""
import math

import numpy as np
import pytest

from oracle import psi_oracle as O

U32_MAX = O.U32_MAX


def test_causal_attention_closed_form():
    # crates/inference-executor-core/src/attn/gqa/reference.rs:84-115
    out = O.projected_gqa_reference(2, 1, 2, 1.0, [0, 2], [0], [1, 0, 1, 0, 0, 2, 0, 2], [[1, 0, 0, 1]],
                                    [[10, 0, 0, 20]])
    f = np.float32
    first = np.exp(f(-2.0), dtype=np.float32)  # the reference forms the expectation in f32 arithmetic
    total = f(first + f(1.0))
    w0, w1 = f(first / total), f(f(1.0) / total)
    expected = np.array([10, 0, 10, 0, f(10) * w0, f(20) * w1, f(10) * w0, f(20) * w1], dtype=np.float32)
    assert np.max(np.abs(out - expected)) < 1e-6


def test_softmax_reference_normalizes_logits():
    # crates/inference-executor-core/src/reference.rs:110-116
    out = O.softmax([0.0, math.log(3.0)])
    assert abs(out[0] - 0.25) < 1e-6 and abs(out[1] - 0.75) < 1e-6
    with pytest.raises(AssertionError):
        O.softmax([float("nan")])


@pytest.mark.parametrize("np_dtype", [np.uint16, np.float32])
def test_kv_page_write_fixed(np_dtype):
    # crates/inference-backend-metal/src/components/gqa_kv_page_write.rs:344-364
    pages = np.zeros(8, dtype=np_dtype)
    O.kv_page_write(pages, np.array([10, 11], np_dtype), np.array([20, 21], np_dtype), [0], [1], [0], 1, 0,
                    O.Layout(1, 1, 1, 1), 1, 2, pages.nbytes)
    assert pages.tolist() == [0, 0, 10, 11, 0, 0, 20, 21]


def test_kv_page_write_bucketed_preserves_inactive_page():
    # gqa_kv_page_write.rs:284-342: 3 of 4 writes leave page 1 untouched; the 4th touches it.
    sentinel = 0x7777
    layout = O.Layout(2, 1, 1, 1)
    k = np.arange(10, 18, dtype=np.uint16)
    v = np.arange(20, 28, dtype=np.uint16)
    pages = np.full(32, sentinel, dtype=np.uint16)
    O.kv_page_write(pages, k, v, [0, 0, 0, 1], [0, 1, 2, 0], [0, 1], 3, 0, layout, 1, 2, 32)
    assert pages[16:].tolist() == [sentinel] * 16
    assert pages[:16].tolist() == [10, 11, 12, 13, 14, 15, sentinel, sentinel, 20, 21, 22, 23, 24, 25, sentinel,
                                   sentinel]
    pages[:] = sentinel
    O.kv_page_write(pages, k, v, [0, 0, 0, 1], [0, 1, 2, 0], [0, 1], 4, 0, layout, 1, 2, 32)
    assert pages[16:18].tolist() == [16, 17] and pages[24:26].tolist() == [26, 27]


def test_page_gather_inverts_write_with_two_level_table():
    rng = np.random.default_rng(7)
    hkv, d, p, ipb, blocks = 2, 4, 4, 2, 3
    page_bytes = 2 * hkv * p * d * 2
    layout = O.Layout(2, 2, blocks, ipb)
    table = rng.permutation(2 * 2 * blocks * ipb).astype(np.uint32)
    pages = np.zeros(len(table) * page_bytes // 2, dtype=np.uint16)
    n = 19
    k = rng.integers(0, 65535, size=(n, hkv, d)).astype(np.uint16)
    v = rng.integers(0, 65535, size=(n, hkv, d)).astype(np.uint16)
    O.kv_page_write(pages, k, v, [1] * n, list(range(n)), table, n, 1, layout, hkv, d, page_bytes)
    gk, gv = O.page_gather(pages, table, 1, 1, layout, hkv, d, page_bytes, 3, n)
    assert np.array_equal(gk, k[3:]) and np.array_equal(gv, v[3:])


def test_metadata_golden_vectors():
    # crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs:549-613
    md = O.Metadata(8)
    single = O.single_q_variant(8, 32, 1)
    tiled = O.tiled_q_variant(8, 4, 1)
    rs, ti, cu = [2, 5], [7, 20], [0, 2, 5]
    shape = md.update(rs, ti, cu, single)
    assert md.req_slots[:5].tolist() == [2, 2, 5, 5, 5]
    assert md.flat_token_indices[:5].tolist() == [7, 8, 20, 21, 22]
    assert md.kv_splits[:24].tolist() == [0, 0, 8, 1, 0, 9, 2, 0, 8, 2, 8, 21, 3, 0, 8, 3, 8, 22, 4, 0, 8, 4, 8, 23]
    assert md.cu_kv_splits[:6].tolist() == [0, 1, 2, 4, 6, 8]
    assert shape.as_tuple() == (5, 5, 5, 5, 8, 8, 1)
    shape = md.update(rs, ti, cu, tiled)
    assert md.q_token_tiles[:4].tolist() == [0, 2, 2, 5]
    assert md.kv_splits[:12].tolist() == [0, 0, 9, 1, 0, 12, 1, 12, 23, U32_MAX, U32_MAX, U32_MAX]
    assert md.cu_kv_splits[:3].tolist() == [0, 1, 3]
    assert shape.as_tuple() == (5, 5, 2, 2, 3, 4, 1)
    assert md.update(rs, ti, cu, tiled, mode=O.CAP_BUCKETED).as_tuple() == (5, 6, 2, 2, 3, 4, 1)
    assert md.update(rs, ti, cu, tiled, mode=O.CAP_CALLER_TOKENS, caller_tokens=5).as_tuple() == (5, 5, 2, 2, 3, 4, 1)


def test_metadata_bucketed_preserves_poisoned_tail():
    # batch_metadata.rs:617-648
    md = O.Metadata(12)
    md.q_token_tiles[:] = 0xA5A5A5A5
    md.kv_splits[:] = 0xB6B6B6B6
    md.cu_kv_splits[:] = 0xC7C7C7C7
    shape = md.update([2, 5, 7], [0, 0, 0], [0, 4, 8, 9], O.tiled_q_variant(8, 4, 1), mode=O.CAP_BUCKETED)
    assert shape.as_tuple() == (9, 12, 3, 4, 3, 4, 1)
    assert md.q_token_tiles[6:8].tolist() == [0xA5A5A5A5] * 2
    assert md.kv_splits[9:12].tolist() == [U32_MAX] * 3
    assert md.cu_kv_splits[4] == 0xC7C7C7C7


def test_metadata_caller_capacity_contract():
    # batch_metadata.rs:650-678
    md = O.Metadata(12)
    with pytest.raises(AssertionError, match="code 6"):
        md.update([0], [0], [0, 5], O.single_q_variant(8), mode=O.CAP_CALLER_TOKENS, caller_tokens=4)
    with pytest.raises(AssertionError, match="code 7"):
        md.update([0], [0], [0, 5], O.single_q_variant(8), mode=O.CAP_CALLER_TOKENS, caller_tokens=13)


def test_bucket_policy_vectors():
    # crates/inference-executor-core/src/replay.rs:94-180
    base = [1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 56, 64]
    assert O.bucket_policy(64) == base
    assert O.bucket_policy(128) == base + [80, 96, 112, 128]
    assert O.bucket_policy(70)[-1] == 70
    assert O.bucket_policy(6) == [1, 2, 4, 6]
    for cap in [65, 79, 80, 81, 127, 128, 129, U32_MAX]:
        b = O.bucket_policy(cap)
        assert b[-1] == cap and O.bucket_capacity(b, cap) == cap
        assert all(x < y for x, y in zip(b, b[1:]))
    b64 = O.bucket_policy(64)
    assert [O.bucket_capacity(b64, a) for a in (1, 3, 5, 9, 25, 64)] == [1, 4, 6, 12, 32, 64]
    bt = O.bucket_policy(64, [5, 6, 10, 12, 18])
    assert 0 not in bt
    assert [O.bucket_capacity(bt, a) for a in (5, 9, 10, 11, 17, 18)] == [5, 9, 11, 11, 17, 20]
    assert O.bucket_policy(6, [1]) == [1, 2, 4, 6]
    b8 = O.bucket_policy(8, [6])
    assert b8 == [1, 2, 4, 5, 6, 8]
    assert [O.bucket_capacity(b8, a) for a in (5, 6, 7)] == [5, 6, 8]
    b256 = O.bucket_policy(256)
    for active in range(1, 257):
        total = O.bucket_capacity(b256, active)
        assert (total - active) * 4 <= total
    with pytest.raises(AssertionError, match="exceeds capacity"):
        O.bucket_capacity(O.bucket_policy(6), 7)


def _cfg(head_dim, group, tokens_per_page):
    hkv = 2
    return dict(io_dtype=O.BF16, page_bytes=2 * hkv * head_dim * tokens_per_page * 2, num_q_heads=hkv * group,
                num_kv_heads=hkv, head_dim=head_dim)


def test_split_kv_variant_selection_matrix():
    # crates/inference-backend-metal/src/components/gqa_split_kv.rs:177-231
    sel = lambda cfg, t, tiles, **kw: O.split_kv_select(num_tokens=t, num_q_token_tiles=tiles, **cfg, **kw)
    v, mq = sel(_cfg(256, 6, 16), 4, 4)
    assert mq == 8 and v.as_tuple() == (0, 0, 256, 256, 6)
    assert sel(_cfg(256, 6, 8), 4, 4)[1] == 8
    assert sel(_cfg(256, 6, 16), 8, 4)[0].as_tuple() == (1, 8, 16, 0, 3)
    assert sel(_cfg(256, 6, 16), 16, 4)[0].as_tuple() == (1, 8, 16, 0, 6)
    assert sel(_cfg(256, 6, 8), 16, 4)[0].as_tuple() == (1, 8, 16, 0, 6)
    assert sel(_cfg(128, 8, 8), 8, 4)[0].as_tuple() == (1, 8, 16, 0, 8)
    v, mq = sel(_cfg(256, 8, 4), 16, 4)
    assert mq == 1 and v.tiled_q == 0
    v, mq = sel(_cfg(128, 8, 8), 16, 4, dspark_history=True)
    assert mq == 1 and v.tiled_q == 0


def test_allocator_vectors():
    # crates/inference-runtime-core/src/memory/u32_id_allocator.rs:179-217
    a = O.Allocator(65)
    assert a.bitmap() == [0, 0]
    first, second = a.alloc_one(), a.alloc_one()
    assert (first, second) == (0, 1) and a.bitmap() == [0b11, 0]
    a.free_many([first])
    assert a.bitmap() == [0b10, 0]
    a.free_many([second])
    assert a.bitmap() == [0, 0]
    b = O.Allocator(130)
    ids = b.alloc_many(66)
    full = (1 << 64) - 1
    assert b.bitmap() == [full, 0b11, 0]
    b.free_many([1, 63, 64, 65])
    assert b.bitmap() == [full & ~(0b10 | (1 << 63)), 0, 0]
    assert sorted(b.alloc_many(4)) == [1, 63, 64, 65]
    assert b.bitmap() == [full, 0b11, 0]
    b.free_many(ids)
    assert b.bitmap() == [0, 0, 0]
    with pytest.raises(MemoryError):
        O.Allocator(3).alloc_many(4)


def test_bf16_and_f16_rounding_hand_values():
    # IEEE round-to-nearest-even; the reference relies on crate `half` for the same behaviour.
    L = O.lib()
    assert L.psi_oracle_f32_to_bf16(1.0) == 0x3F80
    assert L.psi_oracle_f32_to_bf16(np.float32(1.00390625)) == 0x3F80      # tie -> even
    assert L.psi_oracle_f32_to_bf16(np.float32(1.01171875)) == 0x3F82      # tie -> even (up)
    assert L.psi_oracle_f32_to_bf16(np.float32(1.0039063692092896)) == 0x3F81
    assert L.psi_oracle_f32_to_f16(1.0) == 0x3C00
    assert L.psi_oracle_f32_to_f16(65504.0) == 0x7BFF
    assert L.psi_oracle_f32_to_f16(65520.0) == 0x7C00
    assert L.psi_oracle_f32_to_f16(np.float32(5.9604645e-08)) == 0x0001
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(20000) * 4).astype(np.float32)
    assert np.array_equal(O.encode(x, O.F16), x.astype(np.float16).view(np.uint16))
    assert np.array_equal(O.decode(x.astype(np.float16).view(np.uint16), O.F16), x.astype(np.float16).astype(np.float32))
    import torch
    tb = torch.from_numpy(x).to(torch.bfloat16)
    assert np.array_equal(O.encode(x, O.BF16), tb.view(torch.int16).numpy().view(np.uint16))


def test_paged_attention_matches_contiguous_reference_and_merge():
    from refdata import generated_values, kv_page_values
    hq, hkv, d, p = 4, 2, 2, 4
    page_bytes = 2 * hkv * p * d * 4
    q = generated_values(3 * hq * d, 0xD2056AB9)
    stride = hkv * d
    r0k, r0v = generated_values(2 * stride, 0xD2056ABA), generated_values(2 * stride, 0xD2056ABB)
    r1k, r1v = generated_values(2 * stride, 0xD2056ABC), generated_values(2 * stride, 0xD2056ABD)
    pages = kv_page_values(hkv, d, p, [(r0k, r0v), (r1k, r1v)]).ravel()
    layout = O.Layout(2, 1, 1, 1)
    out, mx, sm = O.paged_attention(pages, O.F32, q, [0, 1, 1], [1, 0, 1], [0, 1], 0, layout, hq, hkv, d, page_bytes,
                                    0.5, want_stats=True)
    ref = O.projected_gqa_reference(hq, hkv, d, 0.5, [0, 1, 3], [1, 0], q, [r0k, r1k], [r0v, r1v])
    assert np.max(np.abs(out.ravel() - ref)) <= 1e-6
    # split the visible range of token 0 (2 keys) into two partials and merge them
    o_a, m_a, s_a = O.paged_attention(pages, O.F32, q, [0, 1, 1], [1, 0, 1], [0, 1], 0, layout, hq, hkv, d,
                                      page_bytes, 0.5, kv_begin=0, kv_end=1, want_stats=True)
    o_b, m_b, s_b = O.paged_attention(pages, O.F32, q, [0, 1, 1], [1, 0, 1], [0, 1], 0, layout, hq, hkv, d,
                                      page_bytes, 0.5, kv_begin=1, kv_end=2, want_stats=True)
    for h in range(hq):
        merged = O.merge_partials(np.stack([o_a[0, h], o_b[0, h]]), [m_a[0, h], m_b[0, h]], [s_a[0, h], s_b[0, h]])
        assert np.max(np.abs(merged - out[0, h])) <= 1e-6


def test_yarn_correction_range_and_long_context_rotation():
    # crates/inference-backend-metal/src/components/rms_norm_rope.rs:394-474
    yarn = O.Yarn(1, 32.0, float(np.float32(1.0) + np.float32(0.1) * np.log(np.float32(32.0))), 32.0, 1.0, 8192, 1)
    inv, factor, low, high = O.rope_parameters(128, 10_000_000.0, yarn)
    assert (low, high) == (14.0, 29.0) and abs(factor - (1.0 + 0.1 * math.log(32.0))) < 1e-6
    x = np.array([((i * 37 % 29) - 14.0) / 8.0 for i in range(128)], dtype=np.float32)
    w = O.encode(np.array([0.75 + (i % 11) / 20.0 for i in range(128)], dtype=np.float32), O.BF16)
    position = 262143
    out = O.rms_norm_rope(x, O.F32, w, [position], 1, 128, 128, 1e-6, inv, factor)
    f = np.float32
    inv_rms = f(1.0) / np.sqrt(f(np.sum(x * x, dtype=np.float32) / f(128) + f(1e-6)))
    wf = O.decode(w, O.BF16)
    for d in range(64):
        ramp = min(max((d - 14.0) / (29.0 - 14.0), 0.0), 1.0)
        inv_freq = f(f(10_000_000.0) ** f(-(d / 64.0))) * f(1.0 + ramp * (1.0 / 32.0 - 1.0))
        theta = f(position) * inv_freq
        first, second = wf[d] * x[d] * inv_rms, wf[d + 64] * x[d + 64] * inv_rms
        assert abs(out[d] - factor * (first * math.cos(theta) - second * math.sin(theta))) < 1e-3
        assert abs(out[d + 64] - factor * (first * math.sin(theta) + second * math.cos(theta))) < 1e-3


def test_bf16_norm_rounding_order_is_bit_exact():
    # rms_norm_rope.rs:476-519: position 0, rope_dim 2 of head_dim 4
    x = O.encode(np.array([0.73046875, -1.171875, 0.43945313, 2.03125], dtype=np.float32), O.BF16)
    w = O.encode(np.array([1.296875, 0.8984375, 1.1015625, 0.703125], dtype=np.float32), O.BF16)
    inv, factor, _, _ = O.rope_parameters(2, 1_000_000.0)
    out = O.rms_norm_rope(x, O.BF16, w, [0], 1, 4, 2, 1e-6, inv, factor)
    xf, wf = O.decode(x, O.BF16), O.decode(w, O.BF16)
    inv_rms = np.float32(1.0) / np.sqrt(np.float32(np.float32(np.sum(xf * xf, dtype=np.float32)) / np.float32(4) + np.float32(1e-6)))
    expected = O.encode(wf * O.decode(O.encode(xf * inv_rms, O.BF16), O.BF16), O.BF16)
    assert out.tolist() == expected.tolist()


def test_activation_gate_sigmoid():
    # crates/inference-backend-metal/src/components/metal/gqa_activation_gate.metal:13-38
    a = np.array([1.0, -2.0, 0.5, 3.0], dtype=np.float32)
    g = np.array([0.0, 2.0, -2.0, 30.0], dtype=np.float32)
    out = O.activation_gate(a, g, O.F32)
    expected = a / (1.0 + np.exp(-g.astype(np.float64)))
    assert np.max(np.abs(out - expected)) < 1e-6
    out16 = O.decode(O.activation_gate(O.encode(a, O.BF16), O.encode(g, O.BF16), O.BF16), O.BF16)
    assert np.max(np.abs(out16 - expected)) < 2e-2


def test_block_sdpa_closed_form_vectors():
    # crates/inference-backend-metal/src/components/gqa_block_attention_test.rs:33-139: block 3, 5 q heads over one
    # KV head, head_dim 32, 6 tokens, ramp inputs; expectations recomputed in float64 from the same formulas
    block, hq, hkv, d, t = 3, 5, 1, 32, 6
    scale = float(np.float32(1.0) / np.sqrt(np.float32(32.0)))
    for dtype, tol in ((O.F32, 1e-5), (O.BF16, 1e-2)):
        q = O.decode(O.encode(np.arange(t * hq * d, dtype=np.float32) * np.float32(0.03125) - np.float32(0.4), dtype), dtype)
        k = O.decode(O.encode(np.arange(t * hkv * d, dtype=np.float32) * np.float32(-0.025) + np.float32(0.3), dtype), dtype)
        v = O.decode(O.encode(np.arange(t * hkv * d, dtype=np.float32) * np.float32(0.05) - np.float32(0.2), dtype), dtype)
        out, pm, ps = O.block_sdpa(O.encode(q, dtype), O.encode(k, dtype), O.encode(v, dtype), dtype, t, block, hq, hkv, d, scale)
        q64, k64, v64 = q.astype(np.float64).reshape(t, hq, d), k.astype(np.float64).reshape(t, d), v.astype(np.float64).reshape(t, d)
        for token in range(t):
            begin = token // block * block
            for head in range(hq):
                scores = (k64[begin:begin + block] @ q64[token, head]) * scale
                weights = np.exp(scores - scores.max())
                assert abs(pm[token, head] - scores.max()) < 1e-4
                assert abs(ps[token, head] - weights.sum()) < 1e-4
                want = weights @ v64[begin:begin + block] / weights.sum()
                assert np.abs(out[token, head] - want).max() < tol


def test_oracle_reproduces_the_committed_fixtures():
    # tests/golden/attention_vectors.npz (written by tests/golden/make_fixtures.py from the reference tests' own
    # deterministic inputs): the oracle must keep producing them
    import importlib.util
    from pathlib import Path
    golden_dir = Path(__file__).resolve().parent / "golden"
    spec = importlib.util.spec_from_file_location("make_fixtures", golden_dir / "make_fixtures.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    stored = np.load(golden_dir / "attention_vectors.npz")
    fresh = module.vectors()
    assert sorted(stored.files) == sorted(fresh)
    for name in stored.files:
        assert stored[name].shape == fresh[name].shape, name
        assert np.abs(stored[name] - fresh[name]).max() <= 1e-6, name


def test_projection_split_vectors():
    # GQAQKVSplitKernel test_fixed (crates/inference-backend-metal/src/components/gqa_qkv_split.rs:212-242):
    # 2 q heads, 1 KV head, head_dim 2, two tokens of 0..15
    x = np.arange(16, dtype=np.float32)
    q, g, k, v = O.projection_split(x, O.F32, False, 2, 2, 1, 2)
    assert g is None
    assert q.reshape(-1).tolist() == [0.0, 1.0, 2.0, 3.0, 8.0, 9.0, 10.0, 11.0]
    assert k.reshape(-1).tolist() == [4.0, 5.0, 12.0, 13.0]
    assert v.reshape(-1).tolist() == [6.0, 7.0, 14.0, 15.0]
    # the gated layout (metal/gqa_qgkv_split.metal:14-42): per head a (q | gate) pair, then k, then v; the same
    # profile widens a token to 2*2*2 + 2*2 = 12 elements
    x = np.arange(24, dtype=np.uint16)
    q, g, k, v = O.projection_split(x, O.BF16, True, 2, 2, 1, 2)
    assert q.reshape(-1).tolist() == [0, 1, 4, 5, 12, 13, 16, 17]
    assert g.reshape(-1).tolist() == [2, 3, 6, 7, 14, 15, 18, 19]
    assert k.reshape(-1).tolist() == [8, 9, 20, 21]
    assert v.reshape(-1).tolist() == [10, 11, 22, 23]
