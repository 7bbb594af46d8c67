"""GPU parity tests: the CUDA path through the C ABI against the CPU oracle on the same inputs.

The fixtures restate the reference's own parity tests for the path (cited per test); larger cases use the seeded
synthetic configurations.  Bit-exact for append / gather / table contents; attention within 2e-5 max-abs for f32 and
within 2e-2 max-abs / 2e-3 mean-abs for 16-bit outputs against the f32 oracle.
"""
import math

import numpy as np
import pytest

import checks
import gpuharness as G
import workloads as W
from oracle import psi_oracle as O
from refdata import fixture_values, generated_half_range_values, generated_values, kv_page_values, pattern

pkg = G.pkg
pytestmark = pytest.mark.gpu

MODES = [(pkg.PLAN_BALANCED, "balanced"), (pkg.PLAN_REFERENCE, "reference")]


def _decode(tensor, dtype):
    return O.decode(G.bits_of(tensor), dtype)


# ---------------------------------------------------------------------------------------------------------------------
# KV append / gather / table / arena
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,np_dtype", [(pkg.BF16, np.uint16), (pkg.F32, np.float32)])
def test_kv_page_write_fixed(dtype, np_dtype):
    # crates/inference-backend-metal/src/components/gqa_kv_page_write.rs:344-364
    import torch
    rig = G.Rig(dtype, 1, 1, 2, 2, 1.0, (1, 1, 1, 1), 1, num_pages=1)
    rig.set_pages(0, 0, [0])
    rig.gqa.prepare([0], [1], [0, 1])
    k = torch.from_numpy(np.array([10, 11], dtype=np_dtype).view(np.int16 if np_dtype == np.uint16 else np.float32)).cuda()
    v = torch.from_numpy(np.array([20, 21], dtype=np_dtype).view(np.int16 if np_dtype == np.uint16 else np.float32)).cuda()
    rig.gqa.kv_page_write(rig.pages, rig.table, 0, k, v)
    rig.ctx.sync()
    assert rig.arena_bits().tolist() == [0, 0, 10, 11, 0, 0, 20, 21]
    rig.close()


def test_kv_page_write_bucketed_preserves_inactive_page():
    # gqa_kv_page_write.rs:284-342: capacity 4, 3 active writes leave page 1 all 0x7777; 4 active writes touch it.
    import torch
    sentinel = 0x7777
    for active_reqs, expect_touched in (([0, 0, 0], False), ([0, 0, 0, 1], True)):
        rig = G.Rig(pkg.BF16, 1, 1, 2, 4, 1.0, (2, 1, 1, 1), 4, arena_bits=np.full(32, sentinel, dtype=np.uint16))
        rig.set_pages(0, 0, [0])
        rig.set_pages(1, 0, [1])
        k = torch.from_numpy(np.arange(10, 18, dtype=np.int16)).cuda()
        v = torch.from_numpy(np.arange(20, 28, dtype=np.int16)).cuda()
        if expect_touched:
            shape = rig.gqa.prepare_bucketed_with_token_capacity([0, 1], [0, 0], [0, 3, 4], 4)
        else:
            shape = rig.gqa.prepare_bucketed_with_token_capacity([0], [0], [0, 3], 4)
        assert shape.num_total_tokens == 4
        rig.gqa.kv_page_write(rig.pages, rig.table, 0, k, v)
        rig.ctx.sync()
        bits = rig.arena_bits()
        assert bits[:16].tolist() == [10, 11, 12, 13, 14, 15, sentinel, sentinel, 20, 21, 22, 23, 24, 25, sentinel,
                                      sentinel]
        if expect_touched:
            assert bits[16:18].tolist() == [16, 17] and bits[24:26].tolist() == [26, 27]
        else:
            assert bits[16:].tolist() == [sentinel] * 16
        rig.close()


@pytest.mark.parametrize("dtype", [pkg.BF16, pkg.F32, pkg.F16])
@pytest.mark.parametrize("head_dim,tokens_per_page,ipb", [(2, 4, 2), (24, 3, 1), (128, 16, 4), (256, 8, 2)])
def test_append_and_gather_bit_exact_with_two_level_table(dtype, head_dim, tokens_per_page, ipb):
    import torch
    rng = np.random.default_rng(head_dim * 7 + ipb)
    hkv, slots, layers, blocks = 2, 3, 2, 5
    pages_per_row = blocks * ipb
    num_pages = slots * layers * pages_per_row
    rig = G.Rig(dtype, 2 * hkv, hkv, head_dim, tokens_per_page, 0.5, (slots, layers, blocks, ipb), 64,
                num_pages=num_pages)
    perm = rng.permutation(num_pages).astype(np.uint32).reshape(slots, layers, pages_per_row)
    for s in range(slots):
        for l in range(layers):
            rig.set_pages(s, l, perm[s, l])
    cap = pages_per_row * tokens_per_page
    lens = [5, 11, 7]
    starts = [0, cap - 11, 3]
    cu = [0, 5, 16, 23]
    t = cu[-1]
    npd = np.float32 if dtype == pkg.F32 else np.uint16
    kbits = rng.integers(1, 60000, size=(t, hkv, head_dim)).astype(npd)
    vbits = rng.integers(1, 60000, size=(t, hkv, head_dim)).astype(npd)
    as_torch = lambda a: torch.from_numpy(a.view(np.int16) if npd == np.uint16 else a).cuda()
    k, v = as_torch(kbits), as_torch(vbits)
    rig.gqa.prepare([0, 1, 2], starts, cu)
    before = rig.arena_bits().copy()
    rig.gqa.kv_page_write(rig.pages, rig.table, 1, k, v)
    rig.ctx.sync()
    expected = before.copy()
    slots_flat, pos_flat = G.flat_metadata([0, 1, 2], starts, cu)
    O.kv_page_write(expected, kbits, vbits, slots_flat, pos_flat, rig.table_host.reshape(-1), t, 1, rig.olayout, hkv,
                    head_dim, rig.page_bytes)
    assert np.array_equal(rig.arena_bits(), expected)
    # gather is the inverse of the append
    for s in range(slots):
        lo, hi = starts[s], starts[s] + lens[s]
        kout = torch.zeros((hi - lo, hkv, head_dim), dtype=G.torch_dtype(dtype), device="cuda:0")
        vout = torch.zeros_like(kout)
        rig.gqa.page_gather(rig.pages, rig.table, s, 1, lo, hi, kout, vout)
        rig.ctx.sync()
        assert np.array_equal(G.bits_of(kout), kbits[cu[s]:cu[s + 1]])
        assert np.array_equal(G.bits_of(vout), vbits[cu[s]:cu[s + 1]])
        ek, ev = O.page_gather(expected, rig.table_host.reshape(-1), s, 1, rig.olayout, hkv, head_dim, rig.page_bytes,
                               lo, hi)
        assert np.array_equal(G.bits_of(kout), ek) and np.array_equal(G.bits_of(vout), ev)
    rig.close()


def test_page_table_lifecycle_on_device():
    # crates/inference-executor-metal/src/attn/gqa/request_page_table.rs:140-174
    import torch
    ctx = pkg.Context(0)
    table = pkg.GQARequestPageTable(ctx, pkg.GQAPageTableLayout(4, 3, 6, 2))
    table.write_page_ids(1, 0, 0, [10, 11])
    table.write_page_ids(1, 0, 1, [12, 13])
    table.write_page_ids(1, 2, 0, [20, 21])
    table.write_page_ids(2, 1, 0, [30, 31])
    table.write_page_ids(3, 0, 0, [40, 41])
    assert table.read_page_ids(1, 0, 0) == [10, 11] and table.read_page_ids(1, 0, 1) == [12, 13]
    assert table.read_page_ids(1, 2, 0) == [20, 21]
    table.reset_req_slot(1)
    assert table.read_page_ids(1, 0, 0) == [0, 0] and table.read_page_ids(1, 0, 1) == [0, 0]
    assert table.read_page_ids(1, 2, 0) == [0, 0]
    assert table.read_page_ids(2, 1, 0) == [30, 31] and table.read_page_ids(3, 0, 0) == [40, 41]
    # role-block write with the page-ID domain check (model/qwen/v3_x/state/gqa.rs:88-106)
    table.write_all_layer_page_ids(0, 2, [1, 2, 3, 4, 5, 6], num_cache_pages=7)
    assert [table.read_page_ids(0, l, 2) for l in range(3)] == [[1, 2], [3, 4], [5, 6]]
    with pytest.raises(pkg.PsiError, match="outside the cache-page buffer"):
        table.write_all_layer_page_ids(0, 2, [1, 2, 3, 4, 5, 7], num_cache_pages=7)
    with pytest.raises(pkg.PsiError, match="must contain all layer page IDs"):
        table.write_all_layer_page_ids(0, 2, [1, 2], num_cache_pages=7)
    with pytest.raises(pkg.PsiError, match="req_slot out of range"):
        table.write_page_ids(4, 0, 0, [1, 2])
    with pytest.raises(pkg.PsiError, match="layer out of range"):
        table.write_page_ids(0, 3, 0, [1, 2])
    with pytest.raises(pkg.PsiError, match="block out of range"):
        table.read_page_ids(0, 0, 6)
    with pytest.raises(pkg.PsiError, match="page-id count must match"):
        table.write_page_ids(0, 0, 0, [1])
    table.close()
    ctx.close()


def test_page_arena_is_zeroed_and_round_trips_selected_ranges():
    # crates/inference-executor-metal/src/model/page_arena.rs:67-153 (full and selected state unload / load)
    ctx = pkg.Context(0)
    arena = pkg.PageArena(ctx, 3, 16)
    assert arena.export_range(0, 3) == bytes(48)
    data = bytes((i * 5 + 3) % 256 for i in range(48))
    arena.import_range(0, 3, data)
    assert arena.export_range(0, 3) == data and arena.export_range(1, 2) == data[16:32]
    arena.release_resources()
    with pytest.raises(pkg.PsiError, match="must be loaded before execution"):
        arena.buffer()
    with pytest.raises(pkg.PsiError, match="not loaded"):
        arena.release_resources()
    arena.allocate_resources()
    assert arena.export_range(0, 3) == bytes(48)
    with pytest.raises(pkg.PsiError, match="already loaded"):
        arena.allocate_resources()
    arena.import_range(2, 3, data[:16])
    assert arena.export_range(0, 3) == bytes(32) + data[:16]
    with pytest.raises(pkg.PsiError, match="outside the page arena"):
        arena.export_range(2, 4)
    arena.close()
    ctx.close()


# ---------------------------------------------------------------------------------------------------------------------
# SingleQ fixtures of the reference (f32, tolerance 2e-5)
# ---------------------------------------------------------------------------------------------------------------------
def _single_q_rig(plan_mode, num_req_slots=1, ipb=1, max_tokens=4):
    # fixture_config(): crates/inference-backend-metal/src/components/gqa_split_kv_single_q_test.rs:267-289
    return dict(dtype=pkg.F32, num_q_heads=4, num_kv_heads=2, head_dim=2, tokens_per_page=4, scale=0.5,
                layout=(num_req_slots, 1, 1, ipb), max_tokens=max_tokens, plan_mode=plan_mode)


def _run_single_q(rig, q, req_slots, token_indices, cu_tokens):
    import torch
    qd = G.to_device(q, pkg.F32).reshape(-1, rig.hq, rig.d)
    out = torch.full_like(qd, -321.0)
    rig.gqa.prepare(req_slots, token_indices, cu_tokens)
    rig.gqa.attend(rig.pages, rig.table, 0, qd, out)
    rig.ctx.sync()
    return out.cpu().numpy().reshape(-1)


@pytest.mark.parametrize("plan_mode,_name", MODES)
@pytest.mark.parametrize("case", ["fixed", "random"])
def test_single_q_fixed_and_random(plan_mode, _name, case):
    # gqa_split_kv_single_q_test.rs:50-83 (fixed) and :145-183 (random)
    n_out, stride = 2 * 4 * 2, 2 * 2
    if case == "fixed":
        q, k, v = fixture_values(n_out, 0.125, 3), fixture_values(2 * stride, 0.0625, 5), fixture_values(2 * stride, 0.25, 7)
    else:
        seed = 0x4C8F17D2
        q, k, v = generated_values(n_out, seed), generated_values(2 * stride, seed + 1), generated_values(2 * stride, seed + 2)
    rig = G.Rig(arena_f32=kv_page_values(2, 2, 4, [(k, v)]), **_single_q_rig(plan_mode))
    rig.set_pages(0, 0, [0])
    actual = _run_single_q(rig, q, [0], [0], [0, 2])
    expected = O.projected_gqa_reference(4, 2, 2, 0.5, [0, 2], [0], q, [k], [v])
    assert np.max(np.abs(actual - expected)) <= 2e-5
    assert np.max(np.abs(actual - checks.golden("single_q_" + case))) <= 2e-5   # the stored vectors
    rig.close()


@pytest.mark.parametrize("plan_mode,_name", MODES)
def test_single_q_ragged_random(plan_mode, _name):
    # gqa_split_kv_single_q_test.rs:185-223: two request slots, flat tokens (slot 0 @1), (slot 1 @0), (slot 1 @1)
    seed = 0xD2056AB9
    stride = 4
    q = generated_values(3 * 4 * 2, seed)
    r0k, r0v = generated_values(2 * stride, seed + 1), generated_values(2 * stride, seed + 2)
    r1k, r1v = generated_values(2 * stride, seed + 3), generated_values(2 * stride, seed + 4)
    rig = G.Rig(arena_f32=kv_page_values(2, 2, 4, [(r0k, r0v), (r1k, r1v)]), **_single_q_rig(plan_mode, num_req_slots=2))
    rig.set_pages(0, 0, [0])
    rig.set_pages(1, 0, [1])
    actual = _run_single_q(rig, q, [0, 1], [1, 0], [0, 1, 3])
    expected = O.projected_gqa_reference(4, 2, 2, 0.5, [0, 1, 3], [1, 0], q, [r0k, r1k], [r0v, r1v])
    assert np.max(np.abs(actual - expected)) <= 2e-5
    assert np.max(np.abs(actual - checks.golden("single_q_ragged"))) <= 2e-5
    rig.close()


@pytest.mark.parametrize("plan_mode,_name", MODES)
def test_single_q_multiple_page_ids_per_block(plan_mode, _name):
    # gqa_split_kv_single_q_test.rs:225-265: one block with two page ids, token index 7 sees 8 keys over two pages
    stride = 4
    q = fixture_values(1 * 4 * 2, 0.125, 3)
    k, v = fixture_values(8 * stride, 0.0625, 5), fixture_values(8 * stride, 0.25, 7)
    arena = kv_page_values(2, 2, 4, [(k[:4 * stride], v[:4 * stride]), (k[4 * stride:], v[4 * stride:])])
    rig = G.Rig(arena_f32=arena, **_single_q_rig(plan_mode, ipb=2))
    rig.set_pages(0, 0, [0, 1])
    actual = _run_single_q(rig, q, [0], [7], [0, 1])
    expected = O.projected_gqa_reference(4, 2, 2, 0.5, [0, 1], [7], q, [k], [v])
    assert np.max(np.abs(actual - expected)) <= 2e-5
    rig.close()


@pytest.mark.parametrize("plan_mode,_name", MODES)
def test_single_q_bucketed_replay_preserves_output_tail(plan_mode, _name):
    # gqa_split_kv_single_q_test.rs:85-143: capacity 4 tokens, 3 then 4 active; inactive output rows keep -321
    import torch
    stride = 4
    q = generated_values(4 * 4 * 2, 0x8B1D5A73)
    k, v = generated_values(4 * stride, 0x8B1D5A74), generated_values(4 * stride, 0x8B1D5A75)
    rig = G.Rig(arena_f32=kv_page_values(2, 2, 4, [(k, v)]), **_single_q_rig(plan_mode))
    rig.set_pages(0, 0, [0])
    qd = G.to_device(q, pkg.F32).reshape(4, 4, 2)
    for active in (3, 4):
        out = torch.full_like(qd, -321.0)
        shape = rig.gqa.prepare_bucketed_with_token_capacity([0], [0], [0, active], 4)
        assert shape.num_tokens == active and shape.num_total_tokens == 4
        rig.gqa.attend(rig.pages, rig.table, 0, qd, out)
        rig.ctx.sync()
        got = out.cpu().numpy().reshape(-1)
        n = active * 8
        expected = O.projected_gqa_reference(4, 2, 2, 0.5, [0, active], [0], q[:n], [k[:active * stride]],
                                             [v[:active * stride]])
        assert np.max(np.abs(got[:n] - expected)) <= 2e-5
        assert np.all(got[n:] == -321.0)
    rig.close()


# ---------------------------------------------------------------------------------------------------------------------
# Multi-query (TiledQ) cases of the reference (bf16, tolerance 2e-2)
# ---------------------------------------------------------------------------------------------------------------------
KERNELS = [(pkg.KERNEL_MMA, "mma"), (pkg.KERNEL_GENERIC, "generic")]


def _run_tiled_case(num_tokens_per_req, num_q_heads, head_dim, tokens_per_page, start, plan_mode, kernel_mode,
                    golden_name=None):
    # run_case(): crates/inference-executor-metal/tests/gqa_split_kv_tiled_q.rs:247-462
    import torch
    reqs = len(num_tokens_per_req)
    num_tokens = sum(num_tokens_per_req)
    num_blocks = -(-(start + max(num_tokens_per_req)) // tokens_per_page)
    q = pattern(num_tokens * num_q_heads * head_dim, 29, 0.015625)
    ks, vs, pages = [], [], []
    for r in range(reqs):
        n = num_blocks * tokens_per_page * head_dim
        k, v = pattern(n, 31 + r, 0.015625), pattern(n, 37 + r, 0.03125)
        ks.append(k)
        vs.append(v)
        for b in range(num_blocks):
            lo, hi = b * tokens_per_page * head_dim, (b + 1) * tokens_per_page * head_dim
            pages.append((k[lo:hi], v[lo:hi]))
    arena = kv_page_values(1, head_dim, tokens_per_page, pages)
    scale = np.float32(1.0) / np.sqrt(np.float32(head_dim))
    rig = G.Rig(pkg.BF16, num_q_heads, 1, head_dim, tokens_per_page, float(scale), (reqs, 1, num_blocks, 1), num_tokens,
                arena_f32=arena, plan_mode=plan_mode, kernel_mode=kernel_mode)
    for r in range(reqs):
        rig.set_pages(r, 0, np.arange(r * num_blocks, (r + 1) * num_blocks))
    cu = [0]
    for n in num_tokens_per_req:
        cu.append(cu[-1] + n)
    qd = G.to_device(q, pkg.BF16).reshape(num_tokens, num_q_heads, head_dim)
    out = torch.zeros_like(qd)
    rig.gqa.prepare(list(range(reqs)), [start] * reqs, cu)
    rig.gqa.attend(rig.pages, rig.table, 0, qd, out)
    rig.ctx.sync()
    bf = lambda x: O.decode(O.encode(x, O.BF16), O.BF16)
    expected = O.projected_gqa_reference(
        num_q_heads, 1, head_dim, float(scale), cu, [start] * reqs, bf(q),
        [bf(ks[r][: (start + num_tokens_per_req[r]) * head_dim]) for r in range(reqs)],
        [bf(vs[r][: (start + num_tokens_per_req[r]) * head_dim]) for r in range(reqs)])
    actual = _decode(out, pkg.BF16).reshape(-1)
    stats = rig.gqa.plan_stats()
    rig.close()
    assert stats["kernel"] == kernel_mode
    assert np.max(np.abs(actual - expected)) <= 0.02, np.max(np.abs(actual - expected))
    assert np.mean(np.abs(actual - expected)) <= 2e-3
    if golden_name is not None:  # the stored vectors keep every 7th element
        assert np.max(np.abs(actual[::7] - checks.golden(golden_name))) <= 0.02


@pytest.mark.parametrize("kernel_mode,_kname", KERNELS)
@pytest.mark.parametrize("plan_mode,_name", MODES)
@pytest.mark.parametrize("case,golden_name", [
    (([16], 8, 256, 16, 17), "tiled_fixed"),                                 # test_fixed
    (([16], 6, 256, 8, 9), "tiled_qwen38_27b"),                              # test_qwen38_27b_profile
    (([1, 2, 4, 6, 8, 11, 16, 16], 6, 256, 16, 17), "tiled_ragged"),         # test_ragged
    (([32, 8], 8, 256, 16, 17), "tiled_multiple_tiles"),                     # test_multiple_tiles
    (([1, 4, 8, 13], 5, 128, 8, 9), "tiled_qwen3"),                          # test_qwen3_profile
])
def test_tiled_q_integration_cases(case, golden_name, plan_mode, _name, kernel_mode, _kname):
    # crates/inference-executor-metal/tests/gqa_split_kv_tiled_q.rs:27-50
    _run_tiled_case(*case, plan_mode, kernel_mode, golden_name)


@pytest.mark.parametrize("kernel_mode,_kname", KERNELS)
def test_tiled_q_bucketed_replay_with_poison_and_canary_tails(kernel_mode, _kname):
    # crates/inference-backend-metal/src/components/gqa_split_kv_tiled_q_test.rs:17-199: one request, 5 -> 8 -> 5
    # active tokens of capacity 8; inactive q / K / V rows are NaN, inactive index entries are u32::MAX, and the
    # inactive output rows must keep the canary (case 0) or the previous full result (case 2).
    import torch
    hq, d, p = 5, 128, 8
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    bf = lambda x: O.decode(O.encode(x, O.BF16), O.BF16)
    qv = bf(generated_half_range_values(8 * hq * d, 0x47514154))
    kv = bf(generated_half_range_values(p * d, 0x47514155))
    vv = bf(generated_half_range_values(p * d, 0x47514156))
    canary = 0x42B6
    rig = G.Rig(pkg.BF16, hq, 1, d, p, scale, (1, 1, 1, 1), 8, num_pages=1, kernel_mode=kernel_mode)
    rig.set_pages(0, 0, [0])
    out = torch.from_numpy(np.full((8, hq, d), canary, dtype=np.uint16).view(np.int16)).cuda().view(torch.bfloat16)
    full_out = None
    for case_index, active in enumerate((5, 8, 5)):
        q_sub, k_sub, v_sub = qv.copy(), kv.copy(), vv.copy()
        q_sub[active * hq * d:] = np.nan
        k_sub[active * d:] = np.nan
        v_sub[active * d:] = np.nan
        rig.arena.copy_(G.to_device(kv_page_values(1, d, p, [(k_sub, v_sub)]).reshape(1, -1), pkg.BF16))
        qd = G.to_device(q_sub, pkg.BF16).reshape(8, hq, d)
        rig.gqa.prepare_bucketed_with_token_capacity([0], [0], [0, active], 8)
        rig.gqa.attend(rig.pages, rig.table, 0, qd, out)
        rig.ctx.sync()
        n = active * hq * d
        expected = O.projected_gqa_reference(hq, 1, d, scale, [0, active], [0], qv[:n], [kv[:active * d]],
                                             [vv[:active * d]])
        bits = G.bits_of(out).reshape(-1)
        actual = O.decode(bits[:n], O.BF16)
        assert np.max(np.abs(actual - expected)) <= 2e-2
        if case_index == 0:
            assert np.all(bits[n:] == canary)
        elif case_index == 1:
            full_out = bits.copy()
        else:
            assert np.array_equal(bits[n:], full_out[n:])
    rig.close()


# ---------------------------------------------------------------------------------------------------------------------
# Benchmark configurations
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kernel_mode,_kname", KERNELS)
def test_config1_append_then_attend(kernel_mode, _kname):
    s = W.Session(W.config(1), kernel_mode=kernel_mode)
    before = checks.to_numpy_bits(s.arena)
    s.step()
    s.ctx.sync()
    expected = checks.expected_arena_after_append(s, before)
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), expected)
    checks.assert_attention_close(s)
    s.close()


@pytest.mark.parametrize("index,scale_down", [(2, 8), (3, 16), (4, 64), (5, 64)])
@pytest.mark.parametrize("plan_mode,_name", MODES)
def test_scaled_configs_full_parity(index, scale_down, plan_mode, _name):
    spec = W.config(index, scale_down=scale_down)
    if plan_mode == pkg.PLAN_REFERENCE and spec.num_tokens > 512:
        pytest.skip("the reference planner's O(max_tokens * tiles) greedy loop is slow at this token count")
    s = W.Session(spec, plan_mode=plan_mode)
    before = checks.to_numpy_bits(s.arena)
    s.step()
    s.ctx.sync()
    expected = checks.expected_arena_after_append(s, before)
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), expected)
    checks.assert_attention_close(s)
    s.close()


@pytest.mark.parametrize("index,scale_down", [(1, 1), (2, 8), (3, 16), (5, 64)])
def test_fused_step_equals_append_then_attend(index, scale_down):
    # one launch (the map kernel appends and reads this step's rows from k / v) against the two-stage order
    import torch
    spec = W.config(index, scale_down=scale_down)
    a, b = W.Session(spec), W.Session(spec)
    assert torch.equal(a.arena.view(torch.int16), b.arena.view(torch.int16))
    a.step()
    b.step_unfused()
    a.ctx.sync()
    b.ctx.sync()
    assert torch.equal(a.arena.view(torch.int16), b.arena.view(torch.int16))
    diff = (a.out.float() - b.out.float()).abs().max().item()
    assert diff <= 1e-2, diff  # same math; partial sums may associate differently across launches
    checks.assert_attention_close(a)
    a.close()
    b.close()


@pytest.mark.parametrize("kernel_mode,_kname", KERNELS)
@pytest.mark.parametrize("page,head_dim", [(16, 256), (8, 128), (32, 64)])
def test_page_and_tile_boundaries(page, head_dim, kernel_mode, _kname):
    # Contexts that end just before, on and just after a page and a 16-token tile boundary, from an empty cache up,
    # with query runs of one to three tokens (a verify run that starts on the last slot of a page appends into two
    # pages): pages bit-exact after the step, attention within tolerance, fused step against the two-stage order.
    contexts = [0, 1, 7, 8, 9, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257]
    runs = [1 + (i % 3) for i in range(len(contexts))]
    spec = W.Spec("boundaries", pkg.BF16, 8, 2, head_dim, page, contexts, runs, seed=29)
    s, t = W.Session(spec, kernel_mode=kernel_mode), W.Session(spec, kernel_mode=kernel_mode)
    before = checks.to_numpy_bits(s.arena)
    s.step()
    t.step_unfused()
    s.ctx.sync()
    t.ctx.sync()
    expected = checks.expected_arena_after_append(s, before)
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), expected)
    assert np.array_equal(checks.to_numpy_bits(t.arena).reshape(-1), expected)
    checks.assert_attention_close(s)
    checks.assert_attention_close(t)
    s.close()
    t.close()


@pytest.mark.parametrize("seed", range(24))
def test_random_profiles_fused_step_against_the_oracle(seed):
    # Seeded draws over the profile space the decode kernels accept: head counts and group sizes (including groups
    # wider than one 16-row tile), head dims, page sizes, dtypes, ragged query runs, contexts from an empty cache up,
    # CTA caps from one CTA to the whole GPU, both plan modes.  Pages bit-exact after the step, attention within
    # tolerance, and the same step again leaves both unchanged.
    import torch
    rng = np.random.default_rng(1000 + seed)
    hkv = int(rng.choice([1, 2, 4, 8]))
    group = int(rng.choice([1, 2, 4, 6, 8, 16, 24]))
    head_dim = int(rng.choice([64, 128, 256]))
    page = int(rng.choice([8, 16, 32, 64]))
    dtype = [pkg.BF16, pkg.F16][int(rng.integers(0, 2))]
    batch = int(rng.integers(1, 24))
    hi = int(rng.choice([40, 700, 5000]))
    contexts = rng.integers(0, hi + 1, size=batch)
    runs = rng.integers(1, 7, size=batch)
    plan_mode = [pkg.PLAN_BALANCED, pkg.PLAN_REFERENCE][int(rng.integers(0, 2))]
    max_ctas = int(rng.choice([0, 1, 3, 37, 148]))
    spec = W.Spec(f"random-{seed}", dtype, hkv * group, hkv, head_dim, page, contexts, runs, seed=seed)
    s = W.Session(spec, plan_mode=plan_mode, max_ctas=max_ctas)
    before = checks.to_numpy_bits(s.arena)
    s.step()
    s.ctx.sync()
    expected = checks.expected_arena_after_append(s, before)
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), expected)
    checks.assert_attention_close(s)
    first = s.out.clone()
    s.step()
    s.ctx.sync()
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), expected)
    assert torch.equal(first.view(torch.int16), s.out.view(torch.int16))
    assert s.gqa.device_status() == 0
    s.close()


@pytest.mark.parametrize("seed", range(20))
def test_random_profiles_on_the_correctness_path_against_the_oracle(seed):
    # The same for what only the CUDA-core kernels take: f32, head dims that are no multiple of 64, page sizes that
    # are no power of two (f32 against the reference's own f32 tolerance).  Head dims that are a multiple of four run
    # on the staged kernel, the others (6, 30) on the one-warp kernel.
    rng = np.random.default_rng(2000 + seed)
    hkv = int(rng.choice([1, 2, 3]))
    group = int(rng.choice([1, 2, 5, 8]))
    head_dim = int(rng.choice([6, 8, 24, 30, 96, 128, 256]))
    page = int(rng.choice([3, 5, 8, 12, 16]))
    dtype = [pkg.F32, pkg.BF16, pkg.F16][int(rng.integers(0, 3))]
    batch = int(rng.integers(1, 12))
    contexts = rng.integers(0, int(rng.choice([30, 400])) + 1, size=batch)
    runs = rng.integers(1, 4, size=batch)
    plan_mode = [pkg.PLAN_BALANCED, pkg.PLAN_REFERENCE][int(rng.integers(0, 2))]
    spec = W.Spec(f"random-generic-{seed}", dtype, hkv * group, hkv, head_dim, page, contexts, runs, seed=seed)
    s = W.Session(spec, plan_mode=plan_mode, kernel_mode=pkg.KERNEL_GENERIC, max_ctas=int(rng.choice([0, 2, 64])))
    before = checks.to_numpy_bits(s.arena)
    s.step()
    s.ctx.sync()
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), checks.expected_arena_after_append(s, before))
    checks.assert_attention_close(s)
    assert s.gqa.device_status() == 0
    s.close()


@pytest.mark.parametrize("index,scale_down,kernel_mode", [
    (2, 1, pkg.KERNEL_AUTO), (3, 4, pkg.KERNEL_AUTO), (5, 8, pkg.KERNEL_AUTO), (5, 8, pkg.KERNEL_MMA_SYNC),
    (3, 8, pkg.KERNEL_GENERIC), (2, 4, pkg.KERNEL_MMA_TMA)])
def test_repeated_launches_are_bit_identical(index, scale_down, kernel_mode):
    # A launch's result depends on nothing but its inputs: cut units are merged in slot order whoever arrives last,
    # and no kernel reads shared or global memory that it has not written in the same launch.  Forty launches of the
    # same step (an L2 sweep in between changes the timing of the loads), every output against the first, bit for bit.
    import torch
    s = W.Session(W.config(index, scale_down=scale_down), kernel_mode=kernel_mode)
    sweep = torch.zeros(48 << 20, dtype=torch.float32, device=s.device)
    s.step()
    s.ctx.sync()
    first = s.out.clone()
    arena = s.arena.clone()
    for launch in range(40):
        if launch % 2:
            sweep.sum()
        s.out.fill_(float("nan"))
        s.step()
        s.ctx.sync()
        assert torch.equal(first.view(torch.int16), s.out.view(torch.int16)), launch
    assert torch.equal(arena.view(torch.int16), s.arena.view(torch.int16))
    assert s.gqa.device_status() == 0
    checks.assert_attention_close(s, seq_ids=list(range(min(4, s.spec.num_seqs))))
    s.close()


@pytest.mark.parametrize("engine", ["tcgen05", "mma_sync"])
@pytest.mark.parametrize("max_ctas", [1, 5, 148])
@pytest.mark.parametrize("heads,head_dim,page", [((16, 2), 256, 16), ((24, 4), 128, 8), ((8, 8), 128, 32)])
def test_long_query_runs_through_the_chunk_kernel(heads, head_dim, page, max_ctas, engine):
    # chunked prefill mixed with decode rows: requests with long query runs take the chunk kernel (one pass over the
    # history for eight query tiles), units cut across CTAs leave partials that the last-arriving warp merges
    hq, hkv = heads
    spec = W.Spec("chunks", pkg.BF16, hq, hkv, head_dim, page, [700, 37, 0, 1500, 260], [96, 1, 40, 33, 2], seed=11)
    s = W.Session(spec, max_ctas=max_ctas, kernel_mode=pkg.KERNEL_MMA if engine == "tcgen05" else pkg.KERNEL_MMA_SYNC)
    stats = s.gqa.plan_stats()
    assert stats["chunk_ctas"] >= 1 and stats["chunk_items"] >= 1
    before = checks.to_numpy_bits(s.arena)
    s.step()
    s.ctx.sync()
    expected = checks.expected_arena_after_append(s, before)
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), expected)
    checks.assert_attention_close(s)
    # the unfused order and the partial (o, m, l) outputs take the same kernels
    fused = s.out.clone()
    s.step_unfused()
    s.ctx.sync()
    assert float((s.out.float() - fused.float()).abs().max()) <= 1e-2
    assert s.gqa.device_status() == 0  # no bounded wait of the tcgen05 kernel ran out
    stats = s.gqa.plan_stats()
    if engine == "tcgen05":
        assert stats["chunk_tcgen05_launches"] >= 2 and stats["chunk_mma_sync_launches"] == 0
    else:
        assert stats["chunk_tcgen05_launches"] == 0 and stats["chunk_mma_sync_launches"] >= 2
    s.close()


@pytest.mark.parametrize("engine", ["tcgen05", "mma_sync"])
def test_long_query_runs_in_f16(engine):
    # the f16 instantiation of both chunk engines (the MMA instruction descriptor carries the element format)
    spec = W.Spec("chunks-f16", pkg.F16, 16, 2, 128, 16, [900, 64, 2000], [128, 1, 70], seed=13)
    s = W.Session(spec, kernel_mode=pkg.KERNEL_MMA if engine == "tcgen05" else pkg.KERNEL_MMA_SYNC)
    assert s.gqa.plan_stats()["chunk_ctas"] >= 1
    before = checks.to_numpy_bits(s.arena)
    s.step()
    s.ctx.sync()
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), checks.expected_arena_after_append(s, before))
    checks.assert_attention_close(s)
    assert s.gqa.device_status() == 0
    key = "chunk_tcgen05_launches" if engine == "tcgen05" else "chunk_mma_sync_launches"
    assert s.gqa.plan_stats()[key] == 1
    s.close()


def test_config2_full_size_parity_and_idempotence():
    import torch
    s = W.Session(W.config(2))
    assert s.gqa.plan_stats()["kernel"] == pkg.KERNEL_MMA
    s.step()
    s.ctx.sync()
    first = s.out.clone()
    checks.assert_attention_close(s)
    # a second pass appends the same rows to the same slots: pages and outputs must not change
    arena = s.arena.clone()
    s.step()
    s.ctx.sync()
    assert torch.equal(arena.view(torch.int16), s.arena.view(torch.int16))
    assert torch.equal(first.view(torch.int16), s.out.view(torch.int16))
    s.close()


def test_config3_full_size_sampled_parity_and_gather_round_trip():
    import torch
    spec = W.config(3)
    s = W.Session(spec)
    s.step()
    s.ctx.sync()
    # a quarter of the batch against the CPU oracle, spread evenly over the length distribution (shortest and longest
    # included)
    order = np.argsort(spec.visible)
    sample = sorted({int(order[i]) for i in np.linspace(0, len(order) - 1, 32).round().astype(int)})
    assert len(sample) >= 30
    checks.assert_attention_close(s, sample)
    sample = sample[::8]
    # size-independent property at full size: gathering the appended positions returns exactly this step's k, v
    cu = np.concatenate([[0], np.cumsum(spec.q_len)])
    for seq in sample:
        lo = int(spec.context_lens[seq])
        kout = torch.zeros((2, spec.num_kv_heads, spec.head_dim), dtype=s.tdtype, device=s.device)
        vout = torch.zeros_like(kout)
        s.gqa.page_gather(s.pages, s.table, seq, 0, lo, lo + 2, kout, vout)
        s.ctx.sync()
        assert torch.equal(kout.view(torch.int16), s.k[cu[seq]:cu[seq] + 2].view(torch.int16))
        assert torch.equal(vout.view(torch.int16), s.v[cu[seq]:cu[seq] + 2].view(torch.int16))
    s.close()


def test_config4_full_size_sampled_parity_and_idempotence():
    # Configuration 4 at full size: four sequences of 262,144 context tokens behind randomly permuted block tables
    # (16,385 table entries each after the append).  Every sequence against the CPU oracle, the appended position read
    # back bit for bit, and a second pass over the same slots leaving pages and outputs unchanged.
    import torch
    spec = W.config(4)
    s = W.Session(spec)
    assert s.gqa.plan_stats()["kernel"] == pkg.KERNEL_MMA
    s.step()
    s.ctx.sync()
    checks.assert_attention_close(s, list(range(spec.num_seqs)))
    first = s.out.clone()
    for seq in range(spec.num_seqs):
        lo = int(spec.context_lens[seq])
        kout = torch.zeros((1, spec.num_kv_heads, spec.head_dim), dtype=s.tdtype, device=s.device)
        vout = torch.zeros_like(kout)
        s.gqa.page_gather(s.pages, s.table, seq, 0, lo, lo + 1, kout, vout)
        s.ctx.sync()
        assert torch.equal(kout.view(torch.int16), s.k[seq:seq + 1].view(torch.int16))
        assert torch.equal(vout.view(torch.int16), s.v[seq:seq + 1].view(torch.int16))
    arena = s.arena.clone()
    s.step()
    s.ctx.sync()
    assert torch.equal(arena.view(torch.int16), s.arena.view(torch.int16))
    assert torch.equal(first.view(torch.int16), s.out.view(torch.int16))
    s.close()


def test_config5_full_size_chunk_engines_agree_and_sample_matches_oracle():
    # Configuration 5 at full size (256 sequences, 30 % with a 512-token query run, contexts up to 131,072): the
    # tcgen05 chunk kernel against the CPU oracle on a sample of long-run sequences, and against the independent
    # mma.sync chunk kernel on every output row (two engines, one plan, same pages after the step).
    import torch
    spec = W.config(5)
    a = W.Session(spec)
    stats = a.gqa.plan_stats()
    assert stats["chunk_ctas"] >= 1
    a.step()
    a.ctx.sync()
    assert a.gqa.device_status() == 0
    assert a.gqa.plan_stats()["chunk_tcgen05_launches"] == 1
    # Against the oracle: the sixteen cheapest long-run sequences, then every further one (cheapest first) while the
    # oracle's work stays within about 40 GB of K/V reads (a 512-token run re-reads its context per query token), and
    # eight decode sequences spread over the length distribution.
    long_runs = np.flatnonzero(spec.q_len > 1)
    by_cost = long_runs[np.argsort(spec.visible[long_runs])]
    row_bytes = 2 * spec.num_kv_heads * spec.head_dim * spec.elem_bytes
    sample, budget = [], 40e9
    for seq in by_cost:
        cost = float(spec.q_len[seq]) * float(spec.visible[seq]) * row_bytes
        if len(sample) >= 16 and cost > budget:
            break
        sample.append(int(seq))
        budget -= cost
    assert len(sample) >= 16
    decode = np.flatnonzero(spec.q_len == 1)
    decode = decode[np.argsort(spec.visible[decode])]
    sample += [int(decode[i]) for i in np.linspace(0, len(decode) - 1, 8).round().astype(int)]
    checks.assert_attention_close(a, sorted(set(sample)))
    out_tcgen05 = a.out.clone()
    arena_after = a.arena.clone() if a.arena.numel() * 2 <= (8 << 30) else None
    a.close()
    b = W.Session(spec, kernel_mode=pkg.KERNEL_MMA_SYNC)
    b.step()
    b.ctx.sync()
    assert b.gqa.plan_stats()["chunk_mma_sync_launches"] == 1
    diff = (b.out.float() - out_tcgen05.float()).abs()
    assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3, (float(diff.max()), float(diff.mean()))
    if arena_after is not None:  # both steps appended the same rows to the same slots
        assert torch.equal(arena_after.view(torch.int16), b.arena.view(torch.int16))
    b.close()


def test_partials_and_combine_match_full_attention():
    # KV-range split of configuration 4 (scaled): two local shards produce (o, m, l); combine equals the unsplit run.
    import torch
    spec = W.config(4, scale_down=64)
    full = W.Session(spec)
    full.step()
    full.ctx.sync()
    checks.assert_attention_close(full)
    t, hq, d = spec.num_tokens, spec.num_q_heads, spec.head_dim
    # shard sessions draw their own K/V; rebuild the unsplit context from both shards' gathered tokens via the oracle
    shards = [W.Session(spec.kv_range_shard(r, 2)) for r in range(2)]
    parts = []
    for sh in shards:
        sh.q.copy_(full.q)
        if sh.spec.do_append:
            sh.append()
        o = torch.zeros((t, hq, d), dtype=torch.float32, device="cuda:0")
        m = torch.zeros((t, hq), dtype=torch.float32, device="cuda:0")
        l = torch.zeros((t, hq), dtype=torch.float32, device="cuda:0")
        sh.gqa.attend_partial(sh.pages, sh.table, 0, sh.q, o, m, l)
        sh.ctx.sync()
        parts.append((o, m, l))
        # each partial against the oracle on the shard's own arena
        prob = checks.host_problem(sh)
        q = checks.to_numpy_bits(sh.q)[prob["tok_rows"]]
        eo, em, es = O.paged_attention(prob["arena"], spec.dtype, q, prob["req_slots"], prob["positions"],
                                       prob["table"], 0, prob["layout"], hq, spec.num_kv_heads, d, spec.page_bytes,
                                       spec.scale, want_stats=True)
        assert np.max(np.abs(o.cpu().numpy() - eo)) <= 2e-2
        assert np.max(np.abs(m.cpu().numpy() - em)) <= 2e-3
        assert np.max(np.abs(l.cpu().numpy() / es - 1.0)) <= 2e-2
    out = torch.zeros_like(full.q)
    shards[0].gqa.combine([p[0] for p in parts], [p[1] for p in parts], [p[2] for p in parts], t, out)
    shards[0].ctx.sync()
    # oracle merge of the oracle partials is the expectation for the combined output
    merged = np.zeros((t, hq, d), dtype=np.float32)
    po = [p[0].cpu().numpy() for p in parts]
    pm = [p[1].cpu().numpy() for p in parts]
    pl = [p[2].cpu().numpy() for p in parts]
    for i in range(t):
        for h in range(hq):
            merged[i, h] = O.merge_partials(np.stack([po[0][i, h], po[1][i, h]]), [pm[0][i, h], pm[1][i, h]],
                                            [pl[0][i, h], pl[1][i, h]])
    assert np.max(np.abs(_decode(out, spec.dtype) - merged)) <= 2e-2
    for sh in shards:
        sh.close()
    full.close()


@pytest.mark.parametrize("pinned", [True, False])
def test_decode_step_through_host_buffers(pinned):
    # pinned buffers are read and written in place by the launch; pageable ones are staged through device copies
    import torch
    spec = W.config(2, scale_down=8)
    s = W.Session(spec)
    before = checks.to_numpy_bits(s.arena)
    pin = (lambda t: t.pin_memory()) if pinned else (lambda t: t)
    kh, vh, qh = pin(s.k.cpu()), pin(s.v.cpu()), pin(s.q.cpu())
    oh = pin(torch.zeros_like(qh))
    s.gqa.decode_step_host(s.pages, s.table, 0, kh, vh, qh, oh)
    expected = checks.expected_arena_after_append(s, before)
    assert np.array_equal(checks.to_numpy_bits(s.arena).reshape(-1), expected)
    s.out.copy_(oh.cuda())
    checks.assert_attention_close(s)
    s.close()


@pytest.mark.parametrize("index,scale_down", [(2, 8), (3, 2)])
@pytest.mark.parametrize("pinned", [True, False])
def test_one_call_host_step_equals_prepare_plus_host_step(pinned, index, scale_down):
    # psi_gqa_step_host plans the step while q/k/v travel; same arena and same output bits as the two separate calls,
    # also on the second call of the same component (the plan's staging buffer is reused).  The second workload
    # (128 verify tokens, 2 MiB of q/k/v) is past the size from which pinned buffers are read in place by the
    # attention launch instead of being pulled into device staging first.
    import torch
    spec = W.config(index, scale_down=scale_down)
    a, b, c = W.Session(spec), W.Session(spec), W.Session(spec)
    pin = (lambda t: t.pin_memory()) if pinned else (lambda t: t)
    kh, vh, qh = pin(a.k.cpu()), pin(a.v.cpu()), pin(a.q.cpu())
    two, one = pin(torch.zeros_like(qh)), pin(torch.zeros_like(qh))
    batch = spec.batch()
    for repeat in range(2):
        slots, starts, cu = batch
        qh.mul_(-0.5)   # another query each time: the outputs differ between the repeats
        before = checks.to_numpy_bits(a.arena) if repeat == 0 else None
        a.gqa.prepare(slots, starts, cu)
        a.gqa.decode_step_host(a.pages, a.table, 0, kh, vh, qh, two)
        b.gqa.step_host(b.pages, b.table, 0, slots, starts, cu, kh, vh, qh, one)
        assert torch.equal(one.view(torch.int16), two.view(torch.int16))
        assert torch.equal(a.arena.view(torch.int16), b.arena.view(torch.int16))
        # the device-resident fused step on the same inputs: the same launch, whichever memory q/k/v are read from
        c.q.copy_(qh)
        c.step()
        c.ctx.sync()
        assert torch.equal(c.out.cpu().view(torch.int16), one.view(torch.int16))
        assert torch.equal(c.arena.view(torch.int16), b.arena.view(torch.int16))
        if before is not None:
            assert not np.array_equal(checks.to_numpy_bits(a.arena), before)   # the step did append
    a.close()
    b.close()
    c.close()
    with pytest.raises(pkg.PsiError):
        c = W.Session(spec)
        try:
            c.gqa.step_host(c.pages, c.table, 0, batch[0], batch[1], batch[2], None, vh, qh, one)
        finally:
            c.close()


def test_layer_index_selects_the_table_row():
    # two layers share one arena; each layer's rows map the same logical pages to different physical pages
    import torch
    rng = np.random.default_rng(3)
    hq, hkv, d, p = 8, 2, 64, 16
    rig = G.Rig(pkg.BF16, hq, hkv, d, p, 0.125, (2, 2, 4, 1), 2,
                arena_f32=rng.standard_normal((16, 2 * hkv * p * d)).astype(np.float32))
    ids = rng.permutation(16).astype(np.uint32).reshape(2, 2, 4)
    for s in range(2):
        for l in range(2):
            rig.set_pages(s, l, ids[s, l])
    q = G.to_device(rng.standard_normal((2, hq, d)).astype(np.float32), pkg.BF16)
    rig.gqa.prepare([0, 1], [40, 63], [0, 1, 2])
    for layer in range(2):
        out = torch.zeros_like(q)
        rig.gqa.attend(rig.pages, rig.table, layer, q, out)
        rig.ctx.sync()
        expected = rig.oracle_attention(q, [0, 1], [40, 63], layer=layer)
        assert np.max(np.abs(_decode(out, pkg.BF16) - expected)) <= 2e-2
    rig.close()


def test_host_side_contracts_on_the_component():
    # the reference's panics, returned as invalid-argument before anything launches
    ctx = pkg.Context(0)
    layout = pkg.GQAPageTableLayout(2, 1, 4, 1)
    good = dict(num_q_heads=4, num_kv_heads=2, head_dim=64, scale=0.125, page_bytes=2 * 2 * 16 * 64 * 2,
                dtype=pkg.BF16, layout=layout, max_tokens=8, plan_mode=0, kernel_mode=0, max_ctas=0)
    def make(**kw):
        return pkg.GQA(ctx, pkg.GQAConfig(**{**good, **kw}))
    with pytest.raises(pkg.PsiError, match="multiple of kv heads"):
        make(num_q_heads=5)
    with pytest.raises(pkg.PsiError, match="divisible by the K/V bytes per token"):
        make(page_bytes=1000)
    with pytest.raises(pkg.PsiError, match="scale must be positive"):
        make(scale=0.0)
    with pytest.raises(pkg.PsiError, match="exceeds the shader u32 count domain"):
        make(max_tokens=1 << 30)
    with pytest.raises(pkg.PsiError, match="does not support this profile"):
        make(dtype=pkg.F32, page_bytes=2 * 2 * 16 * 64 * 4, kernel_mode=pkg.KERNEL_MMA)
    g = make()
    with pytest.raises(pkg.PsiError, match="must be updated before recording"):
        g.plan_stats()
    with pytest.raises(pkg.PsiError, match="exceeds the metadata token capacity"):
        g.prepare([0], [0], [0, 9])
    with pytest.raises(pkg.PsiError, match="does not fit the request page table"):
        g.prepare([0], [60], [0, 5])
    with pytest.raises(pkg.PsiError, match="req_slot out of range"):
        g.prepare([2], [0], [0, 1])
    table = pkg.GQARequestPageTable(ctx, pkg.GQAPageTableLayout(2, 1, 5, 1))
    arena = pkg.PageArena(ctx, 4, good["page_bytes"])
    g.prepare([0], [0], [0, 1])
    with pytest.raises(pkg.PsiError, match="layout differs"):
        g.attend(arena, table, 0, arena.buffer(), arena.buffer())
    for obj in (g, table, arena):
        obj.close()
    ctx.close()


def test_flag_exchange_on_one_device_and_bounded_wait_timeout():
    # Two emulated ranks on one GPU: partials land in "receive" slots, each followed by a flag; the merge waits on
    # the flags (already set: same stream).  Then a flag that nothing sets: the bounded wait gives up, reports a
    # timeout, writes nothing, and the context keeps working.
    import torch
    spec = W.config(4, scale_down=64)
    t, hq, d = spec.num_tokens, spec.num_q_heads, spec.head_dim
    shards = [W.Session(spec.kv_range_shard(r, 2)) for r in range(2)]
    owner = shards[1]
    recv_o = [torch.zeros((t, hq, d), dtype=torch.float32, device="cuda:0") for _ in range(2)]
    recv_m = [torch.zeros((t, hq), dtype=torch.float32, device="cuda:0") for _ in range(2)]
    recv_l = [torch.zeros((t, hq), dtype=torch.float32, device="cuda:0") for _ in range(2)]
    flags = torch.zeros(4, dtype=torch.int32, device="cuda:0")
    expect = torch.zeros_like(owner.q)
    for step in (1, 2):
        for r, sh in enumerate(shards):
            sh.q.copy_(owner.q)
            if sh.spec.do_append:
                sh.append()
            sh.gqa.attend_partial(sh.pages, sh.table, 0, sh.q, recv_o[r], recv_m[r], recv_l[r])
            sh.gqa.signal(flags.data_ptr() + 4 * r, step)
        out = torch.zeros_like(owner.q)
        owner.gqa.combine_wait(recv_o, recv_m, recv_l, t, out, flags, step)
        owner.gqa.combine(recv_o, recv_m, recv_l, t, expect)
        assert owner.gqa.device_status() == 0
        assert torch.equal(out.view(torch.int16), expect.view(torch.int16))
        assert flags[:2].tolist() == [step, step]
    canary = torch.full_like(owner.q, 7.0)
    owner.gqa.combine_wait(recv_o, recv_m, recv_l, t, canary, flags, 3, max_polls=2000)   # nobody publishes step 3
    assert owner.gqa.device_status() == 4                                               # PSI_ERR_TIMEOUT
    assert bool((canary == 7.0).all())
    assert owner.gqa.device_status() == 0                                               # cleared; still usable
    owner.gqa.combine_wait(recv_o, recv_m, recv_l, t, canary, flags, 2)
    assert owner.gqa.device_status() == 0
    assert torch.equal(canary.view(torch.int16), expect.view(torch.int16))
    for sh in shards:
        sh.close()


@pytest.mark.parametrize("spec_args", [
    dict(index=2, scale_down=1),                                  # configuration 2 at full size, fused append
    dict(index=3, scale_down=8),                                  # two query tokens per sequence, 12 rows per item
    dict(custom=(32, 8, 128, 16, 12, 300, 3000, 1)),              # head_dim 128
    dict(custom=(16, 4, 64, 16, 9, 100, 2500, 1)),                # head_dim 64 (one swizzle atom per row group)
    dict(custom=(16, 2, 256, 8, 7, 50, 1500, 2)),                 # 8-token pages: two boxes per tile
    dict(custom=(16, 2, 256, 32, 5, 10, 900, 1)),                 # 32-token pages: a tile is half a page
])
def test_decode_kernel_with_the_tma_feed_matches_the_oracle_and_the_cp_async_feed(spec_args):
    # PSI_KERNEL_MMA_TMA: the same decode kernel with whole K/V tiles brought from their pages as TMA boxes.  Same
    # arithmetic in the same order on the same values, so the outputs equal the default kernel's bit for bit; the
    # ragged last tile of every item and this step's own rows still travel by cp.async into the box layout.
    import torch
    spec = W.config(spec_args["index"], scale_down=spec_args["scale_down"]) if "index" in spec_args else W.W.custom(*spec_args["custom"])
    a = W.Session(spec, kernel_mode=pkg.KERNEL_MMA_TMA)
    before = checks.to_numpy_bits(a.arena)
    a.step()
    a.ctx.sync()
    assert a.gqa.device_status() == 0
    assert np.array_equal(checks.to_numpy_bits(a.arena).reshape(-1), checks.expected_arena_after_append(a, before))
    checks.assert_attention_close(a)
    b = W.Session(spec, kernel_mode=pkg.KERNEL_MMA)
    b.step()
    b.ctx.sync()
    assert torch.equal(a.out.view(torch.int16), b.out.view(torch.int16))
    # the two-stage order (append launch, then attention over pages only) through the TMA feed as well
    a.out.zero_()
    a.step_unfused()
    a.ctx.sync()
    assert torch.equal(a.out.view(torch.int16), b.out.view(torch.int16))
    a.close()
    b.close()
