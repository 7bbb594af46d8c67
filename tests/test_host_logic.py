"""The library's host-side policy against the reference's golden vectors and against the CPU oracle (no GPU)."""
import numpy as np
import pytest

import hostapi as H
from oracle import psi_oracle as O

pkg = H.pkg
U32_MAX = 0xFFFFFFFF


def test_bucket_policy_vectors():
    # crates/inference-executor-core/src/replay.rs:94-180
    base = [1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 56, 64]
    P = pkg.ReplayBucketPolicy
    assert P(64).buckets() == base
    assert P(128).buckets() == base + [80, 96, 112, 128]
    assert P(70).buckets()[-1] == 70 and P(6).buckets() == [1, 2, 4, 6]
    for cap in [65, 79, 80, 81, 127, 128, 129, U32_MAX]:
        b = P(cap).buckets()
        assert b[-1] == cap and P(cap).capacity(cap) == cap and all(x < y for x, y in zip(b, b[1:]))
    assert [P(64).capacity(a) for a in (1, 3, 5, 9, 25, 64)] == [1, 4, 6, 12, 32, 64]
    assert P(64).capacity_allow_zero(0) == 0
    t = P(64, [5, 6, 10, 12, 18])
    assert 0 not in t.buckets()
    assert [t.capacity(a) for a in (5, 9, 10, 11, 17, 18)] == [5, 9, 11, 11, 17, 20]
    assert P(6, [1]).buckets() == [1, 2, 4, 6]
    assert P(8, [6]).buckets() == [1, 2, 4, 5, 6, 8]
    assert [P(8, [6]).capacity(a) for a in (5, 6, 7)] == [5, 6, 8]
    p256 = P(256)
    for active in range(1, 257):
        total = p256.capacity(active)
        assert (total - active) * 4 <= total
    with pytest.raises(pkg.PsiError, match="replay active work exceeds capacity"):
        P(6).capacity(7)
    with pytest.raises(pkg.PsiError, match="replay bucket requires active work"):
        P(6).capacity(0)
    with pytest.raises(pkg.PsiError, match="capacity must be positive"):
        P(0)


def test_bucket_policy_matches_oracle_on_random_inputs():
    rng = np.random.default_rng(11)
    for _ in range(200):
        cap = int(rng.integers(1, 5000))
        bounds = [int(x) for x in rng.integers(1, cap + 10, size=rng.integers(0, 6))]
        assert pkg.ReplayBucketPolicy(cap, bounds).buckets() == O.bucket_policy(cap, bounds)


def _cfg(head_dim, group, tokens_per_page, dtype=pkg.BF16):
    hkv = 2
    return (dtype, 2 * hkv * head_dim * tokens_per_page * 2, hkv * group, hkv, head_dim)


def test_split_kv_variant_selection_matrix():
    # crates/inference-backend-metal/src/components/gqa_split_kv.rs:177-231
    S = pkg.GQASplitKV
    t256 = S(*_cfg(256, 6, 16))
    assert t256.max_q_tokens_per_partial_output() == 8
    assert S(*_cfg(256, 6, 8)).max_q_tokens_per_partial_output() == 8
    assert t256.select(4, 4).as_tuple() == (0, 0, 256, 256, 6)
    assert t256.select(8, 4).as_tuple() == (1, 8, 16, 0, 3)
    assert t256.select(16, 4).as_tuple() == (1, 8, 16, 0, 6)
    assert S(*_cfg(256, 6, 8)).select(16, 4).as_tuple() == (1, 8, 16, 0, 6)
    assert S(*_cfg(128, 8, 8)).select(8, 4).as_tuple() == (1, 8, 16, 0, 8)
    for s in (S(*_cfg(256, 8, 4)), S(*_cfg(128, 8, 8), dspark_history=True)):
        assert s.max_q_tokens_per_partial_output() == 1 and s.select(16, 4).tiled_q == 0
    with pytest.raises(pkg.PsiError, match="GQA K/V bytes per token must fit u32"):
        S(pkg.F32, 65536, U32_MAX, U32_MAX, 2)


def test_split_kv_selector_matches_oracle():
    rng = np.random.default_rng(5)
    for _ in range(300):
        d = int(rng.choice([64, 128, 256]))
        g = int(rng.integers(1, 17))
        p = int(rng.choice([4, 8, 16, 32]))
        dt = int(rng.choice([pkg.F32, pkg.BF16]))
        esz = 4 if dt == pkg.F32 else 2
        hkv = 2
        tokens = int(rng.integers(1, 200))
        tiles = int(rng.integers(1, tokens + 1))
        args = (dt, 2 * hkv * d * p * esz, hkv * g, hkv, d)
        mine = pkg.GQASplitKV(*args).select(tokens, tiles).as_tuple()
        theirs, _ = O.split_kv_select(*args, tokens, tiles)
        assert mine == theirs.as_tuple()


def test_metadata_golden_vectors():
    # crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs:549-613
    md = H.Metadata(8)
    rs, ti, cu = [2, 5], [7, 20], [0, 2, 5]
    shape = md.update(rs, ti, cu, H.single_q(8))
    assert md.req_slots[:5].tolist() == [2, 2, 5, 5, 5]
    assert md.flat_token_indices[:5].tolist() == [7, 8, 20, 21, 22]
    assert md.kv_splits[:24].tolist() == [0, 0, 8, 1, 0, 9, 2, 0, 8, 2, 8, 21, 3, 0, 8, 3, 8, 22, 4, 0, 8, 4, 8, 23]
    assert md.cu_kv_splits[:6].tolist() == [0, 1, 2, 4, 6, 8]
    assert shape.as_tuple() == (5, 5, 5, 5, 8, 8, 1)
    shape = md.update(rs, ti, cu, H.tiled_q(8, 4))
    assert md.q_token_tiles[:4].tolist() == [0, 2, 2, 5]
    assert md.kv_splits[:12].tolist() == [0, 0, 9, 1, 0, 12, 1, 12, 23, U32_MAX, U32_MAX, U32_MAX]
    assert md.cu_kv_splits[:3].tolist() == [0, 1, 3]
    assert shape.as_tuple() == (5, 5, 2, 2, 3, 4, 1)
    assert md.update(rs, ti, cu, H.tiled_q(8, 4), mode=pkg.CAPACITY_BUCKETED).as_tuple() == (5, 6, 2, 2, 3, 4, 1)
    assert md.update(rs, ti, cu, H.tiled_q(8, 4), mode=pkg.CAPACITY_CALLER_TOKENS,
                     caller_tokens=5).as_tuple() == (5, 5, 2, 2, 3, 4, 1)


def test_metadata_bucketed_preserves_poisoned_tail():
    # batch_metadata.rs:617-648
    md = H.Metadata(12)
    md.q_token_tiles[:] = 0xA5A5A5A5
    md.kv_splits[:] = 0xB6B6B6B6
    md.cu_kv_splits[:] = 0xC7C7C7C7
    shape = md.update([2, 5, 7], [0, 0, 0], [0, 4, 8, 9], H.tiled_q(8, 4), mode=pkg.CAPACITY_BUCKETED)
    assert shape.as_tuple() == (9, 12, 3, 4, 3, 4, 1)
    assert md.q_token_tiles[6:8].tolist() == [0xA5A5A5A5] * 2
    assert md.kv_splits[9:12].tolist() == [U32_MAX] * 3
    assert md.cu_kv_splits[4] == 0xC7C7C7C7


def test_metadata_contracts():
    # batch_metadata.rs:650-678 and the asserts of update_with_capacity
    md = H.Metadata(12)
    with pytest.raises(pkg.PsiError, match="GQA active token count must not exceed the caller-owned token capacity"):
        md.update([0], [0], [0, 5], H.single_q(8), mode=pkg.CAPACITY_CALLER_TOKENS, caller_tokens=4)
    with pytest.raises(pkg.PsiError, match="GQA caller-owned token capacity must not exceed the metadata capacity"):
        md.update([0], [0], [0, 5], H.single_q(8), mode=pkg.CAPACITY_CALLER_TOKENS, caller_tokens=13)
    with pytest.raises(pkg.PsiError, match="cu_tokens must start at zero"):
        md.update([0], [0], [1, 5], H.single_q(8))
    with pytest.raises(pkg.PsiError, match="nondecreasing"):
        md.update([0, 1], [0, 0], [0, 5, 3], H.single_q(8))
    with pytest.raises(pkg.PsiError, match="context length must fit u32"):
        md.update([0], [U32_MAX], [0, 1], H.single_q(8))
    with pytest.raises(pkg.PsiError, match="requires tokens"):
        md.update([0], [3], [0, 0], H.single_q(8))


def test_metadata_matches_oracle_on_random_batches():
    rng = np.random.default_rng(21)
    for trial in range(150):
        max_tokens = int(rng.integers(4, 96))
        reqs = int(rng.integers(1, 9))
        lens = rng.integers(0, 6, size=reqs)
        if lens.sum() == 0:
            lens[0] = 1
        while lens.sum() > max_tokens:
            lens[np.argmax(lens)] -= 1
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
        ti = rng.integers(0, 3000, size=reqs)
        rs = rng.integers(0, 64, size=reqs)
        tiled = bool(rng.integers(0, 2))
        mode = int(rng.integers(0, 3))
        caller = int(rng.integers(int(cu[-1]), max_tokens + 1))
        bounds = [int(x) for x in rng.integers(1, max_tokens + 1, size=rng.integers(0, 3))]
        kv_tile = int(rng.choice([4, 16, 128, 256]))
        mine, theirs = H.Metadata(max_tokens), O.Metadata(max_tokens)
        v_mine = H.tiled_q(8, kv_tile) if tiled else H.single_q(kv_tile)
        v_ref = O.tiled_q_variant(8, kv_tile) if tiled else O.single_q_variant(kv_tile)
        s1 = mine.update(rs, ti, cu, v_mine, mode, bounds, caller)
        s2 = theirs.update(rs, ti, cu, v_ref, mode, bounds, caller)
        assert s1.as_tuple() == s2.as_tuple(), trial
        for name in ("req_slots", "flat_token_indices", "q_token_tiles", "kv_splits", "cu_kv_splits"):
            assert np.array_equal(getattr(mine, name), getattr(theirs, name)), (trial, name)


def test_allocator_vectors_and_trace_against_oracle():
    # crates/inference-runtime-core/src/memory/u32_id_allocator.rs:179-217
    a = pkg.U32IDAllocator(65)
    assert a.allocated_ids_bitmap() == [0, 0]
    assert (a.alloc_one(), a.alloc_one()) == (0, 1) and a.allocated_ids_bitmap() == [0b11, 0]
    a.free_one(0)
    assert a.allocated_ids_bitmap() == [0b10, 0]
    a.free_one(1)
    assert a.allocated_ids_bitmap() == [0, 0]
    b = pkg.U32IDAllocator(130)
    ids = b.alloc_many(66)
    full = (1 << 64) - 1
    assert b.allocated_ids_bitmap() == [full, 0b11, 0]
    b.free_many([1, 63, 64, 65])
    assert b.allocated_ids_bitmap() == [full & ~(0b10 | (1 << 63)), 0, 0]
    assert len(b.alloc_many(4)) == 4 and b.allocated_ids_bitmap() == [full, 0b11, 0]
    b.free_many(ids)
    assert b.allocated_ids_bitmap() == [0, 0, 0]
    with pytest.raises(pkg.PsiError, match="not enough ID") as err:
        pkg.U32IDAllocator(3).alloc_many(4)
    assert err.value.status == 2
    # seeded admit/finish trace: both allocators must issue identical ids
    rng = np.random.default_rng(9)
    mine, theirs = pkg.U32IDAllocator(500), O.Allocator(500)
    live = []
    for _ in range(400):
        if live and rng.random() < 0.45:
            k = int(rng.integers(0, len(live)))
            ids = live.pop(k)
            mine.free_many(ids)
            theirs.free_many(ids)
        else:
            n = int(rng.integers(1, 12))
            if mine.free() < n:
                continue
            got = mine.alloc_many(n)
            assert got == theirs.alloc_many(n)
            live.append(got)
        assert mine.free() == theirs.free_count()
    assert mine.allocated_ids_bitmap() == theirs.bitmap()


def _check_plan(hq, hkv, ti, cu, max_ctas, min_tiles=8, start_cost=0):
    items, ctas, counts = H.plan_preview(hq, hkv, ti, cu, max_ctas, min_tiles, start_cost)
    group = hq // hkv
    heads_per_tile = min(group, 16)
    head_tiles = -(-group // heads_per_tile)
    tokens_per_tile = max(1, 16 // heads_per_tile)
    # every (tile, head selection) unit is covered exactly once over [0, context) by adjacent items
    covered = {}
    for i, (tile, sel, b, e, slot, flat_begin) in enumerate(items.tolist()):
        key = (tile, sel)
        prev = covered.get(key)
        assert b % 16 == 0 and e > b
        if prev is None:
            assert b == 0
        else:
            assert prev[0] == b and prev[1] == i - 1, "items of one unit must be adjacent and contiguous"
        covered[key] = (e, i, flat_begin)
    # contexts: the unit of a tile ends at the position of the tile's last token + 1
    ends = {}
    tile = 0
    for r in range(len(ti)):
        begin = int(cu[r])
        while begin < int(cu[r + 1]):
            end = min(int(cu[r + 1]), begin + tokens_per_tile)
            ends[tile] = (int(ti[r]) + end - int(cu[r]), begin)
            begin = end
            tile += 1
    assert int(counts[4]) == tile
    for (t, sel), (e, _, flat_begin) in covered.items():
        assert e == ends[t][0] and flat_begin == ends[t][1] and sel < hkv * head_tiles
    assert len(covered) == tile * hkv * head_tiles
    # shares: contiguous, complete, and equal within one KV tile
    assert ctas[0] == 0 and ctas[-1] == len(items) and np.all(np.diff(ctas.astype(np.int64)) >= 0)
    load, charged = [], []
    for c in range(len(ctas) - 1):
        rows = items[ctas[c]:ctas[c + 1]]
        load.append(int(sum(-(-(int(e) - int(b)) // 16) for _, _, b, e, _, _ in rows.tolist())))
        starts = sum(1 for _, _, b, _, _, _ in rows.tolist() if b == 0)      # items that open a unit in this share
        charged.append(load[-1] + start_cost * starts)
    assert sum(load) == int(counts[5])
    # equal shares of KV tiles plus the start cost per opened unit; a unit's start cost may straddle a share boundary,
    # which this count charges wholly to the later share (up to start_cost too much there, too little before)
    assert max(charged) - min(charged) <= 1 + 2 * start_cost
    assert len(load) <= max_ctas
    # partial slots: exactly the items of units that were cut
    per_unit = {}
    for tile, sel, *_ in items.tolist():
        per_unit[(tile, sel)] = per_unit.get((tile, sel), 0) + 1
    slots = [int(s) for s in items[:, 4]]
    cut_items = sum(n for n in per_unit.values() if n > 1)
    assert sorted(s for s in slots if s != U32_MAX) == list(range(cut_items)) and int(counts[2]) == cut_items
    assert int(counts[3]) == sum(1 for n in per_unit.values() if n > 1)
    return items, ctas, counts


def test_balanced_plan_properties():
    rng = np.random.default_rng(4)
    _check_plan(16, 2, [256], [0, 1], 148)                          # configuration 1 shape class
    ctx = rng.integers(1024, 8193, size=32)
    _check_plan(16, 2, ctx, np.arange(33), 148)                     # configuration 2
    ctx = rng.integers(4096, 32769, size=128)
    _check_plan(24, 4, ctx, np.arange(129) * 2, 148)                # configuration 3 (two query tokens per sequence)
    _check_plan(16, 2, [262144] * 4, np.arange(5), 148)             # configuration 4
    _check_plan(32, 1, [5, 900, 17], [0, 3, 4, 9], 7)               # 32-head group: two head tiles, ragged q lens
    _check_plan(4, 4, [0, 0, 0], [0, 1, 2, 3], 1184, min_tiles=4)   # empty caches, one token each
    for _ in range(40):
        reqs = int(rng.integers(1, 20))
        lens = rng.integers(1, 20, size=reqs)
        cu = np.concatenate([[0], np.cumsum(lens)])
        hkv = int(rng.choice([1, 2, 4]))
        g = int(rng.choice([1, 2, 4, 6, 8, 16, 24]))
        _check_plan(hkv * g, hkv, rng.integers(0, 5000, size=reqs), cu, int(rng.integers(1, 300)),
                    int(rng.choice([1, 4, 8])), int(rng.choice([0, 3, 10])))


def test_rope_parameters_yarn_golden_and_oracle():
    # crates/inference-backend-metal/src/components/rms_norm_rope.rs:394-412 (correction range 14, 29)
    import math
    factor = float(np.float32(1.0) + np.float32(0.1) * np.log(np.float32(32.0)))
    cfg = pkg.NormRopeConfig(128, 1e-6, 10_000_000.0, 1, 32.0, factor, 32.0, 1.0, 8192, 1)
    inv, f, low, high = pkg.rope_parameters(cfg)
    assert (low, high) == (14.0, 29.0) and f == pytest.approx(1.0 + 0.1 * math.log(32.0), abs=1e-6)
    ref_inv, ref_f, ref_low, ref_high = O.rope_parameters(128, 10_000_000.0, O.Yarn(1, 32.0, factor, 32.0, 1.0, 8192, 1))
    assert np.allclose(inv, ref_inv, rtol=1e-6) and (low, high) == (ref_low, ref_high)
    plain = pkg.NormRopeConfig(64, 1e-6, 1_000_000.0, 0, 1.0, 1.0, 1.0, 1.0, 1, 0)
    inv, f, low, high = pkg.rope_parameters(plain)
    assert f == 1.0 and (low, high) == (0.0, 0.0)
    assert np.allclose(inv, O.rope_parameters(64, 1_000_000.0)[0], rtol=1e-6)
    with pytest.raises(pkg.PsiError, match="Yarn rope_theta must be greater than 1"):
        pkg.rope_parameters(pkg.NormRopeConfig(64, 1e-6, 1.0, 1, 2.0, 1.0, 2.0, 1.0, 4096, 0))


@pytest.mark.parametrize("equal_shares", [False, True])
@pytest.mark.parametrize("max_ctas", [1, 7, 148])
def test_chunk_plan_covers_every_unit_once_and_keeps_its_books(equal_shares, max_ctas):
    # long query runs: units = (request, KV head, super-tile of 8 query tiles = 16 tokens at group 8); every unit's KV
    # range [0, context + tokens so far) must be covered exactly once by its pieces, pieces of a cut unit own disjoint
    # partial-slot groups and one group of eight arrival counters, every item belongs to exactly one CTA
    rng = np.random.default_rng(11)
    for trial in range(6):
        n = int(rng.integers(1, 9))
        ctx = rng.integers(0, 20000, size=n)
        runs = rng.integers(10, 700, size=n)
        cu = np.concatenate([[0], np.cumsum(runs)])
        items, ctas, counts = H.chunk_plan_preview(16, 2, ctx, cu, max_ctas, equal_shares)
        assert counts[0] == len(items) and ctas[0] == 0 and ctas[-1] == len(items) and np.all(np.diff(ctas.astype(np.int64)) >= 0)
        assert len(ctas) - 1 <= max_ctas
        units = {}
        for req, head, flat, tokens, kb, ke, slot, pieces, first_slot, counter in items.tolist():
            assert kb < ke and kb % 16 == 0 and 1 <= tokens <= 16
            units.setdefault((req, head, flat), []).append((kb, ke, slot, pieces, first_slot, counter, tokens))
        expected_units = sum(-(-int(r) // 16) for r in runs) * 2
        assert len(units) == expected_units
        slot_groups, counter_groups = set(), set()
        total_tiles = 0
        for (req, head, flat), pieces in units.items():
            pieces.sort()
            done = flat - int(cu[req])                      # tokens of the request before this super-tile
            tokens = pieces[0][6]
            end = int(ctx[req]) + done + tokens             # keys the super-tile's last token sees
            assert pieces[0][0] == 0 and pieces[-1][1] == end
            assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
            assert all(a[1] % 16 == 0 for a in pieces[:-1])
            total_tiles += -(-end // 16)
            if len(pieces) == 1:
                assert pieces[0][2] == 0xFFFFFFFF
            else:
                firsts = {x[4] for x in pieces}
                assert len(firsts) == 1 and {x[3] for x in pieces} == {len(pieces)} and len({x[5] for x in pieces}) == 1
                first = firsts.pop()
                assert sorted(x[2] for x in pieces) == [first + 8 * k for k in range(len(pieces))]
                group = set(range(first, first + 8 * len(pieces)))
                assert not (group & slot_groups)
                slot_groups |= group
                counters = set(range(pieces[0][5], pieces[0][5] + 8))
                assert not (counters & counter_groups)
                counter_groups |= counters
        assert counts[4] == total_tiles
        assert counts[2] == len(slot_groups) and counts[3] == len(counter_groups)
        if equal_shares and len(ctas) - 1 > 1:
            loads = [sum(-(-(int(items[i, 5]) - int(items[i, 4])) // 16) for i in range(ctas[c], ctas[c + 1]))
                     for c in range(len(ctas) - 1)]
            share = total_tiles / (len(ctas) - 1)
            assert max(loads) <= share + 2 * 16 + 8 and min(loads) >= share - 2 * 16 - 8, (min(loads), share, max(loads))
