"""Continuous-batching churn on one GPU: page IDs come from the allocator, finished sequences free their pages, new
sequences reuse them (contents are never cleared), and every step's attention is checked against the CPU oracle on a
host-side shadow of each sequence's K/V that knows nothing about paging.

Scaled-down version of the churn configuration: 24 live sequences, 16/2 heads, head_dim 128, 16-token pages, 30 % of
the sequences append a 40-token chunk per step and the rest one token, 10 % finish per step.  The cache-ownership side
follows crates/inference-runtime-core/src/memory/u32_id_allocator.rs (free IDs first) and
crates/inference-executor-metal/src/attn/gqa/request_page_table.rs (reset on slot reuse)."""
import numpy as np
import pytest

import checks
import gpuharness as G
from oracle import psi_oracle as O

pkg = G.pkg
pytestmark = pytest.mark.gpu


def test_allocator_driven_page_reuse_over_many_steps():
    import torch
    rng = np.random.default_rng(5)
    hq, hkv, d, p = 16, 2, 128, 16
    slots, max_ctx, chunk, steps = 24, 640, 40, 14
    blocks = -(-(max_ctx + chunk) // p)
    pool = slots * blocks // 2                      # tight pool: reuse is the rule, not the exception
    scale = 1.0 / np.sqrt(d)
    rig = G.Rig(pkg.BF16, hq, hkv, d, p, float(scale), (slots, 1, blocks, 1), slots * chunk, num_pages=pool)
    rig.arena.copy_(torch.randn(rig.arena.shape, device="cuda").to(torch.bfloat16))   # stale garbage everywhere
    alloc = pkg.U32IDAllocator(pool)
    shadow_k = [np.zeros((0, hkv, d), np.uint16) for _ in range(slots)]
    shadow_v = [np.zeros((0, hkv, d), np.uint16) for _ in range(slots)]
    pages = [[] for _ in range(slots)]
    reused = 0
    ever_freed = set()

    def grow(slot, new_len):
        nonlocal reused
        while len(pages[slot]) * p < new_len:
            pid = alloc.alloc_one()
            reused += pid in ever_freed
            rig.table.write_page_ids(slot, 0, len(pages[slot]), [pid])
            pages[slot].append(pid)

    def admit(slot):
        """A new sequence arrives with a cached prompt: its K/V rows are appended in bulk, without attention."""
        length = int(min(max_ctx - 200, 16 + rng.zipf(1.3)))
        grow(slot, length)
        k = rng.integers(0, 1 << 16, size=(length, hkv, d)).astype(np.uint16) & 0xBFFF | 0x3000  # finite bf16 values
        v = rng.integers(0, 1 << 16, size=(length, hkv, d)).astype(np.uint16) & 0xBFFF | 0x3000
        shadow_k[slot], shadow_v[slot] = k, v
        for start in range(0, length, slots * chunk):
            n = min(slots * chunk, length - start)
            rig.gqa.prepare([slot], [start], [0, n])
            kd = torch.from_numpy(k[start:start + n].view(np.int16)).cuda()
            vd = torch.from_numpy(v[start:start + n].view(np.int16)).cuda()
            rig.gqa.kv_page_write(rig.pages, rig.table, 0, kd, vd)
            rig.ctx.sync()

    for slot in range(slots):
        admit(slot)

    for step in range(steps):
        # 10 % of the sequences finish: pages go back to the allocator, the slot's table rows are zeroed, a new
        # sequence moves in
        for slot in rng.choice(slots, size=max(1, slots // 10), replace=False):
            slot = int(slot)
            alloc.free_many(pages[slot])
            ever_freed.update(pages[slot])
            pages[slot] = []
            rig.table.reset_req_slot(slot)
            admit(slot)
        q_len = np.where(rng.random(slots) < 0.3, chunk, 1)
        active = [s for s in range(slots) if len(shadow_k[s]) + q_len[s] <= max_ctx + chunk]
        token_indices = [len(shadow_k[s]) for s in active]
        cu = np.concatenate([[0], np.cumsum(q_len[active])]).tolist()
        t = cu[-1]
        for s in active:
            grow(s, len(shadow_k[s]) + int(q_len[s]))
        kq = rng.standard_normal((t, hkv, d)).astype(np.float32)
        vq = rng.standard_normal((t, hkv, d)).astype(np.float32)
        qq = rng.standard_normal((t, hq, d)).astype(np.float32)
        kd, vd, qd = G.to_device(kq, pkg.BF16), G.to_device(vq, pkg.BF16), G.to_device(qq, pkg.BF16)
        out = torch.zeros_like(qd)
        rig.gqa.prepare(active, token_indices, cu)
        if step % 2 == 0:
            rig.gqa.append_attend(rig.pages, rig.table, 0, kd, vd, qd, out)      # one launch
        else:
            rig.gqa.kv_page_write(rig.pages, rig.table, 0, kd, vd)               # the two-stage order
            rig.gqa.attend(rig.pages, rig.table, 0, qd, out)
        rig.ctx.sync()
        kb, vb = G.bits_of(kd), G.bits_of(vd)
        for i, s in enumerate(active):
            shadow_k[s] = np.concatenate([shadow_k[s], kb[cu[i]:cu[i + 1]]])
            shadow_v[s] = np.concatenate([shadow_v[s], vb[cu[i]:cu[i + 1]]])
        # oracle on the shadows of a sample of sequences (always including a chunk when there is one)
        sample = sorted(set([int(np.argmax(q_len[active]))] + rng.choice(len(active), size=4, replace=False).tolist()))
        got = O.decode(G.bits_of(out), O.BF16)
        for i in sample:
            s = active[i]
            n = cu[i + 1] - cu[i]
            expected = O.projected_gqa_reference(hq, hkv, d, float(scale), [0, n], [token_indices[i]],
                                                 O.decode(G.bits_of(qd)[cu[i]:cu[i + 1]], O.BF16),
                                                 [O.decode(shadow_k[s], O.BF16)], [O.decode(shadow_v[s], O.BF16)])
            diff = np.abs(got[cu[i]:cu[i + 1]].reshape(-1) - expected)
            assert diff.max() <= 2e-2 and diff.mean() <= 2e-3, (step, s, diff.max(), diff.mean())
        # gather returns exactly the shadow (bit-exact), across reused pages
        s = active[sample[0]]
        n = len(shadow_k[s])
        kout = torch.zeros((n, hkv, d), dtype=torch.bfloat16, device="cuda")
        vout = torch.zeros_like(kout)
        rig.gqa.page_gather(rig.pages, rig.table, s, 0, 0, n, kout, vout)
        rig.ctx.sync()
        assert np.array_equal(G.bits_of(kout), shadow_k[s]) and np.array_equal(G.bits_of(vout), shadow_v[s])
    assert reused > 50, "the trace must actually recycle page IDs"
    assert alloc.used() == sum(len(x) for x in pages)
    rig.close()


def test_churn_session_trace_matches_the_oracle_and_reuses_pages():
    # The benchmark's churn driver at a small scale: allocator-driven pages in a two-level table (8 page IDs per
    # logical block), slot resets, page reuse without clearing; every step a sample of sequences against the oracle.
    from psi_dec_b200 import workloads as PW
    trace = PW.ChurnTrace(slots=20, steps=10, seed=17, world=1, hi=1500, chunk=48, num_q_heads=16, num_kv_heads=2,
                          head_dim=128)
    churn = PW.ChurnSession(trace, ids_per_block=8)
    assert churn.layout.num_page_ids_per_block == 8
    rng = np.random.default_rng(1)
    for t in range(trace.steps):
        churn.prepare_step(t)
        churn.launch_step()
        churn.ctx.sync()
        assert churn.gqa.device_status() == 0
        q_len = trace.q_len[t]
        picks = set(rng.choice(trace.slots, size=3, replace=False).tolist())
        picks.add(int(np.argmax(q_len)))                      # always one chunked sequence
        picks.update(trace.finished[t - 1][:1] if t else [])  # and one that just moved into a reused slot
        for local in sorted(picks):
            max_abs, mean_abs = checks.churn_sequence_error(churn, t, local)
            assert max_abs <= 2e-2 and mean_abs <= 2e-3, (t, local, max_abs, mean_abs)
        churn.finish_step(t)
    assert churn.reused_pages > 0
    assert churn.allocator.used() == sum(len(ids) for ids in churn.page_ids)
    churn.close()


def test_churn_steps_from_pinned_host_buffers_run_as_overlapping_request_groups():
    # Steps large enough for the grouped host step (more than 64 MB of q + k + v, long query runs present): the output
    # that comes back in the host buffer against a twin session that runs the same trace from device memory (other
    # plans, so other KV splits: tolerance), a sample of sequences against the oracle, and the two arenas bit for bit.
    import torch
    from psi_dec_b200 import workloads as PW
    trace = PW.ChurnTrace(slots=64, steps=3, seed=23, world=1, hi=3000, chunk=512, chunk_fraction=0.4)
    host, twin = PW.ChurnSession(trace), PW.ChurnSession(trace)
    assert torch.equal(host.arena.view(torch.int16), twin.arena.view(torch.int16))
    kh, vh, qh = host.k.cpu().pin_memory(), host.v.cpu().pin_memory(), host.q.cpu().pin_memory()
    oh = torch.zeros_like(qh).pin_memory()
    for t in range(trace.steps):
        host.prepare_step(t, plan=False)
        twin.prepare_step(t)
        n = host.tokens
        assert n * (qh[0].numel() + 2 * kh[0].numel()) * 2 >= 64 << 20
        oh.fill_(float("nan"))
        before = host.ctx.launch_count
        host.host_step(kh, vh, qh, oh)
        assert host.ctx.launch_count - before >= 4, "the step must have run as several groups"
        twin.launch_step()
        twin.ctx.sync()
        assert host.gqa.device_status() == 0
        got, want = oh[:n].float(), twin.out[:n].float().cpu()
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= 2e-2
        assert torch.equal(host.arena.view(torch.int16), twin.arena.view(torch.int16))
        host.out[:n].copy_(oh[:n])   # the oracle helper reads the session's device output
        q_len = trace.q_len[t]
        for local in (0, int(np.argmax(q_len)), trace.slots - 1):
            max_abs, mean_abs = checks.churn_sequence_error(host, t, local)
            assert max_abs <= 2e-2 and mean_abs <= 2e-3, (t, local, max_abs, mean_abs)
        # the component is left unprepared after a grouped step
        with pytest.raises(pkg.PsiError, match="metadata must be updated"):
            host.gqa.attend(host.pages, host.table, 0, host.q[:n], host.out[:n])
        host.finish_step(t)
        twin.finish_step(t)
    host.close()
    twin.close()
