"""The KV-range exchange as one launch per rank (psi_gqa_attend_exchange), on ONE device.

The ranks of a group are emulated by sessions on the same GPU whose launches run one after the other in one stream,
with an ordinary device buffer standing in for the owner's peer-mapped receive area.  A wait in such a launch is either
already satisfied when the launch starts (the producers ran first) or is meant to run out (nothing will publish): no
launch here waits for a launch that comes after it.  The true multi-device run is tests/test_gpu_multi.py.
"""
import numpy as np
import pytest

import checks
import workloads as W
from oracle import psi_oracle as O

pkg = W.pkg
pytestmark = pytest.mark.gpu


class Group:
    """`world` emulated ranks over configuration 4 scaled down; the last rank owns the receive area."""

    def __init__(self, world, scale_down=64, kernel_mode=pkg.KERNEL_AUTO):
        import torch
        self.torch = torch
        self.world = world
        self.whole = W.config(4, scale_down=scale_down)
        self.shards = [W.Session(self.whole.kv_range_shard(r, world), kernel_mode=kernel_mode) for r in range(world)]
        self.owner = self.shards[-1]
        spec = self.whole
        self.rows = spec.num_tokens * spec.num_q_heads
        self.slot = (self.rows * (spec.head_dim + 2) + 3) // 4 * 4
        self.flag_words = (world + 3) // 4 * 4
        self.area = torch.zeros(2 * world * self.slot + self.flag_words + 4, dtype=torch.float32, device="cuda:0")
        self.words = self.area[2 * world * self.slot:].view(torch.int32)

    def descriptor(self, rank, step, max_polls=0):
        base = self.area.data_ptr()
        flags = base + 4 * 2 * self.world * self.slot
        return pkg.KvExchange(rank, self.world, self.world - 1, step, base, self.slot, flags, flags + 4 * self.flag_words,
                              max_polls)

    def flags(self):
        return self.words[: self.world].tolist()

    def consumed(self):
        return int(self.words[self.flag_words])

    def set_queries(self, seed):
        gen = self.torch.Generator(device="cuda:0")
        gen.manual_seed(seed)
        q = self.torch.randn(self.owner.q.shape, generator=gen, device="cuda:0", dtype=self.torch.float32)
        for sh in self.shards:
            sh.q.copy_(q)

    def run_rank(self, rank, step, out=None, max_polls=0):
        sh = self.shards[rank]
        k, v = (sh.k, sh.v) if sh.spec.do_append else (None, None)
        sh.gqa.attend_exchange(sh.pages, sh.table, 0, sh.q, self.descriptor(rank, step, max_polls),
                               out=out if rank == self.world - 1 else None, k=k, v=v)

    def expected(self):
        """The oracle's merge of the oracle's per-rank partials (each rank's own arena and table)."""
        parts = []
        for sh in self.shards:
            sh.ctx.sync()
            prob = checks.host_problem(sh)
            q = checks.to_numpy_bits(sh.q)[prob["tok_rows"]]
            parts.append(O.paged_attention(prob["arena"], sh.spec.dtype, q, prob["req_slots"], prob["positions"],
                                           prob["table"], 0, prob["layout"], sh.spec.num_q_heads, sh.spec.num_kv_heads,
                                           sh.spec.head_dim, sh.spec.page_bytes, sh.spec.scale, want_stats=True))
        t, hq, d = self.whole.num_tokens, self.whole.num_q_heads, self.whole.head_dim
        expected = np.zeros((t, hq, d), dtype=np.float32)
        for i in range(t):
            for h in range(hq):
                expected[i, h] = O.merge_partials(np.stack([p[0][i, h] for p in parts]), [p[1][i, h] for p in parts],
                                                  [p[2][i, h] for p in parts])
        return expected

    def close(self):
        for sh in self.shards:
            sh.close()


def _assert_close(group, out):
    got = O.decode(checks.to_numpy_bits(out), group.whole.dtype)
    diff = np.abs(got - group.expected())
    assert diff.max() <= checks.MAX_ABS_16BIT and diff.mean() <= checks.MEAN_ABS_16BIT, (diff.max(), diff.mean())


@pytest.mark.parametrize("world,kernel_mode", [(2, pkg.KERNEL_AUTO), (4, pkg.KERNEL_AUTO), (8, pkg.KERNEL_AUTO), (2, pkg.KERNEL_GENERIC)])
def test_exchange_merges_every_step_against_the_oracle(world, kernel_mode):
    # Queries change from step to step, so a merge that mixed two steps' partials would miss the oracle.
    import torch
    g = Group(world, kernel_mode=kernel_mode)
    for step in range(1, 6):
        g.set_queries(100 + step)
        out = torch.full_like(g.owner.q, float("nan"))
        for rank in range(world):            # producers first, the owner last: its wait finds every flag set
            g.run_rank(rank, step, out=out)
        assert g.owner.gqa.device_status() == 0
        assert g.flags() == [step] * world and g.consumed() == step
        _assert_close(g, out)
    g.close()


def test_exchange_owner_gives_up_when_a_rank_never_publishes_and_recovers():
    import torch
    g = Group(2)
    g.set_queries(7)
    canary = torch.full_like(g.owner.q, 7.0)
    g.run_rank(1, 1, out=canary, max_polls=2000)          # rank 0 has not run: nothing sets its flag
    assert g.owner.gqa.device_status() == 4               # PSI_ERR_TIMEOUT
    assert bool((canary == 7.0).all())                    # one verdict for the launch: no row was written
    assert g.flags() == [0, 1] and g.consumed() == 0
    assert g.owner.gqa.device_status() == 0               # cleared; the context keeps working
    g.run_rank(0, 1)                                      # the late rank arrives; the owner repeats its step
    out = torch.full_like(g.owner.q, float("nan"))
    g.run_rank(1, 1, out=out)
    assert g.owner.gqa.device_status() == 0
    assert g.flags() == [1, 1] and g.consumed() == 1
    _assert_close(g, out)
    g.close()


def test_exchange_producer_does_not_overwrite_a_slot_the_owner_has_not_merged():
    # Rank 0 runs ahead: steps 1 and 2 fit the two slot parities, step 3 needs the owner to have merged step 1.
    import torch
    g = Group(2)
    g.set_queries(11)
    g.run_rank(0, 1)
    g.run_rank(0, 2)
    g.shards[0].ctx.sync()
    assert g.flags()[0] == 2
    slot_of_step_1 = g.area[g.slot * 2 * 1 + 0 * g.slot: g.slot * 2 * 1 + g.slot].clone()   # parity 1, rank 0
    g.set_queries(12)
    g.run_rank(0, 3, max_polls=2000)                      # consumed is 0 < 1: the bounded wait runs out
    assert g.shards[0].gqa.device_status() == 4
    assert g.flags()[0] == 2                              # step 3 was not published
    assert torch.equal(g.area[g.slot * 2: g.slot * 3], slot_of_step_1)   # and step 1's partial is intact
    # the owner catches up on steps 1 and 2 (queries of step 1 and 2 were seed 11), then step 3 goes through
    g.set_queries(11)
    for step in (1, 2):
        out = torch.full_like(g.owner.q, float("nan"))
        g.run_rank(1, step, out=out)
        assert g.owner.gqa.device_status() == 0
        _assert_close(g, out)
    g.set_queries(12)
    g.run_rank(0, 3)
    out = torch.full_like(g.owner.q, float("nan"))
    g.run_rank(1, 3, out=out)
    assert g.owner.gqa.device_status() == 0 and g.shards[0].gqa.device_status() == 0
    assert g.flags() == [3, 3] and g.consumed() == 3
    _assert_close(g, out)
    g.close()


def test_exchange_argument_contracts():
    import torch
    g = Group(2)
    bad = g.descriptor(0, 0)
    sh = g.shards[0]
    with pytest.raises(pkg.PsiError, match="steps count from 1"):
        sh.gqa.attend_exchange(sh.pages, sh.table, 0, sh.q, bad)
    small = g.descriptor(0, 1)
    small.slot_floats = 8
    with pytest.raises(pkg.PsiError, match="slot_floats"):
        sh.gqa.attend_exchange(sh.pages, sh.table, 0, sh.q, small)
    with pytest.raises(pkg.PsiError, match="owner of the exchange needs an output"):
        g.owner.gqa.attend_exchange(g.owner.pages, g.owner.table, 0, g.owner.q, g.descriptor(1, 1))
    torch.cuda.synchronize()
    assert g.flags() == [0, 0]                            # nothing was launched
    g.close()
