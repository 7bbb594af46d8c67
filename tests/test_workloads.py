"""Host-side checks of the synthetic workload generators (no GPU): the sharding helpers and the churn trace."""
import numpy as np

import workloads as W


def test_churn_trace_keeps_the_books():
    tr = W.W.ChurnTrace(slots=64, steps=12, seed=9, world=4, hi=4096, chunk=64)
    assert tr.context.shape == (12, 64) and tr.q_len.shape == (12, 64)
    for t in range(12):
        q = tr.q_len[t]
        assert set(np.unique(q)) <= {1, 64}
        # 30 % of every rank's sequences carry a chunk
        for r in range(4):
            own = tr.rank_slots(r)
            assert (q[own] == 64).sum() == round(0.3 * len(own))
        assert len(tr.finished[t]) == round(0.1 * 64) and sorted(tr.admitted[t]) == tr.finished[t]
        if t + 1 < 12:
            grown = tr.context[t] + q
            for s in range(64):
                expected = tr.admitted[t][s] if s in tr.admitted[t] else grown[s]
                assert tr.context[t + 1][s] == expected
    assert tr.context.min() >= 128 and tr.max_context() <= 4096 + 12 * 64
    # the same seed gives the same sequence lengths whatever the rank count; only the slot a newcomer takes differs
    one = W.W.ChurnTrace(slots=64, steps=12, seed=9, world=1, hi=4096, chunk=64)
    assert sorted(one.context[0]) == sorted(tr.context[0])


def test_churn_admission_prefers_the_least_loaded_rank():
    tr = W.W.ChurnTrace(slots=64, steps=30, seed=3, world=8, hi=65536, chunk=128)
    blind = []
    for t in range(30):
        assert 1.0 <= tr.step_cost_share(t)
        blind.append(tr.step_cost_share(t))
    assert np.mean(blind) < 3.0
    d, f, n = tr.step_bytes_flops(0, tr.rank_slots(0), tokens_per_tile=2)
    assert d > 0 and f > 0 and n == int(tr.q_len[0][tr.rank_slots(0)].sum())


def test_kv_range_shards_cover_every_token_once():
    whole = W.config(4, scale_down=64)
    for world in (2, 3, 8):
        shards = [whole.kv_range_shard(r, world) for r in range(world)]
        assert sum(int(s.visible.sum()) for s in shards) == int(whole.visible.sum())
        assert [s.do_append for s in shards] == [False] * (world - 1) + [True]
