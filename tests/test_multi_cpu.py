"""World-size-2 gloo tests of the multi-GPU host logic on CPU (no GPU): how sequences and KV ranges are sharded,
and that per-rank partials exchanged between processes merge to the unsplit result."""
import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry

entry.load_package()
from oracle import psi_oracle as O
from psi_dec_b200 import workloads as W


def test_sequence_sharding_partitions_the_batch():
    whole = W.config(3)
    for world in (2, 4, 8):
        shards = [whole.shard(r, world) for r in range(world)]
        assert sum(s.num_seqs for s in shards) == whole.num_seqs
        assert sorted(np.concatenate([s.visible for s in shards]).tolist()) == sorted(whole.visible.tolist())
        loads = [int(s.visible.sum()) for s in shards]
        assert max(loads) <= 1.15 * (sum(loads) / world)


def test_custom_decode_batch_and_its_bench_argument():
    # bench.py --shape HQ,HKV,D,PAGE,BATCH,CTX_LO,CTX_HI[,Q_LEN] builds a seeded decode batch of another model profile
    import argparse
    import bench
    spec = W.custom(32, 8, 128, 8, 12, 100, 900, 2)
    assert (spec.num_q_heads, spec.num_kv_heads, spec.head_dim, spec.tokens_per_page, spec.num_seqs) == (32, 8, 128, 8, 12)
    assert spec.context_lens.min() >= 100 and spec.context_lens.max() <= 900 and np.all(spec.q_len == 2)
    assert np.array_equal(spec.context_lens, W.custom(32, 8, 128, 8, 12, 100, 900, 2).context_lens)   # seeded
    assert len(spec.block_tables) == 12 and all(len(t) == -(-(c + 2) // 8) for t, c in zip(spec.block_tables, spec.context_lens))
    args = argparse.Namespace(shape="32,8,128,8,12,100,900,2", gpus=1, config=2, scale_down=1)
    assert bench.workload(W, args).name == spec.name
    assert bench.workload(W, argparse.Namespace(shape=None, gpus=1, config=2, scale_down=1)).name == W.config(2).name
    with pytest.raises(SystemExit):
        bench.workload(W, argparse.Namespace(shape="1,2,3", gpus=1, config=2, scale_down=1))
    with pytest.raises(SystemExit):
        bench.workload(W, argparse.Namespace(shape="32,8,128,8,12,100,900", gpus=2, config=2, scale_down=1))
    # --shape HQ,HKV,D,PAGE --contexts C1,C2,...: one sequence per listed context (the reference's own bench fixtures)
    ragged = bench.workload(W, argparse.Namespace(shape="32,8,128,16", contexts="128,128,4096", dtype="f32", gpus=1, config=2,
                                                  scale_down=1))
    assert ragged.context_lens.tolist() == [128, 128, 4096] and ragged.dtype == O.F32 and ragged.tokens_per_page == 16


def test_kv_range_sharding_covers_each_context_once():
    whole = W.config(4, scale_down=16)
    for world in (2, 4, 8):
        shards = [whole.kv_range_shard(r, world) for r in range(world)]
        total = sum(s.visible for s in shards)
        assert np.array_equal(total, whole.visible)
        assert [s.do_append for s in shards] == [False] * (world - 1) + [True]
        for s in shards[:-1]:
            assert np.all(s.visible % whole.tokens_per_page == 0)   # page-aligned slices


def _merge_worker(rank, world, port, results):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    # one sequence of 96 tokens in 16-token pages, 4 q heads / 2 kv heads, D=8, f32; every rank builds the same data
    rng = np.random.default_rng(5)
    hq, hkv, d, p, ctx = 4, 2, 8, 16, 96
    pages = rng.standard_normal((6, 2, hkv, p, d)).astype(np.float32).reshape(-1)
    q = rng.standard_normal((1, hq, d)).astype(np.float32)
    layout = O.Layout(1, 1, 6, 1)
    table = np.arange(6, dtype=np.uint32)
    lo, hi = (0, 48) if rank == 0 else (48, 96)
    o, m, s = O.paged_attention(pages, O.F32, q, [0], [ctx - 1], table, 0, layout, hq, hkv, d, 2 * hkv * p * d * 4, 0.3,
                                kv_begin=lo, kv_end=hi, want_stats=True)
    mine = torch.from_numpy(np.concatenate([o.reshape(-1), m.reshape(-1), s.reshape(-1)]))
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    full = O.paged_attention(pages, O.F32, q, [0], [ctx - 1], table, 0, layout, hq, hkv, d, 2 * hkv * p * d * 4, 0.3)
    n = hq * d
    for h in range(hq):
        merged = O.merge_partials(np.stack([g[:n].numpy().reshape(hq, d)[h] for g in gathered]),
                                  [float(g[n + h]) for g in gathered], [float(g[n + hq + h]) for g in gathered])
        assert np.max(np.abs(merged - full[0, h])) <= 1e-5
    dist.barrier()
    dist.destroy_process_group()
    results[rank] = 1


def test_partials_exchanged_between_two_processes_merge_to_the_unsplit_result():
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_merge_worker, args=(2, 29617, results), nprocs=2, join=True)
    assert dict(results) == {0: 1, 1: 1}
