"""Worker of the multi-GPU tests: run under torch.distributed.run with one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        tests/multi_gpu_worker.py kv_range p2p

Modes: ``kv_range p2p|p2p3|nccl`` (configuration 4 scaled down, KV range split across the ranks, partial exchange, merged
output checked against the CPU oracle's merge of per-rank oracle partials), ``kv_range_free_run`` (the one-launch
exchange for a few hundred steps with no host synchronisation between them, so that ranks run ahead of one another
and the protocol's own ordering - two slots by step parity, the consumed word - is what keeps steps apart; every
step's output is checked afterwards) and ``sequence`` (configuration 3 scaled down, sequence-sharded, every rank
checked against the oracle on its own shard).
"""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import numpy as np
import torch
import torch.distributed as dist

import __graft_entry__ as entry

entry.load_package()
import checks
from oracle import psi_oracle as O
from psi_dec_b200 import workloads as W
from psi_dec_b200.distributed import KvRangeExchange


def main():
    kind = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if kind == "sequence":
        spec = W.config(3, scale_down=8).shard(rank, world)
        s = W.Session(spec, device=local)
        s.step()
        s.ctx.sync()
        checks.assert_attention_close(s)
        s.close()
    elif kind == "kv_range_free_run":
        steps, distinct = 300, 6
        spec = W.config(4, scale_down=32).kv_range_shard(rank, world)
        s = W.Session(spec, device=local)
        # a wait bound of seconds: a host that is held up for a moment on a shared machine is not a protocol failure
        ex = KvRangeExchange(s, rank, world, mode="p2p", max_polls=40_000_000)
        prob = checks.host_problem(s)
        queries = []
        for i in range(distinct):      # the same queries on every rank
            gen = torch.Generator(device=s.device)
            gen.manual_seed(777 + i)
            queries.append(torch.randn(s.q.shape, generator=gen, device=s.device, dtype=torch.float32).to(s.q.dtype))
        outs = torch.zeros((steps,) + tuple(s.out.shape), dtype=s.out.dtype, device=s.device) if rank == ex.owner else None
        dist.barrier()
        for step in range(steps):
            s.q.copy_(queries[step % distinct])   # stream-ordered in front of the launch
            ex.step()
            if rank == ex.owner:
                outs[step].copy_(s.out)           # stream-ordered behind it
        torch.cuda.synchronize()
        assert s.gqa.device_status() == 0
        dist.barrier()
        expected = []
        for i in range(distinct):
            q = checks.to_numpy_bits(queries[i])[prob["tok_rows"]]
            part = O.paged_attention(prob["arena"], spec.dtype, q, prob["req_slots"], prob["positions"], prob["table"], 0,
                                     prob["layout"], spec.num_q_heads, spec.num_kv_heads, spec.head_dim,
                                     spec.page_bytes, spec.scale, want_stats=True)
            gathered = [None] * world
            dist.all_gather_object(gathered, part)
            if rank == ex.owner:
                expected.append(checks.merged_oracle_partials(gathered, spec.num_tokens, spec.num_q_heads, spec.head_dim))
        if rank == ex.owner:
            got = O.decode(checks.to_numpy_bits(outs), spec.dtype)
            for step in range(steps):
                diff = np.abs(got[step] - expected[step % distinct])
                assert diff.max() <= 2e-2 and diff.mean() <= 2e-3, (step, diff.max(), diff.mean())
        dist.barrier()
        s.close()
    else:
        mode = sys.argv[2]
        whole = W.config(4, scale_down=32)
        spec = whole.kv_range_shard(rank, world)
        s = W.Session(spec, device=local)
        ex = KvRangeExchange(s, rank, world, mode=mode)
        prob = checks.host_problem(s)
        t, hq, d = spec.num_tokens, spec.num_q_heads, spec.head_dim
        for step in range(1, 5):
            # Every rank uses the same queries, and they change from step to step: a merge that read a slot of another
            # step would miss the oracle.  Only the three-launch mode needs the ranks held together between steps.
            gen = torch.Generator(device=s.device)
            gen.manual_seed(1234 + step)
            s.q.copy_(torch.randn(s.q.shape, generator=gen, device=s.device, dtype=torch.float32))
            if mode == "p2p3":
                torch.cuda.synchronize()
                dist.barrier()
            ex.step()
            s.ctx.sync()
            assert s.gqa.device_status() == 0
            # per-rank oracle partial on the rank's own arena, gathered on the host
            q = checks.to_numpy_bits(s.q)[prob["tok_rows"]]
            eo, em, es = O.paged_attention(prob["arena"], spec.dtype, q, prob["req_slots"], prob["positions"],
                                           prob["table"], 0, prob["layout"], spec.num_q_heads, spec.num_kv_heads,
                                           spec.head_dim, spec.page_bytes, spec.scale, want_stats=True)
            gathered = [None] * world
            dist.all_gather_object(gathered, (eo, em, es))
            if rank == ex.owner or mode == "nccl":
                expected = np.zeros((t, hq, d), dtype=np.float32)
                for i in range(t):
                    for h in range(hq):
                        expected[i, h] = O.merge_partials(np.stack([g[0][i, h] for g in gathered]),
                                                          [g[1][i, h] for g in gathered], [g[2][i, h] for g in gathered])
                got = O.decode(checks.to_numpy_bits(s.out), spec.dtype)
                diff = np.abs(got - expected)
                assert diff.max() <= 2e-2 and diff.mean() <= 2e-3, (step, diff.max(), diff.mean())
                if step == 4:
                    for r, (po, pm, pl) in enumerate(ex.partials_on_owner()):
                        assert np.abs(po - gathered[r][0]).max() <= 2e-2
                        assert np.abs(pm - gathered[r][1]).max() <= 2e-3
        dist.barrier()
        s.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print(f"multi-gpu worker ok: {' '.join(sys.argv[1:])} world={world}")


if __name__ == "__main__":
    main()
