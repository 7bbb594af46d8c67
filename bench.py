"""Benchmark of the paged GQA decode hot path (KV append + split-KV attention) on N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --steps 3 --warmup 1        # the reference arm: CPU restatement on host cores

One step is one pass of the hot path over one batch of seeded synthetic input: append this step's K/V rows into their
pages, then attend over every visible key.  At N GPUs the batch is N times larger and sequence-sharded, one shard per
rank, with no data-path collective (weak scaling).  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for extra in (ROOT, ROOT / "tests"):
    if str(extra) not in sys.path:
        sys.path.insert(0, str(extra))

METRIC = "paged_gqa_decode_kv_read_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1400.0
# dram__bytes_read.sum + dram__bytes_write.sum of one attend_mma_kernel launch divided by the launch's algorithmic
# bytes, from the ncu capture summarised in profiles/attend_mma_cfg2_ncu_full.md (301.27 MB for 296.76 MB).
NCU_DRAM_BYTES_PER_ALGORITHMIC_BYTE = {"cfg2-a3b-layer-decode": 301.27 / 296.76}


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s of a library GEMM timed inside a seconds-long loop (the chunk kernel runs for milliseconds
    per launch under the power cap), else the stated fallback."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["bf16_tflops_sustained"]), "measured (sustained)"
        except Exception:
            pass
    return FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 7]
        os.unlink(self.file.name)
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in rows:
            try:
                sm.append(float(row[0]))
                sm_max.append(float(row[1]))
            except ValueError:
                continue
            for name, value in zip(names, row[4:8]):
                if value.strip().lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def bench_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry
    pkg = entry.load_package()
    from psi_dec_b200 import workloads as W
    from psi_dec_b200.distributed import KvRangeExchange

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} disagrees with WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    # How the job is spread over N GPUs.  The headline configuration (2) grows with N: the global batch is N x 32
    # sequences, sequence-sharded, no collective in the step (weak scaling).  Configurations 3 and 5 shard their fixed
    # batch by sequence, configuration 4 splits every sequence's KV range across the ranks and exchanges partials
    # (strong scaling).
    base = workload(W, args)
    exchange = None
    scaling, parallelism = "weak", f"sequence-sharded x{world}"
    if world == 1:
        spec = base
    elif args.config == 4:
        spec = base.kv_range_shard(rank, world)
        scaling, parallelism = "strong", f"kv-range-split x{world} ({args.exchange} partial exchange)"
    elif args.config in (3, 5):
        spec = base.shard(rank, world)
        scaling = "strong"
    else:
        specs = [W.config(args.config, scale_down=args.scale_down, seed=base.seed + 100 * r) for r in range(world)]
        whole = W.Spec(base.name, base.dtype, base.num_q_heads, base.num_kv_heads, base.head_dim,
                       base.tokens_per_page, np.concatenate([s.context_lens for s in specs]),
                       np.concatenate([s.q_len for s in specs]), base.seed)
        spec = whole.shard(rank, world)
    kernel_mode = {"auto": pkg.KERNEL_AUTO, "mma": pkg.KERNEL_MMA, "generic": pkg.KERNEL_GENERIC,
                   "mma_sync": pkg.KERNEL_MMA_SYNC}[args.kernel]
    session = W.Session(spec, device=local_rank, kernel_mode=kernel_mode)
    if world > 1 and args.config == 4:
        exchange = KvRangeExchange(session, rank, world, mode=args.exchange)
    step = exchange.step if exchange else session.step
    ctx = session.ctx
    alg = spec.algorithmic_bytes()
    # Larger than the 126 MB L2 and swept read-only between timed steps, so that the step's inputs are not resident
    # and no dirty lines are left for the timed kernels to write back.
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=session.device)  # f32: summed without a cast copy

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """Per-step CUDA-event durations (ms) on the launching stream, L2 sweep between steps outside the windows.
        With an exchange in the step every rank enters each step together (barrier), as a serving loop would."""
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        # A few sweeps ahead of the first window keep the GPU busy while the host enqueues it: without them the first
        # window also measures how long the host takes to submit the step after the preceding synchronize.
        for _ in range(4):
            flush.sum()
        for i in range(steps):
            flush.sum()
            if exchange:
                barrier()
            starts[i].record(session.stream)
            fn()
            ends[i].record(session.stream)
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in zip(starts, ends)]

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches_before = ctx.launch_count
    barrier()
    step_ms = timed(step, args.steps)
    barrier()
    launches = ctx.launch_count - launches_before
    # The dominant kernel on its own clock: the same steps again with the library's per-launch event pairs switched
    # on (kept out of the pass above, where the extra events would sit inside the step time).
    ctx.enable_kernel_timing(True)
    timed(step, args.steps)
    map_ms, map_n = ctx.kernel_timing(1)
    append_ms, append_n = ctx.kernel_timing(0)
    reduce_ms, reduce_n = ctx.kernel_timing(2)
    combine_ms, combine_n = ctx.kernel_timing(3)
    chunk_ms, chunk_n = ctx.kernel_timing(5)
    ctx.enable_kernel_timing(False)
    barrier()

    # End to end through the C ABI with host buffers: metadata upload, H2D of q/k/v, append, attend, D2H of out.
    kh, vh, qh = session.k.cpu().pin_memory(), session.v.cpu().pin_memory(), session.q.cpu().pin_memory()
    oh = torch.empty_like(qh).pin_memory()
    batch = spec.batch()

    def e2e_step():
        if exchange:
            session.gqa.prepare(*batch)
            session.q.copy_(qh, non_blocking=True)
            if spec.do_append:
                session.k.copy_(kh, non_blocking=True)
                session.v.copy_(vh, non_blocking=True)
            exchange.step()
            if rank == exchange.owner or args.exchange == "nccl":
                oh.copy_(session.out, non_blocking=True)
            session.stream.synchronize()
        else:
            session.gqa.step_host(session.pages, session.table, spec.layer, *batch, kh, vh, qh, oh)

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_ms = timed(e2e_step, args.steps)
    barrier()
    clocks = sampler.stop() if sampler else None

    total_ms = sum(step_ms)
    e2e_total_ms = sum(e2e_ms)
    h2d = kh.numel() * kh.element_size() * 2 * (1 if spec.do_append else 0) + qh.numel() * qh.element_size()
    d2h = oh.numel() * oh.element_size() if (exchange is None or rank == exchange.owner) else 0
    sums = torch.tensor([float(alg["total"]), float(spec.num_tokens), float(alg["kv"]), float(h2d), float(d2h)],
                        dtype=torch.float64, device=session.device)
    worst = torch.tensor([total_ms, e2e_total_ms], dtype=torch.float64, device=session.device)
    if world > 1:
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    job_bytes, job_tokens, job_kv, job_h2d, job_d2h = (float(x) for x in sums.tolist())
    if exchange:
        job_tokens = float(base.num_tokens)  # every rank works on the same query tokens
    total_ms, e2e_total_ms = (float(x) for x in worst.tolist())

    if rank == 0:
        peak, peak_kind = measured_peak()
        ms_per_step = total_ms / args.steps
        value = job_bytes / (ms_per_step * 1e-3) / 1e9
        map_avg_ms = map_ms / max(map_n, 1)
        achieved = alg["total"] / (map_avg_ms * 1e-3) / 1e9 if map_n else 0.0
        stats = session.gqa.plan_stats()
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "bf16" if spec.dtype == pkg.BF16 else "f16/f32",
            "data": "synthetic",
            "config": {"workload": base.name if args.scale_down == 1 else f"{base.name}/scaled-down-{args.scale_down}",
                       "sequences_rank0": spec.num_seqs, "q_heads": spec.num_q_heads,
                       "kv_heads": spec.num_kv_heads, "head_dim": spec.head_dim,
                       "tokens_per_page": spec.tokens_per_page, "visible_tokens_rank0": int(spec.visible.sum()),
                       "seed": base.seed, "parallelism": parallelism,
                       "l2": "256 MB read-only sweep between timed steps",
                       "kernel": "mma" if stats["kernel"] == 2 else "generic",
                       "ctas": stats["ctas"], "items": stats["items"], "reduce_units": stats["reduce_units"]},
            "tokens_per_s": round(job_tokens / (ms_per_step * 1e-3), 1),
            "kv_gbs": round(job_kv / (ms_per_step * 1e-3) / 1e9, 1),
            "frac_of_nominal_8tbs_per_gpu": round(value / world / NOMINAL_HBM_GBS, 4),
            "roofline": {"bound": "hbm", "kernel": "attend_map (rank 0)", "achieved": round(achieved, 1), "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": round(achieved / peak, 4),
                         "traffic": None, "algorithmic_bytes_per_launch": alg["total"],
                         "avg_launch_ms": round(map_avg_ms, 5), "launches": map_n},
            "kernel_ms_per_step": {"append": round(append_ms / max(append_n, 1), 5),
                                   "attend_map": round(map_avg_ms, 5),
                                   "attend_reduce": round(reduce_ms / max(reduce_n, 1), 5),
                                   "combine": round(combine_ms / max(combine_n, 1), 5),
                                   "attend_chunk": round(chunk_ms / max(chunk_n, 1), 5)},
            "e2e": {"value": round(job_bytes / (e2e_total_ms / args.steps * 1e-3) / 1e9, 1), "unit": UNIT,
                    "ms_per_step": round(e2e_total_ms / args.steps, 5),
                    "tokens_per_s": round(job_tokens / (e2e_total_ms / args.steps * 1e-3), 1),
                    "h2d_bytes_per_step": int(job_h2d), "d2h_bytes_per_step": int(job_d2h)},
            "gpu_launches": int(launches),
            "clocks": clocks,
            # rank 0's per-step distribution (the headline ms_per_step is the mean of the slowest rank)
            "ms_per_step_rank0": {"median": round(statistics.median(step_ms), 5), "min": round(min(step_ms), 5),
                                  "max": round(max(step_ms), 5)},
        }
        if chunk_n and chunk_ms > map_ms:
            # long query runs dominate the step: the chunk kernel is a contraction, bounded by the tensor pipe
            flops = spec.long_run_flops(16 // min(16, spec.num_q_heads // spec.num_kv_heads))
            tensor_peak, tensor_kind = measured_tensor_peak()
            chunk_avg_ms = chunk_ms / chunk_n
            tflops = flops / (chunk_avg_ms * 1e-3) / 1e12
            engine = "tcgen05" if stats["chunk_tcgen05_launches"] else "mma.sync"
            line["roofline"] = {"bound": "tensor", "kernel": f"attend_chunk ({engine}, rank 0)",
                                "achieved": round(tflops, 1), "peak": tensor_peak, "peak_kind": tensor_kind,
                                "unit": "TFLOP/s", "frac": round(tflops / tensor_peak, 4), "traffic": None,
                                "flops_per_launch": flops, "avg_launch_ms": round(chunk_avg_ms, 5),
                                "launches": chunk_n}
            line["config"]["chunk_ctas"] = stats["chunk_ctas"]
            line["config"]["chunk_items"] = stats["chunk_items"]
        per_byte = NCU_DRAM_BYTES_PER_ALGORITHMIC_BYTE.get(base.name)
        if per_byte and stats["kernel"] == 2 and line["roofline"]["bound"] == "hbm":
            line["roofline"]["traffic"] = int(per_byte * alg["total"])
        if world == 1 and line["roofline"]["bound"] == "hbm" and not args.no_read_probe:
            # the ceiling of a kernel that only reads HBM (4 GiB through 16-byte loads), beside the copy figure in `peak`
            probe = session.ctx.read_bandwidth(4 << 30, 5)
            line["roofline"]["read_only_probe_gbs"] = round(probe, 1)
            line["roofline"]["frac_of_read_only_probe"] = round(achieved / probe, 4) if probe > 0 else None
        if world == 1 and not args.no_cpu_baseline:
            import checks
            tok_s, bytes_s, desc, threads = checks.time_oracle_sample(session, seconds_target=12.0)
            line["cpu_baseline"] = {"value": round(bytes_s / 1e9, 4), "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": desc, "tokens_per_s": round(tok_s, 2)}
        print(json.dumps(line), flush=True)
    barrier()
    session.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def bench_reference(args):
    """The reference's own implementation of the path cannot run here (Rust + Metal), so this arm times the CPU
    restatement of its algorithm (the oracle) with every host thread, on a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    import __graft_entry__ as entry
    entry.load_package()
    from oracle import psi_oracle as O
    from psi_dec_b200 import workloads as W

    base = workload(W, args)
    order = np.argsort(base.visible, kind="stable")
    budget = 400_000 * max(1, O.num_threads()) // 8  # visible tokens per step: a step of roughly a second
    chosen, total = [], 0
    for s in order:
        if chosen and total + int(base.visible[s]) > budget:
            break
        chosen.append(int(s))
        total += int(base.visible[s])
    sample = W.Spec(base.name + "/sample", base.dtype, base.num_q_heads, base.num_kv_heads, base.head_dim,
                    base.tokens_per_page, base.context_lens[chosen], base.q_len[chosen], base.seed)
    rng = np.random.default_rng(base.seed)
    page_elems = sample.page_bytes // sample.elem_bytes
    arena = O.encode(rng.standard_normal((sample.num_pages, page_elems), dtype=np.float32), sample.dtype).reshape(-1)
    t = sample.num_tokens
    q = O.encode(rng.standard_normal((t, sample.num_q_heads, sample.head_dim), dtype=np.float32), sample.dtype)
    k = O.encode(rng.standard_normal((t, sample.num_kv_heads, sample.head_dim), dtype=np.float32), sample.dtype)
    v = O.encode(rng.standard_normal((t, sample.num_kv_heads, sample.head_dim), dtype=np.float32), sample.dtype)
    max_pages = int(sample.pages_per_seq().max())
    table = np.zeros((sample.num_seqs, 1, max_pages, 1), dtype=np.uint32)
    for s, ids in enumerate(sample.block_tables):
        table[s, 0, : len(ids), 0] = ids
    layout = O.Layout(sample.num_seqs, 1, max_pages, 1)
    req_slots, positions = [], []
    for s in range(sample.num_seqs):
        for j in range(int(sample.q_len[s])):
            req_slots.append(s)
            positions.append(int(sample.context_lens[s]) + j)

    def step():
        O.kv_page_write(arena, k, v, req_slots, positions, table.reshape(-1), t, 0, layout, sample.num_kv_heads,
                        sample.head_dim, sample.page_bytes)
        O.paged_attention(arena, sample.dtype, q, req_slots, positions, table.reshape(-1), 0, layout,
                          sample.num_q_heads, sample.num_kv_heads, sample.head_dim, sample.page_bytes, sample.scale)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    elapsed = time.perf_counter() - t0
    alg = sample.algorithmic_bytes()
    ms_per_step = elapsed / args.steps * 1e3
    value = alg["total"] / (ms_per_step * 1e-3) / 1e9
    desc = f"{len(chosen)} shortest of {base.num_seqs} sequences ({total} visible tokens) per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": base.name, "sample": desc, "seed": base.seed},
        "tokens_per_s": round(sample.num_tokens / (ms_per_step * 1e-3), 2),
        "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                         "sample": desc},
        "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference algorithm; the reference's Rust + Metal path cannot build or run here",
    }
    print(json.dumps(line), flush=True)


def workload(W, args):
    """The benchmark configuration, or the custom decode batch --shape describes."""
    if args.shape is None:
        return W.config(args.config, scale_down=args.scale_down)
    if args.gpus != 1:
        raise SystemExit("--shape runs on one GPU")
    values = [int(x) for x in args.shape.split(",")]
    if len(values) not in (7, 8):
        raise SystemExit("--shape wants HQ,HKV,D,PAGE,BATCH,CTX_LO,CTX_HI[,Q_LEN]")
    return W.custom(*values)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--config", type=int, default=2, help="benchmark configuration (2 = the headline)")
    parser.add_argument("--scale-down", type=int, default=1,
                        help="divide batch and context sizes (small cases for profiler captures; not a bench value)")
    parser.add_argument("--shape", default=None, metavar="HQ,HKV,D,PAGE,BATCH,CTX_LO,CTX_HI[,Q_LEN]",
                        help="one GPU only: a decode batch of another model profile instead of --config")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-read-probe", action="store_true", help="skip the read-only HBM bandwidth probe")
    parser.add_argument("--kernel", choices=["auto", "mma", "generic", "mma_sync"], default="auto",
                        help="attention kernel: tensor-core kernels (default where supported), the CUDA-core kernel, or "
                             "mma_sync = tensor-core kernels with long query runs kept off the tcgen05 kernel")
    parser.add_argument("--exchange", choices=["p2p", "nccl"], default="p2p",
                        help="partial exchange of the KV-range-split configuration 4")
    args = parser.parse_args()
    if args.impl == "reference":
        bench_reference(args)
    else:
        bench_ours(args)


if __name__ == "__main__":
    main()
