"""Benchmark of the paged GQA decode hot path (KV append + split-KV attention) on N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --steps 3 --warmup 1        # the reference arm: CPU restatement on host cores

One step is one pass of the hot path over one batch of seeded synthetic input: append this step's K/V rows into their
pages, then attend over every visible key.  Rank 0 prints one JSON line.

The line's headline is the layer-decode batch (32 sequences per GPU, sequence-sharded, no collective in the step:
weak scaling).  Beside it, under ``splits``, the same run measures the other ways the path is spread over GPUs: the
verify batch sharded by sequence (strong scaling), the long-context batch split by KV range with the partial exchange
in the attention launch (strong scaling), and the continuous-batching churn trace sharded sticky by request slot.
``--config N`` runs one configuration alone as the headline instead.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "paged_gqa_decode_kv_read_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1400.0
L2_NOTE = "256 MB read-only sweep between timed steps"


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


TRAFFIC_SUMMARY = ROOT / "profiles" / "attend_mma_dram_traffic.txt"
KERNEL_SOURCES = ("attend_mma.cu", "mma_common.cuh", "device_common.cuh")


def kernel_source_hash() -> str:
    digest = hashlib.sha256()
    for name in KERNEL_SOURCES:
        digest.update((ROOT / "psi-dec_b200" / "csrc" / name).read_bytes())
    return digest.hexdigest()


def record_traffic(report: str, workload_name: str, command: str):
    """Reads an ncu report of the decode kernel (here, no GPU needed) and writes the per-launch DRAM traffic beside the
    profiler summaries, with the hash of the kernel sources it was taken with:

        python bench.py --record-traffic prof_attend_mma_cfg2.ncu-rep
    """
    import csv
    raw = subprocess.run(["ncu", "-i", report, "--page", "raw", "--csv"], capture_output=True, text=True, check=True).stdout
    rows = list(csv.reader(raw.splitlines()))
    header, units = rows[0], rows[1]
    col = {name: i for i, name in enumerate(header)}
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    launches = []
    for row in rows[2:]:
        if "attend_mma_kernel" not in row[col["Kernel Name"]]:
            continue
        total = 0.0
        for metric in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
            total += float(row[col[metric]]) * scale[units[col[metric]]]
        launches.append(total)
    if not launches:
        raise SystemExit("the report holds no attend_mma_kernel launch")
    import __graft_entry__ as entry
    entry.load_package()
    from psi_dec_b200 import workloads as W
    spec = {c.name: c for c in (W.config(i) for i in (2, 3, 4))}[workload_name]
    TRAFFIC_SUMMARY.write_text(
        "# DRAM traffic of one attend_mma_kernel launch (ncu: dram__bytes_read.sum + dram__bytes_write.sum, mean of the\n"
        "# captured launches); bench.py scales it by a run's algorithmic bytes for roofline.traffic and ignores it once\n"
        "# the kernel sources named by the hash have changed.  Written by: python bench.py --record-traffic <report>\n"
        f"workload: {workload_name}\n"
        f"captured_launches: {len(launches)}\n"
        f"dram_bytes_per_launch: {int(sum(launches) / len(launches))}\n"
        f"algorithmic_bytes_per_launch: {spec.algorithmic_bytes()['total']}\n"
        f"kernel_sources: {' '.join(KERNEL_SOURCES)}\n"
        f"kernel_source_sha256: {kernel_source_hash()}\n"
        f"capture_command: {command}\n")
    print(TRAFFIC_SUMMARY.read_text())


def recorded_traffic(workload_name: str, algorithmic_bytes: int):
    """DRAM bytes per launch of the decode kernel from the committed profiler summary of this workload, scaled by the
    launch's algorithmic bytes.  The summary names the kernel sources it was taken with (a hash); when they have
    changed since, the figure is stale and None is returned together with that fact."""
    summary = TRAFFIC_SUMMARY
    if not summary.exists():
        return None, "no profiler summary"
    fields = {}
    for line in summary.read_text().splitlines():
        if ":" in line and not line.startswith("#"):
            key, value = line.split(":", 1)
            fields[key.strip()] = value.strip()
    if fields.get("workload") != workload_name:
        return None, "profiler summary covers another workload"
    if fields.get("kernel_source_sha256") != kernel_source_hash():
        return None, "profiler summary predates the current kernel source"
    per_byte = float(fields["dram_bytes_per_launch"]) / float(fields["algorithmic_bytes_per_launch"])
    return int(per_byte * algorithmic_bytes), "ncu dram__bytes_read.sum + dram__bytes_write.sum, scaled by algorithmic bytes"


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


class Job:
    """The process group of one bench run and the helpers every measurement shares."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world > 1:
            raise SystemExit(f"--gpus {args.gpus} disagrees with WORLD_SIZE={self.world}")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            # NCCL only carries barriers and a few scalars here; NVLink multicast objects are not needed for that
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            dist.init_process_group("nccl", device_id=self.device)
        # Larger than the 126 MB L2 and swept read-only between timed steps, so that a step's inputs are not resident
        # and no dirty lines are left for the timed kernels to write back.  f32: summed without a cast copy.
        self.flush = torch.zeros(64 << 20, dtype=torch.float32, device=self.device)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, steps, stream, barrier_each=False):
        """Per-step CUDA-event durations (ms) on the launching stream, L2 sweep between steps outside the windows.
        With an exchange in the step every rank enters each step together (barrier), as a serving loop would."""
        torch = self.torch
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        # A few sweeps ahead of the first window keep the GPU busy while the host enqueues it: without them the first
        # window also measures how long the host takes to submit the step after the preceding synchronize.
        for _ in range(4):
            self.flush.sum()
        for i in range(steps):
            self.flush.sum()
            if barrier_each:
                self.barrier()
            starts[i].record(stream)
            fn()
            ends[i].record(stream)
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in zip(starts, ends)]

    def reduce(self, values, op):
        """All-reduce of a list of floats (float64) over the ranks; op is 'sum', 'max' or 'min'."""
        t = self.torch.tensor([float(v) for v in values], dtype=self.torch.float64, device=self.device)
        if self.world > 1:
            ops = {"sum": self.dist.ReduceOp.SUM, "max": self.dist.ReduceOp.MAX, "min": self.dist.ReduceOp.MIN}
            self.dist.all_reduce(t, op=ops[op])
        return [float(x) for x in t.tolist()]

    def close(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def workload(W, args, index=None):
    """The benchmark configuration, or the custom decode batch --shape describes."""
    if args.shape is None:
        return W.config(index if index is not None else (args.config or 2), scale_down=args.scale_down)
    if args.gpus != 1:
        raise SystemExit("--shape runs on one GPU")
    values = [int(x) for x in args.shape.split(",")]
    if getattr(args, "contexts", None) is not None:
        if len(values) != 4:
            raise SystemExit("with --contexts, --shape wants HQ,HKV,D,PAGE")
        dtype = {"bf16": 1, "f16": 2, "f32": 0}[getattr(args, "dtype", "bf16")]
        return W.explicit(*values, [int(x) for x in args.contexts.split(",")], dtype=dtype)
    if len(values) not in (7, 8):
        raise SystemExit("--shape wants HQ,HKV,D,PAGE,BATCH,CTX_LO,CTX_HI[,Q_LEN]")
    return W.custom(*values)


def spread(W, pkg, base, index, job, args):
    """This rank's part of configuration `index` over the job's GPUs: (spec, scaling, parallelism, whole-job spec)."""
    import numpy as np
    world, rank = job.world, job.rank
    if world == 1:
        return base, "weak", "one GPU", base
    if index == 4:
        return (base.kv_range_shard(rank, world), "strong",
                f"kv-range-split x{world} ({args.exchange} partial exchange)", base)
    if index in (3, 5):
        return base.shard(rank, world), "strong", f"sequence-sharded x{world}", base
    # the headline grows with the GPU count: N x 32 sequences, sequence-sharded
    specs = [W.config(index, scale_down=args.scale_down, seed=base.seed + 100 * r) for r in range(world)]
    whole = W.Spec(base.name, base.dtype, base.num_q_heads, base.num_kv_heads, base.head_dim, base.tokens_per_page,
                   np.concatenate([s.context_lens for s in specs]), np.concatenate([s.q_len for s in specs]), base.seed)
    return whole.shard(rank, world), "weak", f"sequence-sharded x{world}", whole


def config_block(whole, parallelism):
    """The `config` object of a line: what the workload is, the same in this arm and in the reference arm."""
    return {"workload": whole.name, "sequences": int(whole.num_seqs), "q_heads": whole.num_q_heads,
            "kv_heads": whole.num_kv_heads, "head_dim": whole.head_dim, "tokens_per_page": whole.tokens_per_page,
            "visible_tokens": int(whole.visible.sum()), "query_tokens": int(whole.num_tokens), "seed": whole.seed,
            "parallelism": parallelism, "l2": L2_NOTE}


def measure_decode(job, pkg, W, index, main):
    """One configuration of the static kind (a fixed batch stepped repeatedly): device-timed step, the dominant
    kernel's own time, and for the headline the end-to-end leg, the read probe and the CPU baseline."""
    from psi_dec_b200.distributed import KvRangeExchange
    args, torch = job.args, job.torch
    world, rank = job.world, job.rank
    base = workload(W, args, index)
    spec, scaling, parallelism, whole = spread(W, pkg, base, index, job, args)
    kernel_mode = {"auto": pkg.KERNEL_AUTO, "mma": pkg.KERNEL_MMA, "generic": pkg.KERNEL_GENERIC,
                   "mma_sync": pkg.KERNEL_MMA_SYNC, "mma_tma": pkg.KERNEL_MMA_TMA}[args.kernel]
    session = W.Session(spec, device=job.local_rank, kernel_mode=kernel_mode)
    # wait bound of seconds (about 100 ns per poll): a rank whose host is held up for a moment is not a failed step
    exchange = (KvRangeExchange(session, rank, world, mode=args.exchange, max_polls=20_000_000)
                if (world > 1 and index == 4) else None)
    step = exchange.step if exchange else session.step
    ctx = session.ctx
    alg = spec.algorithmic_bytes()
    steps = args.steps if main else min(args.steps, args.split_steps)
    every = exchange is not None

    for _ in range(max(args.warmup, 3)):
        if every:
            job.barrier()
        step()
    job.barrier()
    sampler = ClockSampler(job.local_rank) if (rank == 0 and main) else None
    launches_before = ctx.launch_count
    job.barrier()
    step_ms = job.timed(step, steps, session.stream, barrier_each=every)
    job.barrier()
    launches = ctx.launch_count - launches_before
    # The dominant kernel on its own clock: the same steps again with the library's per-launch event pairs switched
    # on (kept out of the pass above, where the extra events would sit inside the step time).
    ctx.enable_kernel_timing(True)
    job.timed(step, steps, session.stream, barrier_each=every)
    timing = {name: ctx.kernel_timing(cls) for name, cls in
              (("append", 0), ("attend_map", 1), ("attend_reduce", 2), ("combine", 3), ("attend_chunk", 5))}
    ctx.enable_kernel_timing(False)
    job.barrier()
    status = session.gqa.device_status()

    map_ms, map_n = timing["attend_map"]
    map_avg_ms = map_ms / max(map_n, 1)
    peak, peak_kind = measured_peak()
    achieved = alg["total"] / (map_avg_ms * 1e-3) / 1e9 if map_n else 0.0
    frac = achieved / peak

    e2e = None
    if main:
        e2e = measure_e2e(job, session, spec, exchange, steps)
    clocks = sampler.stop() if sampler else None

    total_ms = sum(step_ms)
    job_bytes, job_kv, job_tokens = job.reduce([alg["total"], alg["kv"], spec.num_tokens], "sum")
    if exchange:
        job_tokens = float(base.num_tokens)  # every rank works on the same query tokens
    (worst_total_ms, frac_max, status_max) = job.reduce([total_ms, frac, status], "max")
    (frac_min,) = job.reduce([frac], "min")

    record = None
    if rank == 0:
        ms_per_step = worst_total_ms / steps
        value = job_bytes / (ms_per_step * 1e-3) / 1e9
        stats = session.gqa.plan_stats()
        record = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": {pkg.BF16: "bf16", pkg.F16: "f16", pkg.F32: "f32"}[spec.dtype],
            "data": "synthetic", "config": config_block(whole, parallelism),
            "tokens_per_s": round(job_tokens / (ms_per_step * 1e-3), 1),
            "kv_gbs": round(job_kv / (ms_per_step * 1e-3) / 1e9, 1),
            "frac_of_nominal_8tbs_per_gpu": round(value / world / NOMINAL_HBM_GBS, 4),
            "roofline": {"bound": "hbm", "kernel": "attend_map (rank 0)", "achieved": round(achieved, 1), "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": round(frac, 4),
                         "frac_min_over_ranks": round(frac_min, 4), "frac_max_over_ranks": round(frac_max, 4),
                         "traffic": None, "algorithmic_bytes_per_launch": alg["total"],
                         "avg_launch_ms": round(map_avg_ms, 5), "launches": map_n},
            "kernel_ms_per_step": {name: round(ms / max(n, 1), 5) for name, (ms, n) in timing.items()},
            "plan_rank0": {"sequences": spec.num_seqs, "visible_tokens": int(spec.visible.sum()),
                           "kernel": "mma" if stats["kernel"] == 2 else "generic", "ctas": stats["ctas"],
                           "items": stats["items"], "reduce_units": stats["reduce_units"]},
            "gpu_launches": int(launches),
            "device_status": int(status_max),
            # rank 0's per-step distribution (the headline ms_per_step is the mean of the slowest rank)
            "ms_per_step_rank0": {"median": round(statistics.median(step_ms), 5), "min": round(min(step_ms), 5),
                                  "max": round(max(step_ms), 5)},
        }
        chunk_ms, chunk_n = timing["attend_chunk"]
        if chunk_n and chunk_ms > map_ms:
            # long query runs dominate the step: the chunk kernel is a contraction, bounded by the tensor pipe
            flops = spec.long_run_flops(16 // min(16, spec.num_q_heads // spec.num_kv_heads))
            tensor_peak, tensor_kind = measured_tensor_peak()
            chunk_avg_ms = chunk_ms / chunk_n
            tflops = flops / (chunk_avg_ms * 1e-3) / 1e12
            engine = "tcgen05" if stats["chunk_tcgen05_launches"] else "mma.sync"
            record["roofline"] = {"bound": "tensor", "kernel": f"attend_chunk ({engine}, rank 0)",
                                  "achieved": round(tflops, 1), "peak": tensor_peak, "peak_kind": tensor_kind,
                                  "unit": "TFLOP/s", "frac": round(tflops / tensor_peak, 4), "traffic": None,
                                  "flops_per_launch": flops, "avg_launch_ms": round(chunk_avg_ms, 5),
                                  "launches": chunk_n}
        elif stats["kernel"] == 2:
            traffic, how = recorded_traffic(base.name, alg["total"])
            record["roofline"]["traffic"] = traffic
            record["roofline"]["traffic_source"] = how
        if main:
            record["e2e"] = e2e
            record["clocks"] = clocks
            if world == 1 and record["roofline"]["bound"] == "hbm" and not args.no_read_probe:
                # the ceiling of a kernel that only reads HBM (4 GiB through 16-byte loads), beside the copy figure
                probe = ctx.read_bandwidth(4 << 30, 5)
                record["roofline"]["read_only_probe_gbs"] = round(probe, 1)
                record["roofline"]["frac_of_read_only_probe"] = round(achieved / probe, 4) if probe > 0 else None
            if world == 1 and not args.no_cpu_baseline:
                from oracle import harness
                tok_s, bytes_s, desc, threads = harness.time_oracle_sample(session, seconds_target=12.0)
                record["cpu_baseline"] = {"value": round(bytes_s / 1e9, 4), "unit": UNIT, "cores": threads,
                                          "kind": "port", "sample": desc, "tokens_per_s": round(tok_s, 2)}
    job.barrier()
    session.close()
    return record


def measure_e2e(job, session, spec, exchange, steps):
    """End to end through the C ABI with host buffers: plan, H2D of q/k/v, append, attend, D2H of out, all inside the
    timed region.  Two clocks: CUDA events around the call while the GPU is kept busy in front of it (a serving loop's
    view: the host-side planning overlaps the work queued before the step), and the host's wall clock around the call
    with the GPU idle at entry (the latency of one isolated call).  `prepare_us` is the host-side planning alone."""
    torch = job.torch
    rank = job.rank
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
            if rank == exchange.owner or exchange.mode == "nccl":
                oh.copy_(session.out, non_blocking=True)
            session.stream.synchronize()
        else:
            session.gqa.step_host(session.pages, session.table, spec.layer, *batch, kh, vh, qh, oh)

    every = exchange is not None
    for _ in range(3):
        if every:
            job.barrier()
        e2e_step()
    job.barrier()
    e2e_ms = job.timed(e2e_step, steps, session.stream, barrier_each=every)
    job.barrier()
    wall_us, prepare_us = [], []
    for _ in range(max(steps, 100) if not every else steps):
        job.flush.sum()
        if every:
            job.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e2e_step()
        wall_us.append((time.perf_counter() - t0) * 1e6)
    for _ in range(100):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        session.gqa.prepare(*batch)
        prepare_us.append((time.perf_counter() - t0) * 1e6)
    session.ctx.sync()
    job.barrier()
    alg = spec.algorithmic_bytes()
    h2d = kh.numel() * kh.element_size() * 2 * (1 if spec.do_append else 0) + qh.numel() * qh.element_size()
    d2h = oh.numel() * oh.element_size() if (exchange is None or rank == exchange.owner) else 0
    job_bytes, job_tokens, job_h2d, job_d2h = job.reduce([alg["total"], spec.num_tokens, h2d, d2h], "sum")
    if exchange:
        job_tokens = float(spec.num_tokens)
    worst_ms, worst_wall, worst_prepare = job.reduce([sum(e2e_ms), statistics.median(wall_us),
                                                      statistics.median(prepare_us)], "max")
    ms = worst_ms / steps
    return {"value": round(job_bytes / (ms * 1e-3) / 1e9, 1), "unit": UNIT, "ms_per_step": round(ms, 5),
            "tokens_per_s": round(job_tokens / (ms * 1e-3), 1),
            "h2d_bytes_per_step": int(job_h2d), "d2h_bytes_per_step": int(job_d2h),
            "clock": "CUDA events around the call, GPU busy in front of it (max over ranks of the mean)",
            "wall_us_per_call": round(worst_wall, 2),
            "wall_value": round(job_bytes / (worst_wall * 1e-6) / 1e9, 1),
            "wall_clock": "host perf_counter around the blocking call, GPU idle at entry (max over ranks of the median)",
            "prepare_us": round(worst_prepare, 2)}


def measure_churn(job, pkg, W, main):
    """The continuous-batching trace: `--churn-steps` steps of admit / append / finish over 256 request slots, sticky
    by slot over the ranks, with the page allocator, table resets and page reuse between steps.  Decode rows are
    judged against HBM bandwidth, the 512-token chunk rows against the tensor peak; a few sequences are checked against
    the CPU oracle inside the run."""
    import numpy as np
    args, torch = job.args, job.torch
    world, rank = job.world, job.rank
    scale = max(1, args.scale_down)
    trace = W.ChurnTrace(slots=max(world, 256 // scale), steps=args.churn_steps, world=world, hi=max(256, 131072 // scale),
                         chunk=max(16, 512 // min(scale, 8)))
    kernel_mode = {"auto": pkg.KERNEL_AUTO, "mma": pkg.KERNEL_MMA, "generic": pkg.KERNEL_GENERIC,
                   "mma_sync": pkg.KERNEL_MMA_SYNC, "mma_tma": pkg.KERNEL_MMA_TMA}[args.kernel]
    churn = W.ChurnSession(trace, rank=rank, device=job.local_rank, kernel_mode=kernel_mode)
    ctx = churn.ctx
    mine = churn.mine
    tokens_per_tile = max(1, 16 // min(16, trace.num_q_heads // trace.num_kv_heads))
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(trace.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(trace.steps)]
    table_s, prepare_s, parity = [], [], []
    check_steps = {trace.steps // 4, (3 * trace.steps) // 4} if not args.no_cpu_baseline else set()
    launches_before = ctx.launch_count
    ctx.enable_kernel_timing(True)
    job.barrier()
    wall0 = time.perf_counter()
    for t in range(trace.steps):
        a, b = churn.prepare_step(t)
        table_s.append(a)
        prepare_s.append(b)
        job.flush.sum()
        starts[t].record(churn.stream)
        churn.launch_step()
        ends[t].record(churn.stream)
        if t in check_steps and rank == 0:
            # sampled parity inside the run: the two shortest decode sequences and the shortest chunked one
            from oracle import harness
            churn.ctx.sync()
            ctx_len, q_len = trace.context[t][mine], trace.q_len[t][mine]
            order = np.argsort(ctx_len, kind="stable")
            picks = [int(i) for i in order if q_len[i] == 1][:2] + [int(i) for i in order if q_len[i] > 1][:1]
            for local in picks:
                parity.append(harness.churn_sequence_error(churn, t, local))
        churn.finish_step(t)
    torch.cuda.synchronize()
    wall_s = time.perf_counter() - wall0
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    map_ms, map_n = ctx.kernel_timing(1)
    chunk_ms, chunk_n = ctx.kernel_timing(5)
    append_ms, append_n = ctx.kernel_timing(0)
    ctx.enable_kernel_timing(False)
    launches = ctx.launch_count - launches_before
    status = churn.gqa.device_status()
    stats = churn.gqa.plan_stats()

    warm = min(3, trace.steps - 1)   # the first steps also pay first-use costs (kernel load, scratch growth)
    decode_bytes = flops = tokens = 0
    for t in range(warm, trace.steps):
        d, f, n = trace.step_bytes_flops(t, mine, tokens_per_tile=tokens_per_tile)
        decode_bytes, flops, tokens = decode_bytes + d, flops + f, tokens + n
    timed_ms = sum(step_ms[warm:])
    # kernel event pairs are summed over all steps; scale to the steady-state steps by launch count
    hbm_peak, hbm_kind = measured_peak()
    tensor_peak, tensor_kind = measured_tensor_peak()
    all_decode = sum(trace.step_bytes_flops(t, mine, tokens_per_tile=tokens_per_tile)[0] for t in range(trace.steps))
    all_flops = sum(trace.step_bytes_flops(t, mine, tokens_per_tile=tokens_per_tile)[1] for t in range(trace.steps))
    decode_gbs = all_decode / (map_ms * 1e-3) / 1e9 if map_ms > 0 else 0.0
    chunk_tflops = all_flops / (chunk_ms * 1e-3) / 1e12 if chunk_ms > 0 else 0.0
    shares = [trace.step_cost_share(t) for t in range(trace.steps)]

    job_tokens, job_bytes, job_flops = job.reduce([tokens, decode_bytes, flops], "sum")
    worst_ms, worst_table, worst_prepare, status_max, worst_wall = job.reduce(
        [timed_ms, statistics.median(table_s), statistics.median(prepare_s), status, wall_s], "max")
    decode_frac_min, chunk_frac_min = job.reduce([decode_gbs / hbm_peak, chunk_tflops / tensor_peak], "min")
    reused, = job.reduce([churn.reused_pages], "sum")
    record = None
    if rank == 0:
        n_steps = trace.steps - warm
        ms_per_step = worst_ms / n_steps
        max_abs = max((p[0] for p in parity), default=None)
        mean_abs = max((p[1] for p in parity), default=None)
        record = {
            "metric": "continuous_batching_churn_tokens_per_second", "value": round(job_tokens / (worst_ms * 1e-3), 1),
            "unit": "tokens/s", "n_gpus": world, "steps": n_steps, "warmup": warm, "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg5-churn" if scale == 1 else f"cfg5-churn/scaled-down-{scale}",
                       "slots": trace.slots, "trace_steps": trace.steps, "chunk_tokens": trace.chunk,
                       "chunk_fraction": 0.3, "finish_fraction": 0.1, "context": "Zipf(1.1) over [128, 131072]",
                       "tokens_per_page": churn.p, "page_ids_per_block": churn.ipb, "seed": trace.seed,
                       "parallelism": f"sticky by request slot (slot mod {world})", "l2": L2_NOTE},
            "tokens_per_s": round(job_tokens / (worst_ms * 1e-3), 1),
            "decode_rows": {"bound": "hbm", "kernel": "attend_map (rank 0)", "achieved": round(decode_gbs, 1),
                            "peak": hbm_peak, "peak_kind": hbm_kind, "unit": "GB/s",
                            "frac": round(decode_gbs / hbm_peak, 4), "frac_min_over_ranks": round(decode_frac_min, 4),
                            "ms_per_step": round(map_ms / max(map_n, 1), 5)},
            "chunk_rows": {"bound": "tensor", "kernel": "attend_chunk (%s, rank 0)" %
                           ("tcgen05" if stats["chunk_tcgen05_launches"] else "mma.sync"),
                           "achieved": round(chunk_tflops, 1), "peak": tensor_peak, "peak_kind": tensor_kind,
                           "unit": "TFLOP/s", "frac": round(chunk_tflops / tensor_peak, 4),
                           "frac_min_over_ranks": round(chunk_frac_min, 4),
                           "ms_per_step": round(chunk_ms / max(chunk_n, 1), 5)},
            "append_ms_per_step": round(append_ms / max(append_n, 1), 5),
            "job_decode_gbs": round(job_bytes / (worst_ms * 1e-3) / 1e9, 1),
            "job_chunk_tflops": round(job_flops / (worst_ms * 1e-3) / 1e12, 1),
            "host_us_per_step": {"table_updates": round(worst_table * 1e6, 1), "prepare": round(worst_prepare * 1e6, 1)},
            "wall_s_whole_trace": round(worst_wall, 3),
            "slowest_rank_cost_share": {"mean": round(float(np.mean(shares)), 3), "max": round(float(np.max(shares)), 3)},
            "pages_reused": int(reused), "arena_pages_rank0": churn.num_pages,
            "parity": {"sequences_checked": len(parity), "max_abs": max_abs, "mean_abs": mean_abs,
                       "ok": (all(p[0] <= 2e-2 and p[1] <= 2e-3 for p in parity) if parity else None)},
            "gpu_launches": int(launches), "device_status": int(status_max),
            "ms_per_step_rank0": {"median": round(statistics.median(step_ms[warm:]), 5),
                                  "min": round(min(step_ms[warm:]), 5), "max": round(max(step_ms[warm:]), 5)},
        }
        if main:
            record["vs_baseline"] = None
            record["roofline"] = dict(record["chunk_rows"], traffic=None)
    job.barrier()
    churn.close()
    e2e = measure_churn_e2e(job, W, trace, kernel_mode, warm, min(trace.steps, 50 if main else 16))
    if record is not None:
        record["e2e"] = e2e
    return record


def measure_churn_e2e(job, W, trace, kernel_mode, warm, steps):
    """The first `steps` steps of the same trace again on a fresh session, every step through `psi_gqa_step_host` with
    pinned host buffers: planning, q/k/v over the host link, append, attention and the output's way back inside the
    timed region (CUDA events around the blocking call, and the host's clock)."""
    torch = job.torch
    churn = W.ChurnSession(trace, rank=job.rank, device=job.local_rank, kernel_mode=kernel_mode)
    kh, vh, qh = churn.k.cpu().pin_memory(), churn.v.cpu().pin_memory(), churn.q.cpu().pin_memory()
    oh = torch.empty_like(qh).pin_memory()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    wall, tokens, h2d, d2h = [], [], [], []
    launches_before = churn.ctx.launch_count
    job.barrier()
    for t in range(steps):
        churn.prepare_step(t, plan=False)
        job.flush.sum()
        torch.cuda.synchronize()
        starts[t].record(churn.stream)
        t0 = time.perf_counter()
        churn.host_step(kh, vh, qh, oh)
        wall.append(time.perf_counter() - t0)
        ends[t].record(churn.stream)
        n = churn.tokens
        tokens.append(n)
        h2d.append(n * (qh[0].numel() + 2 * kh[0].numel()) * qh.element_size())
        d2h.append(n * oh[0].numel() * oh.element_size())
        churn.finish_step(t)
    torch.cuda.synchronize()
    ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    launches = churn.ctx.launch_count - launches_before
    status = churn.gqa.device_status()
    churn.close()
    warm = min(warm, steps - 1)
    n_steps = steps - warm
    job_tokens, job_h2d, job_d2h = job.reduce([sum(tokens[warm:]), sum(h2d[warm:]), sum(d2h[warm:])], "sum")
    worst_ms, worst_wall, status_max = job.reduce([sum(ms[warm:]), sum(wall[warm:]) * 1e3, status], "max")
    job.barrier()
    return {"value": round(job_tokens / (worst_ms * 1e-3), 1), "unit": "tokens/s", "steps": n_steps,
            "ms_per_step": round(worst_ms / n_steps, 4), "wall_ms_per_step": round(worst_wall / n_steps, 4),
            "h2d_bytes_per_step": int(job_h2d / n_steps), "d2h_bytes_per_step": int(job_d2h / n_steps),
            "launches_per_step_rank0": round(launches / steps, 1), "device_status": int(status_max),
            "clock": "CUDA events around the blocking psi_gqa_step_host call (max over ranks of the sum); "
                     "large steps run as groups of requests whose transfers and launches overlap"}


SPLIT_KEYS = ("metric", "value", "unit", "scaling", "steps", "ms_per_step", "tokens_per_s", "kv_gbs",
              "frac_of_nominal_8tbs_per_gpu", "config", "roofline", "kernel_ms_per_step", "gpu_launches", "device_status",
              "decode_rows", "chunk_rows", "host_us_per_step", "slowest_rank_cost_share", "pages_reused", "parity",
              "job_decode_gbs", "job_chunk_tflops", "wall_s_whole_trace", "e2e")


def bench_ours(args):
    import __graft_entry__ as entry
    pkg = entry.load_package()
    from psi_dec_b200 import workloads as W
    job = Job(args)
    if args.config == 5 and not args.static:
        line = measure_churn(job, pkg, W, main=True)
    else:
        line = measure_decode(job, pkg, W, args.config or 2, main=True)
    if args.config is None and args.shape is None and not args.no_splits:
        splits = {}
        if job.world > 1:
            # a driver-visible check that the partial exchange over NVLink is right: a scaled-down long-context case
            # through the same exchange, every step against the oracle's merge of per-rank oracle partials
            from oracle import harness
            ok, max_abs, mean_abs = harness.exchange_parity(job.rank, job.world, job.local_rank, mode=args.exchange)
            parity = {"kv_range_exchange_vs_oracle": ok, "max_abs": max_abs, "mean_abs": mean_abs,
                      "case": "long-context configuration scaled down 32x, 3 steps, queries change per step"}
        for name, index in (("cfg3-verify-sequence-sharded", 3), ("cfg4-long-context-kv-range-split", 4)):
            record = measure_decode(job, pkg, W, index, main=False)
            if record is not None:
                splits[name] = {k: record[k] for k in SPLIT_KEYS if k in record}
        record = measure_churn(job, pkg, W, main=False)
        if record is not None:
            splits["cfg5-churn-sticky-by-slot"] = {k: record[k] for k in SPLIT_KEYS if k in record}
        if line is not None:
            if job.world > 1:
                splits["cfg4-long-context-kv-range-split"]["parity"] = parity
            line["splits"] = splits
    if job.rank == 0:
        print(json.dumps(line), flush=True)
    job.close()


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

    index = args.config or 2
    base = workload(W, args, index)
    world = max(1, args.gpus)
    if world > 1 and index == 2 and args.shape is None:
        specs = [W.config(index, scale_down=args.scale_down, seed=base.seed + 100 * r) for r in range(world)]
        whole = W.Spec(base.name, base.dtype, base.num_q_heads, base.num_kv_heads, base.head_dim, base.tokens_per_page,
                       np.concatenate([s.context_lens for s in specs]), np.concatenate([s.q_len for s in specs]), base.seed)
        parallelism = f"sequence-sharded x{world}"
    else:
        whole = base
        parallelism = "one GPU" if world == 1 else (f"kv-range-split x{world} ({args.exchange} partial exchange)"
                                                    if index == 4 else f"sequence-sharded x{world}")
    order = np.argsort(whole.visible, kind="stable")
    budget = 400_000 * max(1, O.num_threads()) // 8  # visible tokens per step: a step of roughly a second
    chosen, total = [], 0
    for s in order:
        if chosen and total + int(whole.visible[s]) > budget:
            break
        chosen.append(int(s))
        total += int(whole.visible[s])
    sample = W.Spec(whole.name + "/sample", whole.dtype, whole.num_q_heads, whole.num_kv_heads, whole.head_dim,
                    whole.tokens_per_page, whole.context_lens[chosen], whole.q_len[chosen], whole.seed)
    rng = np.random.default_rng(whole.seed)
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
    desc = f"{len(chosen)} shortest of {whole.num_seqs} sequences ({total} visible tokens) per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_block(whole, parallelism),
        "tokens_per_s": round(sample.num_tokens / (ms_per_step * 1e-3), 2),
        "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                         "sample": desc},
        "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference algorithm; the reference's Rust + Metal path cannot build or run here",
    }
    print(json.dumps(line), flush=True)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--config", type=int, default=None,
                        help="run one benchmark configuration alone (default: configuration 2 as the headline plus "
                             "configurations 3, 4 and 5 under `splits`)")
    parser.add_argument("--no-splits", action="store_true", help="headline only")
    parser.add_argument("--split-steps", type=int, default=50, help="timed steps of each `splits` record (at most --steps)")
    parser.add_argument("--churn-steps", type=int, default=50, help="steps of the continuous-batching trace")
    parser.add_argument("--static", action="store_true",
                        help="with --config 5: one static step of the churn batch instead of the trace")
    parser.add_argument("--scale-down", type=int, default=1,
                        help="divide batch and context sizes (small cases for profiler captures; not a bench value)")
    parser.add_argument("--shape", default=None, metavar="HQ,HKV,D,PAGE,BATCH,CTX_LO,CTX_HI[,Q_LEN]",
                        help="one GPU only: a decode batch of another model profile instead of --config")
    parser.add_argument("--contexts", default=None, metavar="C1,C2,...",
                        help="with --shape HQ,HKV,D,PAGE: one sequence per listed context length")
    parser.add_argument("--dtype", choices=["bf16", "f16", "f32"], default="bf16", help="storage dtype of --contexts runs")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-read-probe", action="store_true", help="skip the read-only HBM bandwidth probe")
    parser.add_argument("--kernel", choices=["auto", "mma", "generic", "mma_sync", "mma_tma"], default="auto",
                        help="attention kernel: tensor-core kernels (default where supported), the CUDA-core kernel, or "
                             "mma_sync = tensor-core kernels with long query runs kept off the tcgen05 kernel, mma_tma = decode kernel fed by "
                             "TMA boxes instead of cp.async (both kept for A/B measurement)")
    parser.add_argument("--exchange", choices=["p2p", "p2p3", "nccl"], default="p2p",
                        help="partial exchange of the KV-range-split configuration 4: one launch per rank (p2p), the "
                             "same data path as three launches (p2p3), or an NCCL all-gather")
    parser.add_argument("--record-traffic", default=None, metavar="REPORT.ncu-rep",
                        help="no run: read an ncu report of the decode kernel and write profiles/attend_mma_dram_traffic.txt")
    parser.add_argument("--capture-command", default="ncu --set full --clock-control none -k regex:attend_mma -s 4 -c 2 -o "
                        "prof_attend_mma_cfg2 python bench.py --config 2 --steps 3 --warmup 3 --no-cpu-baseline "
                        "--no-read-probe --no-splits", help="with --record-traffic: the command that made the report")
    args = parser.parse_args()
    if args.record_traffic:
        record_traffic(args.record_traffic, {2: "cfg2-a3b-layer-decode", 3: "cfg3-27b-mtp-verify", 4: "cfg4-long-context"}[args.config or 2],
                       args.capture_command)
        return
    if args.impl == "reference":
        bench_reference(args)
    else:
        bench_ours(args)


if __name__ == "__main__":
    main()
