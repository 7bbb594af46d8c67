"""Seeded synthetic decode workloads with the shapes, sizes and value distributions of the benchmark configurations,
and a ``Session`` that lays one of them out on a GPU through the library's public objects.

No public dataset stands behind these configurations: lengths, block tables and values are drawn from seeded
generators (numpy PCG64 for integers, torch's Philox for values), and the seed is part of the spec.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

from . import binding as B

_ELEM_BYTES = {B.F32: 4, B.BF16: 2, B.F16: 2}


@dataclass
class Spec:
    name: str
    dtype: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    tokens_per_page: int
    context_lens: np.ndarray          # tokens already cached per sequence, before this step's append
    q_len: np.ndarray                 # query (= appended) tokens per sequence this step
    seed: int
    pool_factor: float = 1.25
    ids_per_block: int = 1
    num_layers: int = 1
    layer: int = 0
    scale: float = 0.0
    do_append: bool = True                # False: this step's K/V rows are already resident (KV-range shards)
    block_tables: list = field(default_factory=list)   # per sequence: physical page ids in logical order
    num_pages: int = 0

    def __post_init__(self):
        self.context_lens = np.asarray(self.context_lens, dtype=np.int64)
        self.q_len = np.broadcast_to(np.asarray(self.q_len, dtype=np.int64), self.context_lens.shape).copy()
        if self.scale == 0.0:
            self.scale = 1.0 / math.sqrt(self.head_dim)
        if not self.block_tables:
            self._draw_block_tables()

    # -- derived sizes ------------------------------------------------------------------------------------------------
    @property
    def elem_bytes(self) -> int:
        return _ELEM_BYTES[self.dtype]

    @property
    def page_bytes(self) -> int:
        return 2 * self.num_kv_heads * self.tokens_per_page * self.head_dim * self.elem_bytes

    @property
    def num_seqs(self) -> int:
        return len(self.context_lens)

    @property
    def num_tokens(self) -> int:
        return int(self.q_len.sum())

    @property
    def visible(self) -> np.ndarray:
        return self.context_lens + self.q_len

    def pages_per_seq(self) -> np.ndarray:
        return -(-self.visible // self.tokens_per_page)

    def _draw_block_tables(self):
        rng = np.random.default_rng(self.seed)
        pages = self.pages_per_seq()
        total = int(pages.sum())
        self.num_pages = max(int(math.ceil(total * self.pool_factor)), total, 1)
        pool = rng.permutation(self.num_pages).astype(np.uint32)
        start = 0
        for n in pages:
            self.block_tables.append(pool[start:start + int(n)].copy())
            start += int(n)

    # -- batch description in the reference's request-level form ---------------------------------------------------------
    def batch(self):
        """(req_slots, token_indices, cu_tokens) as contiguous uint32 arrays."""
        req_slots = np.arange(self.num_seqs, dtype=np.uint32)
        token_indices = self.context_lens.astype(np.uint32)
        cu = np.concatenate([[0], np.cumsum(self.q_len)]).astype(np.uint32)
        return req_slots, token_indices, cu

    def algorithmic_bytes(self) -> dict:
        """Bytes one step must move: every visible K/V byte once, q in, out out, appended rows in and out, and one
        table entry per visible page."""
        e = self.elem_bytes
        kv = int(self.visible.sum()) * 2 * self.num_kv_heads * self.head_dim * e
        t = self.num_tokens
        q_o = t * self.num_q_heads * self.head_dim * 2 * e
        app = 2 * t * 2 * self.num_kv_heads * self.head_dim * e
        table = int(self.pages_per_seq().sum()) * 4
        return {"kv": kv, "q_o": q_o, "append": app, "table": table, "total": kv + q_o + app + table}

    def long_run_flops(self, tokens_per_tile: int, min_tiles: int = 5) -> int:
        """Multiply-add work (2 flops each, Q K^T and P V) of the requests whose query run is long enough for the
        chunk kernel: query token j of a request sees its context plus the j + 1 tokens appended so far."""
        total = 0
        for ctx, n in zip(self.context_lens.tolist(), self.q_len.tolist()):
            if -(-n // tokens_per_tile) >= min_tiles:
                keys = n * ctx + n * (n + 1) // 2
                total += 4 * self.head_dim * self.num_q_heads * keys
        return total

    def shard(self, rank: int, world: int) -> "Spec":
        """Sequence shard ``rank`` of ``world``: sequences are dealt most-expensive-first to the rank with the least
        work so far, where a sequence costs its K/V bytes at HBM speed plus, for a long query run, its attention
        flops at tensor speed, so every rank carries a similar load.  Each rank owns its sequences' pages in an arena
        of its own."""
        kv_bytes = self.visible * (2 * self.num_kv_heads * self.head_dim * self.elem_bytes)
        tokens_per_tile = max(1, 16 // min(16, self.num_q_heads // self.num_kv_heads))
        long_run = -(-self.q_len // tokens_per_tile) >= 5
        keys = self.q_len * self.context_lens + self.q_len * (self.q_len + 1) // 2
        flops = np.where(long_run, 4 * self.head_dim * self.num_q_heads * keys, 0)
        cost = kv_bytes / 6.5e12 + flops / 1.2e15
        loads = np.zeros(world)
        owner = np.empty(self.num_seqs, dtype=np.int64)
        for seq in np.argsort(-cost, kind="stable"):
            owner[seq] = int(np.argmin(loads))
            loads[owner[seq]] += cost[seq]
        mine = np.flatnonzero(owner == rank)
        return Spec(name=f"{self.name}/shard{rank}of{world}", dtype=self.dtype, num_q_heads=self.num_q_heads,
                    num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, tokens_per_page=self.tokens_per_page,
                    context_lens=self.context_lens[mine], q_len=self.q_len[mine], seed=self.seed * 1000 + rank,
                    pool_factor=self.pool_factor, ids_per_block=self.ids_per_block, num_layers=self.num_layers,
                    layer=self.layer, scale=self.scale)

    def kv_range_shard(self, rank: int, world: int) -> "Spec":
        """KV-range shard for one very long context per sequence: rank j holds the j-th page-aligned slice of every
        sequence's context; the appended token lands on the last rank.  Lengths are in the rank's local coordinates."""
        p = self.tokens_per_page
        pages = -(-self.context_lens // p)
        lo = pages * rank // world * p
        hi = np.minimum(pages * (rank + 1) // world * p, self.context_lens)
        local = hi - lo
        last = rank == world - 1
        return Spec(name=f"{self.name}/kvrange{rank}of{world}", dtype=self.dtype, num_q_heads=self.num_q_heads,
                    num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, tokens_per_page=p,
                    context_lens=local if last else local - self.q_len, q_len=self.q_len,
                    seed=self.seed * 1000 + rank, pool_factor=self.pool_factor, scale=self.scale, do_append=bool(last))


def config(index: int, scale_down: int = 1, seed: int | None = None) -> Spec:
    """The five benchmark configurations; ``scale_down`` divides batch and context sizes for small test runs."""
    s = max(1, scale_down)
    if index == 1:
        return Spec("cfg1-cpu-scale", B.F16, 4, 1, 128, 16, [256], 1, seed or 1, pool_factor=64 / 17)
    if index == 2:
        rng = np.random.default_rng(seed or 2)
        ctx = rng.integers(1024 // s, 8192 // s + 1, size=max(1, 32 // s))
        return Spec("cfg2-a3b-layer-decode", B.BF16, 16, 2, 256, 16, ctx, 1, seed or 2)
    if index == 3:
        rng = np.random.default_rng(seed or 3)
        ctx = np.exp(rng.normal(math.log(8192 / s), 0.5, size=max(1, 128 // s)))
        ctx = np.clip(ctx, 4096 // s, 32768 // s).astype(np.int64)
        return Spec("cfg3-27b-mtp-verify", B.BF16, 24, 4, 256, 16, ctx, 2, seed or 3)
    if index == 4:
        return Spec("cfg4-long-context", B.BF16, 16, 2, 256, 16, [262144 // s] * 4, 1, seed or 4, pool_factor=1.0)
    if index == 5:
        rng = np.random.default_rng(seed or 5)
        n = max(1, 256 // s)
        lo, hi = 128, max(256, 131072 // s)
        support = np.arange(lo, hi + 1, dtype=np.float64)
        weights = support ** -1.1
        cdf = np.cumsum(weights) / weights.sum()
        ctx = lo + np.searchsorted(cdf, rng.random(n))
        q_len = np.where(rng.random(n) < 0.3, 512 // min(s, 8), 1)
        return Spec("cfg5-churn", B.BF16, 16, 2, 256, 16, ctx, q_len, seed or 5)
    raise ValueError(f"unknown configuration {index}")


def custom(num_q_heads: int, num_kv_heads: int, head_dim: int, tokens_per_page: int, batch: int, ctx_lo: int,
           ctx_hi: int, q_len: int = 1, seed: int = 11) -> Spec:
    """A decode batch of another model profile: contexts uniform in [ctx_lo, ctx_hi], ``q_len`` tokens per sequence."""
    rng = np.random.default_rng(seed)
    ctx = rng.integers(ctx_lo, ctx_hi + 1, size=batch)
    name = f"custom-hq{num_q_heads}-hkv{num_kv_heads}-d{head_dim}-p{tokens_per_page}-b{batch}-ctx{ctx_lo}-{ctx_hi}-q{q_len}"
    return Spec(name, B.BF16, num_q_heads, num_kv_heads, head_dim, tokens_per_page, ctx, q_len, seed)


def explicit(num_q_heads: int, num_kv_heads: int, head_dim: int, tokens_per_page: int, contexts, q_len: int = 1,
             seed: int = 11, dtype: int = B.BF16) -> Spec:
    """A decode batch with the given context lengths, one sequence each (the reference's own bench fixtures are of
    this kind: crates/inference-backend-metal/benches/gqa/split_kv.rs:19-54)."""
    name = (f"explicit-hq{num_q_heads}-hkv{num_kv_heads}-d{head_dim}-p{tokens_per_page}-ctx"
            + "+".join(str(int(c)) for c in contexts) + f"-q{q_len}")
    return Spec(name, dtype, num_q_heads, num_kv_heads, head_dim, tokens_per_page, list(contexts), q_len, seed)


class Session:
    """One workload resident on one GPU: arena (random K/V everywhere), block tables, GQA component, q/k/v/out."""

    def __init__(self, spec: Spec, device: int = 0, plan_mode: int = B.PLAN_BALANCED, kernel_mode: int = B.KERNEL_AUTO,
                 max_ctas: int = 0, own_arena: bool = False, fill: str = "normal"):
        import torch
        self.torch = torch
        self.spec = spec
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.stream = torch.cuda.current_stream(self.device)
        self.ctx = B.Context(device, stream=self.stream.cuda_stream)
        tdtype = {B.F32: torch.float32, B.BF16: torch.bfloat16, B.F16: torch.float16}[spec.dtype]
        self.tdtype = tdtype
        page_elems = spec.page_bytes // spec.elem_bytes
        gen = torch.Generator(device=self.device)
        gen.manual_seed(spec.seed)
        if own_arena:
            self.pages = B.PageArena(self.ctx, spec.num_pages, spec.page_bytes)
            self.arena = None
        else:
            self.arena = torch.empty((spec.num_pages, page_elems), dtype=tdtype, device=self.device)
            chunk = max(1, (256 << 20) // (page_elems * 4))
            for start in range(0, spec.num_pages, chunk):
                part = self.arena[start:start + chunk]
                if fill == "normal":
                    part.copy_(torch.randn(part.shape, generator=gen, device=self.device, dtype=torch.float32))
                else:
                    part.zero_()
            self.pages = B.PageArena(self.ctx, spec.num_pages, spec.page_bytes, device_ptr=self.arena)
        pages_per_block = spec.ids_per_block
        max_pages = int(spec.pages_per_seq().max())
        self.layout = B.GQAPageTableLayout(spec.num_seqs, spec.num_layers, -(-max_pages // pages_per_block),
                                           pages_per_block)
        self.table = B.GQARequestPageTable(self.ctx, self.layout)
        for slot, ids in enumerate(spec.block_tables):
            self.table.write_row(slot, spec.layer, ids)
        cfg = B.GQAConfig(spec.num_q_heads, spec.num_kv_heads, spec.head_dim, spec.scale, spec.page_bytes, spec.dtype,
                          self.layout, max(spec.num_tokens, 1), plan_mode, kernel_mode, max_ctas)
        self.gqa = B.GQA(self.ctx, cfg)
        t = spec.num_tokens
        self.q = torch.randn((t, spec.num_q_heads, spec.head_dim), generator=gen, device=self.device,
                             dtype=torch.float32).to(tdtype)
        self.k = torch.randn((t, spec.num_kv_heads, spec.head_dim), generator=gen, device=self.device,
                             dtype=torch.float32).to(tdtype)
        self.v = torch.randn((t, spec.num_kv_heads, spec.head_dim), generator=gen, device=self.device,
                             dtype=torch.float32).to(tdtype)
        self.out = torch.zeros_like(self.q)
        self.shape = self.gqa.prepare(*spec.batch())

    def append(self):
        self.gqa.kv_page_write(self.pages, self.table, self.spec.layer, self.k, self.v)

    def attend(self):
        self.gqa.attend(self.pages, self.table, self.spec.layer, self.q, self.out)

    def step(self):
        """One pass of the hot path with inputs resident in HBM: append this step's K/V and attend, as one launch."""
        if self.spec.do_append:
            self.gqa.append_attend(self.pages, self.table, self.spec.layer, self.k, self.v, self.q, self.out)
        else:
            self.attend()

    def step_unfused(self):
        """The same step as the reference records it: KV page write, then attention, in stream order."""
        if self.spec.do_append:
            self.append()
        self.attend()

    def close(self):
        self.ctx.sync()
        self.gqa.close()
        self.table.close()
        self.pages.close()
        self.ctx.close()


# ---------------------------------------------------------------------------------------------------------------------
# Continuous-batching churn (the fifth benchmark configuration)
# ---------------------------------------------------------------------------------------------------------------------
def _zipf_contexts(rng, n: int, lo: int, hi: int, s: float = 1.1) -> np.ndarray:
    """Inverse-CDF samples of a Zipf(s) law over the integers [lo, hi]."""
    support = np.arange(lo, hi + 1, dtype=np.float64)
    weights = support ** -s
    cdf = np.cumsum(weights) / weights.sum()
    return lo + np.searchsorted(cdf, rng.random(n))


class ChurnTrace:
    """A seeded admit / finish / append trace over a fixed set of request slots, host only.

    Per step: ``chunk_fraction`` of the live sequences append a ``chunk``-token block (causal within the block plus
    the paged history), the others one decode token; then ``finish_fraction`` of the sequences finish and new ones
    (context drawn from Zipf(1.1) over [lo, hi]) move into the slots they leave.  Slot ``s`` belongs to rank
    ``s % world`` for good (its pages live in that rank's arena).  The one freedom a sticky assignment leaves is which
    freed slot a newly admitted sequence takes: the most expensive newcomer goes to the freed slot of the rank that
    carries the least work, under the same cost model as ``Spec.shard``.
    """

    def __init__(self, slots: int = 256, steps: int = 50, seed: int = 5, world: int = 1, chunk: int = 512,
                 lo: int = 128, hi: int = 131072, chunk_fraction: float = 0.3, finish_fraction: float = 0.1,
                 num_q_heads: int = 16, num_kv_heads: int = 2, head_dim: int = 256, elem_bytes: int = 2):
        rng = np.random.default_rng(seed)
        self.slots, self.steps, self.seed, self.world, self.chunk = slots, steps, seed, world, chunk
        self.num_q_heads, self.num_kv_heads, self.head_dim, self.elem_bytes = num_q_heads, num_kv_heads, head_dim, elem_bytes
        self.context = np.zeros((steps, slots), dtype=np.int64)   # tokens cached before the step's append
        self.q_len = np.zeros((steps, slots), dtype=np.int64)
        self.finished = []                                        # per step: slots that finish after it
        self.admitted = []                                        # per step: {slot: context of the newcomer}
        ctx = _zipf_contexts(rng, slots, lo, hi)
        n_finish = max(1, int(round(finish_fraction * slots))) if finish_fraction > 0 else 0
        for t in range(steps):
            # the chunked sequences are drawn rank by rank, so every rank carries its share of them
            q = np.ones(slots, dtype=np.int64)
            for r in range(world):
                own = np.arange(r, slots, world)
                q[rng.choice(own, size=int(round(chunk_fraction * len(own))), replace=False)] = chunk
            self.context[t], self.q_len[t] = ctx, q
            ctx = ctx + q
            leaving = np.sort(rng.choice(slots, size=n_finish, replace=False)) if n_finish else np.zeros(0, dtype=np.int64)
            newcomers = np.sort(_zipf_contexts(rng, len(leaving), lo, hi))[::-1]
            loads = np.zeros(world)
            staying = np.ones(slots, dtype=bool)
            staying[leaving] = False
            cost = self._cost(ctx, np.full(slots, 1 + (chunk - 1) * chunk_fraction))
            for r in range(world):
                loads[r] = cost[staying & (np.arange(slots) % world == r)].sum()
            free = list(int(s) for s in leaving)
            placed = {}
            for c in newcomers:
                slot = min(free, key=lambda s: (loads[s % world], s))
                free.remove(slot)
                placed[slot] = int(c)
                loads[slot % world] += float(self._cost(np.array([c]), np.array([1 + (chunk - 1) * chunk_fraction]))[0])
                ctx[slot] = c
            self.finished.append([int(s) for s in leaving])
            self.admitted.append(placed)

    def _cost(self, context, q_len):
        """Seconds a sequence costs per step: its K/V bytes at HBM speed plus, for a chunk, its flops at tensor speed."""
        kv_bytes = (context + q_len) * (2 * self.num_kv_heads * self.head_dim * self.elem_bytes)
        flops = 4.0 * self.head_dim * self.num_q_heads * (q_len * context + q_len * (q_len + 1) / 2) * (q_len > 1)
        return kv_bytes / 6.5e12 + flops / 1.2e15

    def rank_slots(self, rank: int) -> np.ndarray:
        return np.arange(rank, self.slots, self.world)

    def max_context(self) -> int:
        return int((self.context + self.q_len).max())

    def step_cost_share(self, t: int) -> float:
        """Slowest rank's modelled step cost over the mean (1.0 = perfectly balanced)."""
        cost = self._cost(self.context[t], self.q_len[t])
        per_rank = np.array([cost[self.rank_slots(r)].sum() for r in range(self.world)])
        return float(per_rank.max() / per_rank.mean())

    def step_bytes_flops(self, t: int, slots: np.ndarray, chunk_tiles_min: int = 5, tokens_per_tile: int = 2):
        """(decode-row algorithmic bytes, chunk-row flops, query tokens) of step ``t`` over ``slots``: decode rows are
        the requests the decode kernel takes, chunk rows the long query runs the chunk kernel takes."""
        ctx, q = self.context[t][slots], self.q_len[t][slots]
        is_chunk = -(-q // tokens_per_tile) >= chunk_tiles_min
        e = self.elem_bytes
        row = 2 * self.num_kv_heads * self.head_dim * e
        dec = ~is_chunk
        decode_bytes = int(((ctx + q)[dec]).sum()) * row + int(q[dec].sum()) * (self.num_q_heads * self.head_dim * 2 * e + 2 * row)
        keys = q * ctx + q * (q + 1) // 2
        flops = int(4 * self.head_dim * self.num_q_heads * keys[is_chunk].sum())
        return decode_bytes, flops, int(q.sum())


class ChurnSession:
    """One rank's share of a :class:`ChurnTrace` on one GPU, driven through the library's cache-ownership objects:
    page IDs come from ``U32IDAllocator`` (freed IDs first), a finished slot's table rows are zeroed with
    ``reset_req_slots``, its pages go back to the allocator and are handed out again without being cleared, and the
    table is two-level (``ids_per_block`` page IDs per logical block, written block by block as the reference's
    block-table deltas are)."""

    def __init__(self, trace: ChurnTrace, rank: int = 0, device: int = 0, tokens_per_page: int = 16,
                 ids_per_block: int = 128, kernel_mode: int = B.KERNEL_AUTO, dtype: int = B.BF16):
        import torch
        self.torch, self.trace, self.rank = torch, trace, rank
        self.p, self.ipb = tokens_per_page, ids_per_block
        self.mine = trace.rank_slots(rank)                      # global slot ids; local slot i = self.mine[i]
        self.local_of = {int(s): i for i, s in enumerate(self.mine)}
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.stream = torch.cuda.current_stream(self.device)
        self.ctx = B.Context(device, stream=self.stream.cuda_stream)
        self.dtype = dtype
        self.tdtype = {B.BF16: torch.bfloat16, B.F16: torch.float16}[dtype]
        hq, hkv, d = trace.num_q_heads, trace.num_kv_heads, trace.head_dim
        self.page_bytes = 2 * hkv * tokens_per_page * d * trace.elem_bytes
        # the arena holds the largest number of pages this rank's slots ever own at once, plus one step of slack
        pages_needed = -(-(trace.context + trace.q_len)[:, self.mine] // tokens_per_page)
        self.num_pages = int(pages_needed.sum(axis=1).max()) + len(self.mine) * (-(-trace.chunk // tokens_per_page) + 1)
        page_elems = self.page_bytes // trace.elem_bytes
        gen = torch.Generator(device=self.device)
        gen.manual_seed(trace.seed * 1000 + rank)
        self.arena = torch.empty((self.num_pages, page_elems), dtype=self.tdtype, device=self.device)
        step = max(1, (256 << 20) // (page_elems * 4))
        for start in range(0, self.num_pages, step):
            part = self.arena[start:start + step]
            part.copy_(torch.randn(part.shape, generator=gen, device=self.device, dtype=torch.float32))
        self.pages = B.PageArena(self.ctx, self.num_pages, self.page_bytes, device_ptr=self.arena)
        blocks = -(-(-(-trace.max_context() // tokens_per_page)) // ids_per_block)
        self.layout = B.GQAPageTableLayout(len(self.mine), 1, blocks, ids_per_block)
        self.table = B.GQARequestPageTable(self.ctx, self.layout)
        self.table.set_page_bound(self.num_pages)
        self.allocator = B.U32IDAllocator(self.num_pages)
        self.page_ids = [[] for _ in self.mine]                  # per local slot: physical pages in logical order
        self.max_tokens = int(trace.q_len[:, self.mine].sum(axis=1).max())
        cfg = B.GQAConfig(hq, hkv, d, 1.0 / math.sqrt(d), self.page_bytes, dtype, self.layout, self.max_tokens,
                          B.PLAN_BALANCED, kernel_mode, 0)
        self.gqa = B.GQA(self.ctx, cfg)
        self.q = torch.randn((self.max_tokens, hq, d), generator=gen, device=self.device, dtype=torch.float32).to(self.tdtype)
        self.k = torch.randn((self.max_tokens, hkv, d), generator=gen, device=self.device, dtype=torch.float32).to(self.tdtype)
        self.v = torch.randn((self.max_tokens, hkv, d), generator=gen, device=self.device, dtype=torch.float32).to(self.tdtype)
        self.out = torch.zeros_like(self.q)
        self.reused_pages = 0
        self._ever_freed = np.zeros(self.num_pages, dtype=bool)
        for i in range(len(self.mine)):
            self._grow(i, int(trace.context[0][self.mine[i]]))

    def _grow(self, local: int, tokens: int):
        """Pages for the first ``tokens`` tokens of local slot ``local``: new IDs from the allocator, and the logical
        blocks they fall into written to the table."""
        have = len(self.page_ids[local])
        need = -(-tokens // self.p)
        if need <= have:
            return
        fresh = self.allocator.alloc_many(need - have)
        self.reused_pages += int(self._ever_freed[fresh].sum())
        self.page_ids[local].extend(fresh)
        ids = self.page_ids[local]
        for block in range(have // self.ipb, -(-need // self.ipb)):
            entry = ids[block * self.ipb:(block + 1) * self.ipb]
            self.table.write_page_ids(local, 0, block, entry + [0] * (self.ipb - len(entry)))

    def prepare_step(self, t: int, plan: bool = True):
        """Host work in front of step ``t``: admissions of the previous step's leavers are already done; pages for this
        step's appended tokens are allocated and the plan is uploaded (``plan=False``: left to ``host_step``).
        Returns (table_seconds, prepare_seconds)."""
        import time
        tr = self.trace
        t0 = time.perf_counter()
        for i, s in enumerate(self.mine):
            self._grow(i, int(tr.context[t][s] + tr.q_len[t][s]))
        t1 = time.perf_counter()
        q_len = tr.q_len[t][self.mine]
        cu = np.concatenate([[0], np.cumsum(q_len)]).astype(np.uint32)
        self.tokens = int(cu[-1])
        self.batch = (np.arange(len(self.mine), dtype=np.uint32), tr.context[t][self.mine].astype(np.uint32), cu)
        if plan:
            self.gqa.prepare(*self.batch)
        return t1 - t0, time.perf_counter() - t1

    def launch_step(self):
        """The step on the device: this step's K/V rows into their pages and attention over everything visible."""
        n = self.tokens
        self.gqa.append_attend(self.pages, self.table, 0, self.k[:n], self.v[:n], self.q[:n], self.out[:n])

    def host_step(self, k_host, v_host, q_host, out_host):
        """The same step from host buffers through ``psi_gqa_step_host``: plan, transfers in, append, attention and the
        result's way back in one blocking call (large steps from pinned buffers are cut into groups of requests whose
        transfers and launches overlap)."""
        n = self.tokens
        self.gqa.step_host(self.pages, self.table, 0, *self.batch, k_host[:n], v_host[:n], q_host[:n], out_host[:n])

    def finish_step(self, t: int):
        """After step ``t``: the leavers' pages go back to the allocator, their table rows are zeroed, and the
        newcomers' contexts get pages (possibly the very ones just freed, contents untouched)."""
        tr = self.trace
        leaving = [self.local_of[s] for s in tr.finished[t] if s in self.local_of]
        for local in leaving:
            ids = self.page_ids[local]
            self.allocator.free_many(ids)
            self._ever_freed[ids] = True
            self.page_ids[local] = []
        if leaving:
            self.table.reset_req_slots(leaving)
        for s, context in tr.admitted[t].items():
            if s in self.local_of:
                self._grow(self.local_of[s], context)

    def sequence_view(self, t: int, local: int):
        """What a checker needs for one sequence of step ``t`` (after ``launch_step``): its physical pages in logical
        order, its context length, its query length and the flat row range of its tokens."""
        q_len = self.trace.q_len[t][self.mine]
        begin = int(q_len[:local].sum())
        n = int(q_len[local])
        return dict(pages=list(self.page_ids[local]), context=int(self.trace.context[t][self.mine[local]]), q_len=n,
                    rows=(begin, begin + n))

    def close(self):
        self.ctx.sync()
        self.gqa.close()
        self.table.close()
        self.pages.close()
        self.ctx.close()
