"""Checker-side helpers around the CPU oracle: copy a GPU session's problem to the host, run the oracle on it, compare.

Test infrastructure, like everything under ``oracle/``: used by ``tests/``, by ``__graft_entry__.smoke()`` and by
``bench.py``'s CPU-baseline and parity legs as the checker of GPU results, never as the thing that is measured or
shipped.  Nothing in the product package imports this module.
"""
from __future__ import annotations

import time

import numpy as np

from oracle import psi_oracle as O

# Attention tolerance for 16-bit outputs against the f32 oracle (the reference's own bf16 bound is 2e-2 max-abs:
# crates/inference-backend-metal/src/components/gqa_split_kv_tiled_q_test.rs:131).
MAX_ABS_16BIT = 2e-2
MEAN_ABS_16BIT = 2e-3
MAX_ABS_F32 = 2e-5  # crates/inference-backend-metal/src/components/gqa_split_kv_single_q_test.rs:76


def to_numpy_bits(tensor):
    """Device tensor -> host numpy array of the storage bits (u16 for 16-bit floats, f32 otherwise)."""
    import torch
    t = tensor.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def host_problem(session, seq_ids=None):
    """Copy what the oracle needs for the chosen sequences to the host: a compact arena holding only their pages, a
    renumbered block table, their q rows and per-token metadata."""
    import torch
    spec = session.spec
    seq_ids = list(range(spec.num_seqs)) if seq_ids is None else list(seq_ids)
    pages_per_seq = spec.pages_per_seq()
    wanted, rows = [], []
    for s in seq_ids:
        ids = spec.block_tables[s][: int(pages_per_seq[s])].astype(np.int64)
        rows.append(np.arange(len(wanted), len(wanted) + len(ids), dtype=np.uint32))
        wanted.extend(ids.tolist())
    index = torch.as_tensor(np.asarray(wanted, dtype=np.int64), device=session.device)
    arena = to_numpy_bits(session.arena.index_select(0, index)).reshape(-1)
    max_pages = max(len(r) for r in rows)
    table = np.zeros((len(seq_ids), 1, max_pages, 1), dtype=np.uint32)
    for i, r in enumerate(rows):
        table[i, 0, : len(r), 0] = r
    layout = O.Layout(len(seq_ids), 1, max_pages, 1)
    cu = np.concatenate([[0], np.cumsum(spec.q_len)])
    tok_rows, req_slots, positions = [], [], []
    for i, s in enumerate(seq_ids):
        for j in range(int(spec.q_len[s])):
            tok_rows.append(int(cu[s]) + j)
            req_slots.append(i)
            positions.append(int(spec.context_lens[s]) + j)
    return dict(arena=arena, table=table.reshape(-1), layout=layout, tok_rows=np.asarray(tok_rows),
                req_slots=req_slots, positions=positions)


def oracle_attention(session, seq_ids=None, problem=None):
    """f32 oracle output [n_rows][Hq][D] for the chosen sequences' query tokens, plus the flat rows they occupy."""
    spec = session.spec
    prob = host_problem(session, seq_ids) if problem is None else problem
    q = to_numpy_bits(session.q)[prob["tok_rows"]]
    out = O.paged_attention(prob["arena"], spec.dtype, q, prob["req_slots"], prob["positions"], prob["table"], 0,
                            prob["layout"], spec.num_q_heads, spec.num_kv_heads, spec.head_dim, spec.page_bytes,
                            spec.scale)
    return out, prob["tok_rows"]


def compare_attention(session, seq_ids=None):
    """(max_abs, mean_abs) between the session's GPU output and the oracle on the chosen sequences."""
    expected, rows = oracle_attention(session, seq_ids)
    actual = O.decode(to_numpy_bits(session.out)[rows], session.spec.dtype)
    diff = np.abs(actual.astype(np.float64) - expected.astype(np.float64))
    return float(diff.max()), float(diff.mean())


def assert_attention_close(session, seq_ids=None):
    max_abs, mean_abs = compare_attention(session, seq_ids)
    if session.spec.dtype == O.F32:
        assert max_abs <= MAX_ABS_F32, f"max_abs={max_abs}"
    else:
        assert max_abs <= MAX_ABS_16BIT and mean_abs <= MEAN_ABS_16BIT, f"max_abs={max_abs} mean_abs={mean_abs}"
    return max_abs, mean_abs


def expected_arena_after_append(session, arena_before_bits):
    """Oracle append applied to a host copy of the whole arena (bit-exact expectation)."""
    spec = session.spec
    pages = np.array(arena_before_bits, copy=True).reshape(-1)
    table = np.zeros((spec.num_seqs, spec.num_layers, session.layout.num_blocks, session.layout.num_page_ids_per_block),
                     dtype=np.uint32)
    for s, ids in enumerate(spec.block_tables):
        table[s, spec.layer].reshape(-1)[: len(ids)] = ids
    layout = O.Layout(spec.num_seqs, spec.num_layers, session.layout.num_blocks, session.layout.num_page_ids_per_block)
    req_slots, positions = [], []
    for s in range(spec.num_seqs):
        for j in range(int(spec.q_len[s])):
            req_slots.append(s)
            positions.append(int(spec.context_lens[s]) + j)
    O.kv_page_write(pages, to_numpy_bits(session.k), to_numpy_bits(session.v), req_slots, positions, table.reshape(-1),
                    len(req_slots), spec.layer, layout, spec.num_kv_heads, spec.head_dim, spec.page_bytes)
    return pages


def time_oracle_sample(session, seconds_target=15.0, max_seqs=None):
    """Time the oracle on a bounded sample of the session's workload (shortest sequences first until the estimated
    cost reaches the target).  Returns (tokens_per_second, kv_bytes_per_second, description, threads)."""
    spec = session.spec
    order = np.argsort(spec.visible, kind="stable")
    # calibrate on the shortest sequence, then grow the sample
    t0 = time.perf_counter()
    oracle_attention(session, [int(order[0])])
    per_row_token = (time.perf_counter() - t0) / max(1, int(spec.visible[order[0]]) * int(spec.q_len[order[0]]))
    chosen, cost = [], 0.0
    for s in order:
        c = per_row_token * float(spec.visible[s]) * float(spec.q_len[s])
        if chosen and cost + c > seconds_target:
            break
        chosen.append(int(s))
        cost += c
        if max_seqs and len(chosen) >= max_seqs:
            break
    problem = host_problem(session, chosen)
    t0 = time.perf_counter()
    oracle_attention(session, chosen, problem=problem)
    elapsed = time.perf_counter() - t0
    tokens = int(spec.q_len[chosen].sum())
    kv_bytes = int(spec.visible[chosen].sum()) * 2 * spec.num_kv_heads * spec.head_dim * spec.elem_bytes
    desc = f"{len(chosen)} shortest of {spec.num_seqs} sequences ({int(spec.visible[chosen].sum())} visible tokens)"
    return tokens / elapsed, kv_bytes / elapsed, desc, O.num_threads()


_GOLDEN = None


def golden(name):
    """A stored expectation from tests/golden/attention_vectors.npz (see tests/golden/make_fixtures.py)."""
    global _GOLDEN
    if _GOLDEN is None:
        from pathlib import Path
        _GOLDEN = np.load(Path(__file__).resolve().parent.parent / "tests" / "golden" / "attention_vectors.npz")
    return _GOLDEN[name]


def smoke_check():
    """Configuration 1 (batch 1, 4/1 heads, D128, fp16, 256+1 tokens in 16-token pages) on cuda:0: append one token,
    attend over 257, compare page contents bit-exactly and the output within tolerance against the CPU oracle."""
    from psi_dec_b200 import workloads as W
    s = W.Session(W.config(1))
    before = to_numpy_bits(s.arena)
    s.step()
    s.ctx.sync()
    expected = expected_arena_after_append(s, before)
    assert np.array_equal(to_numpy_bits(s.arena).reshape(-1), expected), "append differs from the oracle"
    max_abs, mean_abs = assert_attention_close(s)
    stats = s.gqa.plan_stats()
    launches = s.ctx.launch_count
    s.close()
    print(f"smoke ok: max_abs={max_abs:.3e} mean_abs={mean_abs:.3e} plan={stats} launches={launches}")


def merged_oracle_partials(parts, num_tokens, num_q_heads, head_dim):
    """The oracle's merge (reference reduce algebra) of per-rank oracle partials ``[(o, m, l), ...]``."""
    expected = np.zeros((num_tokens, num_q_heads, head_dim), dtype=np.float32)
    for i in range(num_tokens):
        for h in range(num_q_heads):
            expected[i, h] = O.merge_partials(np.stack([p[0][i, h] for p in parts]), [p[1][i, h] for p in parts],
                                              [p[2][i, h] for p in parts])
    return expected


def oracle_partial(session):
    """(o, m, l) of the oracle over the session's own arena and tables (one rank's slice of a KV range)."""
    spec = session.spec
    prob = host_problem(session)
    q = to_numpy_bits(session.q)[prob["tok_rows"]]
    return O.paged_attention(prob["arena"], spec.dtype, q, prob["req_slots"], prob["positions"], prob["table"], 0,
                             prob["layout"], spec.num_q_heads, spec.num_kv_heads, spec.head_dim, spec.page_bytes,
                             spec.scale, want_stats=True)


def exchange_parity(rank, world, local_rank, mode="p2p", scale_down=32, steps=3):
    """A scaled-down long-context case split by KV range over the ranks of the default process group, run through the
    partial exchange for a few steps with queries that change per step, each step's merged output compared with the
    oracle's merge of per-rank oracle partials.  Returns (ok, max_abs, mean_abs), meaningful on the owner."""
    import torch
    import torch.distributed as dist
    from psi_dec_b200 import workloads as W
    from psi_dec_b200.distributed import KvRangeExchange
    spec = W.config(4, scale_down=scale_down).kv_range_shard(rank, world)
    s = W.Session(spec, device=local_rank)
    ex = KvRangeExchange(s, rank, world, mode=mode, max_polls=20_000_000)
    worst_max, worst_mean, ok = 0.0, 0.0, True
    for step in range(steps):
        gen = torch.Generator(device=s.device)
        gen.manual_seed(4321 + step)
        s.q.copy_(torch.randn(s.q.shape, generator=gen, device=s.device, dtype=torch.float32))
        ex.step()
        s.ctx.sync()
        ok = ok and s.gqa.device_status() == 0
        gathered = [None] * world
        dist.all_gather_object(gathered, oracle_partial(s))
        if rank == ex.owner:
            expected = merged_oracle_partials(gathered, spec.num_tokens, spec.num_q_heads, spec.head_dim)
            diff = np.abs(O.decode(to_numpy_bits(s.out), spec.dtype) - expected)
            worst_max, worst_mean = max(worst_max, float(diff.max())), max(worst_mean, float(diff.mean()))
    ok = ok and worst_max <= MAX_ABS_16BIT and worst_mean <= MEAN_ABS_16BIT
    result = torch.tensor([1.0 if ok else 0.0, worst_max, worst_mean], dtype=torch.float64, device=s.device)
    dist.broadcast(result, src=ex.owner)
    dist.barrier()
    s.close()
    ok_all, worst_max, worst_mean = result.tolist()
    return bool(ok_all), worst_max, worst_mean


def churn_sequence_error(churn, t, local):
    """(max_abs, mean_abs) of one sequence of a churn step against the oracle: its pages are gathered to the host in
    logical order (a compact arena of its own) and the oracle runs over them with the step's query rows."""
    import torch
    view = churn.sequence_view(t, local)
    tr = churn.trace
    visible = view["context"] + view["q_len"]
    ids = view["pages"][: -(-visible // churn.p)]
    index = torch.as_tensor(np.asarray(ids, dtype=np.int64), device=churn.device)
    arena = to_numpy_bits(churn.arena.index_select(0, index)).reshape(-1)
    table = np.arange(len(ids), dtype=np.uint32)
    layout = O.Layout(1, 1, len(ids), 1)
    begin, end = view["rows"]
    q = to_numpy_bits(churn.q[begin:end])
    positions = [view["context"] + j for j in range(view["q_len"])]
    expected = O.paged_attention(arena, churn.dtype, q, [0] * view["q_len"], positions, table, 0, layout,
                                 tr.num_q_heads, tr.num_kv_heads, tr.head_dim, churn.page_bytes,
                                 1.0 / float(np.sqrt(tr.head_dim)))
    got = O.decode(to_numpy_bits(churn.out[begin:end]), churn.dtype)
    diff = np.abs(got.astype(np.float64) - expected.astype(np.float64))
    return float(diff.max()), float(diff.mean())
