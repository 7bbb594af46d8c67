"""Oracle-side helpers shared by the GPU parity tests, the smoke entry and the benchmark's CPU baseline.

Everything here runs the CPU oracle as the checker; nothing in the product imports this module.
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
        _GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "attention_vectors.npz")
    return _GOLDEN[name]
