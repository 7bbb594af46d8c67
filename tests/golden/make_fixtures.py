"""Writes tests/golden/attention_vectors.npz: expected outputs for the deterministic inputs of the reference's own
parity tests (generators restated in tests/refdata.py), computed by the CPU oracle.

The reference is Rust + Metal and cannot run where these files are made, so the vectors are the oracle's, not the
reference's; the oracle itself is pinned to the reference's closed-form and literal vectors in
tests/test_oracle_golden.py.  The file guards against silent drift of the oracle and gives the GPU parity tests a
second, stored expectation.  Large outputs keep every 7th element.

    python tests/golden/make_fixtures.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from oracle import psi_oracle as O  # noqa: E402
from refdata import fixture_values, generated_values, pattern  # noqa: E402

STRIDE = 7

TILED_CASES = {
    "tiled_fixed": ([16], 8, 256, 16, 17),
    "tiled_qwen38_27b": ([16], 6, 256, 8, 9),
    "tiled_ragged": ([1, 2, 4, 6, 8, 11, 16, 16], 6, 256, 16, 17),
    "tiled_multiple_tiles": ([32, 8], 8, 256, 16, 17),
    "tiled_qwen3": ([1, 4, 8, 13], 5, 128, 8, 9),
}


def single_q_fixed():
    q, k, v = fixture_values(16, 0.125, 3), fixture_values(8, 0.0625, 5), fixture_values(8, 0.25, 7)
    return O.projected_gqa_reference(4, 2, 2, 0.5, [0, 2], [0], q, [k], [v])


def single_q_random():
    seed = 0x4C8F17D2
    q, k, v = generated_values(16, seed), generated_values(8, seed + 1), generated_values(8, seed + 2)
    return O.projected_gqa_reference(4, 2, 2, 0.5, [0, 2], [0], q, [k], [v])


def single_q_ragged():
    seed = 0xD2056AB9
    q = generated_values(24, seed)
    ks = [generated_values(8, seed + 1), generated_values(8, seed + 3)]
    vs = [generated_values(8, seed + 2), generated_values(8, seed + 4)]
    return O.projected_gqa_reference(4, 2, 2, 0.5, [0, 1, 3], [1, 0], q, ks, vs)


def tiled(case):
    num_tokens_per_req, num_q_heads, head_dim, tokens_per_page, start = case
    reqs, num_tokens = len(num_tokens_per_req), sum(num_tokens_per_req)
    num_blocks = -(-(start + max(num_tokens_per_req)) // tokens_per_page)
    bf = lambda x: O.decode(O.encode(x, O.BF16), O.BF16)
    q = pattern(num_tokens * num_q_heads * head_dim, 29, 0.015625)
    n = num_blocks * tokens_per_page * head_dim
    ks = [pattern(n, 31 + r, 0.015625) for r in range(reqs)]
    vs = [pattern(n, 37 + r, 0.03125) for r in range(reqs)]
    cu = np.concatenate([[0], np.cumsum(num_tokens_per_req)]).tolist()
    scale = float(np.float32(1.0) / np.sqrt(np.float32(head_dim)))
    return O.projected_gqa_reference(
        num_q_heads, 1, head_dim, scale, cu, [start] * reqs, bf(q),
        [bf(ks[r][: (start + num_tokens_per_req[r]) * head_dim]) for r in range(reqs)],
        [bf(vs[r][: (start + num_tokens_per_req[r]) * head_dim]) for r in range(reqs)])


def block_sdpa(dtype):
    block, hq, hkv, d, t = 3, 5, 1, 32, 6
    scale = float(np.float32(1.0) / np.sqrt(np.float32(32.0)))
    q = O.encode(np.arange(t * hq * d, dtype=np.float32) * np.float32(0.03125) - np.float32(0.4), dtype)
    k = O.encode(np.arange(t * hkv * d, dtype=np.float32) * np.float32(-0.025) + np.float32(0.3), dtype)
    v = O.encode(np.arange(t * hkv * d, dtype=np.float32) * np.float32(0.05) - np.float32(0.2), dtype)
    out, pm, ps = O.block_sdpa(q, k, v, dtype, t, block, hq, hkv, d, scale)
    return np.concatenate([out.reshape(-1), pm.reshape(-1), ps.reshape(-1)])


def vectors():
    out = {
        "single_q_fixed": single_q_fixed(),
        "single_q_random": single_q_random(),
        "single_q_ragged": single_q_ragged(),
        "block_sdpa_f32": block_sdpa(O.F32),
        "block_sdpa_bf16": block_sdpa(O.BF16),
    }
    for name, case in TILED_CASES.items():
        out[name] = np.asarray(tiled(case), dtype=np.float32).reshape(-1)[::STRIDE]
    return {k: np.asarray(v, dtype=np.float32).reshape(-1) for k, v in out.items()}


if __name__ == "__main__":
    target = Path(__file__).resolve().parent / "attention_vectors.npz"
    np.savez_compressed(target, **vectors())
    print(target, target.stat().st_size, "bytes")
