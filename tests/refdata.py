"""Deterministic input generators that restate the ones the reference's own parity tests use.

Each generator cites the reference test helper it follows (paths relative to the reference project root).
"""
import numpy as np


def fixture_values(count, scale, pattern_offset):
    """crates/inference-backend-metal/src/components/gqa_split_kv_single_q_test.rs:426-430"""
    i = np.arange(count, dtype=np.int64)
    return (((i * 11 + pattern_offset) % 23).astype(np.float32) * np.float32(scale)
            - np.float32(11.0) * np.float32(scale)).astype(np.float32)


def _lcg_states(count, seed):
    out = np.empty(count, dtype=np.uint32)
    state = seed & 0xFFFFFFFF
    for i in range(count):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = state
    return out


def generated_values(count, seed):
    """gqa_split_kv_single_q_test.rs:432-440: v = ((state >> 8) / 2^24) * 2 - 1"""
    s = _lcg_states(count, seed)
    return ((s >> 8).astype(np.float32) / np.float32(16777216.0) * np.float32(2.0) - np.float32(1.0)).astype(
        np.float32)


def generated_half_range_values(count, seed):
    """crates/inference-backend-metal/src/components/gqa_split_kv_tiled_q_test.rs:280-288 before bf16 rounding:
    v = ((state >> 8) / 2^24) - 0.5"""
    s = _lcg_states(count, seed)
    return ((s >> 8).astype(np.float32) / np.float32(16777216.0) - np.float32(0.5)).astype(np.float32)


def pattern(length, modulus, scale):
    """crates/inference-executor-metal/tests/gqa_split_kv_tiled_q.rs:464-468"""
    i = np.arange(length, dtype=np.int64)
    return ((i % modulus).astype(np.float32) * np.float32(scale)
            - np.float32(np.float32(modulus) * np.float32(scale) * np.float32(0.5))).astype(np.float32)


def kv_page_values(num_kv_heads, head_dim, tokens_per_page, pages, fill=0.0):
    """Lay per-page (k, v) token-major value lists out as [page][K/V][Hkv][P][D] f32.
    gqa_split_kv_single_q_test.rs:397-424"""
    stride = num_kv_heads * head_dim
    out = np.full((len(pages), 2, num_kv_heads, tokens_per_page, head_dim), fill, dtype=np.float32)
    for p, (k, v) in enumerate(pages):
        k = np.asarray(k, dtype=np.float32)
        v = np.asarray(v, dtype=np.float32)
        n = k.size // stride
        assert k.size == v.size and k.size % stride == 0 and n <= tokens_per_page
        out[p, 0, :, :n, :] = k.reshape(n, num_kv_heads, head_dim).transpose(1, 0, 2)
        out[p, 1, :, :n, :] = v.reshape(n, num_kv_heads, head_dim).transpose(1, 0, 2)
    return out
