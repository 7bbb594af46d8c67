"""ctypes front-end of the CPU oracle (``psi_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke entry and the benchmark's CPU-baseline / reference arm import this module; the CUDA
library and its Python binding never do.  ``build()`` compiles ``psi_oracle.c`` next to this file with the host C
compiler; every other function is a thin numpy wrapper around one exported C function.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libpsi_oracle.so"
_lib = None

F32, BF16, F16 = 0, 1, 2
CAP_EXACT, CAP_BUCKETED, CAP_CALLER_TOKENS = 0, 1, 2
U32_MAX = 0xFFFFFFFF


class Layout(C.Structure):
    _fields_ = [("num_req_slots", C.c_uint32), ("num_gqa_layers", C.c_uint32), ("num_blocks", C.c_uint32),
                ("num_page_ids_per_block", C.c_uint32)]


class Variant(C.Structure):
    _fields_ = [("tiled_q", C.c_uint32), ("q_token_tile_size", C.c_uint32), ("kv_token_tile_size", C.c_uint32),
                ("num_threads_per_threadblock", C.c_uint32), ("q_head_tile_size", C.c_uint32)]

    def as_tuple(self):
        return (self.tiled_q, self.q_token_tile_size, self.kv_token_tile_size, self.num_threads_per_threadblock,
                self.q_head_tile_size)


class ReplayShape(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "num_tokens", "num_total_tokens", "num_q_token_tiles", "num_total_q_token_tiles",
        "num_sdpa_map_task_templates", "num_total_sdpa_map_task_templates", "reduce_sdpa_partial_outputs")]

    def as_tuple(self):
        return tuple(getattr(self, n) for n, _ in self._fields_)


def build(force: bool = False) -> Path:
    """Compile the oracle if its shared library is missing or older than the source."""
    src = _HERE / "psi_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        cc = "gcc" if not os.environ.get("PSI_ORACLE_CC") else os.environ["PSI_ORACLE_CC"]
        subprocess.run([cc, "-O3", "-march=native", "-pthread", "-fPIC", "-fvisibility=hidden", "-std=c11", "-shared",
                        "-o", str(_LIB_PATH), str(src), "-lm"], check=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(_LIB_PATH))
        _lib.psi_oracle_f32_to_bf16.restype = C.c_uint16
        _lib.psi_oracle_f32_to_bf16.argtypes = [C.c_float]
        _lib.psi_oracle_f32_to_f16.restype = C.c_uint16
        _lib.psi_oracle_f32_to_f16.argtypes = [C.c_float]
        _lib.psi_oracle_bf16_to_f32.restype = C.c_float
        _lib.psi_oracle_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.psi_oracle_f16_to_f32.restype = C.c_float
        _lib.psi_oracle_f16_to_f32.argtypes = [C.c_uint16]
        _lib.psi_oracle_bucket_policy.restype = C.c_int64
        _lib.psi_oracle_build_single_q_kv_splits.restype = C.c_int64
        _lib.psi_oracle_build_tiled_q_kv_splits.restype = C.c_int64
        _lib.psi_oracle_bucket_capacity.restype = C.c_uint32
        _lib.psi_oracle_allocator_new.restype = C.c_void_p
        _lib.psi_oracle_allocator_bitmap.restype = C.c_uint64
        _lib.psi_oracle_allocator_free_count.restype = C.c_uint64
    return _lib


def _p(a, t=C.c_void_p):
    return a.ctypes.data_as(t)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def np_dtype(dtype: int):
    return np.float32 if dtype == F32 else np.uint16


def encode(values, dtype: int) -> np.ndarray:
    """f32 -> storage bits of ``dtype`` (f32 array, or u16 bit patterns for bf16 / f16), round-to-nearest-even."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty(v.shape, dtype=np_dtype(dtype))
    lib().psi_oracle_encode(_p(v), C.c_int(dtype), C.c_size_t(v.size), _p(out))
    return out


def decode(bits, dtype: int) -> np.ndarray:
    b = np.ascontiguousarray(bits, dtype=np_dtype(dtype))
    out = np.empty(b.shape, dtype=np.float32)
    lib().psi_oracle_decode(_p(b), C.c_int(dtype), C.c_size_t(b.size), _p(out))
    return out


def kv_page_write(pages, flat_k, flat_v, req_slots, flat_token_indices, page_ids, num_active, layer, layout: Layout,
                  num_kv_heads, head_dim, page_bytes):
    """In-place append into ``pages`` (a contiguous numpy array of 2- or 4-byte elements)."""
    assert pages.flags.c_contiguous and pages.itemsize in (2, 4)
    k = np.ascontiguousarray(flat_k, dtype=pages.dtype)
    v = np.ascontiguousarray(flat_v, dtype=pages.dtype)
    rs, ti, ids = _u32(req_slots), _u32(flat_token_indices), _u32(page_ids)
    lib().psi_oracle_kv_page_write(_p(pages), C.c_uint32(pages.itemsize), _p(k), _p(v), _p(rs), _p(ti), _p(ids),
                                   C.c_uint32(num_active), C.c_uint32(layer), C.byref(layout),
                                   C.c_uint32(num_kv_heads), C.c_uint32(head_dim), C.c_uint32(page_bytes))


def page_gather(pages, page_ids, req_slot, layer, layout: Layout, num_kv_heads, head_dim, page_bytes, tok_begin,
                tok_end):
    n = tok_end - tok_begin
    k = np.zeros((n, num_kv_heads, head_dim), dtype=pages.dtype)
    v = np.zeros_like(k)
    ids = _u32(page_ids)
    lib().psi_oracle_page_gather(_p(pages), C.c_uint32(pages.itemsize), _p(ids), C.c_uint32(req_slot),
                                 C.c_uint32(layer), C.byref(layout), C.c_uint32(num_kv_heads), C.c_uint32(head_dim),
                                 C.c_uint32(page_bytes), C.c_uint32(tok_begin), C.c_uint32(tok_end), _p(k), _p(v))
    return k, v


def softmax(logits):
    x = np.ascontiguousarray(logits, dtype=np.float32)
    out = np.empty_like(x)
    rc = lib().psi_oracle_softmax(_p(x), C.c_size_t(x.size), _p(out))
    if rc:
        raise AssertionError("softmax reference requires finite positive total")
    return out


def projected_gqa_reference(num_q_heads, num_kv_heads, head_dim, scale, cu_tokens, token_indices, q, k_by_req,
                            v_by_req):
    cu, ti = _u32(cu_tokens), _u32(token_indices)
    qf = np.ascontiguousarray(q, dtype=np.float32).ravel()
    ks = [np.ascontiguousarray(k, dtype=np.float32).ravel() for k in k_by_req]
    vs = [np.ascontiguousarray(v, dtype=np.float32).ravel() for v in v_by_req]
    n = len(ti)
    assert len(cu) == n + 1 and cu[0] == 0 and len(ks) == n and len(vs) == n
    total = int(cu[-1])
    assert qf.size == total * num_q_heads * head_dim
    for r in range(n):
        ctx = int(ti[r]) + int(cu[r + 1] - cu[r])
        assert ks[r].size == ctx * num_kv_heads * head_dim and vs[r].size == ks[r].size
    kp = (C.c_void_p * n)(*[k.ctypes.data for k in ks])
    vp = (C.c_void_p * n)(*[v.ctypes.data for v in vs])
    out = np.zeros(total * num_q_heads * head_dim, dtype=np.float32)
    rc = lib().psi_oracle_projected_gqa_reference(C.c_uint32(num_q_heads), C.c_uint32(num_kv_heads),
                                                  C.c_uint32(head_dim), C.c_float(scale), _p(cu), _p(ti),
                                                  C.c_uint32(n), _p(qf), kp, vp, _p(out))
    if rc:
        raise AssertionError("softmax reference requires finite positive total")
    return out


def paged_attention(pages, dtype, q, req_slots, flat_token_indices, page_ids, layer, layout: Layout, num_q_heads,
                    num_kv_heads, head_dim, page_bytes, scale, kv_begin=0, kv_end=0, want_stats=False):
    """Attention straight from the paged arena; returns f32 ``[T][Hq][D]`` (and natural-log ``max``/``sum``)."""
    rs, ti, ids = _u32(req_slots), _u32(flat_token_indices), _u32(page_ids)
    qq = np.ascontiguousarray(q, dtype=np_dtype(dtype))
    pg = np.ascontiguousarray(pages, dtype=np_dtype(dtype))
    t = len(ti)
    out = np.zeros((t, num_q_heads, head_dim), dtype=np.float32)
    mx = np.zeros((t, num_q_heads), dtype=np.float32)
    sm = np.zeros((t, num_q_heads), dtype=np.float32)
    rc = lib().psi_oracle_paged_attention(_p(pg), C.c_int(dtype), _p(qq), _p(rs), _p(ti), C.c_uint32(t), _p(ids),
                                          C.c_uint32(layer), C.byref(layout), C.c_uint32(num_q_heads),
                                          C.c_uint32(num_kv_heads), C.c_uint32(head_dim), C.c_uint32(page_bytes),
                                          C.c_float(scale), C.c_uint32(kv_begin), C.c_uint32(kv_end), _p(out), _p(mx),
                                          _p(sm))
    if rc:
        raise AssertionError("softmax reference requires finite positive total")
    return (out, mx, sm) if want_stats else out


def set_num_threads(n: int):
    lib().psi_oracle_set_num_threads(C.c_int(n))


def num_threads() -> int:
    return int(lib().psi_oracle_num_threads())


def merge_partials(partial_output, partial_max, partial_sum):
    po = np.ascontiguousarray(partial_output, dtype=np.float32)
    pm = np.ascontiguousarray(partial_max, dtype=np.float32)
    ps = np.ascontiguousarray(partial_sum, dtype=np.float32)
    n, d = po.shape
    out = np.empty(d, dtype=np.float32)
    lib().psi_oracle_merge_partials(_p(po), _p(pm), _p(ps), C.c_uint32(n), C.c_uint32(d), _p(out))
    return out


def bucket_policy(max_capacity, boundaries=()):
    b = _u32(list(boundaries))
    cap = 4096 + len(b)
    out = np.zeros(cap, dtype=np.uint32)
    n = lib().psi_oracle_bucket_policy(C.c_uint32(max_capacity), _p(b), C.c_uint32(len(b)), _p(out), C.c_uint64(cap))
    if n < 0:
        raise AssertionError("replay bucket policy contract violated")
    return out[:n].tolist()


def bucket_capacity(buckets, active):
    b = _u32(buckets)
    c = lib().psi_oracle_bucket_capacity(_p(b), C.c_uint64(len(b)), C.c_uint32(active))
    if c == 0:
        raise AssertionError("replay active work exceeds capacity" if active else "replay bucket requires active work")
    return int(c)


def split_kv_select(io_dtype, page_bytes, num_q_heads, num_kv_heads, head_dim, num_tokens, num_q_token_tiles,
                    dspark_history=False):
    v = Variant()
    mq = C.c_uint32(0)
    rc = lib().psi_oracle_split_kv_select(C.c_int(io_dtype), C.c_uint32(page_bytes), C.c_uint32(num_q_heads),
                                          C.c_uint32(num_kv_heads), C.c_uint32(head_dim),
                                          C.c_int(1 if dspark_history else 0), C.c_uint32(num_tokens),
                                          C.c_uint32(num_q_token_tiles), C.byref(v), C.byref(mq))
    if rc:
        raise AssertionError("invalid SplitKV selection input")
    return v, int(mq.value)


def single_q_variant(kv_tile, threads=32, head_tile=1):
    return Variant(0, 0, kv_tile, threads, head_tile)


def tiled_q_variant(q_tile, kv_tile, head_tile=1):
    return Variant(1, q_tile, kv_tile, 0, head_tile)


class Metadata:
    """Capacity-sized metadata arrays updated in place, like the reference's GQAMetadataBuffers."""

    def __init__(self, max_tokens):
        self.max_tokens = max_tokens
        self.req_slots = np.zeros(max_tokens, dtype=np.uint32)
        self.flat_token_indices = np.zeros(max_tokens, dtype=np.uint32)
        self.q_token_tiles = np.zeros(2 * max_tokens, dtype=np.uint32)
        self.kv_splits = np.zeros(3 * max_tokens, dtype=np.uint32)
        self.cu_kv_splits = np.zeros(max_tokens + 1, dtype=np.uint32)

    def update(self, req_slots, token_indices, cu_tokens, variant: Variant, mode=CAP_EXACT, boundaries=(),
               caller_tokens=0):
        rs, ti, cu = _u32(req_slots), _u32(token_indices), _u32(cu_tokens)
        assert len(rs) == len(ti) and len(cu) == len(rs) + 1
        b = _u32(list(boundaries))
        shape = ReplayShape()
        rc = lib().psi_oracle_metadata_update(C.c_uint32(self.max_tokens), _p(rs), _p(ti), _p(cu), C.c_uint32(len(rs)),
                                              C.byref(variant), C.c_int(mode), _p(b), C.c_uint32(len(b)),
                                              C.c_uint32(caller_tokens), _p(self.req_slots),
                                              _p(self.flat_token_indices), _p(self.q_token_tiles), _p(self.kv_splits),
                                              _p(self.cu_kv_splits), C.byref(shape))
        if rc:
            raise AssertionError(f"GQA metadata contract violated (code {rc})")
        return shape


class Allocator:
    def __init__(self, capacity):
        self._h = C.c_void_p(lib().psi_oracle_allocator_new(C.c_uint64(capacity)))
        self.capacity = capacity

    def __del__(self):
        if getattr(self, "_h", None):
            lib().psi_oracle_allocator_free(self._h)
            self._h = None

    def alloc_many(self, count):
        ids = np.zeros(max(count, 1), dtype=np.uint32)
        rc = lib().psi_oracle_allocator_alloc_many(self._h, C.c_uint64(count), _p(ids))
        if rc:
            raise MemoryError("not enough ID")
        return ids[:count].tolist()

    def alloc_one(self):
        return self.alloc_many(1)[0]

    def free_many(self, ids):
        a = _u32(list(ids))
        lib().psi_oracle_allocator_free_many(self._h, _p(a), C.c_uint64(len(a)))

    def bitmap(self):
        words = np.zeros((self.capacity + 63) // 64, dtype=np.uint64)
        lib().psi_oracle_allocator_bitmap(self._h, _p(words), C.c_uint64(len(words)))
        return [int(w) for w in words]

    def free_count(self):
        return int(lib().psi_oracle_allocator_free_count(self._h))


class Yarn(C.Structure):
    _fields_ = [("enabled", C.c_uint32), ("factor", C.c_float), ("attention_factor", C.c_float),
                ("beta_fast", C.c_float), ("beta_slow", C.c_float), ("original_max_position_embeddings", C.c_uint32),
                ("truncate", C.c_uint32)]


def rope_parameters(rope_dim, rope_theta, yarn: Yarn | None = None):
    """(inverse_frequencies[rope_dim/2], attention_factor, correction_low, correction_high)."""
    inv = np.zeros(rope_dim // 2, dtype=np.float32)
    factor, low, high = C.c_float(), C.c_float(), C.c_float()
    y = yarn if yarn is not None else Yarn(0, 1.0, 1.0, 1.0, 1.0, 1, 0)
    rc = lib().psi_oracle_rope_parameters(C.c_uint32(rope_dim), C.c_float(rope_theta), C.byref(y), _p(inv),
                                          C.byref(factor), C.byref(low), C.byref(high))
    if rc:
        raise AssertionError("invalid rope parameters")
    return inv, factor.value, low.value, high.value


def rms_norm_rope(values_bits, dtype, norm_weight_bf16, positions, num_heads, head_dim, rope_dim, eps, inv_freq,
                  attention_factor=1.0):
    x = np.ascontiguousarray(values_bits, dtype=np_dtype(dtype))
    w = np.ascontiguousarray(norm_weight_bf16, dtype=np.uint16)
    pos = _u32(positions)
    f = np.ascontiguousarray(inv_freq, dtype=np.float32)
    out = np.zeros_like(x)
    lib().psi_oracle_rms_norm_rope(_p(x), C.c_int(dtype), _p(w), _p(pos), C.c_uint32(len(pos)), C.c_uint32(num_heads),
                                   C.c_uint32(head_dim), C.c_uint32(rope_dim), C.c_float(eps), _p(f),
                                   C.c_float(attention_factor), _p(out))
    return out


def projection_split(projection_bits, dtype, gated, num_tokens, num_q_heads, num_kv_heads, head_dim):
    """De-interleave a fused projection output [T][width] into (q, g, k, v); g is None for the ungated layout."""
    x = np.ascontiguousarray(projection_bits, dtype=np_dtype(dtype)).reshape(-1)
    q = np.zeros((num_tokens, num_q_heads, head_dim), dtype=x.dtype)
    g = np.zeros_like(q)
    k = np.zeros((num_tokens, num_kv_heads, head_dim), dtype=x.dtype)
    v = np.zeros_like(k)
    lib().psi_oracle_projection_split(_p(x), C.c_uint32(x.dtype.itemsize), C.c_uint32(1 if gated else 0),
                                      C.c_uint32(num_tokens), C.c_uint32(num_q_heads), C.c_uint32(num_kv_heads),
                                      C.c_uint32(head_dim), _p(q), _p(g), _p(k), _p(v))
    return q, (g if gated else None), k, v


def activation_gate(attention_bits, gate_bits, dtype):
    a = np.ascontiguousarray(attention_bits, dtype=np_dtype(dtype))
    g = np.ascontiguousarray(gate_bits, dtype=np_dtype(dtype))
    out = np.zeros_like(a)
    lib().psi_oracle_activation_gate(_p(a), _p(g), C.c_int(dtype), C.c_size_t(a.size), _p(out))
    return out


def block_sdpa(q_bits, k_bits, v_bits, dtype, num_tokens, block_size, num_q_heads, num_kv_heads, head_dim, scale):
    """Dense bidirectional block attention partials: (output f32 [T][Hq][D], max [T][Hq], exp-sum [T][Hq])."""
    q = np.ascontiguousarray(q_bits, dtype=np_dtype(dtype))
    k = np.ascontiguousarray(k_bits, dtype=np_dtype(dtype))
    v = np.ascontiguousarray(v_bits, dtype=np_dtype(dtype))
    out = np.zeros((num_tokens, num_q_heads, head_dim), dtype=np.float32)
    pm = np.zeros((num_tokens, num_q_heads), dtype=np.float32)
    ps = np.zeros((num_tokens, num_q_heads), dtype=np.float32)
    lib().psi_oracle_block_sdpa(_p(q), _p(k), _p(v), C.c_int(dtype), C.c_uint32(num_tokens), C.c_uint32(block_size),
                                C.c_uint32(num_q_heads), C.c_uint32(num_kv_heads), C.c_uint32(head_dim),
                                C.c_float(scale), _p(out), _p(pm), _p(ps))
    return out, pm, ps
