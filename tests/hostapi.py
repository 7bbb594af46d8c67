"""ctypes helpers for the host-only entry points of libpsi_cuda.so (no device needed)."""
import ctypes as C

import numpy as np

import __graft_entry__ as entry

pkg = entry.load_package()


def lib():
    return pkg.library()


class Metadata:
    """Capacity-sized arrays driven through psi_metadata_update_host (the product's GQAMetadataBuffers::update*)."""

    def __init__(self, max_tokens):
        self.max_tokens = max_tokens
        self.req_slots = np.zeros(max_tokens, dtype=np.uint32)
        self.flat_token_indices = np.zeros(max_tokens, dtype=np.uint32)
        self.q_token_tiles = np.zeros(2 * max_tokens, dtype=np.uint32)
        self.kv_splits = np.zeros(3 * max_tokens, dtype=np.uint32)
        self.cu_kv_splits = np.zeros(max_tokens + 1, dtype=np.uint32)

    def update(self, req_slots, token_indices, cu_tokens, variant, mode=0, boundaries=(), caller_tokens=0):
        p = lambda a: a.ctypes.data_as(C.POINTER(C.c_uint32))
        rs = np.ascontiguousarray(req_slots, dtype=np.uint32)
        ti = np.ascontiguousarray(token_indices, dtype=np.uint32)
        cu = np.ascontiguousarray(cu_tokens, dtype=np.uint32)
        b = np.ascontiguousarray(list(boundaries), dtype=np.uint32)
        shape = pkg.GQAReplayShape()
        status = lib().psi_metadata_update_host(
            C.c_uint32(self.max_tokens), p(rs), p(ti), p(cu), C.c_uint32(len(rs)), C.byref(variant), C.c_uint32(mode),
            p(b), C.c_uint32(len(b)), C.c_uint32(caller_tokens), p(self.req_slots), p(self.flat_token_indices),
            p(self.q_token_tiles), p(self.kv_splits), p(self.cu_kv_splits), C.byref(shape))
        if status:
            buf = C.create_string_buffer(512)
            lib().psi_last_error(buf, C.c_size_t(512))
            raise pkg.PsiError(status, buf.value.decode())
        return shape


def single_q(kv_tile, threads=32, head_tile=1):
    return pkg.GQASplitKVVariant(0, 0, kv_tile, threads, head_tile)


def tiled_q(q_tile, kv_tile, head_tile=1):
    return pkg.GQASplitKVVariant(1, q_tile, kv_tile, 0, head_tile)


def plan_preview(num_q_heads, num_kv_heads, token_indices, cu_tokens, max_ctas, min_tiles=8, start_cost=0):
    p = lambda a: a.ctypes.data_as(C.POINTER(C.c_uint32))
    ti = np.ascontiguousarray(token_indices, dtype=np.uint32)
    cu = np.ascontiguousarray(cu_tokens, dtype=np.uint32)
    counts = np.zeros(6, dtype=np.uint32)
    status = lib().psi_plan_preview(C.c_uint32(num_q_heads), C.c_uint32(num_kv_heads), p(ti), p(cu), C.c_uint32(len(ti)),
                                    C.c_uint32(max_ctas), C.c_uint32(min_tiles), C.c_uint32(start_cost), None, C.c_uint64(0), None,
                                    C.c_uint64(0), p(counts))
    assert status == 0
    items = np.zeros((int(counts[0]), 6), dtype=np.uint32)
    ctas = np.zeros(int(counts[1]) + 1, dtype=np.uint32)
    status = lib().psi_plan_preview(C.c_uint32(num_q_heads), C.c_uint32(num_kv_heads), p(ti), p(cu), C.c_uint32(len(ti)),
                                    C.c_uint32(max_ctas), C.c_uint32(min_tiles), C.c_uint32(start_cost), p(items), C.c_uint64(len(items)),
                                    p(ctas), C.c_uint64(len(ctas)), p(counts))
    assert status == 0
    return items, ctas, counts


def chunk_plan_preview(num_q_heads, num_kv_heads, token_indices, cu_tokens, max_ctas, equal_shares):
    p = lambda a: a.ctypes.data_as(C.POINTER(C.c_uint32))
    ti = np.ascontiguousarray(token_indices, dtype=np.uint32)
    cu = np.ascontiguousarray(cu_tokens, dtype=np.uint32)
    counts = np.zeros(5, dtype=np.uint32)
    args = (C.c_uint32(num_q_heads), C.c_uint32(num_kv_heads), p(ti), p(cu), C.c_uint32(len(ti)), C.c_uint32(max_ctas),
            C.c_uint32(1 if equal_shares else 0))
    assert lib().psi_chunk_plan_preview(*args, None, C.c_uint64(0), None, C.c_uint64(0), p(counts)) == 0
    items = np.zeros((int(counts[0]), 10), dtype=np.uint32)
    ctas = np.zeros(int(counts[1]) + 1, dtype=np.uint32)
    assert lib().psi_chunk_plan_preview(*args, p(items), C.c_uint64(len(items)), p(ctas), C.c_uint64(len(ctas)),
                                        p(counts)) == 0
    return items, ctas, counts
