"""ctypes binding of the C ABI declared in ``include/psi_cuda.h``.

The classes keep the names and argument meaning of the reference's host-side owners of this path
(``GQARequestPageTable``, ``PageArena``, ``GQAMetadataBuffers`` + ``GQA``, ``ReplayBucketPolicy``, ``GQASplitKV``,
``U32IDAllocator``); a violated contract raises :class:`PsiError` where the reference panics.  Device buffers are passed
as integers (device addresses) or as objects with a ``data_ptr()`` method such as torch tensors.  There is no CPU
fallback: the shared library must exist and every compute call needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

F32, BF16, F16 = 0, 1, 2
PLAN_BALANCED, PLAN_REFERENCE = 0, 1
KERNEL_AUTO, KERNEL_GENERIC, KERNEL_MMA, KERNEL_MMA_SYNC, KERNEL_MMA_TMA = 0, 1, 2, 3, 4
CAPACITY_EXACT, CAPACITY_BUCKETED, CAPACITY_CALLER_TOKENS = 0, 1, 2
MD_REQ_SLOTS, MD_FLAT_TOKEN_INDICES, MD_Q_TOKEN_TILES, MD_KV_SPLITS, MD_CU_KV_SPLITS = range(5)

_STATUS = {1: "invalid argument", 2: "resource exhausted", 3: "internal error", 4: "timeout", 5: "CUDA error"}

def _library_file() -> Path:
    """``lib/libpsi_cuda.so``, or what the environment variable PSI_CUDA_LIBRARY names: ``checked`` for the
    bounds-checked build ``lib/libpsi_cuda_checked.so``, or a path."""
    import os
    choice = os.environ.get("PSI_CUDA_LIBRARY", "")
    lib_dir = Path(__file__).resolve().parent / "lib"
    if choice == "checked":
        return lib_dir / "libpsi_cuda_checked.so"
    return Path(choice) if choice else lib_dir / "libpsi_cuda.so"


_LIB_PATH = _library_file()
_lib = None


class PsiError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{_STATUS.get(status, status)}: {message}")
        self.status = status
        self.message = message


class GQAPageTableLayout(C.Structure):
    _fields_ = [("num_req_slots", C.c_uint32), ("num_gqa_layers", C.c_uint32), ("num_blocks", C.c_uint32),
                ("num_page_ids_per_block", C.c_uint32)]


class GQAReplayShape(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "num_tokens", "num_total_tokens", "num_q_token_tiles", "num_total_q_token_tiles",
        "num_sdpa_map_task_templates", "num_total_sdpa_map_task_templates", "reduce_sdpa_partial_outputs")]

    def as_tuple(self):
        return tuple(getattr(self, n) for n, _ in self._fields_)


class GQASplitKVVariant(C.Structure):
    _fields_ = [("tiled_q", C.c_uint32), ("q_token_tile_size", C.c_uint32), ("kv_token_tile_size", C.c_uint32),
                ("num_threads_per_threadblock", C.c_uint32), ("q_head_tile_size", C.c_uint32)]

    def as_tuple(self):
        return tuple(getattr(self, n) for n, _ in self._fields_)


class NormRopeConfig(C.Structure):
    _fields_ = [("rope_dim", C.c_uint32), ("eps", C.c_float), ("rope_theta", C.c_float), ("yarn_enabled", C.c_uint32),
                ("yarn_factor", C.c_float), ("yarn_attention_factor", C.c_float), ("yarn_beta_fast", C.c_float),
                ("yarn_beta_slow", C.c_float), ("yarn_original_max_position_embeddings", C.c_uint32),
                ("yarn_truncate", C.c_uint32)]


def rope_parameters(config: "NormRopeConfig"):
    """(inverse_frequencies, attention_factor, correction_low, correction_high) of a RoPE profile (host only)."""
    inv = (C.c_float * max(config.rope_dim // 2, 1))()
    factor, low, high = C.c_float(), C.c_float(), C.c_float()
    _check(library().psi_rope_parameters(C.byref(config), inv, C.byref(factor), C.byref(low), C.byref(high)))
    return list(inv[: config.rope_dim // 2]), factor.value, low.value, high.value


class KvExchange(C.Structure):
    """``psi_kv_exchange``: one rank's view of a KV-range exchange group (addresses as seen from this rank's device)."""
    _fields_ = [("rank", C.c_uint32), ("world", C.c_uint32), ("owner", C.c_uint32), ("step", C.c_uint32),
                ("slots", C.c_void_p), ("slot_floats", C.c_uint64), ("flags", C.c_void_p), ("consumed", C.c_void_p),
                ("max_polls", C.c_uint32)]


class GQAConfig(C.Structure):
    _fields_ = [("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("scale", C.c_float), ("page_bytes", C.c_uint32), ("dtype", C.c_uint32),
                ("layout", GQAPageTableLayout), ("max_tokens", C.c_uint32), ("plan_mode", C.c_uint32),
                ("kernel_mode", C.c_uint32), ("max_ctas", C.c_uint32)]


def library_path() -> Path:
    return _LIB_PATH


def library():
    """Load ``libpsi_cuda.so``; raises if it has not been built (``python psi-dec_b200/build.py``)."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise FileNotFoundError(f"{_LIB_PATH} is missing: build it with psi-dec_b200/build.py (no CPU fallback)")
        _lib = C.CDLL(str(_LIB_PATH))
    return _lib


def _ptr(x):
    if x is None:
        return C.c_void_p(0)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    return C.c_void_p(int(x))


def _u32_array(values):
    """(pointer, length) of a u32 sequence; a contiguous numpy uint32 array is passed without a copy."""
    if hasattr(values, "ctypes") and getattr(values, "dtype", None) is not None and values.dtype.itemsize == 4 \
            and values.dtype.kind == "u" and values.flags["C_CONTIGUOUS"]:
        return values.ctypes.data_as(C.POINTER(C.c_uint32)), int(values.size)
    values = [int(v) for v in values]
    return (C.c_uint32 * max(len(values), 1))(*values), len(values)


def _check(status: int, ctx=None):
    if status == 0:
        return
    buf = C.create_string_buffer(1024)
    if ctx is not None:
        library().psi_ctx_last_error(ctx, buf, C.c_size_t(len(buf)))
    else:
        library().psi_last_error(buf, C.c_size_t(len(buf)))
    raise PsiError(status, buf.value.decode("utf-8", "replace"))


class Graph:
    """A captured launch sequence (the reference's recorded replay program); ``launch`` replays it on the context's
    stream after the step's ``GQA.prepare``."""

    def __init__(self, ctx, handle):
        self.ctx = ctx
        self._h = handle

    def launch(self):
        _check(library().psi_graph_launch(self._h), self.ctx._h)

    def kernel_count(self) -> int:
        out = C.c_uint64()
        _check(library().psi_graph_kernel_count(self._h, C.byref(out)), self.ctx._h)
        return out.value

    def close(self):
        if getattr(self, "_h", None):
            library().psi_graph_destroy(self._h)
            self._h = None

    __del__ = close


class Context:
    """One device + one stream (the reference's ``Device::system_default()`` + ``Stream``)."""

    def __init__(self, device: int = 0, stream=None):
        self._h = C.c_void_p()
        if stream is None:
            _check(library().psi_ctx_create(C.c_int32(device), C.byref(self._h)))
        else:
            _check(library().psi_ctx_create_on_stream(C.c_int32(device), C.c_void_p(int(stream)), C.byref(self._h)))
        self.device = device

    def close(self):
        if self._h:
            library().psi_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def sync(self):
        _check(library().psi_ctx_sync(self._h), self._h)

    def read_bandwidth(self, num_bytes: int, iterations: int = 5) -> float:
        """GB/s of a kernel that only reads ``num_bytes`` of HBM with 16-byte loads (best of ``iterations`` passes)."""
        out = C.c_double()
        _check(library().psi_ctx_read_bandwidth(self._h, C.c_uint64(num_bytes), C.c_uint32(iterations), C.byref(out)), self._h)
        return float(out.value)

    @property
    def sm_count(self) -> int:
        out = C.c_int32()
        _check(library().psi_ctx_sm_count(self._h, C.byref(out)), self._h)
        return out.value

    @property
    def launch_count(self) -> int:
        out = C.c_uint64()
        _check(library().psi_ctx_launch_count(self._h, C.byref(out)), self._h)
        return out.value

    def capture_begin(self):
        """Start capturing the library's launches on this context's stream (``Stream::create_replay_program``)."""
        _check(library().psi_ctx_capture_begin(self._h), self._h)

    def capture_end(self) -> "Graph":
        handle = C.c_void_p()
        _check(library().psi_ctx_capture_end(self._h, C.byref(handle)), self._h)
        return Graph(self, handle)

    def enable_kernel_timing(self, enable: bool = True):
        _check(library().psi_ctx_enable_kernel_timing(self._h, C.c_int32(1 if enable else 0)), self._h)

    def kernel_timing(self, kernel_class: int):
        """(total milliseconds, launches) of one kernel class (0 append, 1 attend map, 2 attend reduce, 3 combine,
        4 gather) since timing was enabled."""
        ms, n = C.c_float(), C.c_uint64()
        _check(library().psi_ctx_kernel_timing(self._h, C.c_uint32(kernel_class), C.byref(ms), C.byref(n)), self._h)
        return ms.value, n.value

    @property
    def stream(self) -> int:
        out = C.c_void_p()
        _check(library().psi_ctx_stream(self._h, C.byref(out)), self._h)
        return out.value or 0


class PageArena:
    """``num_pages x page_bytes`` of zero-filled device memory (reference ``PageArena``)."""

    def __init__(self, ctx: Context, num_pages: int, page_bytes: int, device_ptr=None):
        self.ctx, self.num_pages, self.page_bytes = ctx, num_pages, page_bytes
        self._h = C.c_void_p()
        if device_ptr is None:
            _check(library().psi_pages_create(ctx._h, C.c_uint64(num_pages), C.c_uint32(page_bytes),
                                              C.byref(self._h)), ctx._h)
        else:
            _check(library().psi_pages_wrap(ctx._h, _ptr(device_ptr), C.c_uint64(num_pages), C.c_uint32(page_bytes),
                                            C.byref(self._h)), ctx._h)

    def close(self):
        if self._h:
            library().psi_pages_destroy(self._h)
            self._h = C.c_void_p()

    def buffer(self) -> int:
        out = C.c_void_p()
        _check(library().psi_pages_device_ptr(self._h, C.byref(out)), self.ctx._h)
        return out.value

    def release_resources(self):
        _check(library().psi_pages_release(self._h), self.ctx._h)

    def allocate_resources(self):
        _check(library().psi_pages_allocate(self._h), self.ctx._h)

    def export_range(self, page_begin: int, page_end: int) -> bytes:
        buf = C.create_string_buffer(max(1, (page_end - page_begin) * self.page_bytes))
        _check(library().psi_pages_export_range(self._h, C.c_uint64(page_begin), C.c_uint64(page_end), buf),
               self.ctx._h)
        return buf.raw[: (page_end - page_begin) * self.page_bytes]

    def import_range(self, page_begin: int, page_end: int, data: bytes):
        assert len(data) == (page_end - page_begin) * self.page_bytes
        _check(library().psi_pages_import_range(self._h, C.c_uint64(page_begin), C.c_uint64(page_end),
                                                C.c_char_p(bytes(data))), self.ctx._h)


class GQARequestPageTable:
    """Device block table ``u32[slots][layers][blocks][ids_per_block]`` (reference ``GQARequestPageTable``)."""

    def __init__(self, ctx: Context, layout: GQAPageTableLayout):
        self.ctx, self.layout = ctx, layout
        self._h = C.c_void_p()
        _check(library().psi_table_create(ctx._h, C.byref(layout), C.byref(self._h)), ctx._h)

    def close(self):
        if self._h:
            library().psi_table_destroy(self._h)
            self._h = C.c_void_p()

    def write_page_ids(self, req_slot, layer_index, block_index, page_ids):
        arr, n = _u32_array(page_ids)
        _check(library().psi_table_write(self._h, C.c_uint32(req_slot), C.c_uint32(layer_index),
                                         C.c_uint32(block_index), arr, C.c_uint32(n)), self.ctx._h)

    def write_all_layer_page_ids(self, req_slot, block_index, page_ids, num_cache_pages):
        arr, n = _u32_array(page_ids)
        _check(library().psi_table_write_all_layers(self._h, C.c_uint32(req_slot), C.c_uint32(block_index), arr,
                                                    C.c_uint32(n), C.c_uint64(num_cache_pages)), self.ctx._h)

    def set_page_bound(self, num_cache_pages: int):
        """Declare the arena's page count: later writes and snapshot loads refuse page IDs at or beyond it."""
        _check(library().psi_table_set_page_bound(self._h, C.c_uint64(num_cache_pages)), self.ctx._h)

    def write_row(self, req_slot, layer_index, page_ids):
        """Bulk load of the leading entries of one (slot, layer) row; ``page_ids`` may be a numpy u32 array."""
        if hasattr(page_ids, "ctypes"):
            import numpy as np
            a = np.ascontiguousarray(page_ids, dtype=np.uint32)
            arr, n = a.ctypes.data_as(C.POINTER(C.c_uint32)), a.size
        else:
            arr, n = _u32_array(page_ids)
        _check(library().psi_table_write_row(self._h, C.c_uint32(req_slot), C.c_uint32(layer_index), arr,
                                             C.c_uint32(n)), self.ctx._h)

    def read_page_ids(self, req_slot, layer_index, block_index):
        n = self.layout.num_page_ids_per_block
        out = (C.c_uint32 * n)()
        _check(library().psi_table_read(self._h, C.c_uint32(req_slot), C.c_uint32(layer_index),
                                        C.c_uint32(block_index), out, C.c_uint32(n)), self.ctx._h)
        return list(out)

    def reset_req_slots(self, req_slots):
        arr, n = _u32_array(req_slots)
        _check(library().psi_table_reset_slots(self._h, arr, C.c_uint32(n)), self.ctx._h)

    def reset_req_slot(self, req_slot):
        self.reset_req_slots([req_slot])

    def page_ids_buffer(self) -> int:
        out = C.c_void_p()
        _check(library().psi_table_device_ptr(self._h, C.byref(out)), self.ctx._h)
        return out.value


class ReplayBucketPolicy:
    """Reference ``ReplayBucketPolicy`` (host only)."""

    def __init__(self, max_capacity: int, topology_boundaries=()):
        self.max_capacity = max_capacity
        self._b, self._nb = _u32_array(topology_boundaries)
        out = (C.c_uint32 * (4096 + self._nb))()
        n = C.c_uint64()
        _check(library().psi_replay_bucket_policy(C.c_uint32(max_capacity), self._b, C.c_uint32(self._nb), out,
                                                  C.c_uint64(len(out)), C.byref(n)))
        self._buckets = list(out[: n.value])

    def buckets(self):
        return list(self._buckets)

    def capacity(self, active: int) -> int:
        out = C.c_uint32()
        _check(library().psi_replay_bucket_capacity(C.c_uint32(self.max_capacity), self._b, C.c_uint32(self._nb),
                                                    C.c_uint32(active), C.byref(out)))
        return out.value

    def capacity_allow_zero(self, active: int) -> int:
        return 0 if active == 0 else self.capacity(active)


class GQASplitKV:
    """Reference ``GQASplitKV`` selector (host only)."""

    def __init__(self, io_dtype, page_bytes, num_q_heads, num_kv_heads, head_dim, dspark_history=False):
        self._args = (C.c_uint32(io_dtype), C.c_uint32(page_bytes), C.c_uint32(num_q_heads), C.c_uint32(num_kv_heads),
                      C.c_uint32(head_dim), C.c_uint32(1 if dspark_history else 0))
        self.select(1, 1)  # validates the configuration like GQASplitKV::new

    def _call(self, num_tokens, num_q_token_tiles):
        v, mq = GQASplitKVVariant(), C.c_uint32()
        _check(library().psi_split_kv_select(*self._args, C.c_uint32(num_tokens), C.c_uint32(num_q_token_tiles),
                                             C.byref(v), C.byref(mq)))
        return v, mq.value

    def select(self, num_tokens, num_q_token_tiles) -> GQASplitKVVariant:
        return self._call(num_tokens, num_q_token_tiles)[0]

    def max_q_tokens_per_partial_output(self) -> int:
        return self._call(1, 1)[1]


class _U32Range(C.Structure):
    _fields_ = [("begin", C.c_uint32), ("end", C.c_uint32)]


class _HibernationPlan(C.Structure):
    _fields_ = [("selected", C.c_uint32), ("request_slot_ranges", C.POINTER(_U32Range)),
                ("num_request_slot_ranges", C.c_uint64), ("page_id_ranges", C.POINTER(_U32Range)),
                ("num_page_id_ranges", C.c_uint64)]


def _ranges(ranges):
    ranges = [(int(b), int(e)) for b, e in ranges]
    arr = (_U32Range * max(len(ranges), 1))(*[_U32Range(b, e) for b, e in ranges])
    return arr, len(ranges)


class ExecutorHibernationPlan:
    """``ExecutorHibernationPlan``: ``all()`` or ``selected(request_slot_ranges, page_id_ranges)`` (half-open ranges)."""

    def __init__(self, selected: bool, request_slot_ranges=(), page_id_ranges=()):
        self.is_selected = selected
        self.request_slot_ranges = [tuple(r) for r in request_slot_ranges]
        self.page_id_ranges = [tuple(r) for r in page_id_ranges]

    @classmethod
    def all(cls):
        return cls(False)

    @classmethod
    def selected(cls, request_slot_ranges, page_id_ranges):
        return cls(True, request_slot_ranges, page_id_ranges)

    def _c(self):
        slots, n_slots = _ranges(self.request_slot_ranges)
        pages, n_pages = _ranges(self.page_id_ranges)
        plan = _HibernationPlan(1 if self.is_selected else 0, slots, n_slots, pages, n_pages)
        return plan, (slots, pages)  # the arrays must outlive the call


# StateSnapshotFile
SNAPSHOT_PAGE_ARENA, SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE, SNAPSHOT_MAIN_GDN_REQUEST_STATE_TABLE = 0, 1, 2
SNAPSHOT_MAIN_GDN_RECURRENT_STATE, SNAPSHOT_MAIN_GDN_CONV_STATE = 3, 4
SNAPSHOT_MTP_GQA_REQUEST_PAGE_TABLE, SNAPSHOT_DSPARK_GQA_REQUEST_PAGE_TABLE = 5, 6


class StateSnapshotWriter:
    """``StateSnapshotWriter``: files go into a temporary directory that ``commit`` publishes by rename."""

    def __init__(self, destination, expected_files, plan: ExecutorHibernationPlan):
        self._h = C.c_void_p()
        files, n = _u32_array(list(expected_files))
        c_plan, keep = plan._c()
        _check(library().psi_snapshot_writer_create(str(destination).encode(), files, C.c_uint64(n), C.byref(c_plan),
                                                    C.byref(self._h)))

    def close(self):
        if getattr(self, "_h", None):
            library().psi_snapshot_writer_destroy(self._h)
            self._h = None

    __del__ = close

    def write_pages(self, snapshot_file: int, pages):
        _check(library().psi_snapshot_write_pages(self._h, C.c_uint32(snapshot_file), pages._h))

    def write_table(self, snapshot_file: int, table):
        _check(library().psi_snapshot_write_table(self._h, C.c_uint32(snapshot_file), table._h))

    def write_full_buffer(self, snapshot_file: int, array):
        _check(library().psi_snapshot_write_host_buffer(self._h, C.c_uint32(snapshot_file), C.c_void_p(array.ctypes.data),
                                                        C.c_uint64(array.nbytes), None, C.c_uint64(0), C.c_uint64(0)))

    def write_selected_buffer(self, snapshot_file: int, array, entry_ranges, entry_bytes: int):
        ranges, n = _ranges(entry_ranges)
        _check(library().psi_snapshot_write_host_buffer(self._h, C.c_uint32(snapshot_file), C.c_void_p(array.ctypes.data),
                                                        C.c_uint64(array.nbytes), ranges, C.c_uint64(n),
                                                        C.c_uint64(entry_bytes)))

    def write_metadata(self, snapshot_file: int, payload: bytes):
        _check(library().psi_snapshot_write_metadata(self._h, C.c_uint32(snapshot_file), payload, C.c_uint64(len(payload))))

    def commit(self):
        _check(library().psi_snapshot_writer_commit(self._h))


class StateSnapshotReader:
    """``StateSnapshotReader``: validates manifest, plan, file set and directory on open; ``finish`` checks that every
    file was read."""

    def __init__(self, path, expected_files, plan: ExecutorHibernationPlan):
        self._h = C.c_void_p()
        files, n = _u32_array(list(expected_files))
        c_plan, keep = plan._c()
        _check(library().psi_snapshot_reader_open(str(path).encode(), files, C.c_uint64(n), C.byref(c_plan),
                                                  C.byref(self._h)))

    def close(self):
        if getattr(self, "_h", None):
            library().psi_snapshot_reader_destroy(self._h)
            self._h = None

    __del__ = close

    def read_pages(self, snapshot_file: int, pages):
        _check(library().psi_snapshot_read_pages(self._h, C.c_uint32(snapshot_file), pages._h))

    def read_table(self, snapshot_file: int, table):
        _check(library().psi_snapshot_read_table(self._h, C.c_uint32(snapshot_file), table._h))

    def read_full_buffer(self, snapshot_file: int, array):
        _check(library().psi_snapshot_read_host_buffer(self._h, C.c_uint32(snapshot_file), C.c_void_p(array.ctypes.data),
                                                       C.c_uint64(array.nbytes), None, C.c_uint64(0), C.c_uint64(0)))

    def read_selected_buffer(self, snapshot_file: int, array, entry_ranges, entry_bytes: int):
        ranges, n = _ranges(entry_ranges)
        _check(library().psi_snapshot_read_host_buffer(self._h, C.c_uint32(snapshot_file), C.c_void_p(array.ctypes.data),
                                                       C.c_uint64(array.nbytes), ranges, C.c_uint64(n),
                                                       C.c_uint64(entry_bytes)))

    def read_metadata(self, snapshot_file: int) -> bytes:
        out = C.create_string_buffer(1 << 20)
        n = C.c_uint64()
        _check(library().psi_snapshot_read_metadata(self._h, C.c_uint32(snapshot_file), out, C.c_uint64(len(out)),
                                                    C.byref(n)))
        return out.raw[:n.value]

    def finish(self):
        _check(library().psi_snapshot_reader_finish(self._h))


class U32IDAllocator:
    """Reference ``U32IDAllocator`` semantics: freed IDs first (oldest first), then fresh IDs."""

    def __init__(self, capacity: int):
        self.capacity = capacity
        self._h = C.c_void_p()
        _check(library().psi_id_allocator_create(C.c_uint64(capacity), C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            library().psi_id_allocator_destroy(self._h)
            self._h = None

    def alloc_many(self, count: int):
        out = (C.c_uint32 * max(count, 1))()
        _check(library().psi_id_allocator_alloc_many(self._h, C.c_uint64(count), out))
        return list(out[:count])

    def alloc_one(self) -> int:
        return self.alloc_many(1)[0]

    def free_many(self, ids):
        arr, n = _u32_array(ids)
        _check(library().psi_id_allocator_free_many(self._h, arr, C.c_uint64(n)))

    def free_one(self, page_id):
        self.free_many([page_id])

    def allocated_ids_bitmap(self):
        words = (self.capacity + 63) // 64
        out = (C.c_uint64 * max(words, 1))()
        n = C.c_uint64()
        _check(library().psi_id_allocator_bitmap(self._h, out, C.c_uint64(words), C.byref(n)))
        return [int(w) for w in out[:words]]

    def free(self) -> int:
        out = C.c_uint64()
        _check(library().psi_id_allocator_free_count(self._h, C.byref(out)))
        return out.value

    def used(self) -> int:
        return self.capacity - self.free()


class GQA:
    """The GQA component: metadata + KV append + split-KV attention (reference ``GQA`` + ``GQAMetadataBuffers``)."""

    def __init__(self, ctx: Context, config: GQAConfig):
        self.ctx, self.config = ctx, config
        self._h = C.c_void_p()
        _check(library().psi_gqa_create(ctx._h, C.byref(config), C.byref(self._h)), ctx._h)

    def close(self):
        if self._h:
            library().psi_gqa_destroy(self._h)
            self._h = C.c_void_p()

    def set_token_topology_boundaries(self, boundaries):
        arr, n = _u32_array(boundaries)
        _check(library().psi_gqa_set_token_topology_boundaries(self._h, arr, C.c_uint32(n)), self.ctx._h)

    def _prepare(self, req_slots, token_indices, cu_tokens, mode, caller_tokens=0) -> GQAReplayShape:
        rs, n = _u32_array(req_slots)
        ti, n2 = _u32_array(token_indices)
        cu, n3 = _u32_array(cu_tokens)
        if n != n2 or n3 != n + 1:
            raise PsiError(1, "req_slots, token_indices and cu_tokens lengths disagree")
        shape = GQAReplayShape()
        _check(library().psi_gqa_prepare(self._h, rs, ti, cu, C.c_uint32(n), C.c_uint32(mode),
                                         C.c_uint32(caller_tokens), C.byref(shape)), self.ctx._h)
        return shape

    def prepare(self, req_slots, token_indices, cu_tokens) -> GQAReplayShape:
        return self._prepare(req_slots, token_indices, cu_tokens, CAPACITY_EXACT)

    def prepare_bucketed(self, req_slots, token_indices, cu_tokens) -> GQAReplayShape:
        return self._prepare(req_slots, token_indices, cu_tokens, CAPACITY_BUCKETED)

    def prepare_bucketed_with_token_capacity(self, req_slots, token_indices, cu_tokens, num_total_tokens):
        return self._prepare(req_slots, token_indices, cu_tokens, CAPACITY_CALLER_TOKENS, num_total_tokens)

    def split_kv_variant(self) -> GQASplitKVVariant:
        v = GQASplitKVVariant()
        _check(library().psi_gqa_split_kv_variant(self._h, C.byref(v)), self.ctx._h)
        return v

    def metadata(self, which: int, offset: int, count: int):
        out = (C.c_uint32 * max(count, 1))()
        _check(library().psi_gqa_metadata_read(self._h, C.c_uint32(which), C.c_uint64(offset), out,
                                               C.c_uint64(count)), self.ctx._h)
        return list(out[:count])

    def write_metadata(self, which: int, offset: int, values):
        arr, n = _u32_array(values)
        _check(library().psi_gqa_metadata_write(self._h, C.c_uint32(which), C.c_uint64(offset), arr, C.c_uint64(n)),
               self.ctx._h)

    def plan_stats(self) -> dict:
        out = (C.c_uint32 * 12)()
        _check(library().psi_gqa_plan_stats(self._h, out, C.c_uint32(12)), self.ctx._h)
        keys = ("ctas", "items", "partial_slots", "reduce_units", "q_tiles", "kernel", "kv_tiles", "rows_per_tile",
                "chunk_ctas", "chunk_items", "chunk_tcgen05_launches", "chunk_mma_sync_launches")
        return dict(zip(keys, out))

    def kv_page_write(self, pages: PageArena, table: GQARequestPageTable, layer: int, k, v):
        _check(library().psi_gqa_kv_append(self._h, pages._h, table._h, C.c_uint32(layer), _ptr(k), _ptr(v)),
               self.ctx._h)

    def attend(self, pages: PageArena, table: GQARequestPageTable, layer: int, q, out):
        _check(library().psi_gqa_attend(self._h, pages._h, table._h, C.c_uint32(layer), _ptr(q), _ptr(out)),
               self.ctx._h)

    def append_attend(self, pages: PageArena, table: GQARequestPageTable, layer: int, k, v, q, out):
        """KV append and attention as one launch (same results as ``kv_page_write`` then ``attend``)."""
        _check(library().psi_gqa_append_attend(self._h, pages._h, table._h, C.c_uint32(layer), _ptr(k), _ptr(v),
                                               _ptr(q), _ptr(out)), self.ctx._h)

    def set_norm_rope(self, config: NormRopeConfig, q_norm_weight_bf16, k_norm_weight_bf16):
        """Fix the q / k RMSNorm + RoPE profile; weights are sequences of ``head_dim`` bf16 bit patterns."""
        qw, nq = (C.c_uint16 * len(q_norm_weight_bf16))(*[int(x) for x in q_norm_weight_bf16]), len(q_norm_weight_bf16)
        kw, nk = (C.c_uint16 * len(k_norm_weight_bf16))(*[int(x) for x in k_norm_weight_bf16]), len(k_norm_weight_bf16)
        if nq != self.config.head_dim or nk != self.config.head_dim:
            raise PsiError(1, "norm weights must hold head_dim values")
        _check(library().psi_gqa_set_norm_rope(self._h, C.byref(config), qw, kw), self.ctx._h)

    def norm_rope_append(self, pages, table, layer, q_in, k_in, v_in, q_out):
        """q norm/rope -> q_out, k norm/rope -> pages, v -> pages: the three stages before attention as one launch."""
        _check(library().psi_gqa_norm_rope_append(self._h, pages._h, table._h, C.c_uint32(layer), _ptr(q_in),
                                                  _ptr(k_in), _ptr(v_in), _ptr(q_out)), self.ctx._h)

    def projection_norm_rope_append(self, pages, table, layer, projection, gated, q_out, gates_out=None):
        """``norm_rope_append`` reading q, k, v (and the gates) in place from the fused projection output ``[T][width]``
        (GQAQGKVSplitKernel / GQAQKVSplitKernel layouts); ``gates_out`` receives the gate rows when ``gated``."""
        _check(library().psi_gqa_projection_norm_rope_append(
            self._h, pages._h, table._h, C.c_uint32(layer), _ptr(projection), C.c_uint32(1 if gated else 0),
            _ptr(q_out), _ptr(gates_out)), self.ctx._h)

    def attend_gated(self, pages, table, layer, q, gates, out):
        """Attention with ``out = attention * sigmoid(gates)`` fused into the epilogue."""
        _check(library().psi_gqa_attend_gated(self._h, pages._h, table._h, C.c_uint32(layer), _ptr(q), _ptr(gates),
                                              _ptr(out)), self.ctx._h)

    def attend_partial(self, pages, table, layer, q, o, m, l):
        _check(library().psi_gqa_attend_partial(self._h, pages._h, table._h, C.c_uint32(layer), _ptr(q), _ptr(o),
                                                _ptr(m), _ptr(l)), self.ctx._h)

    def reserve_replay(self):
        """Fix every offset, scratch size and launch grid for ``max_tokens`` so that captured graphs stay valid."""
        _check(library().psi_gqa_reserve_replay(self._h), self.ctx._h)

    def block_partial(self, q, local_k, local_v, num_tokens: int, block_size: int, o, m, l, slot_indices=None):
        """Dense bidirectional block attention partials (``GQABlockSDPAKernel``) in the ``attend_partial`` ABI."""
        _check(library().psi_gqa_block_partial(self._h, _ptr(q), _ptr(local_k), _ptr(local_v), C.c_uint32(num_tokens),
                                               C.c_uint32(block_size), _ptr(slot_indices), _ptr(o), _ptr(m), _ptr(l)),
               self.ctx._h)

    def combine(self, o_list, m_list, l_list, num_tokens, out):
        n = len(o_list)
        po = (C.c_void_p * n)(*[_ptr(x).value for x in o_list])
        pm = (C.c_void_p * n)(*[_ptr(x).value for x in m_list])
        pl = (C.c_void_p * n)(*[_ptr(x).value for x in l_list])
        _check(library().psi_gqa_combine(self._h, po, pm, pl, C.c_uint32(n), C.c_uint32(num_tokens), _ptr(out)),
               self.ctx._h)

    def signal(self, flag, value: int):
        """Release-store ``value`` to the u32 at device address ``flag`` after all earlier work of the stream."""
        _check(library().psi_gqa_signal(self._h, _ptr(flag), C.c_uint32(value)), self.ctx._h)

    def combine_wait(self, o_list, m_list, l_list, num_tokens, out, flags, flag_value: int, max_polls: int = 0):
        """``combine`` preceded by a bounded device-side wait until each of the n flags reached ``flag_value``."""
        n = len(o_list)
        po = (C.c_void_p * n)(*[_ptr(x).value for x in o_list])
        pm = (C.c_void_p * n)(*[_ptr(x).value for x in m_list])
        pl = (C.c_void_p * n)(*[_ptr(x).value for x in l_list])
        _check(library().psi_gqa_combine_wait(self._h, po, pm, pl, C.c_uint32(n), C.c_uint32(num_tokens), _ptr(out),
                                              _ptr(flags), C.c_uint32(flag_value), C.c_uint32(max_polls)), self.ctx._h)

    def attend_exchange(self, pages, table, layer, q, exchange: "KvExchange", out=None, k=None, v=None):
        """One rank's step of a KV-range exchange as one launch (``psi_gqa_attend_exchange``): the partial goes into
        the rank's slot on the owner, the flag is published, and on the owner the merged output lands in ``out``."""
        _check(library().psi_gqa_attend_exchange(self._h, pages._h, table._h, C.c_uint32(layer), _ptr(k), _ptr(v),
                                                 _ptr(q), C.byref(exchange), _ptr(out)), self.ctx._h)

    def device_status(self) -> int:
        """Waits for the stream; returns 0, or the status a bounded device-side wait recorded (4 = timeout)."""
        out = C.c_int32()
        _check(library().psi_gqa_device_status(self._h, C.byref(out)), self.ctx._h)
        return out.value

    def step_host(self, pages, table, layer, req_slots, token_indices, cu_tokens, k_host, v_host, q_host, out_host):
        """``prepare`` + ``decode_step_host`` in one call: q/k/v travel while the step is planned."""
        rs, n = _u32_array(req_slots)
        ti, _ = _u32_array(token_indices)
        cu, _ = _u32_array(cu_tokens)
        _check(library().psi_gqa_step_host(self._h, pages._h, table._h, C.c_uint32(layer), rs, ti, cu, C.c_uint32(n),
                                           _ptr(k_host), _ptr(v_host), _ptr(q_host), _ptr(out_host)), self.ctx._h)

    def decode_step_host(self, pages, table, layer, k_host, v_host, q_host, out_host):
        _check(library().psi_gqa_decode_step_host(self._h, pages._h, table._h, C.c_uint32(layer), _ptr(k_host),
                                                  _ptr(v_host), _ptr(q_host), _ptr(out_host)), self.ctx._h)

    def page_gather(self, pages, table, req_slot, layer, tok_begin, tok_end, k_out, v_out):
        _check(library().psi_page_gather(self._h, pages._h, table._h, C.c_uint32(req_slot), C.c_uint32(layer),
                                         C.c_uint32(tok_begin), C.c_uint32(tok_end), _ptr(k_out), _ptr(v_out)),
               self.ctx._h)


def attend_static(device, stream, config: GQAConfig, pages, page_table, req_slots, token_indices, cu_tokens, layer, q,
                  out):
    """Split-KV attention without any device allocation (``psi_gqa_attend_static``).

    For hosts that cannot call ``cudaMalloc`` while serving - all HBM already given to the KV arena, device memory
    owned by the host runtime's own pool, or a decode loop that cannot stall on an allocation.  The scratch is one
    fixed device array inside the library; ``pages`` and ``page_table`` are device addresses, the batch arrays are
    host lists as for :meth:`GQA.prepare`.  Calls on one device share that scratch, so keep them on one stream.
    Raises :class:`PsiError` with the library's message when the step exceeds the scratch limits.
    """
    rs, n = _u32_array(req_slots)
    ti, n2 = _u32_array(token_indices)
    cu, n3 = _u32_array(cu_tokens)
    if n != n2 or n3 != n + 1:
        raise PsiError(1, "req_slots, token_indices and cu_tokens lengths disagree")
    err = C.create_string_buffer(512)
    status = library().psi_gqa_attend_static(C.c_int32(device), C.c_void_p(int(stream or 0)), C.byref(config),
                                             _ptr(pages), _ptr(page_table), rs, ti, cu, C.c_uint32(n),
                                             C.c_uint32(layer), _ptr(q), _ptr(out), err, C.c_size_t(len(err)))
    if status:
        raise PsiError(status, err.value.decode("utf-8", "replace"))
