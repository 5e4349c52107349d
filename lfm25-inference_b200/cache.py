"""Host-side cache bookkeeping, named after the reference's ``src/cache``: the physical page allocator and the
fixed per-slot block tables, plus the decode scheduler and the replica dispatcher.  All state lives in the C++
library (``csrc/host_runtime.cu``); these classes only hold the handles."""
from __future__ import annotations

import ctypes

import numpy as np

from . import _abi
from ._abi import check, library


class KvAllocationError(RuntimeError):
    """`KvAllocationError` of the reference (src/cache/allocator.rs:7-24)."""

    MESSAGES = {_abi.KV_PHYSICAL_PAGES_EXHAUSTED: "physical KV pages exhausted",
                _abi.KV_LOGICAL_RESERVATION_EXHAUSTED: "logical KV reservation exhausted",
                _abi.KV_SEQUENCE_CAPACITY_EXCEEDED: "sequence block table capacity exceeded"}

    def __init__(self, code: int):
        super().__init__(self.MESSAGES.get(code, f"KV allocation error {code}"))
        self.code = code


def _count(value: int) -> int:
    if value < 0:
        raise KvAllocationError(int(value))
    return int(value)


def _table_pointer(table: np.ndarray):
    assert table.dtype == np.uint32 and table.flags["C_CONTIGUOUS"]
    return table.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))


class KvPageAllocator:
    """Reference: src/cache/allocator.rs:40-229."""

    def __init__(self, total_pages: int, page_size: int = 16):
        self._handle = ctypes.c_void_p()
        check(library().lfm25_kv_allocator_create(total_pages, page_size, ctypes.byref(self._handle)))

    def try_reserve_tokens(self, maximum_tokens: int) -> int:
        return _count(library().lfm25_kv_allocator_try_reserve_tokens(self._handle, maximum_tokens))

    def try_reserve_pages(self, pages: int) -> int:
        return _count(library().lfm25_kv_allocator_try_reserve_pages(self._handle, pages))

    def release_reservation(self, pages: int) -> None:
        library().lfm25_kv_allocator_release_reservation(self._handle, pages)

    def pin_cached_pages(self, pages) -> None:
        array = np.ascontiguousarray(pages, dtype=np.uint32)
        _count(library().lfm25_kv_allocator_pin_cached_pages(self._handle, _table_pointer(array), array.size))

    def retain_pages(self, pages) -> None:
        array = np.ascontiguousarray(pages, dtype=np.uint32)
        _count(library().lfm25_kv_allocator_retain_pages(self._handle, _table_pointer(array), array.size))

    def grow_sequence(self, current_tokens: int, target_tokens: int, block_table: np.ndarray) -> int:
        return _count(library().lfm25_kv_allocator_grow_sequence(self._handle, current_tokens, target_tokens,
                                                                 _table_pointer(block_table), block_table.size))

    def release_sequence(self, tokens: int, block_table: np.ndarray) -> None:
        library().lfm25_kv_allocator_release_sequence(self._handle, tokens, _table_pointer(block_table),
                                                      block_table.size)

    def snapshot(self) -> dict:
        snapshot = _abi.KvPoolSnapshot()
        library().lfm25_kv_allocator_snapshot(self._handle, ctypes.byref(snapshot))
        return {name: int(getattr(snapshot, name)) for name, _ in _abi.KvPoolSnapshot._fields_}

    def __del__(self):
        if getattr(self, "_handle", None):
            library().lfm25_kv_allocator_destroy(self._handle)
            self._handle = None


class FixedBlockTables:
    """Reference: src/cache/block_table.rs:3-31.  `slot(i)` is a live numpy view of row i."""

    def __init__(self, slots: int, pages_per_slot: int):
        self._handle = ctypes.c_void_p()
        check(library().lfm25_block_tables_create(slots, pages_per_slot, ctypes.byref(self._handle)))
        self.slots = slots
        self.pages_per_slot = pages_per_slot

    def slot(self, slot: int) -> np.ndarray:
        pointer = library().lfm25_block_tables_slot(self._handle, slot)
        if not pointer:
            raise _abi.Lfm25Error(_abi.ERR_INVALID_ARGUMENT, library().lfm25_last_error().decode())
        return np.ctypeslib.as_array(pointer, shape=(self.pages_per_slot,))

    def as_array(self) -> np.ndarray:
        pointer = library().lfm25_block_tables_data(self._handle)
        return np.ctypeslib.as_array(pointer, shape=(self.slots, self.pages_per_slot))

    def __del__(self):
        if getattr(self, "_handle", None):
            library().lfm25_block_tables_destroy(self._handle)
            self._handle = None


def schedule_decode(phases, next_token_deadline_us, context_tokens, now_us: int):
    """Decode half of Scheduler::schedule (src/scheduler/planner.rs:80-113): (slots in deadline order, longest context)."""
    phases = np.ascontiguousarray(phases, dtype=np.uint32)
    deadlines = np.ascontiguousarray(next_token_deadline_us, dtype=np.uint64)
    contexts = np.ascontiguousarray(context_tokens, dtype=np.uint32)
    out = np.zeros(phases.size, dtype=np.uint32)
    maximum = ctypes.c_size_t()
    count = library().lfm25_schedule_decode(
        phases.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), deadlines.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)),
        contexts.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), phases.size, now_us,
        out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), ctypes.byref(maximum))
    return out[:count].copy(), int(maximum.value)


class Dispatcher:
    """Least-loaded dispatch of whole requests over engine replicas with prefix-hash affinity."""

    def __init__(self, replicas: int):
        self._handle = ctypes.c_void_p()
        check(library().lfm25_dispatcher_create(replicas, ctypes.byref(self._handle)))

    def assign(self, estimated_tokens: int, prefix_hash: int | None = None) -> int:
        replica = library().lfm25_dispatcher_assign(self._handle, prefix_hash or 0, int(prefix_hash is not None),
                                                    estimated_tokens)
        check(min(replica, 0))
        return int(replica)

    def complete(self, replica: int, tokens: int) -> None:
        library().lfm25_dispatcher_complete(self._handle, replica, tokens)

    def mark_failed(self, replica: int) -> None:
        library().lfm25_dispatcher_mark_failed(self._handle, replica)

    def load(self, replica: int) -> int:
        return int(library().lfm25_dispatcher_load(self._handle, replica))

    def __del__(self):
        if getattr(self, "_handle", None):
            library().lfm25_dispatcher_destroy(self._handle)
            self._handle = None
