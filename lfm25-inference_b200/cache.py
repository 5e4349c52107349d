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

    def pages_short(self, current_tokens, target_tokens) -> int:
        """Pages missing for growing all the given sequences together (0 = they fit); allocates nothing."""
        current = (ctypes.c_size_t * len(current_tokens))(*current_tokens)
        target = (ctypes.c_size_t * len(target_tokens))(*target_tokens)
        return _count(library().lfm25_kv_allocator_pages_short(self._handle, current, target, len(current_tokens)))

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

    def assign(self, estimated_tokens: int, prefix_hash: int | None = None, slack_tokens: int | None = None) -> int:
        """`slack_tokens`: the prefix's home replica may be at most this many outstanding tokens busier than the
        idlest replica, else the request spills to the idlest one (None = the home always takes it)."""
        if slack_tokens is None:
            replica = library().lfm25_dispatcher_assign(self._handle, prefix_hash or 0, int(prefix_hash is not None),
                                                        estimated_tokens)
        else:
            replica = library().lfm25_dispatcher_assign_bounded(self._handle, prefix_hash or 0,
                                                                int(prefix_hash is not None), estimated_tokens,
                                                                slack_tokens)
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


class PageRadixCache:
    """Reference: src/cache/radix.rs:61-287.  Host-only radix index over page-sized token blocks; a node may carry
    the slot of a convolution-state checkpoint."""

    def __init__(self, page_size: int, max_cached_pages: int):
        self._handle = ctypes.c_void_p()
        self.page_size = page_size
        check(library().lfm25_radix_cache_create(page_size, max_cached_pages, ctypes.byref(self._handle)))

    def _lookup(self, function, tokens, maximum_tokens: int):
        array = np.ascontiguousarray(tokens, dtype=np.uint32)
        capacity = max(1, array.size // self.page_size)
        pages = np.zeros(capacity, dtype=np.uint32)
        count = ctypes.c_size_t(0)
        slot = ctypes.c_uint32(0)
        matched = function(self._handle, _table_pointer(array), array.size, maximum_tokens, _table_pointer(pages),
                           capacity, ctypes.byref(count), ctypes.byref(slot))
        if matched < 0:
            check(int(matched))
        if matched == 0:
            return None
        return int(matched), int(slot.value), pages[:count.value].copy()

    def longest_checkpoint(self, tokens, maximum_tokens: int):
        """(matched tokens, checkpoint slot, physical pages) of the deepest checkpointed prefix, or None; counts a
        hit or a miss."""
        return self._lookup(library().lfm25_radix_cache_longest_checkpoint, tokens, maximum_tokens)

    def probe_checkpoint(self, tokens, maximum_tokens: int):
        """The same lookup without touching the admission statistics."""
        return self._lookup(library().lfm25_radix_cache_probe_checkpoint, tokens, maximum_tokens)

    def can_publish(self, tokens, prefix_tokens: int) -> bool:
        array = np.ascontiguousarray(tokens, dtype=np.uint32)
        return bool(library().lfm25_radix_cache_can_publish(self._handle, _table_pointer(array), array.size,
                                                            prefix_tokens))

    def insert_checkpoint(self, tokens, prefix_tokens: int, physical_pages, checkpoint_slot: int) -> np.ndarray:
        """Indexes the prefix; returns the physical pages that became owned by new nodes (to be pinned)."""
        array = np.ascontiguousarray(tokens, dtype=np.uint32)
        pages = np.ascontiguousarray(physical_pages, dtype=np.uint32)
        fresh = np.zeros(max(1, pages.size), dtype=np.uint32)
        created = library().lfm25_radix_cache_insert_checkpoint(
            self._handle, _table_pointer(array), array.size, prefix_tokens, _table_pointer(pages), pages.size,
            checkpoint_slot, _table_pointer(fresh))
        if created < 0:
            check(int(created))
        return fresh[:created].copy()

    def snapshot(self) -> dict:
        out = _abi.PrefixCacheSnapshot()
        library().lfm25_radix_cache_snapshot(self._handle, ctypes.byref(out))
        return {name: int(getattr(out, name)) for name, _ in out._fields_}

    def close(self) -> None:
        if self._handle:
            library().lfm25_radix_cache_destroy(self._handle)
            self._handle = None


class ConvCheckpointPool:
    """Reference: src/model/prefix.rs:15-129.  Device-resident snapshots of every convolution layer's state."""

    def __init__(self, convolution_layers: int, capacity: int, hidden_size: int = 2048, state_width: int = 2):
        self._handle = ctypes.c_void_p()
        check(library().lfm25_conv_checkpoints_create(convolution_layers, capacity, hidden_size, state_width,
                                                      ctypes.byref(self._handle)))

    def acquire(self):
        slot = library().lfm25_conv_checkpoints_acquire(self._handle)
        return None if slot < 0 else int(slot)

    def release(self, slot: int) -> None:
        library().lfm25_conv_checkpoints_release(self._handle, slot)

    def available(self) -> int:
        return int(library().lfm25_conv_checkpoints_available(self._handle))

    def capacity(self) -> int:
        return int(library().lfm25_conv_checkpoints_capacity(self._handle))

    def capture_layer(self, stream: int, checkpoint_slot: int, convolution_index: int, states, request_slot: int):
        check(library().lfm25_conv_checkpoints_capture_layer(self._handle, stream, checkpoint_slot,
                                                             convolution_index, states.data_ptr(), request_slot,
                                                             states.shape[0]))

    def restore_layer(self, stream: int, checkpoint_slot: int, convolution_index: int, states, request_slot: int):
        check(library().lfm25_conv_checkpoints_restore_layer(self._handle, stream, checkpoint_slot,
                                                             convolution_index, states.data_ptr(), request_slot,
                                                             states.shape[0]))

    def close(self) -> None:
        if self._handle:
            library().lfm25_conv_checkpoints_destroy(self._handle)
            self._handle = None


class HardwareCostModel:
    """Reference: src/scheduler/cost_model.rs:185-231.  Curves are lists of (batch, tokens, context, milliseconds)."""

    CURVES = {"decode_bf16": 0, "decode_fp8": 1, "prefill_bf16": 2}

    def __init__(self, decode_bf16, decode_fp8, prefill_bf16, page_size: int = 16):
        def points(values):
            return (_abi.CostPoint * len(values))(*[_abi.CostPoint(*value) for value in values])

        self._handle = ctypes.c_void_p()
        a, b, c = points(decode_bf16), points(decode_fp8), points(prefill_bf16)
        check(library().lfm25_cost_model_create(a, len(decode_bf16), b, len(decode_fp8), c, len(prefill_bf16),
                                                page_size, ctypes.byref(self._handle)))

    def predict(self, curve: str, batch: int, tokens: int, context: int) -> float:
        return float(library().lfm25_cost_model_predict(self._handle, self.CURVES[curve], batch, tokens, context))

    def predict_decode_ms(self, batch: int, maximum_context: int, fp8: bool) -> float:
        return float(library().lfm25_cost_model_predict_decode_ms(self._handle, batch, maximum_context, int(fp8)))

    def predict_prefill_ms(self, tokens: int) -> float:
        return float(library().lfm25_cost_model_predict_prefill_ms(self._handle, tokens))

    def close(self) -> None:
        if self._handle:
            library().lfm25_cost_model_destroy(self._handle)
            self._handle = None


def schedule(cost: HardwareCostModel, requests, now_us: int, step_budget_ms: float = 40.0,
             ttft_slo_us: int = 400_000, tpot_slo_us: int = 50_000, fp8_decode: bool = True,
             maximum_prefill_tokens: int = 512):
    """Scheduler::schedule (src/scheduler/planner.rs:80-236) with SchedulerConfig's defaults (:17-27).  `requests`:
    one dict per request slot with phase, prompt_len, prefilled, context_tokens, arrival_us,
    first_token_deadline_us, next_token_deadline_us.  Returns (work list of ("decode" | "prefill", slot, tokens),
    plan dict)."""
    views = (_abi.RequestView * max(1, len(requests)))()
    for index, request in enumerate(requests):
        views[index] = _abi.RequestView(request["phase"], request["prompt_len"], request["prefilled"],
                                        request["context_tokens"], request["arrival_us"],
                                        request["first_token_deadline_us"], request["next_token_deadline_us"])
    config = _abi.SchedulerConfig(step_budget_ms, ttft_slo_us, tpot_slo_us, int(fp8_decode), maximum_prefill_tokens)
    work = (_abi.ScheduledWork * max(1, len(requests)))()
    plan = _abi.BatchPlan()
    check(library().lfm25_schedule(cost._handle, ctypes.byref(config), views, len(requests), now_us, work,
                                   len(requests), ctypes.byref(plan)))
    items = [("decode" if work[i].kind == 0 else "prefill", int(work[i].slot), int(work[i].tokens))
             for i in range(plan.work_count)]
    return items, {"predicted_ms": float(plan.predicted_ms), "decode_count": int(plan.decode_count),
                   "prefill_tokens": int(plan.prefill_tokens)}
