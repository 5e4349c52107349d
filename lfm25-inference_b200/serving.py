"""Continuous-batching serving loop over the C ABI: admission with prefix reuse, step planning, mixed prefill /
decode steps, token bookkeeping.

Mirror of the reference's owner loop (src/engine/serving/radix_owner.rs:101-437 with admit_request_radix :549-708,
split_prefill_at_reusable_boundary :526-547 and the publication of page-aligned prefixes :305-322): one engine owns
one GPU's request slots, page allocator, block tables, radix index, convolution checkpoints and executor.  All
policy and bookkeeping live in the library (allocator, radix index, planner, cost curves); this module only wires them
together and moves the step metadata.  Sampling is greedy; the model is whatever `RandomModel` the caller built.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _abi, cache, ops, workloads
from . import model as lfm_model

PAGE = 16


@dataclass
class Request:
    request_id: int
    prompt: np.ndarray               # uint32
    max_new_tokens: int
    arrival_us: int


@dataclass
class SlotState:
    """SequenceRequest of the reference (src/scheduler/request.rs:42-53) plus the response bookkeeping."""

    phase: int = _abi.PHASE_FREE
    request: Request | None = None
    tokens: list = field(default_factory=list)
    prompt_len: int = 0
    prefilled: int = 0
    cached_tokens: int = 0           # tokens whose KV is in the cache (prefilled prompt + decoded tokens)
    reserved_pages: int = 0
    first_token_deadline_us: int = 0
    next_token_deadline_us: int = 0
    first_token_us: int | None = None
    token_times_us: list = field(default_factory=list)
    reused_tokens: int = 0


class ServingEngine:
    def __init__(self, model: lfm_model.RandomModel, device, max_slots: int = 64, max_sequence_tokens: int = 8704,
                 max_prefill_tokens: int = 512, radix_pages: int = 4096, checkpoint_capacity: int = 64,
                 use_fp8: bool = True, ttft_slo_us: int = 400_000, tpot_slo_us: int = 50_000,
                 step_budget_ms: float = 40.0):
        self.model, self.device, self.use_fp8 = model, device, use_fp8
        self.max_slots, self.max_prefill_tokens = max_slots, max_prefill_tokens
        self.ttft_slo_us, self.tpot_slo_us, self.step_budget_ms = ttft_slo_us, tpot_slo_us, step_budget_ms
        assert model.num_request_slots >= max_slots
        self.pages_per_slot = (max_sequence_tokens + PAGE - 1) // PAGE
        self.allocator = cache.KvPageAllocator(model.num_pages)
        self.tables = cache.FixedBlockTables(max_slots, self.pages_per_slot)
        self.radix = cache.PageRadixCache(PAGE, radix_pages)
        self.conv_layers = [layer for layer in model.layers if not layer.is_attention]
        self.checkpoints = cache.ConvCheckpointPool(len(self.conv_layers), checkpoint_capacity)
        self.slots = [SlotState() for _ in range(max_slots)]
        self.free_slots = list(range(max_slots - 1, -1, -1))
        self.queue: list[Request] = []
        self.cost: cache.HardwareCostModel | None = None
        self.blaslt = ops.BlasLt()
        self.max_tokens = max_slots + max_prefill_tokens
        self.executor = lfm_model.DecodeExecutor(self.blaslt, self.max_tokens, maximum_segments=max_slots)
        # fixed device buffers of the step metadata and their pinned staging area
        def device_u32(count):
            return torch.zeros(count, dtype=torch.int32, device=device)
        self.d_token_ids, self.d_positions = device_u32(self.max_tokens), device_u32(self.max_tokens)
        self.d_request_slots = device_u32(self.max_tokens)
        self.d_physical_slots = torch.zeros(self.max_tokens, dtype=torch.int64, device=device)
        self.d_segment_offsets, self.d_segment_slots = device_u32(max_slots + 1), device_u32(max_slots)
        self.d_output_rows = device_u32(max_slots)
        self.d_tables = torch.full((max_slots, self.pages_per_slot), -1, dtype=torch.int32, device=device)
        self.h_meta = torch.zeros(3 * self.max_tokens + 3 * max_slots + 1, dtype=torch.int32).pin_memory()
        self.h_sampled = torch.zeros(max_slots, dtype=torch.int32).pin_memory()
        self.finished: list[dict] = []
        self.tables_dirty = True          # host block tables changed since the last upload
        self.stats = {"steps": 0, "mixed_steps": 0, "decode_steps": 0, "generated": 0, "prefill_tokens": 0,
                      "reused_tokens": 0, "gpu_ms": 0.0}

    # ------------------------------------------------------------------------------------------ calibration

    def calibrate(self) -> None:
        """Measures the cost curves the planner uses (the reference reads them from a hardware profile file,
        src/scheduler/cost_model.rs:198-216): decode steps at a few (batch, context) points and prefill chunks of
        the planner's sizes, on scratch sequences that are released again."""
        decode_points, prefill_points = [], []
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def timed(batch, token_count):
            ids = np.zeros(token_count, dtype=np.uint32)
            self._run_step(batch, ids)                                     # warm-up (plans, attributes)
            start.record()
            self._run_step(batch, ids)
            stop.record()
            stop.synchronize()
            return start.elapsed_time(stop)

        contexts = [context for context in (512, 2048) if context + 1 <= self.pages_per_slot * PAGE]
        for context in contexts:
            for sequences in sorted({1, min(8, self.max_slots), min(32, self.max_slots), self.max_slots}):
                pages = (context + 1 + PAGE - 1) // PAGE
                if sequences * pages > self.model.num_pages:
                    continue
                table = np.full((self.max_slots, self.pages_per_slot), 0xFFFFFFFF, dtype=np.uint32)
                for slot in range(sequences):
                    table[slot, :pages] = np.arange(slot * pages, (slot + 1) * pages)
                batch = workloads.MixedStepBatch(self.model.num_pages, table, np.full(sequences, context),
                                                 np.ones(sequences, dtype=np.int64),
                                                 np.arange(sequences, dtype=np.uint32))
                self._upload_tables(table)
                decode_points.append((sequences, 1, context, timed(batch, sequences)))
        for chunk in (16, 64, 128, 256, 512):
            if chunk > self.max_prefill_tokens:
                continue
            table = np.full((self.max_slots, self.pages_per_slot), 0xFFFFFFFF, dtype=np.uint32)
            pages = (chunk + PAGE - 1) // PAGE
            table[0, :pages] = np.arange(pages)
            batch = workloads.MixedStepBatch(self.model.num_pages, table, np.array([0]), np.array([chunk]),
                                             np.zeros(1, dtype=np.uint32))
            self._upload_tables(table)
            prefill_points.append((1, chunk, chunk, timed(batch, chunk)))
        self.tables_dirty = True
        for layer in self.conv_layers:
            layer.tensors["conv_state"].zero_()
        self.cost = cache.HardwareCostModel(decode_points, decode_points, prefill_points)
        self.calibration = {"decode": decode_points, "prefill": prefill_points}

    # ------------------------------------------------------------------------------------------ admission

    def submit(self, request: Request) -> None:
        self.queue.append(request)

    def _admit(self, now_us: int) -> None:
        """admit_request_radix: a free slot, the longest reusable checkpointed prefix (at most the last full page
        before the final prompt token, so that the forward pass still produces logits), page reservation for the
        rest of the sequence, convolution state restored from the checkpoint or cleared."""
        while self.queue and self.free_slots:
            request = self.queue[0]
            total_tokens = len(request.prompt) + request.max_new_tokens
            if total_tokens > self.pages_per_slot * PAGE:
                raise ValueError("request exceeds the engine's maximum sequence length")
            reusable_limit = (len(request.prompt) - 1) // PAGE * PAGE
            hit = self.radix.probe_checkpoint(request.prompt, reusable_limit) if reusable_limit else None
            matched = hit[0] if hit else 0
            needed_pages = (total_tokens + PAGE - 1) // PAGE - matched // PAGE
            try:
                self.allocator.try_reserve_pages(needed_pages)
            except cache.KvAllocationError:
                return                                                 # back-pressure: keep the queue order
            self.queue.pop(0)
            self.tables_dirty = True
            slot = self.free_slots.pop()
            state = self.slots[slot]
            row = self.tables.slot(slot)
            row[:] = 0xFFFFFFFF
            stream = torch.cuda.current_stream().cuda_stream
            if hit:
                matched, checkpoint_slot, pages = self.radix.longest_checkpoint(request.prompt, reusable_limit)
                self.allocator.retain_pages(pages)
                row[:len(pages)] = pages
                for index, layer in enumerate(self.conv_layers):
                    self.checkpoints.restore_layer(stream, checkpoint_slot, index, layer.tensors["conv_state"], slot)
            else:
                if reusable_limit:
                    self.radix.longest_checkpoint(request.prompt, reusable_limit)   # counts the miss
                for layer in self.conv_layers:
                    layer.tensors["conv_state"][slot].zero_()
            state.phase = _abi.PHASE_QUEUED_PREFILL
            state.request = request
            state.tokens = [int(token) for token in request.prompt]
            state.prompt_len = len(request.prompt)
            state.prefilled = matched
            state.cached_tokens = matched
            state.reused_tokens = matched
            state.reserved_pages = needed_pages
            state.first_token_deadline_us = request.arrival_us + self.ttft_slo_us
            state.next_token_deadline_us = request.arrival_us + self.tpot_slo_us
            state.first_token_us = None
            state.token_times_us = []
            self.stats["reused_tokens"] += matched

    # ------------------------------------------------------------------------------------------ one step

    def _views(self):
        return [dict(phase=state.phase, prompt_len=state.prompt_len, prefilled=state.prefilled,
                     context_tokens=len(state.tokens),
                     arrival_us=state.request.arrival_us if state.request else 0,
                     first_token_deadline_us=state.first_token_deadline_us,
                     next_token_deadline_us=state.next_token_deadline_us) for state in self.slots]

    def _upload_tables(self, table: np.ndarray) -> None:
        self.d_tables.copy_(torch.from_numpy(np.ascontiguousarray(table).view(np.int32)), non_blocking=False)

    def _run_step(self, batch: workloads.MixedStepBatch, token_ids: np.ndarray) -> None:
        """Uploads the step metadata from pinned memory and enqueues the step."""
        tokens, segments = batch.num_tokens, batch.num_segments
        meta = self.h_meta.numpy().view(np.uint32)
        cursor = 0
        pieces = []
        for values, target in ((token_ids, self.d_token_ids), (batch.positions, self.d_positions),
                               (batch.request_slots, self.d_request_slots),
                               (batch.segment_offsets, self.d_segment_offsets),
                               (batch.segment_slots, self.d_segment_slots), (batch.output_rows, self.d_output_rows)):
            count = len(values)
            meta[cursor:cursor + count] = values
            pieces.append((cursor, count, target))
            cursor += count
        for begin, count, target in pieces:
            target[:count].copy_(self.h_meta[begin:begin + count], non_blocking=True)
        struct = _abi.RaggedBatch(
            self.d_token_ids.data_ptr(), self.d_positions.data_ptr(), self.d_request_slots.data_ptr(),
            self.d_physical_slots.data_ptr(), self.d_segment_offsets.data_ptr(), self.d_segment_slots.data_ptr(),
            self.d_output_rows.data_ptr(), self.d_tables.data_ptr(), self.pages_per_slot, self.max_slots, tokens,
            segments, *lfm_model.leading_decode_segments(batch))
        self.blaslt.bind_current_stream()
        if segments == tokens:
            # pure decode: the decode executor's path (fused append + attention, split-K policy)
            decode = _abi.DecodeBatch(
                self.d_token_ids.data_ptr(), self.d_positions.data_ptr(), self.d_request_slots.data_ptr(),
                self.d_physical_slots.data_ptr(), self.d_tables.data_ptr(), self.pages_per_slot, self.max_slots,
                tokens, int(batch.positions.max()) + 1)
            _abi.check(_abi.library().lfm25_decode_executor_forward(self.executor._handle, self.model.struct, decode,
                                                                    int(self.use_fp8), 0))
        else:
            _abi.check(_abi.library().lfm25_decode_executor_forward_ragged(self.executor._handle, self.model.struct,
                                                                           struct, int(self.use_fp8)))

    def step(self, now_us: int):
        """Admits, plans and runs one step.  Returns (events, gpu_ms): events are (request_id, token, finished)."""
        if self.cost is None:
            raise RuntimeError("calibrate() (or a cost model) is needed before the first step")
        self._admit(now_us)
        work, _ = cache.schedule(self.cost, self._views(), now_us, step_budget_ms=self.step_budget_ms,
                                 ttft_slo_us=self.ttft_slo_us, tpot_slo_us=self.tpot_slo_us,
                                 fp8_decode=self.use_fp8, maximum_prefill_tokens=self.max_prefill_tokens)
        if not work:
            return [], 0.0
        prefixes, chunks, segment_slots, token_ids = [], [], [], []
        for kind, slot, count in work:
            state = self.slots[slot]
            if kind == "prefill":
                # split_prefill_at_reusable_boundary: end the chunk at the last full page before the final prompt
                # token, so that the prefix published there can serve a later identical prompt
                reusable_limit = (state.prompt_len - 1) // PAGE * PAGE
                if reusable_limit and state.prefilled < reusable_limit < state.prefilled + count:
                    count = reusable_limit - state.prefilled
                begin = state.prefilled
                token_ids.extend(state.tokens[begin:begin + count])
            else:
                begin = len(state.tokens) - 1
                token_ids.append(state.tokens[-1])
                count = 1
            if self.allocator.grow_sequence(state.cached_tokens, begin + count, self.tables.slot(slot)) > 0:
                self.tables_dirty = True
            prefixes.append(begin)
            chunks.append(count)
            segment_slots.append(slot)
        if self.tables_dirty:
            self._upload_tables(self.tables.as_array())
            self.tables_dirty = False
        batch = workloads.MixedStepBatch(self.model.num_pages, self.tables.as_array(), np.array(prefixes),
                                         np.array(chunks), np.array(segment_slots, dtype=np.uint32))
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        self._run_step(batch, np.array(token_ids, dtype=np.uint32))
        stop.record()
        self.executor.download_sampled(self.h_sampled)
        stream = torch.cuda.current_stream()
        stream.synchronize()
        gpu_ms = start.elapsed_time(stop)
        sampled = self.h_sampled.numpy().view(np.uint32)
        done_us = now_us + int(gpu_ms * 1000)

        events = []
        self.stats["steps"] += 1
        self.stats["mixed_steps" if batch.num_segments != batch.num_tokens else "decode_steps"] += 1
        self.stats["gpu_ms"] += gpu_ms
        for row_index, ((kind, slot, _), count) in enumerate(zip(work, chunks)):
            state = self.slots[slot]
            state.cached_tokens = prefixes[row_index] + count
            if kind == "prefill":
                state.prefilled += count
                self.stats["prefill_tokens"] += count
                if state.prefilled % PAGE == 0:
                    self._publish(slot, state)
                if state.prefilled < state.prompt_len:
                    continue
            token = int(sampled[row_index])
            state.tokens.append(token)
            state.phase = _abi.PHASE_DECODING
            state.next_token_deadline_us = done_us + self.tpot_slo_us
            state.token_times_us.append(done_us)
            if state.first_token_us is None:
                state.first_token_us = done_us
            self.stats["generated"] += 1
            generated = len(state.tokens) - state.prompt_len
            finished = generated >= state.request.max_new_tokens
            events.append((state.request.request_id, token, finished))
            if finished:
                self._release(slot, state)
        return events, gpu_ms

    def _publish(self, slot: int, state: SlotState) -> None:
        """publish_prefix_checkpoint: index the page-aligned prefix and snapshot the convolution states that go
        with it, when the radix budget and a checkpoint slot allow."""
        prompt = np.asarray(state.tokens[:state.prompt_len], dtype=np.uint32)
        if not self.radix.can_publish(prompt, state.prefilled):
            return
        checkpoint = self.checkpoints.acquire()
        if checkpoint is None:
            return
        stream = torch.cuda.current_stream().cuda_stream
        for index, layer in enumerate(self.conv_layers):
            self.checkpoints.capture_layer(stream, checkpoint, index, layer.tensors["conv_state"], slot)
        pages = self.tables.slot(slot)[:state.prefilled // PAGE].copy()
        self.allocator.pin_cached_pages(self.radix.insert_checkpoint(prompt, state.prefilled, pages, checkpoint))

    def _release(self, slot: int, state: SlotState) -> None:
        self.finished.append(state_summary(state))
        row = self.tables.slot(slot)
        # BatchModelCache::release (src/model/lfm2_base.rs:262-277): the pages go back (shared ones only lose a
        # reference) and the whole logical reservation of the request is returned
        self.allocator.release_sequence(state.cached_tokens, row)
        self.allocator.release_reservation(state.reserved_pages)
        row[:] = 0xFFFFFFFF
        self.slots[slot] = SlotState()
        self.free_slots.append(slot)

    def active(self) -> int:
        return sum(1 for state in self.slots if state.phase != _abi.PHASE_FREE)

    def close(self) -> None:
        self.executor.close()
        self.blaslt.close()
        self.checkpoints.close()
        self.radix.close()


def state_summary(state: SlotState) -> dict:
    times = state.token_times_us
    gaps = np.diff(times) if len(times) > 1 else np.array([])
    return {"request_id": state.request.request_id, "prompt_len": state.prompt_len,
            "generated": len(state.tokens) - state.prompt_len, "reused_tokens": state.reused_tokens,
            "ttft_us": state.first_token_us - state.request.arrival_us,
            "tpot_us": float(gaps.mean()) if gaps.size else 0.0, "tokens": state.tokens[state.prompt_len:]}


def run_trace(engine: ServingEngine, requests: list[Request], realtime: bool = True) -> dict:
    """Drives the engine over a list of requests ordered by arrival time.  The clock is the wall clock of this
    process since the call (`realtime`), jumped forward to the next arrival whenever the engine is idle."""
    engine.finished = []
    pending = sorted(requests, key=lambda request: request.arrival_us)
    origin = time.perf_counter()
    skipped_us = 0
    cursor = 0
    idle_rounds = 0
    while cursor < len(pending) or engine.queue or engine.active():
        now_us = int((time.perf_counter() - origin) * 1e6) + skipped_us
        if not engine.queue and not engine.active() and cursor < len(pending) and pending[cursor].arrival_us > now_us:
            skipped_us += pending[cursor].arrival_us - now_us          # idle: jump to the next arrival
            now_us = pending[cursor].arrival_us
        while cursor < len(pending) and pending[cursor].arrival_us <= now_us:
            engine.submit(pending[cursor])
            cursor += 1
        events, _ = engine.step(now_us)
        idle_rounds = 0 if (events or engine.active()) else idle_rounds + 1
        if idle_rounds > 1000:
            raise RuntimeError("the engine makes no progress: a queued request does not fit the page pool")
    makespan_us = int((time.perf_counter() - origin) * 1e6) + skipped_us
    return {"makespan_us": makespan_us, "wall_s": time.perf_counter() - origin, "requests": engine.finished,
            "stats": dict(engine.stats), "prefix_cache": engine.radix.snapshot()}
