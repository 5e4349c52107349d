"""Seeded synthetic inputs for the benchmark configurations and the parity tests.

Everything is generated with numpy from an explicit seed and kept as raw bit patterns (bf16 as
uint16), so the CPU oracle and the GPU kernels see identical bytes.  No dataset is involved: the
shapes, sizes and value distributions follow the decode workloads the library is measured on.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

PAGE_SIZE = 16
Q_HEADS = 32
KV_HEADS = 8
HEAD_DIM = 64


def f32_to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit patterns."""
    array = np.ascontiguousarray(values, dtype=np.float32)
    bits = array.view(np.uint32)
    with np.errstate(over="ignore"):
        rounded = ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
    nan = (bits & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    if nan.any():
        rounded[nan] = 0x7FFF
    return rounded.reshape(array.shape)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    array = np.ascontiguousarray(bits, dtype=np.uint16)
    return (array.astype(np.uint32) << 16).view(np.float32).reshape(array.shape)


def bf16_normal(rng: np.random.Generator, shape, std: float = 1.0) -> np.ndarray:
    return f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


def patterned_bf16(elements: int, mul: int, modulus: int, center: float, scale: float) -> np.ndarray:
    """bf16(((i * mul) % modulus - center) / scale): the patterned tensors of the reference's attention tests
    (src/ops/attention_async_fast_tests.rs:21-25)."""
    index = np.arange(elements, dtype=np.int64)
    values = ((index * mul) % modulus).astype(np.float32)
    return f32_to_bf16_bits((values - np.float32(center)) / np.float32(scale))


@dataclass
class RaggedDecodeBatch:
    """A decode batch over a paged pool: one new token per sequence per step."""

    num_pages: int
    block_tables: np.ndarray      # uint32 [sequences, stride], 0xffffffff = unassigned
    contexts: np.ndarray          # int64 [sequences]: tokens already cached before the first step
    request_slots: np.ndarray     # uint32 [sequences]

    @property
    def num_sequences(self) -> int:
        return int(self.contexts.shape[0])

    @property
    def stride(self) -> int:
        return int(self.block_tables.shape[1])

    def positions(self, step: int) -> np.ndarray:
        """Index of the token appended at `step` (0-based) = context length before it."""
        return (self.contexts + step).astype(np.uint32)

    def physical_slots(self, step: int) -> np.ndarray:
        positions = self.positions(step).astype(np.int64)
        pages = self.block_tables[np.arange(self.num_sequences), positions // PAGE_SIZE].astype(np.int64)
        return pages * PAGE_SIZE + positions % PAGE_SIZE

    def kv_bytes(self, step: int) -> int:
        """Algorithmic KV bytes read by attention at `step`: 2048 B per valid key."""
        return int(((self.contexts + step + 1) * (KV_HEADS * HEAD_DIM * 2 * 2)).sum())


def ragged_decode_batch(seed: int, num_sequences: int, context_low: int, context_high: int, num_pages: int,
                        steps: int) -> RaggedDecodeBatch:
    """Contexts uniform in [low, high]; block tables are consecutive slices of one seeded shuffle of the pool."""
    rng = np.random.default_rng(seed)
    contexts = rng.integers(context_low, context_high + 1, size=num_sequences, dtype=np.int64)
    pages_needed = (contexts + steps + PAGE_SIZE - 1) // PAGE_SIZE
    stride = int((context_high + steps + PAGE_SIZE - 1) // PAGE_SIZE)
    if int(pages_needed.sum()) > num_pages:
        raise ValueError("page pool too small for the batch")
    shuffle = rng.permutation(num_pages).astype(np.uint32)
    tables = np.full((num_sequences, stride), 0xFFFFFFFF, dtype=np.uint32)
    cursor = 0
    for sequence in range(num_sequences):
        count = int(pages_needed[sequence])
        tables[sequence, :count] = shuffle[cursor:cursor + count]
        cursor += count
    return RaggedDecodeBatch(num_pages, tables, contexts, np.arange(num_sequences, dtype=np.uint32))


def single_step_c0(seed: int = 0):
    """Batch 1, context 40 after the append (39 cached + 1 new), 3 pages drawn from a 64-page pool."""
    rng = np.random.default_rng(seed)
    table = rng.permutation(64).astype(np.uint32)[:3].reshape(1, 3)
    cached_key = bf16_normal(rng, (39, KV_HEADS, HEAD_DIM))
    cached_value = bf16_normal(rng, (39, KV_HEADS, HEAD_DIM))
    new_key = bf16_normal(rng, (1, KV_HEADS, HEAD_DIM))
    new_value = bf16_normal(rng, (1, KV_HEADS, HEAD_DIM))
    query = bf16_normal(rng, (1, Q_HEADS, HEAD_DIM))
    positions = np.arange(39, dtype=np.int64)
    cached_slots = table[0, positions // PAGE_SIZE].astype(np.int64) * PAGE_SIZE + positions % PAGE_SIZE
    new_slot = np.array([int(table[0, 2]) * PAGE_SIZE + 7], dtype=np.int64)
    return {
        "num_pages": 64, "block_table": table, "cached_key": cached_key, "cached_value": cached_value,
        "cached_slots": cached_slots, "new_key": new_key, "new_value": new_value, "new_slot": new_slot,
        "query": query, "position": np.array([39], dtype=np.uint32), "request_slot": np.array([0], dtype=np.uint32),
    }


def fill_pool_for_batch(rng: np.random.Generator, batch: RaggedDecodeBatch):
    """K and V pools [pages, 8, 16, 64] (bf16 bits), N(0,1) in every page a sequence owns, zero elsewhere."""
    shape = (batch.num_pages, KV_HEADS, PAGE_SIZE, HEAD_DIM)
    key = np.zeros(shape, dtype=np.uint16)
    value = np.zeros(shape, dtype=np.uint16)
    owned = batch.block_tables[batch.block_tables != 0xFFFFFFFF].astype(np.int64)
    key[owned] = bf16_normal(rng, (owned.size, KV_HEADS, PAGE_SIZE, HEAD_DIM))
    value[owned] = bf16_normal(rng, (owned.size, KV_HEADS, PAGE_SIZE, HEAD_DIM))
    return key, value


@dataclass
class MixedStepBatch:
    """One step that mixes prefill chunks and decode tokens: segment s holds `chunks[s]` consecutive tokens of the
    sequence in request slot `segment_slots[s]`, whose first `prefixes[s]` tokens are already in the paged cache
    (a decode token is a segment of one token)."""

    num_pages: int
    block_tables: np.ndarray      # uint32 [request slots, stride], 0xffffffff = unassigned
    prefixes: np.ndarray          # int64 [segments]
    chunks: np.ndarray            # int64 [segments]
    segment_slots: np.ndarray     # uint32 [segments]

    @property
    def num_segments(self) -> int:
        return int(self.chunks.shape[0])

    @property
    def num_tokens(self) -> int:
        return int(self.chunks.sum())

    @property
    def stride(self) -> int:
        return int(self.block_tables.shape[1])

    @property
    def segment_offsets(self) -> np.ndarray:
        return np.concatenate([[0], np.cumsum(self.chunks)]).astype(np.uint32)

    @property
    def request_slots(self) -> np.ndarray:
        return np.repeat(self.segment_slots, self.chunks).astype(np.uint32)

    @property
    def positions(self) -> np.ndarray:
        return np.concatenate([prefix + np.arange(chunk) for prefix, chunk in zip(self.prefixes, self.chunks)]).astype(
            np.uint32)

    @property
    def physical_slots(self) -> np.ndarray:
        positions = self.positions.astype(np.int64)
        pages = self.block_tables[self.request_slots.astype(np.int64), positions // PAGE_SIZE].astype(np.int64)
        return pages * PAGE_SIZE + positions % PAGE_SIZE

    @property
    def output_rows(self) -> np.ndarray:
        """Row of each segment's last token: the rows whose logits a serving step needs."""
        return (np.cumsum(self.chunks) - 1).astype(np.uint32)


def mixed_step_batch(seed: int, prefixes, chunks, num_pages: int, shuffle_slots: bool = True) -> MixedStepBatch:
    """Block tables are consecutive slices of one seeded shuffle of the pool, sized for prefix + chunk tokens; the
    request slots are a seeded permutation of 0..segments-1 unless `shuffle_slots` is off."""
    rng = np.random.default_rng(seed)
    prefixes = np.asarray(prefixes, dtype=np.int64)
    chunks = np.asarray(chunks, dtype=np.int64)
    pages_needed = (prefixes + chunks + PAGE_SIZE - 1) // PAGE_SIZE
    if int(pages_needed.sum()) > num_pages:
        raise ValueError("page pool too small for the batch")
    stride = int(pages_needed.max())
    shuffle = rng.permutation(num_pages).astype(np.uint32)
    slots = rng.permutation(len(chunks)).astype(np.uint32) if shuffle_slots else np.arange(len(chunks),
                                                                                         dtype=np.uint32)
    tables = np.full((len(chunks), stride), 0xFFFFFFFF, dtype=np.uint32)
    cursor = 0
    for segment, slot in enumerate(slots):
        count = int(pages_needed[segment])
        tables[slot, :count] = shuffle[cursor:cursor + count]
        cursor += count
    return MixedStepBatch(num_pages, tables, prefixes, chunks, slots)


def fill_prefixes(rng: np.random.Generator, batch: MixedStepBatch):
    """K and V pools [pages, 8, 16, 64] (bf16 bits) with N(0,1) in the first `prefix` token rows of every segment's
    sequence; rows at and beyond the prefix hold a NaN pattern (0x7fc1), so that a kernel that reads a row it
    must not read shows up in the result."""
    shape = (batch.num_pages, KV_HEADS, PAGE_SIZE, HEAD_DIM)
    key = np.full(shape, 0x7FC1, dtype=np.uint16)
    value = np.full(shape, 0x7FC1, dtype=np.uint16)
    for segment in range(batch.num_segments):
        prefix = int(batch.prefixes[segment])
        if prefix == 0:
            continue
        positions = np.arange(prefix)
        pages = batch.block_tables[int(batch.segment_slots[segment]), positions // PAGE_SIZE].astype(np.int64)
        offsets = positions % PAGE_SIZE
        key[pages, :, offsets, :] = bf16_normal(rng, (prefix, KV_HEADS, HEAD_DIM))
        value[pages, :, offsets, :] = bf16_normal(rng, (prefix, KV_HEADS, HEAD_DIM))
    return key, value
