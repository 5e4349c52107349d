"""Parity of the paged KV append kernels (C ABI) with the CPU oracle and the reference's kernels.
Raw append and V copies are bit-exact; the fused QK-norm + RoPE append is bit-exact against the
reference's kernel and within one bf16 step of the CPU oracle (whose sincosf is the host's)."""
import numpy as np
import pytest
import torch

import cases
from conftest import bits_of, to_bf16, to_i64, to_u32
from lfm25_inference_b200 import ops, workloads
from oracle import oracle, refkernels

pytestmark = pytest.mark.gpu


def test_raw_write_layout(device):
    # src/cuda/kernels/tests/kv_cache.rs:13-66
    source = (np.arange(3 * 8 * 64, dtype=np.uint32) ^ 0x5A5A).astype(np.uint16).reshape(3, 8, 64)
    slots = np.array([0, -1, 16 * 2 + 3], dtype=np.int64)
    arena = ops.PagedKvArena.new(3, device=device)
    arena.write_lfm2(to_bf16(source, device), to_bf16(source, device), to_i64(slots, device))
    key_cache, value_cache = cases.write_cache(source, source, slots, 3)
    assert np.array_equal(bits_of(arena.key), key_cache) and np.array_equal(bits_of(arena.value), value_cache)


@pytest.mark.parametrize("tokens,pages", [(1, 1), (64, 4096), (513, 64), (4096, 300)])
def test_raw_write_random(device, tokens, pages):
    rng = np.random.default_rng(tokens)
    key = workloads.bf16_normal(rng, (tokens, 8, 64))
    value = workloads.bf16_normal(rng, (tokens, 8, 64))
    slots = rng.permutation(pages * 16)[:tokens].astype(np.int64) if tokens <= pages * 16 else None
    if slots is None:
        slots = rng.integers(0, pages * 16, size=tokens).astype(np.int64)
        _, first = np.unique(slots, return_index=True)
        duplicate = np.ones(tokens, dtype=bool)
        duplicate[first] = False
        slots[duplicate] = -1            # keep the write set race-free
    slots[::7] = np.where(np.arange(tokens)[::7] % 2 == 0, slots[::7], pages * 16 + 5)  # some beyond the pool
    arena = ops.PagedKvArena.new(pages, device=device)
    arena.write_lfm2(to_bf16(key, device), to_bf16(value, device), to_i64(slots, device))
    key_cache, value_cache = cases.write_cache(key, value, slots, pages)
    assert np.array_equal(bits_of(arena.key), key_cache) and np.array_equal(bits_of(arena.value), value_cache)
    if refkernels.available():
        ref_key = torch.zeros_like(arena.key)
        ref_value = torch.zeros_like(arena.value)
        refkernels.kv_cache_write(to_bf16(key, device), to_bf16(value, device), ref_key, ref_value,
                                  to_i64(slots, device))
        assert torch.equal(ref_key, arena.key) and torch.equal(ref_value, arena.value)


def run_fused(case, device, function):
    query = to_bf16(case["query"], device)
    arena = ops.PagedKvArena.new(case["num_pages"], device=device)
    function(query, to_bf16(case["key"], device), to_bf16(case["value"], device), to_bf16(case["query_norm"], device),
             to_bf16(case["key_norm"], device), torch.from_numpy(case["inv_freq"]).to(device),
             to_u32(case["position_ids"], device), to_i64(case["slot_mapping"], device), arena, case["eps"])
    return bits_of(query), bits_of(arena.key), bits_of(arena.value)


def ulp_distance(a_bits, b_bits):
    def ordered(bits):
        signed = bits.astype(np.int32)
        return np.where(signed & 0x8000, 0x8000 - signed, signed)
    return np.abs(ordered(a_bits) - ordered(b_bits))


@pytest.mark.parametrize("seed,tokens", [(11, 6), (12, 1), (13, 5)])
def test_fused_qk_norm_rope_append(device, seed, tokens):
    case = cases.qk_postprocess_case(seed, tokens)
    query, key_cache, value_cache = run_fused(case, device, ops.qk_norm_rope_kv_write_arena_decode_bf16)
    want_query = case["query"].copy()
    want_key = np.zeros((case["num_pages"], 8, 16, 64), dtype=np.uint16)
    want_value = np.zeros_like(want_key)
    oracle.qk_norm_rope_kv_write_decode(want_query, case["key"], case["value"], case["query_norm"], case["key_norm"],
                                        case["inv_freq"], case["position_ids"], case["slot_mapping"], want_key,
                                        want_value, case["eps"])
    assert np.array_equal(value_cache, want_value)                       # V: bit copy
    assert ulp_distance(query, want_query).max() <= 1
    assert ulp_distance(key_cache, want_key).max() <= 1
    assert (query != want_query).mean() < 0.01 and (key_cache != want_key).mean() < 0.01
    if refkernels.available():
        def reference(query_t, key, value, qn, kn, inv_freq, positions, slots, arena, eps):
            refkernels.qk_norm_rope_kv_write_decode(query_t, key, value, qn, kn, inv_freq, positions, slots,
                                                    arena.key, arena.value, eps)
        ref_query, ref_key, ref_value = run_fused(case, device, reference)
        assert np.array_equal(query, ref_query) and np.array_equal(key_cache, ref_key)
        assert np.array_equal(value_cache, ref_value)


def test_fused_append_large_batch_against_reference_kernel(device):
    if not refkernels.available():
        pytest.skip("reference kernels were not compiled")
    rng = np.random.default_rng(3)
    tokens, pages = 128, 4096
    batch = workloads.ragged_decode_batch(3, tokens, 128, 4096, pages * 16, 1)
    case = dict(query=workloads.bf16_normal(rng, (tokens, 32, 64)), key=workloads.bf16_normal(rng, (tokens, 8, 64)),
                value=workloads.bf16_normal(rng, (tokens, 8, 64)),
                query_norm=oracle.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(64)),
                key_norm=oracle.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(64)), inv_freq=oracle.rope_inv_freq(),
                position_ids=batch.positions(0), slot_mapping=batch.physical_slots(0), num_pages=pages * 16, eps=1e-5)

    def reference(query_t, key, value, qn, kn, inv_freq, positions, slots, arena, eps):
        refkernels.qk_norm_rope_kv_write_decode(query_t, key, value, qn, kn, inv_freq, positions, slots, arena.key,
                                                arena.value, eps)
    ours = run_fused(case, device, ops.qk_norm_rope_kv_write_arena_decode_bf16)
    theirs = run_fused(case, device, reference)
    for got, want in zip(ours, theirs):
        assert np.array_equal(got, want)
