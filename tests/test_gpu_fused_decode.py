"""The one-kernel decode (QK-norm + RoPE + paged KV append + attention in one launch, the reference's
kernels/attention_fused.cu path) must give exactly the bits of the two-kernel route (stand-alone append, then
attention) -- outputs and caches -- unsplit and split, and treat a token whose slot disagrees with its block table
as a no-op."""
import numpy as np
import pytest
import torch

from conftest import assert_within_oracle, bits_of, to_bf16, to_i64, to_u32
from lfm25_inference_b200 import ops, workloads
from oracle import oracle

pytestmark = pytest.mark.gpu


def build_case(seed, sequences, low, high, pages):
    rng = np.random.default_rng(seed)
    batch = workloads.ragged_decode_batch(seed, sequences, low, high, pages, 1)
    key_cache, value_cache = workloads.fill_pool_for_batch(rng, batch)
    return dict(
        batch=batch, key_cache=key_cache, value_cache=value_cache,
        query=workloads.bf16_normal(rng, (sequences, 32, 64)), key=workloads.bf16_normal(rng, (sequences, 8, 64)),
        value=workloads.bf16_normal(rng, (sequences, 8, 64)),
        query_norm=oracle.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(64)),
        key_norm=oracle.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(64)), inv_freq=oracle.rope_inv_freq(),
        positions=batch.positions(0), slots=batch.physical_slots(0))


def run_two_kernels(case, device, splits):
    arena = ops.PagedKvArena(to_bf16(case["key_cache"], device), to_bf16(case["value_cache"], device))
    query = to_bf16(case["query"], device)
    ops.qk_norm_rope_kv_write_arena_decode_bf16(
        query, to_bf16(case["key"], device), to_bf16(case["value"], device), to_bf16(case["query_norm"], device),
        to_bf16(case["key_norm"], device), torch.from_numpy(case["inv_freq"]).to(device),
        to_u32(case["positions"], device), to_i64(case["slots"], device), arena, 1e-5)
    batch = case["batch"]
    inputs = ops.FastRaggedAttentionInput(query, arena, to_u32(batch.block_tables, device), batch.stride,
                                          to_u32(batch.request_slots, device), to_u32(case["positions"], device))
    output = torch.zeros_like(query)
    if splits > 1:
        partials = torch.empty(ops.splitk_workspace_elements(query.shape[0]), dtype=torch.float32, device=device)
        ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, partials, splits, output)
    else:
        ops.paged_ragged_attention_fast_lfm2_bf16_into(inputs, output)
    return bits_of(output), bits_of(arena.key), bits_of(arena.value), bits_of(query)


def run_fused(case, device, splits, slots=None, sentinel=None, packed=False, in_kernel_merge=False):
    arena = ops.PagedKvArena(to_bf16(case["key_cache"], device), to_bf16(case["value_cache"], device))
    query = to_bf16(case["query"], device)
    key, value = to_bf16(case["key"], device), to_bf16(case["value"], device)
    if packed:
        # the three projections as columns of one [N, 3072] buffer (what a packed q|k|v GEMM writes)
        tokens = query.shape[0]
        rows = torch.cat([query.reshape(tokens, -1), key.reshape(tokens, -1), value.reshape(tokens, -1)], dim=1)
        query = rows[:, :2048].unflatten(1, (32, 64))
        key = rows[:, 2048:2560].unflatten(1, (8, 64))
        value = rows[:, 2560:].unflatten(1, (8, 64))
    batch = case["batch"]
    output = torch.zeros_like(query)
    if sentinel is not None:
        output = torch.zeros(query.shape, dtype=torch.int16, device=device).fill_(sentinel).view(torch.bfloat16)
    partials = None if in_kernel_merge else \
        torch.empty(ops.splitk_workspace_elements(query.shape[0]), dtype=torch.float32, device=device)
    ops.fused_ragged_paged_attention_decode_lfm2_bf16_into(
        query, key, value, to_bf16(case["query_norm"], device),
        to_bf16(case["key_norm"], device), torch.from_numpy(case["inv_freq"]).to(device),
        to_u32(case["positions"], device), to_i64(case["slots"] if slots is None else slots, device), arena,
        to_u32(batch.block_tables, device), batch.stride, to_u32(batch.request_slots, device), 1e-5, output,
        partials=partials, num_splits=splits)
    assert np.array_equal(bits_of(query.contiguous()), case["query"])          # the raw query is not modified
    return bits_of(output), bits_of(arena.key), bits_of(arena.value)


@pytest.mark.parametrize("splits", [1, 2, 4, 8])
@pytest.mark.parametrize("seed,sequences,low,high,pages", [(21, 7, 0, 90, 128), (22, 33, 16, 2048, 8192),
                                                           (23, 128, 128, 4096, 32768)])
def test_fused_equals_two_kernel_route(device, seed, sequences, low, high, pages, splits):
    case = build_case(seed, sequences, low, high, pages)
    want_output, want_key, want_value, rotated_query = run_two_kernels(case, device, splits)
    got_output, got_key, got_value = run_fused(case, device, splits)
    assert np.array_equal(got_key, want_key) and np.array_equal(got_value, want_value)
    assert np.array_equal(got_output, want_output)
    assert ops.device_status()[0] == 0
    if sequences <= 33 and splits == 1:
        # and both agree with the oracle run on the appended cache and the rotated query
        _, exact = oracle.paged_ragged_attention(rotated_query, want_key, want_value, case["batch"].block_tables,
                                                 case["batch"].request_slots, case["positions"], want_exact=True)
        assert_within_oracle(got_output, exact)


@pytest.mark.parametrize("splits", [2, 4, 8])
@pytest.mark.parametrize("packed", [False, True])
def test_fused_with_the_merge_inside_the_kernel(device, splits, packed):
    """No workspace: the splits of a token are one cluster and merge through distributed shared memory.  Output and
    the appended cache rows are bit-identical to the route through records and the merge kernel."""
    case = build_case(25, 41, 3, 3000, 8192)
    want = run_fused(case, device, splits, packed=packed)
    got = run_fused(case, device, splits, packed=packed, in_kernel_merge=True)
    for a, b in zip(got, want):
        assert np.array_equal(a, b)
    assert ops.device_status()[0] == 0


@pytest.mark.parametrize("splits", [1, 4])
def test_token_strided_projections(device, splits):
    """q | k | v side by side in one [N, 3072] buffer give the bits of the dense call."""
    case = build_case(24, 19, 5, 700, 1024)
    dense = run_fused(case, device, splits)
    packed = run_fused(case, device, splits, packed=True)
    for a, b in zip(packed, dense):
        assert np.array_equal(a, b)
    assert ops.device_status()[0] == 0


def test_context_of_one_token(device):
    # position 0: the only key is the row the kernel has just produced; it never reads it back from the cache
    case = build_case(31, 4, 0, 0, 16)
    want = run_two_kernels(case, device, 1)
    got = run_fused(case, device, 1)
    for a, b in zip(got, want[:3]):
        assert np.array_equal(a, b)


def test_slot_that_disagrees_with_the_block_table_is_a_no_op(device):
    # kernels/attention_fused.cu:131-147
    case = build_case(41, 5, 20, 300, 256)
    slots = case["slots"].copy()
    slots[1] = -1
    slots[3] += 1                                                 # right page, wrong offset (or the next page)
    sentinel = 0x1234
    output, key, value = run_fused(case, device, 1, slots=slots, sentinel=sentinel)
    want_output, want_key, want_value, _ = run_two_kernels(case, device, 1)
    for token in range(5):
        page, offset = divmod(int(case["slots"][token]), 16)
        if token in (1, 3):
            assert np.all(output[token] == sentinel)
            assert np.array_equal(key[page, :, offset, :], case["key_cache"][page, :, offset, :])
        else:
            assert np.array_equal(output[token], want_output[token])
            assert np.array_equal(key[page, :, offset, :], want_key[page, :, offset, :])
            assert np.array_equal(value[page, :, offset, :], want_value[page, :, offset, :])
