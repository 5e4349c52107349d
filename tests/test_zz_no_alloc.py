"""The split-K attention entry point that allocates nothing (scratch compiled into the library) must give the
same output as the entry point with a caller-owned workspace.  It exists for hosts that cannot call cudaMalloc
while serving (all memory already handed to the KV pool, or no tolerance for the allocator's device
synchronisation).  Collected last on purpose: it shares one scratch array across calls, and a failure here
should not hide the results of the other tests."""
import numpy as np
import pytest
import torch

import cases
from conftest import assert_close_bf16, bits_of, to_bf16, to_u32
from lfm25_inference_b200 import Lfm25Error, ops

pytestmark = pytest.mark.gpu


def upload(case, device):
    arena = ops.PagedKvArena(to_bf16(case["key_cache"], device), to_bf16(case["value_cache"], device))
    return ops.FastRaggedAttentionInput(
        query=to_bf16(case["query"], device), arena=arena, block_tables=to_u32(case["block_tables"], device),
        block_table_stride=case["block_tables"].shape[1], request_slots=to_u32(case["request_slots"], device),
        position_ids=to_u32(case["position_ids"], device))


def both_ways(case, splits, device):
    inputs = upload(case, device)
    tokens = inputs.query.shape[0]
    workspace = torch.empty((ops.splitk_workspace_elements(tokens),), dtype=torch.float32, device=device)
    expected = torch.zeros_like(inputs.query)
    ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, workspace, splits, expected)
    got = torch.zeros_like(inputs.query)
    ops.paged_ragged_attention_splitk_static_lfm2_bf16_into(inputs, splits, got)
    torch.cuda.synchronize()
    return bits_of(got), bits_of(expected)


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row(device):
    # first call: 33 sequences, 8 splits; second call right after: fewer tokens, fewer splits, so the array
    # still holds records of the first call that the second one must not pick up
    first = cases.random_ragged_case(31, 33, 16, 2048, 8192)
    got, expected = both_ways(first, 8, device)
    assert_close_bf16(got, expected, 2e-2, 1e-2)
    assert np.array_equal(got, expected)
    second = cases.splitk_case()
    got, expected = both_ways(second, 2, device)
    assert_close_bf16(got, expected, 2e-2, 1e-2)
    assert np.array_equal(got, expected)
    # and the first one again, to see that nothing depends on what the array held before
    got, expected = both_ways(first, 4, device)
    assert np.array_equal(got, expected)
    assert ops.device_status()[0] == 0


def test_static_scratch_limits(device):
    case = cases.splitk_case()
    inputs = upload(case, device)
    output = torch.zeros_like(inputs.query)
    with pytest.raises(Lfm25Error, match="2..=8 splits"):
        ops.paged_ragged_attention_splitk_static_lfm2_bf16_into(inputs, 1, output)
    too_many = 129
    big = ops.FastRaggedAttentionInput(
        query=torch.zeros((too_many, 32, 64), dtype=torch.bfloat16, device=device), arena=inputs.arena,
        block_tables=inputs.block_tables, block_table_stride=inputs.block_table_stride,
        request_slots=torch.zeros(too_many, dtype=torch.int32, device=device),
        position_ids=torch.zeros(too_many, dtype=torch.int32, device=device))
    with pytest.raises(Lfm25Error, match="at most 128 tokens"):
        ops.paged_ragged_attention_splitk_static_lfm2_bf16_into(big, 4, torch.zeros_like(big.query))


def test_token_without_result_keeps_its_output_row(device):
    """A valid call, then the same batch with one request slot outside the block tables (a documented no-op, not a
    fault: the CTAs of that token return after marking their records).  The other rows are bit-identical to the
    valid call, the row of the bad token keeps what the caller passed in -- not the first call's values, which the
    shared array still holds -- and no bounded wait has run out.  The entry point with a caller workspace behaves
    the same."""
    case = cases.random_ragged_case(32, 9, 16, 1024, 4096)
    inputs = upload(case, device)
    tokens = inputs.query.shape[0]
    good = torch.zeros_like(inputs.query)
    ops.paged_ragged_attention_splitk_static_lfm2_bf16_into(inputs, 4, good)
    bad_token = 4
    slots = case["request_slots"].copy()
    slots[bad_token] = case["block_tables"].shape[0] + 3
    broken = ops.FastRaggedAttentionInput(
        query=inputs.query, arena=inputs.arena, block_tables=inputs.block_tables,
        block_table_stride=inputs.block_table_stride, request_slots=to_u32(slots, device),
        position_ids=inputs.position_ids)
    sentinel = torch.full_like(inputs.query, 3.0)
    ops.paged_ragged_attention_splitk_static_lfm2_bf16_into(broken, 4, sentinel)
    workspace = torch.zeros((ops.splitk_workspace_elements(tokens),), dtype=torch.float32, device=device)
    with_workspace = torch.full_like(inputs.query, 3.0)
    ops.paged_ragged_attention_splitk_lfm2_bf16_into(broken, workspace, 4, with_workspace)
    torch.cuda.synchronize()
    good_bits, got_bits, workspace_bits = bits_of(good), bits_of(sentinel), bits_of(with_workspace)
    keep = np.arange(tokens) != bad_token
    assert np.array_equal(got_bits[keep], good_bits[keep])
    assert np.array_equal(got_bits[bad_token], bits_of(torch.full((32, 64), 3.0, dtype=torch.bfloat16)))
    assert np.array_equal(workspace_bits, got_bits)
    assert ops.device_status()[0] == 0
