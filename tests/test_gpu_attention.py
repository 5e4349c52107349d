"""Parity of the CUDA decode-attention path (through the C ABI) with the CPU oracle and, where the
reference's kernels were compiled, with the reference's own kernels on the same device buffers.

Tolerance against the fp64 oracle: |y - y*| <= 2e-2 + 1e-2 |y*| and cosine >= 0.9999.
Against the reference's kernels: the bounds the reference's own tests use (0.035/0.025 unsplit,
0.04/0.03 split-K; src/ops/attention_async_fast_tests.rs:58-63, attention_splitk_tests.rs:111-116)."""
import numpy as np
import pytest
import torch

import cases
from conftest import assert_close_bf16, assert_within_oracle, bits_of, to_bf16, to_u32
from lfm25_inference_b200 import Lfm25Error, ops, workloads
from oracle import oracle, refkernels

pytestmark = pytest.mark.gpu


def upload(case, device):
    arena = ops.PagedKvArena(to_bf16(case["key_cache"], device), to_bf16(case["value_cache"], device))
    return ops.FastRaggedAttentionInput(
        query=to_bf16(case["query"], device), arena=arena, block_tables=to_u32(case["block_tables"], device),
        block_table_stride=case["block_tables"].shape[1], request_slots=to_u32(case["request_slots"], device),
        position_ids=to_u32(case["position_ids"], device))


def oracle_exact(case):
    return oracle.paged_ragged_attention(case["query"], case["key_cache"], case["value_cache"], case["block_tables"],
                                         case["request_slots"], case["position_ids"], want_exact=True)


def reference_precise(inputs):
    output = torch.zeros_like(inputs.query)
    refkernels.paged_ragged_attention_precise(inputs.query, inputs.arena.key, inputs.arena.value, inputs.block_tables,
                                              inputs.request_slots, inputs.position_ids, output)
    return bits_of(output)


def run_all_variants(case, device, split_counts=(2, 4, 8)):
    """unsplit + every split count, each checked against the oracle (and the reference kernel when present)."""
    inputs = upload(case, device)
    _, exact = oracle_exact(case)
    reference = reference_precise(inputs) if refkernels.available() else None
    output = ops.paged_ragged_attention_fast_lfm2_bf16(inputs)
    assert_within_oracle(bits_of(output), exact)
    if reference is not None:
        assert_close_bf16(bits_of(output), reference, 0.035, 0.025)
    tokens = case["query"].shape[0]
    partials = torch.full((ops.splitk_workspace_elements(tokens),), float("nan"), dtype=torch.float32, device=device)
    for splits in split_counts:
        split_output = torch.zeros_like(inputs.query)
        ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, partials, splits, split_output)
        assert_within_oracle(bits_of(split_output), exact)
        if reference is not None:
            assert_close_bf16(bits_of(split_output), reference, 0.04, 0.03)
    assert ops.device_status()[0] == 0
    return inputs, exact


@pytest.mark.parametrize("context", cases.SINGLE_CONTEXTS)
def test_single_sequence_contexts(device, context):
    case = cases.single_context_case(context)
    inputs, exact = run_all_variants(case, device)
    # the one-sequence entry point (block-table row 0 for every token)
    output = torch.zeros_like(inputs.query)
    ops.paged_attention_fast_lfm2_bf16_into(inputs.query, inputs.arena.key, inputs.arena.value,
                                            inputs.block_tables.reshape(-1), inputs.position_ids, output)
    assert_within_oracle(bits_of(output), exact)


def test_ragged_reversed_page_order(device):
    run_all_variants(cases.ragged_reversed_case(), device)


def test_splitk_lengths_257_65(device):
    case = cases.splitk_case()
    inputs, _ = run_all_variants(case, device)
    # partial records: same layout and convention as the reference's (max, denominator, acc[64])
    for splits in (2, 8):
        partials = torch.full((2, 32, splits, 66), float("nan"), dtype=torch.float32, device=device)
        output = torch.zeros_like(inputs.query)
        ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, partials, splits, output)
        got = partials.cpu().numpy()
        want = oracle.splitk_partials(case["query"], case["key_cache"], case["value_cache"], case["block_tables"],
                                      case["request_slots"], case["position_ids"], splits)
        empty = want[..., 1] == 0
        assert np.array_equal(got[..., 1] == 0, empty)
        assert np.all(np.isneginf(got[..., 0][empty])) and not got[..., 2:][empty].any()
        live = ~empty
        # max is exact up to fp32 summation order; weights are rounded to bf16 before the sum -> 2^-8 relative
        assert np.allclose(got[..., 0][live], want[..., 0][live], atol=1e-4, rtol=0)
        assert np.allclose(got[..., 1][live], want[..., 1][live], rtol=1e-2)
        assert np.allclose(got[..., 2:][live], want[..., 2:][live], atol=3e-2, rtol=1e-2)
        # the oracle's merge of this library's records against its merge of its own records: same identity, so the
        # bound is the one between the records
        assert_close_bf16(oracle.merge_splitk(got), oracle.merge_splitk(want), 3e-2, 1e-2)
        assert_close_bf16(bits_of(output), oracle.merge_splitk(got), 1e-6, 2 ** -7)


def test_block_table_selection_is_exact(device):
    # src/ops/attention_regression_tests.rs:19-61: Q = K = 0, context 1 -> output is exactly V of the request's page
    values = np.zeros((2, 8, 64), dtype=np.float32)
    for token in range(2):
        for head in range(8):
            values[token, head] = token * 100 + head * 2 + np.arange(64) / 64.0
    value = oracle.f32_to_bf16(values)
    key_cache, value_cache = cases.write_cache(np.zeros((2, 8, 64), dtype=np.uint16), value, [0, 16], 2)
    case = dict(query=np.zeros((2, 32, 64), dtype=np.uint16), key_cache=key_cache, value_cache=value_cache,
                block_tables=np.array([[0], [1]], dtype=np.uint32), request_slots=np.array([0, 1], dtype=np.uint32),
                position_ids=np.zeros(2, dtype=np.uint32))
    output = ops.paged_ragged_attention_fast_lfm2_bf16(upload(case, device))
    assert np.array_equal(bits_of(output), np.repeat(value, 4, axis=1))


def test_config0_single_step(device):
    # batch 1, 3 pages of a 64-page pool, context 40 after appending one token
    c0 = workloads.single_step_c0(0)
    arena = ops.PagedKvArena.new(64, device=device)
    arena.write_lfm2(to_bf16(c0["cached_key"], device), to_bf16(c0["cached_value"], device),
                     torch.from_numpy(c0["cached_slots"]).to(device))
    arena.write_lfm2(to_bf16(c0["new_key"], device), to_bf16(c0["new_value"], device),
                     torch.from_numpy(c0["new_slot"]).to(device))
    key_cache, value_cache = cases.write_cache(c0["cached_key"], c0["cached_value"], c0["cached_slots"], 64)
    oracle.kv_cache_write(c0["new_key"], c0["new_value"], key_cache, value_cache, c0["new_slot"])
    assert np.array_equal(bits_of(arena.key), key_cache) and np.array_equal(bits_of(arena.value), value_cache)
    case = dict(query=c0["query"], key_cache=key_cache, value_cache=value_cache, block_tables=c0["block_table"],
                request_slots=c0["request_slot"], position_ids=c0["position"])
    run_all_variants(case, device)


@pytest.mark.parametrize("seed,sequences,low,high,pages", [(7, 6, 1, 700, 512), (8, 33, 16, 2048, 8192),
                                                           (9, 3, 4000, 8192, 2048)])
def test_random_ragged_batches(device, seed, sequences, low, high, pages):
    run_all_variants(cases.random_ragged_case(seed, sequences, low, high, pages), device, split_counts=(2, 3, 5, 8))


def test_invalid_indices_leave_output_untouched(device):
    # kernels/attention_async_fast.cu:88-111,149-151: bad request slot / position / page -> that token is a no-op
    case = cases.splitk_case()
    sentinel = 0x1234
    for mutate, dead in (
        (lambda c: c.update(request_slots=np.array([0, 7], dtype=np.uint32)), 1),
        (lambda c: c.update(position_ids=np.array([17 * 16, 64], dtype=np.uint32)), 0),
        (lambda c: c["block_tables"].__setitem__((1, 2), 0xFFFFFFFF), 1),
        (lambda c: c["block_tables"].__setitem__((0, 16), 19), 0),  # page 19 of a 22-page pool is valid...
    ):
        mutated = {name: array.copy() for name, array in case.items()}
        mutate(mutated)
        inputs = upload(mutated, device)
        expected = oracle.paged_ragged_attention(mutated["query"], mutated["key_cache"], mutated["value_cache"],
                                                 mutated["block_tables"], mutated["request_slots"],
                                                 mutated["position_ids"],
                                                 output=np.full((2, 32, 64), sentinel, dtype=np.uint16))
        for splits in (1, 4):
            output = torch.full((2, 32, 64), 0, dtype=torch.int16, device=device).fill_(sentinel).view(torch.bfloat16)
            if splits == 1:
                ops.paged_ragged_attention_fast_lfm2_bf16_into(inputs, output)
            else:
                partials = torch.zeros((2 * 32 * splits * 66,), dtype=torch.float32, device=device)
                ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, partials, splits, output)
            got = bits_of(output)
            untouched = np.all(expected.reshape(2, -1) == sentinel, axis=1)
            if splits == 1:
                assert np.array_equal(np.all(got.reshape(2, -1) == sentinel, axis=1), untouched)
            live = ~untouched
            assert_close_bf16(got[live], expected[live], 2e-2, 1e-2)
    assert ops.device_status()[0] == 0


def test_stale_bits_beyond_the_position_are_ignored(device):
    # the last page is fetched whole; NaN/Inf patterns after the newest token must not reach the output
    case = cases.single_context_case(19)
    poisoned = {name: array.copy() for name, array in case.items()}
    poisoned["key_cache"][1, :, 3:, :] = 0x7FC0
    poisoned["value_cache"][1, :, 3:, :] = 0x7F80
    clean = bits_of(ops.paged_ragged_attention_fast_lfm2_bf16(upload(case, device)))
    dirty = bits_of(ops.paged_ragged_attention_fast_lfm2_bf16(upload(poisoned, device)))
    assert np.array_equal(clean, dirty)


def test_op_layer_shape_checks(device):
    case = cases.single_context_case(17)
    inputs = upload(case, device)
    with pytest.raises(Lfm25Error, match="must have shape"):
        bad = ops.FastRaggedAttentionInput(inputs.query.reshape(1, 64, 32), inputs.arena, inputs.block_tables, 2,
                                           inputs.request_slots, inputs.position_ids)
        ops.paged_ragged_attention_fast_lfm2_bf16(bad)
    with pytest.raises(Lfm25Error, match="stride/shape mismatch"):
        bad = ops.FastRaggedAttentionInput(inputs.query, inputs.arena, inputs.block_tables, 3, inputs.request_slots,
                                           inputs.position_ids)
        ops.paged_ragged_attention_fast_lfm2_bf16(bad)
    with pytest.raises(Lfm25Error, match="2..=8 splits"):
        ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, torch.zeros(32 * 9 * 66, device=device), 9,
                                                         torch.zeros_like(inputs.query))


def test_full_size_ragged_batch_properties(device):
    """BASELINE config 1 at full size: 64 sequences, contexts in [16, 8192], 2^16-page pool.  Checked through
    size-independent properties: split-K at every count agrees with the unsplit result, a permutation of the
    physical pages leaves the result unchanged, and a sample of tokens matches the oracle."""
    batch = workloads.ragged_decode_batch(1, 64, 16, 8192, 1 << 16, 16)
    generator = torch.Generator(device=device).manual_seed(1)
    shape = (1 << 16, 8, 16, 64)
    arena = ops.PagedKvArena(torch.randn(shape, generator=generator, device=device, dtype=torch.bfloat16),
                             torch.randn(shape, generator=generator, device=device, dtype=torch.bfloat16))
    query = torch.randn((64, 32, 64), generator=generator, device=device, dtype=torch.bfloat16)
    inputs = ops.FastRaggedAttentionInput(query, arena, to_u32(batch.block_tables, device), batch.stride,
                                          to_u32(batch.request_slots, device), to_u32(batch.positions(0), device))
    unsplit = bits_of(ops.paged_ragged_attention_fast_lfm2_bf16(inputs))
    partials = torch.empty((ops.splitk_workspace_elements(64),), dtype=torch.float32, device=device)
    for splits in (2, 4, 8):
        output = torch.zeros_like(query)
        ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, partials, splits, output)
        assert_close_bf16(bits_of(output), unsplit, 4e-3, 2 ** -6)
    # oracle on 3 sequences (shortest, longest, one more), pool pages copied to the host on demand
    order = np.argsort(batch.contexts)
    for sequence in (int(order[0]), int(order[-1]), int(order[31])):
        pages = batch.block_tables[sequence]
        owned = pages[pages != 0xFFFFFFFF].astype(np.int64)
        index = torch.from_numpy(owned).to(device)
        sub_case = dict(query=bits_of(query[sequence:sequence + 1]), key_cache=bits_of(arena.key[index]),
                        value_cache=bits_of(arena.value[index]),
                        block_tables=np.arange(owned.size, dtype=np.uint32).reshape(1, -1),
                        request_slots=np.zeros(1, dtype=np.uint32),
                        position_ids=batch.positions(0)[sequence:sequence + 1])
        _, exact = oracle_exact(sub_case)
        assert_within_oracle(unsplit[sequence], exact[0])
    # relabel the physical pages: move every page to a new place and rewrite the tables accordingly
    permutation = torch.randperm(1 << 16, generator=generator, device=device)
    moved = ops.PagedKvArena(torch.empty_like(arena.key), torch.empty_like(arena.value))
    moved.key[permutation] = arena.key
    moved.value[permutation] = arena.value
    tables = torch.from_numpy(batch.block_tables.astype(np.int64)).to(device)
    valid = tables != 0xFFFFFFFF
    tables[valid] = permutation[tables[valid]]
    moved_inputs = ops.FastRaggedAttentionInput(query, moved, tables.to(torch.int32), batch.stride,
                                                inputs.request_slots, inputs.position_ids)
    assert np.array_equal(bits_of(ops.paged_ragged_attention_fast_lfm2_bf16(moved_inputs)), unsplit)
    assert ops.device_status()[0] == 0


def test_context_order_is_a_stable_descending_sort(device):
    rng = np.random.default_rng(31)
    for count in (1, 2, 64, 257, 2048):
        positions = rng.integers(0, 50, size=count).astype(np.uint32)        # many ties
        order = torch.full((count,), 0x7fffffff, dtype=torch.int32, device=device)
        ops.context_order_desc_into(to_u32(positions, device), order)
        want = np.argsort(-positions.astype(np.int64), kind="stable")
        assert np.array_equal(order.cpu().numpy(), want)
    with pytest.raises(Lfm25Error):
        ops.context_order_desc_into(torch.zeros(2049, dtype=torch.int32, device=device),
                                    torch.zeros(2049, dtype=torch.int32, device=device))


def test_token_order_changes_no_result(device):
    """The optional token order only changes which CTA takes which token: outputs are bit-identical for the
    longest-first order, for a random permutation, and without one; an entry outside the batch is a no-op."""
    case = cases.random_ragged_case(12, 37, 5, 1500, 8192)
    inputs = upload(case, device)
    tokens = case["query"].shape[0]
    plain = bits_of(ops.paged_ragged_attention_fast_lfm2_bf16(inputs))
    longest_first = torch.zeros(tokens, dtype=torch.int32, device=device)
    ops.context_order_desc_into(inputs.position_ids, longest_first)
    shuffled = to_u32(np.random.default_rng(12).permutation(tokens).astype(np.uint32), device)
    partials = torch.empty((ops.splitk_workspace_elements(tokens),), dtype=torch.float32, device=device)
    plain_split = torch.zeros_like(inputs.query)
    ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, partials, 4, plain_split)
    for order in (longest_first, shuffled):
        output = torch.zeros_like(inputs.query)
        ops.paged_ragged_attention_fast_lfm2_bf16_into(inputs, output, token_order=order)
        assert np.array_equal(bits_of(output), plain)
        output = torch.zeros_like(inputs.query)
        ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, partials, 4, output, token_order=order)
        assert np.array_equal(bits_of(output), bits_of(plain_split))
    # one entry points outside the batch: that group of CTAs does nothing, the token it displaced keeps the fill
    broken = shuffled.clone()
    victim = int(broken[5])
    broken[5] = tokens + 3
    output = torch.full_like(inputs.query, 7.0)
    ops.paged_ragged_attention_fast_lfm2_bf16_into(inputs, output, token_order=broken)
    got = bits_of(output)
    untouched = bits_of(torch.full((1,), 7.0, dtype=torch.bfloat16))[0]
    assert np.all(got[victim] == untouched)
    keep = np.arange(tokens) != victim
    assert np.array_equal(got[keep], plain[keep])
    with pytest.raises(Lfm25Error):
        ops.paged_ragged_attention_fast_lfm2_bf16_into(inputs, output, token_order=shuffled[:tokens - 1])
    assert ops.device_status()[0] == 0


@pytest.mark.parametrize("splits", [2, 4, 8])
@pytest.mark.parametrize("sequences,low,high", [(1, 3000, 3000), (9, 1, 700), (24, 16, 4096), (70, 100, 2048)])
def test_merge_inside_the_kernel_gives_the_bits_of_the_merge_kernel(device, splits, sequences, low, high):
    """Without a workspace the splits of a token run as one thread-block cluster and merge through distributed shared
    memory; the output must be bit-identical to records + merge kernel, with short contexts (empty splits) in the
    batch, with and without a token order."""
    case = cases.random_ragged_case(50 + sequences, sequences, low, high, 8192)
    inputs = upload(case, device)
    tokens = case["query"].shape[0]
    workspace = torch.empty((ops.splitk_workspace_elements(tokens),), dtype=torch.float32, device=device)
    expected = torch.zeros_like(inputs.query)
    ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, workspace, splits, expected)
    got = torch.zeros_like(inputs.query)
    ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, None, splits, got)
    assert np.array_equal(bits_of(got), bits_of(expected))
    order = torch.zeros(tokens, dtype=torch.int32, device=device)
    ops.context_order_desc_into(inputs.position_ids, order)
    ordered = torch.zeros_like(inputs.query)
    ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, None, splits, ordered, token_order=order)
    assert np.array_equal(bits_of(ordered), bits_of(expected))
    assert ops.device_status()[0] == 0


def test_merge_inside_the_kernel_leaves_a_token_without_result_alone(device):
    """One request slot outside the block tables (every CTA of that token's clusters returns at once) and one
    unassigned page in the middle of another sequence (only the split that meets it gives up; its partners still
    pass the cluster barrier): both rows keep what the caller passed in, the others match the valid run."""
    case = cases.random_ragged_case(61, 12, 600, 2000, 4096)
    inputs = upload(case, device)
    tokens = case["query"].shape[0]
    good = torch.zeros_like(inputs.query)
    ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, None, 4, good)
    slots = case["request_slots"].copy()
    slots[3] = case["block_tables"].shape[0] + 5
    tables = case["block_tables"].copy()
    tables[int(case["request_slots"][7]), 20] = 0xFFFFFFFF
    broken = ops.FastRaggedAttentionInput(
        query=inputs.query, arena=inputs.arena, block_tables=to_u32(tables, device),
        block_table_stride=inputs.block_table_stride, request_slots=to_u32(slots, device),
        position_ids=inputs.position_ids)
    output = torch.full_like(inputs.query, 5.0)
    ops.paged_ragged_attention_splitk_lfm2_bf16_into(broken, None, 4, output)
    got, want = bits_of(output), bits_of(good)
    fill = bits_of(torch.full((32, 64), 5.0, dtype=torch.bfloat16))
    assert np.array_equal(got[3], fill) and np.array_equal(got[7], fill)
    keep = ~np.isin(np.arange(tokens), [3, 7])
    assert np.array_equal(got[keep], want[keep])
    with pytest.raises(Lfm25Error, match="2, 4 or 8 splits"):
        ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, None, 3, output)
    assert ops.device_status()[0] == 0
