"""Attention of a mixed prefill / decode step (the reference's hybrid_ragged_gqa_lfm2_bf16 path) through the C ABI:
against the exact oracle, against the reference's own kernel on the same device buffers, in both key sources
(paged prefix + contiguous chunk, everything from the cache), with token-strided projections, and the tokens the
reference leaves untouched."""
import numpy as np
import pytest
import torch

import cases
from conftest import HYBRID_ATTENTION_KERNELS, assert_close_bf16, assert_within_oracle, bits_of, to_bf16, to_u32
from lfm25_inference_b200 import ops, workloads
from oracle import oracle, refkernels

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["mma", "umma"], autouse=True)
def kernel_choice(request, library_option):
    """Every case runs through both kernels: mma.sync (16 tokens per CTA) and tcgen05 (32 tokens per CTA)."""
    library_option("hybrid_attention", HYBRID_ATTENTION_KERNELS[request.param])
    return request.param


def run_hybrid(case, device, from_cache=False, packed=False, sentinel=None, positions=None, tables=None):
    key_cache, value_cache = case["key_cache"], case["value_cache"]
    if from_cache:
        key_cache, value_cache = key_cache.copy(), value_cache.copy()
        oracle.kv_cache_write(case["current_key"], case["current_value"], key_cache, value_cache,
                              case["batch"].physical_slots)
    arena = ops.PagedKvArena(to_bf16(key_cache, device), to_bf16(value_cache, device))
    query = to_bf16(case["query"], device)
    key, value = to_bf16(case["current_key"], device), to_bf16(case["current_value"], device)
    if packed:
        tokens = query.shape[0]
        rows = torch.cat([query.reshape(tokens, -1), key.reshape(tokens, -1), value.reshape(tokens, -1)], dim=1)
        query = rows[:, :2048].unflatten(1, (32, 64))
        key = rows[:, 2048:2560].unflatten(1, (8, 64))
        value = rows[:, 2560:].unflatten(1, (8, 64))
    output = torch.zeros((case["query"].shape[0], 32, 64), dtype=torch.bfloat16, device=device)
    if sentinel is not None:
        output = torch.zeros(output.shape, dtype=torch.int16, device=device).fill_(sentinel).view(torch.bfloat16)
    block_tables = case["block_tables"] if tables is None else tables
    ops.hybrid_ragged_attention_lfm2_bf16_into(
        query, None if from_cache else key, None if from_cache else value, arena, to_u32(block_tables, device),
        block_tables.shape[1], to_u32(case["request_slots"], device),
        to_u32(case["position_ids"] if positions is None else positions, device),
        to_u32(case["segment_offsets"], device), output)
    torch.cuda.synchronize()
    return bits_of(output)


def oracle_exact(case):
    arguments = {name: value for name, value in case.items() if name != "batch"}
    return oracle.hybrid_ragged_attention(**arguments, want_exact=True)[1]


def test_known_answer(device):
    # src/ops/attention_regression_tests.rs:64-111
    case = cases.hybrid_known_answer_case()
    case["batch"] = None
    output = oracle.bf16_to_f32(run_hybrid(case, device))
    assert np.abs(output[0] - 10.0 / 3.0).max() < 0.02
    assert np.abs(output[1] - 4.0).max() < 0.02


MIXES = [
    (5, *cases.MIXED_SMALL, 64),
    (6, [0], [1], 4),                                        # a sequence's very first token
    (7, [0], [16], 4), (8, [0], [17], 4), (9, [15], [1], 4), (10, [16], [16], 4), (11, [31], [34], 8),
    (12, [100, 0, 257, 16, 1000, 63], [64, 128, 1, 1, 33, 200], 256),
    (13, list(range(0, 40)), [1] * 40, 128),                 # decode only
    (14, [4000], [512], 512),                                # one long chunk on a long prefix
]


@pytest.mark.parametrize("from_cache", [False, True])
@pytest.mark.parametrize("seed,prefixes,chunks,pages", MIXES)
def test_against_the_oracle(device, seed, prefixes, chunks, pages, from_cache):
    case = cases.mixed_step_case(seed, prefixes, chunks, pages)
    got = run_hybrid(case, device, from_cache=from_cache)
    assert_within_oracle(got, oracle_exact(case))
    assert ops.device_status()[0] == 0


def test_token_strided_projections(device):
    case = cases.mixed_step_case(15, [20, 0, 300], [40, 5, 1], 64)
    assert np.array_equal(run_hybrid(case, device, packed=True), run_hybrid(case, device))


def test_against_the_reference_kernel(device):
    if not refkernels.available():
        pytest.skip("reference kernels were not built (make -C oracle ref)")
    case = cases.mixed_step_case(16, [100, 0, 257, 16], [64, 40, 1, 33], 64)
    arguments = [to_bf16(case[name], device) for name in ("query", "current_key", "current_value", "key_cache",
                                                          "value_cache")]
    arguments += [to_u32(case[name], device) for name in ("block_tables", "request_slots", "position_ids",
                                                          "segment_offsets")]
    reference = torch.zeros((case["query"].shape[0], 32, 64), dtype=torch.bfloat16, device=device)
    refkernels.hybrid_ragged_attention(*arguments, reference)
    torch.cuda.synchronize()
    # the bound the reference uses between its precise and its fast kernels
    assert_close_bf16(run_hybrid(case, device), bits_of(reference), 0.035, 0.025)


def test_tokens_the_reference_leaves_untouched(device):
    # kernels/attention.cu:419-423 (position below the offset) and :465-468 (unassigned page)
    case = cases.mixed_step_case(6, [20, 3], [4, 2], 16)
    positions = case["position_ids"].copy()
    positions[2] = 1
    tables = case["block_tables"].copy()
    tables[case["request_slots"][4], 0] = 0xFFFFFFFF
    got = run_hybrid(case, device, sentinel=0x1234, positions=positions, tables=tables)
    untouched = [bool((got[token] == 0x1234).all()) for token in range(6)]
    assert untouched == [False, False, True, False, True, True]
    want = oracle.hybrid_ragged_attention(case["query"], case["current_key"], case["current_value"],
                                          case["key_cache"], case["value_cache"], tables, case["request_slots"],
                                          positions, case["segment_offsets"], want_exact=True)[1]
    for token in (0, 1, 3):
        assert_within_oracle(got[token], want[token])


def test_shape_checks(device):
    case = cases.mixed_step_case(17, [3], [2], 4)
    arena = ops.PagedKvArena(to_bf16(case["key_cache"], device), to_bf16(case["value_cache"], device))
    query = to_bf16(case["query"], device)
    key, value = to_bf16(case["current_key"], device), to_bf16(case["current_value"], device)
    tables = to_u32(case["block_tables"], device)
    common = (arena, tables, tables.shape[1], to_u32(case["request_slots"], device),
              to_u32(case["position_ids"], device))
    output = torch.zeros_like(query)
    with pytest.raises(ops.Lfm25Error, match="segments are empty"):
        ops.hybrid_ragged_attention_lfm2_bf16_into(query, key, value, *common, to_u32(np.zeros(1, np.uint32), device),
                                                   output)
    with pytest.raises(ops.Lfm25Error, match="K/V shape mismatch"):
        ops.hybrid_ragged_attention_lfm2_bf16_into(query, key[:1], value[:1], *common,
                                                   to_u32(case["segment_offsets"], device), output)
    with pytest.raises(ops.Lfm25Error, match="position mismatch"):
        ops.hybrid_ragged_attention_lfm2_bf16_into(query, key, value, arena, tables, tables.shape[1], common[3],
                                                   common[4][:1], to_u32(case["segment_offsets"], device), output)
