"""Pins the CPU oracle to the known-answer tests that the reference project holds for the decode path.

Each test names the reference test it re-expresses (file:line inside the reference project).  The
reference runs these on its GPU kernels; here the same inputs go through the oracle, and wherever the
reference states an exact expectation the oracle must meet it exactly.
"""
import numpy as np
import pytest

from lfm25_inference_b200 import workloads
from oracle import oracle

import cases
from conftest import assert_close_bf16


def bf16(values):
    return oracle.f32_to_bf16(np.asarray(values, dtype=np.float32))


# ---------------------------------------------------------------------------------- E4M3


def test_quantize_known_codes():
    # src/cuda/tests/blaslt_fp8.rs:60-82  quantize_bf16_to_e4m3_correctness
    codes = oracle.quantize_bf16_e4m3(bf16([1.0, -1.0, 0.5, -0.5]), 1.0)
    assert codes.tolist() == [0x38, 0xB8, 0x30, 0xB0]


def test_e4m3_matches_ml_dtypes_for_every_bf16_value():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    bits = np.arange(65536, dtype=np.uint16)
    values = oracle.bf16_to_f32(bits)
    finite = np.isfinite(values)
    for scale in (1.0, 0.37, 448.0 / 3.0, 9.75):
        got = oracle.quantize_bf16_e4m3(bits, scale)
        with np.errstate(all="ignore"):
            scaled = (values * np.float32(scale)).astype(np.float32)
        expected = np.clip(scaled, -448.0, 448.0).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
        assert np.array_equal(got[finite], expected[finite])
    # saturation and NaN (the conversion is __NV_SATFINITE: kernels/fp8_quantize.cu:25-37)
    assert oracle.e4m3_from_f32(449.0) == 0x7E
    assert oracle.e4m3_from_f32(480.0) == 0x7E
    assert oracle.e4m3_from_f32(1e9) == 0x7E
    assert oracle.e4m3_from_f32(float("inf")) == 0x7E
    assert oracle.e4m3_from_f32(-float("inf")) == 0xFE
    assert oracle.e4m3_from_f32(float("nan")) & 0x7F == 0x7F


def test_e4m3_decode_round_trip():
    table = oracle.e4m3_decode_table()
    for code in range(256):
        if code & 0x7F == 0x7F:
            assert np.isnan(table[code])
            continue
        assert oracle.e4m3_from_f32(float(table[code])) == code


def test_scalar_scale():
    # src/model/quantization.rs:180-194  scalar_scale_round_trips / zero_scale_is_identity
    q, d = oracle.scalar_scale(2.0)
    assert abs(q - 224.0) < np.finfo(np.float32).eps
    assert abs(q * d - 1.0) < 1e-6
    assert oracle.scalar_scale(0.0) == (1.0, 1.0)
    assert oracle.scalar_scale(float("nan")) == (1.0, 1.0)
    assert oracle.scalar_scale(-1.0) == (1.0, 1.0)


def test_linear_fp8_exact_32():
    # src/cuda/tests/blaslt_fp8.rs:25-57  linear_fp8_e4m3_correctness: +-1.0 codes, every output exactly K
    m, n, k = 1, 16, 32
    x = np.array([0x38 if i % 2 == 0 else 0xB8 for i in range(m * k)], dtype=np.uint8).reshape(m, k)
    w = np.array([0x38 if i % 2 == 0 else 0xB8 for i in range(n * k)], dtype=np.uint8).reshape(n, k)
    out = oracle.linear_fp8(x, w, 1.0)
    assert np.all(oracle.bf16_to_f32(out) == float(k))


def _hashed(index, seed):
    # src/cuda/tests/blaslt_fp8.rs:91-100 deterministic_value
    value = (np.asarray(index, dtype=np.uint64) + seed) & 0xFFFFFFFF
    value ^= value >> 16
    value = (value * 0x7FEB352D) & 0xFFFFFFFF
    value ^= value >> 15
    value = (value * 0x846CA68B) & 0xFFFFFFFF
    value ^= value >> 16
    unit = (value & 0xFFFF).astype(np.float32) / np.float32(65535.0)
    return bf16((unit - np.float32(0.5)) * np.float32(1.5))


def test_tensorwide_fp8_error_is_bounded():
    # src/cuda/tests/blaslt_fp8.rs:85-167  tensorwide_fp8_numerical_error_is_bounded: NRMSE < 0.08, cosine > 0.995
    m, n, k = 4, 64, 128
    x = _hashed(np.arange(m * k), 0x12345678).reshape(m, k)
    w = _hashed(np.arange(n * k), 0x9ABCDEF0).reshape(n, k)
    xf = oracle.bf16_to_f32(x).astype(np.float64)
    wf = oracle.bf16_to_f32(w).astype(np.float64)
    xq, xd = oracle.scalar_scale(float(np.abs(xf).max()))
    wq, wd = oracle.scalar_scale(float(np.abs(wf).max()))
    out = oracle.linear_fp8(oracle.quantize_bf16_e4m3(x, xq), oracle.quantize_bf16_e4m3(w, wq), xd * wd)
    dense = xf @ wf.T
    got = oracle.bf16_to_f32(out).astype(np.float64)
    nrmse = np.sqrt(np.mean((got - dense) ** 2)) / np.sqrt(np.mean(dense ** 2))
    cosine = float((got * dense).sum() / (np.linalg.norm(got) * np.linalg.norm(dense)))
    assert nrmse < 0.08 and cosine > 0.995


def test_fused_silu_mul_fp8_equals_unfused_pipeline():
    # src/ops/silu_mul.rs:177-205: fused SiLU->E4M3 equals silu kernel then quantise kernel, even and odd widths
    rng = np.random.default_rng(5)
    for rows, width in ((3, 64), (2, 7), (1, 8192)):
        packed = workloads.bf16_normal(rng, (rows, 2 * width), std=2.0)
        hidden, codes = oracle.silu_mul_packed(packed, 9.75)
        assert np.array_equal(codes, oracle.quantize_bf16_e4m3(hidden, 9.75))
        g = oracle.bf16_to_f32(packed[:, :width]).astype(np.float64)
        u = oracle.bf16_to_f32(packed[:, width:]).astype(np.float64)
        assert_close_bf16(hidden, bf16(g / (1 + np.exp(-g)) * u), 1e-6, 1e-2)


# ---------------------------------------------------------------------------------- KV append


@pytest.mark.parametrize("page_size", [16, 32])
def test_kv_cache_raw_layout(page_size):
    # src/cuda/kernels/tests/kv_cache.rs:13-66  kv_cache_raw_correctness_ps{16,32}
    tokens, pages = 3, 3
    source = (np.arange(tokens * 8 * 64, dtype=np.uint32) ^ 0x5A5A).astype(np.uint16).reshape(tokens, 8, 64)
    slots = np.array([0, -1, page_size * 2 + 3], dtype=np.int64)
    key_cache = np.zeros((pages, 8, page_size, 64), dtype=np.uint16)
    value_cache = np.zeros_like(key_cache)
    oracle.kv_cache_write(source, source, key_cache, value_cache, slots, page_size)
    flat = key_cache.reshape(-1)
    written = np.zeros(flat.size, dtype=bool)
    for token in (0, 2):
        slot = int(slots[token])
        for head in range(8):
            destination = ((slot // page_size * 8 + head) * page_size + slot % page_size) * 64
            assert np.array_equal(flat[destination:destination + 64], source[token, head])
            written[destination:destination + 64] = True
    assert np.all(flat[~written] == 0)  # slot -1 skipped, nothing else touched
    assert np.array_equal(key_cache, value_cache)


@pytest.mark.parametrize("page_size", [16, 32])
def test_paged_kv_write_preserves_bits(page_size):
    # src/cache/kv_cache.rs:159-209  paged_kv_write_ps{16,32}_preserves_bits_and_layout
    key = bf16(np.arange(2 * 8 * 64) / 64.0).reshape(2, 8, 64)
    value = bf16(-np.arange(2 * 8 * 64) / 64.0).reshape(2, 8, 64)
    slots = np.array([0, page_size + 1], dtype=np.int64)
    key_cache = np.zeros((2, 8, page_size, 64), dtype=np.uint16)
    value_cache = np.zeros_like(key_cache)
    oracle.kv_cache_write(key, value, key_cache, value_cache, slots, page_size)
    for token, slot in enumerate(slots):
        page, offset = divmod(int(slot), page_size)
        assert np.array_equal(key_cache[page, :, offset, :], key[token])
        assert np.array_equal(value_cache[page, :, offset, :], value[token])


def test_out_of_pool_slot_is_skipped():
    # kernels/kv_cache.cu:45-59
    key = workloads.bf16_normal(np.random.default_rng(0), (2, 8, 64))
    key_cache = np.zeros((2, 8, 16, 64), dtype=np.uint16)
    value_cache = np.zeros_like(key_cache)
    oracle.kv_cache_write(key, key, key_cache, value_cache, np.array([2 * 16, 5], dtype=np.int64))
    assert not key_cache[:, :, :5].any() and not key_cache[1].any()
    assert np.array_equal(key_cache[0, :, 5, :], key[1])


# ---------------------------------------------------------------------------------- attention


def _write_sequence_major(key, value, slots, pages, page_size=16):
    key_cache = np.zeros((pages, 8, page_size, 64), dtype=np.uint16)
    value_cache = np.zeros_like(key_cache)
    oracle.kv_cache_write(key, value, key_cache, value_cache, np.asarray(slots, dtype=np.int64), page_size)
    return key_cache, value_cache


def test_ragged_attention_selects_each_request_block_table():
    # src/ops/attention_regression_tests.rs:19-61: Q = K = 0, context 1 -> output is V of the request's own page
    query = np.zeros((2, 32, 64), dtype=np.uint16)
    key = np.zeros((2, 8, 64), dtype=np.uint16)
    values = np.zeros((2, 8, 64), dtype=np.float32)
    for token in range(2):
        for head in range(8):
            values[token, head] = token * 100 + head * 2 + np.arange(64) / 64.0
    value = bf16(values)
    key_cache, value_cache = _write_sequence_major(key, value, [0, 16], 2)
    out = oracle.paged_ragged_attention(query, key_cache, value_cache, np.array([[0], [1]], dtype=np.uint32),
                                        np.array([0, 1], dtype=np.uint32), np.array([0, 0], dtype=np.uint32))
    expected = np.repeat(value, 4, axis=1)  # query head q reads KV head q // 4
    assert np.array_equal(out, expected)


def _dense_causal_last_row(query_last, key, value):
    q = oracle.bf16_to_f32(query_last).astype(np.float64)            # [32, 64]
    k = oracle.bf16_to_f32(key).astype(np.float64)                   # [T, 8, 64]
    v = oracle.bf16_to_f32(value).astype(np.float64)
    out = np.zeros((32, 64))
    for head in range(32):
        scores = k[:, head // 4, :] @ q[head] * 0.125
        weights = np.exp(scores - scores.max())
        out[head] = weights @ v[:, head // 4, :] / weights.sum()
    return out


def test_paged_attention_matches_dense_across_page_boundaries():
    # src/ops/attention_regression_tests.rs:111-175: 33 tokens, patterned inputs, identity and permuted [2,0,1] tables
    tokens = 33
    query = workloads.patterned_bf16(tokens * 32 * 64, 17, 101, 50.0, 64.0).reshape(tokens, 32, 64)
    key = workloads.patterned_bf16(tokens * 8 * 64, 13, 89, 44.0, 64.0).reshape(tokens, 8, 64)
    value = workloads.patterned_bf16(tokens * 8 * 64, 7, 79, 39.0, 32.0).reshape(tokens, 8, 64)
    dense = bf16(_dense_causal_last_row(query[-1], key, value))
    for table in ([0, 1, 2], [2, 0, 1]):
        slots = [table[p // 16] * 16 + p % 16 for p in range(tokens)]
        key_cache, value_cache = _write_sequence_major(key, value, slots, 3)
        out = oracle.paged_ragged_attention(query[-1:].copy(), key_cache, value_cache,
                                            np.array([table], dtype=np.uint32), None,
                                            np.array([tokens - 1], dtype=np.uint32))
        assert_close_bf16(out[0], dense, 0.03, 0.02)
        assert np.array_equal(out[0], dense)  # both are the same exact softmax rounded once


@pytest.mark.parametrize("context", [1, 16, 17, 33, 67, 128])
def test_single_sequence_contexts(context):
    # src/ops/attention_async_fast_tests.rs:27-65: contexts {1, PS, PS+1, 2PS+1, 4PS+3, 128}
    key = workloads.patterned_bf16(context * 8 * 64, 13 + context, 89, 44.0, 64.0).reshape(context, 8, 64)
    value = workloads.patterned_bf16(context * 8 * 64, 7 + context, 79, 39.0, 32.0).reshape(context, 8, 64)
    query = workloads.patterned_bf16(32 * 64, 17 + context, 101, 50.0, 64.0).reshape(1, 32, 64)
    pages = (context + 15) // 16
    key_cache, value_cache = _write_sequence_major(key, value, list(range(context)), pages)
    out = oracle.paged_ragged_attention(query, key_cache, value_cache,
                                        np.arange(pages, dtype=np.uint32).reshape(1, pages), None,
                                        np.array([context - 1], dtype=np.uint32))
    assert np.array_equal(out[0], bf16(_dense_causal_last_row(query[0], key, value)))


def _splitk_case():
    # src/ops/attention_splitk_tests.rs:21-132: lengths [257, 65]
    lengths = [257, 65]
    pages = [(length + 15) // 16 for length in lengths]
    stride = max(pages)
    total_tokens = sum(lengths)
    index = np.arange(2 * 32 * 64, dtype=np.int64)
    query = bf16(((index * 17 % 113).astype(np.float32) - 56.0) / 96.0).reshape(2, 32, 64)
    index = np.arange(total_tokens * 8 * 64, dtype=np.int64)
    key = bf16(((index * 13 % 97).astype(np.float32) - 48.0) / 96.0).reshape(total_tokens, 8, 64)
    value = bf16(((index * 7 % 89).astype(np.float32) - 44.0) / 48.0).reshape(total_tokens, 8, 64)
    tables = np.full((2, stride), 0xFFFFFFFF, dtype=np.uint32)
    slots = []
    base = 0
    for request, (length, count) in enumerate(zip(lengths, pages)):
        tables[request, :count] = base + np.arange(count)
        slots += [(base + p // 16) * 16 + p % 16 for p in range(length)]
        base += count
    key_cache, value_cache = _write_sequence_major(key, value, slots, base)
    positions = np.array([lengths[0] - 1, lengths[1] - 1], dtype=np.uint32)
    return query, key_cache, value_cache, tables, np.array([0, 1], dtype=np.uint32), positions


@pytest.mark.parametrize("splits", [2, 4, 8])
def test_splitk_merge_equals_unsplit(splits):
    query, key_cache, value_cache, tables, slots, positions = _splitk_case()
    reference = oracle.paged_ragged_attention(query, key_cache, value_cache, tables, slots, positions)
    partials = oracle.splitk_partials(query, key_cache, value_cache, tables, slots, positions, splits)
    merged = oracle.merge_splitk(partials)
    assert_close_bf16(merged, reference, 0.04, 0.03)   # the reference's own bound
    assert_close_bf16(merged, reference, 1e-6, 2 ** -7)  # and in fact within one bf16 step
    # empty splits follow the (-inf, 0, 0...) convention: request 1 has 5 pages, so 8 splits leave 3 empty
    if splits == 8:
        records = partials[1, 0]
        empty = [s for s in range(8) if 5 * s // 8 == 5 * (s + 1) // 8]
        assert len(empty) == 3
        for s in empty:
            assert records[s, 0] == -np.inf and records[s, 1] == 0 and not records[s, 2:].any()


def test_skipped_tokens_leave_output_untouched():
    # kernels/attention_async_fast.cu:88-111,149-151: invalid row / position / page -> silent return
    query, key_cache, value_cache, tables, slots, positions = _splitk_case()
    sentinel = np.full((2, 32, 64), 0x1234, dtype=np.uint16)
    out = oracle.paged_ragged_attention(query, key_cache, value_cache, tables, np.array([0, 7], dtype=np.uint32),
                                        positions, output=sentinel.copy())
    assert np.all(out[1] == 0x1234) and not np.all(out[0] == 0x1234)
    out = oracle.paged_ragged_attention(query, key_cache, value_cache, tables, slots,
                                        np.array([17 * 16, 64], dtype=np.uint32), output=sentinel.copy())
    assert np.all(out[0] == 0x1234)
    broken = tables.copy()
    broken[1, 2] = 0xFFFFFFFF
    out = oracle.paged_ragged_attention(query, key_cache, value_cache, broken, slots, positions, output=sentinel.copy())
    assert np.all(out[1] == 0x1234) and not np.all(out[0] == 0x1234)


def test_physical_slots():
    # src/model/lfm2_base.rs:371-378
    batch = workloads.ragged_decode_batch(1, 4, 16, 100, 64, 2)
    for step in range(2):
        got = oracle.physical_slots(batch.block_tables, batch.request_slots, batch.positions(step))
        assert np.array_equal(got, batch.physical_slots(step))
    tables = np.array([[3, 0xFFFFFFFF]], dtype=np.uint32)
    got = oracle.physical_slots(tables, np.array([0, 0, 1], dtype=np.uint32), np.array([5, 16, 0], dtype=np.uint32))
    assert got.tolist() == [3 * 16 + 5, -1, -1]


# ---------------------------------------------------------------------------------- QK norm + RoPE


def test_qk_postprocess_against_plain_formulas():
    # src/ops/qk_postprocess.rs:189-275: fused path == rms_norm -> rope -> write_lfm2; V bit-exact
    rng = np.random.default_rng(11)
    tokens = 5
    query = workloads.bf16_normal(rng, (tokens, 32, 64))
    key = workloads.bf16_normal(rng, (tokens, 8, 64))
    value = workloads.bf16_normal(rng, (tokens, 8, 64))
    q_norm = bf16(1.0 + 0.1 * rng.standard_normal(64))
    k_norm = bf16(1.0 + 0.1 * rng.standard_normal(64))
    inv_freq = oracle.rope_inv_freq()
    positions = np.array([0, 14, 15, 16, 33], dtype=np.uint32)
    slots = np.array([16 + 0, 16 + 14, 16 + 15, 0, 2 * 16 + 1], dtype=np.int64)  # crosses a page boundary
    key_cache = np.zeros((3, 8, 16, 64), dtype=np.uint16)
    value_cache = np.zeros_like(key_cache)
    rotated_query = query.copy()
    oracle.qk_norm_rope_kv_write_decode(rotated_query, key, value, q_norm, k_norm, inv_freq, positions, slots,
                                        key_cache, value_cache, 1e-5)

    def plain(x, weight, position):
        xf = oracle.bf16_to_f32(x).astype(np.float64)
        normed = xf / np.sqrt((xf ** 2).mean(-1, keepdims=True) + 1e-5)
        normed = oracle.bf16_to_f32(bf16(normed)).astype(np.float64) * oracle.bf16_to_f32(weight).astype(np.float64)
        normed = oracle.bf16_to_f32(bf16(normed)).astype(np.float64)
        angle = np.float64(position) * inv_freq.astype(np.float64)
        first, second = normed[..., :32], normed[..., 32:]
        return np.concatenate([first * np.cos(angle) - second * np.sin(angle),
                               second * np.cos(angle) + first * np.sin(angle)], axis=-1)

    for token in range(tokens):
        page, offset = divmod(int(slots[token]), 16)
        assert_close_bf16(rotated_query[token], bf16(plain(query[token], q_norm, positions[token])), 0.03, 0.02)
        assert_close_bf16(key_cache[page, :, offset, :], bf16(plain(key[token], k_norm, positions[token])), 0.03, 0.02)
        assert np.array_equal(value_cache[page, :, offset, :], value[token])
    # a skipped token leaves its query untouched
    untouched = query.copy()
    oracle.qk_norm_rope_kv_write_decode(untouched, key, value, q_norm, k_norm, inv_freq, positions,
                                        np.full(tokens, -1, dtype=np.int64), key_cache.copy(), value_cache.copy(), 1e-5)
    assert np.array_equal(untouched, query)


def test_hybrid_attention_uses_paged_prefix_and_contiguous_current_chunk():
    # src/ops/attention_regression_tests.rs:64-111
    case = cases.hybrid_known_answer_case()
    output = oracle.bf16_to_f32(oracle.hybrid_ragged_attention(**case))
    assert np.abs(output[0] - 10.0 / 3.0).max() < 0.02
    assert np.abs(output[1] - 4.0).max() < 0.02


def test_hybrid_attention_equals_paged_attention_after_the_append():
    """Appending the step's K/V to the cache and attending through the block tables is the same function."""
    prefixes, chunks = cases.MIXED_SMALL
    case = cases.mixed_step_case(5, prefixes, chunks, 64)
    batch = case.pop("batch")
    _, hybrid = oracle.hybrid_ragged_attention(**case, want_exact=True)
    key_cache, value_cache = case["key_cache"].copy(), case["value_cache"].copy()
    oracle.kv_cache_write(case["current_key"], case["current_value"], key_cache, value_cache, batch.physical_slots)
    _, paged = oracle.paged_ragged_attention(case["query"], key_cache, value_cache, case["block_tables"],
                                             case["request_slots"], case["position_ids"], want_exact=True)
    assert np.isfinite(hybrid).all()          # no NaN-pattern row of the pool was read
    assert np.abs(hybrid - paged).max() < 1e-12


def test_hybrid_attention_skips_inconsistent_tokens():
    # kernels/attention.cu:419-423 (position < offset) and :465-468 (unassigned page)
    prefixes, chunks = [20, 3], [4, 2]
    case = cases.mixed_step_case(6, prefixes, chunks, 16)
    case.pop("batch")
    positions = case["position_ids"].copy()
    positions[2] = 1                          # third token of its segment cannot sit at position 1
    tables = case["block_tables"].copy()
    tables[case["request_slots"][4], 0] = 0xFFFFFFFF
    sentinel = np.full((6, 32, 64), 0x1234, dtype=np.uint16)
    got = oracle.hybrid_ragged_attention(case["query"], case["current_key"], case["current_value"],
                                         case["key_cache"], case["value_cache"], tables, case["request_slots"],
                                         positions, case["segment_offsets"], output=sentinel.copy())
    untouched = [bool((got[token] == 0x1234).all()) for token in range(6)]
    assert untouched == [False, False, True, False, True, True]


def test_short_conv_segmented_equals_token_steps_with_fp32_carry():
    """kernels/short_conv.cu:100-143: inside a segment the state is carried unrounded."""
    case = cases.short_conv_segmented_case()
    states = case["states"].copy()
    got = oracle.short_conv_segmented_bf16(case["projected"], case["weight"], states, case["segment_offsets"],
                                           case["segment_slots"])
    hidden = case["weight"].shape[0]
    projected = oracle.bf16_to_f32(case["projected"]).astype(np.float32)
    weight = oracle.bf16_to_f32(case["weight"]).astype(np.float32)
    want_states = case["states"].copy()
    want = np.zeros_like(got)
    for segment, slot in enumerate(case["segment_slots"]):
        if slot >= want_states.shape[0]:
            continue
        state = oracle.bf16_to_f32(want_states[slot]).astype(np.float32)
        s0, s1 = state[:, 0].copy(), state[:, 1].copy()
        for token in range(case["segment_offsets"][segment], case["segment_offsets"][segment + 1]):
            b, c, x = (projected[token, :hidden], projected[token, hidden:2 * hidden], projected[token, 2 * hidden:])
            gated = b * x
            convolved = (weight[:, 0] * s0 + weight[:, 1] * s1) + weight[:, 2] * gated
            want[token] = oracle.f32_to_bf16(c * convolved)
            s0, s1 = s1, gated
        want_states[slot, :, 0] = oracle.f32_to_bf16(s0)
        want_states[slot, :, 1] = oracle.f32_to_bf16(s1)
    assert np.array_equal(got, want)
    assert np.array_equal(states, want_states)
    skipped = slice(int(case["segment_offsets"][2]), int(case["segment_offsets"][3]))
    assert not got[skipped].any()
