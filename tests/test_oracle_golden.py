"""Pins the CPU oracle to outputs of the reference project's own CUDA kernels.

tests/golden/reference_b200.npz holds what the reference's unmodified kernels (rebuilt for sm_100a) produced
on a B200 for the inputs of tests/cases.py (generator: tests/golden/make_golden.py).  Bounds are the ones the
reference's tests use between its own kernels."""
import os

import numpy as np
import pytest

import cases
from conftest import assert_close_bf16
from oracle import oracle

GOLDEN_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.npz")
pytestmark = pytest.mark.skipif(not os.path.exists(GOLDEN_PATH), reason="golden fixture not generated yet")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN_PATH)


def oracle_attention(case):
    return oracle.paged_ragged_attention(case["query"], case["key_cache"], case["value_cache"], case["block_tables"],
                                         case["request_slots"], case["position_ids"])


def check_attention(golden, prefix, case, splits=()):
    ours = oracle_attention(case)
    assert_close_bf16(golden[f"{prefix}_precise"], ours, 1e-6, 2 ** -7)   # exp vs exp: one bf16 step
    assert_close_bf16(golden[f"{prefix}_fast"], ours, 0.035, 0.025)
    for count in splits:
        assert_close_bf16(golden[f"{prefix}_splitk{count}"], ours, 0.04, 0.03)
        want = oracle.splitk_partials(case["query"], case["key_cache"], case["value_cache"], case["block_tables"],
                                      case["request_slots"], case["position_ids"], count)
        got = golden[f"{prefix}_partials{count}"]
        empty = want[..., 1] == 0
        assert np.array_equal(got[..., 1] == 0, empty)
        assert np.all(np.isneginf(got[..., 0][empty]))
        assert np.allclose(got[..., :2][~empty], want[..., :2][~empty], rtol=2e-3, atol=1e-4)
        assert np.allclose(got[..., 2:][~empty], want[..., 2:][~empty], rtol=2e-3, atol=2e-3)
        assert_close_bf16(oracle.merge_splitk(got), golden[f"{prefix}_splitk{count}"], 1e-6, 2 ** -7)


@pytest.mark.parametrize("context", cases.SINGLE_CONTEXTS)
def test_single_contexts(golden, context):
    check_attention(golden, f"single{context}", cases.single_context_case(context))


def test_reversed_tables(golden):
    check_attention(golden, "reversed", cases.ragged_reversed_case())


def test_splitk_lengths(golden):
    check_attention(golden, "splitk", cases.splitk_case(), splits=(2, 4, 8))


def test_random_batch(golden):
    check_attention(golden, "random", cases.random_ragged_case(7, 6, 1, 700, 512), splits=(4,))


def test_fused_qk_postprocess(golden):
    case = cases.qk_postprocess_case()
    query = case["query"].copy()
    key_cache = np.zeros((case["num_pages"], 8, 16, 64), dtype=np.uint16)
    value_cache = np.zeros_like(key_cache)
    oracle.qk_norm_rope_kv_write_decode(query, case["key"], case["value"], case["query_norm"], case["key_norm"],
                                        case["inv_freq"], case["position_ids"], case["slot_mapping"], key_cache,
                                        value_cache, case["eps"])
    assert np.array_equal(value_cache, golden["qk_value_cache"])
    for ours, theirs in ((query, golden["qk_query"]), (key_cache, golden["qk_key_cache"])):
        assert_close_bf16(ours, theirs, 1e-6, 2 ** -7)        # at most one bf16 step (sincosf differs)
        assert (ours != theirs).mean() < 0.01


def test_fp8_producers(golden):
    values, packed = cases.fp8_inputs()
    assert np.array_equal(oracle.quantize_bf16_e4m3(values, 3.25), golden["quantize_codes"])
    hidden, codes = oracle.silu_mul_packed(packed, 9.75)
    assert (hidden != golden["silu_hidden"]).mean() <= 1e-3
    assert (codes != golden["silu_codes"]).mean() <= 1e-3


def test_hybrid_attention(golden):
    """kernels/attention.cu hybrid_ragged_gqa_lfm2_bf16_ps16 (expf, sequential online softmax) against the exact
    oracle: one bf16 step, as for the reference's precise paged kernel."""
    for name, case in (("hybrid_known", cases.hybrid_known_answer_case()),
                       ("hybrid_mixed", cases.mixed_step_case(5, *cases.MIXED_SMALL, 64))):
        if name not in golden:
            pytest.skip("fixture predates the mixed-step cases")
        case.pop("batch", None)
        assert_close_bf16(golden[name], oracle.hybrid_ragged_attention(**case), 1e-6, 2 ** -7)


def test_short_conv_segmented(golden):
    if "conv_segmented_output" not in golden:
        pytest.skip("fixture predates the mixed-step cases")
    case = cases.short_conv_segmented_case()
    states = case["states"].copy()
    output = oracle.short_conv_segmented_bf16(case["projected"], case["weight"], states, case["segment_offsets"],
                                              case["segment_slots"])
    assert np.array_equal(golden["conv_segmented_output"], output)
    assert np.array_equal(golden["conv_segmented_states"], states)


@pytest.mark.parametrize("m", cases.FP8_GEMM_BATCHES)
@pytest.mark.parametrize("site", sorted(cases.FP8_GEMM_SITES))
def test_fp8_linear_against_cublaslt(golden, site, m):
    """The oracle's FP8 linear against what cuBLASLt (the library behind the reference's BlasLt::linear_fp8_scaled,
    src/cuda/blaslt/mod.rs:212-298) returned on a B200 for the 15 points of the decode sweep, on a sample of 128
    output columns: both round one fp32 sum of exact products to bf16, so they agree to one bf16 step."""
    key = f"fp8_{site}_{m}"
    if key not in golden.files:
        pytest.skip("fixture predates the cuBLASLt section of make_golden.py")
    x_codes, scale, _ = cases.fp8_gemm_point(site, m)
    ours = oracle.linear_fp8(x_codes, cases.fp8_gemm_sampled_weights(site), scale)
    atol = float(np.abs(oracle.bf16_to_f32(ours)).max()) * 2 ** -10      # fp32 sums in another order
    assert_close_bf16(golden[key], ours, atol, 2 ** -7)
