"""The cost curves and the step planner (host-only), restated from the reference's own tests:
src/scheduler/cost_model.rs:233-306 and src/scheduler/planner.rs:238-439."""
import pytest

from lfm25_inference_b200 import cache
from lfm25_inference_b200._abi import PHASE_DECODING, PHASE_FREE, PHASE_QUEUED_PREFILL, Lfm25Error


def single_curve(points):
    return cache.HardwareCostModel(points, points, points)


def test_measured_points_are_exact_and_unmeasured_interior_is_conservative():
    model = single_curve([(1, 1, 128, 7.0), (8, 1, 128, 8.0)])
    assert model.predict("decode_bf16", 1, 1, 128) == 7.0
    assert model.predict("decode_bf16", 4, 1, 128) == 8.0
    assert model.predict("decode_bf16", 16, 1, 128) >= 16.0


def test_decode_interpolation_preserves_measurements_and_removes_batch_cliffs():
    model = single_curve([(16, 1, 2048, 11.0), (32, 1, 2048, 16.0), (64, 1, 2048, 24.0), (16, 1, 8192, 22.0)])
    assert model.predict_decode_ms(32, 2048, True) == 16.0
    assert 16.0 < model.predict_decode_ms(33, 2048, True) < 24.0
    assert 11.0 < model.predict_decode_ms(16, 2049, False) < 22.0


def test_decode_interpolation_extrapolates_conservatively_outside_grid():
    model = single_curve([(16, 1, 2048, 12.0)])
    assert model.predict_decode_ms(32, 2048, True) >= 24.0
    assert model.predict_decode_ms(16, 4096, True) >= 24.0


def test_invalid_curves_are_rejected():
    with pytest.raises(Lfm25Error, match="requires measured points"):
        cache.HardwareCostModel([], [(1, 1, 1, 1.0)], [(1, 1, 1, 1.0)])
    with pytest.raises(Lfm25Error, match="invalid point"):
        single_curve([(0, 1, 1, 1.0)])
    with pytest.raises(Lfm25Error, match="invalid point"):
        single_curve([(1, 1, 1, float("nan"))])


def planner_cost_model():
    # src/scheduler/planner.rs:243-273
    decode = [(1, 1, 128, 6.0), (64, 1, 2048, 20.0)]
    return cache.HardwareCostModel(decode, decode, [(1, 128, 128, 10.0)])


def request(phase=PHASE_FREE, prompt_len=0, prefilled=0, context=0, now=0):
    # SequenceRequest::initialize (src/scheduler/request.rs:71-91) with the default SLOs
    return dict(phase=phase, prompt_len=prompt_len, prefilled=prefilled, context_tokens=context, arrival_us=now,
                first_token_deadline_us=now + 400_000, next_token_deadline_us=now + 50_000)


def test_decode_is_scheduled_before_aged_prefill():
    requests = [request(PHASE_DECODING, 1, 1, 1), request(PHASE_QUEUED_PREFILL, 256, 0, 256), request()]
    work, plan = cache.schedule(planner_cost_model(), requests, 10_000)
    assert work[0] == ("decode", 0, 1)
    assert plan["prefill_tokens"] > 0 and plan["decode_count"] == 1


def test_packs_multiple_short_prefills_into_one_step():
    requests = [request(PHASE_QUEUED_PREFILL, 32, 0, 32) for _ in range(3)] + [request()]
    work, plan = cache.schedule(planner_cost_model(), requests, 10_000)
    assert [kind for kind, _, _ in work] == ["prefill"] * 3
    assert plan["prefill_tokens"] == 96
    assert plan["predicted_ms"] <= 40.0


def tail_requests(count, long_count=None):
    requests = []
    for index in range(count):
        if long_count is None or index < long_count:
            requests.append(request(PHASE_QUEUED_PREFILL, 2048, 2032, 2048))
        else:
            requests.append(request(PHASE_QUEUED_PREFILL, 128, 112, 128))
    return requests


def test_large_long_context_tail_burst_is_decode_only():
    work, plan = cache.schedule(planner_cost_model(), tail_requests(24), 10_000)
    assert len(work) == 24 and all(item[0] == "prefill" and item[2] == 1 for item in work)
    assert plan["prefill_tokens"] == 24 and plan["predicted_ms"] < 40.0


def test_long_tail_pressure_forces_short_cached_tails_to_singletons_too():
    work, _ = cache.schedule(planner_cost_model(), tail_requests(24, long_count=4), 10_000)
    assert len(work) == 24 and all(item[2] == 1 for item in work)


def test_small_long_context_tail_batch_keeps_chunked_prefill():
    work, _ = cache.schedule(planner_cost_model(), tail_requests(8), 10_000)
    assert len(work) == 8 and all(item[0] == "prefill" and item[2] == 16 for item in work)


def test_decode_order_and_budget_exhaustion():
    model = planner_cost_model()
    requests = [request(PHASE_DECODING, 8, 8, 100), request(PHASE_DECODING, 8, 8, 50),
                request(PHASE_QUEUED_PREFILL, 600, 0, 600)]
    requests[0]["next_token_deadline_us"] = 90_000
    requests[1]["next_token_deadline_us"] = 20_000
    work, plan = cache.schedule(model, requests, 10_000)
    assert work[:2] == [("decode", 1, 1), ("decode", 0, 1)]            # earliest deadline first
    # the prefill curve has one point (128 tokens at context 128: 10 ms) and extrapolates by the product of the
    # token and the context ratio: 256 tokens would cost 40 ms, more than the budget left after the decode part
    assert work[2] == ("prefill", 2, 128)
    # a step budget below the decode cost leaves no room for prefill at all
    work, plan = cache.schedule(model, requests, 10_000, step_budget_ms=1.0)
    assert [kind for kind, _, _ in work] == ["decode", "decode"] and plan["prefill_tokens"] == 0
    with pytest.raises(Lfm25Error, match="step budget must be positive"):
        cache.schedule(model, requests, 0, step_budget_ms=0.0)
