// Step planner of the serving loop: the measured cost curves and Scheduler::schedule.
//
// Replaces, in the reference: CostCurve / HardwareCostModel (src/scheduler/cost_model.rs:7-231) and
// Scheduler::schedule (src/scheduler/planner.rs:80-236).  Pure host code; it lives in the library so that a host in
// any language plans its steps through the same C ABI as it launches them.  The request table is passed in as an
// array of plain views (the fields of SequenceRequest the planner reads), so the caller keeps ownership of its
// request slots.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <new>
#include <vector>

#include "../../include/lfm25_b200.h"
#include "kernels.h"

namespace {

constexpr size_t kDecodeTailContextThreshold = 1536;   // src/scheduler/planner.rs:5-6
constexpr size_t kDecodeTailQueueThreshold = 24;

struct Curve {
    std::vector<lfm25_cost_point> points;

    // CostCurve::predict (src/scheduler/cost_model.rs:33-86): an exact point, else the nearest point that dominates
    // the query in every dimension, else a conservative extrapolation from the nearest point
    double predict(size_t batch, size_t tokens, size_t context) const {
        batch = std::max<size_t>(batch, 1);
        tokens = std::max<size_t>(tokens, 1);
        context = std::max<size_t>(context, 1);
        for (const lfm25_cost_point& point : points) {
            if (point.batch == batch && point.tokens == tokens && point.context == context) {
                return point.milliseconds;
            }
        }
        const lfm25_cost_point* dominating = nullptr;
        double best_distance = std::numeric_limits<double>::infinity();
        for (const lfm25_cost_point& point : points) {
            if (point.batch < batch || point.tokens < tokens || point.context < context) {
                continue;
            }
            const double distance = std::log(static_cast<double>(point.batch) / batch) +
                                    std::log(static_cast<double>(point.tokens) / tokens) +
                                    std::log(static_cast<double>(point.context) / context);
            if (distance < best_distance ||
                (distance == best_distance && (dominating == nullptr || point.milliseconds > dominating->milliseconds))) {
                best_distance = distance;
                dominating = &point;
            }
        }
        if (dominating != nullptr) {
            return dominating->milliseconds;
        }
        const lfm25_cost_point* nearest = &points[0];
        best_distance = std::numeric_limits<double>::infinity();
        for (const lfm25_cost_point& point : points) {
            const double distance = std::fabs(std::log(static_cast<double>(batch) / point.batch)) +
                                    std::fabs(std::log(static_cast<double>(tokens) / point.tokens)) +
                                    std::fabs(std::log(static_cast<double>(context) / point.context));
            if (distance < best_distance) {
                best_distance = distance;
                nearest = &point;
            }
        }
        const double batch_scale = std::max(static_cast<double>(batch) / nearest->batch, 1.0);
        const double token_scale = std::max(static_cast<double>(tokens) / nearest->tokens, 1.0);
        const double context_scale = std::max(static_cast<double>(context) / nearest->context, 1.0);
        return nearest->milliseconds * batch_scale * token_scale * context_scale;
    }

    // interpolate_decode_batch (:150-183): along the batch axis at one measured context; false when that context
    // has no decode point at all
    bool interpolate_batch(size_t batch, size_t context, double* out) const {
        const lfm25_cost_point* lower = nullptr;
        const lfm25_cost_point* upper = nullptr;
        for (const lfm25_cost_point& point : points) {
            if (point.tokens != 1 || point.context != context) {
                continue;
            }
            if (point.batch == batch) {
                *out = point.milliseconds;
                return true;
            }
            if (point.batch < batch && (lower == nullptr || point.batch > lower->batch)) lower = &point;
            if (point.batch > batch && (upper == nullptr || point.batch < upper->batch)) upper = &point;
        }
        if (lower != nullptr && upper != nullptr) {
            const double weight = static_cast<double>(batch - lower->batch) / static_cast<double>(upper->batch - lower->batch);
            *out = lower->milliseconds + (upper->milliseconds - lower->milliseconds) * weight;
            return true;
        }
        if (lower != nullptr) {
            *out = lower->milliseconds * std::max(static_cast<double>(batch) / lower->batch, 1.0);
            return true;
        }
        if (upper != nullptr) {
            *out = upper->milliseconds;
            return true;
        }
        return false;
    }

    double batch_or_predict(size_t batch, size_t context) const {
        double value = 0.0;
        return interpolate_batch(batch, context, &value) ? value : predict(batch, 1, context);
    }

    // predict_decode_interpolated (:94-148): bilinear inside the measured (batch, context) grid of decode points
    double predict_decode(size_t batch, size_t context) const {
        batch = std::max<size_t>(batch, 1);
        context = std::max<size_t>(context, 1);
        for (const lfm25_cost_point& point : points) {
            if (point.tokens == 1 && point.batch == batch && point.context == context) {
                return point.milliseconds;
            }
        }
        bool has_lower = false;
        bool has_upper = false;
        size_t lower = 0;
        size_t upper = 0;
        for (const lfm25_cost_point& point : points) {
            if (point.tokens != 1) continue;
            if (point.context <= context && (!has_lower || point.context > lower)) {
                has_lower = true;
                lower = point.context;
            }
            if (point.context >= context && (!has_upper || point.context < upper)) {
                has_upper = true;
                upper = point.context;
            }
        }
        if (has_lower && has_upper) {
            if (lower == upper) {
                return batch_or_predict(batch, lower);
            }
            const double lower_ms = batch_or_predict(batch, lower);
            const double upper_ms = batch_or_predict(batch, upper);
            const double weight = static_cast<double>(context - lower) / static_cast<double>(upper - lower);
            return lower_ms + (upper_ms - lower_ms) * weight;
        }
        if (has_lower) {
            return batch_or_predict(batch, lower) * std::max(static_cast<double>(context) / lower, 1.0);
        }
        if (has_upper) {
            return batch_or_predict(batch, upper);
        }
        return predict(batch, 1, context);
    }
};

bool valid_points(const lfm25_cost_point* points, size_t count) {
    if (points == nullptr || count == 0) return false;
    for (size_t index = 0; index < count; ++index) {
        const lfm25_cost_point& point = points[index];
        if (point.batch == 0 || point.tokens == 0 || point.context == 0 || !std::isfinite(point.milliseconds) ||
            point.milliseconds < 0.0) {
            return false;
        }
    }
    return true;
}

uint64_t saturating_sub(uint64_t a, uint64_t b) { return a > b ? a - b : 0; }

}  // namespace

struct lfm25_cost_model {
    Curve decode_bf16;
    Curve decode_fp8;
    Curve prefill_bf16;
    size_t page_size;
};

extern "C" {

int32_t lfm25_cost_model_create(const lfm25_cost_point* decode_bf16, size_t decode_bf16_points,
                                const lfm25_cost_point* decode_fp8, size_t decode_fp8_points,
                                const lfm25_cost_point* prefill_bf16, size_t prefill_bf16_points, size_t page_size,
                                lfm25_cost_model** out) {
    if (out == nullptr) return lfm25::report_error(LFM25_ERR_NULL_POINTER, "cost model output is null");
    if (!decode_bf16_points || !decode_fp8_points || !prefill_bf16_points) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "cost curve requires measured points");
    }
    if (!valid_points(decode_bf16, decode_bf16_points) || !valid_points(decode_fp8, decode_fp8_points) ||
        !valid_points(prefill_bf16, prefill_bf16_points)) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "cost curve contains invalid point");
    }
    if (page_size != 16 && page_size != 32) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "hardware profile has invalid page size");
    }
    lfm25_cost_model* self = new (std::nothrow) lfm25_cost_model();
    if (self == nullptr) return lfm25::report_error(LFM25_ERR_CUDA, "out of host memory");
    self->decode_bf16.points.assign(decode_bf16, decode_bf16 + decode_bf16_points);
    self->decode_fp8.points.assign(decode_fp8, decode_fp8 + decode_fp8_points);
    self->prefill_bf16.points.assign(prefill_bf16, prefill_bf16 + prefill_bf16_points);
    self->page_size = page_size;
    *out = self;
    return LFM25_OK;
}

void lfm25_cost_model_destroy(lfm25_cost_model* self) { delete self; }

double lfm25_cost_model_predict(const lfm25_cost_model* self, uint32_t curve, size_t batch, size_t tokens,
                                size_t context) {
    if (self == nullptr) return std::numeric_limits<double>::quiet_NaN();
    const Curve& chosen = curve == LFM25_CURVE_DECODE_FP8    ? self->decode_fp8
                          : curve == LFM25_CURVE_PREFILL_BF16 ? self->prefill_bf16
                                                              : self->decode_bf16;
    return chosen.predict(batch, tokens, context);
}

double lfm25_cost_model_predict_decode_ms(const lfm25_cost_model* self, size_t batch, size_t maximum_context,
                                          uint32_t fp8) {
    if (self == nullptr) return std::numeric_limits<double>::quiet_NaN();
    return (fp8 ? self->decode_fp8 : self->decode_bf16).predict_decode(batch, maximum_context);
}

double lfm25_cost_model_predict_prefill_ms(const lfm25_cost_model* self, size_t tokens) {
    if (self == nullptr) return std::numeric_limits<double>::quiet_NaN();
    return self->prefill_bf16.predict(1, tokens, tokens);
}

// Scheduler::schedule (src/scheduler/planner.rs:80-236)
int32_t lfm25_schedule(const lfm25_cost_model* cost, const lfm25_scheduler_config* config,
                       const lfm25_request_view* requests, size_t num_requests, uint64_t now_us,
                       lfm25_scheduled_work* work, size_t work_capacity, lfm25_batch_plan* plan) {
    if (cost == nullptr || config == nullptr || (requests == nullptr && num_requests > 0) || plan == nullptr ||
        (work == nullptr && work_capacity > 0)) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "scheduler received a null argument");
    }
    if (!std::isfinite(config->step_budget_ms) || config->step_budget_ms <= 0.0) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "scheduler step budget must be positive");
    }
    if (work_capacity < num_requests) {
        return lfm25::report_error(LFM25_ERR_BUFFER_TOO_SMALL, "scheduler work buffer smaller than the request table");
    }
    plan->predicted_ms = 0.0;
    plan->decode_count = 0;
    plan->prefill_tokens = 0;
    plan->work_count = 0;
    size_t count = 0;
    size_t maximum_context = 1;
    for (size_t index = 0; index < num_requests; ++index) {
        if (requests[index].phase == LFM25_PHASE_DECODING) {
            work[count].kind = LFM25_WORK_DECODE;
            work[count].slot = static_cast<uint32_t>(index);
            work[count].tokens = 1;
            ++count;
            maximum_context = std::max(maximum_context, requests[index].context_tokens);
        }
    }
    // sort_unstable_by_key on the time to the next-token deadline; ties are kept in slot order here
    std::stable_sort(work, work + count, [&](const lfm25_scheduled_work& a, const lfm25_scheduled_work& b) {
        return saturating_sub(requests[a.slot].next_token_deadline_us, now_us) <
               saturating_sub(requests[b.slot].next_token_deadline_us, now_us);
    });
    plan->decode_count = count;
    const double decode_ms =
        count == 0 ? 0.0 : lfm25_cost_model_predict_decode_ms(cost, count, maximum_context, config->fp8_decode);
    plan->predicted_ms = decode_ms;
    plan->work_count = count;
    const double remaining_budget = std::max(config->step_budget_ms - decode_ms, 0.0);
    if (remaining_budget <= 0.0 || config->maximum_prefill_tokens == 0) {
        return LFM25_OK;
    }

    struct Waiting {
        uint64_t urgency;
        uint32_t slot;
    };
    std::vector<Waiting> order;
    order.reserve(num_requests);
    for (size_t index = 0; index < num_requests; ++index) {
        const lfm25_request_view& request = requests[index];
        if (request.phase != LFM25_PHASE_QUEUED_PREFILL || request.prefilled >= request.prompt_len) {
            continue;
        }
        const uint64_t urgency = saturating_sub(saturating_sub(request.first_token_deadline_us, now_us),
                                                saturating_sub(now_us, request.arrival_us) / 4);
        order.push_back({urgency, static_cast<uint32_t>(index)});
    }
    std::stable_sort(order.begin(), order.end(), [](const Waiting& a, const Waiting& b) { return a.urgency < b.urgency; });

    const size_t page_size = cost->page_size;
    bool tail_pressure = false;
    if (order.size() >= kDecodeTailQueueThreshold) {
        for (const Waiting& entry : order) {
            const lfm25_request_view& request = requests[entry.slot];
            const size_t remaining = request.prompt_len - request.prefilled;
            if (request.prefilled >= kDecodeTailContextThreshold && remaining > 0 && remaining <= page_size) {
                tail_pressure = true;
                break;
            }
        }
    }
    if (tail_pressure) {
        // Keep the step decode-shaped: single-token prefill tails ride along with the decode batch, because any
        // longer prefill segment would send the whole ragged batch down the generic prefill path.
        size_t singletons = 0;
        size_t singleton_context = maximum_context;
        for (const Waiting& entry : order) {
            const lfm25_request_view& request = requests[entry.slot];
            const size_t remaining = request.prompt_len - request.prefilled;
            if (request.prefilled == 0 || remaining == 0 || remaining > page_size) {
                continue;
            }
            const size_t projected_count = plan->decode_count + singletons + 1;
            const size_t projected_context = std::max(singleton_context, request.prefilled + 1);
            const double projected_ms =
                lfm25_cost_model_predict_decode_ms(cost, projected_count, projected_context, config->fp8_decode);
            if (projected_ms >= config->step_budget_ms ||
                projected_ms * 1000.0 >= static_cast<double>(config->tpot_slo_us)) {
                break;
            }
            work[count].kind = LFM25_WORK_PREFILL;
            work[count].slot = entry.slot;
            work[count].tokens = 1;
            ++count;
            plan->prefill_tokens += 1;
            singletons += 1;
            singleton_context = projected_context;
            plan->predicted_ms = projected_ms;
        }
        plan->work_count = count;
        return LFM25_OK;
    }

    static const size_t kChunks[] = {512, 256, 128, 64, 32, 16, 8, 4, 2, 1};
    for (const Waiting& entry : order) {
        if (plan->prefill_tokens >= config->maximum_prefill_tokens) {
            break;
        }
        const lfm25_request_view& request = requests[entry.slot];
        const size_t remaining = std::min(request.prompt_len - request.prefilled,
                                          config->maximum_prefill_tokens - plan->prefill_tokens);
        if (remaining == 0) {
            continue;
        }
        size_t chunk = 0;
        for (size_t candidate : kChunks) {
            if (candidate > remaining) {
                continue;
            }
            if (lfm25_cost_model_predict_prefill_ms(cost, plan->prefill_tokens + candidate) <= remaining_budget) {
                chunk = candidate;
                break;
            }
        }
        if (chunk == 0) {
            break;
        }
        work[count].kind = LFM25_WORK_PREFILL;
        work[count].slot = entry.slot;
        work[count].tokens = chunk;
        ++count;
        plan->prefill_tokens += chunk;
    }
    if (plan->prefill_tokens > 0) {
        plan->predicted_ms = decode_ms + lfm25_cost_model_predict_prefill_ms(cost, plan->prefill_tokens);
    }
    plan->work_count = count;
    return LFM25_OK;
}

}  // extern "C"
