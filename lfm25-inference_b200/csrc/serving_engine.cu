// The GPU-owner loop of continuous batching behind the C ABI: request slots, admission with prefix reuse, step
// planning, the step's device metadata, mixed prefill / decode steps, token bookkeeping.
//
// Replaces, in the reference: the owner loop of src/engine/serving/radix_owner.rs (run_owner_radix :101-437,
// refresh / split of prefill work :464-547, admit_request_radix :549-708), RequestSlots / SequenceRequest
// (src/scheduler/slots.rs, src/scheduler/request.rs) and BatchModelCache's per-request bookkeeping
// (src/model/lfm2_base.rs:262-388).  It is built from the library's own parts: page allocator and block tables,
// radix index and convolution checkpoints, cost curves and planner, and the executor's decode and mixed steps.
// One engine serves one GPU from one host thread; nothing here is shared between engines.
//
// Per step the host writes one pinned block of metadata (token ids, positions, request slots, segment offsets /
// slots / output rows), issues one upload for it (plus the block tables when they changed), the step, and one
// download of the sampled ids, then synchronises once to read them.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <new>
#include <vector>

#include "../../include/lfm25_b200.h"
#include "kernels.h"
#include "options.h"

namespace {

constexpr size_t kPage = 16;
constexpr size_t kHidden = 2048;

struct Slot {
    uint32_t phase = LFM25_PHASE_FREE;
    uint64_t request_id = 0;
    std::vector<uint32_t> tokens;
    size_t prompt_len = 0;
    size_t prefilled = 0;
    size_t cached_tokens = 0;   // tokens whose K/V are in the cache
    size_t reserved_pages = 0;
    size_t max_new_tokens = 0;
    size_t reused_tokens = 0;
    uint64_t arrival_us = 0;
    uint64_t first_token_deadline_us = 0;
    uint64_t next_token_deadline_us = 0;
};

struct Pending {
    uint64_t request_id;
    std::vector<uint32_t> prompt;
    size_t max_new_tokens;
    uint64_t arrival_us;
};

int32_t cuda_failure(cudaError_t status, const char* what) {
    return lfm25::report_error(LFM25_ERR_CUDA, status == cudaSuccess ? what : cudaGetErrorString(status));
}

#define ENGINE_TRY(expression)          \
    do {                                \
        const int32_t rc_ = (expression); \
        if (rc_ != LFM25_OK) return rc_; \
    } while (0)

}  // namespace

struct lfm25_engine {
    lfm25_blaslt* blaslt = nullptr;
    const lfm25_model* model = nullptr;
    lfm25_engine_config config{};
    size_t pages_per_slot = 0;
    size_t max_tokens = 0;
    lfm25_kv_allocator* allocator = nullptr;
    lfm25_block_tables* tables = nullptr;
    lfm25_radix_cache* radix = nullptr;
    lfm25_conv_checkpoints* checkpoints = nullptr;
    std::vector<size_t> grow_from;       // per work item of the step being built: tokens cached before ...
    std::vector<size_t> grow_to;         // ... and after it
    lfm25_cost_model* cost = nullptr;
    lfm25_decode_executor* executor = nullptr;
    std::vector<uint32_t> conv_layers;   // indices of the gated-convolution layers in the model
    std::vector<Slot> slots;
    std::vector<uint32_t> free_slots;
    std::deque<Pending> queue;
    // device metadata, one allocation: [token_ids | positions | request_slots | segment_offsets | segment_slots |
    // output_rows] as u32, then physical slots (i64), then the block tables
    uint32_t* d_meta = nullptr;
    int64_t* d_physical_slots = nullptr;
    uint32_t* d_tables = nullptr;
    uint32_t* h_meta = nullptr;      // pinned mirror of d_meta
    uint32_t* h_sampled = nullptr;   // pinned
    size_t meta_words = 0;
    bool tables_dirty = true;
    bool graph_decode = true;        // LFM25_ENGINE_GRAPH=0: pure decode steps launch eagerly
    cudaEvent_t start = nullptr;
    cudaEvent_t stop = nullptr;
    lfm25_engine_stats stats{};
    // scratch of one step
    std::vector<lfm25_request_view> views;
    std::vector<lfm25_scheduled_work> work;
    std::vector<uint32_t> lookup_pages;
    std::vector<uint32_t> fresh_pages;

    uint32_t* token_ids() const { return d_meta; }
    uint32_t* positions() const { return d_meta + max_tokens; }
    uint32_t* request_slots() const { return d_meta + 2 * max_tokens; }
    uint32_t* segment_offsets() const { return d_meta + 3 * max_tokens; }
    uint32_t* segment_slots() const { return d_meta + 3 * max_tokens + config.max_slots + 1; }
    uint32_t* output_rows() const { return d_meta + 3 * max_tokens + 2 * config.max_slots + 1; }
    cudaStream_t stream() const { return static_cast<cudaStream_t>(lfm25_blaslt_stream(blaslt)); }
};

namespace {

size_t reusable_limit(size_t prompt_len) { return prompt_len == 0 ? 0 : (prompt_len - 1) / kPage * kPage; }

// One step described on the host: per segment (prefix, chunk, slot), tokens in segment order.
struct StepShape {
    std::vector<size_t> prefixes;
    std::vector<size_t> chunks;
    std::vector<uint32_t> segment_slots;
    std::vector<uint32_t> token_ids;
};

int32_t upload_tables(lfm25_engine* self, const uint32_t* table) {
    const size_t bytes = self->config.max_slots * self->pages_per_slot * sizeof(uint32_t);
    const cudaError_t status = cudaMemcpyAsync(self->d_tables, table, bytes, cudaMemcpyHostToDevice, self->stream());
    return status == cudaSuccess ? LFM25_OK : cuda_failure(status, "block table upload failed");
}

// Writes the step's metadata into the pinned block, uploads it and enqueues the step (the decode executor's path
// when every segment is one token, the mixed step otherwise).
int32_t enqueue_step(lfm25_engine* self, const StepShape& shape) {
    const size_t segments = shape.chunks.size();
    size_t tokens = 0;
    size_t decode_segments = 0;
    size_t decode_context = 0;
    bool leading = true;
    uint32_t* meta = self->h_meta;
    uint32_t* h_positions = meta + self->max_tokens;
    uint32_t* h_request_slots = meta + 2 * self->max_tokens;
    uint32_t* h_offsets = meta + 3 * self->max_tokens;
    uint32_t* h_segment_slots = h_offsets + self->config.max_slots + 1;
    uint32_t* h_output_rows = h_segment_slots + self->config.max_slots;
    for (size_t segment = 0; segment < segments; ++segment) {
        h_offsets[segment] = static_cast<uint32_t>(tokens);
        h_segment_slots[segment] = shape.segment_slots[segment];
        for (size_t index = 0; index < shape.chunks[segment]; ++index) {
            h_positions[tokens] = static_cast<uint32_t>(shape.prefixes[segment] + index);
            h_request_slots[tokens] = shape.segment_slots[segment];
            ++tokens;
        }
        h_output_rows[segment] = static_cast<uint32_t>(tokens - 1);
        if (leading && shape.chunks[segment] == 1) {
            ++decode_segments;
            decode_context = std::max(decode_context, shape.prefixes[segment] + 1);
        } else {
            leading = false;
        }
    }
    h_offsets[segments] = static_cast<uint32_t>(tokens);
    std::memcpy(meta, shape.token_ids.data(), tokens * sizeof(uint32_t));
    cudaError_t status = cudaMemcpyAsync(self->d_meta, self->h_meta, self->meta_words * sizeof(uint32_t),
                                         cudaMemcpyHostToDevice, self->stream());
    if (status != cudaSuccess) return cuda_failure(status, "step metadata upload failed");
    if (segments == tokens) {
        lfm25_decode_batch batch;
        batch.token_ids = self->token_ids();
        batch.positions = self->positions();
        batch.request_slots = self->request_slots();
        batch.physical_slots = self->d_physical_slots;
        batch.block_tables = self->d_tables;
        batch.block_table_stride = self->pages_per_slot;
        batch.block_table_rows = self->config.max_slots;
        batch.num_tokens = tokens;
        batch.max_context_tokens = decode_context;
        // a pure decode step replays the captured step of its batch size (the first two steps of a size run eagerly
        // and capture); the metadata was uploaded above, so the step does not advance it on the device
        if (self->graph_decode) {
            return lfm25_decode_executor_step_graph(self->executor, self->model, &batch, self->config.use_fp8, 0);
        }
        return lfm25_decode_executor_forward(self->executor, self->model, &batch, self->config.use_fp8, 0);
    }
    lfm25_ragged_batch batch;
    batch.token_ids = self->token_ids();
    batch.positions = self->positions();
    batch.request_slots = self->request_slots();
    batch.physical_slots = self->d_physical_slots;
    batch.segment_offsets = self->segment_offsets();
    batch.segment_slots = self->segment_slots();
    batch.output_rows = self->output_rows();
    batch.block_tables = self->d_tables;
    batch.block_table_stride = self->pages_per_slot;
    batch.block_table_rows = self->config.max_slots;
    batch.num_tokens = tokens;
    batch.num_segments = segments;
    batch.num_decode_segments = decode_segments;
    batch.max_decode_context_tokens = decode_context;
    return lfm25_decode_executor_forward_ragged(self->executor, self->model, &batch, self->config.use_fp8);
}

int32_t clear_conv_state(lfm25_engine* self, size_t slot) {
    for (uint32_t layer : self->conv_layers) {
        char* state = static_cast<char*>(self->model->layers[layer].conv_state) + slot * kHidden * 2 * 2;
        const cudaError_t status = cudaMemsetAsync(state, 0, kHidden * 2 * 2, self->stream());
        if (status != cudaSuccess) return cuda_failure(status, "convolution state reset failed");
    }
    return LFM25_OK;
}

// admit_request_radix (src/engine/serving/radix_owner.rs:549-708): a free slot, the longest reusable checkpointed
// prefix (at most the last full page before the final prompt token, so that the forward pass still yields logits),
// a page reservation for the rest of the sequence, convolution states restored from the checkpoint or cleared.
// With admission control (the reference's behaviour) every queued request is decided now: the checks run in the
// reference's order and a request that fails one leaves the queue with a rejection event; `rejections` holds at
// most `rejection_capacity` of them per call, the rest of the queue waits for the next step.  Without admission
// control a request that does not fit yet stays at the head of the queue.
int32_t admit(lfm25_engine* self, uint64_t now_us, lfm25_engine_event* rejections, size_t rejection_capacity,
              size_t* rejected) {
    const bool control = self->config.admission_control != 0;
    auto reject = [&](const Pending& request, uint32_t reason) {
        lfm25_engine_event& event = rejections[(*rejected)++];
        event.request_id = request.request_id;
        event.time_us = now_us;
        event.token = 0;
        event.finished = 1;
        event.reused_tokens = 0;
        event.rejected = reason;
        self->stats.rejected_requests += 1;
        self->queue.pop_front();
    };
    while (!self->queue.empty() && (control ? *rejected < rejection_capacity : !self->free_slots.empty())) {
        Pending& request = self->queue.front();
        const size_t limit = reusable_limit(request.prompt.size());
        if (control) {
            if (request.prompt.size() + request.max_new_tokens > self->config.max_sequence_tokens) {
                reject(request, LFM25_REJECT_SEQUENCE_CAPACITY);
                continue;
            }
            if (self->config.interactive_prompt_limit != 0 &&
                request.prompt.size() > self->config.interactive_prompt_limit) {
                reject(request, LFM25_REJECT_PROMPT_LIMIT);
                continue;
            }
        }
        size_t pages_found = 0;
        uint32_t checkpoint = 0;
        int64_t matched = 0;
        if (limit > 0) {
            matched = lfm25_radix_cache_probe_checkpoint(self->radix, request.prompt.data(), request.prompt.size(), limit,
                                                         self->lookup_pages.data(), self->lookup_pages.size(),
                                                         &pages_found, &checkpoint);
            if (matched < 0) return static_cast<int32_t>(matched);
        }
        const size_t total_tokens = request.prompt.size() + request.max_new_tokens;
        if (control) {
            // one more decoding sequence must keep the predicted decode step inside the step budget and the TPOT
            // SLO, and the prefill work queued in front of this prompt must leave its first token inside the TTFT SLO
            size_t decode_count = 1;
            size_t maximum_context = total_tokens;
            double prefill_queue_ms =
                lfm25_cost_model_predict_prefill_ms(self->cost, request.prompt.size() - static_cast<size_t>(matched));
            for (const Slot& other : self->slots) {
                if (other.phase == LFM25_PHASE_DECODING) {
                    decode_count += 1;
                    maximum_context = std::max(maximum_context, other.tokens.size());
                } else if (other.phase == LFM25_PHASE_QUEUED_PREFILL) {
                    prefill_queue_ms += lfm25_cost_model_predict_prefill_ms(self->cost, other.prompt_len - other.prefilled);
                }
            }
            const double decode_ms =
                lfm25_cost_model_predict_decode_ms(self->cost, decode_count, maximum_context, self->config.use_fp8);
            if (decode_ms >= self->config.step_budget_ms ||
                decode_ms * 1000.0 >= static_cast<double>(self->config.tpot_slo_us)) {
                reject(request, LFM25_REJECT_DECODE_BUDGET);
                continue;
            }
            const double waited_ms =
                now_us > request.arrival_us ? static_cast<double>(now_us - request.arrival_us) / 1000.0 : 0.0;
            if (waited_ms + prefill_queue_ms >= static_cast<double>(self->config.ttft_slo_us) / 1000.0) {
                reject(request, LFM25_REJECT_TTFT);
                continue;
            }
            if (self->free_slots.empty()) {
                reject(request, LFM25_REJECT_SLOTS);
                continue;
            }
        }
        const size_t needed_pages = (total_tokens + kPage - 1) / kPage - static_cast<size_t>(matched) / kPage;
        if (lfm25_kv_allocator_try_reserve_pages(self->allocator, needed_pages) < 0) {
            if (control) {
                reject(request, LFM25_REJECT_KV_PAGES);
                continue;
            }
            return LFM25_OK;   // back-pressure: the queue keeps its order
        }
        if (limit > 0) {       // the admission lookup proper: counts the hit or the miss
            (void)lfm25_radix_cache_longest_checkpoint(self->radix, request.prompt.data(), request.prompt.size(), limit,
                                                       self->lookup_pages.data(), self->lookup_pages.size(),
                                                       &pages_found, &checkpoint);
        }
        const uint32_t slot_index = self->free_slots.back();
        self->free_slots.pop_back();
        Slot& slot = self->slots[slot_index];
        uint32_t* row = lfm25_block_tables_slot(self->tables, slot_index);
        std::fill(row, row + self->pages_per_slot, 0xffffffffu);
        self->tables_dirty = true;
        if (matched > 0) {
            ENGINE_TRY(lfm25_kv_allocator_retain_pages(self->allocator, self->lookup_pages.data(), pages_found));
            std::copy(self->lookup_pages.begin(), self->lookup_pages.begin() + pages_found, row);
            for (size_t index = 0; index < self->conv_layers.size(); ++index) {
                ENGINE_TRY(lfm25_conv_checkpoints_restore_layer(
                    self->checkpoints, self->stream(), checkpoint, index,
                    self->model->layers[self->conv_layers[index]].conv_state, slot_index, self->config.max_slots));
            }
        } else {
            ENGINE_TRY(clear_conv_state(self, slot_index));
        }
        slot.phase = LFM25_PHASE_QUEUED_PREFILL;
        slot.request_id = request.request_id;
        slot.tokens = std::move(request.prompt);
        slot.prompt_len = slot.tokens.size();
        slot.prefilled = static_cast<size_t>(matched);
        slot.cached_tokens = slot.prefilled;
        slot.reused_tokens = slot.prefilled;
        slot.reserved_pages = needed_pages;
        slot.max_new_tokens = request.max_new_tokens;
        slot.arrival_us = request.arrival_us;
        slot.first_token_deadline_us = request.arrival_us + self->config.ttft_slo_us;
        slot.next_token_deadline_us = request.arrival_us + self->config.tpot_slo_us;
        self->stats.reused_prompt_tokens += slot.prefilled;
        self->queue.pop_front();
    }
    return LFM25_OK;
}

// publish_prefix_checkpoint: index the page-aligned prefix and snapshot the convolution states that belong to
// it, when the radix budget and a checkpoint slot allow.
int32_t publish(lfm25_engine* self, uint32_t slot_index, const Slot& slot) {
    if (!lfm25_radix_cache_can_publish(self->radix, slot.tokens.data(), slot.prompt_len, slot.prefilled)) {
        return LFM25_OK;
    }
    const int64_t checkpoint = lfm25_conv_checkpoints_acquire(self->checkpoints);
    if (checkpoint < 0) {
        return LFM25_OK;
    }
    for (size_t index = 0; index < self->conv_layers.size(); ++index) {
        ENGINE_TRY(lfm25_conv_checkpoints_capture_layer(self->checkpoints, self->stream(), static_cast<uint32_t>(checkpoint),
                                                        index, self->model->layers[self->conv_layers[index]].conv_state,
                                                        slot_index, self->config.max_slots));
    }
    const uint32_t* row = lfm25_block_tables_slot(self->tables, slot_index);
    const size_t pages = slot.prefilled / kPage;
    const int64_t created = lfm25_radix_cache_insert_checkpoint(self->radix, slot.tokens.data(), slot.prompt_len,
                                                                slot.prefilled, row, pages,
                                                                static_cast<uint32_t>(checkpoint), self->fresh_pages.data());
    if (created < 0) return static_cast<int32_t>(created);
    return lfm25_kv_allocator_pin_cached_pages(self->allocator, self->fresh_pages.data(), static_cast<size_t>(created));
}

void release(lfm25_engine* self, uint32_t slot_index) {
    Slot& slot = self->slots[slot_index];
    uint32_t* row = lfm25_block_tables_slot(self->tables, slot_index);
    // BatchModelCache::release (src/model/lfm2_base.rs:262-277): the pages go back (shared ones only lose a
    // reference) and the request's whole logical reservation is returned
    lfm25_kv_allocator_release_sequence(self->allocator, slot.cached_tokens, row, self->pages_per_slot);
    lfm25_kv_allocator_release_reservation(self->allocator, slot.reserved_pages);
    std::fill(row, row + self->pages_per_slot, 0xffffffffu);
    slot = Slot();
    self->free_slots.push_back(slot_index);
    self->tables_dirty = true;
}

}  // namespace

extern "C" {

int32_t lfm25_engine_create(lfm25_blaslt* blaslt, const lfm25_model* model, const lfm25_engine_config* config,
                            lfm25_engine** out) {
    if (blaslt == nullptr || model == nullptr || config == nullptr || out == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "engine received a null argument");
    }
    if (config->max_slots == 0 || config->max_slots > 256 || config->max_slots > model->num_request_slots) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT,
                                   "engine needs 1..=256 request slots, at most the model's state rows");
    }
    if (config->max_prefill_tokens == 0 || config->max_sequence_tokens < kPage ||
        config->max_slots + config->max_prefill_tokens > 8192) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "engine token limits are out of range");
    }
    lfm25_engine* self = new (std::nothrow) lfm25_engine();
    if (self == nullptr) return lfm25::report_error(LFM25_ERR_CUDA, "out of host memory");
    self->blaslt = blaslt;
    self->model = model;
    self->config = *config;
    self->pages_per_slot = (config->max_sequence_tokens + kPage - 1) / kPage;
    self->max_tokens = config->max_slots + config->max_prefill_tokens;
    {
        // graph replay needs a stream of its own (capture is not possible on the legacy default stream)
        cudaStream_t bound = static_cast<cudaStream_t>(lfm25_blaslt_stream(blaslt));
        self->graph_decode = lfm25::option(lfm25::kOptEngineGraph) != 0 && bound != nullptr &&
                             bound != cudaStreamLegacy;
    }
    for (uint32_t layer = 0; layer < model->num_layers; ++layer) {
        if (!model->layers[layer].is_attention) self->conv_layers.push_back(layer);
    }
    int32_t rc = lfm25_kv_allocator_create(model->num_pages, kPage, &self->allocator);
    if (rc == LFM25_OK) rc = lfm25_block_tables_create(config->max_slots, self->pages_per_slot, &self->tables);
    if (rc == LFM25_OK) rc = lfm25_radix_cache_create(kPage, std::max<size_t>(config->radix_pages, 1), &self->radix);
    if (rc == LFM25_OK && !self->conv_layers.empty()) {
        rc = lfm25_conv_checkpoints_create(self->conv_layers.size(), std::max<size_t>(config->checkpoint_capacity, 1),
                                           kHidden, 2, &self->checkpoints);
    }
    if (rc == LFM25_OK) {
        rc = lfm25_decode_executor_create_ragged(blaslt, self->max_tokens, config->max_slots, &self->executor);
    }
    if (rc == LFM25_OK) {
        self->meta_words = 3 * self->max_tokens + 3 * config->max_slots + 1;
        const size_t table_words = config->max_slots * self->pages_per_slot;
        cudaError_t status = cudaMalloc(reinterpret_cast<void**>(&self->d_meta), self->meta_words * sizeof(uint32_t));
        if (status == cudaSuccess) {
            status = cudaMalloc(reinterpret_cast<void**>(&self->d_physical_slots), self->max_tokens * sizeof(int64_t));
        }
        if (status == cudaSuccess) status = cudaMalloc(reinterpret_cast<void**>(&self->d_tables), table_words * sizeof(uint32_t));
        if (status == cudaSuccess) {
            status = cudaMallocHost(reinterpret_cast<void**>(&self->h_meta), self->meta_words * sizeof(uint32_t));
        }
        if (status == cudaSuccess) {
            status = cudaMallocHost(reinterpret_cast<void**>(&self->h_sampled), config->max_slots * sizeof(uint32_t));
        }
        if (status == cudaSuccess) status = cudaEventCreate(&self->start);
        if (status == cudaSuccess) status = cudaEventCreate(&self->stop);
        if (status != cudaSuccess) rc = cuda_failure(status, "engine buffers could not be allocated");
    }
    if (rc != LFM25_OK) {
        lfm25_engine_destroy(self);
        return rc;
    }
    std::memset(self->h_meta, 0, self->meta_words * sizeof(uint32_t));
    self->slots.resize(config->max_slots);
    for (size_t slot = config->max_slots; slot-- > 0;) {
        self->free_slots.push_back(static_cast<uint32_t>(slot));
    }
    self->views.resize(config->max_slots);
    self->work.resize(config->max_slots);
    self->lookup_pages.resize(self->pages_per_slot);
    self->fresh_pages.resize(self->pages_per_slot);
    *out = self;
    return LFM25_OK;
}

void lfm25_engine_destroy(lfm25_engine* self) {
    if (self == nullptr) return;
    lfm25_decode_executor_destroy(self->executor);
    lfm25_conv_checkpoints_destroy(self->checkpoints);
    lfm25_radix_cache_destroy(self->radix);
    if (self->tables != nullptr) lfm25_block_tables_destroy(self->tables);
    if (self->allocator != nullptr) lfm25_kv_allocator_destroy(self->allocator);
    lfm25_cost_model_destroy(self->cost);
    cudaFree(self->d_meta);
    cudaFree(self->d_physical_slots);
    cudaFree(self->d_tables);
    cudaFreeHost(self->h_meta);
    cudaFreeHost(self->h_sampled);
    if (self->start != nullptr) cudaEventDestroy(self->start);
    if (self->stop != nullptr) cudaEventDestroy(self->stop);
    delete self;
}

// Measures the cost curves the planner uses (the reference reads them from a hardware profile file,
// src/scheduler/cost_model.rs:198-216): decode steps at a few (batch, context) points and prefill chunks of the
// planner's sizes, on scratch block tables; the live tables are uploaded again afterwards.
int32_t lfm25_engine_calibrate(lfm25_engine* self) {
    if (self == nullptr) return lfm25::report_error(LFM25_ERR_NULL_POINTER, "engine is null");
    for (const Slot& slot : self->slots) {
        if (slot.phase != LFM25_PHASE_FREE) {
            return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "calibrate needs an idle engine");
        }
    }
    // the curves are measured with eager launches: a first replay would put the capture inside the timed step
    const bool graph_decode = self->graph_decode;
    self->graph_decode = false;
    struct Restore {
        lfm25_engine* engine;
        bool value;
        ~Restore() { engine->graph_decode = value; }
    } restore{self, graph_decode};
    std::vector<lfm25_cost_point> decode_points;
    std::vector<lfm25_cost_point> prefill_points;
    std::vector<uint32_t> table(self->config.max_slots * self->pages_per_slot);
    auto timed = [&](const StepShape& shape, double* milliseconds) -> int32_t {
        ENGINE_TRY(upload_tables(self, table.data()));
        ENGINE_TRY(enqueue_step(self, shape));   // warm-up: plans, function attributes
        cudaEventRecord(self->start, self->stream());
        ENGINE_TRY(enqueue_step(self, shape));
        cudaEventRecord(self->stop, self->stream());
        const cudaError_t status = cudaEventSynchronize(self->stop);
        if (status != cudaSuccess) return cuda_failure(status, "calibration step failed");
        float elapsed = 0.0f;
        cudaEventElapsedTime(&elapsed, self->start, self->stop);
        *milliseconds = elapsed;
        return LFM25_OK;
    };
    const size_t batches[4] = {1, std::min<size_t>(8, self->config.max_slots), std::min<size_t>(32, self->config.max_slots),
                               self->config.max_slots};
    for (size_t context : {size_t(512), size_t(2048)}) {
        if (context + 1 > self->pages_per_slot * kPage) continue;
        const size_t pages = (context + 1 + kPage - 1) / kPage;
        size_t previous = 0;
        for (size_t sequences : batches) {
            if (sequences == previous || sequences * pages > self->model->num_pages) continue;
            previous = sequences;
            std::fill(table.begin(), table.end(), 0xffffffffu);
            StepShape shape;
            for (size_t slot = 0; slot < sequences; ++slot) {
                for (size_t page = 0; page < pages; ++page) {
                    table[slot * self->pages_per_slot + page] = static_cast<uint32_t>(slot * pages + page);
                }
                shape.prefixes.push_back(context);
                shape.chunks.push_back(1);
                shape.segment_slots.push_back(static_cast<uint32_t>(slot));
                shape.token_ids.push_back(0);
            }
            double milliseconds = 0.0;
            ENGINE_TRY(timed(shape, &milliseconds));
            decode_points.push_back({sequences, 1, context, milliseconds});
        }
    }
    for (size_t chunk : {size_t(16), size_t(64), size_t(128), size_t(256), size_t(512)}) {
        if (chunk > self->config.max_prefill_tokens || chunk > self->pages_per_slot * kPage) continue;
        std::fill(table.begin(), table.end(), 0xffffffffu);
        for (size_t page = 0; page < (chunk + kPage - 1) / kPage; ++page) {
            table[page] = static_cast<uint32_t>(page);
        }
        StepShape shape;
        shape.prefixes.push_back(0);
        shape.chunks.push_back(chunk);
        shape.segment_slots.push_back(0);
        shape.token_ids.assign(chunk, 0);
        double milliseconds = 0.0;
        ENGINE_TRY(timed(shape, &milliseconds));
        prefill_points.push_back({1, chunk, chunk, milliseconds});
    }
    if (decode_points.empty() || prefill_points.empty()) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "engine limits leave no point to calibrate on");
    }
    for (size_t slot = 0; slot < self->config.max_slots; ++slot) {
        ENGINE_TRY(clear_conv_state(self, slot));
    }
    self->tables_dirty = true;
    lfm25_cost_model_destroy(self->cost);
    self->cost = nullptr;
    return lfm25_cost_model_create(decode_points.data(), decode_points.size(), decode_points.data(),
                                   decode_points.size(), prefill_points.data(), prefill_points.size(), kPage,
                                   &self->cost);
}

const lfm25_cost_model* lfm25_engine_cost_model(const lfm25_engine* self) {
    return self != nullptr ? self->cost : nullptr;
}

int32_t lfm25_engine_submit(lfm25_engine* self, uint64_t request_id, const uint32_t* prompt, size_t prompt_len,
                            size_t max_new_tokens, uint64_t arrival_us) {
    if (self == nullptr || prompt == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "engine submit received a null argument");
    }
    if (prompt_len == 0) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "request prompt is empty");
    if (max_new_tokens == 0) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "request asks for no tokens");
    // with admission control an oversized request is answered by a rejection event at the next step
    if (self->config.admission_control == 0 && prompt_len + max_new_tokens > self->pages_per_slot * kPage) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "request exceeds fixed token capacity");
    }
    self->queue.push_back({request_id, std::vector<uint32_t>(prompt, prompt + prompt_len), max_new_tokens, arrival_us});
    return LFM25_OK;
}

int32_t lfm25_engine_step(lfm25_engine* self, uint64_t now_us, lfm25_engine_event* events, size_t events_capacity,
                          size_t* num_events, float* gpu_ms) {
    if (self == nullptr || num_events == nullptr || (events == nullptr && events_capacity > 0)) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "engine step received a null argument");
    }
    if (events_capacity < self->config.max_slots * (self->config.admission_control != 0 ? 2 : 1)) {
        return lfm25::report_error(LFM25_ERR_BUFFER_TOO_SMALL,
                                   "event buffer smaller than the request slots (twice that with admission control)");
    }
    if (self->cost == nullptr) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "calibrate the engine before its first step");
    }
    *num_events = 0;
    if (gpu_ms != nullptr) *gpu_ms = 0.0f;
    // rejections go first into the event buffer; the step's token events (at most one per slot) follow them
    size_t rejected = 0;
    ENGINE_TRY(admit(self, now_us, events, events_capacity - self->config.max_slots, &rejected));
    *num_events = rejected;

    for (size_t index = 0; index < self->slots.size(); ++index) {
        const Slot& slot = self->slots[index];
        lfm25_request_view& view = self->views[index];
        view.phase = slot.phase;
        view.prompt_len = slot.prompt_len;
        view.prefilled = slot.prefilled;
        view.context_tokens = slot.tokens.size();
        view.arrival_us = slot.arrival_us;
        view.first_token_deadline_us = slot.first_token_deadline_us;
        view.next_token_deadline_us = slot.next_token_deadline_us;
    }
    lfm25_scheduler_config planner;
    planner.step_budget_ms = self->config.step_budget_ms;
    planner.ttft_slo_us = self->config.ttft_slo_us;
    planner.tpot_slo_us = self->config.tpot_slo_us;
    planner.fp8_decode = self->config.use_fp8;
    planner.maximum_prefill_tokens = self->config.max_prefill_tokens;
    lfm25_batch_plan plan;
    ENGINE_TRY(lfm25_schedule(self->cost, &planner, self->views.data(), self->views.size(), now_us, self->work.data(),
                              self->work.size(), &plan));
    if (plan.work_count == 0) {
        return LFM25_OK;
    }

    StepShape shape;
    self->grow_from.clear();
    self->grow_to.clear();
    for (size_t index = 0; index < plan.work_count; ++index) {
        lfm25_scheduled_work& item = self->work[index];
        Slot& slot = self->slots[item.slot];
        size_t begin;
        size_t count = item.tokens;
        if (item.kind == LFM25_WORK_PREFILL) {
            // split_prefill_at_reusable_boundary: end the chunk at the last full page before the final prompt token,
            // so that the prefix published there can serve a later identical prompt
            const size_t limit = reusable_limit(slot.prompt_len);
            if (limit > 0 && slot.prefilled < limit && limit < slot.prefilled + count) {
                count = limit - slot.prefilled;
            }
            begin = slot.prefilled;
            shape.token_ids.insert(shape.token_ids.end(), slot.tokens.begin() + begin, slot.tokens.begin() + begin + count);
        } else {
            begin = slot.tokens.size() - 1;
            count = 1;
            shape.token_ids.push_back(slot.tokens.back());
        }
        item.tokens = count;
        self->grow_from.push_back(slot.cached_tokens);
        self->grow_to.push_back(begin + count);
        shape.prefixes.push_back(begin);
        shape.chunks.push_back(count);
        shape.segment_slots.push_back(item.slot);
    }
    // All the sequences of the step grow or none does: a shortage found half way would leave rows of the block
    // tables pointing at pages that their slots do not account for yet.
    const int64_t short_by = lfm25_kv_allocator_pages_short(self->allocator, self->grow_from.data(), self->grow_to.data(),
                                                            plan.work_count);
    if (short_by != 0) {
        return lfm25::report_error(short_by < 0 ? static_cast<int32_t>(short_by) : LFM25_KV_PHYSICAL_PAGES_EXHAUSTED,
                                   "KV pages exhausted inside a reservation");
    }
    for (size_t index = 0; index < plan.work_count; ++index) {
        const lfm25_scheduled_work& item = self->work[index];
        const int64_t grown = lfm25_kv_allocator_grow_sequence(self->allocator, self->grow_from[index], self->grow_to[index],
                                                               lfm25_block_tables_slot(self->tables, item.slot),
                                                               self->pages_per_slot);
        if (grown != 0) self->tables_dirty = true;        // also on an error: rows may have changed
        if (grown < 0) return lfm25::report_error(static_cast<int32_t>(grown), "KV pages exhausted inside a reservation");
    }
    if (self->tables_dirty) {
        ENGINE_TRY(upload_tables(self, lfm25_block_tables_data(self->tables)));
        self->tables_dirty = false;
    }
    cudaEventRecord(self->start, self->stream());
    ENGINE_TRY(enqueue_step(self, shape));
    cudaEventRecord(self->stop, self->stream());
    ENGINE_TRY(lfm25_decode_executor_download_sampled(self->executor, self->h_sampled, plan.work_count));
    cudaError_t status = cudaStreamSynchronize(self->stream());
    if (status != cudaSuccess) return cuda_failure(status, "serving step failed");
    float elapsed = 0.0f;
    cudaEventElapsedTime(&elapsed, self->start, self->stop);
    if (gpu_ms != nullptr) *gpu_ms = elapsed;
    const uint64_t done_us = now_us + static_cast<uint64_t>(elapsed * 1000.0f);

    self->stats.steps += 1;
    if (shape.token_ids.size() == plan.work_count) {
        self->stats.decode_steps += 1;
    } else {
        self->stats.mixed_steps += 1;
    }
    self->stats.gpu_ms += elapsed;
    size_t produced = rejected;
    for (size_t index = 0; index < plan.work_count; ++index) {
        const lfm25_scheduled_work& item = self->work[index];
        Slot& slot = self->slots[item.slot];
        slot.cached_tokens = shape.prefixes[index] + shape.chunks[index];
        if (item.kind == LFM25_WORK_PREFILL) {
            slot.prefilled += shape.chunks[index];
            self->stats.prefill_tokens += shape.chunks[index];
            if (slot.prefilled % kPage == 0 && self->checkpoints != nullptr) {
                ENGINE_TRY(publish(self, item.slot, slot));
            }
            if (slot.prefilled < slot.prompt_len) {
                continue;
            }
        }
        const uint32_t token = self->h_sampled[index];
        slot.tokens.push_back(token);
        slot.phase = LFM25_PHASE_DECODING;
        slot.next_token_deadline_us = done_us + self->config.tpot_slo_us;
        self->stats.generated_tokens += 1;
        const bool finished = slot.tokens.size() - slot.prompt_len >= slot.max_new_tokens;
        lfm25_engine_event& event = events[produced++];
        event.request_id = slot.request_id;
        event.token = token;
        event.finished = finished ? 1u : 0u;
        event.reused_tokens = static_cast<uint32_t>(slot.reused_tokens);
        event.rejected = LFM25_REJECT_NONE;
        event.time_us = done_us;
        if (finished) {
            release(self, item.slot);
        }
    }
    *num_events = produced;
    return LFM25_OK;
}

size_t lfm25_engine_active(const lfm25_engine* self) {
    if (self == nullptr) return 0;
    size_t active = 0;
    for (const Slot& slot : self->slots) {
        if (slot.phase != LFM25_PHASE_FREE) ++active;
    }
    return active;
}

size_t lfm25_engine_queued(const lfm25_engine* self) { return self != nullptr ? self->queue.size() : 0; }

void lfm25_engine_get_stats(const lfm25_engine* self, lfm25_engine_stats* stats, lfm25_kv_pool_snapshot* pool,
                            lfm25_prefix_cache_snapshot* prefix) {
    if (self == nullptr) return;
    if (stats != nullptr) *stats = self->stats;
    if (pool != nullptr) lfm25_kv_allocator_snapshot(self->allocator, pool);
    if (prefix != nullptr) lfm25_radix_cache_snapshot(self->radix, prefix);
}

}  // extern "C"
