// Decode executor: one continuous-batching decode step of the LFM2.5-1.2B architecture on fixed-address
// scratch, with the step metadata advanced on the device and the whole step replayed from a CUDA graph.
//
// Replaces the reference's DecodeExecutor (src/model/decode_executor.rs:127-155 scratch, :183-443 step) and
// the host work around it (BatchModelCache::prepare_tokens, src/model/lfm2_base.rs:322-388; GpuBatch::update_*,
// src/scheduler/batch.rs:142-260).  The op sequence is the reference's; what changes is who runs it:
//   * positions, token ids and physical slots live on the device and are advanced by a kernel at the head of
//     the step (the sampled ids of the previous step feed the next one), so a step needs no H2D copy and no
//     host synchronisation;
//   * every kernel argument is a fixed device pointer, so one captured graph per batch size replays unchanged.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>
#include <utility>
#include <vector>

#include "../../include/lfm25_b200.h"
#include "blaslt_handle.h"
#include "kernels.h"
#include "options.h"

namespace {

constexpr size_t kHidden = 2048;
constexpr size_t kQueryWidth = 2048;
constexpr size_t kKvWidth = 512;
constexpr size_t kFfn = 8192;
constexpr size_t kVocab = 65536;

}  // namespace

struct lfm25_decode_executor {
    lfm25_blaslt* blaslt;
    size_t maximum_tokens;
    size_t maximum_rows;   // rows that get logits in one step (= sequences in it): decode tokens / segments
    void* allocation;
    // scratch, fixed addresses (src/model/decode_executor.rs:6-22)
    void* hidden;
    void* normalized;
    void* post_operator;
    void* operator_output;
    void* query;
    void* key;
    void* value;
    void* wide;
    void* activated;
    void* logits;
    void* fp8_input;
    float* partials;
    uint32_t* sampled;
    void* head_input;      // [maximum_rows, 2048]: the rows that go to the LM head in a mixed step
    uint32_t* token_order; // [maximum_rows]: the step's tokens, longest context first (written by the metadata kernel)
    // opt-in region timing (the reference's ModelProfileRecorder, src/model/profile.rs:84-253): CUDA-event pairs
    // around every op of an eager step, summed per region
    bool profiling = false;
    std::vector<std::pair<int, std::pair<cudaEvent_t, cudaEvent_t>>> marks;
    // captured steps: one per (batch size, attention split count, flags, buffers); a serving loop walks through many
    // batch sizes, so the table is large and the least recently used entry is recycled
    struct Captured {
        size_t num_tokens = 0;
        size_t splits = 0;
        uint32_t use_fp8 = 0;
        uint32_t advance = 0;
        uint64_t signature = 0;   // of everything else the graph bakes in, see step_signature()
        bool warmed = false;
        cudaGraphExec_t exec = nullptr;
        size_t kernel_nodes = 0;
        uint64_t last_used = 0;
    } captured[96];
    uint64_t graph_clock = 0;
    size_t last_graph_kernel_nodes = 0;   // of the graph launched most recently
    size_t graph_captures = 0;            // captures made so far
};

namespace {

// Times one op of an eager step when profiling is on; a no-op otherwise (and always during graph capture).
struct RegionTimer {
    lfm25_decode_executor* self;
    cudaEvent_t start = nullptr;
    cudaEvent_t stop = nullptr;
    int region;
    RegionTimer(lfm25_decode_executor* executor, int which) : self(executor), region(which) {
        if (self->profiling && cudaEventCreate(&start) == cudaSuccess && cudaEventCreate(&stop) == cudaSuccess) {
            cudaEventRecord(start, self->blaslt->stream);
        }
    }
    ~RegionTimer() {
        if (self->profiling && start != nullptr && stop != nullptr) {
            cudaEventRecord(stop, self->blaslt->stream);
            self->marks.push_back({region, {start, stop}});
        }
    }
};

// A captured step bakes in every kernel argument: all pointers of the batch (token ids, positions, slots, block
// tables, their stride and row count), the page count inside the TMA tensor maps, and every weight, norm, state and
// cache pointer, shape and scale of the model -- the contents of model->layers, not just its address.  The
// signature hashes all of them (and the switches that change which kernels a step launches), so a caller who
// regrows a block table, resizes the pool or swaps weights under the same array gets a fresh capture instead of a
// replay of stale arguments.
struct Fnv1a {
    uint64_t state = 1469598103934665603ull;
    void word(uint64_t value) { state = (state ^ value) * 1099511628211ull; }
    template <typename Value>
    void add(const Value& value) {   // values of up to 8 bytes are mixed in one step, longer ones word by word
        static_assert(sizeof(Value) % 4 == 0, "hashed fields are 4-byte multiples");
        const unsigned char* cursor = reinterpret_cast<const unsigned char*>(&value);
        for (size_t offset = 0; offset < sizeof(Value); offset += 4) {
            uint32_t part;
            memcpy(&part, cursor + offset, 4);
            word(part);
        }
    }
    void linear(const lfm25_linear_weights& weights) {
        add(weights.bf16);
        add(weights.fp8.data);
        add(weights.fp8.activation_quantize);
        add(weights.fp8.activation_dequantize);
        add(weights.fp8.weight_dequantize);
        add(weights.n);
        add(weights.k);
    }
};

uint64_t step_signature(const lfm25_decode_executor* self, const lfm25_model* model, const lfm25_decode_batch* batch) {
    Fnv1a hash;
    hash.add(batch->token_ids);
    hash.add(batch->positions);
    hash.add(batch->request_slots);
    hash.add(batch->physical_slots);
    hash.add(batch->block_tables);
    hash.add(batch->block_table_stride);
    hash.add(batch->block_table_rows);
    hash.add(model->num_layers);
    hash.add(model->layers);
    hash.add(model->embedding);
    hash.add(model->lm_head_fp8.data);
    hash.add(model->lm_head_fp8.activation_quantize);
    hash.add(model->lm_head_fp8.activation_dequantize);
    hash.add(model->lm_head_fp8.weight_dequantize);
    hash.add(model->final_norm);
    hash.add(model->inv_freq);
    hash.add(model->norm_eps);
    hash.add(model->num_pages);
    hash.add(model->num_request_slots);
    for (uint32_t index = 0; index < model->num_layers; ++index) {
        const lfm25_layer& layer = model->layers[index];
        hash.add(layer.is_attention);
        hash.add(layer.operator_norm);
        hash.add(layer.ffn_norm);
        hash.linear(layer.conv_input);
        hash.add(layer.conv_kernel);
        hash.linear(layer.conv_output);
        hash.add(layer.conv_state);
        hash.linear(layer.query);
        hash.linear(layer.key);
        hash.linear(layer.value);
        hash.linear(layer.output);
        hash.add(layer.query_norm);
        hash.add(layer.key_norm);
        hash.add(layer.key_cache);
        hash.add(layer.value_cache);
        hash.linear(layer.gate_up);
        hash.linear(layer.down);
    }
    for (int which = 0; which < lfm25::kOptCount; ++which) {
        if (which != lfm25::kOptEngineGraph) {
            hash.add(lfm25::option(static_cast<lfm25::Option>(which)));
        }
    }
    hash.add(self->blaslt->tuning_kernel);
    hash.add(self->blaslt->tuning);
    hash.add(self->blaslt->stream);
    return hash.state;
}

int32_t cuda_failure(cudaError_t status, const char* what) {
    char message[200];
    snprintf(message, sizeof message, "%s: %s", what, cudaGetErrorString(status));
    return lfm25::report_error(LFM25_ERR_CUDA, message);
}

#define LFM25_TRY(expression)          \
    do {                               \
        const int32_t rc = (expression); \
        if (rc != LFM25_OK) {          \
            return rc;                 \
        }                              \
    } while (0)

lfm25_slice slice_of(const void* pointer, size_t elements) {
    lfm25_slice slice;
    slice.ptr = const_cast<void*>(pointer);
    slice.len = elements;
    return slice;
}

// linear_decode_into (src/model/decode_executor.rs:78-124): FP8 when the site is promoted and FP8 is on
// (quantise the activation with the site's static scale, then the E4M3 GEMM with alpha = d_x * d_w), else BF16.
// `prequantized`: fp8_input already holds the codes of `input` (the producing norm wrote them).
int32_t linear_decode(lfm25_decode_executor* self, const lfm25_linear_weights& weights, const void* input,
                      void* output, size_t rows, bool use_fp8, bool prequantized = false) {
    if (use_fp8 && weights.fp8.data != nullptr) {
        RegionTimer timer(self, LFM25_REGION_FP8_LINEAR);
        if (!prequantized) {
            LFM25_TRY(lfm25_quantize_bf16_e4m3(self->blaslt->stream, slice_of(input, rows * weights.k),
                                               slice_of(self->fp8_input, self->maximum_tokens * kFfn),
                                               rows * weights.k, weights.fp8.activation_quantize));
        }
        lfm25_fp8_linear_config config;
        config.m = rows;
        config.n = weights.n;
        config.k = weights.k;
        config.scale_mode = LFM25_FP8_SCALE_TENSORWIDE;
        config.output_scale = weights.fp8.activation_dequantize * weights.fp8.weight_dequantize;
        return lfm25_blaslt_linear_fp8_scaled(self->blaslt, slice_of(self->fp8_input, rows * weights.k),
                                              slice_of(weights.fp8.data, weights.n * weights.k),
                                              slice_of(output, rows * weights.n), &config);
    }
    if (weights.bf16 == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "linear site has neither BF16 nor FP8 weights resident");
    }
    RegionTimer timer(self, LFM25_REGION_BF16_LINEAR);
    return lfm25_blaslt_linear_bf16(self->blaslt, slice_of(input, rows * weights.k),
                                    slice_of(weights.bf16, weights.n * weights.k), slice_of(output, rows * weights.n),
                                    rows, weights.n, weights.k);
}

// Whether the KV splits of a token should merge inside the attention kernel (one cluster per token and KV head,
// no records, no merge kernel) or through records and the merge kernel.  The cluster saves a launch, but its CTAs
// leave their SM only together, which costs once the grid runs in several waves.  Whole decode step on a B200, ms per
// step without / with the in-kernel merge (sequences, splits): 1 (8) 0.662 / 0.644, 4 (8) 0.675 / 0.655,
// 8 (8) 0.693 / 0.688, 12 (4) 0.709 / 0.701, 16 (4) 0.715 / 0.726, 24 (4) 0.757 / 0.758, 28 (2) 0.783 / 0.774,
// 48 (2) 0.915 / 0.900, 64 (2) 1.012 / 1.026.
bool merge_in_kernel_preferred(size_t tokens, size_t splits) {
    const size_t ctas = tokens * 8 * splits;
    if (splits == 8) return ctas <= 512;
    if (splits == 4) return ctas <= 384;
    if (splits == 2) return ctas <= 768;
    return false;
}

int32_t forward(lfm25_decode_executor* self, const lfm25_model* model, const lfm25_decode_batch* batch, bool use_fp8,
                bool advance) {
    cudaStream_t stream = self->blaslt->stream;
    const size_t tokens = batch->num_tokens;
    cudaError_t status = cudaSuccess;
    const bool ordered = tokens <= 256;   // the metadata kernel orders the tokens only when one CTA covers the batch
    {
    RegionTimer timer(self, LFM25_REGION_OTHER);
    status = lfm25::launch_decode_metadata(
        stream, batch->token_ids, batch->positions, batch->request_slots, batch->block_tables, self->sampled,
        batch->physical_slots, tokens, batch->block_table_stride, batch->block_table_rows, model->num_pages, advance,
        self->token_order);
    if (status != cudaSuccess) return cuda_failure(status, "step metadata launch failed");
    status = lfm25::launch_embedding_bf16(stream, batch->token_ids, model->embedding, self->hidden, tokens, kVocab,
                                          kHidden);
    if (status != cudaSuccess) return cuda_failure(status, "embedding launch failed");
    status = lfm25::launch_rms_norm_bf16(stream, self->hidden, model->layers[0].operator_norm, self->normalized,
                                         tokens, kHidden, model->norm_eps);
    if (status != cudaSuccess) return cuda_failure(status, "rms_norm launch failed");
    }

    for (uint32_t index = 0; index < model->num_layers; ++index) {
        const lfm25_layer& layer = model->layers[index];
        if (!layer.is_attention) {
            LFM25_TRY(linear_decode(self, layer.conv_input, self->normalized, self->wide, tokens, use_fp8));
            RegionTimer timer(self, LFM25_REGION_OTHER);
            status = lfm25::launch_short_conv_decode(stream, self->wide, layer.conv_kernel, layer.conv_state,
                                                     batch->request_slots, self->post_operator, tokens, kHidden,
                                                     model->num_request_slots);
            if (status != cudaSuccess) return cuda_failure(status, "short_conv launch failed");
            LFM25_TRY(linear_decode(self, layer.conv_output, self->post_operator, self->operator_output, tokens,
                                    use_fp8));
        } else {
            // 0 = two launches, 1 = one kernel, 2 = whichever the measured table prefers for this batch
            const int64_t route = lfm25::option(lfm25::kOptFusedAppend);
            const bool fused_append =
                route == 2 ? lfm25_decode_one_kernel_preferred(16, batch->max_context_tokens, tokens) != 0 : route != 0;
            // One GEMM for the three projections when their BF16 matrices are adjacent in memory (q | k | v rows of
            // one [3072, 2048] allocation): the outputs then sit side by side in `wide`, [tokens, 3072]; the one-kernel
            // attention and the QK-norm + RoPE + append kernel both take token strides.
            const uint16_t* query_weight = static_cast<const uint16_t*>(layer.query.bf16);
            const bool packed_qkv = query_weight != nullptr &&
                                    !(use_fp8 && (layer.query.fp8.data || layer.key.fp8.data || layer.value.fp8.data)) &&
                                    layer.key.bf16 == query_weight + kQueryWidth * kHidden &&
                                    layer.value.bf16 == query_weight + (kQueryWidth + kKvWidth) * kHidden &&
                                    layer.query.k == kHidden && layer.key.k == kHidden && layer.value.k == kHidden;
            constexpr size_t kPackedWidth = kQueryWidth + 2 * kKvWidth;
            if (packed_qkv) {
                lfm25_linear_weights packed = layer.query;
                packed.n = kPackedWidth;
                LFM25_TRY(linear_decode(self, packed, self->normalized, self->wide, tokens, false));
            } else {
                LFM25_TRY(linear_decode(self, layer.query, self->normalized, self->query, tokens, use_fp8));
                LFM25_TRY(linear_decode(self, layer.key, self->normalized, self->key, tokens, use_fp8));
                LFM25_TRY(linear_decode(self, layer.value, self->normalized, self->value, tokens, use_fp8));
            }
            const size_t cache_elements = model->num_pages * 8 * 16 * 64;
            lfm25_qk_postprocess_launch post;
            post.page_size = 16;
            post.query = slice_of(self->query, tokens * kQueryWidth);
            post.key = slice_of(self->key, tokens * kKvWidth);
            post.value = slice_of(self->value, tokens * kKvWidth);
            post.query_norm = slice_of(layer.query_norm, 64);
            post.key_norm = slice_of(layer.key_norm, 64);
            post.inv_freq = slice_of(model->inv_freq, 32);
            post.position_ids = slice_of(batch->positions, tokens);
            post.slot_mapping = slice_of(batch->physical_slots, tokens);
            post.key_cache = slice_of(layer.key_cache, cache_elements);
            post.value_cache = slice_of(layer.value_cache, cache_elements);
            post.num_tokens = tokens;
            post.num_pages = model->num_pages;
            post.eps = model->norm_eps;
            const size_t splits = lfm25_splitk_decode_splits(tokens, batch->max_context_tokens, 16);
            // the splits of a token merge inside the attention kernel (a cluster per token and KV head) instead of
            // through records in global memory and a merge kernel
            const bool in_kernel_merge = lfm25::option(lfm25::kOptSplitkClusterMerge) != 0 &&
                                         merge_in_kernel_preferred(tokens, splits);
            if (fused_append) {
                // one launch: QK-norm + RoPE + paged append + attention (+ merge when split)
                RegionTimer timer(self, LFM25_REGION_ATTENTION);
                lfm25_fused_ragged_decode_launch fused;
                fused.page_size = 16;
                fused.query_raw = post.query;
                fused.key_raw = post.key;
                fused.value_raw = post.value;
                fused.query_norm = post.query_norm;
                fused.key_norm = post.key_norm;
                fused.inv_freq = post.inv_freq;
                fused.key_cache = post.key_cache;
                fused.value_cache = post.value_cache;
                fused.position_ids = post.position_ids;
                fused.slot_mapping = post.slot_mapping;
                fused.output = slice_of(self->post_operator, tokens * kHidden);
                fused.num_tokens = tokens;
                fused.num_pages = model->num_pages;
                fused.eps = model->norm_eps;
                fused.block_tables = slice_of(batch->block_tables, batch->block_table_stride * batch->block_table_rows);
                fused.request_slots = slice_of(batch->request_slots, tokens);
                fused.block_table_stride = batch->block_table_stride;
                fused.partials = in_kernel_merge
                                     ? slice_of(static_cast<float*>(nullptr), 0)
                                     : slice_of(self->partials, lfm25_splitk_workspace_elements(self->maximum_rows));
                fused.num_splits = splits;
                fused.query_token_stride = 0;
                fused.kv_token_stride = 0;
                fused.token_order = slice_of(ordered ? self->token_order : nullptr, ordered ? tokens : 0);
                if (packed_qkv) {
                    uint16_t* packed_rows = static_cast<uint16_t*>(self->wide);
                    const size_t span = (tokens - 1) * kPackedWidth;
                    fused.query_raw = slice_of(packed_rows, span + kQueryWidth);
                    fused.key_raw = slice_of(packed_rows + kQueryWidth, span + kKvWidth);
                    fused.value_raw = slice_of(packed_rows + kQueryWidth + kKvWidth, span + kKvWidth);
                    fused.query_token_stride = kPackedWidth;
                    fused.kv_token_stride = kPackedWidth;
                }
                LFM25_TRY(lfm25_fused_ragged_paged_attention_decode_lfm2_bf16(stream, &fused));
            } else {
            if (packed_qkv) {
                // the packed projection is read in place; the rotated query goes to the dense array attention reads
                RegionTimer timer(self, LFM25_REGION_APPEND);
                const uint16_t* packed_rows = static_cast<const uint16_t*>(self->wide);
                lfm25::QkPostprocessArgs strided;
                strided.query = packed_rows;
                strided.query_out = self->query;
                strided.query_token_stride = kPackedWidth;
                strided.kv_token_stride = kPackedWidth;
                strided.key = packed_rows + kQueryWidth;
                strided.value = packed_rows + kQueryWidth + kKvWidth;
                strided.query_norm = layer.query_norm;
                strided.key_norm = layer.key_norm;
                strided.inv_freq = static_cast<const float*>(model->inv_freq);
                strided.position_ids = static_cast<const uint32_t*>(batch->positions);
                strided.slot_mapping = static_cast<const int64_t*>(batch->physical_slots);
                strided.key_cache = layer.key_cache;
                strided.value_cache = layer.value_cache;
                strided.num_tokens = tokens;
                strided.num_pages = model->num_pages;
                strided.eps = model->norm_eps;
                const cudaError_t status = lfm25::launch_qk_norm_rope_kv_write_decode(stream, strided);
                if (status != cudaSuccess) return cuda_failure(status, "QK postprocess launch failed");
            } else {
                RegionTimer timer(self, LFM25_REGION_APPEND);
                LFM25_TRY(lfm25_qk_norm_rope_kv_write_decode(stream, &post));
            }
            {
            RegionTimer attention_timer(self, LFM25_REGION_ATTENTION);
            lfm25_splitk_ragged_attention_launch attention;
            attention.page_size = 16;
            attention.query = post.query;
            attention.key_cache = post.key_cache;
            attention.value_cache = post.value_cache;
            attention.block_tables = slice_of(batch->block_tables, batch->block_table_stride * batch->block_table_rows);
            attention.request_slots = slice_of(batch->request_slots, tokens);
            attention.position_ids = post.position_ids;
            attention.partials = in_kernel_merge
                                     ? slice_of(static_cast<float*>(nullptr), 0)
                                     : slice_of(self->partials, lfm25_splitk_workspace_elements(self->maximum_rows));
            attention.output = slice_of(self->post_operator, tokens * kHidden);
            attention.num_tokens = tokens;
            attention.num_pages = model->num_pages;
            attention.block_table_stride = batch->block_table_stride;
            attention.num_splits = splits;
            attention.token_order = slice_of(ordered ? self->token_order : nullptr, ordered ? tokens : 0);
            if (splits > 1) {
                LFM25_TRY(lfm25_paged_ragged_attention_splitk_lfm2_bf16(stream, &attention));
            } else {
                lfm25_fast_ragged_attention_launch unsplit;
                unsplit.token_order = attention.token_order;
                unsplit.page_size = 16;
                unsplit.query = attention.query;
                unsplit.key_cache = attention.key_cache;
                unsplit.value_cache = attention.value_cache;
                unsplit.block_tables = attention.block_tables;
                unsplit.request_slots = attention.request_slots;
                unsplit.position_ids = attention.position_ids;
                unsplit.output = attention.output;
                unsplit.num_tokens = tokens;
                unsplit.num_pages = model->num_pages;
                unsplit.block_table_stride = batch->block_table_stride;
                LFM25_TRY(lfm25_paged_ragged_attention_fast_lfm2_bf16(stream, &unsplit));
            }
            }
            }
            LFM25_TRY(linear_decode(self, layer.output, self->post_operator, self->operator_output, tokens, use_fp8));
        }

        // the norm in front of an FP8 Gate/Up also writes the E4M3 codes the GEMM reads (one launch less)
        const bool gate_up_fp8 = use_fp8 && layer.gate_up.fp8.data != nullptr && layer.gate_up.k == kHidden;
        {
            RegionTimer timer(self, LFM25_REGION_OTHER);
            status = lfm25::launch_residual_rms_norm_bf16(
                stream, self->hidden, self->operator_output, layer.ffn_norm, self->post_operator, self->normalized,
                tokens, kHidden, model->norm_eps, gate_up_fp8 ? self->fp8_input : nullptr,
                gate_up_fp8 ? layer.gate_up.fp8.activation_quantize : 1.0f);
        }
        if (status != cudaSuccess) return cuda_failure(status, "residual_rms_norm launch failed");

        // An FP8 Gate/Up whose shape the tensor-core kernel takes runs with SiLU(gate) * up in its epilogue: the
        // packed projection is never written, and the activation arrives as the Down site's E4M3 codes or as bf16.
        const bool fuse_gate = lfm25::option(lfm25::kOptFusedSilu) != 0;
        const bool down_fp8 = use_fp8 && layer.down.fp8.data != nullptr;
        bool gate_fused = false;
        if (fuse_gate && gate_up_fp8 && layer.gate_up.n == 2 * kFfn && (down_fp8 || layer.down.bf16 != nullptr)) {
            RegionTimer timer(self, LFM25_REGION_FP8_LINEAR);
            lfm25_fp8_linear_config config;
            config.m = tokens;
            config.n = 2 * kFfn;
            config.k = kHidden;
            config.scale_mode = LFM25_FP8_SCALE_TENSORWIDE;
            config.output_scale = layer.gate_up.fp8.activation_dequantize * layer.gate_up.fp8.weight_dequantize;
            // the codes of the normalised rows are in fp8_input; the activation's codes go to `activated` (the Down
            // GEMM reads them from there), the bf16 activation too
            const int32_t rc = lfm25_blaslt_linear_fp8_silu_mul(
                self->blaslt, slice_of(self->fp8_input, tokens * kHidden),
                slice_of(layer.gate_up.fp8.data, 2 * kFfn * kHidden),
                slice_of(self->activated, down_fp8 ? tokens * kFfn * 2 : tokens * kFfn), &config,
                down_fp8 ? layer.down.fp8.activation_quantize : 1.0f, down_fp8 ? 1u : 0u);
            if (rc == LFM25_OK) {
                gate_fused = true;
            } else if (rc != LFM25_ERR_UNSUPPORTED) {
                return rc;
            }
        }
        if (!gate_fused && fuse_gate && !gate_up_fp8 && layer.gate_up.bf16 != nullptr && layer.gate_up.n == 2 * kFfn &&
            layer.gate_up.k == kHidden && (down_fp8 || layer.down.bf16 != nullptr) &&
            lfm25::option(lfm25::kOptFusedSiluBf16) != 0) {
            // the same fusion for a Gate/Up site that stays in BF16 (batch-major tcgen05 kernel)
            RegionTimer timer(self, LFM25_REGION_BF16_LINEAR);
            const int32_t rc = lfm25_blaslt_linear_bf16_silu_mul(
                self->blaslt, slice_of(self->normalized, tokens * kHidden), slice_of(layer.gate_up.bf16, 2 * kFfn * kHidden),
                slice_of(self->activated, down_fp8 ? tokens * kFfn * 2 : tokens * kFfn), tokens, 2 * kFfn, kHidden,
                down_fp8 ? layer.down.fp8.activation_quantize : 1.0f, down_fp8 ? 1u : 0u);
            if (rc == LFM25_OK) {
                gate_fused = true;
            } else if (rc != LFM25_ERR_UNSUPPORTED) {
                return rc;
            }
        }
        if (gate_fused) {
            if (down_fp8) {
                RegionTimer timer(self, LFM25_REGION_FP8_LINEAR);
                lfm25_fp8_linear_config config;
                config.m = tokens;
                config.n = kHidden;
                config.k = kFfn;
                config.scale_mode = LFM25_FP8_SCALE_TENSORWIDE;
                config.output_scale = layer.down.fp8.activation_dequantize * layer.down.fp8.weight_dequantize;
                LFM25_TRY(lfm25_blaslt_linear_fp8_scaled(self->blaslt, slice_of(self->activated, tokens * kFfn),
                                                         slice_of(layer.down.fp8.data, kHidden * kFfn),
                                                         slice_of(self->operator_output, tokens * kHidden), &config));
            } else {
                RegionTimer timer(self, LFM25_REGION_BF16_LINEAR);
                LFM25_TRY(lfm25_blaslt_linear_bf16(self->blaslt, slice_of(self->activated, tokens * kFfn),
                                                   slice_of(layer.down.bf16, kHidden * kFfn),
                                                   slice_of(self->operator_output, tokens * kHidden), tokens, kHidden,
                                                   kFfn));
            }
        } else {
        LFM25_TRY(linear_decode(self, layer.gate_up, self->normalized, self->wide, tokens, use_fp8, gate_up_fp8));
        if (use_fp8 && layer.down.fp8.data != nullptr) {
            RegionTimer timer(self, LFM25_REGION_FP8_LINEAR);
            LFM25_TRY(lfm25_silu_mul_packed_bf16_to_e4m3(stream, slice_of(self->wide, tokens * 2 * kFfn),
                                                         slice_of(self->fp8_input, self->maximum_tokens * kFfn),
                                                         tokens, kFfn, layer.down.fp8.activation_quantize));
            lfm25_fp8_linear_config config;
            config.m = tokens;
            config.n = kHidden;
            config.k = kFfn;
            config.scale_mode = LFM25_FP8_SCALE_TENSORWIDE;
            config.output_scale = layer.down.fp8.activation_dequantize * layer.down.fp8.weight_dequantize;
            LFM25_TRY(lfm25_blaslt_linear_fp8_scaled(self->blaslt, slice_of(self->fp8_input, tokens * kFfn),
                                                     slice_of(layer.down.fp8.data, kHidden * kFfn),
                                                     slice_of(self->operator_output, tokens * kHidden), &config));
        } else {
            RegionTimer timer(self, LFM25_REGION_BF16_LINEAR);
            LFM25_TRY(lfm25_silu_mul_packed_bf16(stream, slice_of(self->wide, tokens * 2 * kFfn),
                                                 slice_of(self->activated, tokens * kFfn), tokens, kFfn));
            if (layer.down.bf16 == nullptr) {
                return lfm25::report_error(LFM25_ERR_NULL_POINTER, "Down site has no BF16 weights resident");
            }
            LFM25_TRY(lfm25_blaslt_linear_bf16(self->blaslt, slice_of(self->activated, tokens * kFfn),
                                               slice_of(layer.down.bf16, kHidden * kFfn),
                                               slice_of(self->operator_output, tokens * kHidden), tokens, kHidden,
                                               kFfn));
        }
        }

        const bool last_layer = index + 1 == model->num_layers;
        const void* next_norm = last_layer ? model->final_norm : model->layers[index + 1].operator_norm;
        const bool head_fp8 = last_layer && use_fp8 && model->lm_head_fp8.data != nullptr;
        {
            RegionTimer timer(self, LFM25_REGION_OTHER);
            status = lfm25::launch_residual_rms_norm_bf16(
                stream, self->post_operator, self->operator_output, next_norm, self->hidden, self->normalized, tokens,
                kHidden, model->norm_eps, head_fp8 ? self->fp8_input : nullptr,
                head_fp8 ? model->lm_head_fp8.activation_quantize : 1.0f);
        }
        if (status != cudaSuccess) return cuda_failure(status, "residual_rms_norm launch failed");
    }

    // tied LM head: the embedding matrix, FP8 when promoted
    lfm25_linear_weights head;
    head.bf16 = model->embedding;
    head.fp8 = model->lm_head_fp8;
    head.n = kVocab;
    head.k = kHidden;
    LFM25_TRY(linear_decode(self, head, self->normalized, self->logits, tokens, use_fp8,
                            use_fp8 && model->lm_head_fp8.data != nullptr));
    {
        RegionTimer timer(self, LFM25_REGION_OTHER);
        status = lfm25::launch_argmax_rows_bf16(stream, self->logits, self->sampled, tokens, kVocab);
    }
    if (status != cudaSuccess) return cuda_failure(status, "argmax launch failed");
    return LFM25_OK;
}

// The mixed prefill / decode step: Lfm2Model::forward_prepared_batch (src/model/lfm2_base.rs:924-997) with
// attention_batch's prefill branch (:1794-1829) and short_conv_batch (:1511-1530).  Differences from that op list:
// QK-norm, RoPE and the paged append are the one fused kernel of the decode route, applied to every token, and the
// attention kernel then reads all keys through the block tables (the chunk is already in the cache).
int32_t forward_ragged(lfm25_decode_executor* self, const lfm25_model* model, const lfm25_ragged_batch* batch,
                       bool use_fp8) {
    cudaStream_t stream = self->blaslt->stream;
    const size_t tokens = batch->num_tokens;
    const size_t segments = batch->num_segments;
    // FP8 sites only up to the batch the FP8 GEMM covers, as the reference does with maximum_fp8_batch
    // (src/model/lfm2_base.rs:929); larger steps run every site in BF16
    use_fp8 = use_fp8 && tokens <= 256;
    cudaError_t status = cudaSuccess;
    {
        RegionTimer timer(self, LFM25_REGION_OTHER);
        status = lfm25::launch_decode_metadata(stream, const_cast<uint32_t*>(batch->token_ids),
                                               const_cast<uint32_t*>(batch->positions), batch->request_slots,
                                               batch->block_tables, self->sampled, batch->physical_slots, tokens,
                                               batch->block_table_stride, batch->block_table_rows, model->num_pages,
                                               false);
        if (status != cudaSuccess) return cuda_failure(status, "step metadata launch failed");
        status = lfm25::launch_embedding_bf16(stream, batch->token_ids, model->embedding, self->hidden, tokens, kVocab,
                                              kHidden);
        if (status != cudaSuccess) return cuda_failure(status, "embedding launch failed");
        status = lfm25::launch_rms_norm_bf16(stream, self->hidden, model->layers[0].operator_norm, self->normalized,
                                             tokens, kHidden, model->norm_eps);
        if (status != cudaSuccess) return cuda_failure(status, "rms_norm launch failed");
    }
    // the leading decode tokens go through the decode attention kernel: order them longest context first, once per
    // step, for all attention layers
    const size_t leading_decodes = batch->num_decode_segments;
    const bool decodes_ordered = leading_decodes > 1 && leading_decodes <= lfm25::kMaxOrderTokens &&
                                 leading_decodes <= self->maximum_rows;
    if (decodes_ordered) {
        RegionTimer timer(self, LFM25_REGION_OTHER);
        status = lfm25::launch_context_order(stream, batch->positions, leading_decodes, self->token_order);
        if (status != cudaSuccess) return cuda_failure(status, "context order launch failed");
    }
    for (uint32_t index = 0; index < model->num_layers; ++index) {
        const lfm25_layer& layer = model->layers[index];
        if (!layer.is_attention) {
            LFM25_TRY(linear_decode(self, layer.conv_input, self->normalized, self->wide, tokens, use_fp8));
            {
                RegionTimer timer(self, LFM25_REGION_OTHER);
                status = lfm25::launch_short_conv_segmented(stream, self->wide, layer.conv_kernel, layer.conv_state,
                                                            batch->segment_offsets, batch->segment_slots,
                                                            self->post_operator, tokens, segments, kHidden,
                                                            model->num_request_slots);
            }
            if (status != cudaSuccess) return cuda_failure(status, "segmented short_conv launch failed");
            LFM25_TRY(linear_decode(self, layer.conv_output, self->post_operator, self->operator_output, tokens,
                                    use_fp8));
        } else {
            LFM25_TRY(linear_decode(self, layer.query, self->normalized, self->query, tokens, use_fp8));
            LFM25_TRY(linear_decode(self, layer.key, self->normalized, self->key, tokens, use_fp8));
            LFM25_TRY(linear_decode(self, layer.value, self->normalized, self->value, tokens, use_fp8));
            const size_t cache_elements = model->num_pages * 8 * 16 * 64;
            lfm25_qk_postprocess_launch post;
            post.page_size = 16;
            post.query = slice_of(self->query, tokens * kQueryWidth);
            post.key = slice_of(self->key, tokens * kKvWidth);
            post.value = slice_of(self->value, tokens * kKvWidth);
            post.query_norm = slice_of(layer.query_norm, 64);
            post.key_norm = slice_of(layer.key_norm, 64);
            post.inv_freq = slice_of(model->inv_freq, 32);
            post.position_ids = slice_of(batch->positions, tokens);
            post.slot_mapping = slice_of(batch->physical_slots, tokens);
            post.key_cache = slice_of(layer.key_cache, cache_elements);
            post.value_cache = slice_of(layer.value_cache, cache_elements);
            post.num_tokens = tokens;
            post.num_pages = model->num_pages;
            post.eps = model->norm_eps;
            {
                RegionTimer timer(self, LFM25_REGION_APPEND);
                LFM25_TRY(lfm25_qk_norm_rope_kv_write_decode(stream, &post));
            }
            const size_t decode_tokens = batch->num_decode_segments;
            const lfm25_slice tables_slice =
                slice_of(batch->block_tables, batch->block_table_stride * batch->block_table_rows);
            if (decode_tokens > 0) {
                // the leading single-token segments: the decode kernel (pages split over warps and, for long
                // contexts, over CTAs) instead of one 16-row tile per token
                RegionTimer timer(self, LFM25_REGION_ATTENTION);
                const size_t splits = lfm25_splitk_decode_splits(decode_tokens, batch->max_decode_context_tokens, 16);
                lfm25_splitk_ragged_attention_launch decode;
                decode.page_size = 16;
                decode.query = slice_of(self->query, decode_tokens * kQueryWidth);
                decode.key_cache = post.key_cache;
                decode.value_cache = post.value_cache;
                decode.block_tables = tables_slice;
                decode.request_slots = slice_of(batch->request_slots, decode_tokens);
                decode.position_ids = slice_of(batch->positions, decode_tokens);
                const bool in_kernel_merge = lfm25::option(lfm25::kOptSplitkClusterMerge) != 0 &&
                                             merge_in_kernel_preferred(decode_tokens, splits);
                decode.partials = in_kernel_merge
                                      ? slice_of(static_cast<float*>(nullptr), 0)
                                      : slice_of(self->partials, lfm25_splitk_workspace_elements(self->maximum_rows));
                decode.output = slice_of(self->post_operator, decode_tokens * kHidden);
                decode.num_tokens = decode_tokens;
                decode.num_pages = model->num_pages;
                decode.block_table_stride = batch->block_table_stride;
                decode.num_splits = splits;
                decode.token_order = slice_of(decodes_ordered ? self->token_order : nullptr,
                                              decodes_ordered ? decode_tokens : 0);
                if (splits > 1) {
                    LFM25_TRY(lfm25_paged_ragged_attention_splitk_lfm2_bf16(stream, &decode));
                } else {
                    lfm25_fast_ragged_attention_launch unsplit;
                    unsplit.page_size = 16;
                    unsplit.query = decode.query;
                    unsplit.key_cache = decode.key_cache;
                    unsplit.value_cache = decode.value_cache;
                    unsplit.block_tables = decode.block_tables;
                    unsplit.request_slots = decode.request_slots;
                    unsplit.position_ids = decode.position_ids;
                    unsplit.output = decode.output;
                    unsplit.num_tokens = decode_tokens;
                    unsplit.num_pages = model->num_pages;
                    unsplit.block_table_stride = batch->block_table_stride;
                    unsplit.token_order = decode.token_order;
                    LFM25_TRY(lfm25_paged_ragged_attention_fast_lfm2_bf16(stream, &unsplit));
                }
            }
            if (decode_tokens < segments) {
                RegionTimer timer(self, LFM25_REGION_ATTENTION);
                lfm25_hybrid_attention_launch attention;
                attention.page_size = 16;
                attention.query = post.query;
                attention.current_key = slice_of(nullptr, 0);
                attention.current_value = slice_of(nullptr, 0);
                attention.key_cache = post.key_cache;
                attention.value_cache = post.value_cache;
                attention.block_tables = tables_slice;
                attention.request_slots = slice_of(batch->request_slots, tokens);
                attention.position_ids = post.position_ids;
                // segment offsets are absolute token indices, so the remaining segments are simply a later start
                attention.segment_offsets = slice_of(batch->segment_offsets + decode_tokens, segments - decode_tokens + 1);
                attention.output = slice_of(self->post_operator, tokens * kHidden);
                attention.num_tokens = tokens;
                attention.num_pages = model->num_pages;
                attention.block_table_stride = batch->block_table_stride;
                attention.num_segments = segments - decode_tokens;
                attention.query_token_stride = 0;
                attention.kv_token_stride = 0;
                LFM25_TRY(lfm25_hybrid_ragged_attention_lfm2_bf16(stream, &attention));
            }
            LFM25_TRY(linear_decode(self, layer.output, self->post_operator, self->operator_output, tokens, use_fp8));
        }

        const bool gate_up_fp8 = use_fp8 && layer.gate_up.fp8.data != nullptr && layer.gate_up.k == kHidden;
        {
            RegionTimer timer(self, LFM25_REGION_OTHER);
            status = lfm25::launch_residual_rms_norm_bf16(
                stream, self->hidden, self->operator_output, layer.ffn_norm, self->post_operator, self->normalized,
                tokens, kHidden, model->norm_eps, gate_up_fp8 ? self->fp8_input : nullptr,
                gate_up_fp8 ? layer.gate_up.fp8.activation_quantize : 1.0f);
        }
        if (status != cudaSuccess) return cuda_failure(status, "residual_rms_norm launch failed");
        LFM25_TRY(linear_decode(self, layer.gate_up, self->normalized, self->wide, tokens, use_fp8, gate_up_fp8));
        if (use_fp8 && layer.down.fp8.data != nullptr) {
            RegionTimer timer(self, LFM25_REGION_FP8_LINEAR);
            LFM25_TRY(lfm25_silu_mul_packed_bf16_to_e4m3(stream, slice_of(self->wide, tokens * 2 * kFfn),
                                                         slice_of(self->fp8_input, self->maximum_tokens * kFfn),
                                                         tokens, kFfn, layer.down.fp8.activation_quantize));
            lfm25_fp8_linear_config config;
            config.m = tokens;
            config.n = kHidden;
            config.k = kFfn;
            config.scale_mode = LFM25_FP8_SCALE_TENSORWIDE;
            config.output_scale = layer.down.fp8.activation_dequantize * layer.down.fp8.weight_dequantize;
            LFM25_TRY(lfm25_blaslt_linear_fp8_scaled(self->blaslt, slice_of(self->fp8_input, tokens * kFfn),
                                                     slice_of(layer.down.fp8.data, kHidden * kFfn),
                                                     slice_of(self->operator_output, tokens * kHidden), &config));
        } else {
            RegionTimer timer(self, LFM25_REGION_BF16_LINEAR);
            LFM25_TRY(lfm25_silu_mul_packed_bf16(stream, slice_of(self->wide, tokens * 2 * kFfn),
                                                 slice_of(self->activated, tokens * kFfn), tokens, kFfn));
            if (layer.down.bf16 == nullptr) {
                return lfm25::report_error(LFM25_ERR_NULL_POINTER, "Down site has no BF16 weights resident");
            }
            LFM25_TRY(lfm25_blaslt_linear_bf16(self->blaslt, slice_of(self->activated, tokens * kFfn),
                                               slice_of(layer.down.bf16, kHidden * kFfn),
                                               slice_of(self->operator_output, tokens * kHidden), tokens, kHidden,
                                               kFfn));
        }
        const bool last_layer = index + 1 == model->num_layers;
        const void* next_norm = last_layer ? model->final_norm : model->layers[index + 1].operator_norm;
        {
            RegionTimer timer(self, LFM25_REGION_OTHER);
            status = lfm25::launch_residual_rms_norm_bf16(stream, self->post_operator, self->operator_output, next_norm,
                                                          self->hidden, self->normalized, tokens, kHidden,
                                                          model->norm_eps);
        }
        if (status != cudaSuccess) return cuda_failure(status, "residual_rms_norm launch failed");
    }

    // logits only for each segment's last token (gather_rows_bf16 on output_rows, lfm2_base.rs:984)
    {
        RegionTimer timer(self, LFM25_REGION_OTHER);
        status = lfm25::launch_gather_rows_bf16(stream, self->normalized, batch->output_rows, self->head_input, segments,
                                                tokens, kHidden);
    }
    if (status != cudaSuccess) return cuda_failure(status, "gather launch failed");
    lfm25_linear_weights head;
    head.bf16 = model->embedding;
    head.fp8 = model->lm_head_fp8;
    head.n = kVocab;
    head.k = kHidden;
    LFM25_TRY(linear_decode(self, head, self->head_input, self->logits, segments, use_fp8));
    {
        RegionTimer timer(self, LFM25_REGION_OTHER);
        status = lfm25::launch_argmax_rows_bf16(stream, self->logits, self->sampled, segments, kVocab);
    }
    if (status != cudaSuccess) return cuda_failure(status, "argmax launch failed");
    return LFM25_OK;
}

int32_t validate(const lfm25_decode_executor* self, const lfm25_model* model, const lfm25_decode_batch* batch) {
    if (self == nullptr || model == nullptr || batch == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "decode executor received a null argument");
    }
    if (batch->num_tokens == 0 || batch->num_tokens > self->maximum_tokens || batch->num_tokens > self->maximum_rows) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "decode executor token count exceeds workspace");
    }
    if (model->num_layers == 0 || model->layers == nullptr || model->embedding == nullptr ||
        model->final_norm == nullptr || model->inv_freq == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "decode executor model is incomplete");
    }
    if (!batch->token_ids || !batch->positions || !batch->request_slots || !batch->physical_slots ||
        !batch->block_tables || batch->block_table_stride == 0 || batch->block_table_rows == 0) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "decode batch metadata is incomplete");
    }
    return LFM25_OK;
}

}  // namespace

extern "C" {

int32_t lfm25_decode_executor_create(lfm25_blaslt* blaslt, size_t maximum_tokens, lfm25_decode_executor** out) {
    if (maximum_tokens == 0 || maximum_tokens > 256) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "decode executor supports 1..=256 tokens per step");
    }
    return lfm25_decode_executor_create_ragged(blaslt, maximum_tokens, maximum_tokens, out);
}

int32_t lfm25_decode_executor_create_ragged(lfm25_blaslt* blaslt, size_t maximum_tokens, size_t maximum_segments,
                                            lfm25_decode_executor** out) {
    if (blaslt == nullptr || out == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "decode executor needs a BlasLt handle and an output");
    }
    if (maximum_segments == 0 || maximum_segments > 256 || maximum_tokens < maximum_segments ||
        maximum_tokens > 8192) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT,
                                   "executor supports 1..=256 sequences and up to 8192 tokens per step");
    }
    lfm25_decode_executor* self = new (std::nothrow) lfm25_decode_executor();
    if (self == nullptr) {
        return lfm25::report_error(LFM25_ERR_CUDA, "failed to allocate the decode executor");
    }
    self->blaslt = blaslt;
    self->maximum_tokens = maximum_tokens;
    self->maximum_rows = maximum_segments;
    const size_t b = maximum_tokens;
    const size_t r = maximum_segments;
    const size_t sizes[15] = {
        b * kHidden * 2, b * kHidden * 2, b * kHidden * 2, b * kHidden * 2,         // hidden .. operator_output
        b * kQueryWidth * 2, b * kKvWidth * 2, b * kKvWidth * 2,                    // query, key, value
        b * 2 * kFfn * 2, b * kFfn * 2, r * kVocab * 2,                             // wide, activated, logits
        b * kFfn,                                                                   // fp8_input
        lfm25_splitk_workspace_elements(r) * sizeof(float), r * sizeof(uint32_t),   // partials, sampled
        r * kHidden * 2,                                                            // head_input
        r * sizeof(uint32_t)};                                                      // token_order
    size_t total = 0;
    size_t offsets[15];
    for (int index = 0; index < 15; ++index) {
        offsets[index] = total;
        total += (sizes[index] + 255) & ~static_cast<size_t>(255);
    }
    cudaError_t status = cudaMalloc(&self->allocation, total);
    if (status == cudaSuccess) {
        status = cudaMemsetAsync(self->allocation, 0, total, blaslt->stream);
    }
    if (status != cudaSuccess) {
        delete self;
        return cuda_failure(status, "failed to allocate decode scratch");
    }
    unsigned char* base = static_cast<unsigned char*>(self->allocation);
    void** fields[15] = {&self->hidden, &self->normalized, &self->post_operator, &self->operator_output, &self->query,
                         &self->key, &self->value, &self->wide, &self->activated, &self->logits, &self->fp8_input,
                         reinterpret_cast<void**>(&self->partials), reinterpret_cast<void**>(&self->sampled),
                         &self->head_input, reinterpret_cast<void**>(&self->token_order)};
    for (int index = 0; index < 15; ++index) {
        *fields[index] = base + offsets[index];
    }
    *out = self;
    return LFM25_OK;
}

void lfm25_decode_executor_destroy(lfm25_decode_executor* self) {
    if (self == nullptr) {
        return;
    }
    for (auto& entry : self->captured) {
        if (entry.exec != nullptr) {
            cudaGraphExecDestroy(entry.exec);
        }
    }
    cudaFree(self->allocation);
    delete self;
}

int32_t lfm25_decode_executor_download_sampled(lfm25_decode_executor* self, uint32_t* host, size_t count) {
    if (self == nullptr || host == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "sampled download received a null argument");
    }
    if (count > self->maximum_rows) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "sampled download exceeds the executor's capacity");
    }
    const cudaError_t status = cudaMemcpyAsync(host, self->sampled, count * sizeof(uint32_t), cudaMemcpyDeviceToHost,
                                               self->blaslt->stream);
    return status == cudaSuccess ? LFM25_OK : cuda_failure(status, "sampled download failed");
}

int32_t lfm25_decode_executor_download_logits(lfm25_decode_executor* self, void* host, size_t rows) {
    if (self == nullptr || host == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "logits download received a null argument");
    }
    if (rows > self->maximum_rows) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "logits download exceeds the executor's capacity");
    }
    const cudaError_t status = cudaMemcpyAsync(host, self->logits, rows * kVocab * 2, cudaMemcpyDeviceToHost,
                                               self->blaslt->stream);
    return status == cudaSuccess ? LFM25_OK : cuda_failure(status, "logits download failed");
}

const uint32_t* lfm25_decode_executor_sampled(const lfm25_decode_executor* self) {
    return self != nullptr ? self->sampled : nullptr;
}

const void* lfm25_decode_executor_logits(const lfm25_decode_executor* self) {
    return self != nullptr ? self->logits : nullptr;
}

int32_t lfm25_decode_executor_profile(lfm25_decode_executor* self, uint32_t enable, float region_ms[LFM25_REGION_COUNT],
                                      uint32_t region_launches[LFM25_REGION_COUNT]) {
    if (self == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "decode executor is null");
    }
    if (region_ms != nullptr) {
        // collect what has been recorded so far (synchronises the stream)
        const cudaError_t status = cudaStreamSynchronize(self->blaslt->stream);
        if (status != cudaSuccess) return cuda_failure(status, "profile synchronisation failed");
        for (int region = 0; region < LFM25_REGION_COUNT; ++region) {
            region_ms[region] = 0.0f;
            if (region_launches != nullptr) region_launches[region] = 0;
        }
        for (auto& mark : self->marks) {
            float elapsed = 0.0f;
            if (cudaEventElapsedTime(&elapsed, mark.second.first, mark.second.second) == cudaSuccess) {
                region_ms[mark.first] += elapsed;
                if (region_launches != nullptr) region_launches[mark.first] += 1;
            }
            cudaEventDestroy(mark.second.first);
            cudaEventDestroy(mark.second.second);
        }
        self->marks.clear();
    }
    self->profiling = enable != 0;
    return LFM25_OK;
}

int32_t lfm25_decode_executor_forward(lfm25_decode_executor* self, const lfm25_model* model,
                                      const lfm25_decode_batch* batch, uint32_t use_fp8, uint32_t advance) {
    LFM25_TRY(validate(self, model, batch));
    return forward(self, model, batch, use_fp8 != 0, advance != 0);
}

int32_t lfm25_decode_executor_forward_ragged(lfm25_decode_executor* self, const lfm25_model* model,
                                             const lfm25_ragged_batch* batch, uint32_t use_fp8) {
    if (self == nullptr || model == nullptr || batch == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "decode executor received a null argument");
    }
    if (batch->num_tokens == 0 || batch->num_tokens > self->maximum_tokens) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "ragged step token count exceeds workspace");
    }
    if (batch->num_segments == 0 || batch->num_segments > self->maximum_rows ||
        batch->num_segments > batch->num_tokens) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "ragged step segment count exceeds workspace");
    }
    if (batch->num_decode_segments > batch->num_segments ||
        (batch->num_decode_segments > 0 && batch->max_decode_context_tokens == 0)) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "ragged step decode-segment count is inconsistent");
    }
    if (model->num_layers == 0 || model->layers == nullptr || model->embedding == nullptr ||
        model->final_norm == nullptr || model->inv_freq == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "decode executor model is incomplete");
    }
    if (!batch->token_ids || !batch->positions || !batch->request_slots || !batch->physical_slots ||
        !batch->segment_offsets || !batch->segment_slots || !batch->output_rows || !batch->block_tables ||
        batch->block_table_stride == 0 || batch->block_table_rows == 0) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "ragged batch metadata is incomplete");
    }
    return forward_ragged(self, model, batch, use_fp8 != 0);
}

int32_t lfm25_decode_executor_step_graph(lfm25_decode_executor* self, const lfm25_model* model,
                                         const lfm25_decode_batch* batch, uint32_t use_fp8, uint32_t advance) {
    LFM25_TRY(validate(self, model, batch));
    // the split count of the attention launches is decided on the host from the longest context, so it is part of
    // what a captured step is valid for
    const size_t splits = lfm25_splitk_decode_splits(batch->num_tokens, batch->max_context_tokens, 16);
    const uint64_t signature = step_signature(self, model, batch);
    lfm25_decode_executor::Captured* entry = nullptr;
    for (auto& candidate : self->captured) {
        if (candidate.num_tokens == batch->num_tokens && candidate.splits == splits && candidate.use_fp8 == use_fp8 &&
            candidate.advance == advance && candidate.signature == signature) {
            entry = &candidate;
            break;
        }
    }
    if (entry == nullptr) {
        // take a free entry, or recycle the least recently used one
        for (auto& candidate : self->captured) {
            if (candidate.num_tokens == 0) {
                entry = &candidate;
                break;
            }
            if (entry == nullptr || candidate.last_used < entry->last_used) {
                entry = &candidate;
            }
        }
        if (entry->exec != nullptr) {
            cudaGraphExecDestroy(entry->exec);
        }
        *entry = lfm25_decode_executor::Captured();
        entry->num_tokens = batch->num_tokens;
        entry->splits = splits;
        entry->use_fp8 = use_fp8;
        entry->advance = advance;
        entry->signature = signature;
    }
    entry->last_used = ++self->graph_clock;
    cudaStream_t stream = self->blaslt->stream;
    if (stream == nullptr || stream == cudaStreamLegacy) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT,
                                   "graph replay needs the BlasLt handle bound to a non-default stream");
    }
    if (!entry->warmed) {
        // The first step of a bucket runs eagerly: cuBLASLt plans, function attributes and symbol lookups happen
        // here, outside any capture.
        entry->warmed = true;
        return forward(self, model, batch, use_fp8 != 0, advance != 0);
    }
    if (entry->exec == nullptr) {
        cudaError_t status = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
        if (status != cudaSuccess) return cuda_failure(status, "stream capture could not begin");
        const bool was_profiling = self->profiling;
        self->profiling = false;
        const int32_t rc = forward(self, model, batch, use_fp8 != 0, advance != 0);
        self->profiling = was_profiling;
        cudaGraph_t graph = nullptr;
        status = cudaStreamEndCapture(stream, &graph);
        if (rc != LFM25_OK) {
            if (graph != nullptr) cudaGraphDestroy(graph);
            return rc;
        }
        if (status != cudaSuccess) return cuda_failure(status, "stream capture failed");
        size_t node_count = 0;
        if (cudaGraphGetNodes(graph, nullptr, &node_count) == cudaSuccess && node_count > 0) {
            std::vector<cudaGraphNode_t> nodes(node_count);
            if (cudaGraphGetNodes(graph, nodes.data(), &node_count) == cudaSuccess) {
                for (size_t node = 0; node < node_count; ++node) {
                    cudaGraphNodeType type;
                    if (cudaGraphNodeGetType(nodes[node], &type) == cudaSuccess && type == cudaGraphNodeTypeKernel) {
                        ++entry->kernel_nodes;
                    }
                }
            }
        }
        status = cudaGraphInstantiate(&entry->exec, graph, 0);
        cudaGraphDestroy(graph);
        if (status != cudaSuccess) return cuda_failure(status, "graph instantiation failed");
        ++self->graph_captures;
    }
    const cudaError_t status = cudaGraphLaunch(entry->exec, stream);
    if (status != cudaSuccess) return cuda_failure(status, "graph launch failed");
    self->last_graph_kernel_nodes = entry->kernel_nodes;
    return LFM25_OK;
}

int32_t lfm25_decode_executor_serve_step(lfm25_decode_executor* self, const lfm25_model* model,
                                         const lfm25_decode_batch* batch, uint32_t use_fp8,
                                         const uint32_t* host_metadata, uint32_t* host_sampled) {
    LFM25_TRY(validate(self, model, batch));
    if (host_metadata == nullptr || host_sampled == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "served step received a null host buffer");
    }
    cudaStream_t stream = self->blaslt->stream;
    const size_t tokens = batch->num_tokens;
    const size_t bytes = tokens * sizeof(uint32_t);
    cudaError_t status;
    if (batch->positions == batch->token_ids + tokens && batch->request_slots == batch->positions + tokens) {
        status = cudaMemcpyAsync(batch->token_ids, host_metadata, 3 * bytes, cudaMemcpyHostToDevice, stream);
    } else {
        status = cudaMemcpyAsync(batch->token_ids, host_metadata, bytes, cudaMemcpyHostToDevice, stream);
        if (status == cudaSuccess) {
            status = cudaMemcpyAsync(batch->positions, host_metadata + tokens, bytes, cudaMemcpyHostToDevice, stream);
        }
        if (status == cudaSuccess) {
            status = cudaMemcpyAsync(const_cast<uint32_t*>(batch->request_slots), host_metadata + 2 * tokens, bytes,
                                     cudaMemcpyHostToDevice, stream);
        }
    }
    if (status != cudaSuccess) return cuda_failure(status, "step metadata upload failed");
    LFM25_TRY(lfm25_decode_executor_step_graph(self, model, batch, use_fp8, 0));
    status = cudaMemcpyAsync(host_sampled, self->sampled, bytes, cudaMemcpyDeviceToHost, stream);
    if (status == cudaSuccess) {
        status = cudaStreamSynchronize(stream);
    }
    return status == cudaSuccess ? LFM25_OK : cuda_failure(status, "served step failed");
}

size_t lfm25_decode_executor_graph_kernels(const lfm25_decode_executor* self) {
    return self != nullptr ? self->last_graph_kernel_nodes : 0;
}

size_t lfm25_decode_executor_graph_captures(const lfm25_decode_executor* self) {
    return self != nullptr ? self->graph_captures : 0;
}

}  // extern "C"
