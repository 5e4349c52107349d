// Prefix reuse for the serving loop: a radix index over page-sized token blocks and a pool of convolution-state
// checkpoints.
//
// Replaces, in the reference: PageRadixCache (src/cache/radix.rs:61-287) and ConvCheckpointPool
// (src/model/prefix.rs:15-129).  The index is host-only: every non-root node stands for one immutable physical KV page
// (which the caller pins in the page allocator with lfm25_kv_allocator_pin_cached_pages) and a node may carry the
// slot of a checkpoint of all gated-convolution states taken exactly after its last token, because a prefix can only
// be reused where both the attention layers' KV pages and the convolution layers' recurrent state are available.
// Checkpoints are device buffers [capacity, hidden, width] per convolution layer, captured and restored with
// same-stream device-to-device copies (no host synchronisation).
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/lfm25_b200.h"
#include "kernels.h"

namespace {

// A block of page_size token ids as a hash-map key (the bytes of the ids).
std::string block_key(const uint32_t* tokens, size_t count) {
    return std::string(reinterpret_cast<const char*>(tokens), count * sizeof(uint32_t));
}

struct RadixNode {
    std::unordered_map<std::string, size_t> children;
    uint32_t physical_page = 0;
    bool has_checkpoint = false;
    uint32_t checkpoint_slot = 0;
    size_t token_len = 0;
    uint64_t last_access = 0;
};

}  // namespace

struct lfm25_radix_cache {
    size_t page_size;
    std::vector<RadixNode> nodes;   // nodes[0] is the root
    size_t max_cached_pages;
    size_t cached_pages = 0;
    size_t checkpoints = 0;
    uint64_t clock = 0;
    uint64_t hits = 0;
    uint64_t misses = 0;
    uint64_t matched_tokens = 0;
};

struct lfm25_conv_checkpoints {
    std::vector<void*> layers;        // device, [capacity, hidden, width] bf16 each
    std::vector<uint32_t> free_slots; // LIFO, pop yields 0, 1, 2, ...
    size_t capacity;
    size_t elements_per_state;
};

namespace {

// src/cache/radix.rs:116-176
int64_t lookup(lfm25_radix_cache* self, const uint32_t* tokens, size_t num_tokens, size_t maximum_tokens,
               uint32_t* physical_pages, size_t pages_capacity, size_t* num_pages, uint32_t* checkpoint_slot,
               bool record_stats) {
    *num_pages = 0;
    const size_t usable = num_tokens < maximum_tokens ? num_tokens : maximum_tokens;
    const size_t page_count = usable / self->page_size;
    if (page_count == 0) {
        if (record_stats) self->misses += 1;
        return 0;
    }
    self->clock += 1;
    size_t node_id = 0;
    size_t walked = 0;
    size_t best_pages = 0;
    size_t best_tokens = 0;
    uint32_t best_slot = 0;
    bool found = false;
    for (size_t page = 0; page < page_count; ++page) {
        const auto child = self->nodes[node_id].children.find(block_key(tokens + page * self->page_size, self->page_size));
        if (child == self->nodes[node_id].children.end()) {
            break;
        }
        node_id = child->second;
        RadixNode& node = self->nodes[node_id];
        node.last_access = self->clock;
        if (walked < pages_capacity) {
            physical_pages[walked] = node.physical_page;
        }
        walked += 1;
        if (node.has_checkpoint) {
            found = true;
            best_pages = walked;
            best_tokens = node.token_len;
            best_slot = node.checkpoint_slot;
        }
    }
    if (!found || best_pages > pages_capacity) {
        if (record_stats) self->misses += 1;
        return found ? -1 : 0;   // -1: a hit that does not fit the caller's page buffer
    }
    *num_pages = best_pages;
    *checkpoint_slot = best_slot;
    if (record_stats) {
        self->hits += 1;
        self->matched_tokens += best_tokens;
    }
    return static_cast<int64_t>(best_tokens);
}

}  // namespace

extern "C" {

int32_t lfm25_radix_cache_create(size_t page_size, size_t max_cached_pages, lfm25_radix_cache** out) {
    if (out == nullptr) return lfm25::report_error(LFM25_ERR_NULL_POINTER, "radix cache output is null");
    if (page_size != 16 && page_size != 32) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "unsupported KV page size");
    if (max_cached_pages == 0) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "radix cache requires a positive page budget");
    }
    lfm25_radix_cache* self = new (std::nothrow) lfm25_radix_cache();
    if (self == nullptr) return lfm25::report_error(LFM25_ERR_CUDA, "out of host memory");
    self->page_size = page_size;
    self->max_cached_pages = max_cached_pages;
    self->nodes.emplace_back();
    *out = self;
    return LFM25_OK;
}

void lfm25_radix_cache_destroy(lfm25_radix_cache* self) { delete self; }

int64_t lfm25_radix_cache_longest_checkpoint(lfm25_radix_cache* self, const uint32_t* tokens, size_t num_tokens,
                                             size_t maximum_tokens, uint32_t* physical_pages, size_t pages_capacity,
                                             size_t* num_pages, uint32_t* checkpoint_slot) {
    if (self == nullptr || (tokens == nullptr && num_tokens > 0) || num_pages == nullptr || checkpoint_slot == nullptr ||
        (physical_pages == nullptr && pages_capacity > 0)) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "radix lookup received a null argument");
    }
    const int64_t matched = lookup(self, tokens, num_tokens, maximum_tokens, physical_pages, pages_capacity, num_pages,
                                   checkpoint_slot, true);
    return matched >= 0 ? matched
                        : lfm25::report_error(LFM25_ERR_BUFFER_TOO_SMALL, "radix lookup page buffer too small");
}

int64_t lfm25_radix_cache_probe_checkpoint(lfm25_radix_cache* self, const uint32_t* tokens, size_t num_tokens,
                                           size_t maximum_tokens, uint32_t* physical_pages, size_t pages_capacity,
                                           size_t* num_pages, uint32_t* checkpoint_slot) {
    if (self == nullptr || (tokens == nullptr && num_tokens > 0) || num_pages == nullptr || checkpoint_slot == nullptr ||
        (physical_pages == nullptr && pages_capacity > 0)) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "radix lookup received a null argument");
    }
    const int64_t matched = lookup(self, tokens, num_tokens, maximum_tokens, physical_pages, pages_capacity, num_pages,
                                   checkpoint_slot, false);
    return matched >= 0 ? matched
                        : lfm25::report_error(LFM25_ERR_BUFFER_TOO_SMALL, "radix lookup page buffer too small");
}

// src/cache/radix.rs:181-206
uint32_t lfm25_radix_cache_can_publish(const lfm25_radix_cache* self, const uint32_t* tokens, size_t num_tokens,
                                       size_t prefix_tokens) {
    if (self == nullptr || tokens == nullptr) return 0;
    if (prefix_tokens == 0 || prefix_tokens > num_tokens || prefix_tokens % self->page_size != 0) {
        return 0;
    }
    const size_t page_count = prefix_tokens / self->page_size;
    size_t node_id = 0;
    size_t existing = 0;
    for (size_t page = 0; page < page_count; ++page) {
        const auto child = self->nodes[node_id].children.find(block_key(tokens + page * self->page_size, self->page_size));
        if (child == self->nodes[node_id].children.end()) {
            break;
        }
        node_id = child->second;
        existing += 1;
    }
    if (existing == page_count && self->nodes[node_id].has_checkpoint) {
        return 0;
    }
    return self->cached_pages + (page_count - existing) <= self->max_cached_pages ? 1u : 0u;
}

// src/cache/radix.rs:210-271
int64_t lfm25_radix_cache_insert_checkpoint(lfm25_radix_cache* self, const uint32_t* tokens, size_t num_tokens,
                                            size_t prefix_tokens, const uint32_t* physical_pages,
                                            size_t num_physical_pages, uint32_t checkpoint_slot,
                                            uint32_t* newly_cached_pages) {
    if (self == nullptr || tokens == nullptr || physical_pages == nullptr || newly_cached_pages == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "radix insert received a null argument");
    }
    if (prefix_tokens == 0) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "cached prefix cannot be empty");
    if (prefix_tokens > num_tokens) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "cached prefix exceeds token input");
    }
    if (prefix_tokens % self->page_size != 0) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "cached prefix must be page aligned");
    }
    const size_t page_count = prefix_tokens / self->page_size;
    if (num_physical_pages != page_count) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "cached prefix physical page count mismatch");
    }
    if (!lfm25_radix_cache_can_publish(self, tokens, num_tokens, prefix_tokens)) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "radix cache prefix cannot be published");
    }
    self->clock += 1;
    size_t node_id = 0;
    size_t created = 0;
    for (size_t page = 0; page < page_count; ++page) {
        const std::string key = block_key(tokens + page * self->page_size, self->page_size);
        const auto child = self->nodes[node_id].children.find(key);
        if (child != self->nodes[node_id].children.end()) {
            node_id = child->second;
            self->nodes[node_id].last_access = self->clock;
            continue;
        }
        const size_t fresh = self->nodes.size();
        self->nodes.emplace_back();
        RadixNode& node = self->nodes.back();
        node.physical_page = physical_pages[page];
        node.token_len = (page + 1) * self->page_size;
        node.last_access = self->clock;
        self->nodes[node_id].children.emplace(key, fresh);
        node_id = fresh;
        newly_cached_pages[created++] = physical_pages[page];
    }
    RadixNode& last = self->nodes[node_id];
    last.has_checkpoint = true;
    last.checkpoint_slot = checkpoint_slot;
    last.last_access = self->clock;
    self->cached_pages += created;
    self->checkpoints += 1;
    return static_cast<int64_t>(created);
}

void lfm25_radix_cache_snapshot(const lfm25_radix_cache* self, lfm25_prefix_cache_snapshot* out) {
    if (self == nullptr || out == nullptr) return;
    out->nodes = self->nodes.size();
    out->cached_pages = self->cached_pages;
    out->checkpoints = self->checkpoints;
    out->hits = self->hits;
    out->misses = self->misses;
    out->matched_tokens = self->matched_tokens;
}

// ------------------------------------------------------------------------------- convolution checkpoints

int32_t lfm25_conv_checkpoints_create(size_t convolution_layers, size_t capacity, size_t hidden_size,
                                      size_t state_width, lfm25_conv_checkpoints** out) {
    if (out == nullptr) return lfm25::report_error(LFM25_ERR_NULL_POINTER, "checkpoint pool output is null");
    if (convolution_layers == 0) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "checkpoint pool needs convolution layers");
    }
    if (capacity == 0) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "checkpoint pool capacity must be positive");
    if (hidden_size == 0 || state_width == 0) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "invalid convolution state shape");
    }
    if (capacity > 0xffffffffull) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "checkpoint capacity exceeds u32");
    lfm25_conv_checkpoints* self = new (std::nothrow) lfm25_conv_checkpoints();
    if (self == nullptr) return lfm25::report_error(LFM25_ERR_CUDA, "out of host memory");
    self->capacity = capacity;
    self->elements_per_state = hidden_size * state_width;
    const size_t bytes = capacity * self->elements_per_state * 2;
    for (size_t layer = 0; layer < convolution_layers; ++layer) {
        void* buffer = nullptr;
        cudaError_t status = cudaMalloc(&buffer, bytes);
        if (status == cudaSuccess) {
            status = cudaMemset(buffer, 0, bytes);
            self->layers.push_back(buffer);
        }
        if (status != cudaSuccess) {
            lfm25_conv_checkpoints_destroy(self);
            return lfm25::report_error(LFM25_ERR_CUDA, cudaGetErrorString(status));
        }
    }
    for (size_t slot = capacity; slot-- > 0;) {
        self->free_slots.push_back(static_cast<uint32_t>(slot));
    }
    *out = self;
    return LFM25_OK;
}

void lfm25_conv_checkpoints_destroy(lfm25_conv_checkpoints* self) {
    if (self == nullptr) return;
    for (void* buffer : self->layers) {
        cudaFree(buffer);
    }
    delete self;
}

int64_t lfm25_conv_checkpoints_acquire(lfm25_conv_checkpoints* self) {
    if (self == nullptr || self->free_slots.empty()) return -1;
    const uint32_t slot = self->free_slots.back();
    self->free_slots.pop_back();
    return slot;
}

void lfm25_conv_checkpoints_release(lfm25_conv_checkpoints* self, uint32_t slot) {
    if (self != nullptr && slot < self->capacity) {
        self->free_slots.push_back(slot);
    }
}

size_t lfm25_conv_checkpoints_available(const lfm25_conv_checkpoints* self) {
    return self != nullptr ? self->free_slots.size() : 0;
}

size_t lfm25_conv_checkpoints_capacity(const lfm25_conv_checkpoints* self) {
    return self != nullptr ? self->capacity : 0;
}

namespace {

int32_t copy_state(lfm25_conv_checkpoints* self, void* stream, uint32_t checkpoint_slot, size_t convolution_index,
                   void* states, size_t request_slot, size_t num_request_slots, bool capture) {
    if (self == nullptr || states == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "checkpoint copy received a null argument");
    }
    if (convolution_index >= self->layers.size()) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "convolution checkpoint layer out of range");
    }
    if (checkpoint_slot >= self->capacity || request_slot >= num_request_slots) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "convolution checkpoint slot out of range");
    }
    const size_t bytes = self->elements_per_state * 2;
    char* pooled = static_cast<char*>(self->layers[convolution_index]) + static_cast<size_t>(checkpoint_slot) * bytes;
    char* live = static_cast<char*>(states) + request_slot * bytes;
    const cudaError_t status = cudaMemcpyAsync(capture ? pooled : live, capture ? live : pooled, bytes,
                                               cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
    return status == cudaSuccess ? LFM25_OK : lfm25::report_error(LFM25_ERR_CUDA, cudaGetErrorString(status));
}

}  // namespace

int32_t lfm25_conv_checkpoints_capture_layer(lfm25_conv_checkpoints* self, void* stream, uint32_t checkpoint_slot,
                                             size_t convolution_index, const void* states, size_t request_slot,
                                             size_t num_request_slots) {
    return copy_state(self, stream, checkpoint_slot, convolution_index, const_cast<void*>(states), request_slot,
                      num_request_slots, true);
}

int32_t lfm25_conv_checkpoints_restore_layer(lfm25_conv_checkpoints* self, void* stream, uint32_t checkpoint_slot,
                                             size_t convolution_index, void* states, size_t request_slot,
                                             size_t num_request_slots) {
    return copy_state(self, stream, checkpoint_slot, convolution_index, states, request_slot, num_request_slots, false);
}

}  // extern "C"
