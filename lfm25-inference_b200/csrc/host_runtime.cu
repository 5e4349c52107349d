// Host-side state of the decode path: physical KV page allocator, per-slot block tables, the decode part of
// the scheduler and the request dispatcher over engine replicas.  Pure C++ (no device code); it lives in the
// library so that a host in any language reaches it through the same C ABI as the kernels.
//
// Replaces, in the reference: KvPageAllocator (src/cache/allocator.rs:40-229), FixedBlockTables
// (src/cache/block_table.rs:3-31), the decode half of Scheduler::schedule (src/scheduler/planner.rs:80-113).
// The dispatcher has no counterpart: the reference drives one GPU.
#include <algorithm>
#include <cstdint>
#include <new>
#include <vector>

#include "../../include/lfm25_b200.h"
#include "kernels.h"

struct lfm25_kv_allocator {
    size_t page_size;
    std::vector<uint32_t> free_pages;  // LIFO: pop yields 0, 1, 2, ... on a fresh pool
    std::vector<uint32_t> page_refs;   // deliberately not atomic: one GPU-owner thread mutates it
    size_t total_pages;
    size_t reserved_pages;
    size_t cached_pages;
    size_t peak_allocated_pages;
};

struct lfm25_block_tables {
    std::vector<uint32_t> entries;
    size_t slots;
    size_t pages_per_slot;
};

struct lfm25_dispatcher {
    struct Replica {
        uint64_t load = 0;  // outstanding tokens assigned and not yet completed
        bool alive = true;
    };
    std::vector<Replica> replicas;
};

namespace {

size_t div_ceil(size_t value, size_t divisor) { return (value + divisor - 1) / divisor; }

}  // namespace

extern "C" {

// ------------------------------------------------------------------------------------------ allocator

int32_t lfm25_kv_allocator_create(size_t total_pages, size_t page_size, lfm25_kv_allocator** out) {
    if (out == nullptr) return lfm25::report_error(LFM25_ERR_NULL_POINTER, "KV page allocator output is null");
    if (total_pages == 0) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "KV page allocator requires physical pages");
    if (total_pages > 0xffffffffull) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "KV physical page count exceeds u32");
    if (page_size != 16 && page_size != 32) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "unsupported KV page size");
    lfm25_kv_allocator* self = new (std::nothrow) lfm25_kv_allocator();
    if (self == nullptr) return lfm25::report_error(LFM25_ERR_CUDA, "out of host memory");
    self->page_size = page_size;
    self->total_pages = total_pages;
    self->free_pages.reserve(total_pages);
    for (size_t page = total_pages; page-- > 0;) {
        self->free_pages.push_back(static_cast<uint32_t>(page));
    }
    self->page_refs.assign(total_pages, 0);
    self->reserved_pages = self->cached_pages = self->peak_allocated_pages = 0;
    *out = self;
    return LFM25_OK;
}

void lfm25_kv_allocator_destroy(lfm25_kv_allocator* self) { delete self; }

int64_t lfm25_kv_allocator_try_reserve_pages(lfm25_kv_allocator* self, size_t pages) {
    const size_t next = self->reserved_pages + pages;
    if (next < self->reserved_pages || next + self->cached_pages < next ||
        next + self->cached_pages > self->total_pages) {
        return LFM25_KV_LOGICAL_RESERVATION_EXHAUSTED;
    }
    self->reserved_pages = next;
    return static_cast<int64_t>(pages);
}

int64_t lfm25_kv_allocator_try_reserve_tokens(lfm25_kv_allocator* self, size_t maximum_tokens) {
    if (maximum_tokens == 0) {
        return LFM25_KV_SEQUENCE_CAPACITY_EXCEEDED;
    }
    return lfm25_kv_allocator_try_reserve_pages(self, div_ceil(maximum_tokens, self->page_size));
}

void lfm25_kv_allocator_release_reservation(lfm25_kv_allocator* self, size_t pages) {
    self->reserved_pages = self->reserved_pages > pages ? self->reserved_pages - pages : 0;
}

static int32_t add_references(lfm25_kv_allocator* self, const uint32_t* pages, size_t count) {
    for (size_t index = 0; index < count; ++index) {
        if (pages[index] >= self->page_refs.size() || self->page_refs[pages[index]] == 0 ||
            self->page_refs[pages[index]] == 0xffffffffu) {
            return LFM25_KV_PHYSICAL_PAGES_EXHAUSTED;
        }
        self->page_refs[pages[index]] += 1;
    }
    return LFM25_OK;
}

int32_t lfm25_kv_allocator_pin_cached_pages(lfm25_kv_allocator* self, const uint32_t* pages, size_t count) {
    if (self->cached_pages + count > self->total_pages) {
        return LFM25_KV_PHYSICAL_PAGES_EXHAUSTED;
    }
    const int32_t status = add_references(self, pages, count);
    if (status != LFM25_OK) {
        return status;
    }
    self->cached_pages += count;
    return LFM25_OK;
}

int32_t lfm25_kv_allocator_retain_pages(lfm25_kv_allocator* self, const uint32_t* pages, size_t count) {
    return add_references(self, pages, count);
}

int64_t lfm25_kv_allocator_grow_sequence(lfm25_kv_allocator* self, size_t current_tokens, size_t target_tokens,
                                         uint32_t* block_table, size_t block_table_len) {
    if (target_tokens < current_tokens) {
        return LFM25_KV_SEQUENCE_CAPACITY_EXCEEDED;
    }
    const size_t current_pages = div_ceil(current_tokens, self->page_size);
    const size_t target_pages = div_ceil(target_tokens, self->page_size);
    if (target_pages > block_table_len) {
        return LFM25_KV_SEQUENCE_CAPACITY_EXCEEDED;
    }
    const size_t needed = target_pages > current_pages ? target_pages - current_pages : 0;
    if (needed > self->free_pages.size()) {
        return LFM25_KV_PHYSICAL_PAGES_EXHAUSTED;
    }
    for (size_t index = current_pages; index < target_pages; ++index) {
        const uint32_t page = self->free_pages.back();
        if (self->page_refs[page] != 0) {
            return LFM25_KV_PHYSICAL_PAGES_EXHAUSTED;
        }
        self->free_pages.pop_back();
        self->page_refs[page] = 1;
        block_table[index] = page;
    }
    self->peak_allocated_pages = std::max(self->peak_allocated_pages, self->total_pages - self->free_pages.size());
    return static_cast<int64_t>(needed);
}

int64_t lfm25_kv_allocator_pages_short(const lfm25_kv_allocator* self, const size_t* current_tokens,
                                       const size_t* target_tokens, size_t sequences) {
    size_t needed = 0;
    for (size_t index = 0; index < sequences; ++index) {
        if (target_tokens[index] < current_tokens[index]) {
            return LFM25_KV_SEQUENCE_CAPACITY_EXCEEDED;
        }
        needed += div_ceil(target_tokens[index], self->page_size) - div_ceil(current_tokens[index], self->page_size);
    }
    return needed > self->free_pages.size() ? static_cast<int64_t>(needed - self->free_pages.size()) : 0;
}

void lfm25_kv_allocator_release_sequence(lfm25_kv_allocator* self, size_t tokens, uint32_t* block_table,
                                         size_t block_table_len) {
    const size_t pages = std::min(div_ceil(tokens, self->page_size), block_table_len);
    for (size_t index = 0; index < pages; ++index) {
        const uint32_t page = block_table[index];
        if (page == 0xffffffffu) {
            continue;
        }
        // a page that is out of range or already free stays unavailable rather than risking a double free
        if (page < self->page_refs.size() && self->page_refs[page] != 0) {
            if (--self->page_refs[page] == 0) {
                self->free_pages.push_back(page);
            }
        }
        block_table[index] = 0xffffffffu;
    }
}

void lfm25_kv_allocator_snapshot(const lfm25_kv_allocator* self, lfm25_kv_pool_snapshot* out) {
    out->total_pages = self->total_pages;
    out->free_pages = self->free_pages.size();
    out->allocated_pages = self->total_pages - self->free_pages.size();
    out->reserved_pages = self->reserved_pages;
    out->cached_pages = self->cached_pages;
    out->peak_allocated_pages = self->peak_allocated_pages;
}

// ------------------------------------------------------------------------------------------ block tables

int32_t lfm25_block_tables_create(size_t slots, size_t pages_per_slot, lfm25_block_tables** out) {
    if (out == nullptr) return lfm25::report_error(LFM25_ERR_NULL_POINTER, "block tables output is null");
    if (slots == 0) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "block tables require request slots");
    if (pages_per_slot == 0) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "block tables require logical pages");
    if (slots > SIZE_MAX / pages_per_slot / sizeof(uint32_t)) {
        return lfm25::report_error(LFM25_ERR_OVERFLOW, "block table size overflow");
    }
    lfm25_block_tables* self = new (std::nothrow) lfm25_block_tables();
    if (self == nullptr) return lfm25::report_error(LFM25_ERR_CUDA, "out of host memory");
    self->entries.assign(slots * pages_per_slot, 0xffffffffu);
    self->slots = slots;
    self->pages_per_slot = pages_per_slot;
    *out = self;
    return LFM25_OK;
}

void lfm25_block_tables_destroy(lfm25_block_tables* self) { delete self; }

uint32_t* lfm25_block_tables_slot(lfm25_block_tables* self, size_t slot) {
    if (self == nullptr || slot >= self->slots) {
        lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "block table slot out of range");
        return nullptr;
    }
    return self->entries.data() + slot * self->pages_per_slot;
}

const uint32_t* lfm25_block_tables_data(const lfm25_block_tables* self) { return self->entries.data(); }

// ------------------------------------------------------------------------------------------ scheduler (decode)

size_t lfm25_schedule_decode(const uint32_t* phases, const uint64_t* next_token_deadline_us,
                             const uint32_t* context_tokens, size_t num_slots, uint64_t now_us, uint32_t* decode_slots,
                             size_t* maximum_context_tokens) {
    size_t count = 0;
    size_t maximum_context = 1;
    for (size_t slot = 0; slot < num_slots; ++slot) {
        if (phases[slot] == LFM25_PHASE_DECODING) {
            decode_slots[count++] = static_cast<uint32_t>(slot);
            maximum_context = std::max<size_t>(maximum_context, context_tokens[slot]);
        }
    }
    // earliest deadline first; the slack saturates at zero, equal slacks keep slot order
    std::stable_sort(decode_slots, decode_slots + count, [&](uint32_t a, uint32_t b) {
        const uint64_t slack_a = next_token_deadline_us[a] > now_us ? next_token_deadline_us[a] - now_us : 0;
        const uint64_t slack_b = next_token_deadline_us[b] > now_us ? next_token_deadline_us[b] - now_us : 0;
        return slack_a < slack_b;
    });
    if (maximum_context_tokens != nullptr) {
        *maximum_context_tokens = maximum_context;
    }
    return count;
}

// ------------------------------------------------------------------------------------------ replica dispatcher

int32_t lfm25_dispatcher_create(size_t replicas, lfm25_dispatcher** out) {
    if (out == nullptr) return lfm25::report_error(LFM25_ERR_NULL_POINTER, "dispatcher output is null");
    if (replicas == 0) return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "dispatcher requires replicas");
    lfm25_dispatcher* self = new (std::nothrow) lfm25_dispatcher();
    if (self == nullptr) return lfm25::report_error(LFM25_ERR_CUDA, "out of host memory");
    self->replicas.resize(replicas);
    *out = self;
    return LFM25_OK;
}

void lfm25_dispatcher_destroy(lfm25_dispatcher* self) { delete self; }

int32_t lfm25_dispatcher_assign(lfm25_dispatcher* self, uint64_t prefix_hash, uint32_t has_prefix,
                                uint64_t estimated_tokens) {
    const size_t count = self->replicas.size();
    size_t best = count;
    if (has_prefix) {
        // requests that share a prompt prefix go to the replica whose prefix cache holds it, while it lives
        const size_t home = static_cast<size_t>(prefix_hash % count);
        if (self->replicas[home].alive) {
            best = home;
        }
    }
    if (best == count) {
        for (size_t index = 0; index < count; ++index) {
            if (self->replicas[index].alive && (best == count || self->replicas[index].load < self->replicas[best].load)) {
                best = index;
            }
        }
    }
    if (best == count) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "no live replica");
    }
    self->replicas[best].load += estimated_tokens;
    return static_cast<int32_t>(best);
}

int32_t lfm25_dispatcher_assign_bounded(lfm25_dispatcher* self, uint64_t prefix_hash, uint32_t has_prefix,
                                        uint64_t estimated_tokens, uint64_t slack_tokens) {
    const size_t count = self->replicas.size();
    size_t least = count;
    for (size_t index = 0; index < count; ++index) {
        if (self->replicas[index].alive && (least == count || self->replicas[index].load < self->replicas[least].load)) {
            least = index;
        }
    }
    if (least == count) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "no live replica");
    }
    size_t best = least;
    if (has_prefix) {
        // the prefix's home keeps the request while it is not more than `slack_tokens` busier than the idlest
        // replica; past that the request spills there (and that replica's prefix cache learns the prefix)
        const size_t home = static_cast<size_t>(prefix_hash % count);
        if (self->replicas[home].alive && self->replicas[home].load - self->replicas[least].load <= slack_tokens) {
            best = home;
        }
    }
    self->replicas[best].load += estimated_tokens;
    return static_cast<int32_t>(best);
}

void lfm25_dispatcher_complete(lfm25_dispatcher* self, size_t replica, uint64_t tokens) {
    if (replica < self->replicas.size()) {
        uint64_t& load = self->replicas[replica].load;
        load = load > tokens ? load - tokens : 0;
    }
}

void lfm25_dispatcher_mark_failed(lfm25_dispatcher* self, size_t replica) {
    if (replica < self->replicas.size()) {
        self->replicas[replica].alive = false;
        self->replicas[replica].load = 0;
    }
}

uint64_t lfm25_dispatcher_load(const lfm25_dispatcher* self, size_t replica) {
    return replica < self->replicas.size() ? self->replicas[replica].load : 0;
}

}  // extern "C"
