// The library's switch table (see options.h) and its two C-ABI accessors.
#include "options.h"

#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "../../include/lfm25_b200.h"
#include "kernels.h"

namespace lfm25 {

namespace {

struct Entry {
    const char* name;
    const char* variable;
    int64_t value;
    int64_t minimum;
    int64_t maximum;
};

Entry g_options[kOptCount] = {
    {"pdl", "LFM25_PDL", 1, 0, 1},
    {"fused_append", "LFM25_FUSED_APPEND", 2, 0, 2},
    {"fused_silu", "LFM25_FUSED_SILU", 1, 0, 1},
    {"fused_silu_bf16", "LFM25_FUSED_SILU_BF16", 0, 0, 1},
    {"kv_evict_first", "LFM25_KV_EVICT_FIRST", 1, 0, 1},
    {"weights_evict_first", "LFM25_WEIGHTS_EVICT_FIRST", 1, 0, 1},
    {"splitk_cluster_merge", "LFM25_SPLITK_CLUSTER_MERGE", 1, 0, 1},
    {"engine_graph", "LFM25_ENGINE_GRAPH", 1, 0, 1},
    {"hybrid_attention", "LFM25_HYBRID_ATTENTION", 0, 0, 2},
    {"fp8_gemm_path", "LFM25_FP8_GEMM_PATH", 0, 0, 4},
    {"bf16_gemm", "LFM25_BF16_GEMM", 0, 0, 3},
    {"decode_splits", "LFM25_DECODE_SPLITS", 0, 0, 8},
    {"wait_limit_ns", "LFM25_WAIT_LIMIT_NS", 1000000000ll, 1000, 60000000000ll},
    {"wait_selftest_drop", "LFM25_WAIT_SELFTEST_DROP", 0, 0, 1},
};

std::once_flag g_once;

int64_t parse(int which, const char* text) {
    struct Named {
        int option;
        const char* word;
        int64_t value;
    };
    static const Named names[] = {
        {kOptHybridAttention, "auto", 0}, {kOptHybridAttention, "umma", 1}, {kOptHybridAttention, "mma", 2},
        {kOptFp8GemmPath, "auto", 0},     {kOptFp8GemmPath, "stream", 1},   {kOptFp8GemmPath, "umma", 2},
        {kOptFp8GemmPath, "generic", 3},  {kOptFp8GemmPath, "rows", 4},     {kOptBf16Gemm, "auto", 0},
        {kOptBf16Gemm, "umma", 1},        {kOptBf16Gemm, "cublaslt", 2},    {kOptBf16Gemm, "rows", 3},
    };
    for (const Named& named : names) {
        if (named.option == which && strcmp(named.word, text) == 0) {
            return named.value;
        }
    }
    return strtoll(text, nullptr, 10);
}

void initialise() {
    for (int which = 0; which < kOptCount; ++which) {
        const char* text = getenv(g_options[which].variable);
        if (text != nullptr && text[0] != '\0') {
            const int64_t value = parse(which, text);
            if (value >= g_options[which].minimum && value <= g_options[which].maximum) {
                g_options[which].value = value;
            }
        }
    }
}

}  // namespace

int64_t option(Option which) {
    std::call_once(g_once, initialise);
    return g_options[which].value;
}

bool set_option_by_name(const char* name, int64_t value) {
    std::call_once(g_once, initialise);
    for (Entry& entry : g_options) {
        if (strcmp(entry.name, name) == 0) {
            if (value < entry.minimum || value > entry.maximum) {
                return false;
            }
            entry.value = value;
            return true;
        }
    }
    return false;
}

bool get_option_by_name(const char* name, int64_t* value) {
    std::call_once(g_once, initialise);
    for (const Entry& entry : g_options) {
        if (strcmp(entry.name, name) == 0) {
            *value = entry.value;
            return true;
        }
    }
    return false;
}

}  // namespace lfm25

extern "C" {

int32_t lfm25_set_option(const char* name, int64_t value) {
    if (name == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "option name is null");
    }
    if (!lfm25::set_option_by_name(name, value)) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "unknown option or value out of range");
    }
    return LFM25_OK;
}

int32_t lfm25_get_option(const char* name, int64_t* value) {
    if (name == nullptr || value == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "option name or output is null");
    }
    if (!lfm25::get_option_by_name(name, value)) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "unknown option");
    }
    return LFM25_OK;
}

}  // extern "C"
