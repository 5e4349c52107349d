// extern "C" boundary of the library: host-side validation (the reference wrappers' `ensure!`
// checks, in the same order) followed by the kernel launch.  Nothing is launched on error.
#include <stdarg.h>
#include <stdio.h>

#include <stdlib.h>
#include <string.h>

#include <cmath>
#include <limits>
#include <new>

#include "../../include/lfm25_b200.h"
#include "blaslt_handle.h"
#include "common.cuh"
#include "kernels.h"
#include "options.h"

namespace {

thread_local char g_last_error[256] = "";

int32_t fail(int32_t code, const char* format, ...) {
    va_list arguments;
    va_start(arguments, format);
    vsnprintf(g_last_error, sizeof g_last_error, format, arguments);
    va_end(arguments);
    return code;
}

#define LFM25_ENSURE(condition, code, ...) \
    do {                                   \
        if (!(condition)) {                \
            return fail(code, __VA_ARGS__); \
        }                                  \
    } while (0)

bool checked_mul(size_t a, size_t b, size_t* out) {
    if (a != 0 && b > std::numeric_limits<size_t>::max() / a) {
        return false;
    }
    *out = a * b;
    return true;
}

// pages * 8 * page_size * 64 elements
bool cache_elements(size_t num_pages, size_t page_size, size_t* out) {
    size_t value = 0;
    return checked_mul(num_pages, 8, &value) && checked_mul(value, page_size, &value) &&
           checked_mul(value, 64, out);
}

int32_t cuda_result(cudaError_t status, const char* what) {
    if (status == cudaSuccess) {
        return LFM25_OK;
    }
    return fail(LFM25_ERR_CUDA, "%s: %s", what, cudaGetErrorString(status));
}

// Device status words shared by all kernels with bounded waits.
__device__ unsigned int g_device_status[4];

unsigned int* device_status_pointer() {
    // One address per device; looked up on first use with that device current.
    static thread_local int cached_device = -1;
    static thread_local unsigned int* cached_pointer = nullptr;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) {
        return nullptr;
    }
    if (device != cached_device) {
        void* pointer = nullptr;
        if (cudaGetSymbolAddress(&pointer, g_device_status) != cudaSuccess) {
            return nullptr;
        }
        cached_pointer = static_cast<unsigned int*>(pointer);
        cached_device = device;
    }
    return cached_pointer;
}

// Checks shared by the three attention entry points that take block tables per request
// (src/cuda/kernels/attention_async_fast.rs:215-282).
int32_t validate_ragged_common(size_t page_size, const lfm25_slice& query, const lfm25_slice& key_cache,
                               const lfm25_slice& value_cache, const lfm25_slice& block_tables,
                               const lfm25_slice* request_slots, const lfm25_slice& position_ids,
                               const lfm25_slice& output, size_t num_tokens, size_t num_pages,
                               size_t block_table_stride) {
    LFM25_ENSURE(num_tokens > 0, LFM25_ERR_INVALID_ARGUMENT, "fast-exp ragged attention requires tokens");
    LFM25_ENSURE(num_pages > 0, LFM25_ERR_INVALID_ARGUMENT, "fast-exp ragged attention requires cache pages");
    LFM25_ENSURE(page_size == 16 || page_size == 32, LFM25_ERR_INVALID_ARGUMENT,
                 "unsupported fast-exp ragged page size %zu", page_size);
    LFM25_ENSURE(page_size == 16, LFM25_ERR_UNSUPPORTED, "page size 32 is not built; use 16");
    LFM25_ENSURE(block_table_stride > 0, LFM25_ERR_INVALID_ARGUMENT,
                 "fast-exp ragged block table stride must be positive");
    LFM25_ENSURE(block_tables.len >= block_table_stride, LFM25_ERR_BUFFER_TOO_SMALL,
                 "fast-exp ragged block tables too small");
    LFM25_ENSURE(block_tables.len % block_table_stride == 0, LFM25_ERR_INVALID_ARGUMENT,
                 "fast-exp ragged block tables not row aligned");
    LFM25_ENSURE(request_slots == nullptr || request_slots->len >= num_tokens, LFM25_ERR_BUFFER_TOO_SMALL,
                 "fast-exp ragged request slots too small");
    LFM25_ENSURE(position_ids.len >= num_tokens, LFM25_ERR_BUFFER_TOO_SMALL, "fast-exp ragged positions too small");
    size_t q_required = 0;
    LFM25_ENSURE(checked_mul(num_tokens, 32 * 64, &q_required), LFM25_ERR_OVERFLOW,
                 "fast-exp ragged query size overflow");
    size_t cache_required = 0;
    LFM25_ENSURE(cache_elements(num_pages, page_size, &cache_required), LFM25_ERR_OVERFLOW,
                 "fast-exp ragged cache size overflow");
    LFM25_ENSURE(query.len >= q_required, LFM25_ERR_BUFFER_TOO_SMALL, "fast-exp ragged query storage too small");
    LFM25_ENSURE(output.len >= q_required, LFM25_ERR_BUFFER_TOO_SMALL, "fast-exp ragged output storage too small");
    LFM25_ENSURE(key_cache.len >= cache_required, LFM25_ERR_BUFFER_TOO_SMALL, "fast-exp ragged K cache too small");
    LFM25_ENSURE(value_cache.len >= cache_required, LFM25_ERR_BUFFER_TOO_SMALL, "fast-exp ragged V cache too small");
    LFM25_ENSURE(query.ptr && output.ptr && key_cache.ptr && value_cache.ptr && block_tables.ptr &&
                     (request_slots == nullptr || request_slots->ptr) && position_ids.ptr,
                 LFM25_ERR_NULL_POINTER, "fast-exp ragged attention received a null device pointer");
    // Limits of this implementation's 32-bit grid and TMA row coordinates.
    LFM25_ENSURE(num_tokens <= (1u << 24), LFM25_ERR_INVALID_ARGUMENT, "attention grid size exceeds u32");
    LFM25_ENSURE(num_pages <= (1u << 24), LFM25_ERR_INVALID_ARGUMENT, "attention page pool exceeds 2^24 pages");
    LFM25_ENSURE((reinterpret_cast<uintptr_t>(key_cache.ptr) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(value_cache.ptr) & 15) == 0,
                 LFM25_ERR_INVALID_ARGUMENT, "KV cache must be 16-byte aligned");
    return LFM25_OK;
}

// Validation of Fp8MatmulKey::new + BlasLt::linear_fp8_scaled (src/cuda/blaslt/fp8.rs:23-40,
// src/cuda/blaslt/mod.rs:222-262), then the choice of kernel:
//   through a handle, N % 16 == 0, K % 128 == 0, M in the range where it measured ahead (see rows_preferred)
//                                          batch-major tcgen05 kernel (gemm_rows_umma.cu)
//   M <= 256, N % 128 == 0, K % 128 == 0   weight-major tcgen05 kernel (K split over a thread-block cluster when
//                                          there are few tiles and the caller is a handle with an exchange buffer)
//   M <= 8 otherwise, or few tiles without a handle   weight-streaming mma.sync kernel
//   anything else                          generic kernel
// The option fp8_gemm_path = stream | umma | generic | rows overrides the choice where the shape allows.
// `handle` is null for the handle-free entry point, which has no exchange buffer and never splits K.
int32_t linear_fp8_dispatch(cudaStream_t stream, lfm25_slice x, lfm25_slice weight, lfm25_slice out,
                            const lfm25_fp8_linear_config* config, const lfm25_blaslt* handle) {
    void* exchange = handle != nullptr ? handle->exchange : nullptr;
    const size_t exchange_bytes = handle != nullptr ? handle->exchange_bytes : 0;
    LFM25_ENSURE(config != nullptr, LFM25_ERR_NULL_POINTER, "FP8 linear config is null");
    const size_t m = config->m;
    const size_t n = config->n;
    const size_t k = config->k;
    LFM25_ENSURE(m > 0, LFM25_ERR_INVALID_ARGUMENT, "FP8 matmul M must be > 0");
    LFM25_ENSURE(n > 0, LFM25_ERR_INVALID_ARGUMENT, "FP8 matmul N must be > 0");
    LFM25_ENSURE(k > 0, LFM25_ERR_INVALID_ARGUMENT, "FP8 matmul K must be > 0");
    LFM25_ENSURE(config->scale_mode == LFM25_FP8_SCALE_TENSORWIDE || config->scale_mode == LFM25_FP8_SCALE_BLOCK32,
                 LFM25_ERR_INVALID_ARGUMENT, "unknown FP8 scale mode %u", config->scale_mode);
    LFM25_ENSURE(config->scale_mode != LFM25_FP8_SCALE_BLOCK32 || k % 32 == 0, LFM25_ERR_INVALID_ARGUMENT,
                 "MXFP8 matmul K must be divisible by 32, got %zu", k);
    LFM25_ENSURE(config->scale_mode == LFM25_FP8_SCALE_TENSORWIDE, LFM25_ERR_UNSUPPORTED,
                 "Block32 (MXFP8) scaling is not built; use the tensor-wide mode");
    LFM25_ENSURE(std::isfinite(config->output_scale) && config->output_scale > 0.0f, LFM25_ERR_INVALID_ARGUMENT,
                 "FP8 output scale must be finite and positive");
    size_t x_required = 0;
    size_t weight_required = 0;
    size_t out_required = 0;
    LFM25_ENSURE(checked_mul(m, k, &x_required), LFM25_ERR_OVERFLOW, "FP8 linear input size overflow");
    LFM25_ENSURE(checked_mul(n, k, &weight_required), LFM25_ERR_OVERFLOW, "FP8 linear weight size overflow");
    LFM25_ENSURE(checked_mul(m, n, &out_required), LFM25_ERR_OVERFLOW, "FP8 linear output size overflow");
    LFM25_ENSURE(x.len >= x_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "FP8 linear input storage too small: required=%zu, actual=%zu", x_required, x.len);
    LFM25_ENSURE(weight.len >= weight_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "FP8 linear weight storage too small: required=%zu, actual=%zu", weight_required, weight.len);
    LFM25_ENSURE(out.len >= out_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "FP8 linear output storage too small: required=%zu, actual=%zu", out_required, out.len);
    LFM25_ENSURE(x.ptr && weight.ptr && out.ptr, LFM25_ERR_NULL_POINTER,
                 "FP8 linear received a null device pointer");
    LFM25_ENSURE(m <= 0x7fffffffu && n <= 0x7fffffffu && k <= 0x7fffffffu, LFM25_ERR_INVALID_ARGUMENT,
                 "FP8 linear dimension exceeds i32");
    const bool aligned = ((reinterpret_cast<uintptr_t>(x.ptr) | reinterpret_cast<uintptr_t>(weight.ptr) |
                           reinterpret_cast<uintptr_t>(out.ptr)) &
                          15) == 0;
    const bool stream_ok = aligned && lfm25::fp8_gemm_stream_supports(m, n, k);
    const bool umma_ok = aligned && lfm25::fp8_gemm_umma_supports(m, n, k);
    // The tcgen05 kernel is at least as fast as the streaming kernel from M = 1 on once it can occupy the machine
    // (LM head at M = 1: 24.1 against 29.2 us), i.e. with at least 100 weight tiles or with an exchange buffer to
    // split K through; without either (few tiles, handle-free call) small batches stay on the streaming kernel.
    const bool umma_occupies = umma_ok && (n / 128 >= 100 || exchange != nullptr);
    const bool rows_ok = aligned && lfm25::gemm_rows_supports(m, n, k);
    enum { kStream, kUmma, kGeneric, kRows } path = kGeneric;
    if (rows_ok && handle != nullptr && lfm25::fp8_rows_preferred(m, n, k)) {
        path = kRows;
    } else if (umma_occupies || (umma_ok && !(stream_ok && m <= 8))) {
        path = kUmma;
    } else if (stream_ok) {
        path = kStream;
    }
    const int64_t forced = handle != nullptr && handle->tuning_kernel != 0 ? handle->tuning_kernel
                                                                           : lfm25::option(lfm25::kOptFp8GemmPath);
    if (forced == lfm25::kPathStream && stream_ok) path = kStream;
    if (forced == lfm25::kPathUmma && umma_ok) path = kUmma;
    if (forced == lfm25::kPathGeneric) path = kGeneric;
    if (forced == lfm25::kPathRows && rows_ok) path = kRows;
    cudaError_t status;
    if (path == kRows) {
        unsigned int* status_words = device_status_pointer();
        LFM25_ENSURE(status_words != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
        status = lfm25::launch_fp8_gemm_rows(stream, x.ptr, weight.ptr, out.ptr, m, n, k, config->output_scale,
                                             exchange, exchange_bytes, status_words,
                                             handle != nullptr ? handle->tuning : lfm25::GemmRowsTuning());
    } else if (path == kStream) {
        status = lfm25::launch_fp8_gemm_stream(stream, x.ptr, weight.ptr, out.ptr, m, n, k, config->output_scale);
    } else if (path == kUmma) {
        unsigned int* status_words = device_status_pointer();
        LFM25_ENSURE(status_words != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
        status = lfm25::launch_fp8_gemm_umma(stream, x.ptr, weight.ptr, out.ptr, m, n, k, config->output_scale,
                                             exchange, exchange_bytes, status_words);
    } else {
        status = lfm25::launch_fp8_gemm_generic(stream, x.ptr, weight.ptr, out.ptr, m, n, k, config->output_scale);
    }
    return cuda_result(status, "FP8 linear launch failed");
}

}  // namespace

namespace lfm25 {
int32_t report_error(int32_t code, const char* message) { return fail(code, "%s", message); }
}  // namespace lfm25

extern "C" {

const char* lfm25_last_error(void) { return g_last_error; }

const char* lfm25_version(void) { return "lfm25_b200 0.1 sm_100a"; }

int32_t lfm25_device_status(void* stream, uint32_t out[4]) {
    LFM25_ENSURE(out != nullptr, LFM25_ERR_NULL_POINTER, "device status output is null");
    unsigned int* pointer = device_status_pointer();
    LFM25_ENSURE(pointer != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
    cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
    cudaError_t status = cudaMemcpyAsync(out, pointer, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost, cuda_stream);
    if (status == cudaSuccess) {
        status = cudaMemsetAsync(pointer, 0, 4 * sizeof(uint32_t), cuda_stream);
    }
    if (status == cudaSuccess) {
        status = cudaStreamSynchronize(cuda_stream);
    }
    return cuda_result(status, "device status read failed");
}

int32_t lfm25_kv_cache_write_lfm2_bf16(void* stream, const lfm25_kv_cache_write_launch* launch) {
    LFM25_ENSURE(launch != nullptr, LFM25_ERR_NULL_POINTER, "KV cache write launch is null");
    const lfm25_kv_cache_write_launch& l = *launch;
    LFM25_ENSURE(l.num_tokens > 0, LFM25_ERR_INVALID_ARGUMENT, "KV cache write requires at least one token");
    LFM25_ENSURE(l.num_pages > 0, LFM25_ERR_INVALID_ARGUMENT, "KV cache requires at least one page");
    size_t required = 0;
    LFM25_ENSURE(checked_mul(l.num_tokens, 8 * 64, &required), LFM25_ERR_OVERFLOW, "KV input size overflow");
    size_t cache_required = 0;
    LFM25_ENSURE(cache_elements(l.num_pages, l.page_size, &cache_required), LFM25_ERR_OVERFLOW,
                 "KV cache size overflow");
    LFM25_ENSURE(l.key.len >= required, LFM25_ERR_BUFFER_TOO_SMALL, "K storage too small");
    LFM25_ENSURE(l.value.len >= required, LFM25_ERR_BUFFER_TOO_SMALL, "V storage too small");
    LFM25_ENSURE(l.key_cache.len >= cache_required, LFM25_ERR_BUFFER_TOO_SMALL, "K cache storage too small");
    LFM25_ENSURE(l.value_cache.len >= cache_required, LFM25_ERR_BUFFER_TOO_SMALL, "V cache storage too small");
    LFM25_ENSURE(l.slot_mapping.len >= l.num_tokens, LFM25_ERR_BUFFER_TOO_SMALL, "slot mapping storage too small");
    LFM25_ENSURE(l.page_size == 16 || l.page_size == 32, LFM25_ERR_INVALID_ARGUMENT, "unsupported KV page size %zu",
                 l.page_size);
    LFM25_ENSURE(l.page_size == 16, LFM25_ERR_UNSUPPORTED, "page size 32 is not built; use 16");
    LFM25_ENSURE(l.key.ptr && l.value.ptr && l.key_cache.ptr && l.value_cache.ptr && l.slot_mapping.ptr,
                 LFM25_ERR_NULL_POINTER, "KV cache write received a null device pointer");
    LFM25_ENSURE(l.num_tokens <= 0x7fffffffu, LFM25_ERR_INVALID_ARGUMENT, "KV cache write grid size exceeds u32");
    LFM25_ENSURE(((reinterpret_cast<uintptr_t>(l.key.ptr) | reinterpret_cast<uintptr_t>(l.value.ptr) |
                   reinterpret_cast<uintptr_t>(l.key_cache.ptr) | reinterpret_cast<uintptr_t>(l.value_cache.ptr)) &
                  15) == 0,
                 LFM25_ERR_INVALID_ARGUMENT, "KV cache write buffers must be 16-byte aligned");
    return cuda_result(
        lfm25::launch_kv_cache_write(static_cast<cudaStream_t>(stream), l.key.ptr, l.value.ptr, l.key_cache.ptr,
                                     l.value_cache.ptr, static_cast<const int64_t*>(l.slot_mapping.ptr), l.num_tokens,
                                     l.num_pages),
        "KV cache write launch failed");
}

int32_t lfm25_qk_norm_rope_kv_write_decode(void* stream, const lfm25_qk_postprocess_launch* launch) {
    LFM25_ENSURE(launch != nullptr, LFM25_ERR_NULL_POINTER, "fused QK postprocess launch is null");
    const lfm25_qk_postprocess_launch& l = *launch;
    LFM25_ENSURE(l.num_tokens > 0, LFM25_ERR_INVALID_ARGUMENT, "fused QK postprocess requires tokens");
    LFM25_ENSURE(l.num_pages > 0, LFM25_ERR_INVALID_ARGUMENT, "fused QK postprocess requires cache pages");
    size_t q_required = 0;
    LFM25_ENSURE(checked_mul(l.num_tokens, 32 * 64, &q_required), LFM25_ERR_OVERFLOW, "fused Q storage overflow");
    size_t kv_required = 0;
    LFM25_ENSURE(checked_mul(l.num_tokens, 8 * 64, &kv_required), LFM25_ERR_OVERFLOW, "fused KV storage overflow");
    size_t cache_required = 0;
    LFM25_ENSURE(cache_elements(l.num_pages, l.page_size, &cache_required), LFM25_ERR_OVERFLOW,
                 "fused cache storage overflow");
    LFM25_ENSURE(l.query.len >= q_required, LFM25_ERR_BUFFER_TOO_SMALL, "fused Q storage too small");
    LFM25_ENSURE(l.key.len >= kv_required, LFM25_ERR_BUFFER_TOO_SMALL, "fused K storage too small");
    LFM25_ENSURE(l.value.len >= kv_required, LFM25_ERR_BUFFER_TOO_SMALL, "fused V storage too small");
    LFM25_ENSURE(l.query_norm.len >= 64, LFM25_ERR_BUFFER_TOO_SMALL, "query norm weight too small");
    LFM25_ENSURE(l.key_norm.len >= 64, LFM25_ERR_BUFFER_TOO_SMALL, "key norm weight too small");
    LFM25_ENSURE(l.inv_freq.len >= 32, LFM25_ERR_BUFFER_TOO_SMALL, "RoPE frequency storage too small");
    LFM25_ENSURE(l.position_ids.len >= l.num_tokens, LFM25_ERR_BUFFER_TOO_SMALL, "position storage too small");
    LFM25_ENSURE(l.slot_mapping.len >= l.num_tokens, LFM25_ERR_BUFFER_TOO_SMALL, "slot mapping storage too small");
    LFM25_ENSURE(l.key_cache.len >= cache_required, LFM25_ERR_BUFFER_TOO_SMALL, "K cache storage too small");
    LFM25_ENSURE(l.value_cache.len >= cache_required, LFM25_ERR_BUFFER_TOO_SMALL, "V cache storage too small");
    LFM25_ENSURE(l.page_size == 16 || l.page_size == 32, LFM25_ERR_INVALID_ARGUMENT,
                 "unsupported fused QK page size %zu", l.page_size);
    LFM25_ENSURE(l.page_size == 16, LFM25_ERR_UNSUPPORTED, "page size 32 is not built; use 16");
    LFM25_ENSURE(l.num_tokens <= 0x7fffffffu, LFM25_ERR_INVALID_ARGUMENT, "fused QK grid size exceeds u32");
    LFM25_ENSURE(l.query.ptr && l.key.ptr && l.value.ptr && l.query_norm.ptr && l.key_norm.ptr && l.inv_freq.ptr &&
                     l.position_ids.ptr && l.slot_mapping.ptr && l.key_cache.ptr && l.value_cache.ptr,
                 LFM25_ERR_NULL_POINTER, "fused QK postprocess received a null device pointer");
    lfm25::QkPostprocessArgs args;
    args.query = l.query.ptr;
    args.query_out = l.query.ptr;
    args.query_token_stride = 32 * 64;
    args.kv_token_stride = 8 * 64;
    args.key = l.key.ptr;
    args.value = l.value.ptr;
    args.query_norm = l.query_norm.ptr;
    args.key_norm = l.key_norm.ptr;
    args.inv_freq = static_cast<const float*>(l.inv_freq.ptr);
    args.position_ids = static_cast<const uint32_t*>(l.position_ids.ptr);
    args.slot_mapping = static_cast<const int64_t*>(l.slot_mapping.ptr);
    args.key_cache = l.key_cache.ptr;
    args.value_cache = l.value_cache.ptr;
    args.num_tokens = l.num_tokens;
    args.num_pages = l.num_pages;
    args.eps = l.eps;
    return cuda_result(lfm25::launch_qk_norm_rope_kv_write_decode(static_cast<cudaStream_t>(stream), args),
                       "fused QK postprocess launch failed");
}

int32_t lfm25_paged_attention_fast_lfm2_bf16(void* stream, const lfm25_paged_attention_launch* launch) {
    LFM25_ENSURE(launch != nullptr, LFM25_ERR_NULL_POINTER, "fast-exp attention launch is null");
    const lfm25_paged_attention_launch& l = *launch;
    LFM25_ENSURE(l.num_tokens > 0, LFM25_ERR_INVALID_ARGUMENT, "fast-exp attention requires tokens");
    LFM25_ENSURE(l.num_pages > 0, LFM25_ERR_INVALID_ARGUMENT, "fast-exp attention requires cache pages");
    LFM25_ENSURE(l.block_table.len > 0, LFM25_ERR_INVALID_ARGUMENT, "fast-exp attention block table is empty");
    // One sequence is the ragged form with a single row that every token reads.
    const int32_t status = validate_ragged_common(l.page_size, l.query, l.key_cache, l.value_cache, l.block_table,
                                                  nullptr, l.position_ids, l.output, l.num_tokens, l.num_pages,
                                                  l.block_table.len);
    if (status != LFM25_OK) {
        return status;
    }
    lfm25::AttentionLaunch args = {};
    args.query = l.query.ptr;
    args.key_cache = l.key_cache.ptr;
    args.value_cache = l.value_cache.ptr;
    args.block_tables = static_cast<const uint32_t*>(l.block_table.ptr);
    args.request_slots = nullptr;
    args.position_ids = static_cast<const uint32_t*>(l.position_ids.ptr);
    args.output = l.output.ptr;
    args.partials = nullptr;
    args.status = device_status_pointer();
    args.num_tokens = l.num_tokens;
    args.num_pages = l.num_pages;
    args.block_table_stride = l.block_table.len;
    args.block_table_rows = 1;
    args.num_splits = 1;
    LFM25_ENSURE(args.status != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
    return cuda_result(lfm25::launch_ragged_decode_attention(static_cast<cudaStream_t>(stream), args),
                       "fast-exp attention launch failed");
}

namespace {
// The optional token order of a decode attention launch: null, or at least num_tokens entries.
int32_t take_token_order(const lfm25_slice& order, size_t num_tokens, const uint32_t** out) {
    *out = nullptr;
    if (order.ptr == nullptr) {
        return LFM25_OK;
    }
    LFM25_ENSURE(order.len >= num_tokens, LFM25_ERR_BUFFER_TOO_SMALL,
                 "token order too small: required=%zu, actual=%zu", num_tokens, order.len);
    *out = static_cast<const uint32_t*>(order.ptr);
    return LFM25_OK;
}
}  // namespace

int32_t lfm25_context_order_desc(void* stream, lfm25_slice position_ids, size_t num_tokens, lfm25_slice order) {
    LFM25_ENSURE(num_tokens > 0 && num_tokens <= lfm25::kMaxOrderTokens, LFM25_ERR_INVALID_ARGUMENT,
                 "context order takes 1..=%zu tokens, got %zu", lfm25::kMaxOrderTokens, num_tokens);
    LFM25_ENSURE(position_ids.ptr != nullptr && order.ptr != nullptr, LFM25_ERR_NULL_POINTER,
                 "context order received a null device pointer");
    LFM25_ENSURE(position_ids.len >= num_tokens && order.len >= num_tokens, LFM25_ERR_BUFFER_TOO_SMALL,
                 "context order buffers too small for %zu tokens", num_tokens);
    return cuda_result(lfm25::launch_context_order(static_cast<cudaStream_t>(stream),
                                                   static_cast<const uint32_t*>(position_ids.ptr), num_tokens,
                                                   static_cast<uint32_t*>(order.ptr)),
                       "context order launch failed");
}

int32_t lfm25_paged_ragged_attention_fast_lfm2_bf16(void* stream, const lfm25_fast_ragged_attention_launch* launch) {
    LFM25_ENSURE(launch != nullptr, LFM25_ERR_NULL_POINTER, "fast-exp ragged attention launch is null");
    const lfm25_fast_ragged_attention_launch& l = *launch;
    const int32_t status =
        validate_ragged_common(l.page_size, l.query, l.key_cache, l.value_cache, l.block_tables, &l.request_slots,
                               l.position_ids, l.output, l.num_tokens, l.num_pages, l.block_table_stride);
    if (status != LFM25_OK) {
        return status;
    }
    lfm25::AttentionLaunch args = {};
    args.query = l.query.ptr;
    args.key_cache = l.key_cache.ptr;
    args.value_cache = l.value_cache.ptr;
    args.block_tables = static_cast<const uint32_t*>(l.block_tables.ptr);
    args.request_slots = static_cast<const uint32_t*>(l.request_slots.ptr);
    args.position_ids = static_cast<const uint32_t*>(l.position_ids.ptr);
    args.output = l.output.ptr;
    args.partials = nullptr;
    args.status = device_status_pointer();
    args.num_tokens = l.num_tokens;
    args.num_pages = l.num_pages;
    args.block_table_stride = l.block_table_stride;
    args.block_table_rows = l.block_tables.len / l.block_table_stride;
    args.num_splits = 1;
    {
        const int32_t order_status = take_token_order(l.token_order, l.num_tokens, &args.token_order);
        if (order_status != LFM25_OK) return order_status;
    }
    LFM25_ENSURE(args.status != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
    return cuda_result(lfm25::launch_ragged_decode_attention(static_cast<cudaStream_t>(stream), args),
                       "fast-exp ragged attention launch failed");
}

int32_t lfm25_paged_ragged_attention_splitk_lfm2_bf16(void* stream,
                                                      const lfm25_splitk_ragged_attention_launch* launch) {
    LFM25_ENSURE(launch != nullptr, LFM25_ERR_NULL_POINTER, "split-K ragged attention launch is null");
    const lfm25_splitk_ragged_attention_launch& l = *launch;
    const int32_t status =
        validate_ragged_common(l.page_size, l.query, l.key_cache, l.value_cache, l.block_tables, &l.request_slots,
                               l.position_ids, l.output, l.num_tokens, l.num_pages, l.block_table_stride);
    if (status != LFM25_OK) {
        return status;
    }
    LFM25_ENSURE(l.num_splits >= 2 && l.num_splits <= 8, LFM25_ERR_INVALID_ARGUMENT,
                 "split-K ragged attention requires 2..=8 splits");
    size_t partial_required = 0;
    LFM25_ENSURE(checked_mul(l.num_tokens, 32, &partial_required) &&
                     checked_mul(partial_required, l.num_splits, &partial_required) &&
                     checked_mul(partial_required, 66, &partial_required),
                 LFM25_ERR_OVERFLOW, "split-K partial workspace size overflow");
    // No workspace at all (null pointer, zero length): the splits of a token merge inside the kernel, as one
    // thread-block cluster per (token, KV head), and no records are written.
    const bool in_kernel_merge = l.partials.ptr == nullptr && l.partials.len == 0;
    if (in_kernel_merge) {
        LFM25_ENSURE(l.num_splits == 2 || l.num_splits == 4 || l.num_splits == 8, LFM25_ERR_INVALID_ARGUMENT,
                     "split-K ragged attention without a workspace takes 2, 4 or 8 splits");
    } else {
        LFM25_ENSURE(l.partials.len >= partial_required, LFM25_ERR_BUFFER_TOO_SMALL,
                     "split-K partial workspace too small: need %zu, have %zu", partial_required, l.partials.len);
        LFM25_ENSURE(l.partials.ptr != nullptr, LFM25_ERR_NULL_POINTER, "split-K partial workspace is null");
    }
    lfm25::AttentionLaunch args = {};
    args.query = l.query.ptr;
    args.key_cache = l.key_cache.ptr;
    args.value_cache = l.value_cache.ptr;
    args.block_tables = static_cast<const uint32_t*>(l.block_tables.ptr);
    args.request_slots = static_cast<const uint32_t*>(l.request_slots.ptr);
    args.position_ids = static_cast<const uint32_t*>(l.position_ids.ptr);
    args.output = l.output.ptr;
    args.partials = static_cast<float*>(l.partials.ptr);
    args.status = device_status_pointer();
    args.num_tokens = l.num_tokens;
    args.num_pages = l.num_pages;
    args.block_table_stride = l.block_table_stride;
    args.block_table_rows = l.block_tables.len / l.block_table_stride;
    args.num_splits = static_cast<uint32_t>(l.num_splits);
    {
        const int32_t order_status = take_token_order(l.token_order, l.num_tokens, &args.token_order);
        if (order_status != LFM25_OK) return order_status;
    }
    LFM25_ENSURE(args.status != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
    return cuda_result(lfm25::launch_ragged_decode_attention(static_cast<cudaStream_t>(stream), args),
                       "split-K ragged attention launch failed");
}

int32_t lfm25_fused_ragged_paged_attention_decode_lfm2_bf16(void* stream,
                                                            const lfm25_fused_ragged_decode_launch* launch) {
    LFM25_ENSURE(launch != nullptr, LFM25_ERR_NULL_POINTER, "fused ragged decode launch is null");
    const lfm25_fused_ragged_decode_launch& l = *launch;
    const int32_t status =
        validate_ragged_common(l.page_size, l.query_raw, l.key_cache, l.value_cache, l.block_tables, &l.request_slots,
                               l.position_ids, l.output, l.num_tokens, l.num_pages, l.block_table_stride);
    if (status != LFM25_OK) {
        return status;
    }
    size_t kv_required = 0;
    LFM25_ENSURE(checked_mul(l.num_tokens, 8 * 64, &kv_required), LFM25_ERR_OVERFLOW, "fused KV storage overflow");
    const size_t query_stride = l.query_token_stride == 0 ? 32 * 64 : l.query_token_stride;
    const size_t kv_stride = l.kv_token_stride == 0 ? 8 * 64 : l.kv_token_stride;
    LFM25_ENSURE(query_stride >= 32 * 64 && kv_stride >= 8 * 64 && query_stride % 2 == 0 && kv_stride % 2 == 0,
                 LFM25_ERR_INVALID_ARGUMENT, "fused token strides must be even and at least 2048 / 512 elements");
    if (l.num_tokens > 0) {
        size_t query_required = 0;
        LFM25_ENSURE(checked_mul(l.num_tokens - 1, query_stride, &query_required) &&
                         checked_mul(l.num_tokens - 1, kv_stride, &kv_required),
                     LFM25_ERR_OVERFLOW, "fused strided storage overflow");
        query_required += 32 * 64;
        kv_required += 8 * 64;
        LFM25_ENSURE(l.query_raw.len >= query_required, LFM25_ERR_BUFFER_TOO_SMALL, "fused Q storage too small");
    }
    LFM25_ENSURE(l.key_raw.len >= kv_required, LFM25_ERR_BUFFER_TOO_SMALL, "fused K storage too small");
    LFM25_ENSURE(l.value_raw.len >= kv_required, LFM25_ERR_BUFFER_TOO_SMALL, "fused V storage too small");
    LFM25_ENSURE(l.query_norm.len >= 64, LFM25_ERR_BUFFER_TOO_SMALL, "query norm weight too small");
    LFM25_ENSURE(l.key_norm.len >= 64, LFM25_ERR_BUFFER_TOO_SMALL, "key norm weight too small");
    LFM25_ENSURE(l.inv_freq.len >= 32, LFM25_ERR_BUFFER_TOO_SMALL, "RoPE frequency storage too small");
    LFM25_ENSURE(l.slot_mapping.len >= l.num_tokens, LFM25_ERR_BUFFER_TOO_SMALL, "slot mapping storage too small");
    LFM25_ENSURE(l.key_raw.ptr && l.value_raw.ptr && l.query_norm.ptr && l.key_norm.ptr && l.inv_freq.ptr &&
                     l.slot_mapping.ptr,
                 LFM25_ERR_NULL_POINTER, "fused ragged decode received a null device pointer");
    const size_t splits = l.num_splits == 0 ? 1 : l.num_splits;
    LFM25_ENSURE(splits <= 8, LFM25_ERR_INVALID_ARGUMENT, "split-K ragged attention requires 2..=8 splits");
    if (splits > 1) {
        size_t partial_required = 0;
        LFM25_ENSURE(checked_mul(l.num_tokens, 32, &partial_required) &&
                         checked_mul(partial_required, splits, &partial_required) &&
                         checked_mul(partial_required, 66, &partial_required),
                     LFM25_ERR_OVERFLOW, "split-K partial workspace size overflow");
        if (l.partials.ptr == nullptr && l.partials.len == 0) {
            // no workspace: the splits merge inside the kernel (one cluster per token and KV head)
            LFM25_ENSURE(splits == 2 || splits == 4 || splits == 8, LFM25_ERR_INVALID_ARGUMENT,
                         "fused decode attention without a workspace takes 1, 2, 4 or 8 splits");
        } else {
            LFM25_ENSURE(l.partials.ptr != nullptr && l.partials.len >= partial_required, LFM25_ERR_BUFFER_TOO_SMALL,
                         "split-K partial workspace too small: need %zu, have %zu", partial_required, l.partials.len);
        }
    }
    lfm25::AttentionLaunch args = {};
    args.query = l.query_raw.ptr;
    args.key_cache = l.key_cache.ptr;
    args.value_cache = l.value_cache.ptr;
    args.block_tables = static_cast<const uint32_t*>(l.block_tables.ptr);
    args.request_slots = static_cast<const uint32_t*>(l.request_slots.ptr);
    args.position_ids = static_cast<const uint32_t*>(l.position_ids.ptr);
    args.output = l.output.ptr;
    args.partials = static_cast<float*>(l.partials.ptr);
    args.status = device_status_pointer();
    args.num_tokens = l.num_tokens;
    args.num_pages = l.num_pages;
    args.block_table_stride = l.block_table_stride;
    args.block_table_rows = l.block_tables.len / l.block_table_stride;
    args.num_splits = static_cast<uint32_t>(splits);
    args.key_raw = l.key_raw.ptr;
    args.value_raw = l.value_raw.ptr;
    args.query_norm = l.query_norm.ptr;
    args.key_norm = l.key_norm.ptr;
    args.inv_freq = static_cast<const float*>(l.inv_freq.ptr);
    args.slot_mapping = static_cast<const int64_t*>(l.slot_mapping.ptr);
    args.eps = l.eps;
    args.query_token_stride = query_stride;
    args.kv_token_stride = kv_stride;
    {
        const int32_t order_status = take_token_order(l.token_order, l.num_tokens, &args.token_order);
        if (order_status != LFM25_OK) return order_status;
    }
    LFM25_ENSURE(args.status != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
    return cuda_result(lfm25::launch_ragged_decode_attention(static_cast<cudaStream_t>(stream), args),
                       "fused ragged decode launch failed");
}

int32_t lfm25_hybrid_ragged_attention_lfm2_bf16(void* stream, const lfm25_hybrid_attention_launch* launch) {
    LFM25_ENSURE(launch != nullptr, LFM25_ERR_NULL_POINTER, "hybrid attention launch is null");
    const lfm25_hybrid_attention_launch& l = *launch;
    // src/cuda/kernels/attention.rs:153-196
    LFM25_ENSURE(l.page_size == 16 || l.page_size == 32, LFM25_ERR_INVALID_ARGUMENT,
                 "unsupported hybrid attention page size %zu", l.page_size);
    LFM25_ENSURE(l.page_size == 16, LFM25_ERR_UNSUPPORTED, "page size 32 is not built; use 16");
    LFM25_ENSURE(l.num_tokens > 0, LFM25_ERR_INVALID_ARGUMENT, "hybrid ragged attention requires tokens");
    LFM25_ENSURE(l.num_segments > 0, LFM25_ERR_INVALID_ARGUMENT, "hybrid ragged attention requires segments");
    LFM25_ENSURE(l.num_pages > 0, LFM25_ERR_INVALID_ARGUMENT, "hybrid ragged attention requires cache pages");
    LFM25_ENSURE(l.block_table_stride > 0, LFM25_ERR_INVALID_ARGUMENT, "hybrid block table is empty");
    LFM25_ENSURE(l.request_slots.len >= l.num_tokens, LFM25_ERR_BUFFER_TOO_SMALL, "request slots too small");
    LFM25_ENSURE(l.position_ids.len >= l.num_tokens, LFM25_ERR_BUFFER_TOO_SMALL, "positions too small");
    LFM25_ENSURE(l.segment_offsets.len > l.num_segments, LFM25_ERR_BUFFER_TOO_SMALL, "segment offsets too small");
    LFM25_ENSURE(l.num_tokens <= 0x7fffffffu && l.num_pages <= 0x00ffffffu && l.num_segments <= 0x7fffffffu,
                 LFM25_ERR_INVALID_ARGUMENT, "hybrid attention sizes exceed the kernel's index range");
    const size_t query_stride = l.query_token_stride == 0 ? 32 * 64 : l.query_token_stride;
    const size_t kv_stride = l.kv_token_stride == 0 ? 8 * 64 : l.kv_token_stride;
    LFM25_ENSURE(query_stride >= 32 * 64 && query_stride % 2 == 0 && kv_stride >= 8 * 64 && kv_stride % 8 == 0,
                 LFM25_ERR_INVALID_ARGUMENT,
                 "hybrid token strides: query even and >= 2048, K/V a multiple of 8 and >= 512 elements");
    size_t q_dense = 0;
    size_t q_required = 0;
    size_t kv_required = 0;
    size_t cache_required = 0;
    LFM25_ENSURE(checked_mul(l.num_tokens, 32 * 64, &q_dense) &&
                     checked_mul(l.num_tokens - 1, query_stride, &q_required) &&
                     checked_mul(l.num_tokens - 1, kv_stride, &kv_required),
                 LFM25_ERR_OVERFLOW, "hybrid query size overflow");
    q_required += 32 * 64;
    kv_required += 8 * 64;
    LFM25_ENSURE(checked_mul(l.num_pages, 8 * 16 * 64, &cache_required), LFM25_ERR_OVERFLOW,
                 "hybrid cache size overflow");
    LFM25_ENSURE(l.query.len >= q_required && l.output.len >= q_dense, LFM25_ERR_BUFFER_TOO_SMALL,
                 "hybrid Q/O storage too small");
    const bool contiguous = l.current_key.ptr != nullptr;
    if (contiguous) {
        LFM25_ENSURE(l.current_value.ptr != nullptr, LFM25_ERR_NULL_POINTER, "hybrid current V is null");
        LFM25_ENSURE(l.current_key.len >= kv_required && l.current_value.len >= kv_required,
                     LFM25_ERR_BUFFER_TOO_SMALL, "hybrid contiguous KV storage too small");
        LFM25_ENSURE(((reinterpret_cast<uintptr_t>(l.current_key.ptr) |
                       reinterpret_cast<uintptr_t>(l.current_value.ptr)) & 15) == 0,
                     LFM25_ERR_INVALID_ARGUMENT, "hybrid contiguous K/V must be 16-byte aligned");
    }
    LFM25_ENSURE(l.key_cache.len >= cache_required && l.value_cache.len >= cache_required,
                 LFM25_ERR_BUFFER_TOO_SMALL, "hybrid paged KV storage too small");
    LFM25_ENSURE(l.block_tables.len >= l.block_table_stride, LFM25_ERR_BUFFER_TOO_SMALL,
                 "hybrid block table storage too small");
    LFM25_ENSURE(l.query.ptr && l.output.ptr && l.key_cache.ptr && l.value_cache.ptr && l.block_tables.ptr &&
                     l.request_slots.ptr && l.position_ids.ptr && l.segment_offsets.ptr,
                 LFM25_ERR_NULL_POINTER, "hybrid attention received a null device pointer");
    LFM25_ENSURE(((reinterpret_cast<uintptr_t>(l.key_cache.ptr) | reinterpret_cast<uintptr_t>(l.value_cache.ptr)) &
                  127) == 0,
                 LFM25_ERR_INVALID_ARGUMENT, "hybrid paged K/V must be 128-byte aligned");
    lfm25::HybridAttentionLaunch args = {};
    args.query = l.query.ptr;
    args.current_key = contiguous ? l.current_key.ptr : nullptr;
    args.current_value = contiguous ? l.current_value.ptr : nullptr;
    args.key_cache = l.key_cache.ptr;
    args.value_cache = l.value_cache.ptr;
    args.block_tables = static_cast<const uint32_t*>(l.block_tables.ptr);
    args.request_slots = static_cast<const uint32_t*>(l.request_slots.ptr);
    args.position_ids = static_cast<const uint32_t*>(l.position_ids.ptr);
    args.segment_offsets = static_cast<const uint32_t*>(l.segment_offsets.ptr);
    args.output = l.output.ptr;
    args.status = device_status_pointer();
    args.num_tokens = l.num_tokens;
    args.num_pages = l.num_pages;
    args.block_table_stride = l.block_table_stride;
    args.block_table_rows = l.block_tables.len / l.block_table_stride;
    args.num_segments = l.num_segments;
    args.query_token_stride = query_stride;
    args.kv_token_stride = kv_stride;
    LFM25_ENSURE(args.status != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
    // Two kernels: tcgen05 / TMEM with 32 tokens x 4 heads per CTA (191 us per layer on eight 512-token chunks) and
    // mma.sync with 16 tokens per CTA (326 us there, but less padding on short segments).  The tcgen05 kernel takes
    // the step when its segments average at least 16 tokens; the option hybrid_attention = umma | mma forces one.
    const int64_t choice = lfm25::option(lfm25::kOptHybridAttention);
    const bool umma_possible = (reinterpret_cast<uintptr_t>(l.query.ptr) & 15) == 0 && query_stride % 8 == 0;
    bool use_umma = l.num_tokens >= 16 * l.num_segments;
    if (choice == 1) use_umma = true;
    if (choice == 2) use_umma = false;
    if (use_umma && umma_possible) {
        return cuda_result(lfm25::launch_hybrid_attention_umma(static_cast<cudaStream_t>(stream), args),
                           "hybrid ragged attention launch failed");
    }
    return cuda_result(lfm25::launch_hybrid_ragged_attention(static_cast<cudaStream_t>(stream), args),
                       "hybrid ragged attention launch failed");
}

size_t lfm25_splitk_workspace_elements(size_t maximum_tokens) {
    size_t value = 0;
    if (!checked_mul(maximum_tokens, 32, &value) || !checked_mul(value, 8, &value) ||
        !checked_mul(value, 66, &value)) {
        return 0;
    }
    return value;
}

size_t lfm25_splitk_decode_splits(size_t num_tokens, size_t maximum_context_tokens, size_t page_size) {
    if (num_tokens == 0 || page_size != 16) {
        return 1;
    }
    // A B200 keeps 148 SMs x 3 CTAs = 444 (token, KV head, split) items resident, and the callers hand the CTAs out
    // longest context first, so a little more than one wave of items is enough.  Measured on the full decode step
    // (contexts 128..4096, splits -> ms per step): 8 sequences 2/4/8 -> 0.766/0.727/0.725; 16: 2/4/8 ->
    // 0.788/0.750/0.782; 32: 1/2/4/8 -> 0.943/0.874/0.883/0.925; 48: 1/2/4 -> 1.002/0.957/0.992; 64: 1/2/4 ->
    // 1.050/1.030/1.066; 96: 1/2 -> 1.197/1.229; 128: 1/2/3/4 -> 1.336/1.377/1.404/1.441.  With contexts up to 8192
    // (64 sequences, attention alone, 1/2/4/8 -> 113/100/99/105 us) one more doubling pays.  Never below 8 pages
    // (128 tokens) per split.
    const int64_t forced = lfm25::option(lfm25::kOptDecodeSplits);   // 0 = by the table below
    if (forced >= 1 && forced <= 8) {
        return static_cast<size_t>(forced);
    }
    const size_t pages = (maximum_context_tokens + page_size - 1) / page_size;
    size_t splits = num_tokens <= 8 ? 8 : (num_tokens <= 24 ? 4 : (num_tokens <= 80 ? 2 : 1));
    if (num_tokens > 24 && num_tokens <= 80 && maximum_context_tokens > 6144) {
        splits = 4;
    }
    while (splits > 1 && pages / splits < 8) {
        splits /= 2;
    }
    return splits;
}

size_t lfm25_bf16_own_kernel_max_rows(void) {
    // Whole decode step, every BF16 site on the weight-major tcgen05 kernel against every one through cuBLASLt
    // (ms per step on a B200): 32 sequences 1.023 / 1.046, 40: 0.882 / 0.918, 48: 0.918 / 0.941, 64: 1.012 / 1.012,
    // 80: 1.166 / 1.120, 128: 1.415 / 1.322.  A choice per site above 48 rows (own kernel for Down up to 96 rows and
    // Gate/Up up to 112, where its kernel time inside an all-own step is the shorter one; cuBLASLt for the sites with
    // few weight tiles) was measured too: 64 sequences 1.009, 80 1.138 (cuBLASLt for all: 1.120), 96 1.186 (1.189) --
    // an own kernel between two library kernels loses the overlap with its neighbours that makes it faster.
    return 48;
}

uint64_t lfm25_blaslt_library_calls(void) { return lfm25::cublaslt_bf16_calls(); }

int32_t lfm25_decode_one_kernel_preferred(size_t page_size, size_t context_tokens, size_t batch_size) {
    if (page_size != 16 || batch_size == 0) {
        return 0;
    }
    if (lfm25::option(lfm25::kOptPdl) == 0) {
        // Without programmatic dependent launch the boundary between the append and the attention kernel costs a
        // full launch gap, as it did where the reference measured its table (src/ops/mok_dispatch.rs:12-18).
        return (context_tokens <= 16 || (context_tokens <= 32 && batch_size <= 32) ||
                (context_tokens <= 64 && batch_size <= 8))
                   ? 1
                   : 0;
    }
    // Measured on a B200 inside the whole decode step (graph replay, 6 attention layers; microseconds per attention
    // layer that the one kernel costs more (+) or less (-) than QK-norm + RoPE + append followed by attention):
    //   sequences   ctx 16   ctx 64   ctx 128   ctx 512   ctx 2048   ctx 128..4096 (ragged)
    //        1       +0.7     +0.4     +0.4      +0.4      +0.8       +0.8
    //        4       +0.2     -0.2     -0.2      -0.3      -0.2       -0.4
    //        8       +0.2     +0.3     +0.2      -0.1      +1.8       +1.8
    //       16       -0.4     -0.6     -0.6      +2.0      +1.8       -1.5
    //       32       -1.5     -0.9     -2.1      +2.4      +2.1       -2.2
    //       64       +0.8     +1.2     +1.5      +3.6      +2.1       +2.5
    //      128       +2.5     +2.3     +3.2      +2.5      +1.9       -0.7
    // The dependent launch hides the boundary between the two kernels, so the one kernel wins only where its
    // per-CTA prologue (norm, rotation and append before the first page can be read) is hidden as well: 16 to 32
    // sequences with short contexts, and batches whose maximum context is long, which in serving means a ragged
    // batch -- the CTAs are handed out longest context first, so the short sequences' prologues run in the shadow
    // of the long ones.  (One attention layer alone, both routes in a graph of 32 repetitions, uniform contexts:
    // two launches / one kernel = 10.2 / 14.2 us at 128 sequences x 16 tokens, 89.6 / 90.5 us at 128 x 2048,
    // 5.0 / 5.1 us at 1 x 40.)
    const bool mid_batch = batch_size >= 16 && batch_size <= 32;
    const bool large_batch = batch_size > 64;
    return ((mid_batch && (context_tokens <= 128 || context_tokens > 2048)) || (large_batch && context_tokens > 2048))
               ? 1
               : 0;
}

int32_t lfm25_quantize_bf16_e4m3(void* stream, lfm25_slice input, lfm25_slice output, size_t numel, float scale) {
    LFM25_ENSURE(numel > 0, LFM25_ERR_INVALID_ARGUMENT, "FP8 quantization requires at least one element");
    LFM25_ENSURE(input.len >= numel, LFM25_ERR_BUFFER_TOO_SMALL, "FP8 quantization input storage too small");
    LFM25_ENSURE(output.len >= numel, LFM25_ERR_BUFFER_TOO_SMALL, "FP8 quantization output storage too small");
    LFM25_ENSURE(std::isfinite(scale) && scale > 0.0f, LFM25_ERR_INVALID_ARGUMENT, "invalid FP8 quantization scale");
    LFM25_ENSURE(input.ptr && output.ptr, LFM25_ERR_NULL_POINTER, "FP8 quantization received a null device pointer");
    return cuda_result(
        lfm25::launch_quantize_bf16_e4m3(static_cast<cudaStream_t>(stream), input.ptr, output.ptr, numel, scale),
        "FP8 quantization launch failed");
}

int32_t lfm25_silu_mul_packed_bf16(void* stream, lfm25_slice packed, lfm25_slice out, size_t rows,
                                   size_t intermediate_size) {
    LFM25_ENSURE(rows > 0 && intermediate_size > 0, LFM25_ERR_INVALID_ARGUMENT,
                 "packed silu_mul requires non-empty dimensions");
    size_t output_elements = 0;
    LFM25_ENSURE(checked_mul(rows, intermediate_size, &output_elements), LFM25_ERR_OVERFLOW,
                 "packed silu_mul output size overflow");
    size_t packed_elements = 0;
    LFM25_ENSURE(checked_mul(output_elements, 2, &packed_elements), LFM25_ERR_OVERFLOW,
                 "packed silu_mul input size overflow");
    LFM25_ENSURE(packed.len >= packed_elements, LFM25_ERR_BUFFER_TOO_SMALL, "packed silu_mul input storage too small");
    LFM25_ENSURE(out.len >= output_elements, LFM25_ERR_BUFFER_TOO_SMALL, "packed silu_mul output storage too small");
    LFM25_ENSURE(packed.ptr && out.ptr, LFM25_ERR_NULL_POINTER, "packed silu_mul received a null device pointer");
    return cuda_result(lfm25::launch_silu_mul_packed_bf16(static_cast<cudaStream_t>(stream), packed.ptr, out.ptr,
                                                          rows, intermediate_size),
                       "packed silu_mul launch failed");
}

int32_t lfm25_silu_mul_packed_bf16_to_e4m3(void* stream, lfm25_slice packed, lfm25_slice out, size_t rows,
                                           size_t intermediate_size, float scale) {
    LFM25_ENSURE(rows > 0 && intermediate_size > 0, LFM25_ERR_INVALID_ARGUMENT,
                 "packed silu_mul FP8 fusion requires non-empty dimensions");
    LFM25_ENSURE(std::isfinite(scale) && scale > 0.0f, LFM25_ERR_INVALID_ARGUMENT,
                 "packed silu_mul FP8 fusion requires a finite positive scale");
    size_t output_elements = 0;
    LFM25_ENSURE(checked_mul(rows, intermediate_size, &output_elements), LFM25_ERR_OVERFLOW,
                 "packed silu_mul FP8 output size overflow");
    size_t packed_elements = 0;
    LFM25_ENSURE(checked_mul(output_elements, 2, &packed_elements), LFM25_ERR_OVERFLOW,
                 "packed silu_mul FP8 input size overflow");
    LFM25_ENSURE(packed.len >= packed_elements, LFM25_ERR_BUFFER_TOO_SMALL,
                 "packed silu_mul FP8 input storage too small");
    LFM25_ENSURE(out.len >= output_elements, LFM25_ERR_BUFFER_TOO_SMALL,
                 "packed silu_mul FP8 output storage too small");
    LFM25_ENSURE(packed.ptr && out.ptr, LFM25_ERR_NULL_POINTER,
                 "packed silu_mul FP8 fusion received a null device pointer");
    return cuda_result(lfm25::launch_silu_mul_packed_bf16_to_e4m3(static_cast<cudaStream_t>(stream), packed.ptr,
                                                                  out.ptr, rows, intermediate_size, scale),
                       "packed silu_mul FP8 fusion launch failed");
}

int32_t lfm25_embedding_bf16(void* stream, lfm25_slice token_ids, lfm25_slice weight, lfm25_slice out,
                             size_t num_tokens, size_t vocab_size, size_t hidden_size) {
    LFM25_ENSURE(num_tokens > 0 && vocab_size > 0 && hidden_size > 0, LFM25_ERR_INVALID_ARGUMENT,
                 "embedding requires non-empty dimensions");
    size_t out_required = 0;
    size_t weight_required = 0;
    LFM25_ENSURE(checked_mul(num_tokens, hidden_size, &out_required) &&
                     checked_mul(vocab_size, hidden_size, &weight_required),
                 LFM25_ERR_OVERFLOW, "embedding size overflow");
    LFM25_ENSURE(token_ids.len >= num_tokens, LFM25_ERR_BUFFER_TOO_SMALL, "embedding token ids too small");
    LFM25_ENSURE(weight.len >= weight_required, LFM25_ERR_BUFFER_TOO_SMALL, "embedding weight storage too small");
    LFM25_ENSURE(out.len >= out_required, LFM25_ERR_BUFFER_TOO_SMALL, "embedding output storage too small");
    LFM25_ENSURE(token_ids.ptr && weight.ptr && out.ptr, LFM25_ERR_NULL_POINTER,
                 "embedding received a null device pointer");
    return cuda_result(lfm25::launch_embedding_bf16(static_cast<cudaStream_t>(stream),
                                                    static_cast<const uint32_t*>(token_ids.ptr), weight.ptr, out.ptr,
                                                    num_tokens, vocab_size, hidden_size),
                       "embedding launch failed");
}

int32_t lfm25_rms_norm_bf16(void* stream, lfm25_slice x, lfm25_slice weight, lfm25_slice out, size_t rows,
                            size_t hidden_size, float eps) {
    LFM25_ENSURE(rows > 0 && hidden_size > 0, LFM25_ERR_INVALID_ARGUMENT, "rms_norm requires non-empty dimensions");
    LFM25_ENSURE(hidden_size % 2 == 0, LFM25_ERR_UNSUPPORTED, "rms_norm requires an even hidden size");
    size_t required = 0;
    LFM25_ENSURE(checked_mul(rows, hidden_size, &required), LFM25_ERR_OVERFLOW, "rms_norm size overflow");
    LFM25_ENSURE(x.len >= required, LFM25_ERR_BUFFER_TOO_SMALL, "rms_norm input storage too small");
    LFM25_ENSURE(out.len >= required, LFM25_ERR_BUFFER_TOO_SMALL, "rms_norm output storage too small");
    LFM25_ENSURE(weight.len >= hidden_size, LFM25_ERR_BUFFER_TOO_SMALL, "rms_norm weight storage too small");
    LFM25_ENSURE(x.ptr && weight.ptr && out.ptr, LFM25_ERR_NULL_POINTER, "rms_norm received a null device pointer");
    return cuda_result(lfm25::launch_rms_norm_bf16(static_cast<cudaStream_t>(stream), x.ptr, weight.ptr, out.ptr, rows,
                                                   hidden_size, eps),
                       "rms_norm launch failed");
}

namespace {

int32_t residual_rms_norm(void* stream, lfm25_slice residual, lfm25_slice update, lfm25_slice weight,
                          lfm25_slice residual_out, lfm25_slice normalized_out, const lfm25_slice* codes_out,
                          size_t rows, size_t hidden_size, float eps, float scale) {
    LFM25_ENSURE(rows > 0 && hidden_size > 0, LFM25_ERR_INVALID_ARGUMENT,
                 "residual rms_norm requires non-empty dimensions");
    LFM25_ENSURE(hidden_size % 2 == 0, LFM25_ERR_UNSUPPORTED, "residual rms_norm requires an even hidden size");
    size_t required = 0;
    LFM25_ENSURE(checked_mul(rows, hidden_size, &required), LFM25_ERR_OVERFLOW, "residual rms_norm size overflow");
    LFM25_ENSURE(residual.len >= required && update.len >= required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "residual rms_norm input storage too small");
    LFM25_ENSURE(residual_out.len >= required && normalized_out.len >= required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "residual rms_norm output storage too small");
    LFM25_ENSURE(weight.len >= hidden_size, LFM25_ERR_BUFFER_TOO_SMALL, "residual rms_norm weight storage too small");
    LFM25_ENSURE(residual.ptr && update.ptr && weight.ptr && residual_out.ptr && normalized_out.ptr,
                 LFM25_ERR_NULL_POINTER, "residual rms_norm received a null device pointer");
    if (codes_out != nullptr) {
        LFM25_ENSURE(codes_out->ptr != nullptr, LFM25_ERR_NULL_POINTER, "residual rms_norm codes output is null");
        LFM25_ENSURE(codes_out->len >= required, LFM25_ERR_BUFFER_TOO_SMALL,
                     "residual rms_norm codes storage too small");
        LFM25_ENSURE(std::isfinite(scale) && scale > 0.0f, LFM25_ERR_INVALID_ARGUMENT,
                     "FP8 quantize scale must be finite and positive");
    }
    return cuda_result(
        lfm25::launch_residual_rms_norm_bf16(static_cast<cudaStream_t>(stream), residual.ptr, update.ptr, weight.ptr,
                                             residual_out.ptr, normalized_out.ptr, rows, hidden_size, eps,
                                             codes_out != nullptr ? codes_out->ptr : nullptr, scale),
        "residual rms_norm launch failed");
}

}  // namespace

int32_t lfm25_residual_rms_norm_bf16(void* stream, lfm25_slice residual, lfm25_slice update, lfm25_slice weight,
                                     lfm25_slice residual_out, lfm25_slice normalized_out, size_t rows,
                                     size_t hidden_size, float eps) {
    return residual_rms_norm(stream, residual, update, weight, residual_out, normalized_out, nullptr, rows,
                             hidden_size, eps, 1.0f);
}

int32_t lfm25_residual_rms_norm_bf16_e4m3(void* stream, lfm25_slice residual, lfm25_slice update, lfm25_slice weight,
                                          lfm25_slice residual_out, lfm25_slice normalized_out, lfm25_slice codes_out,
                                          size_t rows, size_t hidden_size, float eps, float scale) {
    return residual_rms_norm(stream, residual, update, weight, residual_out, normalized_out, &codes_out, rows,
                             hidden_size, eps, scale);
}

int32_t lfm25_short_conv_segmented_lfm2_bf16(void* stream, lfm25_slice projected, lfm25_slice weight,
                                             lfm25_slice states, lfm25_slice segment_offsets,
                                             lfm25_slice segment_slots, lfm25_slice output, size_t num_tokens,
                                             size_t num_segments, size_t hidden_size, size_t num_request_slots) {
    LFM25_ENSURE(num_tokens > 0 && num_segments > 0 && hidden_size > 0 && num_request_slots > 0,
                 LFM25_ERR_INVALID_ARGUMENT, "segmented short conv requires non-empty dimensions");
    size_t projected_required = 0;
    size_t output_required = 0;
    size_t state_required = 0;
    LFM25_ENSURE(checked_mul(num_tokens, hidden_size, &output_required) &&
                     checked_mul(output_required, 3, &projected_required) &&
                     checked_mul(num_request_slots, hidden_size, &state_required) &&
                     checked_mul(state_required, 2, &state_required),
                 LFM25_ERR_OVERFLOW, "segmented short conv size overflow");
    LFM25_ENSURE(projected.len >= projected_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "segmented short conv input storage too small");
    LFM25_ENSURE(output.len >= output_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "segmented short conv output storage too small");
    LFM25_ENSURE(states.len >= state_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "segmented short conv state storage too small");
    LFM25_ENSURE(weight.len >= hidden_size * 3, LFM25_ERR_BUFFER_TOO_SMALL,
                 "segmented short conv weight storage too small");
    LFM25_ENSURE(segment_offsets.len > num_segments && segment_slots.len >= num_segments, LFM25_ERR_BUFFER_TOO_SMALL,
                 "segmented short conv segment metadata too small");
    LFM25_ENSURE(projected.ptr && weight.ptr && states.ptr && segment_offsets.ptr && segment_slots.ptr && output.ptr,
                 LFM25_ERR_NULL_POINTER, "segmented short conv received a null device pointer");
    return cuda_result(
        lfm25::launch_short_conv_segmented(static_cast<cudaStream_t>(stream), projected.ptr, weight.ptr, states.ptr,
                                           static_cast<const uint32_t*>(segment_offsets.ptr),
                                           static_cast<const uint32_t*>(segment_slots.ptr), output.ptr, num_tokens,
                                           num_segments, hidden_size, num_request_slots),
        "segmented short conv launch failed");
}

int32_t lfm25_gather_rows_bf16(void* stream, lfm25_slice input, lfm25_slice row_indices, lfm25_slice output,
                               size_t output_rows, size_t input_rows, size_t columns) {
    LFM25_ENSURE(output_rows > 0 && input_rows > 0 && columns > 0, LFM25_ERR_INVALID_ARGUMENT,
                 "gather requires non-empty dimensions");
    LFM25_ENSURE(columns % 2 == 0, LFM25_ERR_UNSUPPORTED, "gather requires an even number of columns");
    size_t input_required = 0;
    size_t output_required = 0;
    LFM25_ENSURE(checked_mul(input_rows, columns, &input_required) &&
                     checked_mul(output_rows, columns, &output_required),
                 LFM25_ERR_OVERFLOW, "gather size overflow");
    LFM25_ENSURE(input.len >= input_required && output.len >= output_required && row_indices.len >= output_rows,
                 LFM25_ERR_BUFFER_TOO_SMALL, "gather storage too small");
    LFM25_ENSURE(input.ptr && row_indices.ptr && output.ptr, LFM25_ERR_NULL_POINTER,
                 "gather received a null device pointer");
    return cuda_result(lfm25::launch_gather_rows_bf16(static_cast<cudaStream_t>(stream), input.ptr,
                                                      static_cast<const uint32_t*>(row_indices.ptr), output.ptr,
                                                      output_rows, input_rows, columns),
                       "gather launch failed");
}

int32_t lfm25_short_conv_decode_bf16(void* stream, lfm25_slice projected, lfm25_slice weight, lfm25_slice states,
                                     lfm25_slice request_slots, lfm25_slice output, size_t num_tokens,
                                     size_t hidden_size, size_t num_request_slots) {
    LFM25_ENSURE(num_tokens > 0 && hidden_size > 0 && num_request_slots > 0, LFM25_ERR_INVALID_ARGUMENT,
                 "short conv requires non-empty dimensions");
    size_t out_required = 0;
    size_t state_required = 0;
    LFM25_ENSURE(checked_mul(num_tokens, hidden_size, &out_required) &&
                     checked_mul(num_request_slots, hidden_size * 2, &state_required),
                 LFM25_ERR_OVERFLOW, "short conv size overflow");
    LFM25_ENSURE(projected.len >= out_required * 3, LFM25_ERR_BUFFER_TOO_SMALL, "short conv input storage too small");
    LFM25_ENSURE(weight.len >= hidden_size * 3, LFM25_ERR_BUFFER_TOO_SMALL, "short conv weight storage too small");
    LFM25_ENSURE(states.len >= state_required, LFM25_ERR_BUFFER_TOO_SMALL, "short conv state storage too small");
    LFM25_ENSURE(request_slots.len >= num_tokens, LFM25_ERR_BUFFER_TOO_SMALL, "short conv slot storage too small");
    LFM25_ENSURE(output.len >= out_required, LFM25_ERR_BUFFER_TOO_SMALL, "short conv output storage too small");
    LFM25_ENSURE(projected.ptr && weight.ptr && states.ptr && request_slots.ptr && output.ptr, LFM25_ERR_NULL_POINTER,
                 "short conv received a null device pointer");
    return cuda_result(lfm25::launch_short_conv_decode(static_cast<cudaStream_t>(stream), projected.ptr, weight.ptr,
                                                       states.ptr, static_cast<const uint32_t*>(request_slots.ptr),
                                                       output.ptr, num_tokens, hidden_size, num_request_slots),
                       "short conv launch failed");
}

int32_t lfm25_argmax_rows_bf16(void* stream, lfm25_slice logits, lfm25_slice sampled, size_t rows,
                               size_t vocab_size) {
    LFM25_ENSURE(rows > 0 && vocab_size > 0, LFM25_ERR_INVALID_ARGUMENT, "argmax requires non-empty dimensions");
    LFM25_ENSURE(vocab_size <= 65536, LFM25_ERR_UNSUPPORTED, "argmax supports a vocabulary of at most 65536");
    size_t required = 0;
    LFM25_ENSURE(checked_mul(rows, vocab_size, &required), LFM25_ERR_OVERFLOW, "argmax size overflow");
    LFM25_ENSURE(logits.len >= required, LFM25_ERR_BUFFER_TOO_SMALL, "argmax logits storage too small");
    LFM25_ENSURE(sampled.len >= rows, LFM25_ERR_BUFFER_TOO_SMALL, "argmax output storage too small");
    LFM25_ENSURE(logits.ptr && sampled.ptr, LFM25_ERR_NULL_POINTER, "argmax received a null device pointer");
    return cuda_result(lfm25::launch_argmax_rows_bf16(static_cast<cudaStream_t>(stream), logits.ptr,
                                                      static_cast<uint32_t*>(sampled.ptr), rows, vocab_size),
                       "argmax launch failed");
}

int32_t lfm25_decode_step_metadata(void* stream, const lfm25_decode_batch* batch, lfm25_slice sampled,
                                   size_t num_pages, uint32_t advance) {
    LFM25_ENSURE(batch != nullptr, LFM25_ERR_NULL_POINTER, "decode batch is null");
    LFM25_ENSURE(batch->num_tokens > 0, LFM25_ERR_INVALID_ARGUMENT, "GPU batch needs tokens");
    LFM25_ENSURE(batch->block_table_stride > 0 && batch->block_table_rows > 0, LFM25_ERR_INVALID_ARGUMENT,
                 "GPU batch needs block tables");
    LFM25_ENSURE(batch->token_ids && batch->positions && batch->request_slots && batch->physical_slots &&
                     batch->block_tables,
                 LFM25_ERR_NULL_POINTER, "decode batch metadata is incomplete");
    LFM25_ENSURE(!advance || (sampled.ptr != nullptr && sampled.len >= batch->num_tokens), LFM25_ERR_BUFFER_TOO_SMALL,
                 "sampled ids are needed to advance the batch");
    return cuda_result(
        lfm25::launch_decode_metadata(static_cast<cudaStream_t>(stream), batch->token_ids, batch->positions,
                                      batch->request_slots, batch->block_tables,
                                      static_cast<const uint32_t*>(sampled.ptr), batch->physical_slots,
                                      batch->num_tokens, batch->block_table_stride, batch->block_table_rows, num_pages,
                                      advance != 0),
        "step metadata launch failed");
}

int32_t lfm25_linear_fp8_scaled(void* stream, lfm25_slice x, lfm25_slice weight, lfm25_slice out,
                                const lfm25_fp8_linear_config* config) {
    return linear_fp8_dispatch(static_cast<cudaStream_t>(stream), x, weight, out, config, nullptr);
}

int32_t lfm25_blaslt_create(void* stream, lfm25_blaslt** out) {
    LFM25_ENSURE(out != nullptr, LFM25_ERR_NULL_POINTER, "BlasLt output handle is null");
    lfm25_blaslt* handle = new (std::nothrow) lfm25_blaslt();
    LFM25_ENSURE(handle != nullptr, LFM25_ERR_CUDA, "failed to allocate the BlasLt handle");
    handle->stream = static_cast<cudaStream_t>(stream);
    handle->library_workspace_bytes = 32u * 1024u * 1024u;   // src/cuda/blaslt/mod.rs:53-57
    handle->exchange_bytes = lfm25::kUmmaExchangeBytes;
    const size_t total = handle->library_workspace_bytes + handle->exchange_bytes;
    cudaError_t status = cudaMalloc(&handle->allocation, total);
    if (status == cudaSuccess) {
        status = cudaMemsetAsync(handle->allocation, 0, total, handle->stream);
    }
    if (status != cudaSuccess) {
        if (handle->allocation != nullptr) {
            cudaFree(handle->allocation);
        }
        delete handle;
        return cuda_result(status, "failed to allocate the GEMM workspace");
    }
    handle->library_workspace = handle->allocation;
    handle->exchange = static_cast<char*>(handle->allocation) + handle->library_workspace_bytes;
    handle->cublaslt = nullptr;
    *out = handle;
    return LFM25_OK;
}

void lfm25_blaslt_destroy(lfm25_blaslt* handle) {
    if (handle != nullptr) {
        lfm25::cublaslt_bf16_destroy(handle->cublaslt);
        cudaFree(handle->allocation);
        delete handle;
    }
}

int32_t lfm25_blaslt_set_stream(lfm25_blaslt* handle, void* stream) {
    LFM25_ENSURE(handle != nullptr, LFM25_ERR_NULL_POINTER, "BlasLt handle is null");
    handle->stream = static_cast<cudaStream_t>(stream);
    return LFM25_OK;
}

void* lfm25_blaslt_stream(const lfm25_blaslt* handle) { return handle != nullptr ? handle->stream : nullptr; }

size_t lfm25_blaslt_workspace_size(const lfm25_blaslt* handle) {
    return handle != nullptr ? handle->library_workspace_bytes : 0;
}

int32_t lfm25_blaslt_linear_bf16(lfm25_blaslt* handle, lfm25_slice x, lfm25_slice weight, lfm25_slice out, size_t m,
                                 size_t n, size_t k) {
    LFM25_ENSURE(handle != nullptr, LFM25_ERR_NULL_POINTER, "BlasLt handle is null");
    LFM25_ENSURE(m > 0 && n > 0 && k > 0, LFM25_ERR_INVALID_ARGUMENT, "linear does not support empty tensors");
    size_t x_required = 0;
    size_t weight_required = 0;
    size_t out_required = 0;
    LFM25_ENSURE(checked_mul(m, k, &x_required) && checked_mul(n, k, &weight_required) &&
                     checked_mul(m, n, &out_required),
                 LFM25_ERR_OVERFLOW, "linear size overflow");
    LFM25_ENSURE(x.len >= x_required, LFM25_ERR_BUFFER_TOO_SMALL, "linear input storage too small");
    LFM25_ENSURE(weight.len >= weight_required, LFM25_ERR_BUFFER_TOO_SMALL, "linear weight storage too small");
    LFM25_ENSURE(out.len >= out_required, LFM25_ERR_BUFFER_TOO_SMALL, "linear output storage too small");
    LFM25_ENSURE(x.ptr && weight.ptr && out.ptr, LFM25_ERR_NULL_POINTER, "linear received a null device pointer");
    // Which kernel: this library's tcgen05 kernels where they measured ahead of cuBLASLt on the step (the
    // weight-major one up to lfm25_bf16_own_kernel_max_rows() rows where N % 128 == 0 and K % 64 == 0, the
    // batch-major one where bf16_rows_preferred says so), cuBLASLt otherwise, as the reference does.  The option bf16_gemm (or the
    // handle's tuning) = umma | cublaslt | rows forces one.
    const bool aligned = ((reinterpret_cast<uintptr_t>(x.ptr) | reinterpret_cast<uintptr_t>(weight.ptr) |
                           reinterpret_cast<uintptr_t>(out.ptr)) &
                          15) == 0;
    const bool umma_ok = aligned && lfm25::bf16_gemm_umma_supports(m, n, k);
    const bool rows_ok = aligned && lfm25::gemm_rows_supports(m, n, k * 2);
    enum { kLibrary, kUmma, kRows } path = kLibrary;
    if (rows_ok && lfm25::bf16_rows_preferred(m, n, k)) {
        path = kRows;
    } else if (umma_ok && m <= lfm25_bf16_own_kernel_max_rows()) {
        path = kUmma;
    }
    int64_t forced = lfm25::option(lfm25::kOptBf16Gemm);
    if (handle->tuning_kernel == lfm25::kPathUmma) forced = lfm25::kBf16Umma;
    if (handle->tuning_kernel == lfm25::kPathRows) forced = lfm25::kBf16Rows;
    if (handle->tuning_kernel == lfm25::kPathGeneric) forced = lfm25::kBf16CublasLt;
    if (forced == lfm25::kBf16Umma && umma_ok) path = kUmma;
    if (forced == lfm25::kBf16Rows && rows_ok) path = kRows;
    if (forced == lfm25::kBf16CublasLt) path = kLibrary;
    if (path != kLibrary) {
        unsigned int* status_words = device_status_pointer();
        LFM25_ENSURE(status_words != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
        if (path == kRows) {
            return cuda_result(
                lfm25::launch_bf16_gemm_rows(handle->stream, x.ptr, weight.ptr, out.ptr, m, n, k, handle->exchange,
                                             handle->exchange_bytes, status_words, handle->tuning),
                "BF16 linear launch failed");
        }
        return cuda_result(
            lfm25::launch_bf16_gemm_umma(handle->stream, x.ptr, weight.ptr, out.ptr, m, n, k, handle->exchange,
                                         handle->exchange_bytes, status_words),
            "BF16 linear launch failed");
    }
    if (handle->cublaslt == nullptr) {
        handle->cublaslt = lfm25::cublaslt_bf16_create(handle->library_workspace, handle->library_workspace_bytes);
        LFM25_ENSURE(handle->cublaslt != nullptr, LFM25_ERR_CUDA, "cuBLASLt could not be opened");
    }
    return cuda_result(
        lfm25::cublaslt_bf16_linear(handle->cublaslt, handle->stream, x.ptr, weight.ptr, out.ptr, m, n, k),
        "cuBLASLt BF16 matmul failed");
}

int32_t lfm25_blaslt_set_gemm_tuning(lfm25_blaslt* handle, const lfm25_gemm_tuning* tuning) {
    LFM25_ENSURE(handle != nullptr, LFM25_ERR_NULL_POINTER, "BlasLt handle is null");
    if (tuning == nullptr) {
        handle->tuning_kernel = 0;
        handle->tuning = lfm25::GemmRowsTuning();
        return LFM25_OK;
    }
    LFM25_ENSURE(tuning->kernel <= 4, LFM25_ERR_INVALID_ARGUMENT, "unknown GEMM kernel %u", tuning->kernel);
    LFM25_ENSURE(tuning->n_tile % 16 == 0 && tuning->n_tile <= 256, LFM25_ERR_INVALID_ARGUMENT,
                 "n_tile must be a multiple of 16 up to 256, got %u", tuning->n_tile);
    LFM25_ENSURE(tuning->splits <= 8 && tuning->stages <= 12 && tuning->ctas_per_sm <= 2 && tuning->batch_slices <= 8 &&
                     (tuning->issuers == 0 || tuning->issuers == 1 || tuning->issuers == 2 || tuning->issuers == 4),
                 LFM25_ERR_INVALID_ARGUMENT, "GEMM tuning value out of range");
    handle->tuning_kernel = tuning->kernel;
    handle->tuning.n_tile = tuning->n_tile;
    handle->tuning.splits = tuning->splits;
    handle->tuning.stages = tuning->stages;
    handle->tuning.issuers = tuning->issuers;
    handle->tuning.slices = tuning->batch_slices;
    handle->tuning.ctas_per_sm = tuning->ctas_per_sm;
    handle->tuning.smem_bytes = tuning->shared_memory_bytes;
    return LFM25_OK;
}

int32_t lfm25_blaslt_gemm_plan(const lfm25_blaslt* handle, size_t m, size_t n, size_t k_bytes, uint32_t gated,
                               uint32_t out[8]) {
    LFM25_ENSURE(handle != nullptr && out != nullptr, LFM25_ERR_NULL_POINTER, "GEMM plan query received a null argument");
    LFM25_ENSURE(lfm25::gemm_rows_supports(m, gated != 0 ? 2 * n : n, k_bytes), LFM25_ERR_UNSUPPORTED,
                 "shape outside the batch-major kernel");
    const lfm25::GemmRowsPlan plan =
        lfm25::gemm_rows_plan(m, n, k_bytes, gated != 0, handle->exchange_bytes, handle->tuning);
    LFM25_ENSURE(plan.valid, LFM25_ERR_UNSUPPORTED, "no valid plan for this shape and tuning");
    out[0] = plan.n_tile;
    out[1] = plan.splits;
    out[2] = plan.tiles;
    out[3] = plan.stages;
    out[4] = plan.issuers;
    out[5] = plan.ctas_per_sm;
    out[6] = plan.smem_bytes;
    out[7] = plan.slices;
    return LFM25_OK;
}

int32_t lfm25_blaslt_linear_bf16_silu_mul(lfm25_blaslt* handle, lfm25_slice x, lfm25_slice weight,
                                          lfm25_slice activation, size_t m, size_t n, size_t k,
                                          float activation_scale, uint32_t e4m3_output) {
    LFM25_ENSURE(handle != nullptr, LFM25_ERR_NULL_POINTER, "BlasLt handle is null");
    LFM25_ENSURE(m > 0 && n > 0 && k > 0, LFM25_ERR_INVALID_ARGUMENT, "gated BF16 linear is empty");
    LFM25_ENSURE(n % 2 == 0, LFM25_ERR_INVALID_ARGUMENT, "packed Gate/Up width must be even, got %zu", n);
    LFM25_ENSURE(std::isfinite(activation_scale) && activation_scale > 0.0f, LFM25_ERR_INVALID_ARGUMENT,
                 "activation scale must be finite and positive");
    size_t x_required = 0;
    size_t weight_required = 0;
    size_t out_required = 0;
    LFM25_ENSURE(checked_mul(m, k, &x_required) && checked_mul(n, k, &weight_required) &&
                     checked_mul(m, n / 2, &out_required),
                 LFM25_ERR_OVERFLOW, "gated BF16 linear size overflow");
    LFM25_ENSURE(x.len >= x_required, LFM25_ERR_BUFFER_TOO_SMALL, "gated BF16 linear input storage too small");
    LFM25_ENSURE(weight.len >= weight_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "gated BF16 linear weight storage too small");
    LFM25_ENSURE(activation.len >= out_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "gated BF16 linear output storage too small");
    LFM25_ENSURE(x.ptr && weight.ptr && activation.ptr, LFM25_ERR_NULL_POINTER,
                 "gated BF16 linear received a null device pointer");
    const bool aligned = ((reinterpret_cast<uintptr_t>(x.ptr) | reinterpret_cast<uintptr_t>(weight.ptr) |
                           reinterpret_cast<uintptr_t>(activation.ptr)) &
                          15) == 0;
    LFM25_ENSURE(aligned && (n / 2) % 8 == 0 && lfm25::gemm_rows_supports(m, n, k * 2), LFM25_ERR_UNSUPPORTED,
                 "gated BF16 linear: shape or alignment outside the tensor-core kernel");
    unsigned int* status_words = device_status_pointer();
    LFM25_ENSURE(status_words != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
    return cuda_result(
        lfm25::launch_bf16_gemm_rows_gated(handle->stream, x.ptr, weight.ptr, activation.ptr, m, n / 2, k,
                                           activation_scale, e4m3_output != 0, status_words, handle->tuning),
        "gated BF16 linear launch failed");
}

int32_t lfm25_blaslt_linear_fp8_scaled(lfm25_blaslt* handle, lfm25_slice x, lfm25_slice weight, lfm25_slice out,
                                       const lfm25_fp8_linear_config* config) {
    LFM25_ENSURE(handle != nullptr, LFM25_ERR_NULL_POINTER, "BlasLt handle is null");
    return linear_fp8_dispatch(handle->stream, x, weight, out, config, handle);
}

int32_t lfm25_blaslt_linear_fp8_silu_mul(lfm25_blaslt* handle, lfm25_slice x, lfm25_slice weight,
                                         lfm25_slice activation, const lfm25_fp8_linear_config* config,
                                         float activation_scale, uint32_t e4m3_output) {
    LFM25_ENSURE(handle != nullptr, LFM25_ERR_NULL_POINTER, "BlasLt handle is null");
    LFM25_ENSURE(config != nullptr, LFM25_ERR_NULL_POINTER, "FP8 linear config is null");
    const size_t m = config->m;
    const size_t n = config->n;
    const size_t k = config->k;
    LFM25_ENSURE(m > 0 && n > 0 && k > 0, LFM25_ERR_INVALID_ARGUMENT, "gated FP8 linear is empty");
    LFM25_ENSURE(n % 2 == 0, LFM25_ERR_INVALID_ARGUMENT, "packed Gate/Up width must be even, got %zu", n);
    LFM25_ENSURE(config->scale_mode == LFM25_FP8_SCALE_TENSORWIDE, LFM25_ERR_UNSUPPORTED,
                 "Block32 (MXFP8) scaling is not built; use the tensor-wide mode");
    LFM25_ENSURE(std::isfinite(config->output_scale) && config->output_scale > 0.0f, LFM25_ERR_INVALID_ARGUMENT,
                 "FP8 output scale must be finite and positive");
    LFM25_ENSURE(std::isfinite(activation_scale) && activation_scale > 0.0f, LFM25_ERR_INVALID_ARGUMENT,
                 "activation scale must be finite and positive");
    size_t x_required = 0;
    size_t weight_required = 0;
    size_t out_required = 0;
    LFM25_ENSURE(checked_mul(m, k, &x_required), LFM25_ERR_OVERFLOW, "gated FP8 linear input size overflow");
    LFM25_ENSURE(checked_mul(n, k, &weight_required), LFM25_ERR_OVERFLOW, "gated FP8 linear weight size overflow");
    LFM25_ENSURE(checked_mul(m, n / 2, &out_required), LFM25_ERR_OVERFLOW, "gated FP8 linear output size overflow");
    LFM25_ENSURE(x.len >= x_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "gated FP8 linear input storage too small: required=%zu, actual=%zu", x_required, x.len);
    LFM25_ENSURE(weight.len >= weight_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "gated FP8 linear weight storage too small: required=%zu, actual=%zu", weight_required, weight.len);
    LFM25_ENSURE(activation.len >= out_required, LFM25_ERR_BUFFER_TOO_SMALL,
                 "gated FP8 linear output storage too small: required=%zu, actual=%zu", out_required,
                 activation.len);
    LFM25_ENSURE(x.ptr && weight.ptr && activation.ptr, LFM25_ERR_NULL_POINTER,
                 "gated FP8 linear received a null device pointer");
    const bool aligned = ((reinterpret_cast<uintptr_t>(x.ptr) | reinterpret_cast<uintptr_t>(weight.ptr) |
                           reinterpret_cast<uintptr_t>(activation.ptr)) &
                          15) == 0;
    const bool umma_ok = aligned && lfm25::fp8_gemm_umma_gated_supports(m, n, k);
    const bool rows_ok = aligned && (n / 2) % 8 == 0 && lfm25::gemm_rows_supports(m, n, k);
    LFM25_ENSURE(umma_ok || rows_ok, LFM25_ERR_UNSUPPORTED,
                 "gated FP8 linear: shape or alignment outside the tensor-core kernels");
    unsigned int* status_words = device_status_pointer();
    LFM25_ENSURE(status_words != nullptr, LFM25_ERR_CUDA, "device status words are not reachable");
    bool use_rows = rows_ok && (!umma_ok || lfm25::fp8_gated_rows_preferred(m, n / 2, k));
    const int64_t forced = handle->tuning_kernel != 0 ? handle->tuning_kernel : lfm25::option(lfm25::kOptFp8GemmPath);
    if (forced == lfm25::kPathRows && rows_ok) use_rows = true;
    if (forced == lfm25::kPathUmma && umma_ok) use_rows = false;
    if (use_rows) {
        return cuda_result(
            lfm25::launch_fp8_gemm_rows_gated(handle->stream, x.ptr, weight.ptr, activation.ptr, m, n / 2, k,
                                              config->output_scale, activation_scale, e4m3_output != 0, status_words,
                                              handle->tuning),
            "gated FP8 linear launch failed");
    }
    return cuda_result(lfm25::launch_fp8_gemm_umma_gated(handle->stream, x.ptr, weight.ptr, activation.ptr, m, n, k,
                                                         config->output_scale, activation_scale, e4m3_output != 0,
                                                         status_words),
                       "gated FP8 linear launch failed");
}

}  // extern "C"
