/*
 * lfm25_b200 -- C ABI of the B200-native decode path of the LFM2.5-1.2B runtime.
 *
 * This is the drop-in boundary: one entry point per launch method of the reference's
 * `src/cuda/kernels/*.rs` wrappers and `src/cuda/blaslt` calls that lie on the decode path.
 * Each `*_launch` struct has the fields of the Rust `XLaunch<'_>` struct it replaces, in the
 * same order, with every `&CudaSlice<T>` turned into (device pointer, element count).
 * A Rust host binds these with `#[repr(C)]` structs and an `extern "C"` block.
 *
 * Conventions (kept from the reference):
 *  - the caller owns every buffer; no entry point allocates, frees or synchronises;
 *  - every entry point validates on the host first and launches nothing on error
 *    (the reference's `ensure!` checks); the return value is 0 or a negative LFM25_ERR_*,
 *    and lfm25_last_error() returns the message of the calling thread's last failure;
 *  - work is enqueued on `stream` (a CUstream / cudaStream_t passed as void*);
 *  - indices that are invalid on the device (negative slot, page >= num_pages, request slot
 *    >= rows, position beyond the table) make the affected token a silent no-op;
 *  - bf16 is the raw 16-bit pattern, E4M3 codes are bytes, positions / slots / tables are
 *    uint32, physical slots are int64, sizes are size_t.
 *
 * Citations are file:line inside the reference project.
 */
#ifndef LFM25_B200_H
#define LFM25_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LFM25_OK 0
#define LFM25_ERR_INVALID_ARGUMENT (-1) /* a size, count or scalar fails an `ensure!` of the reference */
#define LFM25_ERR_BUFFER_TOO_SMALL (-2) /* a slice holds fewer elements than the launch needs */
#define LFM25_ERR_UNSUPPORTED (-3)      /* page size other than 16, or a scale mode that is not built */
#define LFM25_ERR_OVERFLOW (-4)         /* a size computation overflowed */
#define LFM25_ERR_CUDA (-5)             /* the CUDA runtime refused the launch */
#define LFM25_ERR_NULL_POINTER (-6)

/* `&CudaSlice<T>`: device pointer + number of elements of T it holds. */
typedef struct lfm25_slice {
    void* ptr;
    size_t len;
} lfm25_slice;

/* Message of the last failing call made by this thread ("" if none).  Never NULL. */
const char* lfm25_last_error(void);

/* Library version string, e.g. "lfm25_b200 0.1 sm_100a". */
const char* lfm25_version(void);

/*
 * Reads and clears the device status words written by kernels whose bounded waits ran out:
 * out[0] = number of waits that gave up since the last read, out[1] = tag of the kernel,
 * out[2] = detail (CTA / stage), out[3] = reserved.  Synchronises `stream`.
 * No counterpart in the reference (its kernels have no waits on asynchronous copies).
 */
int32_t lfm25_device_status(void* stream, uint32_t out[4]);

/* ------------------------------------------------------------------------------------------
 * Paged KV append
 * ------------------------------------------------------------------------------------------ */

/* Replaces KvCacheWriteLaunch + KvCacheKernels::launch_write_lfm2_bf16
 * (src/cuda/kernels/kv_cache.rs:13-22, :48-106; kernel kernels/kv_cache.cu:30-120). */
typedef struct lfm25_kv_cache_write_launch {
    size_t page_size;         /* 16 (32 is rejected with LFM25_ERR_UNSUPPORTED) */
    lfm25_slice key;          /* bf16 [num_tokens, 8, 64] */
    lfm25_slice value;        /* bf16 [num_tokens, 8, 64] */
    lfm25_slice key_cache;    /* bf16 [num_pages, 8, page_size, 64], written */
    lfm25_slice value_cache;  /* bf16 [num_pages, 8, page_size, 64], written */
    lfm25_slice slot_mapping; /* i64 [num_tokens]; < 0 or page >= num_pages skips the token */
    size_t num_tokens;
    size_t num_pages;
} lfm25_kv_cache_write_launch;
int32_t lfm25_kv_cache_write_lfm2_bf16(void* stream, const lfm25_kv_cache_write_launch* launch);

/* Replaces QkPostprocessLaunch + QkPostprocessKernels::launch_decode
 * (src/cuda/kernels/qk_postprocess.rs:13-28, :65-156; kernel kernels/qk_postprocess.cu:44-151):
 * Q RMSNorm + RoPE in place, K RMSNorm + RoPE into the paged cache, V copied. */
typedef struct lfm25_qk_postprocess_launch {
    size_t page_size;
    lfm25_slice query;        /* bf16 [num_tokens, 32, 64], rewritten in place */
    lfm25_slice key;          /* bf16 [num_tokens, 8, 64] */
    lfm25_slice value;        /* bf16 [num_tokens, 8, 64] */
    lfm25_slice query_norm;   /* bf16 [64] */
    lfm25_slice key_norm;     /* bf16 [64] */
    lfm25_slice inv_freq;     /* f32 [32] */
    lfm25_slice position_ids; /* u32 [num_tokens] */
    lfm25_slice slot_mapping; /* i64 [num_tokens] */
    lfm25_slice key_cache;
    lfm25_slice value_cache;
    size_t num_tokens;
    size_t num_pages;
    float eps;
} lfm25_qk_postprocess_launch;
int32_t lfm25_qk_norm_rope_kv_write_decode(void* stream, const lfm25_qk_postprocess_launch* launch);

/* ------------------------------------------------------------------------------------------
 * Paged GQA decode attention
 * ------------------------------------------------------------------------------------------ */

/* Replaces PagedAttentionLaunch + AsyncAttentionFastKernels::launch_lfm2_bf16
 * (src/cuda/kernels/attention.rs PagedAttentionLaunch; attention_async_fast.rs:139-213;
 * kernel kernels/attention_async_fast.cu:423-459): one sequence, block-table row 0. */
typedef struct lfm25_paged_attention_launch {
    size_t page_size;
    lfm25_slice query;        /* bf16 [num_tokens, 32, 64] */
    lfm25_slice key_cache;
    lfm25_slice value_cache;
    lfm25_slice block_table;  /* u32 [block_table.len] logical -> physical page */
    lfm25_slice position_ids; /* u32 [num_tokens], index of the newest key of each token */
    lfm25_slice output;       /* bf16 [num_tokens, 32, 64], written */
    size_t num_tokens;
    size_t num_pages;
} lfm25_paged_attention_launch;
int32_t lfm25_paged_attention_fast_lfm2_bf16(void* stream, const lfm25_paged_attention_launch* launch);

/* Replaces FastRaggedAttentionLaunch + launch_ragged_lfm2_bf16
 * (src/cuda/kernels/attention_async_fast.rs:14-26, :284-341; kernel
 * kernels/attention_async_fast.cu:72-205,461-501). */
typedef struct lfm25_fast_ragged_attention_launch {
    size_t page_size;
    lfm25_slice query;         /* bf16 [num_tokens, 32, 64] */
    lfm25_slice key_cache;
    lfm25_slice value_cache;
    lfm25_slice block_tables;  /* u32 [rows, block_table_stride], rows = len / stride */
    lfm25_slice request_slots; /* u32 [num_tokens] row of each token */
    lfm25_slice position_ids;  /* u32 [num_tokens] */
    lfm25_slice output;        /* bf16 [num_tokens, 32, 64], written */
    size_t num_tokens;
    size_t num_pages;
    size_t block_table_stride;
} lfm25_fast_ragged_attention_launch;
int32_t lfm25_paged_ragged_attention_fast_lfm2_bf16(void* stream, const lfm25_fast_ragged_attention_launch* launch);

/* Replaces SplitKRaggedAttentionLaunch + launch_splitk_ragged_lfm2_bf16
 * (src/cuda/kernels/attention_async_fast.rs:28-42, :343-437; kernels
 * kernels/attention_async_fast.cu:211-358 and :362-419).  `partials` keeps the reference's
 * record layout f32 [num_tokens, 32, num_splits, 66] = (max, denominator, acc[64]). */
typedef struct lfm25_splitk_ragged_attention_launch {
    size_t page_size;
    lfm25_slice query;
    lfm25_slice key_cache;
    lfm25_slice value_cache;
    lfm25_slice block_tables;
    lfm25_slice request_slots;
    lfm25_slice position_ids;
    lfm25_slice partials;      /* f32, >= num_tokens * 32 * num_splits * 66, written */
    lfm25_slice output;
    size_t num_tokens;
    size_t num_pages;
    size_t block_table_stride;
    size_t num_splits;         /* 2..=8 */
} lfm25_splitk_ragged_attention_launch;
int32_t lfm25_paged_ragged_attention_splitk_lfm2_bf16(void* stream, const lfm25_splitk_ragged_attention_launch* launch);

/* Split-K decode attention for hosts that must not allocate device memory after start-up (an engine that
 * gave all free memory to its KV pool, a loop that cannot afford cudaMalloc's device synchronisation, an
 * embedder whose own allocator is the only one allowed).  Same inputs, outputs and results as
 * lfm25_paged_ragged_attention_splitk_lfm2_bf16, but the split records go to an array compiled into the
 * library (8,650,752 bytes per device, held until exit) instead of a caller workspace.  Limits: at most 128
 * tokens per call (more is rejected with LFM25_ERR_INVALID_ARGUMENT), 2..=8 splits.  The first call on a
 * device looks up the array's device address; make that call before any stream capture begins.  All calls
 * share the one array and it keeps whatever the last call wrote, so calls must not overlap on the GPU: keep
 * them ordered on one stream.  Nothing needs clearing between calls: each call writes every record it later
 * reads.  This entry point has no counterpart in the reference, whose split-K path always takes a
 * caller-allocated `partials` tensor. */
int32_t lfm25_paged_ragged_attention_splitk_static_lfm2_bf16(void* stream,
                                                             const lfm25_fast_ragged_attention_launch* launch,
                                                             size_t num_splits);

/* Replaces splitk_workspace_elements (src/ops/attention_async_fast.rs:24-30):
 * maximum_tokens * 32 * 8 * 66 f32 elements; 0 on overflow. */
size_t lfm25_splitk_workspace_elements(size_t maximum_tokens);

/* Replaces splitk_decode_splits (src/ops/splitk_policy.rs:15-78): number of KV-axis splits
 * for a decode batch (1 = use the unsplit kernel).  Re-derived for B200: the reference's table
 * was measured on a 36-SM laptop part. */
size_t lfm25_splitk_decode_splits(size_t num_tokens, size_t maximum_context_tokens, size_t page_size);

/* ------------------------------------------------------------------------------------------
 * FP8 (E4M3) producers
 * ------------------------------------------------------------------------------------------ */

/* Replaces Fp8QuantizeKernels::launch_bf16_e4m3 (src/cuda/kernels/fp8_quantize.rs:31-66;
 * kernel kernels/fp8_quantize.cu:9-45): output[i] = e4m3_rn_satfinite(float(input[i]) * scale). */
int32_t lfm25_quantize_bf16_e4m3(void* stream, lfm25_slice input, lfm25_slice output, size_t numel, float scale);

/* Replaces SiluMulKernels::launch_packed_bf16 (src/cuda/kernels/silu_mul.rs:40-76;
 * kernel kernels/silu_mul.cu:13-61): out[r, c] = bf16(silu(packed[r, c]) * packed[r, I + c]). */
int32_t lfm25_silu_mul_packed_bf16(void* stream, lfm25_slice packed, lfm25_slice out, size_t rows,
                                   size_t intermediate_size);

/* Replaces SiluMulKernels::launch_packed_bf16_to_e4m3 (src/cuda/kernels/silu_mul.rs:78-125;
 * kernel kernels/silu_mul.cu:68-133). */
int32_t lfm25_silu_mul_packed_bf16_to_e4m3(void* stream, lfm25_slice packed, lfm25_slice out, size_t rows,
                                           size_t intermediate_size, float scale);

/* ------------------------------------------------------------------------------------------
 * FP8 (E4M3) linear
 * ------------------------------------------------------------------------------------------ */

#define LFM25_FP8_SCALE_TENSORWIDE 0 /* Fp8ScaleMode::Tensorwide */
#define LFM25_FP8_SCALE_BLOCK32 1    /* Fp8ScaleMode::Block32 (research-only in the reference): not built */

/* Replaces Fp8LinearConfig (src/cuda/blaslt/mod.rs:21-28). */
typedef struct lfm25_fp8_linear_config {
    size_t m;
    size_t n;
    size_t k;
    uint32_t scale_mode;
    float output_scale; /* d_x * d_w, applied to the fp32 sum before rounding to bf16 */
} lfm25_fp8_linear_config;

/* Replaces BlasLt::linear_fp8_scaled (src/cuda/blaslt/mod.rs:212-298, cuBLASLt descriptor
 * src/cuda/blaslt/fp8.rs:312-353): out[M,N] = bf16(output_scale * x[M,K] * weight[N,K]^T), E4M3 codes in,
 * fp32 accumulation.  No plan cache and no workspace are needed. */
int32_t lfm25_linear_fp8_scaled(void* stream, lfm25_slice x, lfm25_slice weight, lfm25_slice out,
                                const lfm25_fp8_linear_config* config);

#ifdef __cplusplus
}
#endif

#endif /* LFM25_B200_H */
