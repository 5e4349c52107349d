/*
 * lfm25_b200 -- C ABI of the B200-native decode path of the LFM2.5-1.2B runtime.
 *
 * This is the drop-in boundary: one entry point per launch method of the reference's
 * `src/cuda/kernels/` wrappers (one .rs file per kernel family) and `src/cuda/blaslt` calls that lie on the decode path.
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

/*
 * Process-wide switches, in the place of the reference's environment-driven feature toggles
 * (LFM25_* variables read in src/model/lfm2_base.rs and src/engine/serving/radix_owner.rs).  Each switch has a
 * default, may be preset by the environment variable LFM25_<NAME> (read once) and changed at run time here; a
 * change applies to launches issued afterwards and is not recorded in CUDA graphs that are already captured.
 *   pdl, fused_silu, kv_evict_first, weights_evict_first, engine_graph 0 | 1 (default 1)
 *   splitk_cluster_merge   0 | 1 (default 1): the decode executor merges the KV splits of a token inside the attention
 *                          kernel (a cluster per token and KV head) where that measured faster, else never
 *   fused_append           0 two launches | 1 one kernel | 2 auto (default): how the decode executor runs an
 *                          attention layer -- QK-norm + RoPE + append as a kernel of their own before the attention
 *                          kernel, or inside it; auto asks lfm25_decode_one_kernel_preferred()
 *   fused_silu_bf16        0 | 1 (default 0): SiLU * Up in the epilogue of a BF16 Gate/Up linear as well
 *   hybrid_attention       0 auto | 1 umma | 2 mma
 *   fp8_gemm_path          0 auto | 1 stream | 2 umma (weight-major) | 3 generic | 4 rows (batch-major)
 *   bf16_gemm              0 auto | 1 umma (weight-major) | 2 cublaslt | 3 rows (batch-major)
 *   decode_splits          0 auto | 1..8
 *   wait_limit_ns          limit of every bounded device-side wait, default 1000000000
 *   wait_selftest_drop     0 | 1: a self-test of the bounded waits -- kernels with a TMA ring arm one barrier
 *                          whose copy they never issue, so that the wait runs out after wait_limit_ns; the kernel
 *                          then records the event (lfm25_device_status), stores nothing and returns normally
 * Unknown names and values out of range are refused with LFM25_ERR_INVALID_ARGUMENT.
 */
int32_t lfm25_set_option(const char* name, int64_t value);
int32_t lfm25_get_option(const char* name, int64_t* value);

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
    /* Extension (no counterpart in the reference's launch struct): optional u32 [num_tokens] permutation of the
     * tokens.  CTAs are handed out in this order; listing the longest contexts first (lfm25_context_order_desc)
     * keeps the tail of the grid short on ragged batches.  Results do not depend on it.  ptr NULL = as given. */
    lfm25_slice token_order;
} lfm25_fast_ragged_attention_launch;
int32_t lfm25_paged_ragged_attention_fast_lfm2_bf16(void* stream, const lfm25_fast_ragged_attention_launch* launch);
/* order[r] = index of the token with the r-th largest position (ties: lower index first), for the `token_order`
 * field of the decode attention launches.  At most 2048 tokens.  No counterpart in the reference, whose kernels take
 * the batch in the order given. */
int32_t lfm25_context_order_desc(void* stream, lfm25_slice position_ids, size_t num_tokens, lfm25_slice order);

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
    lfm25_slice partials;      /* f32, >= num_tokens * 32 * num_splits * 66, written; or {NULL, 0}: no records are
                                * written, the splits of a token run as one thread-block cluster and merge through
                                * distributed shared memory (num_splits 2, 4 or 8; same output bits) */
    lfm25_slice output;
    size_t num_tokens;
    size_t num_pages;
    size_t block_table_stride;
    size_t num_splits;         /* 2..=8 */
    lfm25_slice token_order;   /* optional, as in lfm25_fast_ragged_attention_launch */
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
 * combines into an output row.  A token that has no result (request slot outside the block tables, position
 * outside its row, unassigned page, a wait that ran out -- the last one also shows in lfm25_device_status) keeps
 * the output row the caller passed in, in this entry point and in the one with a caller workspace alike: its
 * records carry a "no result" mark, so values of an earlier call never reach the output.  If a call fails with
 * LFM25_ERR_CUDA the cached device address is dropped and looked up again by the next call (a host that reset
 * the device gets a valid address again).  This entry point has no counterpart in the reference, whose split-K
 * path always takes a caller-allocated `partials` tensor. */
int32_t lfm25_paged_ragged_attention_splitk_static_lfm2_bf16(void* stream,
                                                             const lfm25_fast_ragged_attention_launch* launch,
                                                             size_t num_splits);

/* Replaces FusedAttentionCommon + FusedRaggedDecodeLaunch + FusedAttentionKernels::launch_ragged_decode
 * (src/cuda/kernels/attention_fused.rs:13-41, :226-323; kernel kernels/attention_fused.cu:89-348): the one-kernel
 * decode.  Raw Q/K/V projections in; Q RMSNorm + RoPE in registers (query_raw is not modified), K RMSNorm + RoPE and V
 * written into the paged cache at slot_mapping[t], attention over the updated context, output written.  A token whose
 * slot is negative or disagrees with block_tables[row][position / 16] and position % 16 is a silent no-op.
 * Beyond the reference: with num_splits in 2..=8 and a partials workspace the same fused kernel runs split over the
 * KV axis (num_splits == 1 or 0: one kernel, partials unused).  Results are bit-identical to
 * lfm25_qk_norm_rope_kv_write_decode followed by the unfused attention entry points. */
typedef struct lfm25_fused_ragged_decode_launch {
    size_t page_size;
    lfm25_slice query_raw;     /* bf16 [num_tokens, 32, 64] */
    lfm25_slice key_raw;       /* bf16 [num_tokens, 8, 64] */
    lfm25_slice value_raw;     /* bf16 [num_tokens, 8, 64] */
    lfm25_slice query_norm;    /* bf16 [64] */
    lfm25_slice key_norm;      /* bf16 [64] */
    lfm25_slice inv_freq;      /* f32 [32] */
    lfm25_slice key_cache;     /* written */
    lfm25_slice value_cache;   /* written */
    lfm25_slice position_ids;  /* u32 [num_tokens] */
    lfm25_slice slot_mapping;  /* i64 [num_tokens] */
    lfm25_slice output;        /* bf16 [num_tokens, 32, 64], written */
    size_t num_tokens;
    size_t num_pages;
    float eps;
    lfm25_slice block_tables;  /* u32 [rows, block_table_stride] */
    lfm25_slice request_slots; /* u32 [num_tokens] */
    size_t block_table_stride;
    lfm25_slice partials;      /* f32 [num_tokens, 32, num_splits, 66] when num_splits > 1 */
    size_t num_splits;
    /* Extension (no counterpart in the reference's launch struct): elements between consecutive tokens of
     * query_raw and of key_raw / value_raw, for projections that one packed GEMM wrote side by side
     * ([num_tokens, 3072] = q | k | v).  0 = dense (2048 and 512). */
    size_t query_token_stride;
    size_t kv_token_stride;
    lfm25_slice token_order;   /* optional, as in lfm25_fast_ragged_attention_launch */
} lfm25_fused_ragged_decode_launch;
int32_t lfm25_fused_ragged_paged_attention_decode_lfm2_bf16(void* stream,
                                                            const lfm25_fused_ragged_decode_launch* launch);

/* Replaces AttentionKernels::launch_hybrid_ragged_lfm2_bf16 with HybridAttentionLaunch
 * (src/cuda/kernels/attention.rs:41-57,131-226; kernel kernels/attention.cu:389-585): attention of a step that
 * mixes prefill chunks and decode tokens.  Token t of the segment [segment_offsets[s], segment_offsets[s+1]) that
 * contains it, at offset o and position p, attends to the p - o tokens of its sequence already in the paged cache
 * (through block_tables[request_slots[t]]) and to the step's own tokens segment_begin..t in current_key /
 * current_value.  A token with p < o, or whose key range meets a block-table entry >= num_pages, is left untouched;
 * the tokens of a segment must sit at consecutive positions of one request slot (GpuBatch::update_segments,
 * src/scheduler/batch.rs:142-215): a token that does not continue its 16-token tile is left untouched as well.
 * Extensions: current_key.ptr == NULL reads every key up to each token's position from the cache (the step's K/V
 * were appended first); query_token_stride / kv_token_stride (elements, 0 = dense 2048 / 512) accept projections
 * that one packed GEMM wrote side by side. */
typedef struct lfm25_hybrid_attention_launch {
    size_t page_size;
    lfm25_slice query;            /* bf16 [num_tokens, 32, 64] */
    lfm25_slice current_key;      /* bf16 [num_tokens, 8, 64] (16-byte aligned) or ptr NULL */
    lfm25_slice current_value;
    lfm25_slice key_cache;        /* bf16 [num_pages, 8, 16, 64] */
    lfm25_slice value_cache;
    lfm25_slice block_tables;     /* u32 [rows, block_table_stride] */
    lfm25_slice request_slots;    /* u32 [num_tokens] */
    lfm25_slice position_ids;     /* u32 [num_tokens] */
    lfm25_slice segment_offsets;  /* u32 [num_segments + 1] */
    lfm25_slice output;           /* bf16 [num_tokens, 32, 64], written */
    size_t num_tokens;
    size_t num_pages;
    size_t block_table_stride;
    size_t num_segments;
    size_t query_token_stride;
    size_t kv_token_stride;
} lfm25_hybrid_attention_launch;
int32_t lfm25_hybrid_ragged_attention_lfm2_bf16(void* stream, const lfm25_hybrid_attention_launch* launch);

/* Replaces splitk_workspace_elements (src/ops/attention_async_fast.rs:24-30):
 * maximum_tokens * 32 * 8 * 66 f32 elements; 0 on overflow. */
size_t lfm25_splitk_workspace_elements(size_t maximum_tokens);

/* Replaces splitk_decode_splits (src/ops/splitk_policy.rs:15-78): number of KV-axis splits
 * for a decode batch (1 = use the unsplit kernel).  Re-derived for B200: the reference's table
 * was measured on a 36-SM laptop part. */
size_t lfm25_splitk_decode_splits(size_t num_tokens, size_t maximum_context_tokens, size_t page_size);

/* Replaces should_use_mok_one_kernel (src/ops/mok_dispatch.rs:7-27): 1 when a decode step of `batch_size`
 * sequences with at most `context_tokens` cached tokens should run lfm25_fused_ragged_paged_attention_decode_lfm2_bf16
 * (one kernel), 0 when it should run lfm25_qk_norm_rope_kv_write_decode followed by the attention kernel.  The
 * thresholds are measured on a B200 (the table is in the definition); with the `pdl` switch off the reference's own
 * thresholds apply.  Page sizes other than 16 answer 0. */
int32_t lfm25_decode_one_kernel_preferred(size_t page_size, size_t context_tokens, size_t batch_size);

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
 * fp32 accumulation.  No plan cache and no workspace are needed.  Kernel choice without a handle: M <= 8
 * weight-streaming mma.sync kernel, 9..256 tcgen05/TMEM kernel, other shapes a generic kernel; the switch
 * fp8_gemm_path (lfm25_set_option) overrides it for measurements. */
int32_t lfm25_linear_fp8_scaled(void* stream, lfm25_slice x, lfm25_slice weight, lfm25_slice out,
                                const lfm25_fp8_linear_config* config);

/* Replaces the `BlasLt` object (src/cuda/blaslt/mod.rs:30-70): bound to one stream, owns the 32 MiB device
 * workspace that cuBLASLt uses for the BF16 linears and the exchange buffer through which the tcgen05 kernels
 * combine the partial sums of a split K axis, both allocated once at creation.  A handle serves ONE stream at a
 * time: two launches through the same handle must not overlap on the GPU (different streams, or graphs replayed
 * concurrently), because they would share the workspace and the exchange buffer; give every stream its own handle.
 * If a bounded wait runs out in one CTA of a split-K cluster, the whole cluster stores nothing (the CTA publishes
 * the event to its partners before the cluster barrier) and lfm25_device_status reports it. */
typedef struct lfm25_blaslt lfm25_blaslt;
int32_t lfm25_blaslt_create(void* stream, lfm25_blaslt** out);
void lfm25_blaslt_destroy(lfm25_blaslt* handle);
/* Rebinds the handle to another stream (the reference binds at construction only; work already enqueued on the
 * old stream that uses the workspace must have been ordered before new work by the caller). */
int32_t lfm25_blaslt_set_stream(lfm25_blaslt* handle, void* stream);
size_t lfm25_blaslt_workspace_size(const lfm25_blaslt* handle);
/* The stream the handle is bound to. */
void* lfm25_blaslt_stream(const lfm25_blaslt* handle); /* BlasLt::workspace_size */
int32_t lfm25_blaslt_linear_fp8_scaled(lfm25_blaslt* handle, lfm25_slice x, lfm25_slice weight, lfm25_slice out,
                                       const lfm25_fp8_linear_config* config);
/* The packed Gate/Up FP8 linear with the gated activation in its epilogue: one launch for
 * linear_decode_prequantized_fp8_into on the Gate/Up site + silu_mul_packed_bf16_to_e4m3_into (or
 * silu_mul_packed_bf16_into when `e4m3_output` is 0) of the decode step (src/model/decode_executor.rs:378-402,
 * kernels/silu_mul.cu:68-133).  `weight` [config->n = 2 * intermediate, config->k] E4M3 with the gate rows first,
 * `activation` [config->m, intermediate]: E4M3 codes of bf16(silu(bf16(gate)) * bf16(up)) * activation_scale, or
 * that bf16 value.  Same bits as the two-launch route (the projections are rounded to bf16 before the activation).
 * LFM25_ERR_UNSUPPORTED when the shape is outside the tensor-core kernel (n % 128, k % 128, m <= 256, 16-byte
 * aligned buffers): the caller then takes the two-launch route. */
int32_t lfm25_blaslt_linear_fp8_silu_mul(lfm25_blaslt* handle, lfm25_slice x, lfm25_slice weight,
                                         lfm25_slice activation, const lfm25_fp8_linear_config* config,
                                         float activation_scale, uint32_t e4m3_output);
/* Replaces BlasLt::linear_bf16 (src/cuda/blaslt/mod.rs:113-186): out[M,N] = x[M,K] * weight[N,K]^T in bf16 with
 * fp32 accumulation.  This library's tcgen05 kernels take the call where they measured ahead on the decode step;
 * elsewhere it goes through cuBLASLt (opened lazily; plans cached per shape), as the reference does for the
 * sites that are not promoted to FP8. */
int32_t lfm25_blaslt_linear_bf16(lfm25_blaslt* handle, lfm25_slice x, lfm25_slice weight, lfm25_slice out, size_t m,
                                 size_t n, size_t k);
/* The largest batch (rows of x) that lfm25_blaslt_linear_bf16 sends to this library's own tensor-core kernel when
 * nothing forces a route; larger batches go through cuBLASLt.  The value is measured on the whole decode step (the
 * figures are in the definition).  No counterpart in the reference, which always calls cuBLASLt. */
size_t lfm25_bf16_own_kernel_max_rows(void);
/* How many matmuls this process has handed to cuBLASLt so far (calls made while a stream is being captured count
 * once, replays of the captured graph do not): the benchmark's account of library launches per step. */
uint64_t lfm25_blaslt_library_calls(void);
/* The BF16 packed Gate/Up linear with the gated activation in its epilogue, for the layers whose Gate/Up site is
 * not promoted to FP8: linear_decode_into + silu_mul_packed_bf16_into (or ..._to_e4m3_into when `e4m3_output` is
 * set, for an FP8 Down site) of the decode step in one launch (src/model/decode_executor.rs:378-402,
 * kernels/silu_mul.cu:13-133).  `weight` [n = 2 * intermediate, k] bf16 with the gate rows first, `activation`
 * [m, intermediate]; same bits as the two-launch route.  LFM25_ERR_UNSUPPORTED outside the tensor-core kernel
 * (m <= 256, intermediate % 8 == 0, k % 64 == 0, 16-byte aligned buffers). */
int32_t lfm25_blaslt_linear_bf16_silu_mul(lfm25_blaslt* handle, lfm25_slice x, lfm25_slice weight,
                                          lfm25_slice activation, size_t m, size_t n, size_t k,
                                          float activation_scale, uint32_t e4m3_output);

/* Kernel and tile choice of the linears of one handle, in the place of the algorithm selection a cuBLASLt caller
 * has (cublasLtMatmulAlgoGetHeuristic in src/cuda/blaslt/plan.rs): every field 0 = the library's choice.
 * `kernel`: 1 weight-streaming mma.sync kernel (E4M3, M <= 8), 2 weight-major tcgen05 kernel, 3 generic kernel
 * (E4M3) / cuBLASLt (BF16), 4 batch-major tcgen05 kernel.  The other fields apply to the batch-major kernel:
 * weight rows per CTA (a multiple of 16 up to 256), K splits (1..8), ring slots (<= 12), warps that issue
 * tcgen05.mma (1, 2 or 4), CTAs per SM the tile count is fitted to (1 or 2), shared-memory budget per CTA in bytes,
 * batch slices (1..8 CTAs that share a weight tile, each with a part of the batch rows).
 * A choice the shape does not allow is ignored.  Passing NULL restores the defaults.  bench.py --workload gemm
 * uses it to sweep. */
typedef struct lfm25_gemm_tuning {
    uint32_t kernel;
    uint32_t n_tile;
    uint32_t splits;
    uint32_t stages;
    uint32_t issuers;
    uint32_t ctas_per_sm;
    uint32_t shared_memory_bytes;
    uint32_t batch_slices;
} lfm25_gemm_tuning;
int32_t lfm25_blaslt_set_gemm_tuning(lfm25_blaslt* handle, const lfm25_gemm_tuning* tuning);
/* What the batch-major kernel would launch for a problem under the handle's tuning (the counterpart of reading back
 * a cuBLASLt heuristic result): out = {n_tile, K splits, tiles, ring slots, issuing warps, CTAs per SM,
 * shared-memory bytes per CTA, batch slices}.  `k_bytes` is the row length in bytes (K for E4M3, 2 K for BF16); for
 * the gated form `n` is the intermediate width.  Launches nothing. */
int32_t lfm25_blaslt_gemm_plan(const lfm25_blaslt* handle, size_t m, size_t n, size_t k_bytes, uint32_t gated,
                               uint32_t out[8]);

/* ------------------------------------------------------------------------------------------
 * Remaining ops of the decode step
 * ------------------------------------------------------------------------------------------ */

/* Replaces EmbeddingKernels::launch (kernels/embedding.cu:65): out[t,:] = weight[token_ids[t],:]; an id >= vocab
 * leaves the row untouched. */
int32_t lfm25_embedding_bf16(void* stream, lfm25_slice token_ids, lfm25_slice weight, lfm25_slice out,
                             size_t num_tokens, size_t vocab_size, size_t hidden_size);
/* Replaces rms_norm_bf16 (kernels/rms_norm.cu:342): out = bf16(bf16(x * inv_rms) * weight), hidden_size even. */
int32_t lfm25_rms_norm_bf16(void* stream, lfm25_slice x, lfm25_slice weight, lfm25_slice out, size_t rows,
                            size_t hidden_size, float eps);
/* Replaces residual_rms_norm_bf16 (kernels/rms_norm.cu:364-463): residual_out = bf16(residual + update);
 * normalized_out = bf16(float(residual_out) * inv_rms * weight), the variance taken from the unrounded sums. */
int32_t lfm25_residual_rms_norm_bf16(void* stream, lfm25_slice residual, lfm25_slice update, lfm25_slice weight,
                                     lfm25_slice residual_out, lfm25_slice normalized_out, size_t rows,
                                     size_t hidden_size, float eps);
/* residual_rms_norm_bf16 (kernels/rms_norm.cu:364-463) and quantize_bf16_e4m3 (kernels/fp8_quantize.cu:9-45) of
 * its normalised output in one launch, for a norm whose consumer is an FP8 linear: codes_out (u8 [rows, hidden]) =
 * cvt.rn.satfinite.e4m3(float(normalized_out) * scale), bit-identical to the two launches. */
int32_t lfm25_residual_rms_norm_bf16_e4m3(void* stream, lfm25_slice residual, lfm25_slice update, lfm25_slice weight,
                                          lfm25_slice residual_out, lfm25_slice normalized_out, lfm25_slice codes_out,
                                          size_t rows, size_t hidden_size, float eps, float scale);
/* Replaces short_conv_segmented_lfm2_bf16 (kernels/short_conv.cu:100-143, src/cuda/kernels/short_conv.rs) for
 * segments of any length: projected [num_tokens, 3*hidden] = (b | c | x), weight [hidden, 3], states
 * [num_request_slots, hidden, 2] updated in place, segment_offsets u32 [num_segments + 1], segment_slots u32
 * [num_segments]; inside a segment the carried values stay unrounded fp32, the stored state is bf16.  A segment
 * whose slot is beyond the state table is skipped. */
int32_t lfm25_short_conv_segmented_lfm2_bf16(void* stream, lfm25_slice projected, lfm25_slice weight,
                                             lfm25_slice states, lfm25_slice segment_offsets,
                                             lfm25_slice segment_slots, lfm25_slice output, size_t num_tokens,
                                             size_t num_segments, size_t hidden_size, size_t num_request_slots);
/* Replaces gather_rows_bf16 (kernels/gather.cu): output[r] = input[row_indices[r]] for r < output_rows; an index
 * >= input_rows leaves the output row untouched.  columns must be even. */
int32_t lfm25_gather_rows_bf16(void* stream, lfm25_slice input, lfm25_slice row_indices, lfm25_slice output,
                               size_t output_rows, size_t input_rows, size_t columns);
/* Replaces short_conv_segmented_lfm2_bf16 (kernels/short_conv.cu:100-143) for decode (one token per segment):
 * projected [T, 3*hidden] = (b | c | x), weight [hidden, 3], states [request_slots, hidden, 2] updated in place. */
int32_t lfm25_short_conv_decode_bf16(void* stream, lfm25_slice projected, lfm25_slice weight, lfm25_slice states,
                                     lfm25_slice request_slots, lfm25_slice output, size_t num_tokens,
                                     size_t hidden_size, size_t num_request_slots);
/* Replaces argmax_rows_bf16 and its atomic variant (kernels/sampling.cu:53-217): greedy argmax per row with the
 * legacy tie order (smaller column % 256, then smaller column / 256; NaN and -inf never win; +-0 equal). */
int32_t lfm25_argmax_rows_bf16(void* stream, lfm25_slice logits, lfm25_slice sampled, size_t rows, size_t vocab_size);

/* ------------------------------------------------------------------------------------------
 * Decode step: device-resident batch metadata and the executor
 * ------------------------------------------------------------------------------------------ */

/* Device-resident step metadata (the tensors of GpuBatch, src/scheduler/batch.rs:126-140).  One token per
 * sequence.  `positions[t]` is the index of the token being decoded (= context length before it). */
typedef struct lfm25_decode_batch {
    uint32_t* token_ids;           /* u32 [num_tokens] */
    uint32_t* positions;           /* u32 [num_tokens] */
    const uint32_t* request_slots; /* u32 [num_tokens] block-table / conv-state row of each token */
    int64_t* physical_slots;       /* i64 [num_tokens], written by the step */
    const uint32_t* block_tables;  /* u32 [block_table_rows, block_table_stride] */
    size_t block_table_stride;
    size_t block_table_rows;
    size_t num_tokens;
    size_t max_context_tokens;     /* upper bound used to choose the number of KV splits */
} lfm25_decode_batch;

/* Replaces BatchModelCache::prepare_tokens + GpuBatch::update_step/update_segments + scatter_batch_metadata
 * (src/model/lfm2_base.rs:322-388, src/scheduler/batch.rs:142-260, kernels/metadata.cu:12-69) for pure decode:
 * physical_slots[t] = block_tables[slot][pos/16]*16 + pos%16 (or -1 when not mapped), computed on the device.
 * With advance != 0 every sequence first moves on by one token: token_ids[t] = sampled[t], positions[t] += 1.
 * No host loop, no H2D copy, no synchronisation. */
int32_t lfm25_decode_step_metadata(void* stream, const lfm25_decode_batch* batch, lfm25_slice sampled,
                                   size_t num_pages, uint32_t advance);

/* One linear site: BF16 weights, and/or E4M3 weights with their static scales (Fp8LinearWeight of the reference:
 * activation_scale = (448/c_x, c_x/448), weight_scale dequantize = c_w/448).  data == NULL: site not promoted. */
typedef struct lfm25_fp8_site {
    const void* data; /* u8 [n, k] */
    float activation_quantize;
    float activation_dequantize;
    float weight_dequantize;
} lfm25_fp8_site;
typedef struct lfm25_linear_weights {
    const void* bf16; /* bf16 [n, k], may be NULL when the FP8 copy is the only one resident */
    lfm25_fp8_site fp8;
    size_t n;
    size_t k;
} lfm25_linear_weights;

/* One decoder layer with its cache (LayerWeights + BatchLayerCache of the reference). */
typedef struct lfm25_layer {
    uint32_t is_attention;
    const void* operator_norm; /* bf16 [2048] */
    const void* ffn_norm;      /* bf16 [2048] */
    lfm25_linear_weights conv_input;  /* [6144, 2048] */
    const void* conv_kernel;          /* bf16 [2048, 3] */
    lfm25_linear_weights conv_output; /* [2048, 2048] */
    void* conv_state;                 /* bf16 [request_slots, 2048, 2] */
    /* When the BF16 query, key and value matrices are adjacent in memory in this order (one [3072, 2048]
     * allocation) the executor computes the three projections with one GEMM. */
    lfm25_linear_weights query;       /* [2048, 2048] */
    lfm25_linear_weights key;         /* [512, 2048] */
    lfm25_linear_weights value;       /* [512, 2048] */
    lfm25_linear_weights output;      /* [2048, 2048] */
    const void* query_norm;           /* bf16 [64] */
    const void* key_norm;             /* bf16 [64] */
    void* key_cache;                  /* bf16 [num_pages, 8, 16, 64] */
    void* value_cache;
    lfm25_linear_weights gate_up;     /* [16384, 2048], rows packed gate | up */
    lfm25_linear_weights down;        /* [2048, 8192] */
} lfm25_layer;

typedef struct lfm25_model {
    uint32_t num_layers;
    const lfm25_layer* layers;
    const void* embedding;      /* bf16 [65536, 2048]; tied LM head */
    lfm25_fp8_site lm_head_fp8; /* u8 [65536, 2048] when promoted */
    const void* final_norm;     /* bf16 [2048] */
    const float* inv_freq;      /* f32 [32] */
    float norm_eps;
    size_t num_pages;
    size_t num_request_slots;
} lfm25_model;

/* Replaces DecodeExecutor (src/model/decode_executor.rs): persistent scratch for up to maximum_tokens (<= 256)
 * tokens, allocated once here; the step itself allocates nothing. */
typedef struct lfm25_decode_executor lfm25_decode_executor;
int32_t lfm25_decode_executor_create(lfm25_blaslt* blaslt, size_t maximum_tokens, lfm25_decode_executor** out);
void lfm25_decode_executor_destroy(lfm25_decode_executor* executor);
/* DecodeExecutor::forward_prepared (:183-443) preceded by the device-side metadata step: enqueues one decode step
 * on the BlasLt handle's stream; sampled ids land in the executor's `sampled` buffer. */
int32_t lfm25_decode_executor_forward(lfm25_decode_executor* executor, const lfm25_model* model,
                                      const lfm25_decode_batch* batch, uint32_t use_fp8, uint32_t advance);
/* Device-resident metadata of a step that mixes prefill chunks and decode tokens (GpuBatch after
 * update_segments, src/scheduler/batch.rs:126-215): segment s holds tokens [segment_offsets[s],
 * segment_offsets[s+1]) of the sequence in request slot segment_slots[s], at consecutive positions;
 * output_rows[s] is the row of its last token.  physical_slots is written by the step. */
typedef struct lfm25_ragged_batch {
    const uint32_t* token_ids;       /* u32 [num_tokens] */
    const uint32_t* positions;       /* u32 [num_tokens] */
    const uint32_t* request_slots;   /* u32 [num_tokens] */
    int64_t* physical_slots;         /* i64 [num_tokens], written */
    const uint32_t* segment_offsets; /* u32 [num_segments + 1] */
    const uint32_t* segment_slots;   /* u32 [num_segments] */
    const uint32_t* output_rows;     /* u32 [num_segments] */
    const uint32_t* block_tables;    /* u32 [block_table_rows, block_table_stride] */
    size_t block_table_stride;
    size_t block_table_rows;
    size_t num_tokens;
    size_t num_segments;
    /* Extension: the first num_decode_segments segments are single-token decode segments (segment_offsets[i] == i
     * for i <= num_decode_segments, which is how Scheduler::schedule orders its work: decodes first).  Their
     * attention then runs in the decode kernel (KV-axis splits chosen from max_decode_context_tokens, the longest
     * context among them) and only the remaining segments in the hybrid kernel.  0: everything in the hybrid kernel. */
    size_t num_decode_segments;
    size_t max_decode_context_tokens;
} lfm25_ragged_batch;
/* An executor for steps of up to maximum_tokens tokens (<= 8192) in up to maximum_segments sequences (<= 256):
 * lfm25_decode_executor_create is the case maximum_tokens == maximum_segments. */
int32_t lfm25_decode_executor_create_ragged(lfm25_blaslt* blaslt, size_t maximum_tokens, size_t maximum_segments,
                                            lfm25_decode_executor** out);
/* Lfm2Model::forward_prepared_batch (src/model/lfm2_base.rs:924-997) for a mixed step: embedding, 16 layers
 * (segmented short conv; q/k/v, fused QK-norm + RoPE + paged append of every token, hybrid ragged attention over
 * the cache), logits and greedy ids for each segment's last token: row s of the executor's `logits` / `sampled`
 * belongs to segment s.  FP8 sites are used for steps of up to 256 tokens; larger steps run in BF16, as the
 * reference does above its maximum FP8 batch. */
int32_t lfm25_decode_executor_forward_ragged(lfm25_decode_executor* executor, const lfm25_model* model,
                                             const lfm25_ragged_batch* batch, uint32_t use_fp8);
/* The same step replayed from a CUDA graph captured per (batch size, flags, every value the step bakes in -- see
 * lfm25_decode_executor_graph_captures): the first call
 * of a bucket runs eagerly, the second captures, later ones only launch the graph.  With advance != 0 the step
 * feeds itself (ids and positions move on the device); with advance == 0 the caller refreshes the metadata
 * buffers between steps.  The handle must be bound to a non-default stream.  No counterpart in the reference, which
 * launches ~170 kernels and synchronises the host every step (src/engine/serving/radix_owner.rs:230-259). */
int32_t lfm25_decode_executor_step_graph(lfm25_decode_executor* executor, const lfm25_model* model,
                                         const lfm25_decode_batch* batch, uint32_t use_fp8, uint32_t advance);
/* One decode step as a serving loop runs it, in one call: uploads the step's metadata from pinned host memory
 * (`host_metadata`: token ids | positions | request slots, 3 * num_tokens u32; one copy when the batch's three device
 * arrays are adjacent in that order, three copies otherwise), replays the captured step (advance = 0), downloads the
 * sampled ids to `host_sampled` (num_tokens u32, pinned) and synchronises the stream: the sequence of
 * src/engine/serving/radix_owner.rs:230-259 (update_segments, forward, enqueue_sampled_download, synchronise). */
int32_t lfm25_decode_executor_serve_step(lfm25_decode_executor* executor, const lfm25_model* model,
                                         const lfm25_decode_batch* batch, uint32_t use_fp8,
                                         const uint32_t* host_metadata, uint32_t* host_sampled);
/* Kernel nodes of the CUDA graph that the last lfm25_decode_executor_step_graph call replayed (0 before the first
 * replay): the number of GPU kernels one step launches, this library's and cuBLASLt's together. */
size_t lfm25_decode_executor_graph_kernels(const lfm25_decode_executor* executor);
/* How many steps this executor has captured so far.  A captured step is replayed only while everything it baked in
 * is unchanged: batch size, split count, flags, every pointer, stride and row count of the batch, the model's page
 * count and every pointer, shape and scale inside model->layers, the library's switches and the handle's stream and
 * tuning; any change makes the next call run eagerly once and capture again. */
size_t lfm25_decode_executor_graph_captures(const lfm25_decode_executor* executor);
/* Opt-in region timing of eager steps (the reference's ModelProfileRecorder, src/model/profile.rs:84-253): while
 * enabled, every op of lfm25_decode_executor_forward is bracketed by CUDA events.  A call with region_ms != NULL
 * synchronises, returns the milliseconds and op counts accumulated per region since the last collection, and then
 * applies `enable`.  Graph-replayed steps are never instrumented. */
#define LFM25_REGION_ATTENTION 0   /* ragged paged attention (+ merge) */
#define LFM25_REGION_APPEND 1      /* QK-norm + RoPE + paged KV append */
#define LFM25_REGION_FP8_LINEAR 2  /* quantise / SiLU->E4M3 + E4M3 GEMM */
#define LFM25_REGION_BF16_LINEAR 3 /* cuBLASLt BF16 GEMM (+ SiLU for BF16 Down) */
#define LFM25_REGION_OTHER 4       /* metadata, embedding, norms, short conv, argmax */
#define LFM25_REGION_COUNT 5
int32_t lfm25_decode_executor_profile(lfm25_decode_executor* executor, uint32_t enable,
                                      float region_ms[LFM25_REGION_COUNT],
                                      uint32_t region_launches[LFM25_REGION_COUNT]);
/* Enqueues device-to-host copies of the last step's sampled ids (u32 [count]) or logits (bf16 [rows, 65536]) on
 * the executor's stream; the caller synchronises (the reference's pinned-ring download,
 * src/engine/serving/radix_owner.rs:441-462). */
int32_t lfm25_decode_executor_download_sampled(lfm25_decode_executor* executor, uint32_t* host, size_t count);
int32_t lfm25_decode_executor_download_logits(lfm25_decode_executor* executor, void* host, size_t rows);
const uint32_t* lfm25_decode_executor_sampled(const lfm25_decode_executor* executor); /* u32 [maximum_tokens] */
const void* lfm25_decode_executor_logits(const lfm25_decode_executor* executor);      /* bf16 [maximum_tokens, 65536] */

/* ------------------------------------------------------------------------------------------
 * Host-side state: page allocator, block tables, decode scheduling, replica dispatch (no device work)
 * ------------------------------------------------------------------------------------------ */

/* KvAllocationError (src/cache/allocator.rs:7-24) as negative return values. */
#define LFM25_KV_PHYSICAL_PAGES_EXHAUSTED (-11)
#define LFM25_KV_LOGICAL_RESERVATION_EXHAUSTED (-12)
#define LFM25_KV_SEQUENCE_CAPACITY_EXCEEDED (-13)

/* KvPoolSnapshot (src/cache/allocator.rs:28-35). */
typedef struct lfm25_kv_pool_snapshot {
    size_t total_pages;
    size_t free_pages;
    size_t allocated_pages;
    size_t reserved_pages;
    size_t cached_pages;
    size_t peak_allocated_pages;
} lfm25_kv_pool_snapshot;

/* Replaces KvPageAllocator (src/cache/allocator.rs:40-229): LIFO free list (a fresh pool hands out 0, 1, 2, ...),
 * per-page reference counts, reservation accounting, cache pins.  Single owner thread, as in the reference.
 * Functions returning int64_t give the count on success or a negative LFM25_KV_* code. */
typedef struct lfm25_kv_allocator lfm25_kv_allocator;
int32_t lfm25_kv_allocator_create(size_t total_pages, size_t page_size, lfm25_kv_allocator** out);
void lfm25_kv_allocator_destroy(lfm25_kv_allocator* allocator);
int64_t lfm25_kv_allocator_try_reserve_tokens(lfm25_kv_allocator* allocator, size_t maximum_tokens);
int64_t lfm25_kv_allocator_try_reserve_pages(lfm25_kv_allocator* allocator, size_t pages);
void lfm25_kv_allocator_release_reservation(lfm25_kv_allocator* allocator, size_t pages);
int32_t lfm25_kv_allocator_pin_cached_pages(lfm25_kv_allocator* allocator, const uint32_t* pages, size_t count);
int32_t lfm25_kv_allocator_retain_pages(lfm25_kv_allocator* allocator, const uint32_t* pages, size_t count);
int64_t lfm25_kv_allocator_grow_sequence(lfm25_kv_allocator* allocator, size_t current_tokens, size_t target_tokens,
                                         uint32_t* block_table, size_t block_table_len);
/* How many physical pages are missing for growing `sequences` sequences from current_tokens[i] to target_tokens[i]
 * all together (0 = every one of them fits); nothing is allocated.  A step that grows several sequences asks this
 * first, so that a shortage is reported before any block-table row has been changed.  No counterpart in the
 * reference, which grows the sequences of a step one by one (src/model/lfm2_base.rs:215-260). */
int64_t lfm25_kv_allocator_pages_short(const lfm25_kv_allocator* allocator, const size_t* current_tokens,
                                       const size_t* target_tokens, size_t sequences);
void lfm25_kv_allocator_release_sequence(lfm25_kv_allocator* allocator, size_t tokens, uint32_t* block_table,
                                         size_t block_table_len);
void lfm25_kv_allocator_snapshot(const lfm25_kv_allocator* allocator, lfm25_kv_pool_snapshot* out);

/* Replaces FixedBlockTables (src/cache/block_table.rs:3-31): u32 [slots, pages_per_slot], 0xffffffff = unassigned. */
typedef struct lfm25_block_tables lfm25_block_tables;
int32_t lfm25_block_tables_create(size_t slots, size_t pages_per_slot, lfm25_block_tables** out);
void lfm25_block_tables_destroy(lfm25_block_tables* tables);
uint32_t* lfm25_block_tables_slot(lfm25_block_tables* tables, size_t slot); /* NULL when out of range */
const uint32_t* lfm25_block_tables_data(const lfm25_block_tables* tables);

/* Replaces the decode half of Scheduler::schedule (src/scheduler/planner.rs:80-113): every slot whose phase is
 * LFM25_PHASE_DECODING decodes this step, ordered by time to its next-token deadline; also returns the longest
 * context (used to choose the KV splits).  Returns the number of decode slots written to decode_slots. */
#define LFM25_PHASE_FREE 0
#define LFM25_PHASE_QUEUED_PREFILL 1
#define LFM25_PHASE_DECODING 2
size_t lfm25_schedule_decode(const uint32_t* phases, const uint64_t* next_token_deadline_us,
                             const uint32_t* context_tokens, size_t num_slots, uint64_t now_us, uint32_t* decode_slots,
                             size_t* maximum_context_tokens);

/* Replaces CostCurve / HardwareCostModel (src/scheduler/cost_model.rs:7-231): measured step times as points
 * (batch, tokens per sequence, context) -> milliseconds, one curve each for BF16 decode, FP8 decode and BF16
 * prefill.  predict: an exact point, else the nearest point that dominates the query in every dimension, else a
 * conservative extrapolation; predict_decode_ms: bilinear interpolation inside the measured decode grid
 * (predict_decode_interpolated); predict_prefill_ms(tokens) = prefill curve at (1, tokens, tokens). */
typedef struct lfm25_cost_point {
    size_t batch;
    size_t tokens;
    size_t context;
    double milliseconds;
} lfm25_cost_point;
typedef struct lfm25_cost_model lfm25_cost_model;
#define LFM25_CURVE_DECODE_BF16 0
#define LFM25_CURVE_DECODE_FP8 1
#define LFM25_CURVE_PREFILL_BF16 2
int32_t lfm25_cost_model_create(const lfm25_cost_point* decode_bf16, size_t decode_bf16_points,
                                const lfm25_cost_point* decode_fp8, size_t decode_fp8_points,
                                const lfm25_cost_point* prefill_bf16, size_t prefill_bf16_points, size_t page_size,
                                lfm25_cost_model** out);
void lfm25_cost_model_destroy(lfm25_cost_model* model);
double lfm25_cost_model_predict(const lfm25_cost_model* model, uint32_t curve, size_t batch, size_t tokens,
                                size_t context);
double lfm25_cost_model_predict_decode_ms(const lfm25_cost_model* model, size_t batch, size_t maximum_context,
                                          uint32_t fp8);
double lfm25_cost_model_predict_prefill_ms(const lfm25_cost_model* model, size_t tokens);

/* Replaces Scheduler::schedule (src/scheduler/planner.rs:80-236).  `requests` is the request-slot table as plain
 * views (the fields of SequenceRequest the planner reads; context_tokens = tokens().len()).  Every decoding slot
 * decodes, ordered by time to its next-token deadline; the rest of the step budget goes to queued prefills, most
 * urgent first (time to the first-token deadline, aged by a quarter of the waiting time), in chunks of the largest
 * power of two <= 512 that the cost model fits into the budget; with >= 24 queued prefills of which one is a short
 * tail (<= one page left) of a long context (>= 1536 cached) the step stays decode-shaped and takes one token of
 * every such tail instead.  work needs room for num_requests entries. */
#define LFM25_WORK_DECODE 0
#define LFM25_WORK_PREFILL 1
typedef struct lfm25_scheduler_config {
    double step_budget_ms;
    uint64_t ttft_slo_us;
    uint64_t tpot_slo_us;
    uint32_t fp8_decode;
    size_t maximum_prefill_tokens;
} lfm25_scheduler_config;
typedef struct lfm25_request_view {
    uint32_t phase;                   /* LFM25_PHASE_* */
    size_t prompt_len;
    size_t prefilled;
    size_t context_tokens;
    uint64_t arrival_us;
    uint64_t first_token_deadline_us;
    uint64_t next_token_deadline_us;
} lfm25_request_view;
typedef struct lfm25_scheduled_work {
    uint32_t kind;                    /* LFM25_WORK_* */
    uint32_t slot;
    size_t tokens;
} lfm25_scheduled_work;
typedef struct lfm25_batch_plan {
    double predicted_ms;
    size_t decode_count;
    size_t prefill_tokens;
    size_t work_count;
} lfm25_batch_plan;
int32_t lfm25_schedule(const lfm25_cost_model* cost, const lfm25_scheduler_config* config,
                       const lfm25_request_view* requests, size_t num_requests, uint64_t now_us,
                       lfm25_scheduled_work* work, size_t work_capacity, lfm25_batch_plan* plan);

/* Replaces PageRadixCache (src/cache/radix.rs:61-287): host-only radix index over page-sized token blocks.  Every
 * non-root node stands for one immutable physical KV page (the caller pins newly indexed pages with
 * lfm25_kv_allocator_pin_cached_pages); a node may carry the slot of a convolution-state checkpoint taken right
 * after its last token.  One owner thread, like the allocator. */
typedef struct lfm25_radix_cache lfm25_radix_cache;
typedef struct lfm25_prefix_cache_snapshot {
    size_t nodes;
    size_t cached_pages;
    size_t checkpoints;
    uint64_t hits;
    uint64_t misses;
    uint64_t matched_tokens;
} lfm25_prefix_cache_snapshot;
int32_t lfm25_radix_cache_create(size_t page_size, size_t max_cached_pages, lfm25_radix_cache** out);
void lfm25_radix_cache_destroy(lfm25_radix_cache* cache);
/* longest_checkpoint (:100-107): the deepest indexed prefix of tokens[0 .. min(num_tokens, maximum_tokens)) that has
 * a checkpoint.  Returns its length in tokens (0 = miss) and fills physical_pages[0 .. *num_pages) and
 * *checkpoint_slot; counts a hit or a miss.  Negative: error (page buffer too small for the hit). */
int64_t lfm25_radix_cache_longest_checkpoint(lfm25_radix_cache* cache, const uint32_t* tokens, size_t num_tokens,
                                             size_t maximum_tokens, uint32_t* physical_pages, size_t pages_capacity,
                                             size_t* num_pages, uint32_t* checkpoint_slot);
/* probe_checkpoint (:109-114): the same lookup without touching the hit / miss counters. */
int64_t lfm25_radix_cache_probe_checkpoint(lfm25_radix_cache* cache, const uint32_t* tokens, size_t num_tokens,
                                           size_t maximum_tokens, uint32_t* physical_pages, size_t pages_capacity,
                                           size_t* num_pages, uint32_t* checkpoint_slot);
/* can_publish (:181-206): 1 when the page-aligned prefix is not yet checkpointed and its new pages fit the budget. */
uint32_t lfm25_radix_cache_can_publish(const lfm25_radix_cache* cache, const uint32_t* tokens, size_t num_tokens,
                                       size_t prefix_tokens);
/* insert_checkpoint (:210-271): indexes the prefix; newly_cached_pages (room for prefix_tokens / page_size entries)
 * receives the physical pages that became owned by new nodes, their count is the return value (negative: error). */
int64_t lfm25_radix_cache_insert_checkpoint(lfm25_radix_cache* cache, const uint32_t* tokens, size_t num_tokens,
                                            size_t prefix_tokens, const uint32_t* physical_pages,
                                            size_t num_physical_pages, uint32_t checkpoint_slot,
                                            uint32_t* newly_cached_pages);
void lfm25_radix_cache_snapshot(const lfm25_radix_cache* cache, lfm25_prefix_cache_snapshot* out);

/* Replaces ConvCheckpointPool (src/model/prefix.rs:15-129): `capacity` snapshots of every gated-convolution layer's
 * recurrent state, [capacity, hidden_size, state_width] bf16 per layer on the device.  acquire: a free slot or -1;
 * capture / restore: same-stream device-to-device copy between slot `checkpoint_slot` of layer `convolution_index`
 * and row `request_slot` of that layer's live state tensor [num_request_slots, hidden_size, state_width]. */
typedef struct lfm25_conv_checkpoints lfm25_conv_checkpoints;
int32_t lfm25_conv_checkpoints_create(size_t convolution_layers, size_t capacity, size_t hidden_size,
                                      size_t state_width, lfm25_conv_checkpoints** out);
void lfm25_conv_checkpoints_destroy(lfm25_conv_checkpoints* pool);
int64_t lfm25_conv_checkpoints_acquire(lfm25_conv_checkpoints* pool);
void lfm25_conv_checkpoints_release(lfm25_conv_checkpoints* pool, uint32_t slot);
size_t lfm25_conv_checkpoints_available(const lfm25_conv_checkpoints* pool);
size_t lfm25_conv_checkpoints_capacity(const lfm25_conv_checkpoints* pool);
int32_t lfm25_conv_checkpoints_capture_layer(lfm25_conv_checkpoints* pool, void* stream, uint32_t checkpoint_slot,
                                             size_t convolution_index, const void* states, size_t request_slot,
                                             size_t num_request_slots);
int32_t lfm25_conv_checkpoints_restore_layer(lfm25_conv_checkpoints* pool, void* stream, uint32_t checkpoint_slot,
                                             size_t convolution_index, void* states, size_t request_slot,
                                             size_t num_request_slots);

/* Request dispatcher over engine replicas (one replica per GPU; the model and every sequence's KV fit one GPU, so
 * nothing is sharded and no collective runs on the step path).  A request goes to the live replica with the least
 * outstanding tokens, except that requests sharing a prompt prefix go to the replica that prefix hashes to, so
 * that its prefix cache is hit.  No counterpart in the reference, which drives a single GPU. */
typedef struct lfm25_dispatcher lfm25_dispatcher;
int32_t lfm25_dispatcher_create(size_t replicas, lfm25_dispatcher** out);
void lfm25_dispatcher_destroy(lfm25_dispatcher* dispatcher);
int32_t lfm25_dispatcher_assign(lfm25_dispatcher* dispatcher, uint64_t prefix_hash, uint32_t has_prefix,
                                uint64_t estimated_tokens); /* replica index, or a negative error */
/* The same with bounded imbalance: the prefix's home replica takes the request only while its outstanding tokens
 * exceed those of the least-loaded live replica by at most slack_tokens; otherwise the least-loaded replica does. */
int32_t lfm25_dispatcher_assign_bounded(lfm25_dispatcher* dispatcher, uint64_t prefix_hash, uint32_t has_prefix,
                                        uint64_t estimated_tokens, uint64_t slack_tokens);
void lfm25_dispatcher_complete(lfm25_dispatcher* dispatcher, size_t replica, uint64_t tokens);
void lfm25_dispatcher_mark_failed(lfm25_dispatcher* dispatcher, size_t replica);
uint64_t lfm25_dispatcher_load(const lfm25_dispatcher* dispatcher, size_t replica);

/* The GPU-owner loop of continuous batching (src/engine/serving/radix_owner.rs:101-708 with RequestSlots /
 * SequenceRequest, src/scheduler/{slots,request}.rs): request slots, admission with prefix reuse, planning, mixed
 * prefill / decode steps, token bookkeeping, built from the parts above.  One engine per GPU, driven from one host
 * thread; `model` and `blaslt` must outlive it.  lfm25_engine_calibrate measures the planner's cost curves on the
 * idle engine (needed once before the first step).  lfm25_engine_step admits what fits, plans and runs one step on
 * the handle's stream, synchronises once and reports the tokens it produced: one event per sequence that got a
 * token (events needs room for max_slots entries); gpu_ms (may be NULL) is the step's GPU time.  Greedy sampling. */
typedef struct lfm25_engine lfm25_engine;
typedef struct lfm25_engine_config {
    size_t max_slots;             /* concurrent sequences, <= 256 and <= model->num_request_slots */
    size_t max_sequence_tokens;   /* prompt + generated tokens per sequence */
    size_t max_prefill_tokens;    /* per step (the planner's maximum_prefill_tokens) */
    size_t radix_pages;           /* page budget of the prefix index */
    size_t checkpoint_capacity;   /* convolution-state checkpoints */
    uint32_t use_fp8;
    uint64_t ttft_slo_us;
    uint64_t tpot_slo_us;
    double step_budget_ms;
    /* SLO admission (admit_request_radix, src/engine/serving/radix_owner.rs:549-708).  0: a request that does not
     * fit yet waits in the queue, in order (back-pressure).  1: every queued request is decided at the next step,
     * admitted or rejected with one of the LFM25_REJECT_* reasons, as the reference answers "overloaded". */
    uint32_t admission_control;
    size_t interactive_prompt_limit;   /* longest admitted prompt when admission_control is on; 0 = no limit */
} lfm25_engine_config;
/* Why a request was turned away (lfm25_engine_event.rejected), in the order the reference checks them. */
#define LFM25_REJECT_NONE 0u
#define LFM25_REJECT_SEQUENCE_CAPACITY 1u /* prompt + new tokens exceed max_sequence_tokens */
#define LFM25_REJECT_PROMPT_LIMIT 2u      /* prompt longer than interactive_prompt_limit */
#define LFM25_REJECT_DECODE_BUDGET 3u     /* predicted decode step with one more sequence >= step budget or TPOT SLO */
#define LFM25_REJECT_TTFT 4u              /* time already waited + predicted prefill queue >= TTFT SLO */
#define LFM25_REJECT_SLOTS 5u             /* no free request slot */
#define LFM25_REJECT_KV_PAGES 6u          /* the page reservation for the whole sequence failed */
typedef struct lfm25_engine_event {
    uint64_t request_id;
    uint64_t time_us;             /* now_us of the step + its GPU time */
    uint32_t token;
    uint32_t finished;            /* the request produced its last token and left its slot */
    uint32_t reused_tokens;       /* prompt tokens this request took from the prefix index */
    uint32_t rejected;            /* LFM25_REJECT_*: nonzero = the request was not admitted (token 0, finished 1) */
} lfm25_engine_event;
typedef struct lfm25_engine_stats {
    uint64_t steps;
    uint64_t decode_steps;
    uint64_t mixed_steps;
    uint64_t generated_tokens;
    uint64_t prefill_tokens;
    uint64_t reused_prompt_tokens;
    double gpu_ms;
    uint64_t rejected_requests;
} lfm25_engine_stats;
int32_t lfm25_engine_create(lfm25_blaslt* blaslt, const lfm25_model* model, const lfm25_engine_config* config,
                            lfm25_engine** out);
void lfm25_engine_destroy(lfm25_engine* engine);
int32_t lfm25_engine_calibrate(lfm25_engine* engine);
const lfm25_cost_model* lfm25_engine_cost_model(const lfm25_engine* engine);
int32_t lfm25_engine_submit(lfm25_engine* engine, uint64_t request_id, const uint32_t* prompt, size_t prompt_len,
                            size_t max_new_tokens, uint64_t arrival_us);
int32_t lfm25_engine_step(lfm25_engine* engine, uint64_t now_us, lfm25_engine_event* events, size_t events_capacity,
                          size_t* num_events, float* gpu_ms);
size_t lfm25_engine_active(const lfm25_engine* engine);
size_t lfm25_engine_queued(const lfm25_engine* engine);
void lfm25_engine_get_stats(const lfm25_engine* engine, lfm25_engine_stats* stats, lfm25_kv_pool_snapshot* pool,
                            lfm25_prefix_cache_snapshot* prefix);

#ifdef __cplusplus
}
#endif

#endif /* LFM25_B200_H */
