// Host-side launch functions of the CUDA kernels (internal to the library; the public
// boundary is include/lfm25_b200.h).  Arguments are already validated by the callers in api.cu.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lfm25 {

struct AttentionLaunch {
    const void* query;            // bf16 [T,32,64]
    const void* key_cache;        // bf16 [pages,8,16,64]
    const void* value_cache;
    const uint32_t* block_tables; // [rows, stride]
    const uint32_t* request_slots;// [T] or nullptr (row 0)
    const uint32_t* position_ids; // [T]
    void* output;                 // bf16 [T,32,64]
    float* partials;              // f32 [T,32,S,66] when num_splits > 1
    unsigned int* status;
    size_t num_tokens;
    size_t num_pages;
    size_t block_table_stride;
    size_t block_table_rows;
    uint32_t num_splits;          // 1 = unsplit
    // fused mode (key_raw != nullptr): raw projections in, new cache row produced inside the kernel
    const void* key_raw = nullptr;      // bf16 [T,8,64]
    const void* value_raw = nullptr;    // bf16 [T,8,64]
    const void* query_norm = nullptr;   // bf16 [64]
    const void* key_norm = nullptr;     // bf16 [64]
    const float* inv_freq = nullptr;    // f32 [32]
    const int64_t* slot_mapping = nullptr;
    float eps = 0.0f;
    size_t query_token_stride = 32 * 64;   // elements between tokens of `query`
    size_t kv_token_stride = 8 * 64;       // elements between tokens of key_raw / value_raw
    // optional permutation of the tokens: CTAs are handed out in this order (longest context first evens out the
    // tail of the grid); nullptr = as given
    const uint32_t* token_order = nullptr;
};
cudaError_t launch_ragged_decode_attention(cudaStream_t stream, const AttentionLaunch& launch);
// order[r] = index of the token with the r-th largest position (ties by index); at most kMaxOrderTokens tokens
constexpr size_t kMaxOrderTokens = 2048;
cudaError_t launch_context_order(cudaStream_t stream, const uint32_t* positions, size_t num_tokens, uint32_t* order);

// Attention of a mixed prefill / decode step (hybrid_attention.cu).  `current_key` == nullptr: every key up to a
// token's position is read from the cache; otherwise the segment's own tokens come from current_key / current_value.
struct HybridAttentionLaunch {
    const void* query;             // bf16 [T,32,64], rows query_token_stride apart
    const void* current_key;       // bf16 [T,8,64], rows kv_token_stride apart, or nullptr
    const void* current_value;
    const void* key_cache;         // bf16 [pages,8,16,64]
    const void* value_cache;
    const uint32_t* block_tables;  // [rows, stride]
    const uint32_t* request_slots; // [T]
    const uint32_t* position_ids;  // [T]
    const uint32_t* segment_offsets;  // [S + 1]
    void* output;                  // bf16 [T,32,64], dense
    unsigned int* status;
    size_t num_tokens;
    size_t num_pages;
    size_t block_table_stride;
    size_t block_table_rows;
    size_t num_segments;
    size_t query_token_stride = 32 * 64;
    size_t kv_token_stride = 8 * 64;
};
cudaError_t launch_hybrid_ragged_attention(cudaStream_t stream, const HybridAttentionLaunch& launch);
// The same function on tcgen05 / TMEM, 32 tokens x 4 heads per CTA (hybrid_attention_umma.cu); needs the query
// 16-byte aligned with a token stride that is a multiple of 8 elements.
cudaError_t launch_hybrid_attention_umma(cudaStream_t stream, const HybridAttentionLaunch& launch);

cudaError_t launch_kv_cache_write(cudaStream_t stream, const void* key, const void* value, void* key_cache,
                                  void* value_cache, const int64_t* slot_mapping, size_t num_tokens,
                                  size_t num_pages);

struct QkPostprocessArgs {
    const void* query;            // [tokens] rows of 32 x 64, `query_token_stride` elements apart
    void* query_out;              // dense [tokens, 32, 64]; may alias `query` when that is dense
    size_t query_token_stride;
    size_t kv_token_stride;       // of `key` and `value` rows (8 x 64 each)
    const void* key;
    const void* value;
    const void* query_norm;
    const void* key_norm;
    const float* inv_freq;
    const uint32_t* position_ids;
    const int64_t* slot_mapping;
    void* key_cache;
    void* value_cache;
    size_t num_tokens;
    size_t num_pages;
    float eps;
};
cudaError_t launch_qk_norm_rope_kv_write_decode(cudaStream_t stream, const QkPostprocessArgs& args);

cudaError_t launch_quantize_bf16_e4m3(cudaStream_t stream, const void* input, void* output, size_t numel,
                                      float scale);
cudaError_t launch_silu_mul_packed_bf16(cudaStream_t stream, const void* packed, void* out, size_t rows,
                                        size_t intermediate);
cudaError_t launch_silu_mul_packed_bf16_to_e4m3(cudaStream_t stream, const void* packed, void* out, size_t rows,
                                                size_t intermediate, float scale);

// FP8 linear: Y[M,N] = bf16(alpha * Xq[M,K] * Wq[N,K]^T)
bool fp8_gemm_stream_supports(size_t m, size_t n, size_t k);
cudaError_t launch_fp8_gemm_stream(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                   size_t n, size_t k, float alpha);
cudaError_t launch_fp8_gemm_generic(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                    size_t n, size_t k, float alpha);

bool fp8_gemm_umma_supports(size_t m, size_t n, size_t k);
// Packed Gate/Up GEMM with SiLU(gate) * up in the epilogue: `weight` [n = 2 * intermediate, k] (gate rows first),
// `activation` [m, n / 2] as E4M3 codes of the bf16 activation times `code_scale`, or as bf16.
bool fp8_gemm_umma_gated_supports(size_t m, size_t n, size_t k);
cudaError_t launch_fp8_gemm_umma_gated(cudaStream_t stream, const void* x, const void* weight, void* activation,
                                       size_t m, size_t n, size_t k, float alpha, float code_scale, bool e4m3,
                                       unsigned int* status);
// `exchange` (may be null: K is then not split) is scratch for split-K partial tiles, owned by the caller and
// used by one stream at a time; kUmmaExchangeBytes covers every supported shape.
constexpr size_t kUmmaExchangeBytes = 148u * 256u * 128u * 4u;
cudaError_t launch_fp8_gemm_umma(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                 size_t n, size_t k, float alpha, void* exchange, size_t exchange_bytes,
                                 unsigned int* status);

// Batch-major tcgen05 GEMM (gemm_rows_umma.cu): the batch on the TMEM lanes, a tile of n_tile weight rows as the
// N operand.  A tuning field that is 0 is chosen by gemm_rows_plan().
struct GemmRowsTuning {
    uint32_t n_tile = 0;       // weight rows per CTA, a multiple of 16 up to 256
    uint32_t splits = 0;       // K splits (cluster size), 1..8
    uint32_t stages = 0;       // ring slots (one 128-byte K block of activations and weights each), <= 12
    uint32_t issuers = 0;      // warps that issue tcgen05.mma, each into an accumulator of its own: 1, 2 or 4
    uint32_t slices = 0;       // CTAs that share a weight tile, each with 1 / slices of the batch rows: 1..8
    uint32_t ctas_per_sm = 0;  // 1 or 2: which wave size the tile count is fitted to
    uint32_t smem_bytes = 0;   // shared-memory budget of one CTA
};
struct GemmRowsPlan {
    uint32_t n_tile, splits, tiles, a_tiles, a_rows, slices, slice_rows, stages, issuers, ctas_per_sm;
    uint32_t stage_bytes, control_offset, smem_bytes;
    bool valid;
};
// `k_bytes`: length of a weight / activation row in bytes (K for E4M3, 2 K for BF16); `n`: output features, for
// the gated form the intermediate width
bool gemm_rows_supports(size_t m, size_t n, size_t k_bytes);
GemmRowsPlan gemm_rows_plan(size_t m, size_t n, size_t k_bytes, bool gated, size_t exchange_bytes,
                            const GemmRowsTuning& tuning);
// Where the batch-major kernel measured ahead of the other routes (the weight-major tcgen05 kernel, cuBLASLt)
bool fp8_rows_preferred(size_t m, size_t n, size_t k);
bool bf16_rows_preferred(size_t m, size_t n, size_t k);
bool fp8_gated_rows_preferred(size_t m, size_t intermediate, size_t k);
cudaError_t launch_fp8_gemm_rows(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                 size_t n, size_t k, float alpha, void* exchange, size_t exchange_bytes,
                                 unsigned int* status, const GemmRowsTuning& tuning);
// packed Gate/Up weights [2 * intermediate, k] (gate rows first); activation [m, intermediate] as E4M3 codes of the
// bf16 activation times code_scale, or as bf16
cudaError_t launch_fp8_gemm_rows_gated(cudaStream_t stream, const void* x, const void* weight, void* activation,
                                       size_t m, size_t intermediate, size_t k, float alpha, float code_scale,
                                       bool e4m3, unsigned int* status, const GemmRowsTuning& tuning);
cudaError_t launch_bf16_gemm_rows(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                  size_t n, size_t k, void* exchange, size_t exchange_bytes, unsigned int* status,
                                  const GemmRowsTuning& tuning);
cudaError_t launch_bf16_gemm_rows_gated(cudaStream_t stream, const void* x, const void* weight, void* activation,
                                        size_t m, size_t intermediate, size_t k, float code_scale, bool e4m3,
                                        unsigned int* status, const GemmRowsTuning& tuning);

cudaError_t launch_embedding_bf16(cudaStream_t stream, const uint32_t* token_ids, const void* table, void* out,
                                  size_t num_tokens, size_t vocab_size, size_t hidden);
cudaError_t launch_rms_norm_bf16(cudaStream_t stream, const void* x, const void* weight, void* out, size_t rows,
                                 size_t hidden, float eps);
// `codes` (optional): the normalised rows also as E4M3 with multiplier `code_scale`, bit-identical to quantising
// `normalized_out` afterwards.
cudaError_t launch_residual_rms_norm_bf16(cudaStream_t stream, const void* residual, const void* update,
                                          const void* weight, void* residual_out, void* normalized_out, size_t rows,
                                          size_t hidden, float eps, void* codes = nullptr, float code_scale = 1.0f);
cudaError_t launch_short_conv_decode(cudaStream_t stream, const void* projected, const void* weight, void* states,
                                     const uint32_t* request_slots, void* output, size_t num_tokens, size_t hidden,
                                     size_t num_request_slots);
cudaError_t launch_short_conv_segmented(cudaStream_t stream, const void* projected, const void* weight, void* states,
                                        const uint32_t* segment_offsets, const uint32_t* segment_slots, void* output,
                                        size_t num_tokens, size_t num_segments, size_t hidden,
                                        size_t num_request_slots);
cudaError_t launch_gather_rows_bf16(cudaStream_t stream, const void* input, const uint32_t* row_indices, void* output,
                                    size_t output_rows, size_t input_rows, size_t columns);
cudaError_t launch_argmax_rows_bf16(cudaStream_t stream, const void* logits, uint32_t* sampled, size_t rows,
                                    size_t vocab);
cudaError_t launch_decode_metadata(cudaStream_t stream, uint32_t* token_ids, uint32_t* positions,
                                   const uint32_t* request_slots, const uint32_t* block_tables, const uint32_t* sampled,
                                   int64_t* physical_slots, size_t num_tokens, size_t block_table_stride,
                                   size_t block_table_rows, size_t num_pages, bool advance,
                                   uint32_t* token_order = nullptr);

bool bf16_gemm_umma_supports(size_t m, size_t n, size_t k);
cudaError_t launch_bf16_gemm_umma(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                  size_t n, size_t k, void* exchange, size_t exchange_bytes, unsigned int* status);

// Stores `message` as the calling thread's last error (what lfm25_last_error() returns) and returns `code`.
int32_t report_error(int32_t code, const char* message);

}  // namespace lfm25
