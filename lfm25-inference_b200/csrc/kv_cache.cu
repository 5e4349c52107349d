// Paged KV append kernels for sm_100a.
//
// raw append      : replaces kernels/kv_cache.cu:30-120 of the reference (bit copy of K and V
//                   [T,8,64] into the arena [pages,8,16,64] at slot_mapping[t]).
// fused post-proc : replaces kernels/qk_postprocess.cu:44-151 (Q RMSNorm + RoPE in place,
//                   K RMSNorm + RoPE written straight into the arena, V copied).
//
// Both are latency-bound (a few KiB per token); they exist to be bit-exact and cheap to launch.
#include "common.cuh"
#include "qk_norm_rope.cuh"
#include "kernels.h"
#include "launch.h"

namespace lfm25 {

namespace {

// One CTA per token, 128 threads, 16 bytes per thread: threads 0..63 move K, 64..127 move V.
// A token's K (8 heads x 128 B) is contiguous in the source and lands as 8 runs of 128 B.
__global__ void __launch_bounds__(128)
kv_cache_write_kernel(const uint4* __restrict__ key, const uint4* __restrict__ value, uint4* __restrict__ key_cache,
                      uint4* __restrict__ value_cache, const int64_t* __restrict__ slot_mapping, size_t num_tokens,
                      size_t num_pages) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t token = blockIdx.x;
    if (token >= num_tokens) {
        return;
    }
    const int64_t slot = slot_mapping[token];
    if (slot < 0) {
        return;
    }
    const size_t page = static_cast<size_t>(slot) / kPageSize;
    const size_t offset = static_cast<size_t>(slot) % kPageSize;
    if (page >= num_pages) {
        return;
    }
    const uint32_t vector = threadIdx.x & 63;      // 16-byte vector inside the token: 8 per head
    const uint32_t head = vector >> 3;
    const uint32_t piece = vector & 7;
    const size_t source = token * 64 + vector;
    const size_t destination = ((page * kKvHeads + head) * kPageSize + offset) * 8 + piece;
    if (threadIdx.x < 64) {
        key_cache[destination] = key[source];
    } else {
        value_cache[destination] = value[source];
    }
}

// One CTA per token, 10 warps: warps 0..7 each take 4 query heads, warps 8..9 each take 4 KV
// heads (K normalised + rotated into the arena, V copied).  The three inputs take a token stride (in elements), so
// they may be columns of one packed [tokens, 3072] projection; the rotated query goes to a dense [tokens, 32, 64]
// array, which may be the input itself.  Every warp evaluates the 32 RoPE
// coefficients of the token itself (one sincosf per lane), so the CTA needs no barrier.
constexpr uint32_t kPostWarps = 10;
__global__ void __launch_bounds__(kPostWarps * 32)
qk_norm_rope_kv_write_decode_kernel(const __nv_bfloat16* query, __nv_bfloat16* query_out,
                                    const __nv_bfloat16* __restrict__ key, const __nv_bfloat16* __restrict__ value,
                                    size_t query_token_stride, size_t kv_token_stride,
                                    const __nv_bfloat16* __restrict__ query_norm,
                                    const __nv_bfloat16* __restrict__ key_norm, const float* __restrict__ inv_freq,
                                    const uint32_t* __restrict__ position_ids,
                                    const int64_t* __restrict__ slot_mapping, __nv_bfloat16* __restrict__ key_cache,
                                    __nv_bfloat16* __restrict__ value_cache, size_t num_tokens, size_t num_pages,
                                    float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t token = blockIdx.x;
    if (token >= num_tokens) {
        return;
    }
    const int64_t slot = slot_mapping[token];
    if (slot < 0) {
        return;
    }
    const size_t page = static_cast<size_t>(slot) / kPageSize;
    const size_t offset = static_cast<size_t>(slot) % kPageSize;
    if (page >= num_pages) {
        return;
    }
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = threadIdx.x >> 5;
    float sin_value;
    float cos_value;
    sincosf(static_cast<float>(position_ids[token]) * inv_freq[lane], &sin_value, &cos_value);

    if (warp < 8) {
        const __nv_bfloat16 weight0 = query_norm[lane];
        const __nv_bfloat16 weight1 = query_norm[lane + kHalfDim];
#pragma unroll
        for (uint32_t index = 0; index < 4; ++index) {
            const __nv_bfloat16* row = query + token * query_token_stride + (warp * 4 + index) * kHeadDim;
            __nv_bfloat16* row_out = query_out + (token * kQHeads + warp * 4 + index) * kHeadDim;
            __nv_bfloat16 out0, out1;
            norm_rope(__bfloat162float(row[lane]), __bfloat162float(row[lane + kHalfDim]), weight0, weight1,
                      sin_value, cos_value, eps, out0, out1);
            row_out[lane] = out0;
            row_out[lane + kHalfDim] = out1;
        }
    } else {
        const __nv_bfloat16 weight0 = key_norm[lane];
        const __nv_bfloat16 weight1 = key_norm[lane + kHalfDim];
#pragma unroll
        for (uint32_t index = 0; index < 4; ++index) {
            const uint32_t head = (warp - 8) * 4 + index;
            const size_t source = token * kv_token_stride + head * kHeadDim;
            const size_t destination = ((page * kKvHeads + head) * kPageSize + offset) * kHeadDim;
            __nv_bfloat16 out0, out1;
            norm_rope(__bfloat162float(key[source + lane]), __bfloat162float(key[source + lane + kHalfDim]), weight0,
                      weight1, sin_value, cos_value, eps, out0, out1);
            key_cache[destination + lane] = out0;
            key_cache[destination + lane + kHalfDim] = out1;
            // V: 128 bytes per head, 4 bytes per lane
            reinterpret_cast<uint32_t*>(value_cache + destination)[lane] =
                reinterpret_cast<const uint32_t*>(value + source)[lane];
        }
    }
}

}  // namespace

cudaError_t launch_kv_cache_write(cudaStream_t stream, const void* key, const void* value, void* key_cache,
                                  void* value_cache, const int64_t* slot_mapping, size_t num_tokens,
                                  size_t num_pages) {
    return launch_kernel(kv_cache_write_kernel, static_cast<unsigned int>(num_tokens), 128, 0, stream, 1, 
        static_cast<const uint4*>(key), static_cast<const uint4*>(value), static_cast<uint4*>(key_cache),
        static_cast<uint4*>(value_cache), slot_mapping, num_tokens, num_pages);
}

cudaError_t launch_qk_norm_rope_kv_write_decode(cudaStream_t stream, const QkPostprocessArgs& args) {
    return launch_kernel(qk_norm_rope_kv_write_decode_kernel, static_cast<unsigned int>(args.num_tokens), kPostWarps * 32, 0, stream, 1, 
        static_cast<const __nv_bfloat16*>(args.query), static_cast<__nv_bfloat16*>(args.query_out),
        static_cast<const __nv_bfloat16*>(args.key), static_cast<const __nv_bfloat16*>(args.value),
        args.query_token_stride, args.kv_token_stride, static_cast<const __nv_bfloat16*>(args.query_norm),
        static_cast<const __nv_bfloat16*>(args.key_norm), args.inv_freq, args.position_ids, args.slot_mapping,
        static_cast<__nv_bfloat16*>(args.key_cache), static_cast<__nv_bfloat16*>(args.value_cache), args.num_tokens,
        args.num_pages, args.eps);
}

}  // namespace lfm25
