// The remaining small ops of a decode step (everything between the GEMMs and the attention):
// embedding rows, RMSNorm, residual add + RMSNorm, gated short convolution, greedy argmax, and the
// device-side step metadata that replaces the reference's per-step host loop and H2D slab.
//
// They replace, in the reference: kernels/embedding.cu:65, kernels/rms_norm.cu:342 and :364,
// kernels/short_conv.cu:100 (one token per segment, the decode case), kernels/sampling.cu:53-217
// (tie order of the legacy argmax), kernels/metadata.cu:12-69 + src/model/lfm2_base.rs:338-380.
// All are a few hundred KiB of traffic per launch at decode batch sizes: they are written to be
// cheap to launch (one CTA per row, 16-byte accesses), not tuned against a roofline.
#include <float.h>

#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace lfm25 {

namespace {

constexpr uint32_t kRowThreads = 256;

__device__ __forceinline__ float block_sum_256(float value, float* scratch) {
#pragma unroll
    for (uint32_t delta = 16; delta > 0; delta >>= 1) {
        value += __shfl_xor_sync(0xffffffffu, value, delta);
    }
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    if (lane == 0) {
        scratch[warp] = value;
    }
    __syncthreads();
    float total = lane < (blockDim.x >> 5) ? scratch[lane] : 0.0f;
#pragma unroll
    for (uint32_t delta = 4; delta > 0; delta >>= 1) {
        total += __shfl_xor_sync(0xffffffffu, total, delta);
    }
    return __shfl_sync(0xffffffffu, total, 0);
}

// out[t, :] = table[token_ids[t], :]; an id beyond the vocabulary leaves the row untouched.
__global__ void __launch_bounds__(kRowThreads)
embedding_kernel(const uint32_t* __restrict__ token_ids, const __nv_bfloat16* __restrict__ table,
                 __nv_bfloat16* __restrict__ out, size_t num_tokens, size_t vocab_size, size_t hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t token = blockIdx.x;
    if (token >= num_tokens) {
        return;
    }
    const uint32_t id = token_ids[token];
    if (id >= vocab_size) {
        return;
    }
    const __nv_bfloat16* source = table + static_cast<size_t>(id) * hidden;
    __nv_bfloat16* destination = out + token * hidden;
    if (hidden % 8 == 0) {
        for (size_t vector = threadIdx.x; vector < hidden / 8; vector += blockDim.x) {
            reinterpret_cast<uint4*>(destination)[vector] = __ldg(reinterpret_cast<const uint4*>(source) + vector);
        }
    } else {
        for (size_t index = threadIdx.x; index < hidden; index += blockDim.x) {
            destination[index] = source[index];
        }
    }
}

// RESIDUAL == false: out = bf16(bf16(x * inv_rms) * weight)                    (kernels/rms_norm.cu:268-278)
// RESIDUAL == true : r = bf16(residual + update) stored to residual_out; the variance uses the unrounded fp32
//                    sums; out = bf16(float(r) * inv_rms * float(weight))       (kernels/rms_norm.cu:394-453)
// `codes` (may be null): the normalised row again as E4M3, code = cvt.rn.satfinite(float(out) * code_scale) -- what
// quantize_bf16_e4m3 would produce from `out` -- for a consumer that is an FP8 linear.
template <bool RESIDUAL>
__global__ void __launch_bounds__(kRowThreads)
rms_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ update,
                const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ residual_out,
                __nv_bfloat16* __restrict__ out, uint8_t* __restrict__ codes, float code_scale, size_t rows,
                size_t hidden, float eps) {
    pdl_launch_dependents();
    __shared__ float scratch[8];
    const size_t row = blockIdx.x;
    const uintptr_t alignment = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(update) |
                                reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(residual_out) |
                                reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(codes);
    if (hidden == 8 * kRowThreads && blockDim.x == kRowThreads && (alignment & 15) == 0) {
        // The model's width (2048): every thread keeps its 8 consecutive elements in registers between the two
        // passes, all accesses are 16 bytes wide, and the norm weights (constants) are fetched before the
        // dependency wait.
        const uint4 weight_raw = *reinterpret_cast<const uint4*>(weight + threadIdx.x * 8);
        pdl_wait();
        if (row >= rows) {
            return;
        }
        const size_t base = row * hidden + threadIdx.x * 8;
        const uint4 x_raw = *reinterpret_cast<const uint4*>(x + base);
        const __nv_bfloat162* x_pairs = reinterpret_cast<const __nv_bfloat162*>(&x_raw);
        const __nv_bfloat162* weight_pairs = reinterpret_cast<const __nv_bfloat162*>(&weight_raw);
        float2 value[4];
        __nv_bfloat162 source[4];   // what the second pass normalises: x, or the rounded residual
        float local = 0.0f;
        if (RESIDUAL) {
            const uint4 update_raw = *reinterpret_cast<const uint4*>(update + base);
            const __nv_bfloat162* update_pairs = reinterpret_cast<const __nv_bfloat162*>(&update_raw);
#pragma unroll
            for (uint32_t pair = 0; pair < 4; ++pair) {
                const float2 a = __bfloat1622float2(x_pairs[pair]);
                const float2 b = __bfloat1622float2(update_pairs[pair]);
                value[pair] = make_float2(a.x + b.x, a.y + b.y);
                source[pair] = __floats2bfloat162_rn(value[pair].x, value[pair].y);
            }
            *reinterpret_cast<uint4*>(residual_out + base) = *reinterpret_cast<const uint4*>(source);
        } else {
#pragma unroll
            for (uint32_t pair = 0; pair < 4; ++pair) {
                value[pair] = __bfloat1622float2(x_pairs[pair]);
                source[pair] = x_pairs[pair];
            }
        }
#pragma unroll
        for (uint32_t pair = 0; pair < 4; ++pair) {
            local = fmaf(value[pair].x, value[pair].x, local);
            local = fmaf(value[pair].y, value[pair].y, local);
        }
        const float total = block_sum_256(local, scratch);
        const float inv_rms = __frsqrt_rn(total / static_cast<float>(hidden) + eps);
        __nv_bfloat162 result[4];
#pragma unroll
        for (uint32_t pair = 0; pair < 4; ++pair) {
            const float2 r = __bfloat1622float2(source[pair]);
            if (RESIDUAL) {
                const float2 w = __bfloat1622float2(weight_pairs[pair]);
                result[pair] = __floats2bfloat162_rn(r.x * inv_rms * w.x, r.y * inv_rms * w.y);
            } else {
                result[pair] = __hmul2(__floats2bfloat162_rn(r.x * inv_rms, r.y * inv_rms), weight_pairs[pair]);
            }
        }
        *reinterpret_cast<uint4*>(out + base) = *reinterpret_cast<const uint4*>(result);
        if (codes != nullptr) {
            uint16_t packed[4];
#pragma unroll
            for (uint32_t pair = 0; pair < 4; ++pair) {
                const float2 rounded = __bfloat1622float2(result[pair]);
                asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;"
                    : "=h"(packed[pair])
                    : "f"(rounded.x * code_scale), "f"(rounded.y * code_scale));
            }
            *reinterpret_cast<uint2*>(codes + base) = *reinterpret_cast<const uint2*>(packed);
        }
        return;
    }
    pdl_wait();
    if (row >= rows) {
        return;
    }
    const __nv_bfloat16* x_row = x + row * hidden;
    float local = 0.0f;
    for (size_t index = threadIdx.x * 2; index < hidden; index += blockDim.x * 2) {
        // hidden is even for every model shape; odd sizes are rejected by the caller
        float2 value = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x_row + index));
        if (RESIDUAL) {
            const float2 add = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(update + row * hidden + index));
            value.x += add.x;
            value.y += add.y;
            *reinterpret_cast<__nv_bfloat162*>(residual_out + row * hidden + index) =
                __floats2bfloat162_rn(value.x, value.y);
        }
        local = fmaf(value.x, value.x, local);
        local = fmaf(value.y, value.y, local);
    }
    const float total = block_sum_256(local, scratch);
    const float inv_rms = __frsqrt_rn(total / static_cast<float>(hidden) + eps);
    const __nv_bfloat16* normal_source = RESIDUAL ? residual_out + row * hidden : x_row;
    for (size_t index = threadIdx.x * 2; index < hidden; index += blockDim.x * 2) {
        const __nv_bfloat162 raw = *reinterpret_cast<const __nv_bfloat162*>(normal_source + index);
        const __nv_bfloat162 scale = *reinterpret_cast<const __nv_bfloat162*>(weight + index);
        const float2 value = __bfloat1622float2(raw);
        __nv_bfloat162 result;
        if (RESIDUAL) {
            const float2 w = __bfloat1622float2(scale);
            result = __floats2bfloat162_rn(value.x * inv_rms * w.x, value.y * inv_rms * w.y);
        } else {
            result = __hmul2(__floats2bfloat162_rn(value.x * inv_rms, value.y * inv_rms), scale);
        }
        *reinterpret_cast<__nv_bfloat162*>(out + row * hidden + index) = result;
        if (codes != nullptr) {
            const float2 rounded = __bfloat1622float2(result);
            uint16_t pair;
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;"
                : "=h"(pair)
                : "f"(rounded.x * code_scale), "f"(rounded.y * code_scale));
            *reinterpret_cast<uint16_t*>(codes + row * hidden + index) = pair;
        }
    }
}

// Decode step of the gated depthwise convolution (width 3): one new token per sequence.
//   projected[t] = [b | c | x] (3 * hidden);  gated = b * x;
//   y = c * (w0 * s0 + w1 * s1 + w2 * gated);  state <- (s1, gated), all per channel, fp32 math on bf16 storage.
__global__ void __launch_bounds__(kRowThreads)
short_conv_decode_kernel(const __nv_bfloat16* __restrict__ projected, const __nv_bfloat16* __restrict__ weight,
                         __nv_bfloat16* __restrict__ states, const uint32_t* __restrict__ request_slots,
                         __nv_bfloat16* __restrict__ output, size_t num_tokens, size_t hidden,
                         size_t num_request_slots) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t work = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (work >= num_tokens * hidden) {
        return;
    }
    const size_t token = work / hidden;
    const size_t channel = work % hidden;
    const size_t slot = request_slots[token];
    if (slot >= num_request_slots) {
        return;
    }
    __nv_bfloat162* state = reinterpret_cast<__nv_bfloat162*>(states) + slot * hidden + channel;
    const float2 previous = __bfloat1622float2(*state);
    const float w0 = __bfloat162float(weight[channel * 3]);
    const float w1 = __bfloat162float(weight[channel * 3 + 1]);
    const float w2 = __bfloat162float(weight[channel * 3 + 2]);
    const size_t base = token * hidden * 3;
    const float b = __bfloat162float(projected[base + channel]);
    const float c = __bfloat162float(projected[base + hidden + channel]);
    const float x = __bfloat162float(projected[base + hidden * 2 + channel]);
    const float gated = b * x;
    const float convolved = w0 * previous.x + w1 * previous.y + w2 * gated;
    output[token * hidden + channel] = __float2bfloat16_rn(c * convolved);
    *state = __floats2bfloat162_rn(previous.y, gated);
}

// Sortable key of one logit: larger key wins.  Ties resolve to the smaller (column % 256), then the smaller
// (column / 256); NaN and -inf map to 0 and never win; +0 and -0 are equal (kernels/sampling.cu:101-134).
__device__ __forceinline__ uint32_t argmax_key(uint16_t bits, uint32_t column) {
    const uint16_t magnitude = bits & 0x7fffu;
    if (magnitude > 0x7f80u || bits == 0xff80u) {
        return 0u;
    }
    if (magnitude == 0u) {
        bits = 0u;
    }
    const uint16_t ordered = (bits & 0x8000u) ? static_cast<uint16_t>(~bits) : static_cast<uint16_t>(bits ^ 0x8000u);
    return (static_cast<uint32_t>(ordered) << 16) | ((0xffu - (column & 0xffu)) << 8) | (0xffu - (column >> 8));
}

// Greedy sampling over one row per CTA, in two passes so that the per-element work is one packed instruction each:
// pass 1 finds the row's largest value with bf16x2 maxima (NaN never wins: maxNum semantics), pass 2 forms the
// tie-ordered key only for the few elements that equal it.  A row of 8 * kArgmaxThreads * kArgmaxBatch values
// (65536: the model's vocabulary) is loaded once, all loads in flight together, and stays in registers for pass 2;
// other lengths re-read the row in pass 2.
constexpr uint32_t kArgmaxThreads = 1024;
constexpr uint32_t kArgmaxBatch = 8;

__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t word) {
    return *reinterpret_cast<const __nv_bfloat162*>(&word);
}

__device__ __forceinline__ __nv_bfloat162 max_of_vector(const uint4& raw, __nv_bfloat162 running) {
    running = __hmax2(running, as_bf162(raw.x));
    running = __hmax2(running, as_bf162(raw.y));
    running = __hmax2(running, as_bf162(raw.z));
    return __hmax2(running, as_bf162(raw.w));
}

// keys of the elements of one 8-value vector that equal `wanted` (both halves hold the row maximum)
__device__ __forceinline__ uint32_t keys_of_matches(const uint4& raw, size_t vector, __nv_bfloat162 wanted,
                                                    uint32_t best) {
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (uint32_t pair = 0; pair < 4; ++pair) {
        const unsigned mask = __heq2_mask(as_bf162(words[pair]), wanted);
        if (mask != 0u) {
            const uint32_t column = static_cast<uint32_t>(vector) * 8 + pair * 2;
            if (mask & 0xffffu) {
                best = max(best, argmax_key(static_cast<uint16_t>(words[pair] & 0xffffu), column));
            }
            if (mask >> 16) {
                best = max(best, argmax_key(static_cast<uint16_t>(words[pair] >> 16), column + 1));
            }
        }
    }
    return best;
}

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_rows_kernel(const __nv_bfloat16* __restrict__ logits, uint32_t* __restrict__ sampled, size_t rows,
                   size_t vocab) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ uint32_t warp_best[32];
    __shared__ uint32_t warp_max[32];
    const size_t row = blockIdx.x;
    if (row >= rows) {
        return;
    }
    const uint16_t* row_bits = reinterpret_cast<const uint16_t*>(logits) + row * vocab;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t warps = blockDim.x >> 5;
    uint32_t best = 0;
    if (vocab % 8 == 0) {
        const uint4* vectors = reinterpret_cast<const uint4*>(row_bits);
        const size_t count = vocab / 8;
        const bool resident = count == static_cast<size_t>(kArgmaxBatch) * blockDim.x;
        const __nv_bfloat16 lowest = __ushort_as_bfloat16(static_cast<unsigned short>(0xff80u));   // -inf
        __nv_bfloat162 running = __halves2bfloat162(lowest, lowest);
        uint4 raw[kArgmaxBatch];
        if (resident) {
#pragma unroll
            for (uint32_t index = 0; index < kArgmaxBatch; ++index) {
                raw[index] = __ldg(vectors + threadIdx.x + index * blockDim.x);
            }
#pragma unroll
            for (uint32_t index = 0; index < kArgmaxBatch; ++index) {
                running = max_of_vector(raw[index], running);
            }
        } else {
            for (size_t vector = threadIdx.x; vector < count; vector += blockDim.x) {
                running = max_of_vector(__ldg(vectors + vector), running);
            }
        }
        // the row's maximum: thread -> warp -> CTA
        __nv_bfloat16 top = __hmax(__low2bfloat16(running), __high2bfloat16(running));
#pragma unroll
        for (uint32_t delta = 16; delta > 0; delta >>= 1) {
            const unsigned short other = __shfl_xor_sync(0xffffffffu, __bfloat16_as_ushort(top), delta);
            top = __hmax(top, __ushort_as_bfloat16(other));
        }
        if (lane == 0) {
            warp_max[warp] = __bfloat16_as_ushort(top);
        }
        __syncthreads();
        top = __ushort_as_bfloat16(static_cast<unsigned short>(warp_max[lane < warps ? lane : 0]));
#pragma unroll
        for (uint32_t delta = 16; delta > 0; delta >>= 1) {
            const unsigned short other = __shfl_xor_sync(0xffffffffu, __bfloat16_as_ushort(top), delta);
            top = __hmax(top, __ushort_as_bfloat16(other));
        }
        const __nv_bfloat162 wanted = __halves2bfloat162(top, top);
        if (resident) {
#pragma unroll
            for (uint32_t index = 0; index < kArgmaxBatch; ++index) {
                best = keys_of_matches(raw[index], threadIdx.x + index * blockDim.x, wanted, best);
            }
        } else {
            for (size_t vector = threadIdx.x; vector < count; vector += blockDim.x) {
                best = keys_of_matches(__ldg(vectors + vector), vector, wanted, best);
            }
        }
    } else {
        for (size_t column = threadIdx.x; column < vocab; column += blockDim.x) {
            best = max(best, argmax_key(row_bits[column], static_cast<uint32_t>(column)));
        }
    }
#pragma unroll
    for (uint32_t delta = 16; delta > 0; delta >>= 1) {
        best = max(best, __shfl_xor_sync(0xffffffffu, best, delta));
    }
    if (lane == 0) {
        warp_best[warp] = best;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < warps ? warp_best[threadIdx.x] : 0u;
#pragma unroll
        for (uint32_t delta = 16; delta > 0; delta >>= 1) {
            best = max(best, __shfl_xor_sync(0xffffffffu, best, delta));
        }
        if (threadIdx.x == 0) {
            // key 0: every logit was NaN or -inf; the legacy kernel then answers column 0
            sampled[row] = best == 0u ? 0u : (((0xffu - (best & 0xffu)) << 8) | (0xffu - ((best >> 8) & 0xffu)));
        }
    }
}

// Step metadata on the device.  For token t of the batch: physical_slot = table[slot][pos / 16] * 16 + pos % 16
// (src/model/lfm2_base.rs:371-378), or -1 when the request slot, the position or the table entry is not valid
// (the append kernels skip negative slots).  With `advance` the kernel first moves every sequence on by one
// token: token id <- the id sampled by the previous step, position <- position + 1.  No host round trip.
// How many entries of `held` come before (`mine`, `index`) in descending order of value, ties by index.  `held` is
// 16-byte aligned and padded with zeros up to a multiple of four entries: a zero behind the batch is never larger
// than a value and never has a smaller index, so it is not counted.
__device__ __forceinline__ uint32_t rank_descending(const uint32_t* held, uint32_t count, uint32_t index,
                                                    uint32_t mine) {
    uint32_t rank = 0;
    const uint4* quads = reinterpret_cast<const uint4*>(held);
    const uint32_t groups = (count + 3) / 4;
#pragma unroll 4
    for (uint32_t group = 0; group < groups; ++group) {
        const uint4 q = quads[group];
        const uint32_t base = group * 4;
        rank += (q.x > mine || (q.x == mine && base + 0 < index)) ? 1u : 0u;
        rank += (q.y > mine || (q.y == mine && base + 1 < index)) ? 1u : 0u;
        rank += (q.z > mine || (q.z == mine && base + 2 < index)) ? 1u : 0u;
        rank += (q.w > mine || (q.w == mine && base + 3 < index)) ? 1u : 0u;
    }
    return rank;
}

__global__ void __launch_bounds__(kRowThreads)
decode_metadata_kernel(uint32_t* __restrict__ token_ids, uint32_t* __restrict__ positions,
                       const uint32_t* __restrict__ request_slots, const uint32_t* __restrict__ block_tables,
                       const uint32_t* __restrict__ sampled, int64_t* __restrict__ physical_slots, size_t num_tokens,
                       size_t block_table_stride, size_t block_table_rows, size_t num_pages, uint32_t advance,
                       uint32_t* __restrict__ token_order) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) uint32_t step_positions[kRowThreads];
    const size_t token = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    uint32_t position = 0;
    if (token < num_tokens) {
        position = positions[token];
        if (advance) {
            position += 1;
            positions[token] = position;
            token_ids[token] = sampled[token];
        }
        const size_t row = request_slots[token];
        int64_t slot = -1;
        const size_t page_index = position / kPageSize;
        if (row < block_table_rows && page_index < block_table_stride) {
            const uint32_t page = block_tables[row * block_table_stride + page_index];
            if (page < num_pages) {
                slot = static_cast<int64_t>(page) * kPageSize + position % kPageSize;
            }
        }
        physical_slots[token] = slot;
    }
    // Optional (single-CTA launches only): the tokens ordered by context length, longest first, for the attention
    // kernel to hand its CTAs out in -- rank by counting, at most 256 x 256 comparisons.
    if (token_order != nullptr && gridDim.x == 1) {
        step_positions[threadIdx.x] = position;      // 0 beyond the batch: never counted (see rank_descending)
        __syncthreads();
        if (token < num_tokens) {
            token_order[rank_descending(step_positions, static_cast<uint32_t>(num_tokens), threadIdx.x, position)] =
                static_cast<uint32_t>(token);
        }
    }
}

// order[r] = index of the token with the r-th largest position (ties: lower index first).  One CTA; the positions sit
// in shared memory and every thread ranks its tokens by counting.
constexpr uint32_t kOrderThreads = 1024;
__global__ void __launch_bounds__(kOrderThreads)
context_order_kernel(const uint32_t* __restrict__ positions, uint32_t num_tokens, uint32_t* __restrict__ order) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) uint32_t held[kMaxOrderTokens];
    for (uint32_t token = threadIdx.x; token < ((num_tokens + 3) & ~3u); token += blockDim.x) {
        held[token] = token < num_tokens ? positions[token] : 0u;
    }
    __syncthreads();
    for (uint32_t token = threadIdx.x; token < num_tokens; token += blockDim.x) {
        order[rank_descending(held, num_tokens, token, held[token])] = token;
    }
}

}  // namespace

// Gated short convolution over token segments (prefill chunks and decode tokens in one batch), the reference's
// short_conv_segmented_lfm2_bf16 (kernels/short_conv.cu:100-143) without its loop over the tokens of a segment:
// the "state" it carries is just the gated inputs g = b * x of the two previous tokens, kept unrounded inside a
// segment, so y[t] = c[t] * (w0 g[t-2] + w1 g[t-1] + w2 g[t]) can be evaluated per token, operation for operation.
// One CTA per token.  Only a segment's first two tokens need the stored state and only its first token's CTA
// touches it: that CTA produces y for offsets 0 and 1 and then stores the new state (the gated inputs of the
// segment's last two tokens, rounded to bf16), so no CTA reads a state another one writes.
__global__ void __launch_bounds__(kRowThreads)
short_conv_segmented_kernel(const __nv_bfloat16* __restrict__ projected, const __nv_bfloat16* __restrict__ weight,
                            __nv_bfloat16* __restrict__ states, const uint32_t* __restrict__ segment_offsets,
                            const uint32_t* __restrict__ segment_slots, __nv_bfloat16* __restrict__ output,
                            size_t num_tokens, size_t num_segments, size_t hidden, size_t num_request_slots) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t token = blockIdx.x;
    if (token >= num_tokens) {
        return;
    }
    size_t begin = 0;
    size_t end = 0;
    size_t slot = num_request_slots;
    for (size_t segment = 0; segment < num_segments; ++segment) {
        const size_t first = segment_offsets[segment];
        const size_t last = segment_offsets[segment + 1];
        if (token >= first && token < last) {
            begin = first;
            end = last < num_tokens ? last : num_tokens;
            slot = segment_slots[segment];
            break;
        }
    }
    if (slot >= num_request_slots) {
        return;   // not in any segment, or a slot beyond the state table: the reference skips the segment
    }
    const size_t offset = token - begin;
    if (offset == 1) {
        return;   // produced by the CTA of the segment's first token
    }
    const size_t row = hidden * 3;
    for (size_t channel = threadIdx.x; channel < hidden; channel += blockDim.x) {
        const float w0 = __bfloat162float(weight[channel * 3]);
        const float w1 = __bfloat162float(weight[channel * 3 + 1]);
        const float w2 = __bfloat162float(weight[channel * 3 + 2]);
        auto gated_at = [&](size_t at) {
            return __bfloat162float(projected[at * row + channel]) * __bfloat162float(projected[at * row + 2 * hidden + channel]);
        };
        auto gate_at = [&](size_t at) { return __bfloat162float(projected[at * row + hidden + channel]); };
        if (offset >= 2) {
            const float convolved = w0 * gated_at(token - 2) + w1 * gated_at(token - 1) + w2 * gated_at(token);
            output[token * hidden + channel] = __float2bfloat16_rn(gate_at(token) * convolved);
            continue;
        }
        __nv_bfloat162* state = reinterpret_cast<__nv_bfloat162*>(states) + slot * hidden + channel;
        const float2 previous = __bfloat1622float2(*state);
        const float g0 = gated_at(token);
        output[token * hidden + channel] = __float2bfloat16_rn(gate_at(token) * (w0 * previous.x + w1 * previous.y + w2 * g0));
        float state0 = previous.y;
        float state1 = g0;
        if (token + 1 < end) {
            const float g1 = gated_at(token + 1);
            output[(token + 1) * hidden + channel] =
                __float2bfloat16_rn(gate_at(token + 1) * (w0 * previous.y + w1 * g0 + w2 * g1));
            state0 = g0;
            state1 = g1;
            if (token + 2 < end) {
                state0 = gated_at(end - 2);
                state1 = gated_at(end - 1);
            }
        }
        *state = __floats2bfloat162_rn(state0, state1);
    }
}

// Row gather (kernels/gather.cu): output[r] = input[row_indices[r]]; an index beyond the input leaves the row as is.
__global__ void __launch_bounds__(kRowThreads)
gather_rows_kernel(const __nv_bfloat16* __restrict__ input, const uint32_t* __restrict__ row_indices,
                   __nv_bfloat16* __restrict__ output, size_t output_rows, size_t input_rows, size_t columns) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = blockIdx.x;
    if (row >= output_rows) {
        return;
    }
    const size_t source = row_indices[row];
    if (source >= input_rows) {
        return;
    }
    const uint32_t* from = reinterpret_cast<const uint32_t*>(input + source * columns);
    uint32_t* to = reinterpret_cast<uint32_t*>(output + row * columns);
    for (size_t pair = threadIdx.x; pair < columns / 2; pair += blockDim.x) {
        to[pair] = from[pair];
    }
}

cudaError_t launch_embedding_bf16(cudaStream_t stream, const uint32_t* token_ids, const void* table, void* out,
                                  size_t num_tokens, size_t vocab_size, size_t hidden) {
    return launch_kernel(embedding_kernel, static_cast<unsigned int>(num_tokens), kRowThreads, 0, stream, 1, token_ids,
                         static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), num_tokens,
                         vocab_size, hidden);
}

cudaError_t launch_rms_norm_bf16(cudaStream_t stream, const void* x, const void* weight, void* out, size_t rows,
                                 size_t hidden, float eps) {
    return launch_kernel(rms_norm_kernel<false>, static_cast<unsigned int>(rows), kRowThreads, 0, stream, 1, 
        static_cast<const __nv_bfloat16*>(x), nullptr, static_cast<const __nv_bfloat16*>(weight), nullptr,
        static_cast<__nv_bfloat16*>(out), static_cast<uint8_t*>(nullptr), 1.0f, rows, hidden, eps);
}

cudaError_t launch_residual_rms_norm_bf16(cudaStream_t stream, const void* residual, const void* update,
                                          const void* weight, void* residual_out, void* normalized_out, size_t rows,
                                          size_t hidden, float eps, void* codes, float code_scale) {
    return launch_kernel(rms_norm_kernel<true>, static_cast<unsigned int>(rows), kRowThreads, 0, stream, 1, 
        static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(update),
        static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(residual_out),
        static_cast<__nv_bfloat16*>(normalized_out), static_cast<uint8_t*>(codes), code_scale, rows, hidden, eps);
}

cudaError_t launch_short_conv_decode(cudaStream_t stream, const void* projected, const void* weight, void* states,
                                     const uint32_t* request_slots, void* output, size_t num_tokens, size_t hidden,
                                     size_t num_request_slots) {
    const size_t work = num_tokens * hidden;
    return launch_kernel(short_conv_decode_kernel, static_cast<unsigned int>((work + kRowThreads - 1) / kRowThreads), kRowThreads, 0, stream, 1, static_cast<const __nv_bfloat16*>(projected),
                                         static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(states),
                                         request_slots, static_cast<__nv_bfloat16*>(output), num_tokens, hidden,
                                         num_request_slots);
}

cudaError_t launch_argmax_rows_bf16(cudaStream_t stream, const void* logits, uint32_t* sampled, size_t rows,
                                    size_t vocab) {
    return launch_kernel(argmax_rows_kernel, static_cast<unsigned int>(rows), kArgmaxThreads, 0, stream, 1, 
        static_cast<const __nv_bfloat16*>(logits), sampled, rows, vocab);
}

cudaError_t launch_decode_metadata(cudaStream_t stream, uint32_t* token_ids, uint32_t* positions,
                                   const uint32_t* request_slots, const uint32_t* block_tables, const uint32_t* sampled,
                                   int64_t* physical_slots, size_t num_tokens, size_t block_table_stride,
                                   size_t block_table_rows, size_t num_pages, bool advance, uint32_t* token_order) {
    const unsigned int blocks = static_cast<unsigned int>((num_tokens + kRowThreads - 1) / kRowThreads);
    return launch_kernel(decode_metadata_kernel, blocks, kRowThreads, 0, stream, 1, token_ids, positions,
                         request_slots, block_tables, sampled, physical_slots, num_tokens, block_table_stride,
                         block_table_rows, num_pages, advance ? 1u : 0u, blocks == 1 ? token_order : nullptr);
}

cudaError_t launch_context_order(cudaStream_t stream, const uint32_t* positions, size_t num_tokens, uint32_t* order) {
    if (num_tokens == 0 || num_tokens > kMaxOrderTokens) {
        return cudaErrorInvalidValue;
    }
    return launch_kernel(context_order_kernel, 1, kOrderThreads, 0, stream, 1, positions,
                         static_cast<uint32_t>(num_tokens), order);
}

cudaError_t launch_short_conv_segmented(cudaStream_t stream, const void* projected, const void* weight, void* states,
                                        const uint32_t* segment_offsets, const uint32_t* segment_slots, void* output,
                                        size_t num_tokens, size_t num_segments, size_t hidden,
                                        size_t num_request_slots) {
    return launch_kernel(short_conv_segmented_kernel, static_cast<unsigned int>(num_tokens), kRowThreads, 0, stream, 1,
                         static_cast<const __nv_bfloat16*>(projected), static_cast<const __nv_bfloat16*>(weight),
                         static_cast<__nv_bfloat16*>(states), segment_offsets, segment_slots,
                         static_cast<__nv_bfloat16*>(output), num_tokens, num_segments, hidden, num_request_slots);
}

cudaError_t launch_gather_rows_bf16(cudaStream_t stream, const void* input, const uint32_t* row_indices, void* output,
                                    size_t output_rows, size_t input_rows, size_t columns) {
    return launch_kernel(gather_rows_kernel, static_cast<unsigned int>(output_rows), kRowThreads, 0, stream, 1,
                         static_cast<const __nv_bfloat16*>(input), row_indices, static_cast<__nv_bfloat16*>(output),
                         output_rows, input_rows, columns);
}

}  // namespace lfm25
