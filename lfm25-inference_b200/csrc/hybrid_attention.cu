// Attention of a mixed prefill / decode step over the paged KV cache ("hybrid ragged attention").
//
// Replaces the reference's hybrid_ragged_gqa_lfm2_bf16_ps16 (kernels/attention.cu:389-585, launched from
// src/cuda/kernels/attention.rs:131-226): token t of the segment [begin, end) that contains it, at offset
// o = t - begin and position p, attends to the p - o tokens of its sequence that are already in the paged cache
// (found through block_tables[request_slots[t]]) and to the tokens begin..t of the step's own contiguous K/V.
// The reference runs one CTA per (token, KV head) and re-reads every key for every token; here one CTA owns a
// tile of 16 consecutive tokens of one segment and one KV head, so a key is staged once per 16 tokens x 4 heads:
//
//   warp 4      producer: one thread walks the tile's key range -- pages of the cached prefix, then 16-token slabs
//               of the step's own K/V -- and issues TMA tile loads (128-byte swizzle, mbarrier complete_tx) into a
//               ring of 3 stages of 64 keys shared by the CTA; a stage is refilled once the four compute warps have
//               released it
//   warps 0-3   4 tokens x 4 query heads each = the 16 rows of one mma.sync.m16n8k16 tile; per stage S = Q K^T
//               (32 MMAs), causal mask per row, one online-softmax update in the exp2 domain for the 64 keys with
//               two rows per thread, O += P V (32 MMAs)
//
// With current_key == nullptr the kernel reads every key up to each token's position from the cache (the caller
// appended the step's K/V first, which is what the decode executor's fused append does); with it, the prefix comes
// from the cache and the segment's own tokens from the contiguous buffers, as in the reference.
//
// Conventions kept from the reference: a token whose position is smaller than its offset, or whose key range
// meets a block-table entry >= num_pages, is left untouched.  Narrower than the reference: the tokens of a tile
// must sit at consecutive positions of one request slot (what GpuBatch::update_segments produces,
// src/scheduler/batch.rs:142-215); a token that does not continue its tile's first token is left untouched too.
// Every mbarrier wait is bounded; a wait that runs out is recorded in the device status words and the CTA
// stores nothing.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "launch.h"
#include "tensor_map.h"

namespace lfm25 {

namespace {

constexpr uint32_t kTileTokens = 16;
constexpr uint32_t kComputeWarps = 4;
constexpr uint32_t kHybridThreads = (kComputeWarps + 1) * 32;
constexpr uint32_t kHybridStages = 3;
constexpr uint32_t kSubTiles = 4;                            // 16-key tiles per stage: softmax works on 64 keys
constexpr uint32_t kSlabBytes = kPageSize * kHeadDim * 2;   // one K or V tile: 16 keys x 128 B
constexpr uint32_t kSubTileBytes = 2 * kSlabBytes;          // K tile then V tile
constexpr uint32_t kHybridStageBytes = kSubTiles * kSubTileBytes;
constexpr uint32_t kHybridSmem = kHybridStages * kHybridStageBytes + 2 * kHybridStages * 8 + 16 + 1024;

struct HybridParams {
    const __nv_bfloat16* query;
    __nv_bfloat16* output;
    const uint32_t* block_tables;
    const uint32_t* request_slots;
    const uint32_t* position_ids;
    const uint32_t* segment_offsets;
    unsigned int* status;
    uint64_t block_table_stride;
    uint64_t block_table_rows;
    uint32_t num_tokens;
    uint32_t num_pages;
    uint32_t num_segments;
    uint32_t query_token_stride;
    uint32_t contiguous_current;   // 1: the segment's own K/V come from the contiguous buffers
};

__global__ void __launch_bounds__(kHybridThreads, 3)
hybrid_ragged_attention_kernel(const __grid_constant__ CUtensorMap key_map, const __grid_constant__ CUtensorMap value_map,
                               const __grid_constant__ CUtensorMap current_key_map,
                               const __grid_constant__ CUtensorMap current_value_map, const HybridParams p) {
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();

    // ---- which (segment, 16-token tile, KV head) this CTA owns; every early exit is CTA-uniform ----
    // Later tiles of a segment (and, in a typical batch, later segments) have longer key ranges: the grid is walked
    // backwards so that the long CTAs start first and the short ones fill the tail.
    const uint32_t kv_head = blockIdx.x % kKvHeads;
    uint32_t tile_slot = (gridDim.x - 1 - blockIdx.x) / kKvHeads;
    uint32_t segment_begin = 0;
    uint32_t segment_end = 0;
    bool found = false;
    for (uint32_t segment = 0; segment < p.num_segments; ++segment) {
        const uint32_t begin = __ldg(p.segment_offsets + segment);
        const uint32_t end = __ldg(p.segment_offsets + segment + 1);
        if (end <= begin || end > p.num_tokens) {
            continue;
        }
        const uint32_t tiles = (end - begin + kTileTokens - 1) / kTileTokens;
        if (tile_slot < tiles) {
            segment_begin = begin;
            segment_end = end;
            found = true;
            break;
        }
        tile_slot -= tiles;
    }
    if (!found) {
        return;
    }
    const uint32_t tile_begin = segment_begin + tile_slot * kTileTokens;
    const uint32_t tile_end = min(tile_begin + kTileTokens, segment_end);
    const uint32_t first_offset = tile_begin - segment_begin;
    const uint32_t first_position = p.position_ids[tile_begin];
    if (first_position < first_offset) {
        return;   // no token of this tile can be consistent with it
    }
    const uint32_t prefix = first_position - first_offset;   // tokens of the sequence cached before this step
    const uint64_t table_row = p.request_slots[tile_begin];
    const uint32_t last_offset = tile_end - 1 - segment_begin;
    const uint64_t last_position = static_cast<uint64_t>(prefix) + last_offset;
    if (table_row >= p.block_table_rows || last_position >= p.block_table_stride * kPageSize) {
        return;
    }
    const uint32_t* __restrict__ table = p.block_tables + table_row * p.block_table_stride;

    // key tiles: `paged_tiles` pages through the block table, then `current_tiles` slabs of the step's own K/V
    const uint32_t paged_keys = p.contiguous_current ? prefix : static_cast<uint32_t>(last_position) + 1;
    const uint32_t paged_tiles = (paged_keys + kPageSize - 1) / kPageSize;
    const uint32_t current_tiles = p.contiguous_current ? last_offset / kPageSize + 1 : 0;
    const uint32_t total_tiles = paged_tiles + current_tiles;
    const uint32_t macro_tiles = (total_tiles + kSubTiles - 1) / kSubTiles;   // stages of up to 64 keys

    extern __shared__ uint8_t hybrid_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(hybrid_smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t ring = smem_u32(smem);
    const uint32_t bar_full = ring + kHybridStages * kHybridStageBytes;
    const uint32_t bar_empty = bar_full + kHybridStages * 8;
    volatile uint32_t* flags = reinterpret_cast<volatile uint32_t*>(smem + kHybridStages * kHybridStageBytes +
                                                                    2 * kHybridStages * 8);   // [0] bad, [1] abort
    if (threadIdx.x == 0) {
        flags[0] = 0;
        flags[1] = 0;
        for (uint32_t stage = 0; stage < kHybridStages; ++stage) {
            mbar_init(bar_full + stage * 8, 1);
            mbar_init(bar_empty + stage * 8, kComputeWarps);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncthreads();

    if (warp == kComputeWarps) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            const int32_t head_row = static_cast<int32_t>(kv_head * kPageSize);
            for (uint32_t macro = 0; macro < macro_tiles; ++macro) {
                const uint32_t stage = macro % kHybridStages;
                if (macro >= kHybridStages) {
                    if (flags[1] || !mbar_wait_bounded(bar_empty + stage * 8, ((macro / kHybridStages) - 1) & 1)) {
                        if (!flags[1]) {
                            flags[1] = 1;
                            record_wait_timeout(p.status, kTagHybridAttention, (blockIdx.x << 1) | 1);
                        }
                        break;
                    }
                    fence_proxy_async_smem();
                }
                const uint32_t bar = bar_full + stage * 8;
                const uint32_t first_tile = macro * kSubTiles;
                const uint32_t count = min(kSubTiles, total_tiles - first_tile);
                mbar_arrive_expect_tx(bar, count * kSubTileBytes);
                for (uint32_t sub = 0; sub < count; ++sub) {
                    const uint32_t tile = first_tile + sub;
                    const uint32_t dst = ring + stage * kHybridStageBytes + sub * kSubTileBytes;
                    if (tile < paged_tiles) {
                        uint32_t entry = __ldg(table + tile);
                        if (entry >= p.num_pages) {
                            flags[0] = 1;   // unassigned page: keep the pipeline uniform, discard the result
                            entry = 0;
                        }
                        const int32_t row =
                            static_cast<int32_t>(entry) * static_cast<int32_t>(kKvHeads * kPageSize) + head_row;
                        tma_load_2d(dst, &key_map, bar, 0, row);
                        tma_load_2d(dst + kSlabBytes, &value_map, bar, 0, row);
                    } else {
                        // rows past the last token of the step are filled with zeros by the copy engine
                        const int32_t token_row =
                            static_cast<int32_t>(segment_begin + (tile - paged_tiles) * kPageSize);
                        const int32_t column = static_cast<int32_t>(kv_head * kHeadDim);
                        tma_load_2d(dst, &current_key_map, bar, column, token_row);
                        tma_load_2d(dst + kSlabBytes, &current_value_map, bar, column, token_row);
                    }
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- compute warps
        const uint32_t group = lane >> 2;   // accumulator rows group and group + 8
        const uint32_t quad = lane & 3;
        const uint32_t head = group & 3;
        // row -> token: rows 4j..4j+3 are the heads of the warp's j-th token
        uint32_t row_token[2];
        int64_t row_position[2];   // last key (index in the sequence) the row may see
        bool row_live[2];
        uint32_t warp_last_position = 0;
        bool warp_live = false;
#pragma unroll
        for (uint32_t half = 0; half < 2; ++half) {
            const uint32_t token = tile_begin + warp * 4 + (group >> 2) + half * 2;
            row_token[half] = token;
            bool live = token < tile_end;
            if (live) {
                // the token must continue the tile's first token: same request slot, consecutive position
                live = p.request_slots[token] == table_row &&
                       p.position_ids[token] == prefix + (token - segment_begin);
            }
            row_live[half] = live;
            row_position[half] = live ? static_cast<int64_t>(prefix) + (token - segment_begin)
                                      : static_cast<int64_t>(last_position);
        }
        {
            const uint32_t warp_first = tile_begin + warp * 4;
            if (warp_first < tile_end) {
                warp_live = true;
                warp_last_position = prefix + (min(warp_first + 4, tile_end) - 1 - segment_begin);
            }
        }

        uint32_t qa[4][4];
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) {
            qa[ks][0] = qa[ks][1] = qa[ks][2] = qa[ks][3] = 0;
        }
#pragma unroll
        for (uint32_t half = 0; half < 2; ++half) {
            if (row_token[half] < tile_end) {
                const __nv_bfloat16* q_row = p.query + static_cast<size_t>(row_token[half]) * p.query_token_stride +
                                             (kv_head * kQPerKv + head) * kHeadDim;
#pragma unroll
                for (uint32_t ks = 0; ks < 4; ++ks) {
                    qa[ks][half] = *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + quad * 2);
                    qa[ks][half + 2] = *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + 8 + quad * 2);
                }
            }
        }

        constexpr float kScaleLog2 = kAttnScale * kLog2e;
        float running_max[2] = {-INFINITY, -INFINITY};   // in units of the raw dot product
        float running_sum[2] = {0.0f, 0.0f};             // this thread's share; reduced over the quad at the end
        float acc[8][4];
#pragma unroll
        for (uint32_t nt = 0; nt < 8; ++nt) {
            acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
        }
        const uint32_t ld_matrix = lane >> 3;
        const uint32_t ld_row = lane & 7;
        const uint32_t k_token = ((ld_matrix >> 1) << 3) + ld_row;
        const uint32_t k_chunk = ld_matrix & 1;
        const uint32_t v_token = ((ld_matrix & 1) << 3) + ld_row;
        const uint32_t v_chunk = ld_matrix >> 1;

        bool timed_out = false;
        uint32_t failed_macro = 0;
        for (uint32_t macro = 0; macro < macro_tiles; ++macro) {
            const uint32_t stage = macro % kHybridStages;
            const bool ready = !flags[1] && mbar_wait_bounded(bar_full + stage * 8, (macro / kHybridStages) & 1);
            if (!__all_sync(0xffffffffu, ready)) {
                timed_out = true;
                failed_macro = macro;
                break;
            }
            const uint32_t stage_base = ring + stage * kHybridStageBytes;
            const uint32_t first_tile = macro * kSubTiles;
            const uint32_t count = min(kSubTiles, total_tiles - first_tile);
            bool wrote_stage = false;

            // index in the sequence of a tile's first key, and the last key of the tile that exists at all
            auto tile_first_key = [&](uint32_t tile) -> int64_t {
                return tile < paged_tiles ? static_cast<int64_t>(tile) * kPageSize
                                          : static_cast<int64_t>(prefix) + (tile - paged_tiles) * kPageSize;
            };
            auto tile_last_key = [&](uint32_t tile) -> int64_t {
                return tile < paged_tiles ? static_cast<int64_t>(paged_keys) - 1 : static_cast<int64_t>(last_position);
            };
            // The common stage -- four tiles, every key of them exists and the warp sees all four -- runs with
            // compile-time trip counts, so that the MMAs of the four tiles (eight independent accumulator chains)
            // are interleaved; the edge stages take the same code with per-tile tests.
            const uint32_t last_tile = first_tile + kSubTiles - 1;
            const bool fast = count == kSubTiles && warp_live &&
                              tile_first_key(last_tile) <= static_cast<int64_t>(warp_last_position) &&
                              tile_last_key(first_tile) >= tile_first_key(first_tile) + kPageSize - 1 &&
                              tile_last_key(last_tile) >= tile_first_key(last_tile) + kPageSize - 1 &&
                              (first_tile >= paged_tiles || last_tile < paged_tiles ||
                               tile_last_key(paged_tiles - 1) >= tile_first_key(paged_tiles - 1) + kPageSize - 1);

            float s[2 * kSubTiles][4];
            bool used[kSubTiles];
            auto scores = [&](auto fast_tag) {
                constexpr bool kFast = decltype(fast_tag)::value;
#pragma unroll
                for (uint32_t sub = 0; sub < kSubTiles; ++sub) {
                    const uint32_t tile = first_tile + sub;
                    used[sub] = kFast || (sub < count && warp_live &&
                                          tile_first_key(tile) <= static_cast<int64_t>(warp_last_position));
#pragma unroll
                    for (uint32_t nt = 0; nt < 2; ++nt) {
                        const float fill = used[sub] ? 0.0f : -INFINITY;
                        s[sub * 2 + nt][0] = s[sub * 2 + nt][1] = s[sub * 2 + nt][2] = s[sub * 2 + nt][3] = fill;
                    }
                    if (!kFast && used[sub]) {
                        const int64_t first_key = tile_first_key(tile);
                        const int64_t tile_limit = tile_last_key(tile);
                        if (tile_limit < first_key + kPageSize - 1) {
                            // Keys past the limit do not exist (or are not this tile's to read): their V rows may
                            // hold anything, so clear them; every warp does it for itself before its own reads.
                            wrote_stage = true;
                            const uint32_t v_base = stage_base + sub * kSubTileBytes + kSlabBytes;
                            for (int64_t row = tile_limit - first_key + 1; row < kPageSize; ++row) {
                                asm volatile("st.shared.u32 [%0], %1;" ::"r"(v_base + static_cast<uint32_t>(row) * 128 + lane * 4),
                                             "r"(0u) : "memory");
                            }
                        }
                    }
                }
#pragma unroll
                for (uint32_t ks = 0; ks < 4; ++ks) {
#pragma unroll
                    for (uint32_t sub = 0; sub < kSubTiles; ++sub) {
                        if (kFast || used[sub]) {
                            uint32_t b0, b1, b2, b3;
                            const uint32_t chunk = ks * 2 + k_chunk;
                            ldmatrix_x4(stage_base + sub * kSubTileBytes + k_token * 128 + ((chunk ^ ld_row) << 4), b0, b1,
                                        b2, b3);
                            mma_bf16_16816(s[sub * 2], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                            mma_bf16_16816(s[sub * 2 + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
                        }
                    }
                }
                // causal mask: row r sees key k iff k <= min(row position, last key of the tile)
#pragma unroll
                for (uint32_t sub = 0; sub < kSubTiles; ++sub) {
                    if (kFast || used[sub]) {
                        const uint32_t tile = first_tile + sub;
                        const int64_t first_key = tile_first_key(tile);
                        const int64_t tile_limit = kFast ? first_key + kPageSize - 1 : tile_last_key(tile);
#pragma unroll
                        for (uint32_t half = 0; half < 2; ++half) {
                            const int64_t limit = row_position[half] < tile_limit ? row_position[half] : tile_limit;
                            if (limit < first_key + kPageSize - 1) {
#pragma unroll
                                for (uint32_t nt = 0; nt < 2; ++nt) {
                                    const int64_t key = first_key + nt * 8 + quad * 2;
                                    if (key > limit) s[sub * 2 + nt][half * 2] = -INFINITY;
                                    if (key + 1 > limit) s[sub * 2 + nt][half * 2 + 1] = -INFINITY;
                                }
                            }
                        }
                    }
                }
            };
            if (fast) {
                scores(std::true_type{});
            } else {
                scores(std::false_type{});
            }
            if (wrote_stage) {
                __syncwarp();
            }

            // ---- online softmax over the stage's keys, two rows per thread ----
            uint32_t pa[kSubTiles][4];
            float rescale[2];
#pragma unroll
            for (uint32_t half = 0; half < 2; ++half) {
                float maximum = -INFINITY;
#pragma unroll
                for (uint32_t nt = 0; nt < 2 * kSubTiles; ++nt) {
                    maximum = fmaxf(maximum, fmaxf(s[nt][half * 2], s[nt][half * 2 + 1]));
                }
                maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, 1));
                maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, 2));
                const float new_max = fmaxf(running_max[half], maximum);
                const float base = new_max == -INFINITY ? 0.0f : new_max;   // a row that has seen no key yet
                rescale[half] = fast_exp2((running_max[half] - base) * kScaleLog2);
                const float offset = -base * kScaleLog2;
                float tile_sum = 0.0f;
#pragma unroll
                for (uint32_t sub = 0; sub < kSubTiles; ++sub) {
                    pa[sub][half] = pack_bf16x2(fast_exp2(fmaf(s[sub * 2][half * 2], kScaleLog2, offset)),
                                                fast_exp2(fmaf(s[sub * 2][half * 2 + 1], kScaleLog2, offset)));
                    pa[sub][half + 2] = pack_bf16x2(fast_exp2(fmaf(s[sub * 2 + 1][half * 2], kScaleLog2, offset)),
                                                    fast_exp2(fmaf(s[sub * 2 + 1][half * 2 + 1], kScaleLog2, offset)));
                    // the denominator sums the same bf16-rounded weights that multiply V
                    const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pa[sub][half]));
                    const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pa[sub][half + 2]));
                    tile_sum += (w0.x + w0.y) + (w1.x + w1.y);
                }
                running_sum[half] = fmaf(running_sum[half], rescale[half], tile_sum);
                running_max[half] = new_max;
            }
#pragma unroll
            for (uint32_t nt = 0; nt < 8; ++nt) {
                acc[nt][0] *= rescale[0];
                acc[nt][1] *= rescale[0];
                acc[nt][2] *= rescale[1];
                acc[nt][3] *= rescale[1];
            }

            // ---- O += P V ----
            auto weighted_values = [&](auto fast_tag) {
                constexpr bool kFast = decltype(fast_tag)::value;
#pragma unroll
                for (uint32_t sub = 0; sub < kSubTiles; ++sub) {
                    if (kFast || used[sub]) {
                        const uint32_t v_base = stage_base + sub * kSubTileBytes + kSlabBytes;
#pragma unroll
                        for (uint32_t pair = 0; pair < 4; ++pair) {
                            uint32_t b0, b1, b2, b3;
                            const uint32_t chunk = pair * 2 + v_chunk;
                            ldmatrix_x4_trans(v_base + v_token * 128 + ((chunk ^ ld_row) << 4), b0, b1, b2, b3);
                            mma_bf16_16816(acc[pair * 2], pa[sub][0], pa[sub][1], pa[sub][2], pa[sub][3], b0, b1);
                            mma_bf16_16816(acc[pair * 2 + 1], pa[sub][0], pa[sub][1], pa[sub][2], pa[sub][3], b2, b3);
                        }
                    }
                }
            };
            if (fast) {
                weighted_values(std::true_type{});
            } else {
                weighted_values(std::false_type{});
            }
            if (wrote_stage) {
                fence_proxy_async_smem();   // the stage is refilled by the copy engine after plain stores to it
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_empty + stage * 8);
            }
        }
        if (timed_out) {
            // give the copies still in flight a bounded chance to land before the shared memory is released
            for (uint32_t pending = failed_macro; pending < macro_tiles && pending < failed_macro + kHybridStages;
                 ++pending) {
                (void)mbar_wait_bounded(bar_full + (pending % kHybridStages) * 8, (pending / kHybridStages) & 1);
            }
            if (lane == 0 && !flags[1]) {
                flags[1] = 1;
                record_wait_timeout(p.status, kTagHybridAttention, blockIdx.x << 1);
            }
        }

        __syncthreads();   // the producer has issued (or given up on) every tile; flags are final
        if (flags[0] == 0 && flags[1] == 0) {
#pragma unroll
            for (uint32_t half = 0; half < 2; ++half) {
                float sum = running_sum[half];
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if (row_live[half]) {
                    const float inverse = 1.0f / sum;
                    __nv_bfloat16* out_row = p.output + (static_cast<size_t>(row_token[half]) * kQHeads +
                                                         kv_head * kQPerKv + head) * kHeadDim;
#pragma unroll
                    for (uint32_t nt = 0; nt < 8; ++nt) {
                        *reinterpret_cast<uint32_t*>(out_row + nt * 8 + quad * 2) =
                            pack_bf16x2(acc[nt][half * 2] * inverse, acc[nt][half * 2 + 1] * inverse);
                    }
                }
            }
        }
        return;
    }
    __syncwarp();      // the producer ran its loop on one lane: whole warps reach the CTA barrier
    __syncthreads();   // producer warp: matches the barrier of the compute warps
}

}  // namespace

cudaError_t launch_hybrid_ragged_attention(cudaStream_t stream, const HybridAttentionLaunch& launch) {
    CUtensorMap key_map;
    CUtensorMap value_map;
    CUtensorMap current_key_map;
    CUtensorMap current_value_map;
    const uint64_t cache_rows = static_cast<uint64_t>(launch.num_pages) * kKvHeads * kPageSize;
    if (!make_swizzled_2d_map(&key_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, launch.key_cache, cache_rows,
                              kHeadDim * 2, kPageSize) ||
        !make_swizzled_2d_map(&value_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, launch.value_cache, cache_rows,
                              kHeadDim * 2, kPageSize)) {
        return cudaErrorInvalidValue;
    }
    const bool contiguous = launch.current_key != nullptr;
    if (contiguous) {
        if (!make_swizzled_2d_map_width(&current_key_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, launch.current_key,
                                        launch.num_tokens, kKvHeads * kHeadDim, launch.kv_token_stride * 2,
                                        kPageSize) ||
            !make_swizzled_2d_map_width(&current_value_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                        launch.current_value, launch.num_tokens, kKvHeads * kHeadDim,
                                        launch.kv_token_stride * 2, kPageSize)) {
            return cudaErrorInvalidValue;
        }
    } else {
        current_key_map = key_map;
        current_value_map = value_map;
    }
    const cudaError_t attribute_status = cudaFuncSetAttribute(
        hybrid_ragged_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kHybridSmem));
    if (attribute_status != cudaSuccess) {
        return attribute_status;
    }
    HybridParams params;
    params.query = static_cast<const __nv_bfloat16*>(launch.query);
    params.output = static_cast<__nv_bfloat16*>(launch.output);
    params.block_tables = launch.block_tables;
    params.request_slots = launch.request_slots;
    params.position_ids = launch.position_ids;
    params.segment_offsets = launch.segment_offsets;
    params.status = launch.status;
    params.block_table_stride = launch.block_table_stride;
    params.block_table_rows = launch.block_table_rows;
    params.num_tokens = static_cast<uint32_t>(launch.num_tokens);
    params.num_pages = static_cast<uint32_t>(launch.num_pages);
    params.num_segments = static_cast<uint32_t>(launch.num_segments);
    params.query_token_stride = static_cast<uint32_t>(launch.query_token_stride);
    params.contiguous_current = contiguous ? 1u : 0u;
    // at most floor(T / 16) + S tiles of 16 tokens cover S segments with T tokens in total
    const uint64_t tiles = launch.num_tokens / kTileTokens + launch.num_segments;
    return launch_kernel(hybrid_ragged_attention_kernel, static_cast<unsigned int>(tiles * kKvHeads), kHybridThreads,
                         kHybridSmem, stream, 1, key_map, value_map, current_key_map, current_value_map, params);
}

}  // namespace lfm25
