// Attention of a mixed prefill / decode step on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// Same function as hybrid_attention.cu (the reference's hybrid_ragged_gqa_lfm2_bf16_ps16, kernels/attention.cu:389-585)
// for segments long enough to fill a 128-row MMA: one CTA owns 32 consecutive tokens of one segment and one KV head,
// i.e. 32 tokens x 4 query heads = the 128 rows of a tcgen05.mma tile.
//
//   warp 0      producer: the Q tile (one 3-D TMA copy: 64 dims x 4 heads x 32 tokens) and then the key range in stages
//               of 64 keys (4 pages, or 4 slabs of the step's own K/V), K rows then V rows, 128-byte swizzle
//   warp 1      allocates 256 TMEM columns; one thread issues, per stage, S = Q K^T (4 x tcgen05.mma kind::f16, both
//               operands K-major from shared memory, fp32 accumulator S in TMEM) and, once the softmax warps have put
//               the weights back, PV = P V (one MMA per 16 keys: A = bf16 P read from TMEM, B = the V rows as an
//               MN-major operand -- the page layout [key][dim] needs no transposition).  S / P and PV are double
//               buffered in TMEM and S of the next stage is issued before this stage's weights are awaited, so the
//               tensor core works while the softmax warps do
//   warps 2-5   one thread per row: tcgen05.ld S (two passes: row maximum, then weights), causal mask, exp2 online
//               softmax without any shuffle, bf16 P written over the S columns it came from with tcgen05.st, and
//               O (64 fp32 registers per thread) <- (O + PV of the previous stage) * rescale, one stage late, so that
//               the PV product is never waited for
//
// Keys that do not exist or may not be read are masked by assignment, and their V rows are cleared in shared memory
// before the PV MMA (a zero weight times a stale NaN pattern is NaN).  Every mbarrier wait is bounded; a wait that
// runs out raises an abort flag that every role polls, is recorded in the device status words, and the CTA still
// frees its TMEM and stores nothing.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "launch.h"
#include "tcgen05.cuh"
#include "tensor_map.h"

namespace lfm25 {

namespace {

constexpr uint32_t kTokensPerTile = 32;
constexpr uint32_t kTileRows = kTokensPerTile * kQPerKv;     // 128 = UMMA M
constexpr uint32_t kUmmaThreads = 192;
constexpr uint32_t kUmmaStages = 4;
constexpr uint32_t kPagesPerStage = 4;                       // 64 keys per stage
constexpr uint32_t kPageBytes = kPageSize * kHeadDim * 2;    // one K or V tile of 16 keys: 2048 B
constexpr uint32_t kHalfStageBytes = kPagesPerStage * kPageBytes;   // the K rows (or the V rows) of a stage
constexpr uint32_t kStageBytesUmma = 2 * kHalfStageBytes;
constexpr uint32_t kQBytes = kTileRows * kHeadDim * 2;       // 16 KiB
constexpr uint32_t kUmmaSmem = kQBytes + kUmmaStages * kStageBytesUmma + 256 + 1024;
constexpr uint32_t kTmemColumns = 256;
constexpr uint32_t kColumnS = 0;      // two buffers of 64 fp32 columns; the bf16 P of a stage overwrites the first
                                      // 32 columns of the S buffer it was computed from
constexpr uint32_t kColumnPV = 128;   // two buffers of 64 fp32 columns

struct UmmaAttentionParams {
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
    uint32_t contiguous_current;
};

// D[tmem] (+)= A[smem] * B[smem], bf16 operands
__device__ __forceinline__ void umma_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem], bf16 operands
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tensor_map, uint32_t bar, int32_t x, int32_t y,
                                            int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__global__ void __launch_bounds__(kUmmaThreads, 2)
hybrid_attention_umma_kernel(const __grid_constant__ CUtensorMap query_map, const __grid_constant__ CUtensorMap key_map,
                             const __grid_constant__ CUtensorMap value_map,
                             const __grid_constant__ CUtensorMap current_key_map,
                             const __grid_constant__ CUtensorMap current_value_map, const UmmaAttentionParams p) {
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();

    // ---- which (segment, 32-token tile, KV head); later tiles have longer key ranges, so the grid runs backwards ----
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
        const uint32_t tiles = (end - begin + kTokensPerTile - 1) / kTokensPerTile;
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
    const uint32_t tile_begin = segment_begin + tile_slot * kTokensPerTile;
    const uint32_t tile_end = min(tile_begin + kTokensPerTile, segment_end);
    const uint32_t first_offset = tile_begin - segment_begin;
    const uint32_t first_position = p.position_ids[tile_begin];
    if (first_position < first_offset) {
        return;
    }
    const uint32_t prefix = first_position - first_offset;
    const uint64_t table_row = p.request_slots[tile_begin];
    const uint32_t last_offset = tile_end - 1 - segment_begin;
    const uint64_t last_position = static_cast<uint64_t>(prefix) + last_offset;
    if (table_row >= p.block_table_rows || last_position >= p.block_table_stride * kPageSize) {
        return;
    }
    const uint32_t* __restrict__ table = p.block_tables + table_row * p.block_table_stride;
    const uint32_t paged_keys = p.contiguous_current ? prefix : static_cast<uint32_t>(last_position) + 1;
    const uint32_t paged_tiles = (paged_keys + kPageSize - 1) / kPageSize;
    const uint32_t current_tiles = p.contiguous_current ? last_offset / kPageSize + 1 : 0;
    const uint32_t total_tiles = paged_tiles + current_tiles;
    const uint32_t macro_tiles = (total_tiles + kPagesPerStage - 1) / kPagesPerStage;

    extern __shared__ uint8_t umma_attention_smem[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(umma_attention_smem) + 1023) & ~uintptr_t(1023));
    const uint32_t q_base = smem_u32(smem);
    const uint32_t ring = q_base + kQBytes;
    uint8_t* control = smem + kQBytes + kUmmaStages * kStageBytesUmma;
    const uint32_t bar_full = smem_u32(control);
    const uint32_t bar_empty = bar_full + 8 * kUmmaStages;
    const uint32_t bar_q = bar_empty + 8 * kUmmaStages;
    const uint32_t bar_s = bar_q + 8;      // [2]: S of an even / odd stage is complete
    const uint32_t bar_p = bar_s + 16;     // [2]: its weights are in TMEM
    const uint32_t bar_pv = bar_p + 16;    // [2]: its PV product is complete
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(control + 8 * (2 * kUmmaStages + 7));
    volatile uint32_t* flags = tmem_slot + 1;   // [0] unassigned page met, [1] abort

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&query_map);
        tma_prefetch_descriptor(&key_map);
        tma_prefetch_descriptor(&value_map);
        for (uint32_t stage = 0; stage < kUmmaStages; ++stage) {
            mbar_init(bar_full + 8 * stage, 1);
            mbar_init(bar_empty + 8 * stage, 1);
        }
        mbar_init(bar_q, 1);
        for (uint32_t buffer = 0; buffer < 2; ++buffer) {
            mbar_init(bar_s + 8 * buffer, 1);
            mbar_init(bar_p + 8 * buffer, 4);
            mbar_init(bar_pv + 8 * buffer, 1);
        }
        flags[0] = 0;
        flags[1] = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_allocate(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemColumns);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto tile_first_key = [&](uint32_t tile) -> int64_t {
        return tile < paged_tiles ? static_cast<int64_t>(tile) * kPageSize
                                  : static_cast<int64_t>(prefix) + (tile - paged_tiles) * kPageSize;
    };
    auto tile_last_key = [&](uint32_t tile) -> int64_t {
        return tile < paged_tiles ? static_cast<int64_t>(paged_keys) - 1 : static_cast<int64_t>(last_position);
    };

    if (warp == 0) {
        // ------------------------------------------------------------------------------------ producer
        if (lane == 0) {
            mbar_arrive_expect_tx(bar_q, kQBytes);
            tma_load_3d(q_base, &query_map, bar_q, 0, static_cast<int32_t>(kv_head * kQPerKv),
                        static_cast<int32_t>(tile_begin));
            const int32_t head_row = static_cast<int32_t>(kv_head * kPageSize);
            for (uint32_t macro = 0; macro < macro_tiles; ++macro) {
                const uint32_t stage = macro % kUmmaStages;
                if (macro >= kUmmaStages) {
                    if (flags[1] || !mbar_wait_bounded(bar_empty + 8 * stage, ((macro / kUmmaStages) - 1) & 1)) {
                        if (!flags[1]) {
                            flags[1] = 1;
                            record_wait_timeout(p.status, kTagHybridAttention, (blockIdx.x << 2) | 1);
                        }
                        break;
                    }
                }
                const uint32_t bar = bar_full + 8 * stage;
                const uint32_t first_tile = macro * kPagesPerStage;
                const uint32_t count = min(kPagesPerStage, total_tiles - first_tile);
                // block-table entries first: an unassigned page is flagged before anything of the stage is
                // announced, and page 0 is read in its place so that the pipeline stays uniform
                uint32_t entries[kPagesPerStage];
#pragma unroll
                for (uint32_t sub = 0; sub < kPagesPerStage; ++sub) {
                    entries[sub] = 0;
                    if (sub < count && first_tile + sub < paged_tiles) {
                        entries[sub] = __ldg(table + first_tile + sub);
                        if (entries[sub] >= p.num_pages) {
                            flags[0] = 1;
                            entries[sub] = 0;
                        }
                    }
                }
                mbar_arrive_expect_tx(bar, count * 2 * kPageBytes);
#pragma unroll
                for (uint32_t sub = 0; sub < kPagesPerStage; ++sub) {
                    if (sub >= count) {
                        continue;
                    }
                    const uint32_t tile = first_tile + sub;
                    const uint32_t k_dst = ring + stage * kStageBytesUmma + sub * kPageBytes;
                    const uint32_t v_dst = k_dst + kHalfStageBytes;
                    if (tile < paged_tiles) {
                        const int32_t row =
                            static_cast<int32_t>(entries[sub]) * static_cast<int32_t>(kKvHeads * kPageSize) + head_row;
                        tma_load_2d(k_dst, &key_map, bar, 0, row);
                        tma_load_2d(v_dst, &value_map, bar, 0, row);
                    } else {
                        const int32_t token_row =
                            static_cast<int32_t>(segment_begin + (tile - paged_tiles) * kPageSize);
                        const int32_t column = static_cast<int32_t>(kv_head * kHeadDim);
                        tma_load_2d(k_dst, &current_key_map, bar, column, token_row);
                        tma_load_2d(v_dst, &current_value_map, bar, column, token_row);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptors: D = f32, A = B = bf16, M = 128; QK^T: both K-major, N = keys of the stage;
            // PV: B (the V rows) MN-major, N = 64 dims
            const uint32_t idesc_common = (1u << 4) | (1u << 7) | (1u << 10) | ((kTileRows >> 4) << 24);
            const uint32_t idesc_pv = idesc_common | (1u << 16) | ((kHeadDim >> 3) << 17);
            bool ok = !flags[1] && mbar_wait_bounded(bar_q, 0);
            if (!ok && !flags[1]) {
                flags[1] = 1;
                record_wait_timeout(p.status, kTagHybridAttention, (blockIdx.x << 2) | 2);
            }
            const uint64_t q_desc = smem_descriptor(q_base);
            // S = Q K^T of one stage into S buffer (macro & 1); needs the stage's K rows
            auto issue_scores = [&](uint32_t macro) -> bool {
                const uint32_t stage = macro % kUmmaStages;
                const uint32_t count = min(kPagesPerStage, total_tiles - macro * kPagesPerStage);
                if (flags[1] || !mbar_wait_bounded(bar_full + 8 * stage, (macro / kUmmaStages) & 1)) {
                    return false;
                }
                tcgen05_fence_after();
                const uint64_t k_desc = smem_descriptor(ring + stage * kStageBytesUmma);
                const uint32_t idesc_qk = idesc_common | (((count * kPageSize) >> 3) << 17);
                const uint32_t target = tmem_base + kColumnS + (macro & 1) * 64;
#pragma unroll
                for (uint32_t ks = 0; ks < 4; ++ks) {   // 16 dims = 32 bytes inside the swizzle row per step
                    umma_bf16_ss(target, q_desc + ks * 2, k_desc + ks * 2, idesc_qk, ks);
                }
                umma_commit(bar_s + 8 * (macro & 1));
                return true;
            };
            ok = ok && macro_tiles > 0 && issue_scores(0);
            for (uint32_t macro = 0; macro < macro_tiles && ok; ++macro) {
                const uint32_t stage = macro % kUmmaStages;
                const uint32_t count = min(kPagesPerStage, total_tiles - macro * kPagesPerStage);
                const uint32_t buffer = macro & 1;
                // the next stage's scores first: the tensor core computes them while this stage's softmax runs.
                // Their buffer is free: its previous weights were consumed by the PV product issued before, and MMAs
                // execute in issue order.
                if (macro + 1 < macro_tiles && !issue_scores(macro + 1)) {
                    ok = false;
                    break;
                }
                if (flags[1] || !mbar_wait_bounded(bar_p + 8 * buffer, (macro >> 1) & 1)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint64_t v_desc = smem_descriptor(ring + stage * kStageBytesUmma + kHalfStageBytes);
                for (uint32_t step = 0; step < count; ++step) {   // 16 keys per step: 8 packed columns of P, 2 KiB of V
                    umma_bf16_ts(tmem_base + kColumnPV + buffer * 64, tmem_base + kColumnS + buffer * 64 + step * 8,
                                 v_desc + step * (kPageBytes >> 4), idesc_pv, step);
                }
                umma_commit(bar_pv + 8 * buffer);
                umma_commit(bar_empty + 8 * stage);
            }
            if (!ok && !flags[1]) {
                flags[1] = 1;
                record_wait_timeout(p.status, kTagHybridAttention, (blockIdx.x << 2) | 3);
            }
        }
    } else {
        // ------------------------------------------------------------------------------------ softmax / output
        const uint32_t quadrant = warp & 3;                 // the TMEM lanes this warp may touch
        const uint32_t row = quadrant * 32 + lane;
        const uint32_t token = tile_begin + (row >> 2);
        const uint32_t head = row & 3;
        bool live = token < tile_end;
        if (live) {
            live = p.request_slots[token] == table_row && p.position_ids[token] == prefix + (token - segment_begin);
        }
        const int64_t row_position = live ? static_cast<int64_t>(prefix) + (token - segment_begin)
                                          : static_cast<int64_t>(last_position);
        const uint32_t lane_address = tmem_base + ((quadrant * 32) << 16);
        const uint32_t softmax_thread = threadIdx.x - 64;   // 0..127, for cooperative shared-memory writes
        constexpr float kScaleLog2 = kAttnScale * kLog2e;
        float running_max = -INFINITY;
        float running_sum = 0.0f;
        float out[kHeadDim];
#pragma unroll
        for (uint32_t dim = 0; dim < kHeadDim; ++dim) {
            out[dim] = 0.0f;
        }
        bool ok = true;
        // O <- (O + PV of stage `macro`) * factor: the PV product is folded in one stage late
        auto fold = [&](uint32_t macro, float factor) -> bool {
            const bool ready = !flags[1] && mbar_wait_bounded(bar_pv + 8 * (macro & 1), (macro >> 1) & 1);
            if (!__all_sync(0xffffffffu, ready)) {
                return false;
            }
            tcgen05_fence_after();
            const uint32_t source = lane_address + kColumnPV + (macro & 1) * 64;
            const bool unchanged = __all_sync(0xffffffffu, factor == 1.0f);   // no row of this warp moved its maximum
#pragma unroll
            for (uint32_t half = 0; half < 2; ++half) {
                uint32_t raw[2][16];
                tmem_load16_nowait(source + half * 32, raw[0]);
                tmem_load16_nowait(source + half * 32 + 16, raw[1]);
                tmem_load_wait();
                if (unchanged) {
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) {
                        out[half * 32 + j] += __uint_as_float(raw[j >> 4][j & 15]);
                    }
                } else {
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) {
                        out[half * 32 + j] = (out[half * 32 + j] + __uint_as_float(raw[j >> 4][j & 15])) * factor;
                    }
                }
            }
            return true;
        };
        for (uint32_t macro = 0; macro < macro_tiles; ++macro) {
            const uint32_t stage = macro % kUmmaStages;
            const uint32_t first_tile = macro * kPagesPerStage;
            const uint32_t count = min(kPagesPerStage, total_tiles - first_tile);
            const uint32_t buffer = macro & 1;
            ok = !flags[1] && mbar_wait_bounded(bar_s + 8 * buffer, (macro >> 1) & 1);
            if (!__all_sync(0xffffffffu, ok)) {
                ok = false;
                break;
            }
            tcgen05_fence_after();
            const uint32_t scores = lane_address + kColumnS + buffer * 64;
            // The common stage: four full tiles of consecutive keys, all of them visible to every row of this warp.
            const int64_t stage_first = tile_first_key(first_tile);
            const bool regular = count == kPagesPerStage &&
                                 tile_first_key(first_tile + kPagesPerStage - 1) == stage_first + 3 * kPageSize &&
                                 tile_last_key(first_tile) >= stage_first + kPageSize - 1 &&
                                 tile_last_key(first_tile + kPagesPerStage - 1) >= stage_first + 4 * kPageSize - 1;
            const bool fast = __all_sync(0xffffffffu, regular && row_position >= stage_first + 4 * kPageSize - 1);
            bool clear_values = false;
            float rescale;
            float new_max;
            float stage_sum = 0.0f;
            if (fast) {
                // four independent chains for the maximum and for the sum: the 64 values of a row would otherwise
                // form one dependent chain per pass
                float lane_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (uint32_t half = 0; half < 2; ++half) {
                    uint32_t raw[2][16];
                    tmem_load16_nowait(scores + half * 32, raw[0]);
                    tmem_load16_nowait(scores + half * 32 + 16, raw[1]);
                    tmem_load_wait();
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) {
                        lane_max[j & 3] = fmaxf(lane_max[j & 3], __uint_as_float(raw[j >> 4][j & 15]));
                    }
                }
                const float maximum = fmaxf(fmaxf(lane_max[0], lane_max[1]), fmaxf(lane_max[2], lane_max[3]));
                new_max = fmaxf(running_max, maximum);
                rescale = fast_exp2((running_max - new_max) * kScaleLog2);
                const float offset = -new_max * kScaleLog2;
                float lane_sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (uint32_t half = 0; half < 2; ++half) {
                    uint32_t raw[2][16];
                    tmem_load16_nowait(scores + half * 32, raw[0]);
                    tmem_load16_nowait(scores + half * 32 + 16, raw[1]);
                    tmem_load_wait();
                    uint32_t packed[16];
#pragma unroll
                    for (uint32_t j = 0; j < 32; j += 2) {
                        const float w0 = fast_exp2(fmaf(__uint_as_float(raw[j >> 4][j & 15]), kScaleLog2, offset));
                        const float w1 = fast_exp2(fmaf(__uint_as_float(raw[j >> 4][(j & 15) + 1]), kScaleLog2, offset));
                        packed[j / 2] = pack_bf16x2(w0, w1);
                        lane_sum[(j >> 1) & 3] += w0 + w1;   // unrounded here: the rounding of 64 weights averages out
                    }
                    tmem_store16(scores + half * 16, packed);
                }
                stage_sum = (lane_sum[0] + lane_sum[1]) + (lane_sum[2] + lane_sum[3]);
            } else {
            // how many keys of each 16-key tile this row may see (its keys are consecutive from the tile's first)
            int32_t visible[kPagesPerStage];
#pragma unroll
            for (uint32_t sub = 0; sub < kPagesPerStage; ++sub) {
                const uint32_t tile = first_tile + sub;
                const int64_t first = tile_first_key(tile);
                const int64_t exists = sub < count ? tile_last_key(tile) : first - 1;
                const int64_t limit = row_position < exists ? row_position : exists;
                const int64_t seen = limit - first + 1;
                visible[sub] = seen < 0 ? 0 : (seen > static_cast<int64_t>(kPageSize) ? static_cast<int32_t>(kPageSize)
                                                                                      : static_cast<int32_t>(seen));
                clear_values = clear_values || (sub < count && exists < first + kPageSize - 1);
            }
            // pass 1: row maximum of the masked scores
            float maximum = -INFINITY;
#pragma unroll
            for (uint32_t half = 0; half < 2; ++half) {
                uint32_t raw[2][16];
                tmem_load16_nowait(scores + half * 32, raw[0]);
                tmem_load16_nowait(scores + half * 32 + 16, raw[1]);
                tmem_load_wait();
#pragma unroll
                for (uint32_t part = 0; part < 2; ++part) {
#pragma unroll
                    for (uint32_t j = 0; j < 16; ++j) {
                        if (static_cast<int32_t>(j) < visible[half * 2 + part]) {
                            maximum = fmaxf(maximum, __uint_as_float(raw[part][j]));
                        }
                    }
                }
            }
            new_max = fmaxf(running_max, maximum);
            const float base = new_max == -INFINITY ? 0.0f : new_max;
            rescale = fast_exp2((running_max - base) * kScaleLog2);
            const float offset = -base * kScaleLog2;
            // pass 2: weights, rounded to bf16, written over the scores they came from as the A operand of P V
#pragma unroll
            for (uint32_t half = 0; half < 2; ++half) {
                uint32_t raw[2][16];
                tmem_load16_nowait(scores + half * 32, raw[0]);
                tmem_load16_nowait(scores + half * 32 + 16, raw[1]);
                tmem_load_wait();
                uint32_t packed[16];
#pragma unroll
                for (uint32_t part = 0; part < 2; ++part) {
                    const int32_t seen = visible[half * 2 + part];
#pragma unroll
                    for (uint32_t j = 0; j < 16; j += 2) {
                        const float w0 = static_cast<int32_t>(j) < seen
                                             ? fast_exp2(fmaf(__uint_as_float(raw[part][j]), kScaleLog2, offset)) : 0.0f;
                        const float w1 = static_cast<int32_t>(j + 1) < seen
                                             ? fast_exp2(fmaf(__uint_as_float(raw[part][j + 1]), kScaleLog2, offset)) : 0.0f;
                        const uint32_t pair = pack_bf16x2(w0, w1);
                        packed[part * 8 + j / 2] = pair;
                        // the denominator sums the same bf16-rounded weights that multiply V
                        const float2 rounded = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pair));
                        stage_sum += rounded.x + rounded.y;
                    }
                }
                tmem_store16(scores + half * 16, packed);
            }
            }
            tmem_store_wait();
            if (clear_values) {
                // V rows of keys that do not exist (or are not this tile's to read) may hold anything: clear them
                const uint32_t v_base = ring + stage * kStageBytesUmma + kHalfStageBytes;
#pragma unroll
                for (uint32_t sub = 0; sub < kPagesPerStage; ++sub) {
                    const int64_t exists = tile_last_key(first_tile + sub);
                    const int64_t key = tile_first_key(first_tile + sub) + (softmax_thread >> 3);
                    if (sub < count && key > exists) {
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(
                                         v_base + sub * kPageBytes + (softmax_thread >> 3) * 128 + (softmax_thread & 7) * 16),
                                     "r"(0u)
                                     : "memory");
                    }
                }
                fence_proxy_async_smem();
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_p + 8 * buffer);
            }
            // fold in the previous stage's PV product (it was computed with the previous maximum): both it and
            // the accumulator move to the new maximum together
            if (macro > 0) {
                if (!fold(macro - 1, rescale)) {
                    ok = false;
                    break;
                }
            }
            running_sum = fmaf(running_sum, rescale, stage_sum);
            running_max = new_max;
        }
        if (ok && macro_tiles > 0) {
            ok = fold(macro_tiles - 1, 1.0f);
        }
        if (!ok && lane == 0 && !flags[1]) {
            flags[1] = 1;
            record_wait_timeout(p.status, kTagHybridAttention, (blockIdx.x << 2) | 0);
        }
        if (ok && live) {
            // flags[0] is final once the last stage was consumed: the producer raised it before that stage's loads
            if (flags[0] == 0 && flags[1] == 0) {
                const float inverse = 1.0f / running_sum;
                uint4* out_row = reinterpret_cast<uint4*>(p.output + (static_cast<size_t>(token) * kQHeads +
                                                                      kv_head * kQPerKv + head) * kHeadDim);
#pragma unroll
                for (uint32_t chunk = 0; chunk < kHeadDim / 8; ++chunk) {
                    uint4 value;
                    value.x = pack_bf16x2(out[chunk * 8] * inverse, out[chunk * 8 + 1] * inverse);
                    value.y = pack_bf16x2(out[chunk * 8 + 2] * inverse, out[chunk * 8 + 3] * inverse);
                    value.z = pack_bf16x2(out[chunk * 8 + 4] * inverse, out[chunk * 8 + 5] * inverse);
                    value.w = pack_bf16x2(out[chunk * 8 + 6] * inverse, out[chunk * 8 + 7] * inverse);
                    out_row[chunk] = value;
                }
            }
        }
    }

    // the producer and MMA warps ran their loops on one lane: the warp meets again here, so that the CTA barrier
    // below is reached by whole warps (a barrier reached by part of a warp is not defined behaviour, and it was seen
    // to let the early lanes through before the late one arrived)
    __syncwarp();
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_free(tmem_base, kTmemColumns);
    }
}

// 3-D tensor map over the query buffer: (64 dims, 32 heads, T tokens), boxes of (64, 4, 32) with 128-byte swizzle,
// i.e. a shared-memory tile of 128 rows of 128 bytes ordered (token, head).
bool make_query_map(CUtensorMap* map, const void* query, uint64_t num_tokens, uint64_t token_stride_elements) {
    EncodeTiledFn encode = encode_tiled_entry();
    if (encode == nullptr) {
        return false;
    }
    const cuuint64_t dims[3] = {kHeadDim, kQHeads, num_tokens};
    const cuuint64_t strides[2] = {kHeadDim * 2, token_stride_elements * 2};
    const cuuint32_t box[3] = {kHeadDim, kQPerKv, kTokensPerTile};
    const cuuint32_t element_strides[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(query), dims, strides, box,
                  element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t launch_hybrid_attention_umma(cudaStream_t stream, const HybridAttentionLaunch& launch) {
    CUtensorMap query_map;
    CUtensorMap key_map;
    CUtensorMap value_map;
    CUtensorMap current_key_map;
    CUtensorMap current_value_map;
    const uint64_t cache_rows = static_cast<uint64_t>(launch.num_pages) * kKvHeads * kPageSize;
    if (!make_query_map(&query_map, launch.query, launch.num_tokens, launch.query_token_stride) ||
        !make_swizzled_2d_map(&key_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, launch.key_cache, cache_rows,
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
        hybrid_attention_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kUmmaSmem));
    if (attribute_status != cudaSuccess) {
        return attribute_status;
    }
    UmmaAttentionParams params;
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
    params.contiguous_current = contiguous ? 1u : 0u;
    const uint64_t tiles = launch.num_tokens / kTokensPerTile + launch.num_segments;
    return launch_kernel(hybrid_attention_umma_kernel, static_cast<unsigned int>(tiles * kKvHeads), kUmmaThreads,
                         kUmmaSmem, stream, 1, query_map, key_map, value_map, current_key_map, current_value_map,
                         params);
}

}  // namespace lfm25
