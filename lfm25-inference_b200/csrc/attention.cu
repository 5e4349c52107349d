// Ragged paged GQA decode attention for sm_100a.
//
// Replaces the reference's kernels/attention_async_fast.cu (unsplit :72-205, split-K :211-358,
// merge :362-419).  The arithmetic contract is the same -- per token t and query head q,
// O = softmax(0.125 * Q K^T) V over keys 0..=position[t] of KV head q/4, found through
// block_tables[request_slots[t]] -- but the execution model is new:
//
//  * one CTA per (token, KV head[, split]); its 4 warps take the pages of the range
//    round-robin and each warp runs an independent online-softmax stream;
//  * every physical page (16 tokens x 64 dims of K and of V, 2 KiB each) is fetched ONCE per
//    KV head by a TMA tile copy (128-byte swizzle, mbarrier completion, no multicast) into a
//    per-warp ring of shared-memory stages, and is shared by the 4 grouped query heads, which
//    occupy rows 0..3 of the M=16 operand of mma.sync.m16n8k16 (bf16 in, fp32 accumulate);
//  * softmax runs on the accumulator fragments with quad shuffles; the 4 warps are combined
//    through shared memory with the exact log-sum-exp identity, which is also the split-K
//    record format of the reference ((max, denominator, acc[64]) per (token, head, split)).
//
// HBM traffic per CTA is the K/V pages of its range (valid or not, the last page is read whole),
// 512 B of Q, and either 512 B of output or 4 x 264 B of partial records.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "launch.h"
#include "options.h"
#include "qk_norm_rope.cuh"
#include "tensor_map.h"

namespace lfm25 {

namespace {

constexpr uint32_t kWarps = 4;
constexpr uint32_t kThreads = kWarps * 32;
constexpr uint32_t kStages = 4;                        // ring depth per warp
constexpr uint32_t kStageBytes = 2 * kPageTileBytes;   // K tile then V tile
constexpr uint32_t kRingBytes = kStages * kStageBytes; // per warp
constexpr uint32_t kMergeFloats = kWarps * kQPerKv * kPartialStride;
constexpr uint32_t kClusterRecordFloats = kQPerKv * kPartialStride;   // this CTA's four split records, for its cluster
constexpr uint32_t kSmemBytes = kWarps * kRingBytes + kMergeFloats * 4 + kWarps * kStages * 8 + 16 +
                                kClusterRecordFloats * 4;
constexpr uint32_t kSmemAlloc = kSmemBytes + 1024;     // room to align the rings to 1 KiB

struct AttentionParams {
    const __nv_bfloat16* query;
    const uint32_t* block_tables;
    const uint32_t* request_slots;  // nullptr: every token uses block-table row 0
    const uint32_t* position_ids;
    __nv_bfloat16* output;
    float* partials;
    unsigned int* status;
    uint64_t block_table_stride;
    uint64_t block_table_rows;
    uint32_t num_tokens;
    uint32_t num_pages;
    uint32_t num_splits;  // 1: write normalised output; >1: write split records
    uint32_t cluster_merge;   // with num_splits > 1: the splits of a (token, KV head) are one thread-block cluster and
                              // merge through distributed shared memory -- no records in global memory, no merge kernel
    uint32_t query_token_stride;  // elements between tokens of `query` (2048 when dense)
    uint32_t kv_token_stride;     // elements between tokens of key_raw / value_raw (512 when dense)
    // fused mode only: the raw projections of the step and what is needed to turn them into the new cache row
    const __nv_bfloat16* key_raw;     // [T, 8, 64]
    const __nv_bfloat16* value_raw;   // [T, 8, 64]
    const __nv_bfloat16* query_norm;  // [64]
    const __nv_bfloat16* key_norm;    // [64]
    const float* inv_freq;            // [32]
    const int64_t* slot_mapping;      // [T]
    __nv_bfloat16* key_cache;
    __nv_bfloat16* value_cache;
    float eps;
    uint32_t kv_evict_first;  // nonzero: the K/V page loads carry the L2 evict-first hint
    uint32_t selftest_drop;   // self-test of the bounded wait: warp 0 arms its first barrier and issues no copy for it
    uint64_t wait_limit_ns;   // limit of every mbarrier wait
    const uint32_t* token_order;  // optional permutation: which token the r-th group of CTAs takes
};

__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// a float of the same shared-memory offset in the CTA of rank `rank` of this cluster
__device__ __forceinline__ float load_from_cluster_cta(uint32_t local_address, uint32_t rank) {
    uint32_t remote;
    float value;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(value) : "r"(remote));
    return value;
}

// A CTA that has no result for its token (request slot outside the block tables, position outside the row, an
// unassigned page, an append slot that contradicts the block table, a wait that ran out) returns without touching the
// output.  With the KV axis split, it first marks its four records: a negative sum tells the merge kernel that the
// token has no result, and the merge then leaves the token's output row as it was -- whatever an earlier launch left
// in the records is never combined into an output.
__device__ __forceinline__ void mark_no_result(const AttentionParams& p, uint32_t token, uint32_t kv_head,
                                               uint32_t split) {
    if (p.num_splits > 1 && p.cluster_merge == 0 && threadIdx.x < kQPerKv) {
        const size_t q_index = static_cast<size_t>(token) * kQHeads + kv_head * kQPerKv + threadIdx.x;
        float* record = p.partials + (q_index * p.num_splits + split) * kPartialStride;
        record[0] = -INFINITY;
        record[1] = -1.0f;
    }
}

// FUSED == false: the query is already normalised and rotated and the newest K/V row is already in the cache.
// FUSED == true : the kernel takes the raw Q/K/V projections of the step (the reference's one-kernel decode,
//   kernels/attention_fused.cu:89-348): every CTA normalises and rotates its four query heads in registers, and
//   the warp that owns the sequence's last page also normalises and rotates the new key, writes it and the new
//   value into the paged cache, and patches them into its staged copy of that page before using it.  The
//   arithmetic is the stand-alone append kernel's, operation for operation, so both routes give the same bits.
template <bool FUSED>
__global__ void __launch_bounds__(kThreads, 3)
ragged_decode_attention_kernel(const __grid_constant__ CUtensorMap key_map,
                               const __grid_constant__ CUtensorMap value_map, const AttentionParams p) {
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();   // positions, block tables, the query and the newest K/V row all come from earlier kernels

    // ---- which (token, KV head, split) this CTA owns; every early exit is CTA-uniform ----
    const uint32_t splits = p.num_splits;
    const uint32_t split = blockIdx.x % splits;
    const uint32_t item = blockIdx.x / splits;
    const uint32_t kv_head = item % kKvHeads;
    if (item / kKvHeads >= p.num_tokens) {
        return;
    }
    // CTAs start in block order: with an order that lists the longest contexts first the short ones fill the end of
    // the grid, and the last wave does not wait for a few long sequences.  An entry outside the batch is a no-op.
    const uint32_t token = p.token_order != nullptr ? p.token_order[item / kKvHeads] : item / kKvHeads;
    if (token >= p.num_tokens) {
        return;
    }
    uint64_t table_row = 0;
    if (p.request_slots != nullptr) {
        table_row = p.request_slots[token];
        if (table_row >= p.block_table_rows) {
            mark_no_result(p, token, kv_head, split);
            return;
        }
    }
    const uint32_t position = p.position_ids[token];
    if (static_cast<uint64_t>(position) >= p.block_table_stride * kPageSize) {
        mark_no_result(p, token, kv_head, split);
        return;
    }
    const uint32_t* __restrict__ table = p.block_tables + table_row * p.block_table_stride;
    const uint32_t total_pages = position / kPageSize + 1;
    uint32_t first_page = 0;
    uint32_t end_page = total_pages;
    if (splits > 1) {
        first_page = static_cast<uint32_t>(static_cast<uint64_t>(total_pages) * split / splits);
        end_page = static_cast<uint32_t>(static_cast<uint64_t>(total_pages) * (split + 1) / splits);
    }
    uint32_t new_row_offset = 0;
    if (FUSED) {
        // the slot given for the new token must be the one the block table implies, else the whole token is a
        // silent no-op (kernels/attention_fused.cu:131-147)
        const uint32_t current_page = table[total_pages - 1];
        const int64_t slot_value = p.slot_mapping[token];
        if (current_page >= p.num_pages || slot_value < 0) {
            mark_no_result(p, token, kv_head, split);
            return;
        }
        new_row_offset = position % kPageSize;
        if (static_cast<uint64_t>(slot_value) / kPageSize != current_page ||
            static_cast<uint64_t>(slot_value) % kPageSize != new_row_offset) {
            mark_no_result(p, token, kv_head, split);
            return;
        }
    }
    const uint32_t range_pages = end_page - first_page;
    // warp w owns pages first_page + w + 4*i
    const uint32_t my_pages = range_pages > warp ? (range_pages - warp + kWarps - 1) / kWarps : 0;

    // ---- shared memory carve-up ----
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t ring = smem_u32(smem) + warp * kRingBytes;
    float* merge = reinterpret_cast<float*>(smem + kWarps * kRingBytes);
    const uint32_t bars = smem_u32(smem + kWarps * kRingBytes + kMergeFloats * 4) + warp * kStages * 8;
    uint32_t* bad_flag = reinterpret_cast<uint32_t*>(smem + kWarps * kRingBytes + kMergeFloats * 4 + kWarps * kStages * 8);
    float* cluster_records =
        reinterpret_cast<float*>(smem + kWarps * kRingBytes + kMergeFloats * 4 + kWarps * kStages * 8 + 16);

    if (threadIdx.x == 0) {
        *bad_flag = 0;
    }
    if (lane == 0) {
        for (uint32_t stage = 0; stage < kStages; ++stage) {
            mbar_init(bars + stage * 8, 1);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncthreads();

    // ---- producer state (lane 0 only): issue TMA for this warp's pages, kStages ahead ----
    const int32_t head_row = static_cast<int32_t>(kv_head * kPageSize);
    uint32_t bad = 0;
    uint32_t next_entry = 0;
    auto table_entry = [&](uint32_t iteration) -> uint32_t {
        return __ldg(table + first_page + warp + iteration * kWarps);
    };
    // every page is read by exactly one warp of one CTA in a step: mark the stream as the first to leave L2, so
    // that it does not displace the weights that the step's GEMMs have had fetched ahead
    const uint64_t stream_policy = l2_evict_first_policy();
    bool dropped = false;
    auto issue = [&](uint32_t stage, uint32_t entry) {
        if (entry >= p.num_pages) {
            // An unassigned or out-of-range page: keep the pipeline uniform by reading page 0,
            // and discard this CTA's result at the end (the reference CTA returns silently).
            bad = 1;
            entry = 0;
        }
        const int32_t row = static_cast<int32_t>(entry) * static_cast<int32_t>(kKvHeads * kPageSize) + head_row;
        const uint32_t bar = bars + stage * 8;
        const uint32_t dst = ring + stage * kStageBytes;
        mbar_arrive_expect_tx(bar, kStageBytes);
        if (p.selftest_drop != 0 && warp == 0 && !dropped) {
            dropped = true;   // nothing will complete this barrier: the wait below has to run out
            return;
        }
        if (p.kv_evict_first != 0) {
            tma_load_2d_hint(dst, &key_map, bar, 0, row, stream_policy);
            tma_load_2d_hint(dst + kPageTileBytes, &value_map, bar, 0, row, stream_policy);
        } else {
            tma_load_2d(dst, &key_map, bar, 0, row);
            tma_load_2d(dst + kPageTileBytes, &value_map, bar, 0, row);
        }
    };
    if (lane == 0) {
        const uint32_t prologue = my_pages < kStages ? my_pages : kStages;
        uint32_t entries[kStages];
#pragma unroll
        for (uint32_t stage = 0; stage < kStages; ++stage) {
            entries[stage] = stage < prologue ? table_entry(stage) : 0;
        }
#pragma unroll
        for (uint32_t stage = 0; stage < kStages; ++stage) {
            if (stage < prologue) {
                issue(stage, entries[stage]);
            }
        }
        if (my_pages > kStages) {
            next_entry = table_entry(kStages);
        }
    }

    // ---- query fragments: heads of this KV group in rows 0..3 of the A operand ----
    const uint32_t group = lane >> 2;   // accumulator row
    const uint32_t quad = lane & 3;     // column pair within a quad
    uint32_t qa[4][2];
#pragma unroll
    for (uint32_t ks = 0; ks < 4; ++ks) {
        qa[ks][0] = 0;
        qa[ks][1] = 0;
    }
    if (group < kQPerKv) {
        const __nv_bfloat16* q_row =
            p.query + static_cast<size_t>(token) * p.query_token_stride + (kv_head * kQPerKv + group) * kHeadDim;
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) {
            qa[ks][0] = *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + quad * 2);
            qa[ks][1] = *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + 8 + quad * 2);
        }
    }
    if (FUSED) {
        // This lane holds dims d = 16*ks + 8*h + 2*quad + e of head `group`; d and d + 32 (ks and ks + 2) are
        // both here, so RMSNorm + RoPE stay inside the quad.  The sum of squares follows the butterfly of
        // warp_tree_sum level by level (16 and 8 are local, 4 and 2 cross the quad, 1 is local again).
        float raw[4][4];
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) {
            const float2 low = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[ks][0]));
            const float2 high = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[ks][1]));
            raw[ks][0] = low.x;
            raw[ks][1] = low.y;
            raw[ks][2] = high.x;
            raw[ks][3] = high.y;
        }
        float level[2];
#pragma unroll
        for (uint32_t e = 0; e < 2; ++e) {
            // t[l] = fma(x[l], x[l], x[l+32]^2) for l = 2*quad + e + 8*h + 16*b  (b = ks & 1 with ks < 2)
            float t[2][2];
#pragma unroll
            for (uint32_t b = 0; b < 2; ++b) {
#pragma unroll
                for (uint32_t h = 0; h < 2; ++h) {
                    t[b][h] = fmaf(raw[b][2 * h + e], raw[b][2 * h + e], raw[b + 2][2 * h + e] * raw[b + 2][2 * h + e]);
                }
            }
            const float pair0 = t[0][0] + t[1][0];   // level 16: l and l ^ 16
            const float pair1 = t[0][1] + t[1][1];
            level[e] = pair0 + pair1;                // level 8: l and l ^ 8
            level[e] += __shfl_xor_sync(0xffffffffu, level[e], 2);   // level 4: quad ^ 2
            level[e] += __shfl_xor_sync(0xffffffffu, level[e], 1);   // level 2: quad ^ 1
        }
        const float inv_rms = __frsqrt_rn((level[0] + level[1]) * (1.0f / 64.0f) + p.eps);   // level 1
        if (group < kQPerKv) {
            const float position_f = static_cast<float>(position);
#pragma unroll
            for (uint32_t b = 0; b < 2; ++b) {
#pragma unroll
                for (uint32_t h = 0; h < 2; ++h) {
                    __nv_bfloat16 rotated[2][2];   // [e][first / second half]
#pragma unroll
                    for (uint32_t e = 0; e < 2; ++e) {
                        const uint32_t dim = 16 * b + 8 * h + 2 * quad + e;   // < 32
                        float sin_value, cos_value;
                        sincosf(position_f * p.inv_freq[dim], &sin_value, &cos_value);
                        rotate_pair(raw[b][2 * h + e], raw[b + 2][2 * h + e], inv_rms, p.query_norm[dim],
                                    p.query_norm[dim + kHalfDim], sin_value, cos_value, rotated[e][0], rotated[e][1]);
                    }
                    const __nv_bfloat162 first = __halves2bfloat162(rotated[0][0], rotated[1][0]);
                    const __nv_bfloat162 second = __halves2bfloat162(rotated[0][1], rotated[1][1]);
                    qa[b][h] = *reinterpret_cast<const uint32_t*>(&first);
                    qa[b + 2][h] = *reinterpret_cast<const uint32_t*>(&second);
                }
            }
        }
    }

    // fused mode: the warp that owns the last page of the sequence produces the new K/V row
    const bool owns_new_row = FUSED && end_page == total_pages && my_pages > 0 &&
                              (first_page + warp + (my_pages - 1) * kWarps == total_pages - 1);
    __nv_bfloat16 new_key0, new_key1;
    uint32_t new_value = 0;
    if (owns_new_row) {
        const size_t source = static_cast<size_t>(token) * p.kv_token_stride + kv_head * kHeadDim;
        float sin_value, cos_value;
        sincosf(static_cast<float>(position) * p.inv_freq[lane], &sin_value, &cos_value);
        norm_rope(__bfloat162float(p.key_raw[source + lane]), __bfloat162float(p.key_raw[source + lane + kHalfDim]),
                  p.key_norm[lane], p.key_norm[lane + kHalfDim], sin_value, cos_value, p.eps, new_key0, new_key1);
        new_value = reinterpret_cast<const uint32_t*>(p.value_raw + source)[lane];
        const size_t destination =
            ((static_cast<size_t>(table[total_pages - 1]) * kKvHeads + kv_head) * kPageSize + new_row_offset) * kHeadDim;
        p.key_cache[destination + lane] = new_key0;
        p.key_cache[destination + lane + kHalfDim] = new_key1;
        reinterpret_cast<uint32_t*>(p.value_cache + destination)[lane] = new_value;
    }

    constexpr float kScaleLog2 = kAttnScale * kLog2e;
    float running_max = -INFINITY;  // in units of the raw dot product
    float running_sum = 0.0f;       // this thread's share; reduced over the quad at the end
    float acc[8][4];
#pragma unroll
    for (uint32_t nt = 0; nt < 8; ++nt) {
        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    }

    // ldmatrix row/chunk of this lane: matrix = lane / 8, row inside the matrix = lane % 8
    const uint32_t ld_matrix = lane >> 3;
    const uint32_t ld_row = lane & 7;
    const uint32_t k_token = ((ld_matrix >> 1) << 3) + ld_row;  // K: matrices 2,3 are tokens 8..15
    const uint32_t k_chunk = ld_matrix & 1;                     //    matrices 1,3 are the upper 8 dims
    const uint32_t v_token = ((ld_matrix & 1) << 3) + ld_row;   // V: matrices 1,3 are tokens 8..15
    const uint32_t v_chunk = ld_matrix >> 1;                    //    matrices 2,3 are the next 8 dims

    bool timed_out = false;
    uint32_t failed_iteration = 0;
    for (uint32_t iteration = 0; iteration < my_pages; ++iteration) {
        const uint32_t stage = iteration % kStages;
        const uint32_t parity = (iteration / kStages) & 1;
        const uint32_t bar = bars + stage * 8;
        const bool ready = mbar_wait_bounded(bar, parity, p.wait_limit_ns);
        if (!__all_sync(0xffffffffu, ready)) {
            timed_out = true;
            failed_iteration = iteration;
            break;
        }
        const uint32_t k_base = ring + stage * kStageBytes;
        const uint32_t v_base = k_base + kPageTileBytes;
        const uint32_t page = first_page + warp + iteration * kWarps;
        const uint32_t valid = (page + 1 == total_pages) ? (position - page * kPageSize + 1) : kPageSize;

        if (owns_new_row && iteration + 1 == my_pages) {
            // the staged copy of the last page predates (or races with) the cache write above: put the new row in
            const uint32_t row_base = new_row_offset * 128;
            const uint32_t swizzle = new_row_offset & 7;
            const uint32_t byte0 = lane * 2;             // dim lane
            const uint32_t byte1 = (lane + kHalfDim) * 2;
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(k_base + row_base + (((byte0 >> 4) ^ swizzle) << 4) + (byte0 & 15)),
                         "h"(__bfloat16_as_ushort(new_key0)) : "memory");
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(k_base + row_base + (((byte1 >> 4) ^ swizzle) << 4) + (byte1 & 15)),
                         "h"(__bfloat16_as_ushort(new_key1)) : "memory");
            const uint32_t value_byte = lane * 4;
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(v_base + row_base + (((value_byte >> 4) ^ swizzle) << 4) + (value_byte & 15)),
                         "r"(new_value) : "memory");
            __syncwarp();
        }

        // S[head, token] = Q K^T over this page: 2 token tiles x 4 dim steps
        float s[2][4];
#pragma unroll
        for (uint32_t nt = 0; nt < 2; ++nt) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
        }
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) {
            uint32_t b0, b1, b2, b3;
            const uint32_t chunk = ks * 2 + k_chunk;
            ldmatrix_x4(k_base + k_token * 128 + ((chunk ^ ld_row) << 4), b0, b1, b2, b3);
            mma_bf16_16816(s[0], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
            mma_bf16_16816(s[1], qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
        }

        if (valid < kPageSize) {
            // Last page of the sequence: tokens beyond the position do not exist.  Mask their
            // scores and clear their V rows so that stale bits (even NaN patterns) cannot leak.
#pragma unroll
            for (uint32_t nt = 0; nt < 2; ++nt) {
                const uint32_t token_in_page = nt * 8 + quad * 2;
                if (token_in_page >= valid) s[nt][0] = -INFINITY;
                if (token_in_page + 1 >= valid) s[nt][1] = -INFINITY;
            }
            for (uint32_t row = valid; row < kPageSize; ++row) {
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(v_base + row * 128 + lane * 4), "r"(0u) : "memory");
            }
            __syncwarp();
        }

        // online softmax on rows 0..3 (rows 4..7 carry zeros and are ignored later)
        float page_max = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        page_max = fmaxf(page_max, __shfl_xor_sync(0xffffffffu, page_max, 1));
        page_max = fmaxf(page_max, __shfl_xor_sync(0xffffffffu, page_max, 2));
        const float new_max = fmaxf(running_max, page_max);
        const float rescale = fast_exp2((running_max - new_max) * kScaleLog2);
        const float offset = -new_max * kScaleLog2;
        const uint32_t pa0 = pack_bf16x2(fast_exp2(fmaf(s[0][0], kScaleLog2, offset)),
                                         fast_exp2(fmaf(s[0][1], kScaleLog2, offset)));
        const uint32_t pa2 = pack_bf16x2(fast_exp2(fmaf(s[1][0], kScaleLog2, offset)),
                                         fast_exp2(fmaf(s[1][1], kScaleLog2, offset)));
        // The denominator sums the same bf16-rounded weights that multiply V, so that the
        // result stays an exact convex combination of the V rows.
        const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pa0));
        const float2 w2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pa2));
        running_sum = fmaf(running_sum, rescale, (w0.x + w0.y) + (w2.x + w2.y));
        running_max = new_max;
#pragma unroll
        for (uint32_t nt = 0; nt < 8; ++nt) {
            acc[nt][0] *= rescale;
            acc[nt][1] *= rescale;
        }

        // O[head, dim] += P V: 8 dim tiles, one 16-token step
#pragma unroll
        for (uint32_t pair = 0; pair < 4; ++pair) {
            uint32_t b0, b1, b2, b3;
            const uint32_t chunk = pair * 2 + v_chunk;
            ldmatrix_x4_trans(v_base + v_token * 128 + ((chunk ^ ld_row) << 4), b0, b1, b2, b3);
            mma_bf16_16816(acc[pair * 2], pa0, 0u, pa2, 0u, b0, b1);
            mma_bf16_16816(acc[pair * 2 + 1], pa0, 0u, pa2, 0u, b2, b3);
        }

        // refill this stage with the page kStages ahead
        __syncwarp();
        if (lane == 0 && iteration + kStages < my_pages) {
            fence_proxy_async_smem();
            issue(stage, next_entry);
            if (iteration + kStages + 1 < my_pages) {
                next_entry = table_entry(iteration + kStages + 1);
            }
        }
    }

    if (timed_out) {
        // Give the copies still in flight a second, bounded chance to land before this CTA's
        // shared memory is released, then report and discard the result.
        for (uint32_t pending = failed_iteration; pending < my_pages && pending < failed_iteration + kStages;
             ++pending) {
            (void)mbar_wait_bounded(bars + (pending % kStages) * 8, (pending / kStages) & 1, p.wait_limit_ns);
        }
        if (lane == 0) {
            record_wait_timeout(p.status, kTagAttention, blockIdx.x);
            bad = 1;
        }
    }
    if (lane == 0 && bad) {
        atomicOr(bad_flag, 1u);
    }

    // ---- per-warp state -> shared memory (heads 0..3 live in lanes 0..15) ----
    running_sum += __shfl_xor_sync(0xffffffffu, running_sum, 1);
    running_sum += __shfl_xor_sync(0xffffffffu, running_sum, 2);
    if (group < kQPerKv) {
        float* record = merge + (warp * kQPerKv + group) * kPartialStride;
        if (quad == 0) {
            record[0] = running_max * kAttnScale;  // maximum of the scaled scores; -inf if no page
            record[1] = running_sum;
        }
#pragma unroll
        for (uint32_t nt = 0; nt < 8; ++nt) {
            *reinterpret_cast<float2*>(record + 2 + nt * 8 + quad * 2) = make_float2(acc[nt][0], acc[nt][1]);
        }
    }
    __syncthreads();
    const bool failed = *bad_flag != 0;
    if (failed && p.cluster_merge == 0) {
        mark_no_result(p, token, kv_head, split);
        return;
    }
    // (in a cluster a failed CTA goes on: its partners wait for it at the cluster barrier, and its record says
    // "no result")

    // ---- combine the 4 warps: thread = (head, dims lane and lane + 32) ----
    const uint32_t head = warp;
    float maximum = -INFINITY;
#pragma unroll
    for (uint32_t w = 0; w < kWarps; ++w) {
        maximum = fmaxf(maximum, merge[(w * kQPerKv + head) * kPartialStride]);
    }
    float denominator = 0.0f;
    float out0 = 0.0f;
    float out1 = 0.0f;
#pragma unroll
    for (uint32_t w = 0; w < kWarps; ++w) {
        const float* record = merge + (w * kQPerKv + head) * kPartialStride;
        const float part_sum = record[1];
        const float scale = part_sum == 0.0f ? 0.0f : fast_exp2((record[0] - maximum) * kLog2e);
        denominator = fmaf(part_sum, scale, denominator);
        out0 = fmaf(record[2 + lane], scale, out0);
        out1 = fmaf(record[2 + lane + 32], scale, out1);
    }
    const size_t q_index = static_cast<size_t>(token) * kQHeads + kv_head * kQPerKv + head;
    if (splits == 1) {
        __nv_bfloat16* out_row = p.output + q_index * kHeadDim;
        out_row[lane] = __float2bfloat16_rn(out0 / denominator);
        out_row[lane + 32] = __float2bfloat16_rn(out1 / denominator);
    } else if (p.cluster_merge == 0) {
        float* record = p.partials + (q_index * splits + split) * kPartialStride;
        if (lane == 0) {
            record[0] = maximum;
            record[1] = denominator;
        }
        record[2 + lane] = out0;
        record[2 + lane + 32] = out1;
    } else {
        // The `splits` CTAs of this (token, KV head) are one cluster, in split order.  Each leaves its four records in
        // its own shared memory; after the cluster barrier the first CTA reads them through distributed shared memory
        // and merges them with the arithmetic of merge_splitk_kernel, in the same order, so the bits are the same.
        float* mine = cluster_records + head * kPartialStride;
        if (lane == 0) {
            mine[0] = failed ? -INFINITY : maximum;
            mine[1] = failed ? -1.0f : denominator;     // a negative sum: this CTA has no result
        }
        mine[2 + lane] = out0;
        mine[2 + lane + 32] = out1;
        cluster_barrier();
        if (split == 0) {
            // all remote loads first (up to 8 splits x 4 values per thread in flight), the arithmetic after them
            constexpr uint32_t kMaxSplits = 8;
            const uint32_t local = smem_u32(mine);
            float peak[kMaxSplits];
            float sum[kMaxSplits];
            float low[kMaxSplits];
            float high[kMaxSplits];
#pragma unroll
            for (uint32_t other = 0; other < kMaxSplits; ++other) {
                if (other < splits) {
                    peak[other] = load_from_cluster_cta(local, other);
                    sum[other] = load_from_cluster_cta(local + 4, other);
                    low[other] = load_from_cluster_cta(local + (2 + lane) * 4, other);
                    high[other] = load_from_cluster_cta(local + (2 + lane + 32) * 4, other);
                }
            }
            float top = -INFINITY;
            bool no_result = false;
#pragma unroll
            for (uint32_t other = 0; other < kMaxSplits; ++other) {
                if (other < splits) {
                    top = fmaxf(top, peak[other]);
                    no_result = no_result || sum[other] < 0.0f;
                }
            }
            if (!no_result) {
                float total = 0.0f;
                float merged0 = 0.0f;
                float merged1 = 0.0f;
#pragma unroll
                for (uint32_t other = 0; other < kMaxSplits; ++other) {
                    if (other < splits && sum[other] != 0.0f) {
                        const float scale = fast_exp2((peak[other] - top) * kLog2e);
                        total = fmaf(sum[other], scale, total);
                        merged0 = fmaf(low[other], scale, merged0);
                        merged1 = fmaf(high[other], scale, merged1);
                    }
                }
                __nv_bfloat16* out_row = p.output + q_index * kHeadDim;
                out_row[lane] = __float2bfloat16_rn(merged0 / total);
                out_row[lane + 32] = __float2bfloat16_rn(merged1 / total);
            }
        }
        cluster_barrier();     // nobody leaves while the first CTA may still be reading its records
    }
}

// Merge of split records, one CTA per (token, KV head), thread = (head, dims lane, lane+32).
// Same identity as kernels/attention_async_fast.cu:362-419 of the reference.
__global__ void __launch_bounds__(kThreads)
merge_splitk_kernel(const float* __restrict__ partials, __nv_bfloat16* __restrict__ output, uint32_t num_tokens,
                    uint32_t num_splits) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t token = blockIdx.x / kKvHeads;
    const uint32_t kv_head = blockIdx.x % kKvHeads;
    if (token >= num_tokens) {
        return;
    }
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t head = threadIdx.x >> 5;
    const size_t q_index = static_cast<size_t>(token) * kQHeads + kv_head * kQPerKv + head;
    const float* records = partials + q_index * num_splits * kPartialStride;
    float maximum = -INFINITY;
    bool no_result = false;
    for (uint32_t split = 0; split < num_splits; ++split) {
        maximum = fmaxf(maximum, records[split * kPartialStride]);
        no_result = no_result || records[split * kPartialStride + 1] < 0.0f;
    }
    if (no_result) {
        return;   // a CTA of this token gave up (see mark_no_result): the output row stays as it was
    }
    float denominator = 0.0f;
    float out0 = 0.0f;
    float out1 = 0.0f;
    for (uint32_t split = 0; split < num_splits; ++split) {
        const float* record = records + split * kPartialStride;
        const float part_sum = record[1];
        if (part_sum != 0.0f) {     // a split without pages wrote (-inf, 0) and nothing else
            const float scale = fast_exp2((record[0] - maximum) * kLog2e);
            denominator = fmaf(part_sum, scale, denominator);
            out0 = fmaf(record[2 + lane], scale, out0);
            out1 = fmaf(record[2 + lane + 32], scale, out1);
        }
    }
    __nv_bfloat16* out_row = output + q_index * kHeadDim;
    out_row[lane] = __float2bfloat16_rn(out0 / denominator);
    out_row[lane + 32] = __float2bfloat16_rn(out1 / denominator);
}

// Tensor map over an arena: rows = pages * 8 heads * 16 tokens, 64 bf16 (128 bytes) per row,
// one box = one (page, KV head) tile.
bool make_page_map(CUtensorMap* map, const void* cache, uint64_t num_pages) {
    return make_swizzled_2d_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cache, num_pages * kKvHeads * kPageSize,
                                kHeadDim * 2, kPageSize);
}

}  // namespace

cudaError_t launch_ragged_decode_attention(cudaStream_t stream, const AttentionLaunch& launch) {
    CUtensorMap key_map;
    CUtensorMap value_map;
    if (!make_page_map(&key_map, launch.key_cache, launch.num_pages) ||
        !make_page_map(&value_map, launch.value_cache, launch.num_pages)) {
        return cudaErrorInvalidValue;
    }
    const bool fused = launch.key_raw != nullptr;
    auto kernel = fused ? ragged_decode_attention_kernel<true> : ragged_decode_attention_kernel<false>;
    // per launch: the attribute belongs to the current device's copy of the kernel
    const cudaError_t attribute_status =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemAlloc));
    if (attribute_status != cudaSuccess) {
        return attribute_status;
    }
    AttentionParams params;
    params.query = static_cast<const __nv_bfloat16*>(launch.query);
    params.block_tables = launch.block_tables;
    params.request_slots = launch.request_slots;
    params.position_ids = launch.position_ids;
    params.output = static_cast<__nv_bfloat16*>(launch.output);
    params.partials = launch.partials;
    params.status = launch.status;
    params.block_table_stride = launch.block_table_stride;
    params.block_table_rows = launch.block_table_rows;
    params.num_tokens = static_cast<uint32_t>(launch.num_tokens);
    params.num_pages = static_cast<uint32_t>(launch.num_pages);
    params.num_splits = launch.num_splits;
    // No workspace for the split records: the splits of a (token, KV head) run as one thread-block cluster and merge
    // through distributed shared memory (cluster sizes 2, 4 and 8; the callers ask for nothing else without a
    // workspace).
    const bool cluster_merge = launch.num_splits > 1 && launch.partials == nullptr;
    if (cluster_merge && launch.num_splits != 2 && launch.num_splits != 4 && launch.num_splits != 8) {
        return cudaErrorInvalidValue;
    }
    params.cluster_merge = cluster_merge ? 1u : 0u;
    params.query_token_stride = static_cast<uint32_t>(launch.query_token_stride);
    params.kv_token_stride = static_cast<uint32_t>(launch.kv_token_stride);
    params.key_raw = static_cast<const __nv_bfloat16*>(launch.key_raw);
    params.value_raw = static_cast<const __nv_bfloat16*>(launch.value_raw);
    params.query_norm = static_cast<const __nv_bfloat16*>(launch.query_norm);
    params.key_norm = static_cast<const __nv_bfloat16*>(launch.key_norm);
    params.inv_freq = launch.inv_freq;
    params.slot_mapping = launch.slot_mapping;
    params.key_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(launch.key_cache));
    params.value_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(launch.value_cache));
    params.eps = launch.eps;
    params.kv_evict_first = option(kOptKvEvictFirst) != 0 ? 1 : 0;
    params.wait_limit_ns = wait_limit_ns();
    params.selftest_drop = wait_selftest_drop() ? 1 : 0;
    params.token_order = launch.token_order;
    const uint64_t blocks = static_cast<uint64_t>(launch.num_tokens) * kKvHeads * launch.num_splits;
    cudaError_t status = launch_kernel(kernel, static_cast<unsigned int>(blocks), kThreads, kSmemAlloc, stream,
                                       cluster_merge ? launch.num_splits : 1u, key_map, value_map, params);
    if (status != cudaSuccess || launch.num_splits == 1 || cluster_merge) {
        return status;
    }
    return launch_kernel(merge_splitk_kernel, static_cast<unsigned int>(launch.num_tokens * kKvHeads), kThreads, 0,
                         stream, 1, static_cast<const float*>(launch.partials),
                         static_cast<__nv_bfloat16*>(launch.output), static_cast<uint32_t>(launch.num_tokens),
                         launch.num_splits);
}

}  // namespace lfm25
