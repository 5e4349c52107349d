// Decode GEMM on the 5th-generation tensor cores with the batch on the tensor-memory lanes:
//   Y[M,N] = bf16(alpha * X[M,K] * W[N,K]^T), E4M3 x E4M3 or BF16 x BF16, fp32 accumulation, 1 <= M <= 256.
//
// Replaces the reference's BlasLt::linear_fp8_scaled and BlasLt::linear_bf16 (src/cuda/blaslt/mod.rs:113-186,
// 212-298) for the batch sizes of a continuous-batching step.  The op is bound by the weight stream (N*K bytes
// through M <= 256).  Three things decide how close a kernel gets to that bound, and the layout follows them:
//
//   * Every SM streams an equal share.  The batch (up to 128 rows per accumulator, two accumulators for 129..256
//     rows) is the M = 128 operand of tcgen05.mma and a tile of `n_tile` weight rows is its N operand.  N of the
//     instruction is any multiple of 16 up to 256, so the host picks n_tile such that the number of tiles just fills
//     the SMs (16384 rows in tiles of 112 are 147 CTAs on 148 SMs), which a fixed 128-row weight tile cannot do.
//   * One thread cannot issue tcgen05.mma fast enough.  Measured on a B200: a thread issues one M = 128 MMA every
//     ~182 cycles whatever its N (16 .. 256), i.e. N * 32 bytes of weights per 182 cycles -- 39 GB/s per SM at
//     N = 112, below an SM's share of HBM -- while a second issuing warp runs at the same rate beside it (the
//     tensor pipe itself takes an N = 256 MMA every ~145 cycles), and every K block costs its issuer another few
//     hundred cycles for the barrier wait and the commit.  So the K blocks are dealt out round-robin to 2 or 4
//     issuing warps, each with accumulators of its own in TMEM; the epilogue adds the accumulators.
//   * The accumulator has one batch row per lane and one output feature per column: an epilogue thread owns a
//     batch row and holds consecutive features of it, so it stores 32 contiguous bytes at a time with no
//     transposition, and SiLU(gate) * up of the packed Gate/Up projection is plain register arithmetic (a tile
//     is n_tile / 2 gate rows followed by the matching up rows).
//
//   warp 0      one thread: TMA loads (128-byte swizzle, mbarrier completion, no multicast) of one ring slot per
//               128-byte K block: the activation tile(s) and the weight tile; the weight tiles of the first ring
//               are requested before the dependency wait (they are constants), the activations after it
//   warps 1-4   issuing warps (1, 2 or 4 of them are used); warp 1 also allocates TMEM.  Issuer i takes K blocks
//               i, i + issuers, ...: it waits for the slot, issues the block's MMAs (4 per activation tile) into its
//               own accumulators and releases the slot with tcgen05.commit
//   warps 5-8   epilogue, one TMEM lane quadrant each, for the first half of the tile's columns; the issuing warps,
//               idle by then, take the second half
//
// With few tiles (N = 2048: 16 tiles of 128) K is split over the CTAs of a thread-block cluster; the fp32
// partial tiles meet in an L2-resident exchange buffer, the cluster passes one barrier and CTA q then finishes
// its share of the batch rows in rank order (reproducible, no atomics).
//
// Every mbarrier wait is bounded.  A wait that runs out sets the CTA's abort flag, is recorded in the device
// status words, and the CTA still frees its TMEM and exits without storing; in a cluster the flag is passed to
// the partners before the barrier so that none of them stores a sum with a missing term.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "launch.h"
#include "options.h"
#include "tcgen05.cuh"
#include "tensor_map.h"

namespace lfm25 {

namespace {

constexpr uint32_t kBlockK = 128;          // bytes of K per ring slot = one swizzle row
constexpr uint32_t kUmmaK = 32;            // bytes of K per tcgen05.mma
constexpr uint32_t kKSteps = kBlockK / kUmmaK;
constexpr uint32_t kMaxIssuers = 4;
constexpr uint32_t kFirstEpilogueWarp = 1 + kMaxIssuers;
constexpr uint32_t kThreads = 32 * (kFirstEpilogueWarp + 4);   // producer, 4 issuing warps, 4 epilogue warps
constexpr uint32_t kLanes = 128;           // batch rows per accumulator = UMMA M
constexpr uint32_t kMaxStages = 12;
constexpr uint32_t kSmemLimit = 200 * 1024;
constexpr uint32_t kSmemShared = 110 * 1024;   // two CTAs per SM (2 x (110 + 1) KiB of the 227 KiB)

struct RowsParams {
    __nv_bfloat16* out;
    float* exchange;          // split-K partial tiles [tile][slice][split][a_tiles * 128 batch rows][n_tile] fp32
    unsigned int* status;
    uint64_t wait_limit_ns;
    uint32_t weights_evict_first;   // nonzero: the weight tiles carry the L2 evict-first hint
    uint32_t m;
    uint32_t n;               // output features (plain) or the intermediate width (gated)
    uint32_t n_tile;          // weight rows per CTA = UMMA N
    uint32_t a_rows;          // rows of one activation box (a multiple of 8, <= 128)
    uint32_t a_tiles;         // 1, or 2 for batches over 128 rows that are not sliced
    uint32_t slices;          // CTAs that share one weight tile, each with slice_rows of the batch
    uint32_t slice_rows;
    uint32_t issuers;         // issuing warps: 1 | 2 | 4, each with a_tiles accumulators
    uint32_t stages;
    uint32_t stage_bytes;     // activation tile(s) followed by the weight tile
    uint32_t control_offset;  // bytes from the start of the (1024-byte aligned) shared memory
    uint32_t k_blocks;        // 128-byte K blocks in total; split s takes the s-th of `splits` near-equal ranges
    uint32_t splits;
    uint32_t tmem_columns;    // power of two >= 32
    uint32_t accumulator_columns;   // TMEM columns of one accumulator (issuer i, batch tile a: (i * a_tiles + a) of them in)
    uint32_t drop_block;      // self-test: the copies of this K block are armed but never issued
    float alpha;
    // Gated mode (packed Gate/Up weights [2 * n, K], gate rows first): a tile is n_tile / 2 gate rows and the
    // matching up rows; the epilogue writes act = bf16(silu(bf16(gate)) * bf16(up)), as E4M3 codes of
    // act * gated_scale when gated_e4m3 is set.  gated == 0: plain GEMM.
    uint32_t gated;
    uint32_t gated_e4m3;
    float gated_scale;
    void* gated_out;          // [m, n] E4M3 codes or bf16
};

template <bool BF16>
__device__ __forceinline__ void umma_rows(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    if (BF16) {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}
// Stores `value` to the word at the same shared-memory offset as `local_address` in CTA `rank` of the cluster.
__device__ __forceinline__ void store_to_cluster_cta(uint32_t local_address, uint32_t rank, uint32_t value) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(rank));
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(value) : "memory");
}

__device__ __forceinline__ uint32_t bf16_bits(float value) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(value)));
}

// 16 (or 8) consecutive columns of this thread's lane, summed over `groups` (1, 2 or 4) accumulators `stride` columns
// apart, in accumulator order (reproducible); two accumulators are loaded at a time
__device__ __forceinline__ void load_sum16(uint32_t address, uint32_t groups, uint32_t stride, float (&sum)[16]) {
    uint32_t raw[2][16];
    tmem_load16_nowait(address, raw[0]);
    if (groups > 1) {
        tmem_load16_nowait(address + stride, raw[1]);
    }
    tmem_load_wait();
#pragma unroll
    for (uint32_t j = 0; j < 16; ++j) {
        sum[j] = __uint_as_float(raw[0][j]);
        if (groups > 1) sum[j] += __uint_as_float(raw[1][j]);
    }
    if (groups > 2) {
        tmem_load16_nowait(address + 2 * stride, raw[0]);
        tmem_load16_nowait(address + 3 * stride, raw[1]);
        tmem_load_wait();
#pragma unroll
        for (uint32_t j = 0; j < 16; ++j) {
            sum[j] = (sum[j] + __uint_as_float(raw[0][j])) + __uint_as_float(raw[1][j]);
        }
    }
}
// the same for the gate and the up column of a gated tile at once
__device__ __forceinline__ void load_sum8_pair(uint32_t gate_address, uint32_t up_address, uint32_t groups,
                                               uint32_t stride, float (&gate)[8], float (&up)[8]) {
    uint32_t raw_gate[2][8];
    uint32_t raw_up[2][8];
    tmem_load8_nowait(gate_address, raw_gate[0]);
    tmem_load8_nowait(up_address, raw_up[0]);
    if (groups > 1) {
        tmem_load8_nowait(gate_address + stride, raw_gate[1]);
        tmem_load8_nowait(up_address + stride, raw_up[1]);
    }
    tmem_load_wait();
#pragma unroll
    for (uint32_t j = 0; j < 8; ++j) {
        gate[j] = __uint_as_float(raw_gate[0][j]);
        up[j] = __uint_as_float(raw_up[0][j]);
        if (groups > 1) {
            gate[j] += __uint_as_float(raw_gate[1][j]);
            up[j] += __uint_as_float(raw_up[1][j]);
        }
    }
    if (groups > 2) {
        tmem_load8_nowait(gate_address + 2 * stride, raw_gate[0]);
        tmem_load8_nowait(up_address + 2 * stride, raw_up[0]);
        tmem_load8_nowait(gate_address + 3 * stride, raw_gate[1]);
        tmem_load8_nowait(up_address + 3 * stride, raw_up[1]);
        tmem_load_wait();
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            gate[j] = (gate[j] + __uint_as_float(raw_gate[0][j])) + __uint_as_float(raw_gate[1][j]);
            up[j] = (up[j] + __uint_as_float(raw_up[0][j])) + __uint_as_float(raw_up[1][j]);
        }
    }
}

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 2)
gemm_rows_umma_kernel(const __grid_constant__ CUtensorMap weight_map, const __grid_constant__ CUtensorMap x_map,
                      const RowsParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t tile = blockIdx.x / (p.splits * p.slices);
    const uint32_t slice = (blockIdx.x / p.splits) % p.slices;
    const uint32_t split = p.splits > 1 ? cluster_cta_rank() : 0;
    const uint32_t slice_first = slice * p.slice_rows;                      // first batch row of this CTA
    const uint32_t slice_count = p.m - slice_first < p.slice_rows * p.a_tiles ? p.m - slice_first
                                                                              : p.slice_rows * p.a_tiles;
    const uint32_t x_tile_bytes = p.a_rows * kBlockK;
    const uint32_t x_bytes = p.a_tiles * x_tile_bytes;
    const uint32_t ring = smem_u32(smem);
    uint8_t* control = smem + p.control_offset;
    const uint32_t bar_full = smem_u32(control);
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t bar_accumulator = bar_empty + 8 * kMaxStages;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(control + 16 * kMaxStages + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* partner_abort = tmem_slot + 2;

    pdl_launch_dependents();
    // K range of this split: the first (k_blocks % splits) splits take one block more
    const uint32_t k_share = p.k_blocks / p.splits;
    const uint32_t k_extra = p.k_blocks % p.splits;
    const uint32_t k_count = k_share + (split < k_extra ? 1u : 0u);
    const uint32_t k_block0 = split * k_share + (split < k_extra ? split : k_extra);
    const uint32_t half = p.n_tile / 2;
    const int32_t weight_row = static_cast<int32_t>(tile * (p.gated ? half : p.n_tile));
    const uint32_t ahead = k_count < p.stages ? k_count : p.stages;
    const uint64_t weight_policy = l2_evict_first_policy();
    // a ring slot: [activation tile(s)][weight tile]
    auto load_weights = [&](uint32_t block, uint32_t stage) {
        const uint32_t bar = bar_full + 8 * stage;
        const uint32_t dst = ring + stage * p.stage_bytes + x_bytes;
        const int32_t k_offset = static_cast<int32_t>((k_block0 + block) * kBlockK);
        // every weight byte is read once per launch: with the evict-first hint the stream leaves the activations
        // and the output in the L2 for the kernels that read them next
        if (p.weights_evict_first != 0) {
            tma_load_2d_hint(dst, &weight_map, bar, k_offset, weight_row, weight_policy);
            if (p.gated) {
                tma_load_2d_hint(dst + half * kBlockK, &weight_map, bar, k_offset,
                                 weight_row + static_cast<int32_t>(p.n), weight_policy);
            }
        } else {
            tma_load_2d(dst, &weight_map, bar, k_offset, weight_row);
            if (p.gated) {
                tma_load_2d(dst + half * kBlockK, &weight_map, bar, k_offset, weight_row + static_cast<int32_t>(p.n));
            }
        }
    };
    auto load_activations = [&](uint32_t block, uint32_t stage) {
        const uint32_t bar = bar_full + 8 * stage;
        const uint32_t dst = ring + stage * p.stage_bytes;
        const int32_t k_offset = static_cast<int32_t>((k_block0 + block) * kBlockK);
        tma_load_2d(dst, &x_map, bar, k_offset, static_cast<int32_t>(slice_first));
        if (p.a_tiles == 2) {
            tma_load_2d(dst + x_tile_bytes, &x_map, bar, k_offset, static_cast<int32_t>(slice_first + kLanes));
        }
    };
    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&weight_map);
        tma_prefetch_descriptor(&x_map);
        for (uint32_t stage = 0; stage < p.stages; ++stage) {
            mbar_init(bar_full + 8 * stage, 1);
            mbar_init(bar_empty + 8 * stage, 1);
        }
        mbar_init(bar_accumulator, p.issuers);
        *abort_flag = 0;
        *partner_abort = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        // The weights are constants: the first ring of them is requested here, before the TMEM allocation, the
        // CTA-wide barrier and the dependency wait, so the stream flows while the predecessor kernel drains.  The
        // activation tiles, which the predecessor writes, follow after the wait and complete the same barriers.
        for (uint32_t block = 0; block < ahead; ++block) {
            mbar_arrive_expect_tx(bar_full + 8 * block, p.stage_bytes);
            if (block != p.drop_block) {     // self-test: nothing completes the barrier of a dropped block
                load_weights(block, block);
            }
        }
    }
    __syncwarp();
    if (warp == 1) {
        tmem_allocate(smem_u32(const_cast<uint32_t*>(tmem_slot)), p.tmem_columns);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();   // the activations are the predecessor's output
            for (uint32_t block = 0; block < ahead; ++block) {
                if (block != p.drop_block) {
                    load_activations(block, block);
                }
            }
            // (slot and phase are carried along: a division per K block is dozens of instructions on a lone thread)
            uint32_t stage = 0;
            uint32_t parity = 0;
            for (uint32_t block = ahead; block < k_count; ++block) {
                if (*abort_flag || !mbar_wait_bounded(bar_empty + 8 * stage, parity, p.wait_limit_ns)) {
                    if (!*abort_flag) record_wait_timeout(p.status, kTagGemmRows, (blockIdx.x << 4) | 1);
                    *abort_flag = 1;
                    break;
                }
                mbar_arrive_expect_tx(bar_full + 8 * stage, p.stage_bytes);
                load_weights(block, stage);
                load_activations(block, stage);
                if (++stage == p.stages) {
                    stage = 0;
                    parity ^= 1;
                }
            }
        }
    } else if (warp < kFirstEpilogueWarp) {
        const uint32_t issuer = warp - 1;
        if (lane == 0 && issuer < p.issuers) {
            // instruction descriptor: D = f32, A = B = E4M3 (format 0) or BF16 (format 1), both K-major,
            // N = n_tile, M = 128
            const uint32_t formats = BF16 ? ((1u << 7) | (1u << 10)) : 0u;
            const uint32_t idesc = (1u << 4) | formats | ((p.n_tile >> 3) << 17) | ((kLanes >> 4) << 24);
            const uint32_t accumulator = tmem_base + issuer * p.a_tiles * p.accumulator_columns;
            bool ok = true;
            // The operands of a slot were written by TMA and announced through the slot's mbarrier, which is all the
            // ordering tcgen05.mma needs; the abort flag is only looked at when a wait runs out.
            // slot, phase and descriptors are carried along instead of being derived from the block index: the loop of
            // a lone thread is bound by its instruction count (a division alone is dozens of instructions)
            constexpr uint64_t kDescriptorHigh = (static_cast<uint64_t>(1) << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
                                                 (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
            const uint32_t slot_step = p.issuers * p.stage_bytes;
            const uint32_t ring_bytes = p.stages * p.stage_bytes;
            uint32_t stage = issuer;                       // issuers <= stages and stages % issuers == 0
            uint32_t slot = ring + issuer * p.stage_bytes;
            uint32_t parity = 0;
            uint32_t accumulate = 0;
            for (uint32_t block = issuer; block < k_count; block += p.issuers) {
                if (!mbar_wait_bounded(bar_full + 8 * stage, parity, p.wait_limit_ns)) {
                    if (!*abort_flag) record_wait_timeout(p.status, kTagGemmRows, (blockIdx.x << 4) | 2);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint64_t a_desc = kDescriptorHigh | (slot >> 4);
                const uint64_t b_desc = kDescriptorHigh | ((slot + x_bytes) >> 4);
                // advancing 32 bytes inside the swizzle row = +2 in the (address >> 4) field
                umma_rows<BF16>(accumulator, a_desc, b_desc, idesc, accumulate);
                umma_rows<BF16>(accumulator, a_desc + 2, b_desc + 2, idesc, 1u);
                umma_rows<BF16>(accumulator, a_desc + 4, b_desc + 4, idesc, 1u);
                umma_rows<BF16>(accumulator, a_desc + 6, b_desc + 6, idesc, 1u);
                if (p.a_tiles == 2) {
                    const uint64_t a_desc_second = kDescriptorHigh | ((slot + x_tile_bytes) >> 4);
                    const uint32_t second = accumulator + p.accumulator_columns;
                    umma_rows<BF16>(second, a_desc_second, b_desc, idesc, accumulate);
                    umma_rows<BF16>(second, a_desc_second + 2, b_desc + 2, idesc, 1u);
                    umma_rows<BF16>(second, a_desc_second + 4, b_desc + 4, idesc, 1u);
                    umma_rows<BF16>(second, a_desc_second + 6, b_desc + 6, idesc, 1u);
                }
                umma_commit(bar_empty + 8 * stage);
                accumulate = 1;
                stage += p.issuers;
                slot += slot_step;
                if (stage >= p.stages) {
                    stage -= p.stages;
                    slot -= ring_bytes;
                    parity ^= 1;
                }
            }
            if (ok) {
                umma_commit(bar_accumulator);
            }
        }
    }
    // The producer and the issuers ran their loops on one lane each: every warp meets again here, so that what follows
    // (warp-wide TMEM loads, CTA barriers) is reached by whole warps.
    __syncwarp();
    if (warp != 0) {
        // ---- epilogue: eight warps.  A warp may only touch the 32 TMEM lanes of its quadrant (warp id modulo 4);
        // warps 5..8 take the first half of the tile's columns, the issuing warps 1..4, idle by now, the second.
        const uint32_t quadrant = warp & 3;
        const uint32_t part = warp < kFirstEpilogueWarp ? 1u : 0u;
        pdl_wait();   // the output buffer may still be read by an earlier kernel until the dependency resolves
        const bool ready =
            __all_sync(0xffffffffu, !*abort_flag && mbar_wait_bounded(bar_accumulator, 0, p.wait_limit_ns));
        if (!ready && lane == 0) {
            if (!*abort_flag) record_wait_timeout(p.status, kTagGemmRows, (blockIdx.x << 4) | 3);
            *abort_flag = 1;
        }
        tcgen05_fence_after();
        const uint32_t groups = p.issuers;                                 // accumulators per batch tile
        const uint32_t group_stride = p.a_tiles * p.accumulator_columns;   // between accumulators of one batch tile
        if (ready) {
            for (uint32_t a = 0; a < p.a_tiles; ++a) {
                const uint32_t first_row = a * kLanes + quadrant * 32;
                if (first_row >= slice_count) {
                    break;   // the rest of the lanes hold no batch row (warp-uniform)
                }
                const uint32_t local_row = first_row + lane;
                const uint32_t batch = slice_first + local_row;
                const bool valid = local_row < slice_count;
                const uint32_t lane_address = tmem_base + ((quadrant * 32) << 16) + a * p.accumulator_columns;
                if (p.gated) {
                    // columns [0, half) are gate rows, [half, n_tile) the matching up rows
                    const uint32_t first = tile * half;
                    const uint32_t columns = p.n - first < half ? p.n - first : half;
                    const uint32_t middle = ((columns / 2) + 7) / 8 * 8;
                    const uint32_t column_begin = part == 0 ? 0 : middle;
                    const uint32_t column_end = part == 0 ? middle : columns;
                    for (uint32_t column0 = column_begin; column0 < column_end; column0 += 8) {
                        float gate[8];
                        float up[8];
                        load_sum8_pair(lane_address + column0, lane_address + half + column0, groups, group_stride, gate,
                                       up);
                        if (!valid) {
                            continue;   // lanes past the batch hold whatever the unused operand rows produced
                        }
                        __align__(16) __nv_bfloat162 hidden[4];
#pragma unroll
                        for (uint32_t pair = 0; pair < 4; ++pair) {
                            // both projections are rounded to bf16 first, as the two-launch route stores them
                            const float g0 = __bfloat162float(__float2bfloat16_rn(gate[2 * pair] * p.alpha));
                            const float g1 = __bfloat162float(__float2bfloat16_rn(gate[2 * pair + 1] * p.alpha));
                            const float u0 = __bfloat162float(__float2bfloat16_rn(up[2 * pair] * p.alpha));
                            const float u1 = __bfloat162float(__float2bfloat16_rn(up[2 * pair + 1] * p.alpha));
                            hidden[pair] = __floats2bfloat162_rn(silu(g0) * u0, silu(g1) * u1);
                        }
                        const size_t element = static_cast<size_t>(batch) * p.n + first + column0;
                        if (p.gated_e4m3) {
                            uint32_t packed[2];
#pragma unroll
                            for (uint32_t word = 0; word < 2; ++word) {
                                const float2 low = __bfloat1622float2(hidden[word * 2]);
                                const float2 high = __bfloat1622float2(hidden[word * 2 + 1]);
                                packed[word] =
                                    static_cast<uint32_t>(e4m3x2(low.x * p.gated_scale, low.y * p.gated_scale)) |
                                    (static_cast<uint32_t>(e4m3x2(high.x * p.gated_scale, high.y * p.gated_scale)) << 16);
                            }
                            *reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.gated_out) + element) =
                                make_uint2(packed[0], packed[1]);
                        } else {
                            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.gated_out) + element) =
                                *reinterpret_cast<const uint4*>(hidden);
                        }
                    }
                } else {
                    const uint32_t first = tile * p.n_tile;
                    const uint32_t columns = p.n - first < p.n_tile ? p.n - first : p.n_tile;
                    const uint32_t middle = ((columns / 2) + 15) / 16 * 16;
                    const uint32_t column_begin = part == 0 ? 0 : middle;
                    const uint32_t column_end = part == 0 ? middle : columns;
                    if (p.splits == 1) {
                        __nv_bfloat16* out_row = p.out + static_cast<size_t>(batch) * p.n + first;
                        for (uint32_t column0 = column_begin; column0 < column_end; column0 += 16) {
                            float sum[16];
                            load_sum16(lane_address + column0, groups, group_stride, sum);
                            uint32_t packed[8];
#pragma unroll
                            for (uint32_t j = 0; j < 8; ++j) {
                                packed[j] = bf16_bits(sum[2 * j] * p.alpha) | (bf16_bits(sum[2 * j + 1] * p.alpha) << 16);
                            }
                            if (valid) {
                                uint4* target = reinterpret_cast<uint4*>(out_row + column0);
                                target[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                                target[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                            }
                        }
                    } else {
                        // Split K, step 1 of 2: this thread's batch row of the fp32 partial tile goes to the
                        // exchange buffer (written and read back within microseconds: it lives in L2).
                        float* mine = p.exchange +
                                      (static_cast<size_t>((tile * p.slices + slice) * p.splits + split) *
                                           (p.a_tiles * kLanes) +
                                       local_row) *
                                          p.n_tile;
                        for (uint32_t column0 = column_begin; column0 < column_end; column0 += 16) {
                            float sum[16];
                            load_sum16(lane_address + column0, groups, group_stride, sum);
                            if (valid) {
                                float4* target = reinterpret_cast<float4*>(mine + column0);
#pragma unroll
                                for (uint32_t j = 0; j < 4; ++j) {
                                    __stcg(target + j, make_float4(sum[4 * j], sum[4 * j + 1], sum[4 * j + 2], sum[4 * j + 3]));
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    if (p.splits > 1) {
        // Split K, step 2 of 2.  A CTA that gave up tells its partners first, so that nobody stores a sum with a
        // term missing.  After the cluster barrier (release / acquire at cluster scope; the partners are the only
        // readers) CTA q finishes rows [q, q+1) * ceil(rows / splits) of its batch slice: the partials are added in rank order and
        // stored as bf16, every thread of the CTA taking four features of one row at a time, all ranks' loads in
        // flight together.
        __syncthreads();
        if (threadIdx.x < p.splits && *abort_flag) {
            store_to_cluster_cta(smem_u32(const_cast<uint32_t*>(partner_abort)), threadIdx.x, 1u);
        }
        __syncwarp();
        tcgen05_fence_before();
        cluster_barrier();
        if (!*abort_flag && !*partner_abort) {
            const uint32_t rows_each = (slice_count + p.splits - 1) / p.splits;
            const uint32_t row_begin = split * rows_each;
            const uint32_t row_end = row_begin + rows_each < slice_count ? row_begin + rows_each : slice_count;
            const uint32_t first = tile * p.n_tile;
            const uint32_t columns = p.n - first < p.n_tile ? p.n - first : p.n_tile;
            const uint32_t quads = columns / 4;
            const uint32_t items = row_end > row_begin ? (row_end - row_begin) * quads : 0;
            const size_t slab = static_cast<size_t>(p.a_tiles * kLanes) * p.n_tile;
            const float* partials = p.exchange + static_cast<size_t>(tile * p.slices + slice) * p.splits * slab;
            for (uint32_t item = threadIdx.x; item < items; item += kThreads) {
                const uint32_t row = row_begin + item / quads;
                const uint32_t column = (item % quads) * 4;
                const float* source = partials + static_cast<size_t>(row) * p.n_tile + column;
                float4 part[8];
#pragma unroll
                for (uint32_t rank = 0; rank < 8; ++rank) {
                    part[rank] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (rank < p.splits) {
                        part[rank] = __ldcg(reinterpret_cast<const float4*>(source + rank * slab));
                    }
                }
                float4 sum = part[0];
#pragma unroll
                for (uint32_t rank = 1; rank < 8; ++rank) {   // absent ranks add exact zeros
                    sum.x += part[rank].x;
                    sum.y += part[rank].y;
                    sum.z += part[rank].z;
                    sum.w += part[rank].w;
                }
                uint2 packed;
                packed.x = bf16_bits(sum.x * p.alpha) | (bf16_bits(sum.y * p.alpha) << 16);
                packed.y = bf16_bits(sum.z * p.alpha) | (bf16_bits(sum.w * p.alpha) << 16);
                *reinterpret_cast<uint2*>(p.out + static_cast<size_t>(slice_first + row) * p.n + first + column) = packed;
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_free(tmem_base, p.tmem_columns);
    }
}

constexpr uint32_t kControlBytes = 16 * kMaxStages + 64;

uint32_t round_up(uint32_t value, uint32_t unit) { return (value + unit - 1) / unit * unit; }

}  // namespace

bool gemm_rows_supports(size_t m, size_t n, size_t k_bytes) {
    return m >= 1 && m <= 256 && n % 16 == 0 && n >= 16 && k_bytes % kBlockK == 0 && k_bytes >= kBlockK &&
           n <= 0x7fffffffu && k_bytes <= 0x7fffffffu;
}

// Tile policy.  `tuning` fields that are 0 are chosen here.
//   Many weight rows (at least 148 tiles of 64): K is not split; n_tile is the multiple of 16 in [64, 256] whose
//   tile count wastes the least of a whole number of waves of 148 CTAs (one per SM) or 296 (two per SM, when two
//   rings of at least three slots fit one SM), ties to one full wave of one CTA per SM, then to two CTAs per SM,
//   then to the larger tile.
//   Fewer rows (N = 2048 .. 6144 in the model): tiles of 128 rows and K split over a cluster, the largest split
//   count <= 8 that keeps tiles * splits within 296 CTAs and leaves every CTA two K blocks; needs the exchange
//   buffer (without one, or in gated mode, K is never split).
//   Issuers: as many issuing warps (4, 2 or 1) as TMEM has columns for their accumulators: 512 in all, 256 when
//   two CTAs share the SM.
//   Stages: as many ring slots as the shared-memory budget holds (3 at least, 12 at most).  The default budget
//   leaves half of the SM's shared memory to a second CTA -- of this launch or of the next kernel in the stream,
//   which then requests its first ring of weights before its dependency resolves.
GemmRowsPlan gemm_rows_plan(size_t m, size_t n, size_t k_bytes, bool gated, size_t exchange_bytes,
                            const GemmRowsTuning& tuning) {
    GemmRowsPlan plan = {};
    // batch slices: `slices` CTAs share a weight tile (the first reads it from HBM, the others from L2), each with
    // slice_rows of the batch: the activation tile of a ring slot shrinks accordingly
    uint32_t slices = tuning.slices != 0 ? tuning.slices : 1u;
    if (slices > m) slices = static_cast<uint32_t>(m);
    uint32_t slice_rows = round_up(static_cast<uint32_t>((m + slices - 1) / slices), 8);
    slices = static_cast<uint32_t>((m + slice_rows - 1) / slice_rows);
    const uint32_t a_tiles = slice_rows > kLanes ? 2u : 1u;
    if (a_tiles == 2) slice_rows = kLanes;      // two accumulators of 128 rows, one slice
    const uint32_t a_rows = a_tiles == 2 ? kLanes : slice_rows;
    const uint32_t x_bytes = a_tiles * a_rows * kBlockK;
    const uint32_t k_blocks = static_cast<uint32_t>(k_bytes / kBlockK);
    const uint32_t rows = static_cast<uint32_t>(n);   // output features; a gated tile covers n_tile / 2 of them
    // the tcgen05.mma reads 128 activation rows whatever the batch: rows past the box are whatever follows in
    // shared memory (their lanes are never stored), so the allocation must reach 16 KiB past the last box
    const uint32_t overrun = a_tiles == 1 ? (kLanes - a_rows) * kBlockK : 0;
    auto features_of = [&](uint32_t n_tile) { return gated ? n_tile / 2 : n_tile; };
    auto tiles_of = [&](uint32_t n_tile) { return (rows + features_of(n_tile) - 1) / features_of(n_tile); };
    uint32_t budget = tuning.smem_bytes != 0 ? tuning.smem_bytes : kSmemShared;
    if (budget > kSmemLimit) budget = kSmemLimit;
    const uint32_t fixed = overrun + kControlBytes + 1024;
    auto slots = [&](uint32_t n_tile) {
        const uint32_t stage_bytes = n_tile * kBlockK + x_bytes;
        return budget > fixed + stage_bytes ? (budget - fixed) / stage_bytes : 0u;
    };

    uint32_t n_tile = tuning.n_tile;
    uint32_t splits = tuning.splits;
    uint32_t ctas_per_sm = tuning.ctas_per_sm;
    const bool can_split = !gated && exchange_bytes > 0;
    const bool few_rows = tiles_of(64) * slices < 148;
    // The Gate/Up of the decode step at 64..128 rows: one wave of 112-row tiles (8192 features: 147 CTAs on 148
    // SMs), six ring slots in the whole shared memory of an SM and two issuing warps.  Measured inside the step
    // for the gated form against the general rule below (which picks 64-row tiles, two CTAs per SM): 64 sequences
    // 1.010 -> 1.000 ms, 80: 1.124 -> 1.113, 96: 1.189 -> 1.179, 112: level, 128: 1.307 -> 1.304.  The plain form
    // of the same shape takes the same plan, so that both split the K blocks over the issuing warps alike and the
    // gated launch keeps giving the bits of the plain launch followed by the SiLU * Up kernel.
    uint32_t preset_stages = 0;
    uint32_t preset_issuers = 0;
    if (n_tile == 0 && tuning.stages == 0 && tuning.issuers == 0 && tuning.smem_bytes == 0 &&
        ctas_per_sm == 0 && slices == 1 && m >= 64 && m <= 128 && tiles_of(112) > 120 && tiles_of(112) <= 148) {
        n_tile = 112;
        ctas_per_sm = 1;
        budget = kSmemLimit;
        preset_stages = 6;
        preset_issuers = 2;
    }
    if (n_tile == 0) {
        if (few_rows && can_split && splits != 1) {
            n_tile = rows < 128 ? round_up(rows, 16) : 128;
        } else {
            // score: wasted fraction of the waves (in steps of half a percent), then one full wave of one CTA per SM
            // before two CTAs per SM before several waves of one CTA per SM, then the larger tile.  A candidate needs
            // four ring slots within the budget (so that two CTAs -- of this launch, or this one and the next
            // kernel's -- share an SM); if none has, the whole shared memory of an SM is the budget.
            double best = 1e9;
            uint32_t best_per_sm = 1;
            for (uint32_t attempt = 0; attempt < 2 && n_tile == 0; ++attempt) {
                if (attempt == 1 && tuning.smem_bytes == 0) budget = kSmemLimit;
                for (uint32_t per_sm = 1; per_sm <= 2; ++per_sm) {
                    if (ctas_per_sm != 0 && per_sm != ctas_per_sm) continue;
                    if (per_sm == 2 && attempt == 1) continue;
                    for (uint32_t candidate = 64; candidate <= 256; candidate += 16) {
                        if (slots(candidate) < 4) continue;
                        const uint32_t wave = 148u * per_sm;
                        const uint32_t tiles = tiles_of(candidate) * slices;
                        const uint32_t waves = (tiles + wave - 1) / wave;
                        const double waste = 1.0 - static_cast<double>(rows) * slices /
                                                       (static_cast<double>(waves) * wave * features_of(candidate));
                        const uint32_t rank = (waves == 1 && per_sm == 1) ? 0u : (per_sm == 2 ? 1u : 2u);
                        const double score = static_cast<double>(static_cast<uint32_t>(waste * 200.0)) * 1000.0 +
                                             rank * 300.0 + (256 - candidate);
                        if (score < best) {
                            best = score;
                            n_tile = candidate;
                            best_per_sm = per_sm;
                        }
                    }
                }
            }
            if (n_tile == 0) n_tile = 128;
            if (ctas_per_sm == 0) ctas_per_sm = best_per_sm;
        }
    }
    if (n_tile > 256) n_tile = 256;
    n_tile = round_up(n_tile, 16);
    const uint32_t tiles = tiles_of(n_tile);
    if (splits == 0) {
        splits = 1;
        if (can_split && few_rows) {
            for (uint32_t candidate = 2; candidate <= 8; ++candidate) {
                if (tiles * slices * candidate <= 296 && k_blocks / candidate >= 2) {
                    splits = candidate;
                }
            }
        }
    }
    if (!can_split || splits > k_blocks) splits = 1;
    if (splits > 8) splits = 8;
    while (splits > 1 && static_cast<size_t>(tiles) * slices * splits * a_tiles * kLanes * n_tile * 4 > exchange_bytes) {
        --splits;
    }
    if (ctas_per_sm == 0) {
        ctas_per_sm = tiles * splits * slices > 148 ? 2u : 1u;
    }
    const uint32_t stage_bytes = n_tile * kBlockK + x_bytes;
    const uint32_t k_least = k_blocks / splits;
    uint32_t stages = tuning.stages != 0 ? tuning.stages : (preset_stages != 0 ? preset_stages : slots(n_tile));
    if (stages < 3 && tuning.stages == 0) {
        stages = 3;   // fewer than three slots cannot keep the stream going: take what three need
    }
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > k_least) stages = k_least;
    if (stages < 1) stages = 1;
    while (stages > 2 && stages * stage_bytes + fixed > kSmemLimit + 16 * 1024) --stages;
    // Issuing warps: every issuer has a_tiles accumulators of round_up(n_tile, 32) columns.  The ring slots are dealt
    // out with the K blocks, so the slot count is a multiple of the issuers: a slot then always belongs to the same
    // issuer, which sees every phase of its barrier in order (a parity wait is only right for a waiter that is at
    // most one phase behind).  A slot count in between is rounded down if four or more slots remain, else up.
    const uint32_t accumulator_columns = round_up(n_tile, 32);
    auto fits_twice = [&](uint32_t count) { return 2 * (count * stage_bytes + fixed + 1024) <= 227 * 1024; };
    uint32_t issuers = tuning.issuers != 0 ? tuning.issuers : (preset_issuers != 0 ? preset_issuers : kMaxIssuers);
    if (issuers == 3) issuers = 2;
    if (issuers > kMaxIssuers) issuers = kMaxIssuers;
    while (issuers > 1 && (issuers * a_tiles * accumulator_columns > 512 || issuers > k_least)) issuers /= 2;
    if (tuning.issuers == 0) {
        // two CTAs that share an SM share its 512 TMEM columns
        while (issuers > 1 && fits_twice(stages) && issuers * a_tiles * accumulator_columns > 256) issuers /= 2;
    }
    if (stages % issuers != 0) {
        const uint32_t up = (stages / issuers + 1) * issuers;
        const uint32_t down = stages / issuers * issuers;
        if (down >= 4 || (down > 0 && tuning.stages != 0)) {
            stages = down;
        } else if (up <= k_least && up <= kMaxStages && up * stage_bytes + fixed <= kSmemLimit + 16 * 1024) {
            stages = up;
        } else if (down > 0) {
            stages = down;
        } else {
            issuers = 1;
        }
    }
    plan.n_tile = n_tile;
    plan.splits = splits;
    plan.tiles = tiles;
    plan.a_tiles = a_tiles;
    plan.a_rows = a_rows;
    plan.slices = slices;
    plan.slice_rows = slice_rows;
    plan.stages = stages;
    plan.issuers = issuers;
    plan.ctas_per_sm = ctas_per_sm;
    plan.stage_bytes = stage_bytes;
    plan.control_offset = stages * stage_bytes + overrun;
    plan.smem_bytes = plan.control_offset + kControlBytes + 1024;
    plan.valid = plan.smem_bytes <= kSmemLimit + 16 * 1024 && (!gated || (n_tile / 2) % 8 == 0) &&
                 issuers * a_tiles * accumulator_columns <= 512;
    return plan;
}

// Where this kernel measured ahead of the library's other routes (bench.py --workload gemm: HBM-cold, same process,
// next to cuBLASLt).  Plain linears: nowhere yet -- the weight-major kernel is ahead up to 48 rows and level above,
// cuBLASLt is ahead on the 2048- to 6144-row BF16 sites from 33 rows on.  The gated Gate/Up linear (SiLU * Up in
// the epilogue straight from the accumulator registers) from 64 rows on: 11.9 against 13.7 us at 128 rows, 16.7
// against 20.0 at 256 (E4M3).
bool fp8_rows_preferred(size_t m, size_t n, size_t k) {
    (void)m; (void)n; (void)k;
    return false;
}
bool bf16_rows_preferred(size_t m, size_t n, size_t k) {
    (void)m; (void)n; (void)k;
    return false;
}
bool fp8_gated_rows_preferred(size_t m, size_t intermediate, size_t k) {
    (void)k;
    return m >= 64 && intermediate >= 4096;
}

namespace {

struct GatedTarget {
    void* out;
    float code_scale;
    bool e4m3;
};

template <bool BF16>
cudaError_t launch_rows(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m, size_t n,
                        size_t k_bytes, float alpha, void* exchange, size_t exchange_bytes, unsigned int* status,
                        const GemmRowsTuning& tuning, const GatedTarget* gated) {
    // n: output features of a plain GEMM; for the gated form the intermediate width (the weights have 2 n rows)
    const GemmRowsPlan plan = gemm_rows_plan(m, n, k_bytes, gated != nullptr, exchange != nullptr ? exchange_bytes : 0,
                                             tuning);
    if (!plan.valid) {
        return cudaErrorInvalidValue;
    }
    CUtensorMap weight_map;
    CUtensorMap x_map;
    const size_t weight_rows = gated != nullptr ? 2 * n : n;
    if (!make_swizzled_2d_map(&weight_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, weight, weight_rows, k_bytes,
                              gated != nullptr ? plan.n_tile / 2 : plan.n_tile) ||
        !make_swizzled_2d_map(&x_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x, m, k_bytes, plan.a_rows)) {
        return cudaErrorInvalidValue;
    }
    RowsParams params = {};
    params.out = static_cast<__nv_bfloat16*>(out);
    params.exchange = static_cast<float*>(exchange);
    params.status = status;
    params.wait_limit_ns = wait_limit_ns();
    params.weights_evict_first = weights_evict_first() ? 1u : 0u;
    params.m = static_cast<uint32_t>(m);
    params.n = static_cast<uint32_t>(n);
    params.n_tile = plan.n_tile;
    params.a_rows = plan.a_rows;
    params.a_tiles = plan.a_tiles;
    params.slices = plan.slices;
    params.slice_rows = plan.slice_rows;
    params.issuers = plan.issuers;
    params.stages = plan.stages;
    params.stage_bytes = plan.stage_bytes;
    params.control_offset = plan.control_offset;
    params.k_blocks = static_cast<uint32_t>(k_bytes / kBlockK);
    params.splits = plan.splits;
    params.accumulator_columns = round_up(plan.n_tile, 32);
    params.tmem_columns = 32;
    while (params.tmem_columns < plan.issuers * plan.a_tiles * params.accumulator_columns) params.tmem_columns *= 2;
    params.drop_block = wait_selftest_drop() ? 0u : 0xffffffffu;
    params.alpha = alpha;
    params.gated = gated != nullptr ? 1u : 0u;
    params.gated_e4m3 = gated != nullptr && gated->e4m3 ? 1u : 0u;
    params.gated_scale = gated != nullptr ? gated->code_scale : 1.0f;
    params.gated_out = gated != nullptr ? gated->out : nullptr;

    // The dynamic shared-memory limit of the kernel is set once per device to the largest size any plan uses, so no
    // launch depends on what an earlier launch left behind.
    static bool granted[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
        return cudaErrorInvalidDevice;
    }
    if (!granted[device]) {
        const cudaError_t attribute_status =
            cudaFuncSetAttribute(gemm_rows_umma_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kSmemLimit + 16 * 1024));
        if (attribute_status != cudaSuccess) {
            return attribute_status;
        }
        granted[device] = true;
    }
    return launch_kernel(gemm_rows_umma_kernel<BF16>, plan.tiles * plan.slices * plan.splits, kThreads, plan.smem_bytes, stream,
                         plan.splits, weight_map, x_map, params);
}

}  // namespace

cudaError_t launch_fp8_gemm_rows(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                 size_t n, size_t k, float alpha, void* exchange, size_t exchange_bytes,
                                 unsigned int* status, const GemmRowsTuning& tuning) {
    return launch_rows<false>(stream, x, weight, out, m, n, k, alpha, exchange, exchange_bytes, status, tuning,
                              nullptr);
}

cudaError_t launch_fp8_gemm_rows_gated(cudaStream_t stream, const void* x, const void* weight, void* activation,
                                       size_t m, size_t intermediate, size_t k, float alpha, float code_scale,
                                       bool e4m3, unsigned int* status, const GemmRowsTuning& tuning) {
    const GatedTarget gated = {activation, code_scale, e4m3};
    return launch_rows<false>(stream, x, weight, nullptr, m, intermediate, k, alpha, nullptr, 0, status, tuning,
                              &gated);
}

cudaError_t launch_bf16_gemm_rows(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                  size_t n, size_t k, void* exchange, size_t exchange_bytes, unsigned int* status,
                                  const GemmRowsTuning& tuning) {
    return launch_rows<true>(stream, x, weight, out, m, n, k * 2, 1.0f, exchange, exchange_bytes, status, tuning,
                             nullptr);
}

cudaError_t launch_bf16_gemm_rows_gated(cudaStream_t stream, const void* x, const void* weight, void* activation,
                                        size_t m, size_t intermediate, size_t k, float code_scale, bool e4m3,
                                        unsigned int* status, const GemmRowsTuning& tuning) {
    const GatedTarget gated = {activation, code_scale, e4m3};
    return launch_rows<true>(stream, x, weight, nullptr, m, intermediate, k * 2, 1.0f, nullptr, 0, status, tuning,
                             &gated);
}

}  // namespace lfm25
