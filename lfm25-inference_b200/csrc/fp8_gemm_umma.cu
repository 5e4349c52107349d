// FP8 (E4M3) decode GEMM on the 5th-generation tensor cores: Y[M,N] = bf16(alpha * Xq[M,K] * Wq[N,K]^T)
// for batches of 9..256 rows.
//
// Replaces the reference's BlasLt::linear_fp8_scaled (src/cuda/blaslt/mod.rs:212-298) for the batch
// sizes where a weight-streaming GEMV no longer keeps up with HBM.  "Swap AB": a tile of 128 weight rows
// is the M=128 operand of tcgen05.mma (kind::f8f6f4, E4M3 x E4M3 -> fp32) and the whole batch, padded
// to a multiple of 16, is its N operand, so no tensor-core work is spent on padding.
//
//   warp 0   one thread issues TMA tile loads (128-byte swizzle, mbarrier completion, no multicast):
//            per stage a 128 x 128 B weight tile and the M_pad x 128 B activation tile of the same K block
//   warp 1   allocates TMEM; one thread issues 4 tcgen05.mma per stage (K = 32 each) into a
//            128-lane x M_pad-column fp32 accumulator and releases the stage with tcgen05.commit
//   warp 6   a second issuer with an accumulator of its own: the two take alternate K blocks (one thread issues an
//            MMA every ~180 cycles whatever its shape, which is 4 KiB of weights, about an SM's share of HBM)
//   warps 2-5  epilogue: tcgen05.ld the accumulators (thread = weight row, registers = batch columns), add them,
//            scale, round to bf16, transpose through shared memory and store 16 bytes per lane
//
// The op is bound by the weight stream (N*K bytes) for every batch size here, so what matters is the number
// of bytes in flight: stages are as deep as shared memory allows (up to 8 x 16 KiB of weights per SM).
// When N/128 tiles cannot occupy the machine (Down: 16 tiles), K is split over the CTAs of a thread-block
// cluster (up to 8 per tile).  The partial tiles are reduce-scattered through distributed shared memory:
// after a cluster barrier each CTA pushes the slice of batch columns that partner q owns straight from its
// TMEM registers into q's shared memory (st.shared::cluster, fire-and-forget), and after a second barrier
// every CTA adds the slices it received in rank order (reproducible, no atomics, no workspace, no second
// launch) and stores its share of the output.
//
// The same kernel serves the BF16 sites (template parameter): a 128-byte swizzle row then holds 64 bf16 values,
// one tcgen05.mma (kind::f16) covers K = 16 of them, i.e. the same 32 bytes, and everything else is unchanged.
//
// Every mbarrier wait is bounded; a wait that runs out sets an abort flag, is recorded in the device
// status words, and the CTA still frees its TMEM and exits.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "launch.h"
#include "options.h"
#include "tcgen05.cuh"
#include "tensor_map.h"

namespace lfm25 {

namespace {

constexpr uint32_t kTileN = 128;    // weight rows per CTA = UMMA M
constexpr uint32_t kBlockK = 128;   // bytes of K per stage = one swizzle row
constexpr uint32_t kUmmaK = 32;     // K of one tcgen05.mma with 8-bit operands
constexpr uint32_t kThreads = 224;    // producer, issuer, 4 epilogue warps, second issuer
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kSmemBudget = 200 * 1024;   // upper bound of the ring of one CTA
constexpr uint32_t kSmemBudgetShared = 98 * 1024;  // two CTAs per SM: one drains its tile while the other streams
constexpr uint32_t kWeightTileBytes = kTileN * kBlockK;

struct UmmaParams {
    __nv_bfloat16* out;
    float* exchange;         // split-K partial tiles [tile][split][batch column][128 rows] fp32 (L2-resident)
    unsigned int* status;
    uint32_t m;
    uint32_t n;
    uint32_t m_pad;          // batch rounded up to 16 = UMMA N
    uint32_t stages;
    uint32_t data_bytes;     // shared memory in front of the control block: the stages, or the parked tile
    uint32_t k_blocks;       // 128-byte K blocks in total; split s takes the s-th of `splits` near-equal ranges
    uint32_t splits;         // CTAs of a cluster that share one weight tile, each with its own K range
    uint32_t tmem_columns;   // power of two >= max(32, issuers * accumulator_columns)
    uint32_t issuers;        // issuing warps (1 or 2): issuer i takes K blocks i, i + issuers, ... into accumulator i
    uint32_t accumulator_columns;   // TMEM columns between the two accumulators
    float alpha;
    uint32_t drop_block;     // self-test: the copy of this K block is armed but never issued
    uint64_t wait_limit_ns;  // limit of every mbarrier wait
    uint32_t weights_evict_first;   // nonzero: the weight tiles carry the L2 evict-first hint (each is read once)
    // Gated mode (packed Gate/Up weights [2 * intermediate, K], gate rows first): a tile is 64 gate rows and the 64
    // up rows that belong to them, and the epilogue writes act = bf16(silu(bf16(gate)) * bf16(up)) -- as E4M3 codes
    // of act * gated_scale when gated_e4m3 is set -- instead of the two projections.  0 = plain GEMM.
    uint32_t intermediate;
    uint32_t gated_e4m3;
    float gated_scale;
    void* gated_out;         // [m, intermediate] E4M3 codes or bf16
};

template <bool BF16>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
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

// 16 consecutive columns of this thread's TMEM lane, summed over the issuers' accumulators (as fp32 bit patterns)
__device__ __forceinline__ void load_accumulators16(uint32_t address, uint32_t issuers, uint32_t stride,
                                                    uint32_t (&raw)[16]) {
    if (issuers == 1) {
        tmem_load16(address, raw);
        return;
    }
    uint32_t other[16];
    tmem_load16_nowait(address, raw);
    tmem_load16_nowait(address + stride, other);
    tmem_load_wait();
#pragma unroll
    for (uint32_t j = 0; j < 16; ++j) {
        raw[j] = __float_as_uint(__uint_as_float(raw[j]) + __uint_as_float(other[j]));
    }
}

// ---- thread-block cluster helpers (split-K partners exchange partial tiles through distributed shared memory)
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}
template <bool BF16>
__global__ void __launch_bounds__(kThreads, 2)
gemm_umma_kernel(const __grid_constant__ CUtensorMap weight_map, const __grid_constant__ CUtensorMap x_map,
                     const UmmaParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t tile = blockIdx.x / p.splits;
    const uint32_t split = p.splits > 1 ? cluster_rank() : 0;
    const uint32_t stage_bytes = kWeightTileBytes + p.m_pad * kBlockK;
    const uint32_t smem_base = smem_u32(smem);
    uint8_t* control = smem + p.data_bytes;
    const uint32_t bar_full = smem_u32(control);
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t bar_accumulator = bar_empty + 8 * kMaxStages;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(control + 16 * kMaxStages + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* partner_abort = tmem_slot + 2;   // set by a split-K partner that gave up

    pdl_launch_dependents();
    // K range of this split: the first (k_blocks % splits) splits take one block more
    const uint32_t k_share = p.k_blocks / p.splits;
    const uint32_t k_extra = p.k_blocks % p.splits;
    const uint32_t k_count = k_share + (split < k_extra ? 1u : 0u);
    const uint32_t k_block0 = split * k_share + (split < k_extra ? split : k_extra);
    const uint32_t ahead = k_count < p.stages ? k_count : p.stages;
    const bool gated = p.intermediate != 0;
    const int32_t tile_row = static_cast<int32_t>(tile * (gated ? kTileN / 2 : kTileN));
    // the weight tile of one K block: one 128-row box, or in gated mode two 64-row boxes (gate rows, up rows)
    // Every weight byte is read once per launch, by one CTA: with the evict-first hint the stream does not push the
    // activations and the output (which the next kernels read) out of the L2.
    const uint64_t weight_policy = l2_evict_first_policy();
    auto load_weight_box = [&](uint32_t dst, uint32_t bar, int32_t k_offset, int32_t row) {
        if (p.weights_evict_first != 0) {
            tma_load_2d_hint(dst, &weight_map, bar, k_offset, row, weight_policy);
        } else {
            tma_load_2d(dst, &weight_map, bar, k_offset, row);
        }
    };
    auto load_weights = [&](uint32_t dst, uint32_t bar, int32_t k_offset) {
        if (gated) {
            load_weight_box(dst, bar, k_offset, tile_row);
            load_weight_box(dst + kWeightTileBytes / 2, bar, k_offset, tile_row + static_cast<int32_t>(p.intermediate));
        } else {
            load_weight_box(dst, bar, k_offset, tile_row);
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
        // The weight tiles are constants: the first ring of them is requested right here -- before the TMEM
        // allocation, the CTA-wide barrier and the dependency wait -- so the stream is flowing while the rest of
        // the CTA sets up and the predecessor kernel drains.  The activation tiles, which the predecessor
        // writes, follow after the wait and complete the same barriers.
        for (uint32_t block = 0; block < ahead; ++block) {
            const uint32_t bar = bar_full + 8 * block;
            mbar_arrive_expect_tx(bar, stage_bytes);
            if (block == p.drop_block) {
                continue;   // self-test: nothing completes this barrier, the bounded wait on it has to run out
            }
            load_weights(smem_base + block * stage_bytes, bar, static_cast<int32_t>((k_block0 + block) * kBlockK));
        }
    }
    __syncwarp();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(p.tmem_columns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();
            for (uint32_t block = 0; block < ahead; ++block) {
                tma_load_2d(smem_base + block * stage_bytes + kWeightTileBytes, &x_map, bar_full + 8 * block,
                            static_cast<int32_t>((k_block0 + block) * kBlockK), 0);
            }
            // (slot and phase are carried along: a division per K block is dozens of instructions on a lone thread)
            uint32_t stage = 0;
            uint32_t parity = 0;
            for (uint32_t block = ahead; block < k_count; ++block) {
                if (*abort_flag || !mbar_wait_bounded(bar_empty + 8 * stage, parity, p.wait_limit_ns)) {
                    *abort_flag = 1;
                    record_wait_timeout(p.status, kTagGemmUmma, (blockIdx.x << 4) | 1);
                    break;
                }
                const uint32_t bar = bar_full + 8 * stage;
                const uint32_t dst = smem_base + stage * stage_bytes;
                const int32_t k_offset = static_cast<int32_t>((k_block0 + block) * kBlockK);
                mbar_arrive_expect_tx(bar, stage_bytes);
                load_weights(dst, bar, k_offset);
                tma_load_2d(dst + kWeightTileBytes, &x_map, bar, k_offset, 0);
                if (++stage == p.stages) {
                    stage = 0;
                    parity ^= 1;
                }
            }
        }
        __syncwarp();   // whole warps reach the CTA barriers below
    } else if (warp == 1 || warp == 6) {
        // One thread issues a tcgen05.mma every ~180 cycles whatever its shape, i.e. 4 KiB of weights per 180 cycles:
        // about an SM's share of HBM and no more.  A second issuing warp with an accumulator of its own runs at the
        // same rate beside it, so the K blocks alternate between the two (the slot count is even: a slot always
        // belongs to the same issuer, which therefore sees every phase of its barrier).
        const uint32_t issuer = warp == 1 ? 0u : 1u;
        if (lane == 0 && issuer < p.issuers) {
            // instruction descriptor: D = f32, A = B = E4M3 (format 0) or BF16 (format 1), both K-major,
            // N = m_pad, M = 128
            const uint32_t formats = BF16 ? ((1u << 7) | (1u << 10)) : 0u;
            const uint32_t idesc = (1u << 4) | formats | ((p.m_pad >> 3) << 17) | ((kTileN >> 4) << 24);
            const uint32_t accumulator = tmem_base + issuer * p.accumulator_columns;
            bool ok = true;
            // slot, phase and descriptors are carried along instead of being derived from the block index: the loop of
            // a lone thread is bound by its instruction count
            constexpr uint64_t kDescriptorHigh = (static_cast<uint64_t>(1) << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
                                                 (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
            const uint32_t slot_step = p.issuers * stage_bytes;
            const uint32_t ring_bytes = p.stages * stage_bytes;
            uint32_t stage = issuer;                       // issuers <= stages and stages % issuers == 0
            uint32_t slot = smem_base + issuer * stage_bytes;
            uint32_t parity = 0;
            uint32_t accumulate = 0;
            for (uint32_t block = issuer; block < k_count; block += p.issuers) {
                if (!mbar_wait_bounded(bar_full + 8 * stage, parity, p.wait_limit_ns)) {
                    if (!*abort_flag) record_wait_timeout(p.status, kTagGemmUmma, (blockIdx.x << 4) | 2);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint64_t a_desc = kDescriptorHigh | (slot >> 4);
                const uint64_t b_desc = kDescriptorHigh | ((slot + kWeightTileBytes) >> 4);
                // advancing 32 bytes inside the swizzle row = +2 in the (address >> 4) field
                umma<BF16>(accumulator, a_desc, b_desc, idesc, accumulate);
                umma<BF16>(accumulator, a_desc + 2, b_desc + 2, idesc, 1u);
                umma<BF16>(accumulator, a_desc + 4, b_desc + 4, idesc, 1u);
                umma<BF16>(accumulator, a_desc + 6, b_desc + 6, idesc, 1u);
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
        __syncwarp();   // whole warps reach the CTA barriers below
    } else {
        // ---- epilogue: 4 warps, each owns the 32 TMEM lanes of its quadrant (warp id modulo 4) ----
        const uint32_t quadrant = warp & 3;
        pdl_wait();   // the output buffer may still be read by an earlier kernel until the dependency resolves
        const bool ready = __all_sync(0xffffffffu, !*abort_flag && mbar_wait_bounded(bar_accumulator, 0, p.wait_limit_ns));
        if (!ready && lane == 0) {
            *abort_flag = 1;
            record_wait_timeout(p.status, kTagGemmUmma, (blockIdx.x << 4) | 3);
        }
        tcgen05_fence_after();
        const uint32_t lane_address = tmem_base + ((quadrant * 32) << 16);
        if (gated) {
            // Rows 0-63 of the tile are gate rows, rows 64-127 the matching up rows.  Every thread rounds its row to
            // bf16 (what the unfused route stores as the packed projection) into staged[column][128 rows]; after a
            // barrier of the four epilogue warps a thread takes 16 consecutive outputs of one batch column.
            uint8_t* staged = smem;
            if (ready) {
                for (uint32_t column0 = 0; column0 < p.m_pad; column0 += 16) {
                    uint32_t raw[16];
                    load_accumulators16(lane_address + column0, p.issuers, p.accumulator_columns, raw);
#pragma unroll
                    for (uint32_t j = 0; j < 16; ++j) {
                        reinterpret_cast<__nv_bfloat16*>(staged + (column0 + j) * 256)[quadrant * 32 + lane] =
                            __float2bfloat16_rn(__uint_as_float(raw[j]) * p.alpha);
                    }
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!*abort_flag) {
                const uint32_t worker = threadIdx.x - 64;     // 0..127 over the four epilogue warps
                const uint32_t part = worker & 3;             // 16 of the tile's 64 outputs
                for (uint32_t batch = worker >> 2; batch < p.m; batch += 32) {
                    const uint4* gate_raw = reinterpret_cast<const uint4*>(staged + batch * 256 + part * 32);
                    const uint4* up_raw = reinterpret_cast<const uint4*>(staged + batch * 256 + 128 + part * 32);
                    __align__(16) __nv_bfloat162 hidden[8];
#pragma unroll
                    for (uint32_t half = 0; half < 2; ++half) {
                        const uint4 g4 = gate_raw[half];
                        const uint4 u4 = up_raw[half];
                        const __nv_bfloat162* g = reinterpret_cast<const __nv_bfloat162*>(&g4);
                        const __nv_bfloat162* u = reinterpret_cast<const __nv_bfloat162*>(&u4);
#pragma unroll
                        for (uint32_t pair = 0; pair < 4; ++pair) {
                            const float2 gv = __bfloat1622float2(g[pair]);
                            const float2 uv = __bfloat1622float2(u[pair]);
                            hidden[half * 4 + pair] = __floats2bfloat162_rn(silu(gv.x) * uv.x, silu(gv.y) * uv.y);
                        }
                    }
                    const size_t element = static_cast<size_t>(batch) * p.intermediate + tile * 64 + part * 16;
                    if (p.gated_e4m3) {
                        uint32_t packed[4];
#pragma unroll
                        for (uint32_t word = 0; word < 4; ++word) {
                            const float2 a = __bfloat1622float2(hidden[word * 2]);
                            const float2 b = __bfloat1622float2(hidden[word * 2 + 1]);
                            packed[word] =
                                static_cast<uint32_t>(e4m3x2(a.x * p.gated_scale, a.y * p.gated_scale)) |
                                (static_cast<uint32_t>(e4m3x2(b.x * p.gated_scale, b.y * p.gated_scale)) << 16);
                        }
                        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.gated_out) + element) =
                            make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    } else {
                        uint4* target = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.gated_out) + element);
                        target[0] = *reinterpret_cast<const uint4*>(&hidden[0]);
                        target[1] = *reinterpret_cast<const uint4*>(&hidden[4]);
                    }
                }
            }
        } else if (p.splits == 1) {
            if (ready) {
                // Transpose through this warp's slice of the (now idle) pipeline memory so that the global stores
                // are 16 bytes wide: staged[column][32 rows] as bf16, then lane -> (column l/4, 8 rows l%4).
                uint8_t* staged = smem + quadrant * (p.m_pad * 64);
                for (uint32_t column0 = 0; column0 < p.m_pad; column0 += 16) {
                    uint32_t raw[16];
                    load_accumulators16(lane_address + column0, p.issuers, p.accumulator_columns, raw);
#pragma unroll
                    for (uint32_t j = 0; j < 16; ++j) {
                        reinterpret_cast<__nv_bfloat16*>(staged + (column0 + j) * 64)[lane] =
                            __float2bfloat16_rn(__uint_as_float(raw[j]) * p.alpha);
                    }
                }
                __syncwarp();
                __nv_bfloat16* out_rows = p.out + tile * kTileN + quadrant * 32 + (lane & 3) * 8;
                for (uint32_t column0 = 0; column0 < p.m; column0 += 8) {
                    const uint32_t batch = column0 + (lane >> 2);
                    if (batch < p.m) {
                        const uint4 value = *reinterpret_cast<const uint4*>(staged + batch * 64 + (lane & 3) * 16);
                        *reinterpret_cast<uint4*>(out_rows + static_cast<size_t>(batch) * p.n) = value;
                    }
                }
            }
        } else {
            // Split K, step 1 of 2: the fp32 partial tile goes to the exchange buffer, one coalesced 128-byte
            // store per warp and batch column.  The buffer is written and read back within microseconds, so it
            // lives in L2.  (Distributed shared memory was measured for this exchange, pushed and pulled: at a
            // cluster of 8 it moved a few GB/s per CTA.)
            if (ready) {
                float* mine = p.exchange + static_cast<size_t>(tile * p.splits + split) * p.m_pad * kTileN +
                              quadrant * 32 + lane;
                for (uint32_t column0 = 0; column0 < p.m; column0 += 16) {
                    uint32_t raw[16];
                    load_accumulators16(lane_address + column0, p.issuers, p.accumulator_columns, raw);
#pragma unroll
                    for (uint32_t j = 0; j < 16; ++j) {
                        if (column0 + j < p.m) {
                            __stcg(mine + (column0 + j) * kTileN, __uint_as_float(raw[j]));
                        }
                    }
                }
            }
        }
    }
    if (p.splits > 1) {
        // Split K, step 2 of 2: after the cluster barrier (release / acquire at cluster scope, and the partners are
        // the only readers) CTA q of the cluster finishes batch columns [q, q+1) * ceil(m / splits): it adds the
        // partials in rank order (reproducible, no atomics) and stores bf16.  A warp covers the 128 rows of one
        // column with 16-byte loads; the loads of all ranks are in flight together.
        // A CTA that gave up tells its partners first (a word in each partner's shared memory), so that nobody
        // stores a sum with a term missing.
        __syncthreads();
        if (threadIdx.x < p.splits && *abort_flag) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                         : "=r"(remote)
                         : "r"(smem_u32(const_cast<uint32_t*>(partner_abort))), "r"(threadIdx.x));
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(1u) : "memory");
        }
        tcgen05_fence_before();
        cluster_sync_all();
        if (warp >= 2 && warp <= 5 && !*abort_flag && !*partner_abort) {
            const uint32_t columns = (p.m + p.splits - 1) / p.splits;
            const uint32_t row4 = lane * 4;
            const float* partials = p.exchange + static_cast<size_t>(tile) * p.splits * p.m_pad * kTileN + row4;
            for (uint32_t column = warp - 2; column < columns; column += 4) {
                const uint32_t batch = split * columns + column;
                if (batch >= p.m) break;
                float4 part[8];
#pragma unroll
                for (uint32_t rank = 0; rank < 8; ++rank) {
                    part[rank] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (rank < p.splits) {
                        part[rank] = __ldcg(reinterpret_cast<const float4*>(
                            partials + (static_cast<size_t>(rank) * p.m_pad + batch) * kTileN));
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
                const __nv_bfloat162 low = __floats2bfloat162_rn(sum.x * p.alpha, sum.y * p.alpha);
                const __nv_bfloat162 high = __floats2bfloat162_rn(sum.z * p.alpha, sum.w * p.alpha);
                uint2 packed;
                packed.x = *reinterpret_cast<const uint32_t*>(&low);
                packed.y = *reinterpret_cast<const uint32_t*>(&high);
                *reinterpret_cast<uint2*>(p.out + static_cast<size_t>(batch) * p.n + tile * kTileN + row4) = packed;
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_columns)
                     : "memory");
    }
}

}  // namespace

bool fp8_gemm_umma_supports(size_t m, size_t n, size_t k) {
    return m >= 1 && m <= 256 && n % kTileN == 0 && k % kBlockK == 0 && n <= 0x7fffffffu && k <= 0x7fffffffu;
}

bool bf16_gemm_umma_supports(size_t m, size_t n, size_t k) { return fp8_gemm_umma_supports(m, n, k * 2); }

namespace {

constexpr uint32_t kControlBytes = 16 * kMaxStages + 64 + 1024;   // barriers, TMEM slot, alignment slack

// How many clusters of `size` CTAs, one CTA per SM with the whole shared-memory budget, the device keeps resident
// at once; asked once per size and kept.  0 when the runtime cannot tell.
template <bool BF16>
uint32_t resident_clusters(uint32_t size) {
    static int known[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
    if (size < 2 || size > 8) return 0;
    if (known[size] < 0) {
        const uint32_t smem_bytes = kSmemBudget + kControlBytes;
        int clusters = 0;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(size, 1, 1);
        config.blockDim = dim3(kThreads, 1, 1);
        config.dynamicSmemBytes = smem_bytes;
        cudaLaunchAttribute attribute;
        attribute.id = cudaLaunchAttributeClusterDimension;
        attribute.val.clusterDim.x = size;
        attribute.val.clusterDim.y = 1;
        attribute.val.clusterDim.z = 1;
        config.attrs = &attribute;
        config.numAttrs = 1;
        if (cudaFuncSetAttribute(gemm_umma_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem_bytes)) != cudaSuccess ||
            cudaOccupancyMaxActiveClusters(&clusters, gemm_umma_kernel<BF16>, &config) != cudaSuccess) {
            (void)cudaGetLastError();
            clusters = 0;
        }
        known[size] = clusters;
    }
    return static_cast<uint32_t>(known[size]);
}

// `k_bytes` is the length of a weight / activation row in bytes (K for E4M3, 2 K for BF16).
// Gated mode of a launch: where the activation goes and how it is encoded (see UmmaParams).
struct GatedOutput {
    void* out;
    float code_scale;
    bool e4m3;
};

template <bool BF16>
cudaError_t launch_umma(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m, size_t n,
                        size_t k_bytes, float alpha, void* exchange, size_t exchange_bytes, unsigned int* status,
                        const GatedOutput* gated = nullptr) {
    const uint32_t m_pad = static_cast<uint32_t>((m + 15) / 16 * 16);
    CUtensorMap weight_map;
    CUtensorMap x_map;
    // gated: n = 2 * intermediate packed rows, fetched as two 64-row boxes per tile
    if (!make_swizzled_2d_map(&weight_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, weight, n, k_bytes,
                              gated != nullptr ? kTileN / 2 : kTileN) ||
        !make_swizzled_2d_map(&x_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x, m, k_bytes, m_pad)) {
        return cudaErrorInvalidValue;
    }
    if (gated != nullptr) {
        exchange = nullptr;      // the fused epilogue needs whole sums in one CTA: K is not split
    }
    const uint32_t tiles = static_cast<uint32_t>(n / kTileN);
    const uint32_t k_blocks_total = static_cast<uint32_t>(k_bytes / kBlockK);
    const uint32_t stage_bytes = kWeightTileBytes + m_pad * kBlockK;
    // Two CTAs share an SM whenever three stages still fit in half the shared memory: with more CTAs than SMs
    // (LM head: 512 tiles) the epilogue of one tile then overlaps the weight stream of the next.
    const bool can_share = kSmemBudgetShared / stage_bytes >= 3;
    // Split K over a cluster of up to 8 CTAs per tile when the tiles alone would leave a third of the SMs idle.
    // Measured on the decode shapes (4, 16, 48 and 64 tiles), the best split count is the largest one that keeps
    // the grid within 256 CTAs at two CTAs per SM (16 tiles: 8, 48: 5, 64: 4).  Where the stages are too large to
    // share an SM (batches over 128) the grid must fit one wave of one CTA per SM, and since a cluster needs its
    // SMs inside one GPC the runtime is asked how many clusters of that size are resident (15 of size 8).  Each
    // CTA keeps at least 2 K blocks.  Needs the exchange buffer.
    uint32_t splits = 1;
    if (exchange != nullptr && tiles < 100) {
        for (uint32_t candidate = 2; candidate <= 8; ++candidate) {
            const bool fits = static_cast<size_t>(tiles) * candidate * m_pad * kTileN * 4 <= exchange_bytes;
            const bool resident = can_share ? tiles * candidate <= 256
                                            : tiles * candidate <= 148 &&
                                                  tiles <= resident_clusters<BF16>(candidate);
            if (fits && resident && k_blocks_total / candidate >= 2) {
                splits = candidate;
            }
        }
    }
    const bool share_sm = can_share && (splits > 1 || tiles > 148);
    // Ring size.  Measured on the decode shapes, a deeper ring than about 98 KiB does not pay even with one CTA per
    // SM (Gate/Up at 1..32 rows: 9.9 us with 11 stages, 9.1 with 8, 8.5 with 5): a CTA that leaves half of the
    // shared memory free lets the CTA of the next kernel in the stream move in beside it and request its own first
    // ring of weights before the dependency resolves, which is worth more than bytes in flight.  Four stages are the
    // floor (128 rows: 4 x 32 KiB).
    uint32_t budget = kSmemBudgetShared;
    if (!share_sm && 4 * stage_bytes > budget) {
        budget = 4 * stage_bytes < kSmemBudget ? 4 * stage_bytes : kSmemBudget;
    }
    uint32_t stages = budget / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    const uint32_t k_blocks_least = k_blocks_total / splits;
    if (stages > k_blocks_least) stages = k_blocks_least;
    // two issuing warps when an even ring still has four slots or more (measured: with two slots the second issuer
    // costs more than it gives) and two accumulators fit the tensor memory that one of two CTAs on an SM may take
    const uint32_t accumulator_columns = (m_pad + 31) / 32 * 32;
    uint32_t issuers = (stages - stages % 2 >= 4 && 2 * accumulator_columns <= (share_sm ? 256u : 512u)) ? 2u : 1u;
    if (issuers == 2) stages -= stages % 2;
    uint32_t data_bytes = stages * stage_bytes;
    if (data_bytes < m_pad * 256) data_bytes = m_pad * 256;   // bf16 staging of the epilogue: 4 warps x m_pad x 64 B
    const uint32_t smem_bytes = data_bytes + kControlBytes;

    UmmaParams params;
    params.out = static_cast<__nv_bfloat16*>(out);
    params.exchange = static_cast<float*>(exchange);
    params.status = status;
    params.m = static_cast<uint32_t>(m);
    params.n = static_cast<uint32_t>(n);
    params.m_pad = m_pad;
    params.stages = stages;
    params.data_bytes = data_bytes;
    params.k_blocks = k_blocks_total;
    params.splits = splits;
    params.issuers = issuers;
    params.accumulator_columns = accumulator_columns;
    params.tmem_columns = 32;
    while (params.tmem_columns < issuers * accumulator_columns) params.tmem_columns *= 2;
    params.alpha = alpha;
    params.drop_block = wait_selftest_drop() ? 0u : 0xffffffffu;
    params.wait_limit_ns = wait_limit_ns();
    params.weights_evict_first = weights_evict_first() ? 1u : 0u;
    params.intermediate = gated != nullptr ? static_cast<uint32_t>(n / 2) : 0;
    params.gated_e4m3 = gated != nullptr && gated->e4m3 ? 1u : 0u;
    params.gated_scale = gated != nullptr ? gated->code_scale : 1.0f;
    params.gated_out = gated != nullptr ? gated->out : nullptr;

    // The dynamic shared-memory limit of the kernel is set once per device to the largest size any launch uses, so
    // that no launch depends on what an earlier one (or the occupancy query above) left behind.
    static bool granted[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
        return cudaErrorInvalidDevice;
    }
    if (!granted[device]) {
        const cudaError_t attribute_status =
            cudaFuncSetAttribute(gemm_umma_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kSmemBudget + kControlBytes));
        if (attribute_status != cudaSuccess) {
            return attribute_status;
        }
        granted[device] = true;
    }
    return launch_kernel(gemm_umma_kernel<BF16>, tiles * splits, kThreads, smem_bytes, stream, splits, weight_map,
                         x_map, params);
}

}  // namespace

cudaError_t launch_fp8_gemm_umma(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                 size_t n, size_t k, float alpha, void* exchange, size_t exchange_bytes,
                                 unsigned int* status) {
    return launch_umma<false>(stream, x, weight, out, m, n, k, alpha, exchange, exchange_bytes, status);
}

bool fp8_gemm_umma_gated_supports(size_t m, size_t n, size_t k) {
    return fp8_gemm_umma_supports(m, n, k) && (n / 2) % (kTileN / 2) == 0 && n % 2 == 0;
}

cudaError_t launch_fp8_gemm_umma_gated(cudaStream_t stream, const void* x, const void* weight, void* activation,
                                       size_t m, size_t n, size_t k, float alpha, float code_scale, bool e4m3,
                                       unsigned int* status) {
    const GatedOutput gated = {activation, code_scale, e4m3};
    return launch_umma<false>(stream, x, weight, nullptr, m, n, k, alpha, nullptr, 0, status, &gated);
}

cudaError_t launch_bf16_gemm_umma(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                  size_t n, size_t k, void* exchange, size_t exchange_bytes, unsigned int* status) {
    return launch_umma<true>(stream, x, weight, out, m, n, k * 2, 1.0f, exchange, exchange_bytes, status);
}

}  // namespace lfm25
