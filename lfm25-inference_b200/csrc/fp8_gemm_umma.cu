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
//   warps 2-5  epilogue: tcgen05.ld the accumulator (thread = weight row, registers = batch columns),
//            scale, round to bf16, store; a warp's store covers 32 consecutive outputs of one batch row
//
// The op is bound by the weight stream (N*K bytes) for every batch size here, so what matters is the number
// of bytes in flight: stages are as deep as shared memory allows (up to 8 x 16 KiB of weights per SM).
// When N/128 tiles cannot occupy the machine (Down: 16 tiles), K is split over the CTAs of a thread-block
// cluster (up to 8 per tile).  Each parks its fp32 partial tile in its own shared memory; after a cluster
// barrier every CTA finishes one slice of the batch columns, reading the partners' tiles through distributed
// shared memory and adding them in rank order (reproducible, no atomics, no workspace, no second launch).
//
// Every mbarrier wait is bounded; a wait that runs out sets an abort flag, is recorded in the device
// status words, and the CTA still frees its TMEM and exits.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "launch.h"
#include "tensor_map.h"

namespace lfm25 {

namespace {

constexpr uint32_t kTileN = 128;    // weight rows per CTA = UMMA M
constexpr uint32_t kBlockK = 128;   // bytes of K per stage = one swizzle row
constexpr uint32_t kUmmaK = 32;     // K of one tcgen05.mma with 8-bit operands
constexpr uint32_t kThreads = 192;
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kSmemBudget = 200 * 1024;   // one CTA per SM
constexpr uint32_t kSmemBudgetShared = 98 * 1024;  // two CTAs per SM: one drains its tile while the other streams
constexpr uint32_t kWeightTileBytes = kTileN * kBlockK;

struct UmmaParams {
    __nv_bfloat16* out;
    unsigned int* status;
    uint32_t m;
    uint32_t n;
    uint32_t m_pad;          // batch rounded up to 16 = UMMA N
    uint32_t stages;
    uint32_t data_bytes;     // shared memory in front of the control block: the stages, or the parked tile
    uint32_t k_blocks;       // 128-byte K blocks per split
    uint32_t splits;         // CTAs of a cluster that share one weight tile, each with its own K range
    uint32_t tmem_columns;   // power of two >= max(32, m_pad)
    float alpha;
};

__device__ __forceinline__ uint64_t smem_descriptor(uint32_t address) {
    // K-major operand, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart
    uint64_t descriptor = static_cast<uint64_t>((address & 0x3ffff) >> 4);
    descriptor |= static_cast<uint64_t>(1) << 16;            // leading byte offset (unused with swizzle)
    descriptor |= static_cast<uint64_t>(1024 >> 4) << 32;    // stride byte offset between 8-row groups
    descriptor |= static_cast<uint64_t>(1) << 46;            // descriptor version of sm_100
    descriptor |= static_cast<uint64_t>(2) << 61;            // SWIZZLE_128B
    return descriptor;
}

__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
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
__device__ __forceinline__ float load_peer_smem(uint32_t local_address, uint32_t peer) {
    uint32_t remote;
    float value;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(peer));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(value) : "r"(remote) : "memory");
    return value;
}

__device__ __forceinline__ void tmem_load16(uint32_t address, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kThreads, 2)
fp8_gemm_umma_kernel(const __grid_constant__ CUtensorMap weight_map, const __grid_constant__ CUtensorMap x_map,
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

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&weight_map);
        tma_prefetch_descriptor(&x_map);
        for (uint32_t stage = 0; stage < p.stages; ++stage) {
            mbar_init(bar_full + 8 * stage, 1);
            mbar_init(bar_empty + 8 * stage, 1);
        }
        mbar_init(bar_accumulator, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
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

    const uint32_t k_block0 = split * p.k_blocks;

    if (warp == 0) {
        if (lane == 0) {
            // The weight tiles are constants: the first ring of them is requested before the dependency wait, so
            // the stream is already flowing while the predecessor kernel drains.  The activation tiles, which the
            // predecessor writes, follow after the wait and complete the same barriers.
            const uint32_t ahead = p.k_blocks < p.stages ? p.k_blocks : p.stages;
            const int32_t tile_row = static_cast<int32_t>(tile * kTileN);
            for (uint32_t block = 0; block < ahead; ++block) {
                const uint32_t bar = bar_full + 8 * block;
                mbar_arrive_expect_tx(bar, stage_bytes);
                tma_load_2d(smem_base + block * stage_bytes, &weight_map, bar,
                            static_cast<int32_t>((k_block0 + block) * kBlockK), tile_row);
            }
            pdl_wait();
            for (uint32_t block = 0; block < ahead; ++block) {
                tma_load_2d(smem_base + block * stage_bytes + kWeightTileBytes, &x_map, bar_full + 8 * block,
                            static_cast<int32_t>((k_block0 + block) * kBlockK), 0);
            }
            for (uint32_t block = ahead; block < p.k_blocks; ++block) {
                const uint32_t stage = block % p.stages;
                if (*abort_flag || !mbar_wait_bounded(bar_empty + 8 * stage, ((block / p.stages) - 1) & 1)) {
                    *abort_flag = 1;
                    record_wait_timeout(p.status, kTagGemmUmma, (blockIdx.x << 4) | 1);
                    break;
                }
                const uint32_t bar = bar_full + 8 * stage;
                const uint32_t dst = smem_base + stage * stage_bytes;
                const int32_t k_offset = static_cast<int32_t>((k_block0 + block) * kBlockK);
                mbar_arrive_expect_tx(bar, stage_bytes);
                tma_load_2d(dst, &weight_map, bar, k_offset, tile_row);
                tma_load_2d(dst + kWeightTileBytes, &x_map, bar, k_offset, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D = f32, A = B = E4M3, both K-major, N = m_pad, M = 128
            const uint32_t idesc = (1u << 4) | ((p.m_pad >> 3) << 17) | ((kTileN >> 4) << 24);
            bool ok = true;
            for (uint32_t block = 0; block < p.k_blocks && ok; ++block) {
                const uint32_t stage = block % p.stages;
                if (*abort_flag || !mbar_wait_bounded(bar_full + 8 * stage, (block / p.stages) & 1)) {
                    *abort_flag = 1;
                    record_wait_timeout(p.status, kTagGemmUmma, (blockIdx.x << 4) | 2);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t a_address = smem_base + stage * stage_bytes;
                const uint64_t a_desc = smem_descriptor(a_address);
                const uint64_t b_desc = smem_descriptor(a_address + kWeightTileBytes);
#pragma unroll
                for (uint32_t step = 0; step < kBlockK / kUmmaK; ++step) {
                    // advancing 32 bytes inside the swizzle row = +2 in the (address >> 4) field
                    umma_f8(tmem_base, a_desc + step * 2, b_desc + step * 2, idesc, (block | step) != 0 ? 1u : 0u);
                }
                umma_commit(bar_empty + 8 * stage);
            }
            if (ok) {
                umma_commit(bar_accumulator);
            }
        }
    } else {
        // ---- epilogue: 4 warps, each owns the 32 TMEM lanes of its quadrant (warp id modulo 4) ----
        const uint32_t quadrant = warp & 3;
        const uint32_t row = tile * kTileN + quadrant * 32 + lane;   // weight row = output column
        pdl_wait();   // the output buffer may still be read by an earlier kernel until the dependency resolves
        const bool ready = !*abort_flag && mbar_wait_bounded(bar_accumulator, 0);
        if (!ready) {
            if (lane == 0) {
                *abort_flag = 1;
                record_wait_timeout(p.status, kTagGemmUmma, (blockIdx.x << 4) | 3);
            }
        } else {
            tcgen05_fence_after();
            const uint32_t lane_address = tmem_base + ((quadrant * 32) << 16);
            for (uint32_t column0 = 0; column0 < p.m_pad; column0 += 16) {
                uint32_t raw[16];
                tmem_load16(lane_address + column0, raw);
                if (p.splits == 1) {
#pragma unroll
                    for (uint32_t j = 0; j < 16; ++j) {
                        const uint32_t batch = column0 + j;
                        if (batch < p.m) {
                            p.out[static_cast<size_t>(batch) * p.n + row] =
                                __float2bfloat16_rn(__uint_as_float(raw[j]) * p.alpha);
                        }
                    }
                } else {
                    // park the partial tile in this CTA's (now idle) pipeline memory as fp32 [column][128 rows]
                    float* parked = reinterpret_cast<float*>(smem);
#pragma unroll
                    for (uint32_t j = 0; j < 16; ++j) {
                        parked[(column0 + j) * kTileN + quadrant * 32 + lane] = __uint_as_float(raw[j]);
                    }
                }
            }
        }
    }

    if (p.splits > 1) {
        // Reduce-scatter across the cluster: rank q finishes the batch columns [q, q+1) * m_pad / splits of the
        // tile, adding the partners' parked tiles in rank order (so the sum is reproducible).
        tcgen05_fence_before();
        cluster_sync_all();
        if (warp >= 2 && !*abort_flag) {
            const uint32_t quadrant = warp & 3;
            const uint32_t row_in_tile = quadrant * 32 + lane;
            const uint32_t columns = p.m_pad / p.splits;
            const uint32_t parked_base = smem_base;
            // columns is even (m_pad is a multiple of 16, splits at most 8).  All remote loads of a column pair
            // are issued before the first add, so their latencies overlap instead of adding up.
            for (uint32_t index = 0; index < columns; index += 2) {
                const uint32_t batch = split * columns + index;
                float part[2][8];
#pragma unroll
                for (uint32_t column = 0; column < 2; ++column) {
#pragma unroll
                    for (uint32_t peer = 0; peer < 8; ++peer) {
                        part[column][peer] = 0.0f;
                        if (peer < p.splits) {
                            part[column][peer] =
                                load_peer_smem(parked_base + ((batch + column) * kTileN + row_in_tile) * 4, peer);
                        }
                    }
                }
#pragma unroll
                for (uint32_t column = 0; column < 2; ++column) {
                    float sum = 0.0f;
#pragma unroll
                    for (uint32_t peer = 0; peer < 8; ++peer) {
                        sum += part[column][peer];   // rank order; absent ranks contribute exact zeros
                    }
                    if (batch + column < p.m) {
                        p.out[static_cast<size_t>(batch + column) * p.n + tile * kTileN + row_in_tile] =
                            __float2bfloat16_rn(sum * p.alpha);
                    }
                }
            }
        }
        cluster_sync_all();   // nobody leaves while a partner may still read its shared memory
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

cudaError_t launch_fp8_gemm_umma(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                 size_t n, size_t k, float alpha, unsigned int* status) {
    const uint32_t m_pad = static_cast<uint32_t>((m + 15) / 16 * 16);
    CUtensorMap weight_map;
    CUtensorMap x_map;
    if (!make_swizzled_2d_map(&weight_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, weight, n, k, kTileN) ||
        !make_swizzled_2d_map(&x_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x, m, k, m_pad)) {
        return cudaErrorInvalidValue;
    }
    const uint32_t tiles = static_cast<uint32_t>(n / kTileN);
    const uint32_t k_blocks_total = static_cast<uint32_t>(k / kBlockK);
    // Split K (cluster of up to 8 CTAs per tile) only while the tiles alone leave most SMs idle.
    uint32_t splits = 1;
    while (splits < 8 && tiles * splits * 2 <= 148 && k_blocks_total % (splits * 2) == 0 &&
           k_blocks_total / (splits * 2) >= 4) {
        splits *= 2;
    }
    const uint32_t stage_bytes = kWeightTileBytes + m_pad * kBlockK;
    // With more CTAs than SMs (LM head: 512 tiles) two CTAs share an SM, so that the epilogue of one tile
    // overlaps the weight stream of the next; otherwise one CTA takes the whole shared memory for depth.
    const bool share_sm = tiles * splits > 148 && kSmemBudgetShared / stage_bytes >= 3;
    uint32_t stages = (share_sm ? kSmemBudgetShared : kSmemBudget) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    const uint32_t k_blocks = k_blocks_total / splits;
    if (stages > k_blocks) stages = k_blocks;
    uint32_t data_bytes = stages * stage_bytes;
    const uint32_t parked_bytes = splits > 1 ? m_pad * kTileN * 4 : 0;
    if (data_bytes < parked_bytes) data_bytes = parked_bytes;
    const uint32_t smem_bytes = data_bytes + 16 * kMaxStages + 64 + 1024;

    UmmaParams params;
    params.out = static_cast<__nv_bfloat16*>(out);
    params.status = status;
    params.m = static_cast<uint32_t>(m);
    params.n = static_cast<uint32_t>(n);
    params.m_pad = m_pad;
    params.stages = stages;
    params.data_bytes = data_bytes;
    params.k_blocks = k_blocks;
    params.splits = splits;
    params.tmem_columns = 32;
    while (params.tmem_columns < m_pad) params.tmem_columns *= 2;
    params.alpha = alpha;

    const cudaError_t attribute_status = cudaFuncSetAttribute(
        fp8_gemm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes));
    if (attribute_status != cudaSuccess) {
        return attribute_status;
    }
    return launch_kernel(fp8_gemm_umma_kernel, tiles * splits, kThreads, smem_bytes, stream, splits, weight_map, x_map,
                         params);
}

}  // namespace lfm25
