// FP8 (E4M3) decode GEMM for small batches: Y[M,N] = bf16(alpha * Xq[M,K] * Wq[N,K]^T), fp32 accumulate.
//
// Replaces the reference's BlasLt::linear_fp8_scaled call into cuBLASLt for decode batches
// (src/cuda/blaslt/mod.rs:212-298; descriptor src/cuda/blaslt/fp8.rs:312-353): both operands are
// row-major E4M3 codes with K contiguous, the per-tensor scale product arrives as alpha.
//
// At M <= 8 the op is a stream of the weight matrix: N*K bytes from HBM against M*K bytes of
// activations that stay in L1/L2.  The kernel is built around that stream:
//  * "swap AB": 16 weight rows are the M=16 operand of mma.sync.m16n8k32 (e4m3 x e4m3 -> f32) and
//    8 batch rows are its N=8 operand, so one instruction consumes 512 weight bytes;
//  * weight fragments go from global memory straight to registers with 16-byte loads that no
//    other warp needs (no shared-memory staging): the reduction index of the MMA may be permuted
//    freely as long as both operands use the same permutation, so a lane takes 16 contiguous
//    bytes of a row where the canonical layout would want 4 + 4 from two places;
//  * each warp keeps kDepth 128-byte row chunks in flight per lane (software pipeline in registers);
//  * one CTA of 16 warps per SM, all resident at once: the weight matrix is cut into one contiguous share per
//    CTA and, inside it, one contiguous share of (tile, chunk) units per warp, so there is a single balanced
//    wave whatever N and K are (Down's 128 tiles x 64 chunks spread over 16 warps each, LM head's 4096 tiles
//    28 to a CTA); partial tiles meet in shared memory.
// Larger batches go to the tcgen05 kernel; shapes outside N % 16 == 0, K % 128 == 0 go to a plain
// one-warp-per-output-row kernel.
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace lfm25 {

namespace {

constexpr uint32_t kWarps = 16;
constexpr uint32_t kThreads = kWarps * 32;
constexpr uint32_t kDepth = 4;        // 128-byte chunks in flight per row per lane
constexpr uint32_t kChunk = 128;      // bytes of K per row per pipeline step = 4 MMAs
constexpr uint32_t kMaxTilesPerCta = 32;
constexpr uint32_t kSmCount = 148;

__device__ __forceinline__ uint4 load_stream(const uint8_t* pointer) {
    // weights are read exactly once: do not keep them in L1
    uint4 value;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
                 : "l"(pointer));
    return value;
}

struct WeightChunk {
    uint4 low_a, low_b;    // row g      : bytes [16c, 16c+16) and [64+16c, 64+16c+16) of the chunk
    uint4 high_a, high_b;  // row g + 8
};

// One CTA per SM, all resident at once (a single balanced wave).  CTA c owns a contiguous range of 16-row
// weight tiles; the (tile, 128-byte chunk) units of that range are dealt to the 16 warps in contiguous,
// equal shares, so every warp streams the same number of bytes and the register pipeline runs across tile
// boundaries.  A warp adds what it has of a tile into the CTA's fp32 tile array in shared memory when it
// moves on; the CTA scales, rounds and stores all its tiles at the end.  M <= 8: one 8-column batch tile.
__global__ void __launch_bounds__(kThreads, 1)
fp8_gemm_stream_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ weight,
                       __nv_bfloat16* __restrict__ out, uint32_t m, uint32_t n, uint32_t k, float alpha) {
    pdl_launch_dependents();
    __shared__ float tile_sums[kMaxTilesPerCta][16][8];
    // a warp's first and last tile may be shared with its neighbours: those partial tiles are parked here and
    // added in warp order afterwards, so the result does not depend on the order in which warps finish
    __shared__ float edge_sums[kWarps][2][16][8];
    __shared__ int edge_tile[kWarps][2];
    extern __shared__ __align__(16) uint8_t x_rows[];   // 8 batch rows of K + 64 bytes (the pad spreads the banks)
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t group = lane >> 2;
    const uint32_t quad = lane & 3;
    const uint32_t tiles = n / 16;
    const uint32_t chunks_per_tile = k / kChunk;
    const uint32_t tile_begin = static_cast<uint32_t>(static_cast<uint64_t>(tiles) * blockIdx.x / gridDim.x);
    const uint32_t tile_end = static_cast<uint32_t>(static_cast<uint64_t>(tiles) * (blockIdx.x + 1) / gridDim.x);
    const uint32_t cta_tiles = tile_end - tile_begin;
    const uint32_t units = cta_tiles * chunks_per_tile;
    const uint32_t unit_begin = static_cast<uint32_t>(static_cast<uint64_t>(units) * warp / kWarps);
    const uint32_t unit_end = static_cast<uint32_t>(static_cast<uint64_t>(units) * (warp + 1) / kWarps);

    const uint8_t* w_lane = weight + static_cast<size_t>(tile_begin * 16 + group) * k + quad * 16;
    const size_t tile_stride = static_cast<size_t>(16) * k;   // bytes between consecutive tiles
    const size_t half_stride = static_cast<size_t>(8) * k;    // row g -> row g + 8
    const uint32_t x_pitch = k + 64;
    const uint32_t x_lane = smem_u32(x_rows) + group * x_pitch + quad * 16;

    auto fetch = [&](WeightChunk& chunk, uint32_t unit) {
        const uint32_t tile = unit / chunks_per_tile;
        const uint32_t offset = (unit % chunks_per_tile) * kChunk;
        const uint8_t* low = w_lane + tile * tile_stride + offset;
        chunk.low_a = load_stream(low);
        chunk.low_b = load_stream(low + 64);
        chunk.high_a = load_stream(low + half_stride);
        chunk.high_b = load_stream(low + half_stride + 64);
    };

    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const bool has_work = unit_begin < unit_end;
    const uint32_t first_tile = has_work ? unit_begin / chunks_per_tile : 0;
    const uint32_t last_tile = has_work ? (unit_end - 1) / chunks_per_tile : 0;
    uint32_t current_tile = first_tile;
    if (lane == 0) {
        edge_tile[warp][0] = has_work ? static_cast<int>(first_tile) : -1;
        edge_tile[warp][1] = has_work && last_tile != first_tile ? static_cast<int>(last_tile) : -1;
    }
    auto flush = [&](uint32_t tile) {
        // accumulator: rows g, g + 8 of the tile; batch columns 2c, 2c + 1.  Interior tiles belong to this warp
        // alone and go straight to the tile array; the first and the last tile go to the warp's edge slots.
        float (*target)[8] = tile == first_tile ? edge_sums[warp][0]
                             : (tile == last_tile ? edge_sums[warp][1] : tile_sums[tile]);
        *reinterpret_cast<float2*>(&target[group][quad * 2]) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2*>(&target[group + 8][quad * 2]) = make_float2(acc[2], acc[3]);
        acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
    };
    auto consume = [&](const WeightChunk& chunk, uint32_t unit) {
        const uint32_t tile = unit / chunks_per_tile;
        if (tile != current_tile) {
            flush(current_tile);
            current_tile = tile;
        }
        uint4 xa;
        uint4 xb;
        const uint32_t x_address = x_lane + (unit % chunks_per_tile) * kChunk;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(xa.x), "=r"(xa.y), "=r"(xa.z), "=r"(xa.w) : "r"(x_address));
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(xb.x), "=r"(xb.y), "=r"(xb.z), "=r"(xb.w) : "r"(x_address + 64));
        mma_e4m3_16832(acc, chunk.low_a.x, chunk.high_a.x, chunk.low_a.y, chunk.high_a.y, xa.x, xa.y);
        mma_e4m3_16832(acc, chunk.low_a.z, chunk.high_a.z, chunk.low_a.w, chunk.high_a.w, xa.z, xa.w);
        mma_e4m3_16832(acc, chunk.low_b.x, chunk.high_b.x, chunk.low_b.y, chunk.high_b.y, xb.x, xb.y);
        mma_e4m3_16832(acc, chunk.low_b.z, chunk.high_b.z, chunk.low_b.w, chunk.high_b.w, xb.z, xb.w);
    };

    // The weight stream starts first; while it is in flight the CTA brings the activations (at most 64 KiB,
    // L2-resident) into shared memory, batch rows beyond M as zeros, and clears its tile sums.
    WeightChunk ring[kDepth];
#pragma unroll
    for (uint32_t stage = 0; stage < kDepth; ++stage) {
        if (unit_begin + stage < unit_end) {
            fetch(ring[stage], unit_begin + stage);
        }
    }
    // Everything above touched only the weights, which no kernel writes; the activations come from the
    // predecessor in the stream, so they are read after the dependency wait.
    pdl_wait();
    {
        const uint32_t vectors_per_row = k / 16;
        for (uint32_t index = threadIdx.x; index < 8 * vectors_per_row; index += kThreads) {
            const uint32_t row = index / vectors_per_row;
            const uint32_t vector = index % vectors_per_row;
            uint4 value = make_uint4(0, 0, 0, 0);
            if (row < m) {
                value = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * k) + vector);
            }
            *reinterpret_cast<uint4*>(x_rows + row * x_pitch + vector * 16) = value;
        }
        for (uint32_t index = threadIdx.x; index < cta_tiles * 128; index += kThreads) {
            (&tile_sums[0][0][0])[index] = 0.0f;
        }
    }
    __syncthreads();
    for (uint32_t base = unit_begin; base < unit_end; base += kDepth) {
#pragma unroll
        for (uint32_t stage = 0; stage < kDepth; ++stage) {
            const uint32_t unit = base + stage;
            if (unit < unit_end) {
                consume(ring[stage], unit);
                if (unit + kDepth < unit_end) {
                    fetch(ring[stage], unit + kDepth);
                }
            }
        }
    }
    if (has_work) {
        flush(current_tile);
    }
    __syncthreads();

    // ---- scale, round, store: thread -> (tile, row, batch) with rows fastest, so stores of one batch row coalesce
    const uint32_t cells = cta_tiles * 16;
    for (uint32_t batch = 0; batch < m; ++batch) {
        for (uint32_t cell = threadIdx.x; cell < cells; cell += kThreads) {
            const uint32_t tile = cell >> 4;
            const uint32_t row = cell & 15;
            float sum = tile_sums[tile][row][batch];
#pragma unroll
            for (uint32_t other = 0; other < kWarps; ++other) {
                if (edge_tile[other][0] == static_cast<int>(tile)) sum += edge_sums[other][0][row][batch];
                if (edge_tile[other][1] == static_cast<int>(tile)) sum += edge_sums[other][1][row][batch];
            }
            out[static_cast<size_t>(batch) * n + (tile_begin + tile) * 16 + row] = __float2bfloat16_rn(sum * alpha);
        }
    }
}

// Any shape: one warp per output row, 256-entry decode table in shared memory, fp32 accumulate.
__global__ void __launch_bounds__(256)
fp8_gemm_generic_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ weight,
                        __nv_bfloat16* __restrict__ out, uint32_t m, uint32_t n, uint32_t k, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float table[256];
    {
        const uint32_t code = threadIdx.x;
        const uint32_t exponent = (code >> 3) & 0xf;
        const uint32_t mantissa = code & 7;
        float magnitude;
        if (exponent == 0xf && mantissa == 7) {
            magnitude = __int_as_float(0x7fc00000);
        } else if (exponent == 0) {
            magnitude = ldexpf(static_cast<float>(mantissa), -9);
        } else {
            magnitude = ldexpf(1.0f + static_cast<float>(mantissa) * 0.125f, static_cast<int>(exponent) - 7);
        }
        table[code] = (code & 0x80) ? -magnitude : magnitude;
    }
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31;
    const size_t row = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (row >= n) {
        return;
    }
    const uint8_t* w_row = weight + row * k;
    for (uint32_t batch = 0; batch < m; ++batch) {
        const uint8_t* x_row = x + static_cast<size_t>(batch) * k;
        float sum = 0.0f;
        for (uint32_t inner = lane; inner < k; inner += 32) {
            sum = fmaf(table[x_row[inner]], table[w_row[inner]], sum);
        }
#pragma unroll
        for (uint32_t delta = 16; delta > 0; delta >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, delta);
        }
        if (lane == 0) {
            out[static_cast<size_t>(batch) * n + row] = __float2bfloat16_rn(sum * alpha);
        }
    }
}

}  // namespace

bool fp8_gemm_stream_supports(size_t m, size_t n, size_t k) {
    return m >= 1 && m <= 8 && n % 16 == 0 && k % kChunk == 0 && n <= 0x7fffffffu && k <= 16384 &&
           n / 16 <= static_cast<size_t>(kMaxTilesPerCta) * kSmCount;
}

cudaError_t launch_fp8_gemm_stream(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                   size_t n, size_t k, float alpha) {
    const uint32_t tiles = static_cast<uint32_t>(n / 16);
    const uint32_t blocks = tiles < kSmCount ? tiles : kSmCount;
    const size_t x_bytes = 8 * (k + 64);
    const cudaError_t attribute_status = cudaFuncSetAttribute(
        fp8_gemm_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(x_bytes));
    if (attribute_status != cudaSuccess) {
        return attribute_status;
    }
    return launch_kernel(fp8_gemm_stream_kernel, blocks, kThreads, x_bytes, stream, 1, 
        static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(weight), static_cast<__nv_bfloat16*>(out),
        static_cast<uint32_t>(m), static_cast<uint32_t>(n), static_cast<uint32_t>(k), alpha);
}

cudaError_t launch_fp8_gemm_generic(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                    size_t n, size_t k, float alpha) {
    const unsigned int blocks = static_cast<unsigned int>((n + 7) / 8);
    return launch_kernel(fp8_gemm_generic_kernel, blocks, 256, 0, stream, 1, 
        static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(weight), static_cast<__nv_bfloat16*>(out),
        static_cast<uint32_t>(m), static_cast<uint32_t>(n), static_cast<uint32_t>(k), alpha);
}

}  // namespace lfm25
