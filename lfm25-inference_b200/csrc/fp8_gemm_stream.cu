// FP8 (E4M3) decode GEMM for small batches: Y[M,N] = bf16(alpha * Xq[M,K] * Wq[N,K]^T), fp32 accumulate.
//
// Replaces the reference's BlasLt::linear_fp8_scaled call into cuBLASLt for decode batches
// (src/cuda/blaslt/mod.rs:212-298; descriptor src/cuda/blaslt/fp8.rs:312-353): both operands are
// row-major E4M3 codes with K contiguous, the per-tensor scale product arrives as alpha.
//
// At M <= 64 the op is a stream of the weight matrix: N*K bytes from HBM against M*K bytes of
// activations that stay in L1/L2.  The kernel is built around that stream:
//  * "swap AB": 16 weight rows are the M=16 operand of mma.sync.m16n8k32 (e4m3 x e4m3 -> f32) and
//    8 batch rows are its N=8 operand, so one instruction consumes 512 weight bytes;
//  * weight fragments go from global memory straight to registers with 16-byte loads that no
//    other warp needs (no shared-memory staging): the reduction index of the MMA may be permuted
//    freely as long as both operands use the same permutation, so a lane takes 16 contiguous
//    bytes of a row where the canonical layout would want 4 + 4 from two places;
//  * each warp keeps kDepth 128-byte row chunks in flight per lane (software pipeline in registers);
//  * K is split over the warps of a CTA when N alone does not give enough warps (Down, K = 8192),
//    partial tiles are combined through shared memory.
// Shapes outside N % 16 == 0, K % 128 == 0 go to a plain one-warp-per-output-row kernel.
#include "common.cuh"
#include "kernels.h"

namespace lfm25 {

namespace {

constexpr uint32_t kWarps = 4;
constexpr uint32_t kThreads = kWarps * 32;
constexpr uint32_t kDepth = 4;        // 128-byte chunks in flight per row per lane
constexpr uint32_t kChunk = 128;      // bytes of K per row per pipeline step = 4 MMAs

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

// NT = number of 8-row batch tiles (M <= 8*NT), KSPLIT = warps of a CTA that share one row tile.
template <uint32_t NT, uint32_t KSPLIT>
__global__ void __launch_bounds__(kThreads)
fp8_gemm_stream_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ weight,
                       __nv_bfloat16* __restrict__ out, uint32_t m, uint32_t n, uint32_t k, float alpha) {
    constexpr uint32_t kTilesPerCta = kWarps / KSPLIT;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t group = lane >> 2;
    const uint32_t quad = lane & 3;
    const uint32_t tile = blockIdx.x * kTilesPerCta + warp / KSPLIT;
    const uint32_t slice = warp % KSPLIT;
    const uint32_t row0 = tile * 16;
    const bool tile_valid = row0 < n;

    const uint32_t k_per_slice = k / KSPLIT;
    const uint32_t k_begin = slice * k_per_slice;
    const uint32_t chunks = k_per_slice / kChunk;

    float acc[NT][4];
#pragma unroll
    for (uint32_t nt = 0; nt < NT; ++nt) {
        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    }

    if (tile_valid) {
        const uint8_t* w_low = weight + static_cast<size_t>(row0 + group) * k + k_begin + quad * 16;
        const uint8_t* w_high = w_low + static_cast<size_t>(8) * k;
        const uint8_t* x_lane = x + static_cast<size_t>(group) * k + k_begin + quad * 16;

        auto fetch = [&](WeightChunk& chunk, uint32_t index) {
            const uint32_t offset = index * kChunk;
            chunk.low_a = load_stream(w_low + offset);
            chunk.low_b = load_stream(w_low + offset + 64);
            chunk.high_a = load_stream(w_high + offset);
            chunk.high_b = load_stream(w_high + offset + 64);
        };
        auto consume = [&](const WeightChunk& chunk, uint32_t index) {
            const uint32_t offset = index * kChunk;
#pragma unroll
            for (uint32_t nt = 0; nt < NT; ++nt) {
                uint4 xa = make_uint4(0, 0, 0, 0);
                uint4 xb = make_uint4(0, 0, 0, 0);
                if (nt * 8 + group < m) {
                    const uint8_t* x_row = x_lane + static_cast<size_t>(nt * 8) * k + offset;
                    xa = __ldg(reinterpret_cast<const uint4*>(x_row));
                    xb = __ldg(reinterpret_cast<const uint4*>(x_row + 64));
                }
                mma_e4m3_16832(acc[nt], chunk.low_a.x, chunk.high_a.x, chunk.low_a.y, chunk.high_a.y, xa.x, xa.y);
                mma_e4m3_16832(acc[nt], chunk.low_a.z, chunk.high_a.z, chunk.low_a.w, chunk.high_a.w, xa.z, xa.w);
                mma_e4m3_16832(acc[nt], chunk.low_b.x, chunk.high_b.x, chunk.low_b.y, chunk.high_b.y, xb.x, xb.y);
                mma_e4m3_16832(acc[nt], chunk.low_b.z, chunk.high_b.z, chunk.low_b.w, chunk.high_b.w, xb.z, xb.w);
            }
        };

        WeightChunk ring[kDepth];
#pragma unroll
        for (uint32_t stage = 0; stage < kDepth; ++stage) {
            if (stage < chunks) {
                fetch(ring[stage], stage);
            }
        }
        for (uint32_t base = 0; base < chunks; base += kDepth) {
#pragma unroll
            for (uint32_t stage = 0; stage < kDepth; ++stage) {
                const uint32_t index = base + stage;
                if (index < chunks) {
                    consume(ring[stage], index);
                    if (index + kDepth < chunks) {
                        fetch(ring[stage], index + kDepth);
                    }
                }
            }
        }
    }

    // ---- combine the K slices of a row tile, scale, round, store ----
    if (KSPLIT > 1) {
        __shared__ float partial[kWarps][NT * 4][32];
#pragma unroll
        for (uint32_t nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (uint32_t index = 0; index < 4; ++index) {
                partial[warp][nt * 4 + index][lane] = acc[nt][index];
            }
        }
        __syncthreads();
        if (slice != 0) {
            return;
        }
#pragma unroll
        for (uint32_t other = 1; other < KSPLIT; ++other) {
#pragma unroll
            for (uint32_t nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (uint32_t index = 0; index < 4; ++index) {
                    acc[nt][index] += partial[warp + other][nt * 4 + index][lane];
                }
            }
        }
    }
    if (!tile_valid) {
        return;
    }
    // accumulator (row g / g+8 of the weight tile, batch columns 2c, 2c+1 of batch tile nt)
#pragma unroll
    for (uint32_t nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (uint32_t index = 0; index < 4; ++index) {
            const uint32_t batch = nt * 8 + quad * 2 + (index & 1);
            const uint32_t row = row0 + group + ((index >> 1) << 3);
            if (batch < m) {
                out[static_cast<size_t>(batch) * n + row] = __float2bfloat16_rn(acc[nt][index] * alpha);
            }
        }
    }
}

// Any shape: one warp per output row, 256-entry decode table in shared memory, fp32 accumulate.
__global__ void __launch_bounds__(256)
fp8_gemm_generic_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ weight,
                        __nv_bfloat16* __restrict__ out, uint32_t m, uint32_t n, uint32_t k, float alpha) {
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

template <uint32_t NT, uint32_t KSPLIT>
cudaError_t launch_stream(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m, size_t n,
                          size_t k, float alpha) {
    const uint32_t tiles = static_cast<uint32_t>(n / 16);
    const uint32_t tiles_per_cta = kWarps / KSPLIT;
    const uint32_t blocks = (tiles + tiles_per_cta - 1) / tiles_per_cta;
    fp8_gemm_stream_kernel<NT, KSPLIT><<<blocks, kThreads, 0, stream>>>(
        static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(weight), static_cast<__nv_bfloat16*>(out),
        static_cast<uint32_t>(m), static_cast<uint32_t>(n), static_cast<uint32_t>(k), alpha);
    return cudaGetLastError();
}

template <uint32_t NT>
cudaError_t launch_stream_nt(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m, size_t n,
                             size_t k, float alpha) {
    // Enough (row tile, K slice) warps to cover the machine: at least ~16 warps per SM.
    const size_t tiles = n / 16;
    uint32_t ksplit = 1;
    while (ksplit < kWarps && tiles * ksplit < 148 * 16 && (k / (ksplit * 2)) % kChunk == 0 &&
           k / (ksplit * 2) >= 4 * kChunk) {
        ksplit *= 2;
    }
    switch (ksplit) {
        case 1: return launch_stream<NT, 1>(stream, x, weight, out, m, n, k, alpha);
        case 2: return launch_stream<NT, 2>(stream, x, weight, out, m, n, k, alpha);
        default: return launch_stream<NT, 4>(stream, x, weight, out, m, n, k, alpha);
    }
}

}  // namespace

bool fp8_gemm_stream_supports(size_t m, size_t n, size_t k) {
    return m >= 1 && m <= 64 && n % 16 == 0 && k % kChunk == 0 && n <= 0x7fffffffu && k <= 0x7fffffffu;
}

cudaError_t launch_fp8_gemm_stream(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                   size_t n, size_t k, float alpha) {
    if (m <= 8) return launch_stream_nt<1>(stream, x, weight, out, m, n, k, alpha);
    if (m <= 16) return launch_stream_nt<2>(stream, x, weight, out, m, n, k, alpha);
    if (m <= 32) return launch_stream_nt<4>(stream, x, weight, out, m, n, k, alpha);
    return launch_stream_nt<8>(stream, x, weight, out, m, n, k, alpha);
}

cudaError_t launch_fp8_gemm_generic(cudaStream_t stream, const void* x, const void* weight, void* out, size_t m,
                                    size_t n, size_t k, float alpha) {
    const unsigned int blocks = static_cast<unsigned int>((n + 7) / 8);
    fp8_gemm_generic_kernel<<<blocks, 256, 0, stream>>>(
        static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(weight), static_cast<__nv_bfloat16*>(out),
        static_cast<uint32_t>(m), static_cast<uint32_t>(n), static_cast<uint32_t>(k), alpha);
    return cudaGetLastError();
}

}  // namespace lfm25
