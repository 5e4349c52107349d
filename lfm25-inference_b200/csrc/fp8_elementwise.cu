// Element-wise FP8 producers for sm_100a.
//
// quantize         : replaces kernels/fp8_quantize.cu:9-45 of the reference,
//                    code = cvt.rn.satfinite.e4m3(float(x) * scale).
// silu_mul (bf16)  : replaces kernels/silu_mul.cu:13-61, h = bf16(silu(gate) * up) on packed rows.
// silu_mul -> e4m3 : replaces kernels/silu_mul.cu:68-133, code = e4m3(float(h) * scale); h is rounded
//                    to bf16 first, exactly as the unfused pipeline would.
//
// All three are streaming kernels bound by HBM: 16-byte loads, 8 elements per thread, a grid of
// a few CTAs per SM looping with a grid stride.
#include <cuda_fp8.h>

#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace lfm25 {

namespace {

constexpr uint32_t kThreads = 256;

__device__ __forceinline__ uint8_t e4m3x1(float value) {
    return static_cast<uint8_t>(e4m3x2(value, 0.0f) & 0xffu);
}

// 8 bf16 -> 8 codes
__device__ __forceinline__ uint2 quantize8(const uint4 raw, float scale) {
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint32_t packed[2];
#pragma unroll
    for (uint32_t half = 0; half < 2; ++half) {
        const float2 a = __bfloat1622float2(pairs[half * 2]);
        const float2 b = __bfloat1622float2(pairs[half * 2 + 1]);
        packed[half] = static_cast<uint32_t>(e4m3x2(a.x * scale, a.y * scale)) |
                       (static_cast<uint32_t>(e4m3x2(b.x * scale, b.y * scale)) << 16);
    }
    return make_uint2(packed[0], packed[1]);
}

__global__ void __launch_bounds__(kThreads)
quantize_bf16_e4m3_kernel(const __nv_bfloat16* __restrict__ input, uint8_t* __restrict__ output, size_t numel,
                          float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t thread = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(input) & 15) == 0) && ((reinterpret_cast<uintptr_t>(output) & 7) == 0);
    const size_t vectors = aligned ? numel / 8 : 0;
    for (size_t vector = thread; vector < vectors; vector += stride) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(input) + vector);
        reinterpret_cast<uint2*>(output)[vector] = quantize8(raw, scale);
    }
    for (size_t index = vectors * 8 + thread; index < numel; index += stride) {
        output[index] = e4m3x1(__bfloat162float(input[index]) * scale);
    }
}

// FUSED == true writes E4M3 codes, false writes the bf16 activation.
template <bool FUSED>
__global__ void __launch_bounds__(kThreads)
silu_mul_packed_kernel(const __nv_bfloat16* __restrict__ packed, void* __restrict__ out, size_t rows,
                       size_t intermediate, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t thread = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const bool vector_ok = (intermediate % 8 == 0) && ((reinterpret_cast<uintptr_t>(packed) & 15) == 0) &&
                           ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    if (vector_ok) {
        const size_t vectors_per_row = intermediate / 8;
        const size_t vectors = rows * vectors_per_row;
        for (size_t vector = thread; vector < vectors; vector += stride) {
            const size_t row = vector / vectors_per_row;
            const size_t column = vector % vectors_per_row;
            const uint4* gate_row = reinterpret_cast<const uint4*>(packed + row * 2 * intermediate);
            const uint4 gate_raw = __ldg(gate_row + column);
            const uint4 up_raw = __ldg(gate_row + vectors_per_row + column);
            const __nv_bfloat162* gate = reinterpret_cast<const __nv_bfloat162*>(&gate_raw);
            const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&up_raw);
            uint4 hidden;
            __nv_bfloat162* hidden_pairs = reinterpret_cast<__nv_bfloat162*>(&hidden);
#pragma unroll
            for (uint32_t pair = 0; pair < 4; ++pair) {
                const float2 g = __bfloat1622float2(gate[pair]);
                const float2 u = __bfloat1622float2(up[pair]);
                hidden_pairs[pair] = __floats2bfloat162_rn(silu(g.x) * u.x, silu(g.y) * u.y);
            }
            if (FUSED) {
                reinterpret_cast<uint2*>(out)[vector] = quantize8(hidden, scale);
            } else {
                reinterpret_cast<uint4*>(out)[vector] = hidden;
            }
        }
        return;
    }
    const size_t elements = rows * intermediate;
    for (size_t index = thread; index < elements; index += stride) {
        const size_t row = index / intermediate;
        const size_t column = index % intermediate;
        const float g = __bfloat162float(packed[row * 2 * intermediate + column]);
        const float u = __bfloat162float(packed[row * 2 * intermediate + intermediate + column]);
        const __nv_bfloat16 hidden = __float2bfloat16_rn(silu(g) * u);
        if (FUSED) {
            static_cast<uint8_t*>(out)[index] = e4m3x1(__bfloat162float(hidden) * scale);
        } else {
            static_cast<__nv_bfloat16*>(out)[index] = hidden;
        }
    }
}

unsigned int streaming_grid(size_t work_items) {
    const size_t blocks = (work_items + kThreads - 1) / kThreads;
    const size_t cap = 148 * 8;  // 8 resident CTAs of 256 threads per SM
    return static_cast<unsigned int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

cudaError_t launch_quantize_bf16_e4m3(cudaStream_t stream, const void* input, void* output, size_t numel,
                                      float scale) {
    return launch_kernel(quantize_bf16_e4m3_kernel, streaming_grid((numel + 7) / 8), kThreads, 0, stream, 1, 
        static_cast<const __nv_bfloat16*>(input), static_cast<uint8_t*>(output), numel, scale);
}

cudaError_t launch_silu_mul_packed_bf16(cudaStream_t stream, const void* packed, void* out, size_t rows,
                                        size_t intermediate) {
    return launch_kernel(silu_mul_packed_kernel<false>, streaming_grid((rows * intermediate + 7) / 8), kThreads, 0, stream, 1, 
        static_cast<const __nv_bfloat16*>(packed), out, rows, intermediate, 1.0f);
}

cudaError_t launch_silu_mul_packed_bf16_to_e4m3(cudaStream_t stream, const void* packed, void* out, size_t rows,
                                                size_t intermediate, float scale) {
    return launch_kernel(silu_mul_packed_kernel<true>, streaming_grid((rows * intermediate + 7) / 8), kThreads, 0, stream, 1, 
        static_cast<const __nv_bfloat16*>(packed), out, rows, intermediate, scale);
}

}  // namespace lfm25
