// RMSNorm + RoPE of one 64-wide attention head, shared by the stand-alone append kernel and the attention
// kernel's fused mode, so that both produce the same bits.
#pragma once

#include "common.cuh"

namespace lfm25 {

// Sum over the 32 lanes in the association order of a shuffle-down tree read at lane 0
// (16, 8, 4, 2, 1).  The xor butterfly adds the same pairs at every level, and addition is
// commutative, so every lane ends with exactly the bits lane 0 of the tree would hold.
__device__ __forceinline__ float warp_tree_sum(float value) {
#pragma unroll
    for (uint32_t delta = 16; delta > 0; delta >>= 1) {
        value += __shfl_xor_sync(0xffffffffu, value, delta);
    }
    return value;
}

// RMSNorm + RoPE of one 64-wide head held as (dim lane, dim lane+32) per lane.  The rounding
// points are the reference's (kernels/qk_postprocess.cu:21-30,104-112): normalise -> bf16 ->
// bf16 multiply by the weight -> fp32 rotation with fmaf -> bf16.
// The element-wise half of the above once the head's inverse RMS is known: dims d (< 32) and d + 32.
__device__ __forceinline__ void rotate_pair(float raw0, float raw1, float inv_rms, __nv_bfloat16 weight0,
                                            __nv_bfloat16 weight1, float sin_value, float cos_value,
                                            __nv_bfloat16& out0, __nv_bfloat16& out1) {
    const float x0 = __bfloat162float(__hmul(__float2bfloat16_rn(raw0 * inv_rms), weight0));
    const float x1 = __bfloat162float(__hmul(__float2bfloat16_rn(raw1 * inv_rms), weight1));
    out0 = __float2bfloat16_rn(fmaf(-x1, sin_value, x0 * cos_value));
    out1 = __float2bfloat16_rn(fmaf(x0, sin_value, x1 * cos_value));
}

__device__ __forceinline__ void norm_rope(float raw0, float raw1, __nv_bfloat16 weight0, __nv_bfloat16 weight1,
                                          float sin_value, float cos_value, float eps, __nv_bfloat16& out0,
                                          __nv_bfloat16& out1) {
    const float sum = warp_tree_sum(fmaf(raw0, raw0, raw1 * raw1));
    const float inv_rms = __frsqrt_rn(sum * (1.0f / 64.0f) + eps);
    rotate_pair(raw0, raw1, inv_rms, weight0, weight1, sin_value, cos_value, out0, out1);
}

}  // namespace lfm25
