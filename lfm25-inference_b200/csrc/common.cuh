// Shared device helpers for the sm_100a kernels of the LFM2.5 decode path:
// model constants, PTX wrappers (mbarrier, TMA, ldmatrix, mma.sync) and the
// bounded-wait / device-status convention.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lfm25 {

// Model shape of LFM2.5-1.2B attention (fixed in the reference's kernels as well).
constexpr uint32_t kQHeads = 32;
constexpr uint32_t kKvHeads = 8;
constexpr uint32_t kHeadDim = 64;
constexpr uint32_t kHalfDim = 32;
constexpr uint32_t kQPerKv = 4;
constexpr uint32_t kPageSize = 16;
constexpr uint32_t kPartialStride = 66;  // (max, denominator, acc[64]) per split record
constexpr float kAttnScale = 0.125f;
constexpr float kLog2e = 1.4426950408889634f;

// One K (or V) page of one KV head: 16 tokens x 64 dims of bf16, contiguous in the arena.
constexpr uint32_t kPageTileBytes = kPageSize * kHeadDim * 2;  // 2048

// Device status words.  A kernel that gives up on a bounded wait records where, instead of
// trapping or spinning for ever; the host reads the words with lfm25_device_status().  The
// words live in one translation unit (api.cu); kernels receive their device address.
//   [0] number of waits that ran out   [1] kernel tag of the last one   [2] detail (stage / item)
enum StatusTag : uint32_t {
    kTagAttention = 1,
    kTagGemmStream = 2,
    kTagGemmUmma = 3,
    kTagHybridAttention = 4,
    kTagGemmRows = 5
};
__device__ __forceinline__ void record_wait_timeout(unsigned int* status, uint32_t tag, uint32_t detail) {
    atomicAdd(&status[0], 1u);
    status[1] = tag;
    status[2] = detail;
}

// ------------------------------------------------------------------ programmatic dependent launch
// Every kernel of the step is launched so that it may start while its predecessor in the stream is still
// draining.  A kernel announces early that its successor may be scheduled, and must not touch anything another
// kernel of the step writes (activations, caches, metadata) before pdl_wait(), which returns once every
// predecessor grid has finished and its writes are visible.  Only constants (weights) may be read before it.
// Both are no-ops in a launch without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ------------------------------------------------------------------ shared memory / barriers

__device__ __forceinline__ uint32_t smem_u32(const void* pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the async (TMA) proxy.
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders earlier generic-proxy accesses of shared memory before later async-proxy ones.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for a phase of an mbarrier for at most about `limit_ns` of wall time (one second unless the host set another
// limit, see wait_limit_ns() in options.h).  Returns false when the limit is reached (the caller records the
// failure and unwinds); it never spins without bound.  The bound is kept on the SM's cycle counter, which is cheap
// to read (a wait that misses its first probe must not pay for a slow timer before it probes again): the SM clock
// never exceeds 2 GHz, so 2 * limit_ns cycles last at least limit_ns and at most a few times longer.
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const long long start = clock64();
    const long long limit_cycles = static_cast<long long>(limit_ns) * 2;
    for (;;) {
#pragma unroll 1
        for (uint32_t spin = 0; spin < 32; ++spin) {
            if (mbar_try_wait(bar, parity)) {
                return true;
            }
        }
        if (clock64() - start > limit_cycles) {
            return false;
        }
    }
}

// ------------------------------------------------------------------ TMA (no multicast anywhere)

__device__ __forceinline__ void tma_prefetch_descriptor(const void* tensor_map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensor_map)) : "memory");
}

// 2-D tiled load global -> this CTA's shared memory, completion counted in bytes on `bar`.
// x is the innermost coordinate (elements); x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tensor_map, uint32_t bar, int32_t x,
                                            int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// The same load with an L2 eviction-priority hint: a policy from l2_evict_first_policy() marks the lines as the
// first to be replaced, for data that is read once (a KV stream), so that it does not push reusable lines out.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const void* tensor_map, uint32_t bar, int32_t x,
                                                 int32_t y, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

// ------------------------------------------------------------------ E4M3 and SiLU (shared by the element-wise
// kernels and the GEMM epilogue that fuses them, so that both produce the same bits)

// two floats -> two E4M3 codes (round to nearest even, saturate to +-448); `low` lands in the low byte
__device__ __forceinline__ uint16_t e4m3x2(float low, float high) {
    uint16_t codes;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(codes) : "f"(low), "f"(high));
    return codes;
}

// kernels/silu_mul.cu:7-9
__device__ __forceinline__ float silu(float x) {
    return x / (1.0f + __expf(-x));
}

// ------------------------------------------------------------------ tensor-core helpers

__device__ __forceinline__ void ldmatrix_x4(uint32_t address, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(address));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t address, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(address));
}

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D(16x8, f32) += A(16x32, e4m3, row) * B(32x8, e4m3, col)
__device__ __forceinline__ void mma_e4m3_16832(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

}  // namespace lfm25
