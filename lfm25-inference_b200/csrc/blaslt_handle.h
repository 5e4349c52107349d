// Layout of the opaque lfm25_blaslt handle (internal): the stream it is bound to, the one device allocation it
// owns (the cuBLASLt workspace followed by the split-K exchange buffer of this library's tcgen05 GEMM) and the
// lazily opened cuBLASLt state.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "kernels.h"

namespace lfm25 {
struct CublasLtBf16;
CublasLtBf16* cublaslt_bf16_create(void* workspace, size_t workspace_bytes);
void cublaslt_bf16_destroy(CublasLtBf16* self);
cudaError_t cublaslt_bf16_linear(CublasLtBf16* self, cudaStream_t stream, const void* x, const void* weight,
                                 void* out, size_t m, size_t n, size_t k);
uint64_t cublaslt_bf16_calls();   // matmuls handed to cuBLASLt by this process so far
}  // namespace lfm25

struct lfm25_blaslt {
    cudaStream_t stream;
    void* allocation;
    void* library_workspace;        // handed to cuBLASLt (32 MiB, the size the reference uses)
    size_t library_workspace_bytes;
    void* exchange;                 // split-K partial tiles of the tcgen05 GEMM; one stream at a time
    size_t exchange_bytes;
    lfm25::CublasLtBf16* cublaslt;  // null until the first BF16 linear
    // lfm25_blaslt_set_gemm_tuning: which kernel the linears of this handle take (0 = the library's choice; the
    // values of lfm25::GemmPath) and the tile parameters of the batch-major kernel (0 = the library's choice)
    int64_t tuning_kernel = 0;
    lfm25::GemmRowsTuning tuning;
};
