// BF16 linear through cuBLASLt: Y[M,N] = X[M,K] * W[N,K]^T, fp32 accumulate.
//
// The decode step's BF16 GEMMs (q/k/v/o, conv in/out, the MLP sites that are not promoted to FP8) are
// "plain library GEMMs": the reference sends them to cuBLASLt (BlasLt::linear_bf16,
// src/cuda/blaslt/mod.rs:113-186, layouts src/cuda/blaslt/plan.rs:30-79) and so does this library.
// cuBLASLt is opened lazily with dlopen, so the library itself loads on machines without it; a plan
// (descriptor, layouts, heuristic algorithm) is cached per (M, N, K), as the reference does.
#include <cublasLt.h>
#include <dlfcn.h>

#include <atomic>

#include <map>
#include <mutex>
#include <tuple>

#include "kernels.h"

namespace lfm25 {

namespace {

struct Api {
    void* library = nullptr;
    decltype(&cublasLtCreate) create = nullptr;
    decltype(&cublasLtMatmulDescCreate) desc_create = nullptr;
    decltype(&cublasLtMatmulDescSetAttribute) desc_set = nullptr;
    decltype(&cublasLtMatrixLayoutCreate) layout_create = nullptr;
    decltype(&cublasLtMatmulPreferenceCreate) preference_create = nullptr;
    decltype(&cublasLtMatmulPreferenceSetAttribute) preference_set = nullptr;
    decltype(&cublasLtMatmulAlgoGetHeuristic) heuristic = nullptr;
    decltype(&cublasLtMatmul) matmul = nullptr;
    bool ok = false;
};

Api& api() {
    static Api instance = [] {
        Api loaded;
        const char* names[] = {"libcublasLt.so.12", "libcublasLt.so", "/usr/local/cuda/lib64/libcublasLt.so.12"};
        for (const char* name : names) {
            loaded.library = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (loaded.library != nullptr) {
                break;
            }
        }
        if (loaded.library == nullptr) {
            return loaded;
        }
#define LFM25_LOAD(field, symbol) \
    loaded.field = reinterpret_cast<decltype(loaded.field)>(dlsym(loaded.library, #symbol))
        LFM25_LOAD(create, cublasLtCreate);
        LFM25_LOAD(desc_create, cublasLtMatmulDescCreate);
        LFM25_LOAD(desc_set, cublasLtMatmulDescSetAttribute);
        LFM25_LOAD(layout_create, cublasLtMatrixLayoutCreate);
        LFM25_LOAD(preference_create, cublasLtMatmulPreferenceCreate);
        LFM25_LOAD(preference_set, cublasLtMatmulPreferenceSetAttribute);
        LFM25_LOAD(heuristic, cublasLtMatmulAlgoGetHeuristic);
        LFM25_LOAD(matmul, cublasLtMatmul);
#undef LFM25_LOAD
        loaded.ok = loaded.create && loaded.desc_create && loaded.desc_set && loaded.layout_create &&
                    loaded.preference_create && loaded.preference_set && loaded.heuristic && loaded.matmul;
        return loaded;
    }();
    return instance;
}

std::atomic<uint64_t> g_library_calls{0};   // matmuls handed to cuBLASLt so far (also while a stream is captured)

struct Plan {
    cublasLtMatmulDesc_t desc = nullptr;
    cublasLtMatrixLayout_t a = nullptr;  // W as column-major [K, N], used transposed
    cublasLtMatrixLayout_t b = nullptr;  // X as column-major [K, M]
    cublasLtMatrixLayout_t c = nullptr;  // Y as column-major [N, M]
    cublasLtMatmulAlgo_t algo;
};

}  // namespace

struct CublasLtBf16 {
    cublasLtHandle_t handle = nullptr;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    std::map<std::tuple<size_t, size_t, size_t>, Plan> plans;
    std::mutex mutex;
};

CublasLtBf16* cublaslt_bf16_create(void* workspace, size_t workspace_bytes) {
    if (!api().ok) {
        return nullptr;
    }
    CublasLtBf16* self = new CublasLtBf16();
    if (api().create(&self->handle) != CUBLAS_STATUS_SUCCESS) {
        delete self;
        return nullptr;
    }
    self->workspace = workspace;
    self->workspace_bytes = workspace_bytes;
    return self;
}

void cublaslt_bf16_destroy(CublasLtBf16* self) {
    // plans and the handle live as long as the process' CUDA context; releasing them at teardown
    // would need the library to be still loaded, which dlopen order does not guarantee
    delete self;
}

// Row-major X[M,K], W[N,K], Y[M,N] are column-major X^T[K,M], W^T[K,N], Y^T[N,M]:  Y^T = (W^T)^T * X^T.
cudaError_t cublaslt_bf16_linear(CublasLtBf16* self, cudaStream_t stream, const void* x, const void* weight,
                                 void* out, size_t m, size_t n, size_t k) {
    if (self == nullptr) {
        return cudaErrorNotSupported;
    }
    Plan* plan = nullptr;
    {
        std::lock_guard<std::mutex> guard(self->mutex);
        const auto key = std::make_tuple(m, n, k);
        auto found = self->plans.find(key);
        if (found == self->plans.end()) {
            Plan fresh;
            const cublasOperation_t transpose = CUBLAS_OP_T;
            const cublasOperation_t none = CUBLAS_OP_N;
            bool ok = api().desc_create(&fresh.desc, CUBLAS_COMPUTE_32F, CUDA_R_32F) == CUBLAS_STATUS_SUCCESS;
            ok = ok && api().desc_set(fresh.desc, CUBLASLT_MATMUL_DESC_TRANSA, &transpose, sizeof transpose) ==
                           CUBLAS_STATUS_SUCCESS;
            ok = ok && api().desc_set(fresh.desc, CUBLASLT_MATMUL_DESC_TRANSB, &none, sizeof none) ==
                           CUBLAS_STATUS_SUCCESS;
            ok = ok && api().layout_create(&fresh.a, CUDA_R_16BF, k, n, static_cast<int64_t>(k)) ==
                           CUBLAS_STATUS_SUCCESS;
            ok = ok && api().layout_create(&fresh.b, CUDA_R_16BF, k, m, static_cast<int64_t>(k)) ==
                           CUBLAS_STATUS_SUCCESS;
            ok = ok && api().layout_create(&fresh.c, CUDA_R_16BF, n, m, static_cast<int64_t>(n)) ==
                           CUBLAS_STATUS_SUCCESS;
            cublasLtMatmulPreference_t preference = nullptr;
            ok = ok && api().preference_create(&preference) == CUBLAS_STATUS_SUCCESS;
            ok = ok && api().preference_set(preference, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES,
                                            &self->workspace_bytes, sizeof self->workspace_bytes) ==
                           CUBLAS_STATUS_SUCCESS;
            cublasLtMatmulHeuristicResult_t result;
            int returned = 0;
            ok = ok && api().heuristic(self->handle, fresh.desc, fresh.a, fresh.b, fresh.c, fresh.c, preference, 1,
                                       &result, &returned) == CUBLAS_STATUS_SUCCESS &&
                 returned > 0;
            if (!ok) {
                return cudaErrorNotSupported;
            }
            fresh.algo = result.algo;
            found = self->plans.emplace(key, fresh).first;
        }
        plan = &found->second;
    }
    const float alpha = 1.0f;
    const float beta = 0.0f;
    g_library_calls.fetch_add(1, std::memory_order_relaxed);
    const cublasStatus_t status =
        api().matmul(self->handle, plan->desc, &alpha, weight, plan->a, x, plan->b, &beta, out, plan->c, out, plan->c,
                     &plan->algo, self->workspace, self->workspace_bytes, stream);
    return status == CUBLAS_STATUS_SUCCESS ? cudaSuccess : cudaErrorUnknown;
}

uint64_t cublaslt_bf16_calls() { return g_library_calls.load(std::memory_order_relaxed); }

}  // namespace lfm25
