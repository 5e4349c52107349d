// Split-K ragged decode attention that allocates nothing: the partial records live in a fixed
// array inside the library instead of a caller-supplied workspace.
//
// Who needs this: hosts that are not allowed to call cudaMalloc once serving has started.  Typical
// cases are an engine that gave every free byte of the device to its KV page pool at start-up (a
// later allocation would simply fail), a latency-critical loop that cannot tolerate the implicit
// device synchronisation of cudaMalloc / cudaFree, and embedders whose own memory manager is the only
// component permitted to talk to the allocator.  Such a host passes its inputs and its output buffer
// as usual and leaves the scratch to the library.
//
// The price is a fixed capacity: kStaticMaxTokens tokens per call (8,650,752 bytes, held by every
// device that loads the library until the process exits), and one shared array: two calls that
// overlap on the GPU (different streams, or graphs replayed concurrently) would overwrite each other's
// records, so callers must keep calls that use this entry point ordered on one stream.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/lfm25_b200.h"
#include "kernels.h"

namespace {

constexpr size_t kStaticMaxTokens = 128;
constexpr size_t kStaticMaxSplits = 8;
constexpr size_t kStaticScratchFloats = kStaticMaxTokens * 32 * kStaticMaxSplits * 66;

// The scratch itself.  In host code this name is only a handle for the runtime's symbol table, not
// an address a kernel could use; the device address is looked up below, once per device.
static __device__ __align__(256) float g_static_splitk_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device (resolved with that device current).
cudaError_t static_scratch_address(float** address) {
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) {
        return status;
    }
    if (device < 0 || device >= kMaxDevices) {
        return cudaErrorInvalidDevice;
    }
    std::lock_guard<std::mutex> guard(g_scratch_mutex);
    if (g_scratch_address[device] == nullptr) {
        float* pointer = nullptr;
        status = cudaGetSymbolAddress(reinterpret_cast<void**>(&pointer), g_static_splitk_scratch);
        if (status != cudaSuccess) {
            return status;
        }
        g_scratch_address[device] = pointer;
    }
    *address = g_scratch_address[device];
    return cudaSuccess;
}

void forget_static_scratch_address() {
    int device = 0;
    if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < kMaxDevices) {
        std::lock_guard<std::mutex> guard(g_scratch_mutex);
        g_scratch_address[device] = nullptr;
    }
}

}  // namespace

extern "C" int32_t lfm25_paged_ragged_attention_splitk_static_lfm2_bf16(
    void* stream, const lfm25_fast_ragged_attention_launch* launch, size_t num_splits) {
    if (launch == nullptr) {
        return lfm25::report_error(LFM25_ERR_NULL_POINTER, "static split-K attention launch is null");
    }
    if (launch->num_tokens > kStaticMaxTokens) {
        return lfm25::report_error(
            LFM25_ERR_INVALID_ARGUMENT,
            "static split-K attention holds scratch for at most 128 tokens per call; use the entry point "
            "with a caller-owned workspace for larger batches");
    }
    if (num_splits < 2 || num_splits > kStaticMaxSplits) {
        return lfm25::report_error(LFM25_ERR_INVALID_ARGUMENT, "split-K ragged attention requires 2..=8 splits");
    }
    float* scratch = nullptr;
    const cudaError_t status = static_scratch_address(&scratch);
    if (status != cudaSuccess) {
        return lfm25::report_error(LFM25_ERR_CUDA, "static split-K scratch is not reachable on this device");
    }
    // Nothing in the array has to be cleared first.  Every record that the merge combines into an output row was
    // written by this same call: a valid token's CTAs write all of its records, and a token that a CTA gave up on
    // (request slot outside the block tables, position outside its row, unassigned page, a wait that ran out) gets a
    // "no result" mark in place of the record, on which the merge leaves that token's output row as the caller
    // passed it in.  Records of an earlier call are therefore never turned into output.  The one input that can
    // leave a token without any record is a `token_order` that is not a permutation of the batch; the order arrays
    // that lfm25_context_order_desc writes always are.
    lfm25_splitk_ragged_attention_launch full;
    full.page_size = launch->page_size;
    full.query = launch->query;
    full.key_cache = launch->key_cache;
    full.value_cache = launch->value_cache;
    full.block_tables = launch->block_tables;
    full.request_slots = launch->request_slots;
    full.position_ids = launch->position_ids;
    full.partials.ptr = scratch;
    full.partials.len = kStaticScratchFloats;
    full.output = launch->output;
    full.num_tokens = launch->num_tokens;
    full.num_pages = launch->num_pages;
    full.block_table_stride = launch->block_table_stride;
    full.num_splits = num_splits;
    full.token_order = launch->token_order;
    const int32_t result = lfm25_paged_ragged_attention_splitk_lfm2_bf16(stream, &full);
    if (result == LFM25_ERR_CUDA) {
        // The context may have been torn down and rebuilt since the address was resolved (cudaDeviceReset in the
        // host): forget it, so that the next call asks the runtime again.
        forget_static_scratch_address();
    }
    return result;
}
