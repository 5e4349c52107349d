// Kernel launch helper: every kernel of the library goes through cudaLaunchKernelEx with the programmatic
// stream-serialisation attribute (see pdl_wait() in common.cuh), unless the option `pdl` is 0.
#pragma once

#include <cuda_runtime.h>

#include "options.h"

namespace lfm25 {

inline bool pdl_enabled() { return option(kOptPdl) != 0; }

template <typename... Parameters, typename... Arguments>
cudaError_t launch_kernel(void (*kernel)(Parameters...), unsigned int blocks, unsigned int threads, size_t shared_bytes,
                          cudaStream_t stream, unsigned int cluster, Arguments... arguments) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(blocks, 1, 1);
    config.blockDim = dim3(threads, 1, 1);
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    unsigned int count = 0;
    if (pdl_enabled()) {
        attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    if (cluster > 1) {
        attributes[count].id = cudaLaunchAttributeClusterDimension;
        attributes[count].val.clusterDim.x = cluster;
        attributes[count].val.clusterDim.y = 1;
        attributes[count].val.clusterDim.z = 1;
        ++count;
    }
    config.attrs = attributes;
    config.numAttrs = count;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Parameters>(arguments)...);
}

}  // namespace lfm25
