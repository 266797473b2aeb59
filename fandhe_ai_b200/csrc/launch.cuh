// Host-side kernel launch helper: cudaLaunchKernelEx with the optional attributes this library uses -
// a thread-block cluster shape and programmatic dependent launch (the kernel may be scheduled while its
// predecessor in the stream drains; it calls pdl_wait() before touching the predecessor's results).
#pragma once
#include <cuda_runtime.h>

namespace b200 {

// Process-wide switch for programmatic dependent launch (set from the environment variable
// B200_PDL=0/1 at first use; default on).  Defined in backend.cu.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
cudaError_t launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                      bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (pdl && pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace b200
