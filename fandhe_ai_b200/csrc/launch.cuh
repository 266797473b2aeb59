// Host-side kernel launch helper: cudaLaunchKernelEx with the optional attributes this library uses -
// a thread-block cluster shape and programmatic dependent launch (the kernel may be scheduled while its
// predecessor in the stream drains; it calls pdl_wait() before touching the predecessor's results).
#pragma once
#include <cuda_runtime.h>

namespace b200 {

// Process-wide switch for programmatic dependent launch (set from the environment variable
// B200_PDL=0/1 at first use; default on).  Defined in backend.cu.
bool pdl_enabled();

// Number of SMs of the current device (asked once per device ordinal).  Defined in backend.cu.
int current_sm_count();

// Raises a kernel's dynamic shared-memory limit to `bytes` on the current device.  Function attributes belong to
// the device, so the largest value already set is remembered per device ordinal in `cache` (64 entries, zero
// initialised, one array per kernel instantiation).
template <typename K>
cudaError_t ensure_dynamic_smem(K kernel, int bytes, int* cache) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (cache[dev] >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) cache[dev] = bytes;
    return e;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_impl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, dim3 cluster,
                        bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
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

// cluster of `cluster_x` CTAs along grid x (1: no cluster)
template <typename... KArgs, typename... Args>
cudaError_t launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                      bool pdl, Args... args) {
    return launch_impl(kernel, grid, block, smem, stream, dim3(cluster_x, 1, 1), pdl, args...);
}

// cluster of `cluster_z` CTAs along grid z (1: no cluster)
template <typename... KArgs, typename... Args>
cudaError_t launch_ex_z(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_z,
                        bool pdl, Args... args) {
    return launch_impl(kernel, grid, block, smem, stream, dim3(1, 1, cluster_z), pdl, args...);
}

}  // namespace b200
