// Launching with attributes: thread-block clusters, and programmatic dependent launch.
//
// A decode step is a chain of ~120 small kernels, each of which depends on the one before.
// Launched plainly, every link pays the GPU's launch latency after its predecessor has
// drained. With programmatic dependent launch a kernel's CTAs may become resident while
// the predecessor still runs: they do whatever does not depend on it (above all, request
// their weights from HBM), then wait for it with pdl_wait(). A kernel tells the GPU that its
// successor may be brought in with pdl_launch_dependents().
//
// Rules every kernel launched this way keeps: before pdl_wait() it reads only memory that no
// kernel of the step writes (weights, norm weights, tables; and the cache rows of positions
// before the step's own, which only earlier steps wrote), and it writes nothing. A step begins
// with a copy of its numbers from the host, which the stream orders after every kernel of the
// step before; so nothing of an earlier step is still in flight when a kernel of this one runs.
#pragma once

#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

namespace sm {

// Waits until the kernels this one depends on have completed and their writes are visible.
// Without a programmatic dependency this returns at once.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Allows the next kernel in the stream to be launched (it still waits in its own pdl_wait()).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
void launch_kernel(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                   int cluster, bool dependent, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (dependent) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": launch failed: " + cudaGetErrorString(e));
}

}  // namespace sm
