// Launching with programmatic dependent launch.
//
// A kernel launched through rdl_launch may begin while the kernel before it in the stream is
// still draining: its blocks are scheduled as soon as every block of the earlier kernel has
// called rdl_grid_launch_dependents() (or exited), and they run until rdl_grid_wait(), which
// returns only when the earlier kernel has completed and its writes are visible.  That hides the
// launch latency and whatever a kernel can do before it needs its inputs: reading constants
// (weights, the batch description, cache pages of earlier steps) and asking L2 for them.
//
// Rules every kernel launched this way keeps:
//   * rdl_grid_wait() comes before the first read of anything an earlier kernel of the step wrote
//     and before the first write to global memory (a buffer may be recycled memory that the
//     earlier kernel still reads);
//   * before it, only constants are read.
// A kernel launched the ordinary way may contain the two calls; they do nothing then.
#pragma once

#include <cuda_runtime.h>

#include <utility>

// 1: launches carry the programmatic-serialization attribute.  Set through rdl_set_programmatic_launch.
extern int g_rdl_programmatic_launch;

template <typename... KArgs, typename... Args>
inline cudaError_t rdl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rdl_programmatic_launch ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

__device__ __forceinline__ void rdl_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void rdl_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#define RDL_CHECK_EX(call, name)                                            \
    do {                                                                    \
        cudaError_t e_ = (call);                                            \
        if (e_ != cudaSuccess) {                                            \
            rdl_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
            return 2;                                                       \
        }                                                                   \
    } while (0)
