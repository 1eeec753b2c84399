// Shared by the translation units of libkvq.
#pragma once
#include <cuda_runtime.h>

#include "kvq.h"

namespace kvq {

// cudaError_t of the last failed runtime call on this host thread.
int& last_cuda_error_ref();

inline int check_cuda(cudaError_t e) {
    if (e == cudaSuccess) return KVQ_OK;
    last_cuda_error_ref() = (int)e;
    return KVQ_ECUDA;
}

// Launch-configuration errors only; never synchronises.
inline int check_launch() { return check_cuda(cudaGetLastError()); }

int device_sm_count();

// Device-side error flags of the other translation units (each owns its __device__ word): value, optionally
// cleared; negative = KVQ_ECUDA.  kvq_debug_error_flag combines them.
int quantize_error_flag(int reset);
int kivi_error_flag(int reset);

// Launch with programmatic dependent launch: the grid may start while the previous kernel in the
// stream is still running; the kernel itself calls pdl_wait() before it touches anything that
// kernel writes.  KVQ_NO_PDL=1 falls back to ordinary stream order.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

#ifdef __CUDACC__
// Device side of programmatic dependent launch (no-ops when the launch did not ask for it).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

}  // namespace kvq
