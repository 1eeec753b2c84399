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

}  // namespace kvq
