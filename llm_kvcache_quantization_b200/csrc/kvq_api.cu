// Error reporting and device queries of the C ABI.
#include <stdlib.h>

#include "kvq_internal.h"

namespace kvq {

int& last_cuda_error_ref() {
    static thread_local int e = 0;
    return e;
}

int device_sm_count() {
    // one cached value per device ordinal; 148 on B200
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("KVQ_NO_PDL");
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v == 1;
}

}  // namespace kvq

extern "C" const char* kvq_strerror(int code) {
    switch (code) {
        case KVQ_OK: return "ok";
        case KVQ_EINVAL: return "invalid argument (shape, stride, alignment or NULL pointer)";
        case KVQ_EUNSUPPORTED: return "configuration not supported by this build";
        case KVQ_ECUDA: return "CUDA runtime error (see kvq_last_cuda_error)";
        case KVQ_EWORKSPACE: return "workspace too small";
        case KVQ_ELIMIT: return "request exceeds a fixed limit of this entry point";
        default: return "unknown kvq status";
    }
}

extern "C" int kvq_last_cuda_error(void) { return kvq::last_cuda_error_ref(); }
extern "C" int kvq_abi_version(void) { return KVQ_ABI_VERSION; }

extern "C" size_t kvq_struct_size(int which) {
    switch (which) {
        case 0: return sizeof(KvqAppendSide);
        case 1: return sizeof(KvqAppendArgs);
        case 2: return sizeof(KvqCacheSide);
        case 3: return sizeof(KvqAttnArgs);
        case 4: return sizeof(KvqCombineArgs);
        case 5: return sizeof(KvqDequantArgs);
        case 6: return sizeof(KvqKiviArgs);
        case 7: return sizeof(KvqAbsmaxArgs);
        case 8: return sizeof(KvqExchangeArgs);
        case 9: return sizeof(KvqQuantileArgs);
        default: return 0;
    }
}
