// kvq_group_absmax: per (head, channel group) maximum of |x| over all tokens of a K or V tensor -
// the statistic static calibration is built from: scale = percentile over samples of
// (absmax over the sequence) / qmax  (scripts/calibrate_behavior.py:228-260, 764-812).
//
// The result is max-accumulated into `out` (fp32 [H, G], caller zero-fills it once), so that several
// calls - batch rows, chunks of a long sequence, several samples - fold into one table.  |x| of an
// fp16 value is exact in fp32 and the maximum is order-independent, so the table is bit-identical to
// the reference's view(...).abs().amax(3).amax(1).  Non-negative floats order like their bit patterns,
// which turns the accumulation into an integer atomicMax.
//
// grid = (token chunks, H, B); a thread reduces 8 consecutive channels (one 16-byte load) of up to
// kRowsPerThread rows, threads of a group combine through shared memory, one atomic per (CTA, group).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kvq_internal.h"

namespace kvq {

constexpr int kAbsmaxThreads = 256;
constexpr int kAbsmaxRows = 64;          // token rows per CTA

struct AbsmaxParams {
    KvqAbsmaxArgs a;
    int chunks;                           // D / 8
};

__global__ void __launch_bounds__(kAbsmaxThreads) group_absmax_kernel(const AbsmaxParams p) {
    const KvqAbsmaxArgs& a = p.a;
    const int h = blockIdx.y, b = blockIdx.z;
    const int row0 = blockIdx.x * kAbsmaxRows;
    const int G = a.D / a.group_size;
    extern __shared__ float gmax[];       // [G]
    for (int g = threadIdx.x; g < G; g += kAbsmaxThreads) gmax[g] = 0.f;
    __syncthreads();
    const __half* base = (const __half*)a.x + (long long)b * a.stride_b + (long long)h * a.stride_h;
    const int items = kAbsmaxRows * p.chunks;
    for (int i = threadIdx.x; i < items; i += kAbsmaxThreads) {
        const int r = row0 + i / p.chunks, c = i % p.chunks;
        if (r >= a.S) break;
        const uint4 v = *(const uint4*)(base + (long long)r * a.stride_s + 8 * c);
        const __half2* h2 = reinterpret_cast<const __half2*>(&v);
        float m = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(__habs2(h2[j]));
            m = fmaxf(m, fmaxf(f.x, f.y));
        }
        atomicMax(reinterpret_cast<int*>(&gmax[(8 * c) / a.group_size]), __float_as_int(m));
    }
    __syncthreads();
    for (int g = threadIdx.x; g < G; g += kAbsmaxThreads)
        atomicMax(reinterpret_cast<int*>(a.out + (long long)h * G + g), __float_as_int(gmax[g]));
}

}  // namespace kvq

extern "C" int kvq_group_absmax(const KvqAbsmaxArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    const KvqAbsmaxArgs& a = *args;
    if (a.B < 0 || a.H <= 0 || a.S < 0 || a.D <= 0 || (a.D % 8) != 0) return KVQ_EINVAL;
    const int gs = a.group_size == -1 ? a.D : a.group_size;
    if (gs <= 0 || a.D % gs != 0 || gs % 8 != 0) return KVQ_EINVAL;
    if (a.B == 0 || a.S == 0) return KVQ_OK;
    if (!a.x || !a.out) return KVQ_EINVAL;
    if (((uintptr_t)a.x & 15) || (a.stride_b & 7) || (a.stride_h & 7) || (a.stride_s & 7)) return KVQ_EINVAL;
    if (a.H > 65535 || a.B > 65535) return KVQ_ELIMIT;
    AbsmaxParams p;
    p.a = a;
    p.a.group_size = gs;
    p.chunks = a.D / 8;
    dim3 grid((a.S + kAbsmaxRows - 1) / kAbsmaxRows, a.H, a.B);
    const size_t smem = (size_t)(a.D / gs) * sizeof(float);
    group_absmax_kernel<<<grid, kAbsmaxThreads, smem, (cudaStream_t)stream>>>(p);
    return check_launch();
}
