// Host side of kvq_decode_attn / kvq_lse_combine: argument validation, split
// heuristic, kernel selection, and the two combine kernels.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "kvq_decode_generic.cuh"
#include "kvq_internal.h"

namespace kvq {

// ---------------------------------------------------------------------------
// In-GPU combine over KV splits: unnormalised partials (o, m, l) -> fp16 output
// and, optionally, a normalised partial (o/l, m in natural-log units, l) for a
// cross-GPU merge.  grid = (Hq, B), block = D threads.
// ---------------------------------------------------------------------------
__global__ void combine_splits_kernel(const AttnParams p) {
    const KvqAttnArgs& a = p.a;
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const int D = a.D;
    const long long row0 = ((long long)b * a.Hq + h) * p.splits;
    float M = -INFINITY;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, p.ws_ml[(row0 + s) * 2]);
    float o = 0.f, L = 0.f;
    for (int s = 0; s < p.splits; ++s) {
        float ms = p.ws_ml[(row0 + s) * 2];
        float ls = p.ws_ml[(row0 + s) * 2 + 1];
        if (ls > 0.f) {
            float w = exp2f(ms - M);
            o += p.ws_o[(row0 + s) * D + d] * w;
            L += ls * w;
        }
    }
    float r = (L > 0.f) ? o / L : 0.f;
    if (a.out) ((__half*)a.out)[b * a.out_stride_b + h * a.out_stride_h + d] = __float2half_rn(r);
    if (a.part_o) {
        long long idx = (long long)b * a.Hq + h;
        a.part_o[idx * D + d] = r;
        if (d == 0) {
            a.part_m[idx] = (L > 0.f) ? M * 0.6931471805599453f : -INFINITY;
            a.part_l[idx] = L;
        }
    }
}

// Merge of P normalised partials (one per sequence shard).  grid = (Hq, B).
__global__ void lse_combine_kernel(const KvqCombineArgs c) {
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const long long BH = (long long)c.B * c.Hq;
    const long long idx = (long long)b * c.Hq + h;
    float M = -INFINITY;
    for (int p = 0; p < c.P; ++p) {
        float l = c.part_l[p * BH + idx];
        if (l > 0.f) M = fmaxf(M, c.part_m[p * BH + idx]);
    }
    float num = 0.f, den = 0.f;
    for (int p = 0; p < c.P; ++p) {
        float l = c.part_l[p * BH + idx];
        if (l > 0.f) {
            float w = l * expf(c.part_m[p * BH + idx] - M);
            num += c.part_o[(p * BH + idx) * c.D + d] * w;
            den += w;
        }
    }
    float r = den > 0.f ? num / den : 0.f;
    ((__half*)c.out)[b * c.out_stride_b + h * c.out_stride_h + d] = __float2half_rn(r);
}

static bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

static int validate_side(const KvqCacheSide& s, const KvqAttnArgs& a, bool asym) {
    if (!s.payload) return KVQ_EINVAL;
    if (!aligned16(s.payload) || (s.pay_stride_b & 15) || (s.pay_stride_h & 15) || (s.pay_stride_s & 15))
        return KVQ_EINVAL;
    if (a.format != KVQ_FMT_FP16 && !s.scale) return KVQ_EINVAL;
    if (asym && !s.zp) return KVQ_EINVAL;
    if (a.n_out > 0 && !s.side) return KVQ_EINVAL;
    return KVQ_OK;
}

template <int FMT, bool ASYM, int D>
static int launch_generic(const AttnParams& p, cudaStream_t st) {
    dim3 grid(p.splits, p.a.Hkv * p.rep_chunks, p.a.B);
    size_t dyn = (size_t)4 * kHeadsPerCta * D * sizeof(float);
    static bool attr_done = false;
    if (!attr_done && dyn > 48 * 1024) {
        int rc = check_cuda(cudaFuncSetAttribute(decode_split_generic_kernel<FMT, ASYM, D>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
        if (rc) return rc;
        attr_done = true;
    }
    decode_split_generic_kernel<FMT, ASYM, D><<<grid, 128, dyn, st>>>(p);
    return check_launch();
}

template <int FMT, bool ASYM>
static int dispatch_d(const AttnParams& p, cudaStream_t st) {
    switch (p.a.D) {
        case 64: return launch_generic<FMT, ASYM, 64>(p, st);
        case 128: return launch_generic<FMT, ASYM, 128>(p, st);
        case 256: return launch_generic<FMT, ASYM, 256>(p, st);
        default: return KVQ_EUNSUPPORTED;
    }
}

static int dispatch_generic(const AttnParams& p, bool asym, cudaStream_t st) {
    switch (p.a.format) {
        case KVQ_FMT_FP16: return dispatch_d<KVQ_FMT_FP16, false>(p, st);
        case KVQ_FMT_INT8: return asym ? dispatch_d<KVQ_FMT_INT8, true>(p, st) : dispatch_d<KVQ_FMT_INT8, false>(p, st);
        case KVQ_FMT_INT4: return asym ? dispatch_d<KVQ_FMT_INT4, true>(p, st) : dispatch_d<KVQ_FMT_INT4, false>(p, st);
        default: return KVQ_EINVAL;
    }
}

}  // namespace kvq

extern "C" size_t kvq_decode_workspace_bytes(int32_t B, int32_t Hq, int32_t D, int32_t splits) {
    if (B <= 0 || Hq <= 0 || D <= 0 || splits <= 0) return 0;
    size_t rows = (size_t)B * Hq * splits;
    size_t o = rows * D * sizeof(float);
    size_t ml = rows * 2 * sizeof(float);
    return ((o + 255) & ~(size_t)255) + ((ml + 255) & ~(size_t)255);
}

extern "C" int32_t kvq_decode_pick_splits(int32_t B, int32_t Hkv, int32_t max_ctx) {
    if (B <= 0 || Hkv <= 0 || max_ctx <= 0) return 1;
    const int sms = kvq::device_sm_count();
    long long base = (long long)B * Hkv;
    long long want = 4LL * sms;                         // ~4 CTAs per SM in flight
    long long splits = (want + base - 1) / base;
    long long by_len = max_ctx / 256;                   // keep >= 256 tokens per split
    if (by_len < 1) by_len = 1;
    if (splits > by_len) splits = by_len;
    if (splits > 256) splits = 256;
    if (splits < 1) splits = 1;
    return (int32_t)splits;
}

extern "C" int kvq_decode_attn(const KvqAttnArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    const KvqAttnArgs& a = *args;
    if (a.B < 0 || a.Hq <= 0 || a.Hkv <= 0 || a.D <= 0 || a.max_ctx < 0) return KVQ_EINVAL;
    if (a.Hq % a.Hkv != 0) return KVQ_EINVAL;
    if (a.B == 0) return KVQ_OK;
    if (!a.q || !a.context_lens) return KVQ_EINVAL;
    if (!a.out && !a.part_o) return KVQ_EINVAL;
    if ((a.part_o != nullptr) != (a.part_m != nullptr) || (a.part_o != nullptr) != (a.part_l != nullptr))
        return KVQ_EINVAL;
    if (a.D != 64 && a.D != 128 && a.D != 256) return KVQ_EUNSUPPORTED;
    int gs = a.group_size == -1 ? a.D : a.group_size;
    if (a.format == KVQ_FMT_FP16) gs = a.D;
    if (gs <= 0 || a.D % gs != 0 || gs % 8 != 0) return KVQ_EINVAL;
    const bool asym = a.k.zp != nullptr || a.v.zp != nullptr;
    if (a.n_out < 0 || (a.n_out > 0 && (!a.outlier_idx || asym))) return KVQ_EINVAL;
    int rc = validate_side(a.k, a, asym);
    if (rc) return rc;
    rc = validate_side(a.v, a, asym);
    if (rc) return rc;
    if ((a.q_stride_b & 1) || (a.q_stride_h & 1) || (((uintptr_t)a.q) & 3)) return KVQ_EINVAL;

    AttnParams p;
    p.a = a;
    p.a.group_size = gs;
    p.G = a.D / gs;
    p.n_rep = a.Hq / a.Hkv;
    p.rep_chunks = (p.n_rep + kHeadsPerCta - 1) / kHeadsPerCta;
    p.splits = a.splits > 0 ? a.splits : kvq_decode_pick_splits(a.B, a.Hkv, a.max_ctx);
    size_t need = kvq_decode_workspace_bytes(a.B, a.Hq, a.D, p.splits);
    if (!a.workspace || a.workspace_bytes < need || (((uintptr_t)a.workspace) & 15)) return KVQ_EWORKSPACE;
    size_t o_bytes = ((size_t)a.B * a.Hq * p.splits * a.D * sizeof(float) + 255) & ~(size_t)255;
    p.ws_o = (float*)a.workspace;
    p.ws_ml = (float*)((char*)a.workspace + o_bytes);

    cudaStream_t st = (cudaStream_t)stream;
    rc = dispatch_generic(p, asym, st);
    if (rc) return rc;
    combine_splits_kernel<<<dim3(a.Hq, a.B), a.D, 0, st>>>(p);
    return check_launch();
}

extern "C" int kvq_lse_combine(const KvqCombineArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    const KvqCombineArgs& c = *args;
    if (c.P <= 0 || c.B < 0 || c.Hq <= 0 || c.D <= 0 || c.D > 1024) return KVQ_EINVAL;
    if (c.B == 0) return KVQ_OK;
    if (!c.part_o || !c.part_m || !c.part_l || !c.out) return KVQ_EINVAL;
    lse_combine_kernel<<<dim3(c.Hq, c.B), c.D, 0, (cudaStream_t)stream>>>(c);
    return check_launch();
}
