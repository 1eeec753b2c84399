// Host side of kvq_decode_attn / kvq_lse_combine: argument validation, kernel
// selection, wave-aware split heuristic, TMA descriptors, and the two combine kernels.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>

#include <atomic>
#include <stdint.h>
#include <stdlib.h>

#include "kvq_decode_generic.cuh"
#include "kvq_decode_int4.cuh"
#include "kvq_decode_mma.cuh"
#include "kvq_internal.h"

namespace kvq {

// ---------------------------------------------------------------------------
// In-GPU combine over KV splits: unnormalised partials (o, m, l) -> fp16 output
// and, optionally, a normalised partial (o/l, m in natural-log units, l) for a
// cross-GPU merge.  grid = (Hq, B), block = 8 warps.  Every warp first finds the
// global max over all splits (lane s reads split s), then warp w sums the splits
// w, w+8, ... with four independent loads in flight per lane (a lane owns D/32
// channels), and the eight warps are added through shared memory.  The loop over
// splits is latency-bound when run serially; this form keeps it near one round trip.
// ---------------------------------------------------------------------------
// Shared front half: leaves the warps' weighted sums in red[w][0..D) and their
// denominators in red[w][D]; returns the global max (log2 domain) of the row.
constexpr int kCombineWarps = 8;
constexpr int kCombineThreads = kCombineWarps * 32;

// sum over the warps' rows of `red` at column c
template <int N>
__device__ __forceinline__ float red_sum(const float (*red)[N], int c) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kCombineWarps; ++w) v += red[w][c];
    return v;
}

// Merge of the KV splits of one (batch, head) row: warp w takes splits w, w + 8, ... (a lane = EPL channels), eight
// partials in flight per lane, one pass with a running (max, sum) per warp - no separate pass over the maxima, the
// row's latency is one or two round trips to L2.  The warps then agree on the maximum through shared memory and leave
// their sums, scaled to it, in `red` ([warp][channel], column D = the softmax denominator).  Returns the maximum
// (log2 domain, -inf for an empty row).
template <int EPL>   // channels per lane = D / 32
__device__ __forceinline__ float combine_partials(const AttnParams& p, int b, int h, float (*red)[EPL * 32 + 1]) {
    const KvqAttnArgs& a = p.a;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int D = EPL * 32;
    constexpr int U = 8;
    __shared__ float warp_m[kCombineWarps];
    const long long row0 = ((long long)b * a.Hq + h) * p.splits;
    const float2* ml = reinterpret_cast<const float2*>(p.ws_ml) + row0;
    const float* o_base = p.ws_o + row0 * D + lane * EPL;
    float acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
    float M = -INFINITY, L = 0.f;
    for (int s0 = warp; s0 < p.splits; s0 += U * kCombineWarps) {
        float2 mv[U];
        float ov[U][EPL];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + kCombineWarps * u;
            mv[u] = s < p.splits ? ml[s] : make_float2(-INFINITY, 0.f);
            if (s < p.splits) {
                if (EPL == 4) *reinterpret_cast<float4*>(ov[u]) = *reinterpret_cast<const float4*>(o_base + (long long)s * D);
                else {
#pragma unroll
                    for (int e = 0; e < EPL; ++e) ov[u][e] = o_base[(long long)s * D + e];
                }
            }
        }
        float Mn = M;
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (mv[u].y > 0.f) Mn = fmaxf(Mn, mv[u].x);
        if (Mn > M) {                                  // uniform over the warp
            const float c = exp2f(M - Mn);             // exp2f(-inf) = 0 the first time
            L *= c;
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[e] *= c;
            M = Mn;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (mv[u].y > 0.f) {
                const float w = exp2f(mv[u].x - M);
                L += mv[u].y * w;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[e] += ov[u][e] * w;
            }
        }
    }
    if (lane == 0) warp_m[warp] = M;
    __syncthreads();
    float Mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < kCombineWarps; ++w) Mt = fmaxf(Mt, warp_m[w]);
    const float c = (L > 0.f) ? exp2f(M - Mt) : 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) red[warp][lane * EPL + e] = acc[e] * c;
    if (lane == 0) red[warp][D] = L * c;
    __syncthreads();
    return Mt;
}

// One channel of one cached token, dequantised exactly as the split kernels do (any format; runtime
// dispatch - the combine stage touches a single token per row).
__device__ __forceinline__ float cached_value(const KvqAttnArgs& a, const KvqCacheSide& cs, int b, int kvh, int t, int d) {
    const char* row = (const char*)cs.payload + b * cs.pay_stride_b + kvh * cs.pay_stride_h + (long long)t * cs.pay_stride_s;
    if (a.format == KVQ_FMT_FP16) return __half2float(((const __half*)row)[d]);
    for (int j = 0; j < a.n_out; ++j)
        if ((int)a.outlier_idx[kvh * a.n_out + j] == d)
            return __half2float(((const __half*)cs.side)[b * cs.side_stride_b + kvh * cs.side_stride_h +
                                                         (long long)t * cs.side_stride_s + j]);
    int code;
    if (a.format == KVQ_FMT_INT8) code = ((const int8_t*)row)[d];
    else {
        const unsigned byte = ((const uint8_t*)row)[d >> 1];
        code = (int)((d & 1) ? (byte & 15u) : (byte >> 4)) - 8;
    }
    const long long so = b * cs.sc_stride_b + kvh * cs.sc_stride_h + (long long)t * cs.sc_stride_s + d / a.group_size;
    __half v = __hmul_rn(__int2half_rn(code), ((const __half*)cs.scale)[so]);
    if (cs.zp) v = __hadd_rn(v, ((const __half*)cs.zp)[so]);
    return __half2float(v);
}

// The last token of the row's context, attended here instead of in the split kernel (tail_tokens = 1).
// Thread d owns channel d.  tail_load issues the loads (query, the token's K and V rows, their parameters) and
// returns this thread's q.k product and V value; it is called BEFORE the partials are merged so that both sets of
// loads are in flight together.  tail_fold then folds the token into the merged splits, given as (M log2-domain
// max, o_d weighted sum, Lt denominator).  Both are called by every thread of the CTA.
template <int EPL>
__device__ __forceinline__ bool tail_load(const AttnParams& p, int b, int h, float& prod, float& vd) {
    const KvqAttnArgs& a = p.a;
    constexpr int D = EPL * 32;
    prod = 0.f;
    vd = 0.f;
    int ctx = a.context_lens ? a.context_lens[b] : a.max_ctx;
    ctx = max(0, min(ctx, a.max_ctx));
    if (ctx < 1) return false;                            // uniform over the CTA
    const int t = ctx - 1, kvh = h / p.n_rep, d = threadIdx.x;
    if (d < D) {
        __half qv = ((const __half*)a.q)[b * a.q_stride_b + h * a.q_stride_h + d];
        if (a.inv_tau) qv = __hmul(qv, __float2half_rn(a.inv_tau[h]));
        if (a.q_chan_scale)
            qv = __float2half_rn(__half2float(qv) * a.q_chan_scale[b * a.qcs_stride_b + kvh * a.qcs_stride_h + d]);
        prod = __half2float(qv) * cached_value(a, a.k, b, kvh, t, d);
        vd = cached_value(a, a.v, b, kvh, t, d);
    }
    return true;
}

__device__ __forceinline__ void tail_fold(const KvqAttnArgs& a, float* scratch, float prod, float vd, float& M,
                                          float& o_d, float& Lt) {
    prod = warp_sum(prod);
    __syncthreads();                                      // scratch may still be read as `red`
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = prod;
    __syncthreads();
    float dot = 0.f;
#pragma unroll
    for (int w = 0; w < kCombineWarps; ++w) dot += scratch[w];
    const float sv = dot * a.sm_scale * kLog2e;
    const float Mn = fmaxf(M, sv);
    const float wm = (Lt > 0.f) ? exp2f(M - Mn) : 0.f;
    const float wt = exp2f(sv - Mn);
    o_d = o_d * wm + wt * vd;
    Lt = Lt * wm + wt;
    M = Mn;
}

template <int EPL>
__global__ void __launch_bounds__(kCombineThreads) combine_splits_kernel(const AttnParams p) {
    pdl_launch_dependents();      // the next kernel of the stream may be set up; it waits for this one itself
    pdl_wait();                   // the split kernel's partials
    const KvqAttnArgs& a = p.a;
    const int h = blockIdx.x, b = blockIdx.y;
    constexpr int D = EPL * 32;
    __shared__ float red[kCombineWarps][D + 1];
    __shared__ float tail_scratch[kCombineWarps];
    float tprod, tvd;
    const bool has_tail = a.tail_tokens && tail_load<EPL>(p, b, h, tprod, tvd);
    float M = combine_partials<EPL>(p, b, h, red);
    float o = threadIdx.x < D ? red_sum(red, threadIdx.x) : 0.f;      // kCombineThreads >= D: one channel per thread
    float Lt = red_sum(red, D);
    if (has_tail) tail_fold(a, tail_scratch, tprod, tvd, M, o, Lt);
    for (int d = threadIdx.x; d < D; d += kCombineThreads) {
        const float r = (Lt > 0.f) ? o / Lt : 0.f;
        if (a.out) ((__half*)a.out)[b * a.out_stride_b + h * a.out_stride_h + d] = __float2half_rn(r);
        if (a.part_o) {
            const long long idx = (long long)b * a.Hq + h;
            const long long so = a.part_o_stride ? a.part_o_stride : D;
            const long long sm = a.part_ml_stride ? a.part_ml_stride : 1;
            a.part_o[idx * so + d] = r;
            if (d == 0) {
                a.part_m[idx * sm] = (Lt > 0.f) ? M * 0.6931471805599453f : -INFINITY;
                a.part_l[idx * sm] = Lt;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Combine fused with the cross-GPU exchange of a sequence-sharded decode: one kernel per
// rank merges its KV splits into the normalised partial of every (batch, head) row, stores
// that partial straight into every rank's receive buffer over NVLink (plain peer stores),
// raises a per-row flag on every rank, waits for the same row of every other rank, and
// merges the `world` partials into the fp16 output.  It replaces three launches and a
// library collective (combine, all-gather, merge) by one launch whose transfer overlaps the
// other rows' arithmetic.
//
// Receive buffer of a rank (identical layout on every rank, peer-mapped):
//   8-byte words [2 parity][slots][world src][B][Hq][D + 2], word = (fp32 value, epoch), rows [o (D) | m | l]
// Every word carries its own validity stamp and travels as ONE 8-byte store, so no fence and no
// separate flag is needed: the receiver spins on each word until its stamp equals the current epoch
// (the low-latency protocol of collective libraries).  `epoch` (device int, >= 1) is advanced once
// per decode step by the host side; parity = epoch & 1 double-buffers the rows so that a rank one
// step ahead never overwrites a word a slower rank still waits for.  Progress never depends on
// another CTA of the same GPU: a CTA pushes before it waits, and waits only for remote CTAs.  The
// wait is bounded by `wait_ns`; on expiry the thread raises *status and continues with a zero.
// ---------------------------------------------------------------------------
struct ExchangeParams {
    AttnParams p;
    KvqExchangeArgs x;
    unsigned long long* recv[KVQ_MAX_PEERS];
};

__device__ __forceinline__ void st_word(unsigned long long* p, float v, int stamp) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(stamp) : "memory");
}
__device__ __forceinline__ void ld_word(const unsigned long long* p, float& v, int& stamp) {
    unsigned lo;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(stamp) : "l"(p) : "memory");
    v = __uint_as_float(lo);
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

template <int EPL>
__global__ void __launch_bounds__(kCombineThreads) combine_exchange_kernel(const ExchangeParams ep) {
    pdl_launch_dependents();
    pdl_wait();
    const AttnParams& p = ep.p;
    const KvqExchangeArgs& x = ep.x;
    const KvqAttnArgs& a = p.a;
    const int h = blockIdx.x, b = blockIdx.y;
    constexpr int D = EPL * 32;
    constexpr int W = D + 2;
    static_assert(D <= kCombineThreads, "one channel per thread");
    __shared__ float red[kCombineWarps][D + 1];
    __shared__ float pm[KVQ_MAX_PEERS], pl[KVQ_MAX_PEERS];
    __shared__ float tail_scratch[kCombineWarps];
    float tprod, tvd;
    const bool has_tail = a.tail_tokens && tail_load<EPL>(p, b, h, tprod, tvd);
    float M = combine_partials<EPL>(p, b, h, red);
    float o = threadIdx.x < D ? red_sum(red, threadIdx.x) : 0.f;      // one channel per thread
    float Lt = red_sum(red, D);
    if (has_tail) tail_fold(a, tail_scratch, tprod, tvd, M, o, Lt);

    const int epoch = *x.epoch;
    const long long rows = (long long)a.B * a.Hq;
    const long long slot_base = ((long long)(epoch & 1) * x.slots + x.slot) * x.world;     // in units of `rows`
    const long long row_in_slot = (long long)b * a.Hq + h;

    // ---- push this rank's normalised partial of the row to every rank (itself included)
    {
        const float r = (Lt > 0.f) ? o / Lt : 0.f;
        const float m_nat = (Lt > 0.f) ? M * 0.6931471805599453f : -INFINITY;
        const long long my_row = (slot_base + x.rank) * rows + row_in_slot;
        for (int w = threadIdx.x; w < W; w += kCombineThreads) {
            const float val = w < D ? r : (w == D ? m_nat : Lt);       // w < D implies w == threadIdx.x
            for (int q = 0; q < x.world; ++q) st_word(ep.recv[q] + my_row * W + w, val, epoch);
        }
    }

    // ---- collect the same row from every rank: spin on each word's stamp (bounded)
    float vals[KVQ_MAX_PEERS];
    const unsigned long long t0 = global_ns();
    bool expired = false;
    for (int w = threadIdx.x; w < W; w += kCombineThreads) {
#pragma unroll
        for (int q = 0; q < KVQ_MAX_PEERS; ++q) {
            if (q >= x.world) break;
            const unsigned long long* src = ep.recv[x.rank] + ((slot_base + q) * rows + row_in_slot) * W + w;
            float v;
            int stamp;
            ld_word(src, v, stamp);
            while (stamp != epoch && !expired) {
                if (global_ns() - t0 > x.wait_ns) { expired = true; break; }
                __nanosleep(40);
                ld_word(src, v, stamp);
            }
            if (stamp != epoch) v = 0.f;                               // l = 0 removes the rank from the merge
            if (w < D) vals[q] = v;
            else if (w == D) pm[q] = v;
            else pl[q] = v;
        }
    }
    if (expired && x.status) atomicExch(x.status, 1);
    __syncthreads();
    float Mx = -INFINITY;
    for (int q = 0; q < x.world; ++q)
        if (pl[q] > 0.f) Mx = fmaxf(Mx, pm[q]);
    if (threadIdx.x < D) {
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int q = 0; q < KVQ_MAX_PEERS; ++q) {
            if (q >= x.world) break;
            if (pl[q] > 0.f) {
                const float wgt = pl[q] * expf(pm[q] - Mx);
                num += vals[q] * wgt;
                den += wgt;
            }
        }
        const float r = den > 0.f ? num / den : 0.f;
        ((__half*)x.out)[b * x.out_stride_b + h * x.out_stride_h + threadIdx.x] = __float2half_rn(r);
    }
}

static int launch_combine(const AttnParams& p, cudaStream_t st) {
    dim3 grid(p.a.Hq, p.a.B);
    switch (p.a.D) {
        case 64: return launch_pdl(combine_splits_kernel<2>, grid, dim3(kCombineThreads), 0, st, p);
        case 128: return launch_pdl(combine_splits_kernel<4>, grid, dim3(kCombineThreads), 0, st, p);
        case 256: return launch_pdl(combine_splits_kernel<8>, grid, dim3(kCombineThreads), 0, st, p);
        default: return KVQ_EUNSUPPORTED;
    }
}

// Merge of P normalised partials (one per sequence shard).  grid = (Hq, B).
__global__ void lse_combine_kernel(const KvqCombineArgs c) {
    pdl_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const long long BH = (long long)c.B * c.Hq;
    const long long idx = (long long)b * c.Hq + h;
    const long long so = c.part_o_stride ? c.part_o_stride : c.D;
    const long long sm = c.part_ml_stride ? c.part_ml_stride : 1;
    const long long sop = c.part_o_stride_p ? c.part_o_stride_p : BH * so;
    const long long smp = c.part_ml_stride_p ? c.part_ml_stride_p : BH * sm;
    float M = -INFINITY;
    for (int p = 0; p < c.P; ++p) {
        float l = c.part_l[p * smp + idx * sm];
        if (l > 0.f) M = fmaxf(M, c.part_m[p * smp + idx * sm]);
    }
    float num = 0.f, den = 0.f;
    for (int p = 0; p < c.P; ++p) {
        float l = c.part_l[p * smp + idx * sm];
        if (l > 0.f) {
            float w = l * expf(c.part_m[p * smp + idx * sm] - M);
            num += c.part_o[p * sop + idx * so + d] * w;
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

// ---------------------------------------------------------------------------
// Generic kernel dispatch
// ---------------------------------------------------------------------------
template <int FMT, bool ASYM, int D>
static int launch_generic(const AttnParams& p, cudaStream_t st) {
    dim3 grid(p.splits, p.a.Hkv * p.rep_chunks, p.a.B);
    size_t dyn = (size_t)4 * kHeadsPerCta * D * sizeof(float);
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

// ---------------------------------------------------------------------------
// Tensor-core path: eligibility, TMA descriptors, occupancy, launch
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    return fn;
}

// Payload [B, Hkv, S, row_bytes] as a 4-D byte tensor; box = (min(row_bytes, 128), TS, 1, 1), swizzle = box
// width.  Rows at or beyond `s_extent` are zero-filled by the copy engine.
// `pair_rows`: two consecutive 64-byte token rows are mapped as ONE 128-byte row (`s_extent` counts such pairs; the
// caller guarantees tokens are contiguous, pay_stride_s == row_bytes / 2): the copy engine then moves 128-byte
// segments instead of 64-byte ones, which is what the memory system is built for.
static int make_payload_map(CUtensorMap* map, const KvqCacheSide& sd, int row_bytes, int s_extent, int hkv, int b,
                            bool pair_rows = false, int box_tokens = kTS) {
    const int box_bytes = row_bytes > 128 ? 128 : row_bytes;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return KVQ_EUNSUPPORTED;
    cuuint64_t dims[4] = {(cuuint64_t)row_bytes, (cuuint64_t)s_extent, (cuuint64_t)hkv, (cuuint64_t)b};
    cuuint64_t strides[3] = {(cuuint64_t)(pair_rows ? 2 * sd.pay_stride_s : sd.pay_stride_s), (cuuint64_t)sd.pay_stride_h,
                             (cuuint64_t)sd.pay_stride_b};
    cuuint32_t box[4] = {(cuuint32_t)box_bytes, (cuuint32_t)(pair_rows ? box_tokens / 2 : box_tokens), 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(sd.payload), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? KVQ_OK : KVQ_EUNSUPPORTED;
}


// fp16 scales / zero-points [B, Hkv, S, NG] (tokens contiguous) as a 3-D tensor of 2- / 4- / 8-byte elements, one
// (two for NG = 8) per token; box = `box_tokens` tokens.  Tokens at or beyond `s_extent` are zero-filled.
static int make_scale_map(CUtensorMap* map, const void* base, long long stride_h, long long stride_b, int ng, int s_extent,
                          int hkv, int b, int box_tokens) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return KVQ_EUNSUPPORTED;
    const int tok_bytes = ng * 2;
    const int elem = tok_bytes > 8 ? 8 : tok_bytes;
    const int ept = tok_bytes / elem;
    const CUtensorMapDataType ty = elem == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                 : elem == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT64;
    const cuuint64_t row_bytes = (((cuuint64_t)s_extent * tok_bytes) + 15) & ~(cuuint64_t)15;
    cuuint64_t dims[3] = {(cuuint64_t)s_extent * ept, (cuuint64_t)hkv, (cuuint64_t)b};
    // a dimension of extent 1 never advances; give it any legal stride
    cuuint64_t strides[2] = {hkv > 1 ? (cuuint64_t)stride_h * 2 : row_bytes,
                             b > 1 ? (cuuint64_t)stride_b * 2 : row_bytes * (cuuint64_t)hkv};
    cuuint32_t box[3] = {(cuuint32_t)(box_tokens * ept), 1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, ty, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? KVQ_OK : KVQ_EUNSUPPORTED;
}

static bool mma_side_ok(const KvqCacheSide& s, int row_bytes, int hkv, int b, int n_out, int ng) {
    if (s.pay_stride_s < row_bytes || (s.pay_stride_s & 15) || (s.pay_stride_h & 15) || (s.pay_stride_b & 15)) return false;
    if (hkv > 1 && s.pay_stride_h <= 0) return false;
    if (b > 1 && s.pay_stride_b <= 0) return false;
    if (ng == 0) return true;                      // fp16 cache: payload only
    // scales [.., S, NG] with tokens contiguous and 16-byte aligned (b, h) rows
    if (s.sc_stride_s != ng || (s.sc_stride_h & 7) || (s.sc_stride_b & 7)) return false;
    if (((uintptr_t)s.scale & 15) || (s.zp && ((uintptr_t)s.zp & 15))) return false;
    if (n_out > 0) {
        if (!s.side || ((uintptr_t)s.side & 15) || s.side_stride_s != n_out || (s.side_stride_h & 7) ||
            (s.side_stride_b & 7))
            return false;
    }
    return true;
}

static bool mma_eligible(const AttnParams& p, bool asym) {
    const KvqAttnArgs& a = p.a;
    if (getenv("KVQ_FORCE_GENERIC")) return false;
    const int gs = a.group_size;
    if (a.D != 128 || (gs != 16 && gs != 32 && gs != 64 && gs != 128)) return false;
    if (a.n_out > 0 && gs != 32) return false;
    const bool f16 = a.format == KVQ_FMT_FP16;
    if (!f16 && a.format != KVQ_FMT_INT8 && a.format != KVQ_FMT_INT4) return false;
    if (asym && (f16 || (a.format == KVQ_FMT_INT8 && gs != 128))) return false;   // INT8 zero-points: one group per token
    if (a.n_out < 0 || a.n_out > kMaxOut || (a.n_out > 0 && (asym || f16))) return false;
    if (a.max_ctx < 1) return false;
    if (!a.k.payload || !a.v.payload || (!f16 && (!a.k.scale || !a.v.scale))) return false;
    const int rb = f16 ? 256 : a.format == KVQ_FMT_INT8 ? 128 : 64;
    const int ng = f16 ? 0 : 128 / gs;
    if (!mma_side_ok(a.k, rb, a.Hkv, a.B, a.n_out, ng) || !mma_side_ok(a.v, rb, a.Hkv, a.B, a.n_out, ng))
        return false;
    if (((uintptr_t)a.q & 15) || (a.q_stride_b & 7) || (a.q_stride_h & 7)) return false;
    return true;
}

// Launch configuration of one instantiation: stages, shared memory, resident CTAs per SM.
struct MmaConfig {
    int nstage;
    int stage_bytes;
    size_t dyn_smem;
    int ctas_per_sm;
    int rc;
};

static int stages_from_env(int dflt) {
    const char* e = getenv("KVQ_MMA_STAGES");
    if (!e) return dflt;
    int v = atoi(e);
    return (v >= 2 && v <= 8) ? v : dflt;
}

template <int FMT, bool ASYM, bool OUTL, int GS>
struct MmaTag {};

template <int FMT, bool ASYM, bool OUTL, int GS>
static const MmaConfig& mma_config(MmaTag<FMT, ASYM, OUTL, GS>) {
    static MmaConfig cfg = [] {
        MmaConfig c;
        c.nstage = stages_from_env(2);       // measured on B200: 2 stages (one more resident CTA per SM) beat 3
        c.stage_bytes = mma_stage_bytes(FMT, ASYM, OUTL, GS);
        c.dyn_smem = (size_t)kMmaWarps * c.nstage * c.stage_bytes + 1024;
        c.ctas_per_sm = 1;
        c.rc = check_cuda(cudaFuncSetAttribute(decode_split_mma_kernel<FMT, ASYM, OUTL, GS>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.dyn_smem));
        if (c.rc == KVQ_OK) {
            int n = 0;
            c.rc = check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                &n, decode_split_mma_kernel<FMT, ASYM, OUTL, GS>, kMmaWarps * 32, c.dyn_smem));
            if (n > 0) c.ctas_per_sm = n;
        }
        return c;
    }();
    return cfg;
}

// Calls f(MmaTag<...>{}) for the INT8 / fp16 instantiation that serves these arguments.
template <class F>
static int mma_dispatch(const AttnParams& p, bool asym, F&& f) {
    const bool outl = p.a.n_out > 0;
    const int fmt = p.a.format, gs = p.a.group_size;
#define KVQ_MMA_CASE(FMT_, ASYM_, OUTL_, GS_)                                                     \
    if (fmt == FMT_ && asym == ASYM_ && outl == OUTL_ && gs == GS_) return f(MmaTag<FMT_, ASYM_, OUTL_, GS_>{});
    KVQ_MMA_CASE(KVQ_FMT_FP16, false, false, 128)
    KVQ_MMA_CASE(KVQ_FMT_INT8, false, false, 16)
    KVQ_MMA_CASE(KVQ_FMT_INT8, false, false, 32)
    KVQ_MMA_CASE(KVQ_FMT_INT8, false, false, 64)
    KVQ_MMA_CASE(KVQ_FMT_INT8, false, false, 128)
    KVQ_MMA_CASE(KVQ_FMT_INT8, false, true, 32)
    KVQ_MMA_CASE(KVQ_FMT_INT8, true, false, 128)
#undef KVQ_MMA_CASE
    return KVQ_EUNSUPPORTED;
}

static const MmaConfig* mma_config_for(const AttnParams& p, bool asym) {
    const MmaConfig* out = nullptr;
    mma_dispatch(p, asym, [&](auto tag) { out = &mma_config(tag); return KVQ_OK; });
    return out;
}


static bool wide_rows_possible(const KvqAttnArgs& a) {
    return a.format == KVQ_FMT_INT4 && a.k.pay_stride_s == 64 && a.v.pay_stride_s == 64 && a.max_ctx >= 2 &&
           !getenv("KVQ_INT4_NARROW_ROWS");
}
// An odd max_ctx makes the last pair row reach one token slot past max_ctx - 1: fine when that slot belongs to the
// same (batch, head) row of the cache (its bytes are sanitised like any token beyond a row's context), which the head
// stride tells.
static bool wide_rows_room(const KvqAttnArgs& a) {
    const long long need = ((long long)a.max_ctx + 1) * 64;
    return a.k.pay_stride_h >= need && a.v.pay_stride_h >= need;
}
static bool wide_rows_ok(const KvqAttnArgs& a) {
    return wide_rows_possible(a) && ((a.max_ctx & 1) == 0 || a.tail_tokens == 1 || wide_rows_room(a));
}

// ---------------------------------------------------------------------------
// Packed-INT4 kernel (kvq_decode_int4.cuh): configuration, dispatch, launch
// ---------------------------------------------------------------------------
template <bool ASYM, int NOUT, bool FAST, int GS>
struct I4Tag {};

static int i4_stages_from_env(int dflt) {
    const char* e = getenv("KVQ_I4_STAGES");
    if (!e) return dflt;
    int v = atoi(e);
    return (v >= 2 && v <= kI4MaxStages) ? v : dflt;
}

template <bool ASYM, int NOUT, bool FAST, int GS>
static const MmaConfig& i4_config(I4Tag<ASYM, NOUT, FAST, GS>) {
    static MmaConfig cfg = [] {
        MmaConfig c;
        c.nstage = i4_stages_from_env(2);
        c.stage_bytes = int4_stage_bytes(ASYM, NOUT > 0, GS);
        c.dyn_smem = (size_t)c.nstage * c.stage_bytes + 1024;
        c.ctas_per_sm = 1;
        c.rc = check_cuda(cudaFuncSetAttribute(decode_split_int4_kernel<ASYM, NOUT, FAST, GS>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.dyn_smem));
        if (c.rc == KVQ_OK) {
            int n = 0;
            c.rc = check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                &n, decode_split_int4_kernel<ASYM, NOUT, FAST, GS>, kMmaWarps * 32, c.dyn_smem));
            if (n > 0) c.ctas_per_sm = n;
        }
        return c;
    }();
    return cfg;
}

// The factored-scale arithmetic (see kvq_decode_int4.cuh) serves groups of >= 32 channels unless the caller asks for
// the bit-faithful one (fast_dequant = 0 in the C ABI means "library default"; 2 = bit-faithful).
static bool i4_use_fast(const KvqAttnArgs& a) {
    if (a.group_size < 32) return false;
    if (a.fast_dequant == 2) return false;
    if (a.fast_dequant == 1) return true;
    const char* e = getenv("KVQ_INT4_EXACT");
    return !(e && e[0] == '1');
}

template <class F>
static int i4_dispatch(const AttnParams& p, bool asym, F&& f) {
    const bool fast = i4_use_fast(p.a);
    const int gs = p.a.group_size, nout = p.a.n_out;
#define KVQ_I4_CASE(ASYM_, NOUT_, FAST_, GS_)                                              \
    if (asym == ASYM_ && nout == NOUT_ && fast == FAST_ && gs == GS_) return f(I4Tag<ASYM_, NOUT_, FAST_, GS_>{});
#define KVQ_I4_GS(ASYM_, FAST_) KVQ_I4_CASE(ASYM_, 0, FAST_, 32) KVQ_I4_CASE(ASYM_, 0, FAST_, 64) KVQ_I4_CASE(ASYM_, 0, FAST_, 128)
#define KVQ_I4_OUT(FAST_) KVQ_I4_CASE(false, 1, FAST_, 32) KVQ_I4_CASE(false, 2, FAST_, 32) KVQ_I4_CASE(false, 3, FAST_, 32) KVQ_I4_CASE(false, 4, FAST_, 32)
    KVQ_I4_GS(false, true)
    KVQ_I4_GS(true, true)
    KVQ_I4_OUT(true)
    KVQ_I4_GS(false, false)
    KVQ_I4_GS(true, false)
    KVQ_I4_CASE(false, 0, false, 16)
    KVQ_I4_CASE(true, 0, false, 16)
    KVQ_I4_OUT(false)
#undef KVQ_I4_OUT
#undef KVQ_I4_GS
#undef KVQ_I4_CASE
    return KVQ_EUNSUPPORTED;
}

static const MmaConfig* i4_config_for(const AttnParams& p, bool asym) {
    const MmaConfig* out = nullptr;
    i4_dispatch(p, asym, [&](auto tag) { out = &i4_config(tag); return KVQ_OK; });
    return out;
}

template <bool ASYM, int NOUT, bool FAST, int GS>
static int launch_i4(I4Tag<ASYM, NOUT, FAST, GS> tag, const AttnParams& p, cudaStream_t st) {
    const MmaConfig& cfg = i4_config(tag);
    if (cfg.rc) return cfg.rc;
    Int4Params ip;
    ip.p = p;
    ip.nstage = cfg.nstage;
    // Pairs of tokens travel as 128-byte rows when the tokens of a (b, h) row are contiguous.  With an odd max_ctx
    // the last token either belongs to the combine stage (tail_tokens; the pair view then covers floor(max_ctx / 2)
    // pairs), or shares its pair row with the next slot of the same cache row (wide_rows_room); a call with neither
    // keeps the 64-byte rows.
    ip.wide_rows = wide_rows_ok(p.a);
    {
        static const int pf = [] { const char* e = getenv("KVQ_I4_PREFETCH"); int v = e ? atoi(e) : 1; return v < 0 ? 0 : (v > 64 ? 64 : v); }();
        static const int ahead = [] { const char* e = getenv("KVQ_I4_L2_AHEAD"); int v = e ? atoi(e) : 0; return v < 0 ? 0 : (v > 16 ? 16 : v); }();
        ip.prefetch_stages = pf;
        ip.l2_ahead = ahead;
    }
    const KvqAttnArgs& a = p.a;
    const int ext = ip.wide_rows ? (a.max_ctx + (a.tail_tokens ? 0 : 1)) / 2 : a.max_ctx;
    const int ng = 128 / GS;
    CUtensorMap kmap, vmap, ksmap, vsmap, kzmap, vzmap;
    int rc;
    if ((rc = make_payload_map(&kmap, a.k, ip.wide_rows ? 128 : 64, ext, a.Hkv, a.B, ip.wide_rows != 0, kI4Tok))) return rc;
    if ((rc = make_payload_map(&vmap, a.v, ip.wide_rows ? 128 : 64, ext, a.Hkv, a.B, ip.wide_rows != 0, kI4Tok))) return rc;
    if ((rc = make_scale_map(&ksmap, a.k.scale, a.k.sc_stride_h, a.k.sc_stride_b, ng, a.max_ctx, a.Hkv, a.B, kI4Tok))) return rc;
    if ((rc = make_scale_map(&vsmap, a.v.scale, a.v.sc_stride_h, a.v.sc_stride_b, ng, a.max_ctx, a.Hkv, a.B, kI4Tok))) return rc;
    if (ASYM) {
        if ((rc = make_scale_map(&kzmap, a.k.zp, a.k.sc_stride_h, a.k.sc_stride_b, ng, a.max_ctx, a.Hkv, a.B, kI4Tok))) return rc;
        if ((rc = make_scale_map(&vzmap, a.v.zp, a.v.sc_stride_h, a.v.sc_stride_b, ng, a.max_ctx, a.Hkv, a.B, kI4Tok))) return rc;
    } else {
        kzmap = ksmap;
        vzmap = vsmap;
    }
    dim3 grid(p.splits, a.Hkv * p.rep_chunks, a.B);
    return launch_pdl(decode_split_int4_kernel<ASYM, NOUT, FAST, GS>, grid, dim3(kMmaWarps * 32), cfg.dyn_smem, st, ip,
                      kmap, vmap, ksmap, vsmap, kzmap, vzmap);
}

static bool i4_eligible(const AttnParams& p, bool asym) {
    return p.a.format == KVQ_FMT_INT4 && i4_config_for(p, asym) != nullptr;
}

static int dispatch_i4(const AttnParams& p, bool asym, cudaStream_t st) {
    return i4_dispatch(p, asym, [&](auto tag) { return launch_i4(tag, p, st); });
}

template <int FMT, bool ASYM, bool OUTL, int GS>
static int launch_mma(MmaTag<FMT, ASYM, OUTL, GS> tag, const AttnParams& p, cudaStream_t st) {
    constexpr int RB = FMT == KVQ_FMT_FP16 ? 256 : 128;
    const MmaConfig& cfg = mma_config(tag);
    if (cfg.rc) return cfg.rc;
    MmaParams mp;
    mp.p = p;
    mp.nstage = cfg.nstage;
    mp.warp_smem_bytes = cfg.nstage * cfg.stage_bytes;
    CUtensorMap kmap, vmap;
    int rc = make_payload_map(&kmap, p.a.k, RB, p.a.max_ctx, p.a.Hkv, p.a.B);
    if (rc) return rc;
    rc = make_payload_map(&vmap, p.a.v, RB, p.a.max_ctx, p.a.Hkv, p.a.B);
    if (rc) return rc;
    dim3 grid(p.splits, p.a.Hkv * p.rep_chunks, p.a.B);
    return launch_pdl(decode_split_mma_kernel<FMT, ASYM, OUTL, GS>, grid, dim3(kMmaWarps * 32), cfg.dyn_smem, st, mp,
                      kmap, vmap);
}

static int dispatch_mma(const AttnParams& p, bool asym, cudaStream_t st) {
    if (i4_eligible(p, asym)) return dispatch_i4(p, asym, st);
    return mma_dispatch(p, asym, [&](auto tag) { return launch_mma(tag, p, st); });
}

// ---------------------------------------------------------------------------
// Split heuristic.  All CTAs of a launch do the same amount of work when the
// batch rows have equal context, so the launch takes ceil(ctas / slots) "waves"
// (slots = SMs x resident CTAs per SM).  Pick the split count whose last wave
// is fullest, among those that leave at least `min_tokens` per split; prefer
// fewer splits on ties (less workspace traffic, cheaper combine).
// ---------------------------------------------------------------------------
static int pick_splits_waves(long long rows, int max_ctx, int slots, int min_tokens) {
    long long by_len = (max_ctx + min_tokens - 1) / min_tokens;     // a last split may be short
    if (by_len < 1) by_len = 1;
    if (by_len > 256) by_len = 256;
    if (rows >= 8LL * slots) return 1;            // many waves already: the tail is a small fraction
    // Cost of a launch in "token times": waves x (tokens of the busiest warp's share + a fixed
    // per-CTA cost for prologue, first-copy latency and the 4-warp merge, about one 128-token slice).
    const int quantum = kMmaWarps * kTS, fixed = quantum;
    int best = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= by_len; ++s) {
        const long long ctas = rows * s;
        const long long waves = (ctas + slots - 1) / slots;
        if (waves > 8 && s > 1) break;
        const int per = ((max_ctx + s - 1) / s + quantum - 1) / quantum * quantum;
        const double cost = (double)waves * (per + fixed);
        if (cost < best_cost * 0.98) {
            best_cost = cost;
            best = s;
        }
    }
    return best;
}

static int pick_splits_internal(const AttnParams& p, bool asym, bool mma) {
    const long long rows = (long long)p.a.B * p.a.Hkv * p.rep_chunks;
    const int sms = device_sm_count();
    if (mma) {
        const MmaConfig* cfg = i4_eligible(p, asym) ? i4_config_for(p, asym) : mma_config_for(p, asym);
        if (!cfg) return 1;
        // the tokens the split kernel scans: a tail token belongs to the combine stage
        return pick_splits_waves(rows, p.a.max_ctx - (p.a.tail_tokens ? 1 : 0), sms * cfg->ctas_per_sm, kMmaWarps * kTS);
    }
    return pick_splits_waves(rows, p.a.max_ctx - (p.a.tail_tokens ? 1 : 0), sms * 8, 256);
}

static int fill_params(const KvqAttnArgs& a, AttnParams& p, bool& asym) {
    if (a.B < 0 || a.Hq <= 0 || a.Hkv <= 0 || a.D <= 0 || a.max_ctx < 0) return KVQ_EINVAL;
    if (a.Hq % a.Hkv != 0) return KVQ_EINVAL;
    if (a.D != 64 && a.D != 128 && a.D != 256) return KVQ_EUNSUPPORTED;
    int gs = a.group_size == -1 ? a.D : a.group_size;
    if (a.format == KVQ_FMT_FP16) gs = a.D;
    if (gs <= 0 || a.D % gs != 0 || gs % 8 != 0) return KVQ_EINVAL;
    asym = a.k.zp != nullptr || a.v.zp != nullptr;
    p.a = a;
    p.a.group_size = gs;
    p.G = a.D / gs;
    p.n_rep = a.Hq / a.Hkv;
    p.rep_chunks = (p.n_rep + kHeadsPerCta - 1) / kHeadsPerCta;
    p.splits = 1;
    p.ws_o = nullptr;
    p.ws_ml = nullptr;
    return KVQ_OK;
}

}  // namespace kvq

extern "C" size_t kvq_decode_workspace_bytes(int32_t B, int32_t Hq, int32_t D, int32_t splits) {
    if (B <= 0 || Hq <= 0 || D <= 0 || splits <= 0) return 0;
    size_t rows = (size_t)B * Hq * splits;
    size_t o = rows * D * sizeof(float);
    size_t ml = rows * 2 * sizeof(float);
    return ((o + 255) & ~(size_t)255) + ((ml + 255) & ~(size_t)255);
}

extern "C" int32_t kvq_decode_pick_splits(const KvqAttnArgs* args) {
    using namespace kvq;
    if (!args) return 1;
    AttnParams p;
    bool asym = false;
    if (fill_params(*args, p, asym) != KVQ_OK || args->B == 0 || args->max_ctx == 0) return 1;
    return pick_splits_internal(p, asym, mma_eligible(p, asym));
}

extern "C" int kvq_decode_kernel_kind(const KvqAttnArgs* args) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    AttnParams p;
    bool asym = false;
    int rc = fill_params(*args, p, asym);
    if (rc) return rc;
    return mma_eligible(p, asym) ? 1 : 0;
}

extern "C" int kvq_decode_attn(const KvqAttnArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    const KvqAttnArgs& a = *args;
    AttnParams p;
    bool asym = false;
    int rc = fill_params(a, p, asym);
    if (rc) return rc;
    if (a.B == 0) return KVQ_OK;
    if (!a.q) return KVQ_EINVAL;
    if (!a.out && !a.part_o) return KVQ_EINVAL;
    if ((a.part_o != nullptr) != (a.part_m != nullptr) || (a.part_o != nullptr) != (a.part_l != nullptr))
        return KVQ_EINVAL;
    if (a.n_out < 0 || (a.n_out > 0 && (!a.outlier_idx || asym))) return KVQ_EINVAL;
    rc = validate_side(a.k, a, asym);
    if (rc) return rc;
    rc = validate_side(a.v, a, asym);
    if (rc) return rc;
    if ((a.q_stride_b & 1) || (a.q_stride_h & 1) || (((uintptr_t)a.q) & 3)) return KVQ_EINVAL;
    if (a.stages < 0 || a.stages > 2) return KVQ_EINVAL;
    if (a.tail_tokens < 0 || a.tail_tokens > 1) return KVQ_EINVAL;
    if (a.q_chan_scale && (a.format == KVQ_FMT_FP16 || a.n_out > 0)) return KVQ_EUNSUPPORTED;

    const bool mma = mma_eligible(p, asym);
    // whole call over a packed-INT4 cache with an odd token count: hand the last token to the combine stage so that
    // the scan can fetch pairs of tokens as 128-byte rows (see launch_mma)
    if (mma && a.stages == 0 && a.tail_tokens == 0 && (a.max_ctx & 1) && wide_rows_possible(a) && !wide_rows_room(a))
        p.a.tail_tokens = 1;
    p.splits = a.splits > 0 ? a.splits : pick_splits_internal(p, asym, mma);
    size_t need = kvq_decode_workspace_bytes(a.B, a.Hq, a.D, p.splits);
    if (!a.workspace || a.workspace_bytes < need || (((uintptr_t)a.workspace) & 15)) return KVQ_EWORKSPACE;
    size_t o_bytes = ((size_t)a.B * a.Hq * p.splits * a.D * sizeof(float) + 255) & ~(size_t)255;
    p.ws_o = (float*)a.workspace;
    p.ws_ml = (float*)((char*)a.workspace + o_bytes);

    cudaStream_t st = (cudaStream_t)stream;
    if (a.stages != 2) {
        rc = KVQ_EUNSUPPORTED;
        if (mma) rc = dispatch_mma(p, asym, st);
        if (rc == KVQ_EUNSUPPORTED) rc = dispatch_generic(p, asym, st);
        if (rc) return rc;
    }
    if (a.stages != 1) {
        rc = launch_combine(p, st);
    }
    return rc;
}

// ---------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to obtain scratch memory at call time: a
// serving runtime that has already handed every byte of HBM to its own pool and
// forbids cudaMalloc afterwards, or a plugin called from inside a region where the
// allocator must not run.  For them the split-K partials live in a fixed array inside
// the library image instead of a caller-provided workspace.
//
// The array is a file-scope __device__ object: every GPU that loads the library keeps
// its own copy (KVQ_STATIC_WS_BYTES) until the process exits.  In host code the name
// `g_static_workspace` is only a handle for the runtime, not a device address, so the
// address is resolved with cudaGetSymbolAddress, once per device, with that device
// current, and cached.
// ---------------------------------------------------------------------------
#define KVQ_STATIC_WS_BYTES KVQ_STATIC_WORKSPACE_BYTES
static __device__ __align__(256) unsigned char g_static_workspace[KVQ_STATIC_WS_BYTES];

static int static_workspace_ptr(void** out) {
    // one slot per device; concurrent first calls from several host threads all resolve the same address and
    // store the same value, so the relaxed atomics only keep the accesses well defined
    static std::atomic<void*> cached[64];
    int dev = 0;
    int rc = kvq::check_cuda(cudaGetDevice(&dev));
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return KVQ_EUNSUPPORTED;
    void* p = cached[dev].load(std::memory_order_relaxed);
    if (!p) {
        rc = kvq::check_cuda(cudaGetSymbolAddress(&p, g_static_workspace));
        if (rc) return rc;
        if (!p) return KVQ_ECUDA;
        cached[dev].store(p, std::memory_order_relaxed);
    }
    *out = p;
    return KVQ_OK;
}

// Bytes of the array a call may use: all of it, or less when KVQ_STATIC_WS_LIMIT (bytes) says so - a host that
// wants the partials to stay inside a slice of L2, or a test of the shrinking below.
static size_t static_workspace_limit() {
    static const size_t lim = [] {
        const char* e = getenv("KVQ_STATIC_WS_LIMIT");
        long long v = e ? atoll(e) : 0;
        return (v > 0 && (size_t)v < (size_t)KVQ_STATIC_WS_BYTES) ? (size_t)v : (size_t)KVQ_STATIC_WS_BYTES;
    }();
    return lim;
}

extern "C" int kvq_decode_attn_static(const KvqAttnArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    KvqAttnArgs a = *args;
    if (a.B == 0) return KVQ_OK;
    if (a.B < 0 || a.Hq <= 0 || a.D <= 0) return KVQ_EINVAL;
    if (a.splits <= 0) {
        a.splits = kvq_decode_pick_splits(&a);
        // prefer fewer splits over refusing: shrink until the partials fit the fixed array
        while (a.splits > 1 && kvq_decode_workspace_bytes(a.B, a.Hq, a.D, a.splits) > static_workspace_limit()) --a.splits;
    }
    const size_t need = kvq_decode_workspace_bytes(a.B, a.Hq, a.D, a.splits);
    if (need == 0) return KVQ_EINVAL;
    if (need > static_workspace_limit()) return KVQ_ELIMIT;  // B * Hq * splits * (D + 2) * 4 bytes > 8 MiB (or the env limit)
    void* ws = nullptr;
    int rc = static_workspace_ptr(&ws);
    if (rc) return rc;
    a.workspace = ws;
    a.workspace_bytes = static_workspace_limit();
    return kvq_decode_attn(&a, stream);
}

extern "C" size_t kvq_exchange_bytes(int32_t B, int32_t Hq, int32_t D, int32_t slots, int32_t world) {
    if (B <= 0 || Hq <= 0 || D <= 0 || slots <= 0 || world <= 0) return 0;
    const size_t words = (size_t)2 * slots * world * B * Hq * (D + 2);
    return (words * sizeof(unsigned long long) + 255) & ~(size_t)255;
}

extern "C" int kvq_combine_exchange(const KvqExchangeArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    const KvqExchangeArgs& x = *args;
    if (x.B < 0 || x.Hq <= 0 || x.splits <= 0 || x.slots <= 0 || x.slot < 0 || x.slot >= x.slots) return KVQ_EINVAL;
    if (x.world < 1 || x.world > KVQ_MAX_PEERS || x.rank < 0 || x.rank >= x.world) return KVQ_EINVAL;
    if (x.D != 64 && x.D != 128 && x.D != 256) return KVQ_EUNSUPPORTED;
    if (x.B == 0) return KVQ_OK;
    if (!x.peer_base || !x.epoch || !x.out || !x.workspace) return KVQ_EINVAL;
    const size_t need = kvq_decode_workspace_bytes(x.B, x.Hq, x.D, x.splits);
    if (x.workspace_bytes < need || (((uintptr_t)x.workspace) & 15)) return KVQ_EWORKSPACE;
    ExchangeParams ep;
    ep.x = x;
    ep.p.a = KvqAttnArgs();
    ep.p.a.B = x.B; ep.p.a.Hq = x.Hq; ep.p.a.D = x.D;
    ep.p.n_rep = 1;
    if (x.tail_attn && x.tail_attn->tail_tokens) {
        // the stage-1 call left this rank's last token to this kernel: same validation, same derived values
        bool asym = false;
        int rc = fill_params(*x.tail_attn, ep.p, asym);
        if (rc) return rc;
        const KvqAttnArgs& t = *x.tail_attn;
        if (t.B != x.B || t.Hq != x.Hq || t.D != x.D || t.tail_tokens != 1 || !t.q) return KVQ_EINVAL;
        if (t.n_out < 0 || (t.n_out > 0 && (!t.outlier_idx || asym))) return KVQ_EINVAL;
        if ((rc = validate_side(t.k, t, asym)) != 0 || (rc = validate_side(t.v, t, asym)) != 0) return rc;
    }
    ep.p.splits = x.splits;
    const size_t o_bytes = ((size_t)x.B * x.Hq * x.splits * x.D * sizeof(float) + 255) & ~(size_t)255;
    ep.p.ws_o = (float*)x.workspace;
    ep.p.ws_ml = (float*)((char*)x.workspace + o_bytes);
    for (int q = 0; q < KVQ_MAX_PEERS; ++q) {
        char* base = q < x.world ? (char*)x.peer_base[q] : nullptr;
        if (q < x.world && (!base || ((uintptr_t)base & 15))) return KVQ_EINVAL;
        ep.recv[q] = (unsigned long long*)base;
    }
    if (ep.x.wait_ns == 0) ep.x.wait_ns = 1000000000ull;       // one second
    dim3 grid(x.Hq, x.B);
    cudaStream_t st = (cudaStream_t)stream;
    switch (x.D) {
        case 64: return launch_pdl(combine_exchange_kernel<2>, grid, dim3(kCombineThreads), 0, st, ep);
        case 128: return launch_pdl(combine_exchange_kernel<4>, grid, dim3(kCombineThreads), 0, st, ep);
        default: return launch_pdl(combine_exchange_kernel<8>, grid, dim3(kCombineThreads), 0, st, ep);
    }
}

extern "C" int kvq_debug_error_flag(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, kvq::g_kvq_error_flag, sizeof(int)) != cudaSuccess) return KVQ_ECUDA;
    if (reset && v) {
        int z = 0;
        if (cudaMemcpyToSymbol(kvq::g_kvq_error_flag, &z, sizeof(int)) != cudaSuccess) return KVQ_ECUDA;
    }
    const int qf = kvq::quantize_error_flag(reset), kf = kvq::kivi_error_flag(reset);
    if (qf < 0 || kf < 0) return KVQ_ECUDA;
    return (v ? 1 : 0) | (qf ? 2 : 0) | (kf ? 4 : 0);
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
