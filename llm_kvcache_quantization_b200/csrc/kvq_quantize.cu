// Quantize-on-append for the KV cache: one launch quantizes the new tokens of K
// and V and writes payload, fp16 scales (zero-points, outlier side values)
// straight into the cache slots.
//
// Arithmetic contracts (bit-exact with the reference's torch quantizers):
//   INT8   s = RN16(max(s_in,1e-5));  c = clamp(rint(RN16(float(x)/float(s))), -127, 127)
//          (src/quant/int8_basic.py:155-161 - the fp32 quotient is rounded to fp16 first)
//   INT4   s = max(s_in,1e-5) fp32;   c = clamp(rint(float(x)/s), -7, 7); stored scale RN16(s)
//          (src/quant/int4_basic.py:150-156; src/engine/patch_model.py:932-933)
//   asym   rng = max(max-min, 9.1553e-4); s = rng/15; zp = min + 8 s;
//          c = clamp(rint((x - zp)/s), -8, 7)      (src/quant/asymmetric_quant.py:98-141)
//   percentile = torch.quantile's sorted lerp, evaluated as one fma.
//   rotary embedding (optional, K side and the query): rotate-half in fp16, every operation rounded
//          as the eager torch ops are: RN16(RN16(x cos) + RN16(rot(x) sin)), rot(x) = (-x[d + r/2], x[d - r/2])
//          (src/engine/patch_model.py:223-278).
// This translation unit must be compiled WITHOUT fast-math: it relies on IEEE
// fp32 division and fp16 subnormals.
//
// Two work decompositions of the same arithmetic.  Per-token form: one thread per chunk of a
// (side, b, h, t) row; decode-time append traffic is tiny next to the attention scan (B*Hkv rows
// of 256 B), the kernel is launch-latency bound and what matters is that it is ONE launch with no
// host sync.  Bulk form (prefill, thousands of tokens): laid out for bandwidth and for few
// instructions per element, bit-identical results (see quantize_bulk_kernel).

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "kvq_internal.h"

namespace kvq {

__device__ int g_quantize_error_flag = 0;   // 1: an append met a slot at or beyond max_slots


constexpr int kMaxGroup = 256;

struct QuantParams {
    KvqAppendArgs a;
    int G;
    int nsides;   // 2, or 1 when the V side is absent (v.src == NULL)
    long long q_items;   // B * Hq * T * G work items that rotate the query (0 = none)
};

__device__ __forceinline__ float h2f(__half h) { return __half2float(h); }

// One channel of a head row after rotate-half RoPE.  `row` points at channel 0 of the head row,
// `cs` / `sn` at channel 0 of the cos / sin row of this (batch, token).
__device__ __forceinline__ __half rope_one(const __half* row, const __half* cs, const __half* sn, int rd, int d) {
    const __half x = row[d];
    if (d >= rd) return x;
    const int hf = rd >> 1;
    const __half partner = d < hf ? __hneg(row[d + hf]) : row[d - hf];
    return __hadd_rn(__hmul_rn(x, cs[d]), __hmul_rn(partner, sn[d]));
}

// torch.quantile(|x|, q) over n sorted values: rank = q*(n-1) in fp32, fma lerp.
__device__ float group_quantile(const float* v, int n, float q) {
    float pos = __fmul_rn(q, (float)(n - 1));
    int lo = (int)floorf(pos);
    int hi = min(lo + 1, n - 1);
    float w = __fsub_rn(pos, (float)lo);
    float x0 = 0.f, x1 = 0.f;
    for (int i = 0; i < n; ++i) {
        float vi = v[i];
        int rank = 0;
        for (int j = 0; j < n; ++j) {
            float vj = v[j];
            rank += (vj < vi) || (vj == vi && j < i);
        }
        if (rank == lo) x0 = vi;
        if (rank == hi) x1 = vi;
    }
    float diff = __fsub_rn(x1, x0);
    return (w < 0.5f) ? __fmaf_rn(w, diff, x0) : __fmaf_rn(__fsub_rn(w, 1.0f), diff, x1);
}

// torch.quantile over a group when only its two largest values matter (rank floor(q (n-1)) >= n - 2,
// which holds for the usual clipping percentiles: 99.9 % of a group of <= 1000 values):
// same lerp, same rounding, no sort.  m1 >= m2 are the two largest |x| of the group.
__device__ __forceinline__ float top2_quantile(float m1, float m2, int n, float q) {
    float pos = __fmul_rn(q, (float)(n - 1));
    int lo = (int)floorf(pos);
    float w = __fsub_rn(pos, (float)lo);
    float x1 = m1, x0 = (lo >= n - 1) ? m1 : m2;
    float diff = __fsub_rn(x1, x0);
    return (w < 0.5f) ? __fmaf_rn(w, diff, x0) : __fmaf_rn(__fsub_rn(w, 1.0f), diff, x1);
}
__host__ __device__ inline bool top2_applies(int n, float q) {
    float pos = q * (float)(n - 1);          // one IEEE fp32 multiply on either side
    return (int)floorf(pos) >= n - 2;
}

// x / s for a divisor that is fixed per thread: r = RN(1 / s) once, then per element q0 = RN(x r), the exact residual
// e = x - q0 s (one FMA: q0 is within one unit in the last place of the quotient), q = RN(q0 + e r).  With a correctly
// rounded reciprocal this is the correctly rounded quotient (Markstein's correction step), the value __fdiv_rn(x, s)
// gives, at 3 instructions instead of a subroutine.  The residual is NaN exactly when x or s is not finite (r is then
// 0, inf or NaN, or q0 s is inf - inf); q0 already equals IEEE x / s there (inf, 0 or NaN).  kvq_selftest_division
// compares the two over every pair of fp32 significands on request.
struct FastDiv {
    float s, r;
    __device__ __forceinline__ explicit FastDiv(float s_) {
        s = s_;
        r = __frcp_rn(s_);
    }
    __device__ __forceinline__ float operator()(float x) const {
#ifdef KVQ_IEEE_DIV
        return __fdiv_rn(x, s);
#endif
        const float q0 = __fmul_rn(x, r);
        const float e = __fmaf_rn(-q0, s, x);
        const float q = __fmaf_rn(e, r, q0);
        return (e != e) ? q0 : q;
    }
};

// x / Q for Q = 7, 15, 127, 255 (the code ranges): the same reciprocal-and-residual division with the compile-time
// correctly rounded 1 / Q.  `ieee`: x may be infinite or NaN.
template <int Q>
__device__ __forceinline__ float div_const(float x, bool ieee) {
    if (ieee) return __fdiv_rn(x, (float)Q);
    constexpr float r = 1.0f / (float)Q;
    const float q0 = __fmul_rn(x, r);
    return __fmaf_rn(__fmaf_rn(-q0, (float)Q, x), r, q0);
}

// equal as numbers (the sign of a zero quotient is not kept: x = -0 gives +0; the integer code has no sign of zero)
__device__ __forceinline__ bool same_quotient(float x, float s, const FastDiv& d) {
    const float a = d(x), b = __fdiv_rn(x, s);
    return a == b || (a != a && b != b);
}

// mode 0, part 1: blockIdx.x * blockDim.x + threadIdx.x = index of a divisor significand (times stride); every thread
// walks the 65 536 fp16 dividends
__global__ void selftest_div_fp16_kernel(uint32_t stride, uint32_t count, unsigned long long* bad) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float s = __uint_as_float(0x3f800000u | (i * stride));
    const FastDiv d(s);
    unsigned n = 0;
    for (uint32_t h = 0; h < 65536u; ++h) n += !same_quotient(__half2float(__ushort_as_half((unsigned short)h)), s, d);
    if (n) atomicAdd(bad, (unsigned long long)n);
}

// mode 0, part 2: divisor = exponent field e (0 .. 255, which includes 0 / subnormals at e = 0 and inf / NaN at
// e = 255) with a coarse significand sweep
__global__ void selftest_div_binades_kernel(unsigned long long* bad) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;     // 256 exponents x 1024 significands
    if (i >= 256u * 1024u) return;
    const float s = __uint_as_float(((i >> 10) << 23) | ((i & 1023u) * 8191u));
    const FastDiv d(s);
    // 2^-17 .. 2^16 is what a scale can be (the quantizers clamp it to >= 1e-5); inf and NaN come from such inputs
    const bool in_range = (s >= 7.62939453125e-06f && s <= 65536.0f) || (i >> 10) == 255u;
    if (!in_range) return;
    const FastDiv dn(-s);
    unsigned n = 0;
    for (uint32_t h = 0; h < 65536u; ++h) {
        const float x = __half2float(__ushort_as_half((unsigned short)h));
        n += !same_quotient(x, s, d);
        n += !same_quotient(x, -s, dn);
    }
    if (n) atomicAdd(bad, (unsigned long long)n);
}

// mode 0, part 3: every fp32 dividend significand over the constant divisors of the code ranges
__global__ void selftest_div_const_kernel(unsigned long long* bad) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;     // 2^23 dividends
    const float x = __uint_as_float(0x3f800000u | i);
    unsigned n = 0;
    n += div_const<7>(x, false) != __fdiv_rn(x, 7.0f);
    n += div_const<15>(x, false) != __fdiv_rn(x, 15.0f);
    n += div_const<127>(x, false) != __fdiv_rn(x, 127.0f);
    n += div_const<255>(x, false) != __fdiv_rn(x, 255.0f);
    if (n) atomicAdd(bad, (unsigned long long)n);
}

// mode 1: thread = one divisor significand, loop over the dividend significands
__global__ void selftest_div_full_kernel(uint32_t stride, uint32_t first, uint32_t count, unsigned long long* bad) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;     // 2^23 divisors
    const float s = __uint_as_float(0x3f800000u | i);
    const FastDiv d(s);
    unsigned n = 0;
    for (uint32_t k = 0; k < count; ++k) n += !same_quotient(__uint_as_float(0x3f800000u | ((first + k) * stride)), s, d);
    if (n) atomicAdd(bad, (unsigned long long)n);
}

// Work item = one thread = CH consecutive channels of one (side, b, h, token) row.
//   CH > 0: the channels are fetched with 16-byte loads into registers and every loop over them unrolls
//           (the decode-time append is a chain of dependent loads otherwise).  A quantisation group is
//           CH * LPG channels: LPG adjacent lanes (1, 2 or 4) share it and combine their statistics with
//           warp shuffles, so groups of 64 and 128 channels keep the 32-channel register footprint.
//   CH == 0: any group size, one thread per group, element-wise loads.
template <int FMT, int POLICY, int CH, int LPG>
__global__ void __launch_bounds__(128) quantize_append_kernel(const QuantParams p) {
    pdl_launch_dependents();      // the decode kernel that follows may start its prologue now
    pdl_wait();                   // launched early itself: the kernel before it may still produce the new tokens
    const KvqAppendArgs& a = p.a;
    const int G = p.G;
    const int gs = CH ? CH * LPG : a.group_size;
    const int cw = CH ? CH : gs;                            // channels of this work item
    const int cpr = CH ? a.D / CH : G;                      // work items per row
    const long long per_side = (long long)a.B * a.Hkv * a.T * cpr;
    long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool is_kv = gid < p.nsides * per_side;
    // lanes that quantize; groups never straddle this boundary (cpr is a multiple of LPG)
    const unsigned kvmask = __ballot_sync(0xffffffffu, is_kv);
    if (!is_kv) {
        // ---- query rows: rotate and store, nothing to quantize
        gid -= p.nsides * per_side;
        if (gid >= p.q_items) return;
        const int c = (int)(gid % cpr);
        long long r = gid / cpr;
        const int t = (int)(r % a.T); r /= a.T;
        const int h = (int)(r % a.Hq);
        const int b = (int)(r / a.Hq);
        const __half* row = (const __half*)a.q_src + b * a.q_stride_b + h * a.q_stride_h + t * a.q_stride_t;
        const __half* cs = (const __half*)a.rope_cos + b * a.rope_stride_b + t * a.rope_stride_t;
        const __half* sn = (const __half*)a.rope_sin + b * a.rope_stride_b + t * a.rope_stride_t;
        __half* dst = (__half*)a.q_out + b * a.qo_stride_b + h * a.qo_stride_h + t * a.qo_stride_t;
        for (int i = c * cw; i < (c + 1) * cw; ++i) dst[i] = rope_one(row, cs, sn, a.rotary_dim, i);
        return;
    }
    const int sidx = gid >= per_side;
    if (sidx) gid -= per_side;
    const KvqAppendSide& sd = sidx ? a.v : a.k;
    const int c = (int)(gid % cpr);                         // chunk of the row
    const int g = c / LPG;                                  // its quantisation group
    const int cb = c * cw;                                  // its first channel
    long long r = gid / cpr;
    const int t = (int)(r % a.T); r /= a.T;
    const int h = (int)(r % a.Hkv);
    const int b = (int)(r / a.Hkv);
    long long pos = a.write_pos_dev ? (long long)(*a.write_pos_dev) : a.write_pos;
    pos += t;
    // a slot beyond the destination buffers (a graph replayed once too often, a stale device counter): nothing of
    // this token is stored, the flag is raised, and the lane keeps running so that group shuffles stay complete
    const bool in_range = a.max_slots <= 0 || (pos >= 0 && pos < a.max_slots);
    if (!in_range) {
        g_quantize_error_flag = 1;
        pos = 0;
    }

    const __half* src = (const __half*)sd.src + b * sd.src_stride_b + h * sd.src_stride_h +
                        t * sd.src_stride_t + cb;
    // rotary embedding applies to the K side only
    const bool rope = a.rope_cos != nullptr && sidx == 0;
    const __half* rcos = rope ? (const __half*)a.rope_cos + b * a.rope_stride_b + t * a.rope_stride_t : nullptr;
    const __half* rsin = rope ? (const __half*)a.rope_sin + b * a.rope_stride_b + t * a.rope_stride_t : nullptr;
    char* pay = (char*)sd.payload + b * sd.pay_stride_b + h * sd.pay_stride_h + pos * sd.pay_stride_s;

    if (FMT == KVQ_FMT_FP16) {
        __half* dst = (__half*)pay + cb;
        if (!in_range) return;
        if (rope) {
            for (int i = 0; i < cw; ++i) dst[i] = rope_one(src - cb, rcos, rsin, a.rotary_dim, cb + i);
        } else if (CH) {
#pragma unroll
            for (int i = 0; i < (CH ? CH : 8); i += 8) *(uint4*)(dst + i) = *(const uint4*)(src + i);
        } else {
            for (int i = 0; i < cw; ++i) dst[i] = src[i];
        }
        return;
    }

    float xr[CH ? CH : 1];
    if (CH) {
#pragma unroll
        for (int i = 0; i < (CH ? CH : 8); i += 8) {
            const uint4 v = *(const uint4*)(src + i);
            const __half2* h2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                xr[CH ? i + 2 * j : 0] = __low2float(h2[j]);
                xr[CH ? i + 2 * j + 1 : 0] = __high2float(h2[j]);
            }
        }
    }

    if (CH && rope && cb < a.rotary_dim) {
        // the launcher only takes this path when rotary_dim is a multiple of 2 * CH: the partner
        // channels are one whole chunk, rotary_dim / 2 away
        const int hf = a.rotary_dim >> 1;
        const bool low = cb < hf;
        const __half* prt = src + (low ? hf : -hf);
        const __half* cs = rcos + cb;
        const __half* sn = rsin + cb;
#pragma unroll
        for (int i = 0; i < (CH ? CH : 8); i += 8) {
            const uint4 pv = *(const uint4*)(prt + i), cv = *(const uint4*)(cs + i), sv = *(const uint4*)(sn + i);
            const __half* ph = reinterpret_cast<const __half*>(&pv);
            const __half* ch = reinterpret_cast<const __half*>(&cv);
            const __half* sh = reinterpret_cast<const __half*>(&sv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const __half x = __float2half_rn(xr[CH ? i + j : 0]);            // exact: it came from fp16
                const __half partner = low ? __hneg(ph[j]) : ph[j];
                xr[CH ? i + j : 0] = h2f(__hadd_rn(__hmul_rn(x, ch[j]), __hmul_rn(partner, sh[j])));
            }
        }
    }
    // the value the quantizer sees for channel i of this work item, before outlier handling
    auto raw = [&](int i) -> __half {
        return rope ? rope_one(src - cb, rcos, rsin, a.rotary_dim, cb + i) : src[i];
    };

    // outlier channels of this head that fall in this work item: copy raw, treat as 0
    const int16_t* oidx = a.n_out ? a.outlier_idx + h * a.n_out : nullptr;
    if (oidx && sd.side && in_range) {
        __half* side = (__half*)sd.side + b * sd.side_stride_b + h * sd.side_stride_h + pos * sd.side_stride_s;
        for (int j = 0; j < a.n_out; ++j) {
            int ch = oidx[j] - cb;
            if (ch >= 0 && ch < cw) side[j] = raw(ch);
        }
    }
    if (CH && oidx) {
        for (int j = 0; j < a.n_out; ++j) {
            const int ch = oidx[j] - cb;
#pragma unroll
            for (int i = 0; i < (CH ? CH : 1); ++i)
                if (i == ch) xr[CH ? i : 0] = 0.0f;
        }
    }
    auto load = [&](int i) -> float {
        if (CH) return xr[CH ? i : 0];
        if (oidx) {
            for (int j = 0; j < a.n_out; ++j)
                if (oidx[j] == cb + i) return 0.0f;
        }
        return h2f(raw(i));
    };
    // statistics of the whole group: this work item's channels, then the other lanes of the group
    auto group_max = [&](float v) -> float {
#pragma unroll
        for (int o = 1; o < LPG; o <<= 1) v = fmaxf(v, __shfl_xor_sync(kvmask, v, o));
        return v;
    };
    auto group_min = [&](float v) -> float {
#pragma unroll
        for (int o = 1; o < LPG; o <<= 1) v = fminf(v, __shfl_xor_sync(kvmask, v, o));
        return v;
    };
    auto chunk_amax = [&]() -> float {
        float amax = 0.f;   // |x| is exact in fp16, so the fp32 max equals the fp16 amax
#pragma unroll
        for (int i = 0; i < cw; ++i) amax = fmaxf(amax, fabsf(load(i)));
        return amax;
    };

    const long long sc_off = b * sd.sc_stride_b + h * sd.sc_stride_h + pos * sd.sc_stride_s + g;
    float s32 = 1.0f, zp32 = 0.0f;   // scale used for the division (fp32 value)

    if (POLICY == KVQ_SCALE_STATIC) {
        float st = sd.static_scale_is_f32 ? ((const float*)sd.static_scale)[h * G + g]
                                          : h2f(((const __half*)sd.static_scale)[h * G + g]);
        s32 = st;
        if (a.flags & (KVQ_F_ADAPTIVE | KVQ_F_MIXED_RESCUE | KVQ_F_RESCUE_THR)) {
            const float amax = group_max(chunk_amax());
            const float qmax = (FMT == KVQ_FMT_INT8) ? 127.0f : 7.0f;
            float dyn = __fdiv_rn(fmaxf(amax, 1e-5f), qmax);
            s32 = fmaxf(s32, 1e-5f);
            if ((a.flags & KVQ_F_ADAPTIVE) && !(a.flags & (sidx ? KVQ_F_ADAPT_SKIP_V : KVQ_F_ADAPT_SKIP_K)))
                s32 = fmaxf(__fmul_rn(s32, a.adaptive_margin), dyn);
            if (a.flags & KVQ_F_MIXED_RESCUE) s32 = fmaxf(s32, dyn);
            if (a.flags & KVQ_F_RESCUE_THR) {
                float thr = *sd.rescue_threshold;
                if (dyn >= thr) s32 = fmaxf(s32, dyn);
            }
        }
        s32 = fmaxf(s32, 1e-5f);
    } else if (POLICY == KVQ_SCALE_DYNAMIC_PCT) {
        float amax;
        if (a.quantile < 1.0f) {
            if (CH || top2_applies(gs, a.quantile)) {
                // only the two largest magnitudes matter (the launcher checked this for CH > 0)
                float m1 = 0.f, m2 = 0.f;
#pragma unroll
                for (int i = 0; i < cw; ++i) {
                    const float v = fabsf(load(i));
                    m2 = fmaxf(m2, fminf(m1, v));
                    m1 = fmaxf(m1, v);
                }
#pragma unroll
                for (int o = 1; o < LPG; o <<= 1) {
                    const float o1 = __shfl_xor_sync(kvmask, m1, o), o2 = __shfl_xor_sync(kvmask, m2, o);
                    m2 = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
                    m1 = fmaxf(m1, o1);
                }
                amax = fmaxf(top2_quantile(m1, m2, gs, a.quantile), 1e-5f);
            } else {
                float vals[kMaxGroup];
                for (int i = 0; i < gs; ++i) vals[i] = fabsf(load(i));
                amax = fmaxf(group_quantile(vals, gs, a.quantile), 1e-5f);
            }
            if (FMT == KVQ_FMT_INT8) amax = h2f(__float2half_rn(amax));
        } else {
            // the reference clamps the fp16 amax in fp16
            amax = h2f(__float2half_rn(fmaxf(group_max(chunk_amax()), 1e-5f)));
        }
        if (FMT == KVQ_FMT_INT8) {
            s32 = h2f(__float2half_rn(__fdiv_rn(amax, 127.0f)));   // "/127" runs in fp16
        } else {
            s32 = __fdiv_rn(fmaxf(amax, 1e-5f), 7.0f);
        }
    } else {  // KVQ_SCALE_ASYM_MINMAX
        float mn = INFINITY, mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < cw; ++i) {
            float x = load(i);
            mn = fminf(mn, x);
            mx = fmaxf(mx, x);
        }
        mn = group_min(mn);
        mx = group_max(mx);
        const float qspan = (FMT == KVQ_FMT_INT8) ? 255.0f : 15.0f;
        const float qmin = (FMT == KVQ_FMT_INT8) ? -128.0f : -8.0f;
        const float floor_rng = fmaxf(1e-5f, __fmul_rn(6.103515625e-05f, qspan));
        float rng = fmaxf(__fsub_rn(mx, mn), floor_rng);
        s32 = __fdiv_rn(rng, qspan);
        zp32 = __fsub_rn(mn, __fmul_rn(qmin, s32));
    }

    // stored (kernel-facing) scale is fp16; one lane of the group writes it
    __half s16 = __float2half_rn(s32);
    if (FMT == KVQ_FMT_INT8 && POLICY != KVQ_SCALE_ASYM_MINMAX) s32 = h2f(s16);  // INT8 divides by the fp16 scale
    if (!in_range) return;                               // every shuffle of the group is behind us
    if (LPG == 1 || (c % LPG) == 0) {
        ((__half*)sd.scale)[sc_off] = s16;
        if (sd.scale_f32) sd.scale_f32[sc_off] = s32;
        if (POLICY == KVQ_SCALE_ASYM_MINMAX) ((__half*)sd.zp)[sc_off] = __float2half_rn(zp32);
    }

    const FastDiv by_scale(s32);
    auto code_of = [&](int i) -> int {
        float x = load(i);
        float qv;
        if (POLICY == KVQ_SCALE_ASYM_MINMAX) {
            qv = rintf(by_scale(__fsub_rn(x, zp32)));
            return (FMT == KVQ_FMT_INT8) ? (int)fminf(fmaxf(qv, -128.f), 127.f)
                                         : (int)fminf(fmaxf(qv, -8.f), 7.f);
        }
        if (FMT == KVQ_FMT_INT8) {
            qv = rintf(h2f(__float2half_rn(by_scale(x))));
            return (int)fminf(fmaxf(qv, -127.f), 127.f);
        }
        qv = rintf(by_scale(x));
        return (int)fminf(fmaxf(qv, -7.f), 7.f);
    };

    if (FMT == KVQ_FMT_INT8 || (a.flags & KVQ_F_UNPACKED)) {
        int8_t* dst = (int8_t*)pay + cb;
#pragma unroll
        for (int i = 0; i < cw; i += 4) {
            int c0 = code_of(i), c1 = code_of(i + 1), c2 = code_of(i + 2), c3 = code_of(i + 3);
            uint32_t w = (uint32_t)(c0 & 0xff) | ((uint32_t)(c1 & 0xff) << 8) |
                         ((uint32_t)(c2 & 0xff) << 16) | ((uint32_t)(c3 & 0xff) << 24);
            *(uint32_t*)(dst + i) = w;
        }
    } else {
        uint8_t* dst = (uint8_t*)pay + cb / 2;
#pragma unroll
        for (int i = 0; i < cw; i += 8) {
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int c0 = code_of(i + 2 * j) + 8, c1 = code_of(i + 2 * j + 1) + 8;
                w |= (uint32_t)(((c0 & 0xf) << 4) | (c1 & 0xf)) << (8 * j);
            }
            *(uint32_t*)(dst + i / 2) = w;
        }
    }
}

// ---------------------------------------------------------------------------
// Bulk form (prefill: thousands of tokens per launch).  Same results as the kernel above, bit for bit; the work
// decomposition and the instruction sequence are made for throughput (the per-token form spends ~34 instructions per
// element, which at prefill sizes is the bound, not the memory system):
//   thread  = CH = 16 consecutive channels (two 16-byte loads) of one token row; a group is LPG = group_size / 16
//             adjacent lanes (group 16: CH = 8, LPG = 2), statistics combined with shuffles;
//   block   = 256 threads = 256 / (D / CH) token rows per pass, U passes with all loads issued first;
//   grid    = (token tiles, head, side x batch): no per-thread division chain;
//   group statistics on the packed fp16 pairs (min, max and |max| of fp16 values are exact in fp16);
//   x / s   = FastDiv without the NaN select: a chunk with a value that is not finite takes IEEE division;
//   code    = clamp first, then round by adding 1.5 * 2^23 (round-to-nearest-even of the addition is rintf; the
//             bounds are integers, so clamp-then-round equals round-then-clamp, and a NaN quotient still becomes the
//             lower bound through fmaxf) - the integer sits in the low bits of the sum's bit pattern.
// Taken when the source rows allow 16-byte loads, without rotary embedding and query rows.
// ---------------------------------------------------------------------------
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

template <int FMT, int POLICY, int CH, int LPG, int U>
__global__ void __launch_bounds__(256) quantize_bulk_kernel(const QuantParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const KvqAppendArgs& a = p.a;
    constexpr int NW = CH / 2;                             // 32-bit words (fp16 pairs) of a chunk
    const int G = p.G;
    const int cpr_log2 = 31 - __clz(a.D / CH);             // chunks per token row: a power of two (D = 64, 128, 256)
    const int rows = 256 >> cpr_log2;                      // token rows per pass
    const int c = threadIdx.x & ((1 << cpr_log2) - 1), rloc = threadIdx.x >> cpr_log2;
    const int h = blockIdx.y;
    const int sidx = blockIdx.z >= (unsigned)a.B;          // grid.z = side x batch
    const int b = blockIdx.z - (sidx ? a.B : 0);
    const KvqAppendSide sd = sidx ? a.v : a.k;             // by value: the fields used below are selected once
    const int g = c / LPG, cb = c * CH;
    const int flags = a.flags, n_out = a.n_out, T = a.T;
    const long long pos0 = a.write_pos_dev ? (long long)(*a.write_pos_dev) : a.write_pos;
    // tokens [t_lo, t_hi) have a slot inside the destination buffers (slot = pos0 + t); the others store nothing
    const int t_lo = (a.max_slots > 0 && pos0 < 0) ? (int)min(-pos0, (long long)T) : 0;
    const int t_hi = a.max_slots > 0 ? (int)max(0ll, min((long long)T, a.max_slots - pos0)) : T;
    if (t_lo > 0 || t_hi < T) g_quantize_error_flag = 1;
    const int t_base = blockIdx.x * (rows * U) + rloc;
    // everything of token t_base; pass u is u * rows tokens further
    const __half* src_t = (const __half*)sd.src + b * sd.src_stride_b + h * sd.src_stride_h + cb + (long long)t_base * sd.src_stride_t;
    char* pay_t = (char*)sd.payload + b * sd.pay_stride_b + h * sd.pay_stride_h + (pos0 + t_base) * sd.pay_stride_s;
    const long long sc_t = b * sd.sc_stride_b + h * sd.sc_stride_h + g + (pos0 + t_base) * sd.sc_stride_s;
    const long long src_step = (long long)rows * sd.src_stride_t, pay_step = (long long)rows * sd.pay_stride_s,
                    sc_step = (long long)rows * sd.sc_stride_s;
    const int16_t* oidx = n_out ? a.outlier_idx + h * n_out : nullptr;
    const bool wide_store = FMT == KVQ_FMT_INT8 || (flags & KVQ_F_UNPACKED);
    const float quantile = a.quantile, margin = a.adaptive_margin;

    uint32_t raw[U][NW];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int t = t_base + u * rows;
#pragma unroll
        for (int i = 0; i < NW; i += 4) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (t < T) v = __ldcs(reinterpret_cast<const uint4*>(src_t + u * src_step) + i / 4);
            raw[u][i] = v.x; raw[u][i + 1] = v.y; raw[u][i + 2] = v.z; raw[u][i + 3] = v.w;
        }
    }

    float st_scale = 1.0f;                                 // static table entry of this (head, group)
    if (POLICY == KVQ_SCALE_STATIC)
        st_scale = sd.static_scale_is_f32 ? ((const float*)sd.static_scale)[h * G + g]
                                          : h2f(((const __half*)sd.static_scale)[h * G + g]);
    const bool need_amax = POLICY == KVQ_SCALE_DYNAMIC_PCT ||
                           (POLICY == KVQ_SCALE_STATIC && (flags & (KVQ_F_ADAPTIVE | KVQ_F_MIXED_RESCUE | KVQ_F_RESCUE_THR)));

#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int t = t_base + u * rows;
        const bool in_range = t >= t_lo && t < t_hi;       // other rows compute (on zeros past T) and store nothing
        uint32_t* w = raw[u];
        if (oidx) {
            __half* side = sd.side ? (__half*)sd.side + b * sd.side_stride_b + h * sd.side_stride_h + (pos0 + t) * sd.side_stride_s : nullptr;
            for (int j = 0; j < n_out; ++j) {
                const int ch = oidx[j] - cb;
#pragma unroll
                for (int i = 0; i < CH; ++i)
                    if (i == ch) {
                        if (side && in_range) side[j] = __ushort_as_half((unsigned short)((i & 1) ? (w[i >> 1] >> 16) : (w[i >> 1] & 0xffffu)));
                        w[i >> 1] &= (i & 1) ? 0x0000ffffu : 0xffff0000u;
                    }
            }
        }
        // a value that is not finite anywhere in the chunk (or a sum of two that overflows: harmless) -> IEEE division
        bool odd;
        {
            __half2 acc = u32_as_h2(w[0]);                 // inf and NaN survive any sum
#pragma unroll
            for (int i = 1; i < NW; ++i) acc = __hadd2(acc, u32_as_h2(w[i]));
            const float2 f = __half22float2(acc);
            odd = !(fabsf(f.x) <= 3.0e38f && fabsf(f.y) <= 3.0e38f);
        }
        auto group_max = [&](float v) -> float {
#pragma unroll
            for (int o = 1; o < LPG; o <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
            return v;
        };
        auto group_min = [&](float v) -> float {
#pragma unroll
            for (int o = 1; o < LPG; o <<= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
            return v;
        };
        constexpr int gs = CH * LPG;
        float s32 = 1.0f, zp32 = 0.0f;
        float amax = 0.f;
        if (need_amax && !(POLICY == KVQ_SCALE_DYNAMIC_PCT && quantile < 1.0f)) {
            __half2 m = __habs2(u32_as_h2(w[0]));
#pragma unroll
            for (int i = 1; i < NW; ++i) m = __hmax2(m, __habs2(u32_as_h2(w[i])));
            amax = group_max(h2f(__hmax(__low2half(m), __high2half(m))));
        }
        if (POLICY == KVQ_SCALE_STATIC) {
            s32 = st_scale;
            if (flags & (KVQ_F_ADAPTIVE | KVQ_F_MIXED_RESCUE | KVQ_F_RESCUE_THR)) {
                const float dyn = FMT == KVQ_FMT_INT8 ? div_const<127>(fmaxf(amax, 1e-5f), !(amax <= 3.0e38f)) : div_const<7>(fmaxf(amax, 1e-5f), !(amax <= 3.0e38f));
                s32 = fmaxf(s32, 1e-5f);
                if ((flags & KVQ_F_ADAPTIVE) && !(flags & (sidx ? KVQ_F_ADAPT_SKIP_V : KVQ_F_ADAPT_SKIP_K)))
                    s32 = fmaxf(__fmul_rn(s32, margin), dyn);
                if (flags & KVQ_F_MIXED_RESCUE) s32 = fmaxf(s32, dyn);
                if (flags & KVQ_F_RESCUE_THR) {
                    const float thr = *sd.rescue_threshold;
                    if (dyn >= thr) s32 = fmaxf(s32, dyn);
                }
            }
            s32 = fmaxf(s32, 1e-5f);
        } else if (POLICY == KVQ_SCALE_DYNAMIC_PCT) {
            if (quantile < 1.0f) {                       // the launcher checked that the two largest values decide
                float m1 = 0.f, m2 = 0.f;
#pragma unroll
                for (int i = 0; i < NW; ++i) {
                    const float2 f = __half22float2(__habs2(u32_as_h2(w[i])));
                    m2 = fmaxf(m2, fminf(m1, f.x));
                    m1 = fmaxf(m1, f.x);
                    m2 = fmaxf(m2, fminf(m1, f.y));
                    m1 = fmaxf(m1, f.y);
                }
#pragma unroll
                for (int o = 1; o < LPG; o <<= 1) {
                    const float o1 = __shfl_xor_sync(0xffffffffu, m1, o), o2 = __shfl_xor_sync(0xffffffffu, m2, o);
                    m2 = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
                    m1 = fmaxf(m1, o1);
                }
                amax = fmaxf(top2_quantile(m1, m2, gs, quantile), 1e-5f);
                if (FMT == KVQ_FMT_INT8) amax = h2f(__float2half_rn(amax));
            } else {
                amax = h2f(__float2half_rn(fmaxf(amax, 1e-5f)));
            }
            if (FMT == KVQ_FMT_INT8) s32 = h2f(__float2half_rn(div_const<127>(amax, !(amax <= 3.0e38f))));
            else s32 = div_const<7>(fmaxf(amax, 1e-5f), !(amax <= 3.0e38f));
        } else {
            __half2 lo2 = u32_as_h2(w[0]), hi2 = lo2;
#pragma unroll
            for (int i = 1; i < NW; ++i) { lo2 = __hmin2(lo2, u32_as_h2(w[i])); hi2 = __hmax2(hi2, u32_as_h2(w[i])); }
            const float mn = group_min(h2f(__hmin(__low2half(lo2), __high2half(lo2))));
            const float mx = group_max(h2f(__hmax(__low2half(hi2), __high2half(hi2))));
            constexpr float qmin = (FMT == KVQ_FMT_INT8) ? -128.0f : -8.0f;
            // max(1e-5, 2^-14 * span): 2^-14 * 255 and 2^-14 * 15 are exact products, both above 1e-5
            constexpr float floor_rng = 6.103515625e-05f * ((FMT == KVQ_FMT_INT8) ? 255.0f : 15.0f);
            const float rng = fmaxf(__fsub_rn(mx, mn), floor_rng);
            s32 = FMT == KVQ_FMT_INT8 ? div_const<255>(rng, !(rng <= 3.0e38f)) : div_const<15>(rng, !(rng <= 3.0e38f));
            zp32 = __fsub_rn(mn, __fmul_rn(qmin, s32));
        }
        const __half s16 = __float2half_rn(s32);
        if (FMT == KVQ_FMT_INT8 && POLICY != KVQ_SCALE_ASYM_MINMAX) s32 = h2f(s16);
        if (in_range && (c % LPG) == 0) {
            const long long sc_off = sc_t + u * sc_step;
            ((__half*)sd.scale)[sc_off] = s16;
            if (sd.scale_f32) sd.scale_f32[sc_off] = s32;
            if (POLICY == KVQ_SCALE_ASYM_MINMAX) ((__half*)sd.zp)[sc_off] = __float2half_rn(zp32);
        }
        odd = odd || !(fabsf(s32) <= 3.0e38f) || !(fabsf(zp32) <= 3.0e38f);
        const float r32 = __frcp_rn(s32);
        constexpr float lo_b = (POLICY == KVQ_SCALE_ASYM_MINMAX) ? (FMT == KVQ_FMT_INT8 ? -128.f : -8.f) : (FMT == KVQ_FMT_INT8 ? -127.f : -7.f);
        constexpr float hi_b = (FMT == KVQ_FMT_INT8) ? 127.f : 7.f;
        if (!in_range) continue;
        char* pay = pay_t + u * pay_step;
        constexpr float kMagic = 12582912.0f;              // 1.5 * 2^23: ulp 1
        // the codes of the chunk; IEEE = true divides with __fdiv_rn (chunks with a value that is not finite)
        auto emit = [&](auto ieee) {
            constexpr bool IEEE = decltype(ieee)::value;
            auto quotient = [&](float x) -> float {
                if (POLICY == KVQ_SCALE_ASYM_MINMAX) x = __fsub_rn(x, zp32);
                if (IEEE) return __fdiv_rn(x, s32);
                const float q0 = __fmul_rn(x, r32);
                return __fmaf_rn(__fmaf_rn(-q0, s32, x), r32, q0);
            };
            if (FMT == KVQ_FMT_INT8 && POLICY != KVQ_SCALE_ASYM_MINMAX) {
                // the reference rounds the quotient to fp16 first: stay in fp16 pairs.  Clamp, then round by adding
                // 1.5 * 2^10 (ulp 1 in fp16): the bit pattern is 0x6600 + code, the code is its low byte.
                const __half2 lo2 = __float2half2_rn(lo_b), hi2 = __float2half2_rn(hi_b), magic2 = __float2half2_rn(1536.f);
                uint32_t out[CH / 4];
#pragma unroll
                for (int i = 0; i < NW; i += 2) {
                    uint32_t tb[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float2 f = __half22float2(u32_as_h2(w[i + e]));
                        const __half2 q = __floats2half2_rn(quotient(f.x), quotient(f.y));
                        const __half2 t = __hadd2_rn(__hmin2(__hmax2(q, lo2), hi2), magic2);
                        tb[e] = *reinterpret_cast<const uint32_t*>(&t);
                    }
                    out[i / 2] = prmt(tb[0], tb[1], 0x6420u);
                }
#pragma unroll
                for (int i = 0; i < CH / 4; i += 2) __stcs(reinterpret_cast<uint2*>(pay + cb) + i / 2, make_uint2(out[i], out[i + 1]));
            } else if (wide_store) {
                // one code per byte: byte = low 8 bits of (clamped quotient + magic)
                uint32_t out[CH / 4];
#pragma unroll
                for (int i = 0; i < NW; i += 2) {
                    uint32_t tb[4];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float2 f = __half22float2(u32_as_h2(w[i + e]));
                        tb[2 * e] = __float_as_uint(__fadd_rn(fminf(fmaxf(quotient(f.x), lo_b), hi_b), kMagic));
                        tb[2 * e + 1] = __float_as_uint(__fadd_rn(fminf(fmaxf(quotient(f.y), lo_b), hi_b), kMagic));
                    }
                    out[i / 2] = prmt(prmt(tb[0], tb[1], 0x0040u), prmt(tb[2], tb[3], 0x0040u), 0x5410u);
                }
#pragma unroll
                for (int i = 0; i < CH / 4; i += 2) __stcs(reinterpret_cast<uint2*>(pay + cb) + i / 2, make_uint2(out[i], out[i + 1]));
            } else {
                // two codes per byte, channel 2j in the high nibble.  The bit pattern of (clamped quotient + magic + 8)
                // is 0x4B400000 + code + 8, so t_even * 16 + t_odd has the byte in its low 8 bits.
                uint32_t out[CH / 8];
#pragma unroll
                for (int i = 0; i < NW; i += 4) {
                    uint32_t by[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(u32_as_h2(w[i + e]));
                        const uint32_t t0 = __float_as_uint(__fadd_rn(fminf(fmaxf(quotient(f.x), lo_b), hi_b), kMagic + 8.f));
                        const uint32_t t1 = __float_as_uint(__fadd_rn(fminf(fmaxf(quotient(f.y), lo_b), hi_b), kMagic + 8.f));
                        by[e] = t0 * 16u + t1;
                    }
                    out[i / 4] = prmt(prmt(by[0], by[1], 0x0040u), prmt(by[2], by[3], 0x0040u), 0x5410u);
                }
                if (CH == 16) __stcs(reinterpret_cast<uint2*>(pay + cb / 2), make_uint2(out[0], out[CH == 16 ? 1 : 0]));
                else __stcs(reinterpret_cast<uint32_t*>(pay + cb / 2), out[0]);
            }
        };
        if (odd) emit(std::true_type());
        else emit(std::false_type());
    }
}

template <int FMT, int POLICY, int CH, int LPG>
static int launch_bulk(const QuantParams& p, cudaStream_t st) {
    constexpr int U = 4;
    const int cpr = p.a.D / CH, rows = 256 / cpr;
    const long long tiles = ((long long)p.a.T + rows * U - 1) / (rows * U);
    const long long gz = (long long)p.nsides * p.a.B;
    if (tiles > 0x7fffffffLL || p.a.Hkv > 65535 || gz > 65535) return KVQ_EUNSUPPORTED;
    return launch_pdl(quantize_bulk_kernel<FMT, POLICY, CH, LPG, U>, dim3((unsigned)tiles, (unsigned)p.a.Hkv, (unsigned)gz), dim3(256),
                      0, st, p);
}

// Bulk form applies: enough rows to fill the machine, 16-byte loads and 8-byte payload stores possible,
// no rotary embedding / query rows, a percentile that the two largest values decide.
template <int FMT, int POLICY>
static bool bulk_ok(const QuantParams& p) {
    const KvqAppendArgs& a = p.a;
    if (FMT == KVQ_FMT_FP16 || getenv("KVQ_NO_BULK_QUANTIZE")) return false;
    if (a.rope_cos || a.q_src) return false;
    if (a.D != 64 && a.D != 128 && a.D != 256) return false;
    const int gs = a.group_size;
    if (gs != 16 && gs != 32 && gs != 64 && gs != 128) return false;
    if ((long long)a.B * a.Hkv * a.T < 8192) return false;
    if (POLICY == KVQ_SCALE_DYNAMIC_PCT && a.quantile < 1.0f && !top2_applies(gs, a.quantile)) return false;
    for (int s = 0; s < p.nsides; ++s) {
        const KvqAppendSide& sd = s ? a.v : a.k;
        if ((((uintptr_t)sd.src) & 15) || (sd.src_stride_b & 7) || (sd.src_stride_h & 7) || (sd.src_stride_t & 7)) return false;
        if ((((uintptr_t)sd.payload) | (uintptr_t)sd.pay_stride_b | (uintptr_t)sd.pay_stride_h | (uintptr_t)sd.pay_stride_s) & 7)
            return false;                                  // 8-byte payload stores
    }
    return true;
}

static bool side_vec_ok(const KvqAppendSide& s) {
    return !s.src || ((((uintptr_t)s.src) & 15) == 0 && (s.src_stride_b & 7) == 0 && (s.src_stride_h & 7) == 0 &&
                      (s.src_stride_t & 7) == 0);
}

template <int FMT, int POLICY, int CH, int LPG>
static int launch_gs(const QuantParams& p, cudaStream_t st) {
    const int cpr = CH ? p.a.D / CH : p.G;
    const long long per_row_set = (long long)p.a.B * p.a.T * cpr;
    const long long threads = per_row_set * p.a.Hkv * p.nsides + (p.q_items ? per_row_set * p.a.Hq : 0);
    if (threads == 0) return KVQ_OK;
    const int block = 128;
    const long long grid = (threads + block - 1) / block;
    if (grid > 0x7fffffffLL) return KVQ_EINVAL;
    QuantParams q = p;
    q.q_items = p.q_items ? per_row_set * p.a.Hq : 0;
    return launch_pdl(quantize_append_kernel<FMT, POLICY, CH, LPG>, dim3((unsigned)grid), dim3(block), 0, st, q);
}

template <int FMT, int POLICY>
static int launch(const QuantParams& p, cudaStream_t st) {
    const KvqAppendArgs& a = p.a;
    const int gs = a.group_size;
    // a percentile below 100 needs the sorted group unless its rank falls on the two largest values
    const bool dyn_sort = POLICY == KVQ_SCALE_DYNAMIC_PCT && a.quantile < 1.0f && !top2_applies(gs, a.quantile);
    if constexpr (FMT != KVQ_FMT_FP16) if (bulk_ok<FMT, POLICY>(p)) {
        int rc = KVQ_EUNSUPPORTED;
        if (gs == 16) rc = launch_bulk<FMT, POLICY, 8, 2>(p, st);
        if (gs == 32) rc = launch_bulk<FMT, POLICY, 16, 2>(p, st);
        if (gs == 64) rc = launch_bulk<FMT, POLICY, 16, 4>(p, st);
        if (gs == 128) rc = launch_bulk<FMT, POLICY, 16, 8>(p, st);
        if (rc != KVQ_EUNSUPPORTED) return rc;
    }
    const bool rope = a.rope_cos != nullptr;
    const bool rope_vec_ok = !rope || ((a.rotary_dim % 64) == 0 && ((((uintptr_t)a.rope_cos | (uintptr_t)a.rope_sin) & 15) == 0) &&
                                       (a.rope_stride_b & 7) == 0 && (a.rope_stride_t & 7) == 0);
    if (!dyn_sort && side_vec_ok(a.k) && side_vec_ok(a.v) && rope_vec_ok) {
        // register-resident chunks of 32 (or 16) channels; rotary partners are whole chunks
        if (FMT == KVQ_FMT_FP16 && a.D % 32 == 0) return launch_gs<FMT, POLICY, 32, 1>(p, st);   // a plain copy: any chunking
        // a handful of rows (one decode token): spread each group of 32 over two lanes - the per-element division
        // chain of a thread halves, and the launch is a latency chain, not a throughput kernel
        const long long groups = (long long)a.B * a.Hkv * a.T * (a.D / (gs > 0 ? gs : 1)) * p.nsides;
        if (gs == 32 && FMT != KVQ_FMT_FP16 && groups <= 4096) return launch_gs<FMT, POLICY, 16, 2>(p, st);
        if (gs == 32) return launch_gs<FMT, POLICY, 32, 1>(p, st);
        if (gs == 64) return launch_gs<FMT, POLICY, 32, 2>(p, st);
        if (gs == 128) return launch_gs<FMT, POLICY, 32, 4>(p, st);
        if (gs == 16) return launch_gs<FMT, POLICY, 16, 1>(p, st);
    }
    return launch_gs<FMT, POLICY, 0, 1>(p, st);
}

static bool side_ok(const KvqAppendSide& s, const KvqAppendArgs& a) {
    if (!s.src || !s.payload) return false;
    if (a.format != KVQ_FMT_FP16 && !s.scale) return false;
    if (a.policy == KVQ_SCALE_STATIC && a.format != KVQ_FMT_FP16 && !s.static_scale) return false;
    if (a.policy == KVQ_SCALE_ASYM_MINMAX && !s.zp) return false;
    if ((a.flags & KVQ_F_RESCUE_THR) && !s.rescue_threshold) return false;
    if (a.n_out > 0 && !s.side) return false;
    // 4-byte stores into the payload
    if (((uintptr_t)s.payload | (uintptr_t)s.pay_stride_b | (uintptr_t)s.pay_stride_h |
         (uintptr_t)s.pay_stride_s) & 3) return false;
    return true;
}

int quantize_error_flag(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_quantize_error_flag, sizeof(int)) != cudaSuccess) return KVQ_ECUDA;
    if (reset && v) {
        const int z = 0;
        if (cudaMemcpyToSymbol(g_quantize_error_flag, &z, sizeof(int)) != cudaSuccess) return KVQ_ECUDA;
    }
    return v;
}

}  // namespace kvq

extern "C" int kvq_selftest_division(int mode, uint32_t stride, uint64_t* mismatches, uint64_t* pairs) {
    using namespace kvq;
    if (!mismatches || stride == 0 || (mode != 0 && mode != 1)) return KVQ_EINVAL;
    unsigned long long* bad = nullptr;
    int rc = check_cuda(cudaMalloc(&bad, sizeof(unsigned long long)));
    if (rc) return rc;
    rc = check_cuda(cudaMemset(bad, 0, sizeof(unsigned long long)));
    unsigned long long n_pairs = 0;
    if (!rc && mode == 0) {
        const uint32_t count = ((1u << 23) + stride - 1) / stride;
        selftest_div_fp16_kernel<<<(count + 127) / 128, 128>>>(stride, count, bad);
        selftest_div_binades_kernel<<<256 * 1024 / 128, 128>>>(bad);
        selftest_div_const_kernel<<<(1u << 23) / 256, 256>>>(bad);
        n_pairs = (unsigned long long)count * 65536ull + 2ull * 256 * 1024 * 65536ull + (4ull << 23);
        rc = check_launch();
    } else if (!rc) {
        // launches of bounded length: 2^23 threads x `chunk` dividends each
        const uint32_t total = ((1u << 23) + stride - 1) / stride, chunk = 4096;
        for (uint32_t first = 0; first < total && !rc; first += chunk) {
            const uint32_t n = total - first < chunk ? total - first : chunk;
            selftest_div_full_kernel<<<(1u << 23) / 256, 256>>>(stride, first, n, bad);
            rc = check_launch();
            if (!rc) rc = check_cuda(cudaDeviceSynchronize());
        }
        n_pairs = (unsigned long long)total << 23;
    }
    if (!rc) rc = check_cuda(cudaDeviceSynchronize());
    unsigned long long v = 0;
    if (!rc) rc = check_cuda(cudaMemcpy(&v, bad, sizeof(v), cudaMemcpyDeviceToHost));
    cudaFree(bad);
    if (rc) return rc;
    *mismatches = v;
    if (pairs) *pairs = n_pairs;
    return KVQ_OK;
}

extern "C" int kvq_quantize_append(const KvqAppendArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    const KvqAppendArgs& a = *args;
    if (a.B < 0 || a.Hkv <= 0 || a.T < 0 || a.D <= 0) return KVQ_EINVAL;
    if (a.B == 0 || a.T == 0) return KVQ_OK;
    int gs = a.group_size == -1 ? a.D : a.group_size;
    if (gs <= 0 || a.D % gs != 0 || gs % 8 != 0 || gs > kMaxGroup) return KVQ_EINVAL;
    if (a.format != KVQ_FMT_FP16 && a.format != KVQ_FMT_INT8 && a.format != KVQ_FMT_INT4) return KVQ_EINVAL;
    if (a.policy < 0 || a.policy > 2) return KVQ_EINVAL;
    if (a.n_out < 0 || (a.n_out > 0 && !a.outlier_idx)) return KVQ_EINVAL;
    if (a.n_out > 0 && a.policy == KVQ_SCALE_ASYM_MINMAX) return KVQ_EUNSUPPORTED;
    if (a.write_pos < 0 || a.max_slots < 0) return KVQ_EINVAL;
    if (a.max_slots > 0 && !a.write_pos_dev && a.write_pos + a.T > a.max_slots) return KVQ_ELIMIT;
    QuantParams p;
    p.a = a;
    p.a.group_size = gs;
    p.G = a.D / gs;
    p.nsides = a.v.src ? 2 : 1;
    p.q_items = 0;
    if (a.rope_cos || a.rope_sin) {
        if (!a.rope_cos || !a.rope_sin || a.rotary_dim <= 0 || (a.rotary_dim & 1) || a.rotary_dim > a.D) return KVQ_EINVAL;
    }
    if (a.q_src) {
        if (!a.rope_cos || !a.q_out || a.Hq <= 0) return KVQ_EINVAL;
        p.q_items = 1;        // the launcher counts the work items of its chunking
    }
    if (!side_ok(a.k, p.a) || (p.nsides == 2 && !side_ok(a.v, p.a))) return KVQ_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
#define KVQ_DISPATCH(F, P) if (a.format == F && a.policy == P) return launch<F, P>(p, st);
    if (a.format == KVQ_FMT_FP16) return launch<KVQ_FMT_FP16, KVQ_SCALE_STATIC>(p, st);
    KVQ_DISPATCH(KVQ_FMT_INT8, KVQ_SCALE_STATIC)
    KVQ_DISPATCH(KVQ_FMT_INT8, KVQ_SCALE_DYNAMIC_PCT)
    KVQ_DISPATCH(KVQ_FMT_INT8, KVQ_SCALE_ASYM_MINMAX)
    KVQ_DISPATCH(KVQ_FMT_INT4, KVQ_SCALE_STATIC)
    KVQ_DISPATCH(KVQ_FMT_INT4, KVQ_SCALE_DYNAMIC_PCT)
    KVQ_DISPATCH(KVQ_FMT_INT4, KVQ_SCALE_ASYM_MINMAX)
#undef KVQ_DISPATCH
    return KVQ_EUNSUPPORTED;
}
