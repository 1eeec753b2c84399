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
// Work decomposition: one thread per (side, b, h, t, group).  Append traffic is
// tiny next to the attention scan (decode: B*Hkv rows of 256 B), so the kernel is
// launch-latency bound; what matters is that it is ONE launch with no host sync.

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

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

    auto code_of = [&](int i) -> int {
        float x = load(i);
        float qv;
        if (POLICY == KVQ_SCALE_ASYM_MINMAX) {
            qv = rintf(__fdiv_rn(__fsub_rn(x, zp32), s32));
            return (FMT == KVQ_FMT_INT8) ? (int)fminf(fmaxf(qv, -128.f), 127.f)
                                         : (int)fminf(fmaxf(qv, -8.f), 7.f);
        }
        if (FMT == KVQ_FMT_INT8) {
            qv = rintf(h2f(__float2half_rn(__fdiv_rn(x, s32))));
            return (int)fminf(fmaxf(qv, -127.f), 127.f);
        }
        qv = rintf(__fdiv_rn(x, s32));
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
