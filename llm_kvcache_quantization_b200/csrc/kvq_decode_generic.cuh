// Generic split-K decode-attention kernel: any payload format, group size,
// zero-points and outlier side buffer, head_dim 64/128/256, any GQA ratio.
// It is the shape-agnostic path; the tensor-core kernel in kvq_decode_mma.cuh
// takes the shapes it is specialised for.
//
// One CTA = (KV split, kv head x query-head chunk, batch row), 4 warps.  A warp
// walks 32-token chunks: lane = token for q.K (no shuffles), online softmax per
// chunk, then lane = head-dim slice for P.V with the probabilities broadcast by
// shuffle.  Dequantisation is RN16(fp16(code) * scale) (+ zero-point), i.e. the
// same fp16 values the torch reference multiplies (src/engine/patch_model.py:355-362).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "kvq_internal.h"

namespace kvq {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kHeadsPerCta = 8;

struct AttnParams {
    KvqAttnArgs a;
    int G;
    int n_rep;
    int rep_chunks;
    int splits;
    float* ws_o;    // [B, Hq, splits, D]
    float* ws_ml;   // [B, Hq, splits, 2]  (m in log2 domain, l)
};

__device__ __forceinline__ void split_range(int ctx, int splits, int split, int align, int& s0, int& s1) {
    int per = (ctx + splits - 1) / splits;
    per = ((per + align - 1) / align) * align;
    s0 = min(ctx, split * per);
    s1 = min(ctx, s0 + per);
}

// Load N consecutive elements (dims d0..d0+N) of one token row and dequantise
// them to float through the reference's fp16 arithmetic.
template <int FMT, bool ASYM, int N>
__device__ __forceinline__ void load_dequant(const char* row, int d0, __half sc, __half zp, float* out) {
    if (FMT == KVQ_FMT_FP16) {
        const __half* p = (const __half*)row + d0;
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            __half2 v = *(const __half2*)(p + i);
            out[i] = __low2float(v);
            out[i + 1] = __high2float(v);
        }
    } else if (FMT == KVQ_FMT_INT8) {
        const int8_t* p = (const int8_t*)row + d0;
        alignas(8) int8_t c[N];
        if (N == 2) *(uint16_t*)c = *(const uint16_t*)p;
        else if (N == 4) *(uint32_t*)c = *(const uint32_t*)p;
        else { *(uint2*)c = *(const uint2*)p; }
#pragma unroll
        for (int i = 0; i < N; ++i) {
            __half v = __hmul_rn(__int2half_rn((int)c[i]), sc);
            if (ASYM) v = __hadd_rn(v, zp);
            out[i] = __half2float(v);
        }
    } else {
        const uint8_t* p = (const uint8_t*)row + d0 / 2;
        alignas(4) uint8_t c[N / 2];
        if (N == 2) c[0] = *p;
        else if (N == 4) *(uint16_t*)c = *(const uint16_t*)p;
        else { *(uint32_t*)c = *(const uint32_t*)p; }
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            __half v0 = __hmul_rn(__int2half_rn((int)(c[i] >> 4) - 8), sc);
            __half v1 = __hmul_rn(__int2half_rn((int)(c[i] & 15) - 8), sc);
            if (ASYM) { v0 = __hadd_rn(v0, zp); v1 = __hadd_rn(v1, zp); }
            out[2 * i] = __half2float(v0);
            out[2 * i + 1] = __half2float(v1);
        }
    }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int FMT, bool ASYM, int D>
__global__ void __launch_bounds__(128) decode_split_generic_kernel(const AttnParams p) {
    constexpr int EPL = D / 32;          // head-dim elements per lane in the P.V phase
    constexpr int NW = 4;
    constexpr int H = kHeadsPerCta;
    const KvqAttnArgs& a = p.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, b = blockIdx.z;
    const int kvh = blockIdx.y / p.rep_chunks, rc = blockIdx.y % p.rep_chunks;
    const int h0 = kvh * p.n_rep + rc * H;
    const int nh = min(H, p.n_rep - rc * H);
    const int gs = a.group_size;

    int ctx = a.context_lens ? a.context_lens[b] : a.max_ctx;
    ctx = max(0, min(ctx, a.max_ctx) - a.tail_tokens);      // the tail belongs to the combine stage
    int s0, s1;
    split_range(ctx, p.splits, split, 32, s0, s1);

    __shared__ float q_s[H][D];
    __shared__ float red_ml[NW][H][2];
    extern __shared__ float red_acc[];   // [NW][H][D]

    const float qk_scale = a.sm_scale * kLog2e;
    for (int i = tid; i < H * D; i += 128) {
        int h = i / D, d = i % D;
        float v = 0.f;
        if (h < nh) {
            __half qv = ((const __half*)a.q)[b * a.q_stride_b + (h0 + h) * a.q_stride_h + d];
            if (a.inv_tau) qv = __hmul(qv, __float2half_rn(a.inv_tau[h0 + h]));
            if (a.q_chan_scale)
                qv = __float2half_rn(__half2float(qv) * a.q_chan_scale[b * a.qcs_stride_b + kvh * a.qcs_stride_h + d]);
            v = __half2float(qv) * qk_scale;
        }
        q_s[h][d] = v;
    }
    __syncthreads();

    const char* k_base = (const char*)a.k.payload + b * a.k.pay_stride_b + kvh * a.k.pay_stride_h;
    const char* v_base = (const char*)a.v.payload + b * a.v.pay_stride_b + kvh * a.v.pay_stride_h;
    const __half* ks_base = (const __half*)a.k.scale + b * a.k.sc_stride_b + kvh * a.k.sc_stride_h;
    const __half* vs_base = (const __half*)a.v.scale + b * a.v.sc_stride_b + kvh * a.v.sc_stride_h;
    const __half* kz_base = ASYM ? (const __half*)a.k.zp + b * a.k.sc_stride_b + kvh * a.k.sc_stride_h : nullptr;
    const __half* vz_base = ASYM ? (const __half*)a.v.zp + b * a.v.sc_stride_b + kvh * a.v.sc_stride_h : nullptr;
    const int n_out = a.n_out;
    const int16_t* oidx = n_out ? a.outlier_idx + kvh * n_out : nullptr;
    const __half* kside = n_out ? (const __half*)a.k.side + b * a.k.side_stride_b + kvh * a.k.side_stride_h : nullptr;
    const __half* vside = n_out ? (const __half*)a.v.side + b * a.v.side_stride_b + kvh * a.v.side_stride_h : nullptr;

    float m[H], l[H], acc[H][EPL];
#pragma unroll
    for (int h = 0; h < H; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[h][e] = 0.f;
    }

    for (int c = s0 + warp * 32; c < s1; c += NW * 32) {
        const int tok = c + lane;
        const bool valid = tok < s1;
        float s[H];
#pragma unroll
        for (int h = 0; h < H; ++h) s[h] = 0.f;
        if (valid) {
            const char* row = k_base + (long long)tok * a.k.pay_stride_s;
            const __half* srow = (FMT != KVQ_FMT_FP16) ? ks_base + (long long)tok * a.k.sc_stride_s : nullptr;
            const __half* zrow = ASYM ? kz_base + (long long)tok * a.k.sc_stride_s : nullptr;
            for (int d0 = 0; d0 < D; d0 += 8) {
                __half sc = __float2half(1.f), zp = __float2half(0.f);
                if (FMT != KVQ_FMT_FP16) sc = srow[d0 / gs];
                if (ASYM) zp = zrow[d0 / gs];
                float kf[8];
                load_dequant<FMT, ASYM, 8>(row, d0, sc, zp, kf);
#pragma unroll
                for (int h = 0; h < H; ++h) {
                    if (h < nh) {
                        float4 qa = *(const float4*)&q_s[h][d0];
                        float4 qb = *(const float4*)&q_s[h][d0 + 4];
                        s[h] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] +
                                qb.x * kf[4] + qb.y * kf[5] + qb.z * kf[6] + qb.w * kf[7];
                    }
                }
            }
            for (int j = 0; j < n_out; ++j) {
                int dim = oidx[j];
                float kv = __half2float(kside[(long long)tok * a.k.side_stride_s + j]);
#pragma unroll
                for (int h = 0; h < H; ++h)
                    if (h < nh) s[h] += q_s[h][dim] * kv;
            }
        }
#pragma unroll
        for (int h = 0; h < H; ++h) {
            if (h < nh) {
                float sv = valid ? s[h] : -INFINITY;
                float mx = warp_max(sv);           // finite: lane 0 of every chunk is valid
                float m_new = fmaxf(m[h], mx);
                float corr = exp2f(m[h] - m_new);  // exp2(-inf) = 0 on the first chunk
                float pj = valid ? exp2f(sv - m_new) : 0.f;
                l[h] = l[h] * corr + warp_sum(pj);
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[h][e] *= corr;
                m[h] = m_new;
                s[h] = pj;
            }
        }
        const int ntok = min(32, s1 - c);
        for (int j = 0; j < ntok; ++j) {
            const int tj = c + j;
            const char* row = v_base + (long long)tj * a.v.pay_stride_s;
            __half sc = __float2half(1.f), zp = __float2half(0.f);
            if (FMT != KVQ_FMT_FP16) sc = vs_base[(long long)tj * a.v.sc_stride_s + (lane * EPL) / gs];
            if (ASYM) zp = vz_base[(long long)tj * a.v.sc_stride_s + (lane * EPL) / gs];
            float vf[EPL];
            load_dequant<FMT, ASYM, EPL>(row, lane * EPL, sc, zp, vf);
            for (int jo = 0; jo < n_out; ++jo) {
                int dim = oidx[jo];
                if (dim / EPL == lane) {
                    float sv = __half2float(vside[(long long)tj * a.v.side_stride_s + jo]);
#pragma unroll
                    for (int e = 0; e < EPL; ++e)
                        if (e == dim % EPL) vf[e] = sv;
                }
            }
#pragma unroll
            for (int h = 0; h < H; ++h) {
                if (h < nh) {
                    float pj = __shfl_sync(0xffffffffu, s[h], j);
#pragma unroll
                    for (int e = 0; e < EPL; ++e) acc[h][e] += pj * vf[e];
                }
            }
        }
    }

    // merge the 4 warps
#pragma unroll
    for (int h = 0; h < H; ++h) {
        if (lane == 0) { red_ml[warp][h][0] = m[h]; red_ml[warp][h][1] = l[h]; }
#pragma unroll
        for (int e = 0; e < EPL; ++e) red_acc[(warp * H + h) * D + lane * EPL + e] = acc[h][e];
    }
    __syncthreads();
    for (int i = tid; i < nh * D; i += 128) {
        int h = i / D, d = i % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, red_ml[w][h][0]);
        float o = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            float mw = red_ml[w][h][0];
            float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
            o += red_acc[(w * H + h) * D + d] * wgt;
            L += red_ml[w][h][1] * wgt;
        }
        long long row = ((long long)b * a.Hq + (h0 + h)) * p.splits + split;
        p.ws_o[row * D + d] = o;
        if (d == 0) { p.ws_ml[row * 2] = M; p.ws_ml[row * 2 + 1] = L; }
    }
}

}  // namespace kvq
