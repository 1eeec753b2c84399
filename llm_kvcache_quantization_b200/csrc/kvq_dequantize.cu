// kvq_dequantize: quantized cache -> fp16 [B, Hkv, S, D] for the callers that want the
// whole cache back in floating point (get_kv / to_tuple of the cache classes, the
// non-fused "update" fallback of the HF-shaped wrapper, perplexity evaluation).
//
// Values are exactly what the fused decode kernels and the torch reference multiply:
//   symmetric   RN16(fp16(code) * scale_fp16)                 (src/engine/patch_model.py:355-362;
//               equal to the cache's own code.float() * scale -> fp16 for fp16-valued scales,
//               src/cache/int8_cache.py:536-542, src/cache/int4_cache.py get_kv)
//   asymmetric  RN16(RN16(fp16(code) * scale) + zero_point)   (src/quant/asymmetric_quant.py:193-196)
//   outlier channels: the fp16 side value replaces the (code 0) payload entry.
//
// One thread produces 8 consecutive channels of one token row: a 4-byte (packed INT4) or
// 8-byte (INT8) payload load, one scale (group sizes are multiples of 8), a 16-byte store.
// Consecutive threads cover consecutive chunks, so every access is coalesced; index arithmetic
// is 32-bit (the (side, batch, head) part of the index lives in blockIdx.y); the kernel
// is a pure HBM stream (read 0.5 - 1 B and write 2 B per element).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kvq_internal.h"

namespace kvq {

struct DequantParams {
    KvqDequantArgs a;
    int chunks;                  // D / 8
    unsigned per_row_block;      // S * chunks: work items of one (side, b, h)
    int chunk_shift;             // log2(chunks)              } when chunks and group_size are powers of two
    int group_shift;             // log2(group_size / 8)      } (POW2 instantiation: no division per chunk)
};

__device__ __forceinline__ uint32_t dq_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t dq_u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 dq_h(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Integer codes become exact fp16 numbers without the conversion unit: OR the code bits into the
// mantissa of 1024 (0x6400) and subtract the bias with one exact fp16 operation.
// two int8 codes (bytes `sel` of w, sign bits already flipped) -> half2
__device__ __forceinline__ __half2 dq_i8pair(uint32_t w_flipped, uint32_t sel) {
    return __hsub2_rn(dq_h(dq_prmt(w_flipped, 0x64646464u, sel)), dq_h(0x64806480u));          // 1152 + c - 1152
}
__device__ __forceinline__ __half2 dq_nib_lo(uint32_t w) {       // bits 0-3 of each 16-bit half
    return __hsub2_rn(dq_h((w & 0x000F000Fu) | 0x64006400u), dq_h(0x64086408u));               // 1024 + n - 1032
}
__device__ __forceinline__ __half2 dq_nib_hi(uint32_t w) {       // bits 4-7 of each 16-bit half
    return __hfma2(dq_h((w & 0x00F000F0u) | 0x64006400u), dq_h(0x2c002c00u), dq_h(0xd480d480u));   // (1024 + 16 n) / 16 - 72
}

// grid = (ceil(S * D/8 / (256 * kDqUnroll)), B * Hkv * sides); a thread converts kDqUnroll chunks of
// 8 consecutive channels, 256 chunks apart, with all of its loads issued before the first use
// (memory-level parallelism: the kernel has no reuse and little arithmetic).
constexpr int kDqUnroll = 4;

template <int FMT, bool ASYM, bool POW2>
__global__ void __launch_bounds__(256) dequantize_kernel(const DequantParams p) {
    const KvqDequantArgs& a = p.a;
    const int bh = blockIdx.y % (a.B * a.Hkv), side = blockIdx.y / (a.B * a.Hkv);
    const int b = bh / a.Hkv, h = bh - b * a.Hkv;
    const KvqCacheSide& cs = side ? a.v : a.k;
    const char* pay0 = (const char*)cs.payload + b * cs.pay_stride_b + h * cs.pay_stride_h;
    const __half* sc0 = (const __half*)cs.scale + b * cs.sc_stride_b + h * cs.sc_stride_h;
    const __half* zp0 = ASYM ? (const __half*)cs.zp + b * cs.sc_stride_b + h * cs.sc_stride_h : nullptr;
    __half* out0 = (__half*)(side ? a.v_out : a.k_out) + b * a.out_stride_b + h * a.out_stride_h;
    const unsigned base = blockIdx.x * (256u * kDqUnroll) + threadIdx.x;

    int s[kDqUnroll], c[kDqUnroll];
    bool ok[kDqUnroll];
    uint2 w[kDqUnroll];
    __half sc[kDqUnroll], zp[kDqUnroll];
#pragma unroll
    for (int u = 0; u < kDqUnroll; ++u) {
        const unsigned i = base + 256u * u;
        ok[u] = i < p.per_row_block;
        if (POW2) {
            s[u] = (int)(i >> p.chunk_shift);
            c[u] = (int)(i & (unsigned)(p.chunks - 1));
        } else {
            s[u] = (int)(i / (unsigned)p.chunks);
            c[u] = (int)(i - (unsigned)s[u] * (unsigned)p.chunks);
        }
        w[u] = make_uint2(0u, 0u);
        sc[u] = zp[u] = __half();
        if (ok[u]) {
            const char* row = pay0 + s[u] * cs.pay_stride_s;
            if (FMT == KVQ_FMT_INT8) w[u] = *(const uint2*)(row + 8 * c[u]);
            else w[u].x = *(const uint32_t*)(row + 4 * c[u]);
            const long long so = s[u] * cs.sc_stride_s + (POW2 ? (c[u] >> p.group_shift) : (8 * c[u]) / a.group_size);
            sc[u] = sc0[so];
            if (ASYM) zp[u] = zp0[so];
        }
    }
#pragma unroll
    for (int u = 0; u < kDqUnroll; ++u) {
        if (!ok[u]) continue;
        const __half2 sc2 = __half2half2(sc[u]), zp2 = __half2half2(zp[u]);
        __half2 v[4];                                     // channels (8c+0,1) (2,3) (4,5) (6,7)
        if (FMT == KVQ_FMT_INT8) {
            const uint32_t x = w[u].x ^ 0x80808080u, y = w[u].y ^ 0x80808080u;
            v[0] = dq_i8pair(x, 0x5140u); v[1] = dq_i8pair(x, 0x5342u);
            v[2] = dq_i8pair(y, 0x5140u); v[3] = dq_i8pair(y, 0x5342u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[j] = __hmul2_rn(v[j], sc2);
                if (ASYM) v[j] = __hadd2_rn(v[j], zp2);
            }
        } else {
            // byte j of the word = (channel 2j) << 4 | (channel 2j+1)
            const uint32_t x = w[u].x, x8 = x >> 8;
            __half2 t[4] = {dq_nib_hi(x), dq_nib_lo(x), dq_nib_hi(x8), dq_nib_lo(x8)};   // (0,4) (1,5) (2,6) (3,7)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                t[j] = __hmul2_rn(t[j], sc2);
                if (ASYM) t[j] = __hadd2_rn(t[j], zp2);
            }
            v[0] = dq_h(dq_prmt(dq_u(t[0]), dq_u(t[1]), 0x5410u));
            v[1] = dq_h(dq_prmt(dq_u(t[2]), dq_u(t[3]), 0x5410u));
            v[2] = dq_h(dq_prmt(dq_u(t[0]), dq_u(t[1]), 0x7632u));
            v[3] = dq_h(dq_prmt(dq_u(t[2]), dq_u(t[3]), 0x7632u));
        }
        if (a.n_out > 0) {
            const __half* sv = (const __half*)cs.side + b * cs.side_stride_b + h * cs.side_stride_h + s[u] * cs.side_stride_s;
            __half* e = reinterpret_cast<__half*>(v);
            for (int j = 0; j < a.n_out; ++j) {
                const int ch = (int)a.outlier_idx[h * a.n_out + j] - 8 * c[u];
                if (ch >= 0 && ch < 8) {
                    const __half x = sv[j];
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        if (q == ch) e[q] = x;
                }
            }
        }
        uint4 o;
        o.x = dq_u(v[0]); o.y = dq_u(v[1]); o.z = dq_u(v[2]); o.w = dq_u(v[3]);
        *(uint4*)(out0 + s[u] * a.out_stride_s + 8 * c[u]) = o;
    }
}

static bool side_ok(const KvqCacheSide& s, const KvqDequantArgs& a, bool asym) {
    if (!s.payload || !s.scale) return false;
    const int align = a.format == KVQ_FMT_INT8 ? 8 : 4;
    if (((uintptr_t)s.payload % align) || (s.pay_stride_b % align) || (s.pay_stride_h % align) || (s.pay_stride_s % align))
        return false;
    if (asym && !s.zp) return false;
    if (a.n_out > 0 && !s.side) return false;
    return true;
}

}  // namespace kvq

extern "C" int kvq_dequantize(const KvqDequantArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    const KvqDequantArgs& a = *args;
    if (a.B < 0 || a.Hkv <= 0 || a.S < 0 || a.D <= 0 || (a.D % 8) != 0) return KVQ_EINVAL;
    if (a.format != KVQ_FMT_INT8 && a.format != KVQ_FMT_INT4) return KVQ_EUNSUPPORTED;
    const int gs = a.group_size == -1 ? a.D : a.group_size;
    if (gs <= 0 || a.D % gs != 0 || gs % 8 != 0) return KVQ_EINVAL;
    if (a.B == 0 || a.S == 0) return KVQ_OK;
    if (!a.k.payload || !a.k_out) return KVQ_EINVAL;
    const bool two = a.v.payload != nullptr;
    if (two && !a.v_out) return KVQ_EINVAL;
    const bool asym = a.k.zp != nullptr || (two && a.v.zp != nullptr);
    if (a.n_out < 0 || (a.n_out > 0 && (!a.outlier_idx || asym))) return KVQ_EINVAL;
    if (!side_ok(a.k, a, asym) || (two && !side_ok(a.v, a, asym))) return KVQ_EINVAL;
    if (((uintptr_t)a.k_out & 15) || (two && ((uintptr_t)a.v_out & 15)) || (a.out_stride_b & 7) || (a.out_stride_h & 7) ||
        (a.out_stride_s & 7))
        return KVQ_EINVAL;

    if ((long long)a.S * (a.D / 8) > 0x7fffffffLL || (long long)a.B * a.Hkv * 2 > 65535) return KVQ_ELIMIT;
    DequantParams p;
    p.a = a;
    p.a.group_size = gs;
    p.chunks = a.D / 8;
    p.per_row_block = (unsigned)a.S * (unsigned)p.chunks;
    dim3 grid((p.per_row_block + 256u * kDqUnroll - 1u) / (256u * kDqUnroll), (unsigned)(a.B * a.Hkv * (two ? 2 : 1)));
    cudaStream_t st = (cudaStream_t)stream;
    auto is_pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
    auto log2i = [](int v) { int l = 0; while ((1 << l) < v) ++l; return l; };
    const bool pow2 = is_pow2(p.chunks) && is_pow2(gs / 8);
    p.chunk_shift = pow2 ? log2i(p.chunks) : 0;
    p.group_shift = pow2 ? log2i(gs / 8) : 0;
#define KVQ_DQ(F, A)                                                                  \
    if (pow2) dequantize_kernel<F, A, true><<<grid, 256, 0, st>>>(p);                 \
    else dequantize_kernel<F, A, false><<<grid, 256, 0, st>>>(p);
    if (a.format == KVQ_FMT_INT8) {
        if (asym) { KVQ_DQ(KVQ_FMT_INT8, true) } else { KVQ_DQ(KVQ_FMT_INT8, false) }
    } else {
        if (asym) { KVQ_DQ(KVQ_FMT_INT4, true) } else { KVQ_DQ(KVQ_FMT_INT4, false) }
    }
#undef KVQ_DQ
    return check_launch();
}
