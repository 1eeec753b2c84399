// KIVI-format cache: K quantized per channel (one scale / zero-point per (batch, head, channel), fixed by the
// prompt), V quantized per token (one scale / zero-point per (batch, head, token)), both asymmetric with a
// float zero-point, fp32 parameters, INT8 codes or nibble-packed INT4.
//
// Arithmetic (bit-exact with the reference's eager path, src/quant/asymmetric_quant.py:98-141, 144-196 and
// src/cache/kivi_style_cache.py:392-600):
//   rng = max(max - min, max(1e-5, 6.1035e-5 * (qmax - qmin)));  s = rng / (qmax - qmin);  zp = min - qmin * s
//   code = clamp(rint((float(x) - zp) / s), qmin, qmax)          (IEEE fp32 subtract and divide)
//   dequantised value = RN16(fp32(code * s) + zp)                 (fp32 multiply, fp32 add, one fp16 rounding)
// K statistics run over the tokens of the FIRST append of a layer; later appends reuse them (values outside
// the range clip).  V statistics run over head_dim for every token.
//
// Kernels: min/max of K per channel (chunks of tokens per CTA, ordered-integer atomics into the parameter
// buffers), a finalize step turning (min, max) into (scale, zero-point), and one quantize-and-store kernel for
// K and V (a thread owns 8 consecutive channels; the lanes of a token row combine their V statistics with
// shuffles).  Compile without fast-math.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "kvq_internal.h"

namespace kvq {

__device__ int g_kivi_error_flag = 0;   // 1: an append met a slot at or beyond max_slots


// monotone float <-> int mapping so that integer atomicMin / atomicMax order floats
__device__ __forceinline__ int f2ord(float f) {
    const int b = __float_as_int(f);
    return b >= 0 ? b : b ^ 0x7fffffff;
}
__device__ __forceinline__ float ord2f(int o) { return __int_as_float(o >= 0 ? o : o ^ 0x7fffffff); }

struct KiviParams {
    KvqKiviArgs a;
    int chunks;          // D / 8
    float qmin, qspan;
};

__global__ void kivi_stats_init_kernel(const KiviParams p) {
    const KvqKiviArgs& a = p.a;
    const long long n = (long long)a.B * a.H * a.D;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        reinterpret_cast<int*>(a.k_zp)[i] = f2ord(INFINITY);        // running minimum
        reinterpret_cast<int*>(a.k_scale)[i] = f2ord(-INFINITY);    // running maximum
    }
}

// grid = (token chunks, B * H); thread = channel (strided over D)
constexpr int kKiviStatRows = 128;
__global__ void __launch_bounds__(128) kivi_k_stats_kernel(const KiviParams p) {
    const KvqKiviArgs& a = p.a;
    const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int t0 = blockIdx.x * kKiviStatRows, t1 = min(a.T, t0 + kKiviStatRows);
    const __half* base = (const __half*)a.k_src + (long long)b * a.src_stride_b + (long long)h * a.src_stride_h;
    for (int d = threadIdx.x; d < a.D; d += blockDim.x) {
        float mn = INFINITY, mx = -INFINITY;
        for (int t = t0; t < t1; ++t) {
            const float x = __half2float(base[(long long)t * a.src_stride_t + d]);
            mn = fminf(mn, x);
            mx = fmaxf(mx, x);
        }
        const long long o = (long long)bh * a.D + d;
        atomicMin(reinterpret_cast<int*>(a.k_zp) + o, f2ord(mn));
        atomicMax(reinterpret_cast<int*>(a.k_scale) + o, f2ord(mx));
    }
}

__device__ __forceinline__ void kivi_scale_zp(float mn, float mx, float qmin, float qspan, float& s, float& zp) {
    const float floor_rng = fmaxf(1e-5f, __fmul_rn(6.103515625e-05f, qspan));
    const float rng = fmaxf(__fsub_rn(mx, mn), floor_rng);
    s = __fdiv_rn(rng, qspan);
    zp = __fsub_rn(mn, __fmul_rn(qmin, s));
}

__global__ void kivi_k_finalize_kernel(const KiviParams p) {
    const KvqKiviArgs& a = p.a;
    const long long n = (long long)a.B * a.H * a.D;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float mn = a.k_lo ? a.k_lo[i] : ord2f(reinterpret_cast<int*>(a.k_zp)[i]);
        const float mx = a.k_lo ? a.k_hi[i] : ord2f(reinterpret_cast<int*>(a.k_scale)[i]);
        float s, zp;
        kivi_scale_zp(mn, mx, p.qmin, p.qspan, s, zp);
        a.k_scale[i] = s;
        a.k_zp[i] = zp;
    }
}

__device__ __forceinline__ int kivi_code(float x, float s, float zp, float lo, float hi) {
    const float q = rintf(__fdiv_rn(__fsub_rn(x, zp), s));
    return (int)fminf(fmaxf(q, lo), hi);
}

// One thread = 8 consecutive channels of one (side, b, h, token) row.  K rows use the per-channel parameters;
// the D/8 lanes of a V row (a power of two <= 32, aligned in the warp) reduce min / max with shuffles.
template <int BITS>
__global__ void __launch_bounds__(256) kivi_quantize_kernel(const KiviParams p) {
    const KvqKiviArgs& a = p.a;
    const long long per_side = (long long)a.B * a.H * a.T * p.chunks;
    long long gid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const bool live = gid < 2 * per_side;
    if (!live) gid = 2 * per_side - 1;                 // keep the lane for the shuffles, store nothing
    const int side = gid >= per_side;
    long long r = side ? gid - per_side : gid;
    const int c = (int)(r % p.chunks); r /= p.chunks;
    const int t = (int)(r % a.T); r /= a.T;
    const int h = (int)(r % a.H);
    const int b = (int)(r / a.H);
    long long pos = (a.write_pos_dev ? (long long)(*a.write_pos_dev) : a.write_pos) + t;
    // a slot beyond the destination buffers: store nothing for this token, raise the flag, keep the lane for the shuffles
    const bool in_range = a.max_slots <= 0 || (pos >= 0 && pos < a.max_slots);
    if (!in_range) {
        if (live) g_kivi_error_flag = 1;
        pos = 0;
    }
    const __half* src = (const __half*)(side ? a.v_src : a.k_src) + (long long)b * a.src_stride_b +
                        (long long)h * a.src_stride_h + (long long)t * a.src_stride_t + 8 * c;
    const uint4 raw = *(const uint4*)src;
    const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
    float x[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { x[2 * j] = __low2float(h2[j]); x[2 * j + 1] = __high2float(h2[j]); }
    const float lo = p.qmin, hi = p.qmin + p.qspan;
    int code[8];
    if (side == 0) {
        const long long o = ((long long)b * a.H + h) * a.D + 8 * c;
        const float4 s0 = *(const float4*)(a.k_scale + o), s1 = *(const float4*)(a.k_scale + o + 4);
        const float4 z0 = *(const float4*)(a.k_zp + o), z1 = *(const float4*)(a.k_zp + o + 4);
        const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const float z[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) code[j] = kivi_code(x[j], s[j], z[j], lo, hi);
    }
    // V statistics: every lane takes part in the shuffles (K lanes contribute neutral values and ignore the result)
    float mn = INFINITY, mx = -INFINITY;
    if (side == 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { mn = fminf(mn, x[j]); mx = fmaxf(mx, x[j]); }
    }
    for (int o = 1; o < p.chunks; o <<= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (side == 1) {
        if (a.v_lo) {                                  // clipping bounds of this token instead of its minimum / maximum
            const long long o = ((long long)b * a.H + h) * a.T + t;
            mn = a.v_lo[o];
            mx = a.v_hi[o];
        }
        float s, zp;
        kivi_scale_zp(mn, mx, p.qmin, p.qspan, s, zp);
#pragma unroll
        for (int j = 0; j < 8; ++j) code[j] = kivi_code(x[j], s, zp, lo, hi);
        if (live && in_range && c == 0) {
            const long long o = (long long)b * a.vs_stride_b + (long long)h * a.vs_stride_h + pos;
            a.v_scale[o] = s;
            a.v_zp[o] = zp;
            if (a.v_scale_h) {
                ((__half*)a.v_scale_h)[o] = __float2half_rn(s);
                ((__half*)a.v_zp_h)[o] = __float2half_rn(zp);
            }
        }
    }
    if (!live || !in_range) return;
    char* row = (char*)(side ? a.v_payload : a.k_payload) + (long long)b * a.pay_stride_b + (long long)h * a.pay_stride_h +
                pos * a.pay_stride_s;
    if (BITS == 8) {
        uint2 w;
        w.x = (uint32_t)(code[0] & 0xff) | ((uint32_t)(code[1] & 0xff) << 8) | ((uint32_t)(code[2] & 0xff) << 16) |
              ((uint32_t)(code[3] & 0xff) << 24);
        w.y = (uint32_t)(code[4] & 0xff) | ((uint32_t)(code[5] & 0xff) << 8) | ((uint32_t)(code[6] & 0xff) << 16) |
              ((uint32_t)(code[7] & 0xff) << 24);
        *(uint2*)(row + 8 * c) = w;
    } else {
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            w |= (uint32_t)((((code[2 * j] + 8) & 0xf) << 4) | ((code[2 * j + 1] + 8) & 0xf)) << (8 * j);
        *(uint32_t*)(row + 4 * c) = w;
    }
}

// Cache -> fp16: K with per-channel, V with per-token fp32 parameters.  Same work decomposition.
template <int BITS>
__global__ void __launch_bounds__(256) kivi_dequantize_kernel(const KiviParams p) {
    const KvqKiviArgs& a = p.a;
    const long long per_side = (long long)a.B * a.H * a.T * p.chunks;
    const int sides = a.v_out ? 2 : 1;
    long long gid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (gid >= sides * per_side) return;
    const int side = gid >= per_side;
    long long r = side ? gid - per_side : gid;
    const int c = (int)(r % p.chunks); r /= p.chunks;
    const int t = (int)(r % a.T); r /= a.T;
    const int h = (int)(r % a.H);
    const int b = (int)(r / a.H);
    const char* row = (const char*)(side ? a.v_payload : a.k_payload) + (long long)b * a.pay_stride_b +
                      (long long)h * a.pay_stride_h + (long long)t * a.pay_stride_s;
    int code[8];
    if (BITS == 8) {
        const uint2 w = *(const uint2*)(row + 8 * c);
        const int8_t* cb = reinterpret_cast<const int8_t*>(&w);
#pragma unroll
        for (int j = 0; j < 8; ++j) code[j] = cb[j];
    } else {
        const uint32_t w = *(const uint32_t*)(row + 4 * c);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t byte = (w >> (8 * j)) & 0xffu;
            code[2 * j] = (int)(byte >> 4) - 8;
            code[2 * j + 1] = (int)(byte & 15u) - 8;
        }
    }
    float s[8], z[8];
    if (side == 0) {
        const long long o = ((long long)b * a.H + h) * a.D + 8 * c;
#pragma unroll
        for (int j = 0; j < 8; ++j) { s[j] = a.k_scale[o + j]; z[j] = a.k_zp[o + j]; }
    } else {
        const long long o = (long long)b * a.vs_stride_b + (long long)h * a.vs_stride_h + t;
        const float sv = a.v_scale[o], zv = a.v_zp[o];
#pragma unroll
        for (int j = 0; j < 8; ++j) { s[j] = sv; z[j] = zv; }
    }
    __half out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = __float2half_rn(__fadd_rn(__fmul_rn((float)code[j], s[j]), z[j]));
    __half* dst = (__half*)(side ? a.v_out : a.k_out) + (long long)b * a.out_stride_b + (long long)h * a.out_stride_h +
                  (long long)t * a.out_stride_s + 8 * c;
    *(uint4*)dst = *reinterpret_cast<const uint4*>(out);
}

static int kivi_check(const KvqKiviArgs& a, KiviParams& p) {
    if (a.bits != 4 && a.bits != 8) return KVQ_EINVAL;
    if (a.B < 0 || a.H <= 0 || a.T < 0 || a.D <= 0) return KVQ_EINVAL;
    if (a.D != 64 && a.D != 128 && a.D != 256) return KVQ_EUNSUPPORTED;     // D / 8 lanes per row: a power of two <= 32
    if (!a.k_payload || !a.v_payload || !a.k_scale || !a.k_zp || !a.v_scale || !a.v_zp) return KVQ_EINVAL;
    const int al = a.bits == 8 ? 8 : 4;
    if (((uintptr_t)a.k_payload % al) || ((uintptr_t)a.v_payload % al) || (a.pay_stride_b % al) || (a.pay_stride_h % al) ||
        (a.pay_stride_s % al))
        return KVQ_EINVAL;
    if (((uintptr_t)a.k_scale & 15) || ((uintptr_t)a.k_zp & 15)) return KVQ_EINVAL;
    p.a = a;
    p.chunks = a.D / 8;
    p.qmin = a.bits == 8 ? -128.f : -8.f;
    p.qspan = a.bits == 8 ? 255.f : 15.f;
    return KVQ_OK;
}

int kivi_error_flag(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_kivi_error_flag, sizeof(int)) != cudaSuccess) return KVQ_ECUDA;
    if (reset && v) {
        const int z = 0;
        if (cudaMemcpyToSymbol(g_kivi_error_flag, &z, sizeof(int)) != cudaSuccess) return KVQ_ECUDA;
    }
    return v;
}

// torch.quantile's linear interpolation on a sorted row: the rank in fp32, one fused multiply-add for either branch
__device__ __forceinline__ float sorted_quantile(const float* row, int n, float q) {
    const float pos = __fmul_rn(q, (float)(n - 1));
    const int lo = (int)floorf(pos);
    const int hi = min(lo + 1, n - 1);
    const float w = __fsub_rn(pos, (float)lo);
    const float x0 = row[lo], x1 = row[hi];
    const float diff = __fsub_rn(x1, x0);
    return (w < 0.5f) ? __fmaf_rn(w, diff, x0) : __fmaf_rn(__fsub_rn(w, 1.0f), diff, x1);
}

__global__ void sorted_quantile_kernel(const KvqQuantileArgs a) {
    for (long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x; r < a.rows; r += (long long)gridDim.x * blockDim.x) {
        const float* row = a.sorted + r * a.n;
        a.out_lo[r] = sorted_quantile(row, a.n, a.q_lo);
        a.out_hi[r] = sorted_quantile(row, a.n, a.q_hi);
    }
}

}  // namespace kvq

extern "C" int kvq_sorted_quantile(const KvqQuantileArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    const KvqQuantileArgs& a = *args;
    if (a.rows < 0 || a.n <= 0 || !(a.q_lo >= 0.f && a.q_lo <= 1.f) || !(a.q_hi >= 0.f && a.q_hi <= 1.f)) return KVQ_EINVAL;
    if (a.rows == 0) return KVQ_OK;
    if (!a.sorted || !a.out_lo || !a.out_hi) return KVQ_EINVAL;
    const long long blocks = (a.rows + 255) / 256;
    sorted_quantile_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, (cudaStream_t)stream>>>(a);
    return check_launch();
}

extern "C" int kvq_kivi_append(const KvqKiviArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    KiviParams p;
    int rc = kivi_check(*args, p);
    if (rc) return rc;
    const KvqKiviArgs& a = *args;
    if (a.B == 0 || a.T == 0) return KVQ_OK;
    if (!a.k_src || !a.v_src || a.write_pos < 0 || a.max_slots < 0) return KVQ_EINVAL;
    if (a.max_slots > 0 && !a.write_pos_dev && a.write_pos + a.T > a.max_slots) return KVQ_ELIMIT;
    if ((a.v_scale_h != nullptr) != (a.v_zp_h != nullptr)) return KVQ_EINVAL;
    if (((uintptr_t)a.k_src & 15) || ((uintptr_t)a.v_src & 15) || (a.src_stride_b & 7) || (a.src_stride_h & 7) ||
        (a.src_stride_t & 7))
        return KVQ_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    if ((a.k_lo != nullptr) != (a.k_hi != nullptr) || (a.v_lo != nullptr) != (a.v_hi != nullptr)) return KVQ_EINVAL;
    if (a.init_k_params) {
        const long long n = (long long)a.B * a.H * a.D;
        const unsigned g = (unsigned)((n + 255) / 256 < 1024 ? (n + 255) / 256 : 1024);
        if (!a.k_lo) {
            kivi_stats_init_kernel<<<g, 256, 0, st>>>(p);
            dim3 grid((a.T + kKiviStatRows - 1) / kKiviStatRows, a.B * a.H);
            kivi_k_stats_kernel<<<grid, 128, 0, st>>>(p);
        }
        kivi_k_finalize_kernel<<<g, 256, 0, st>>>(p);
        if ((rc = check_launch()) != 0) return rc;
    }
    const long long threads = 2LL * a.B * a.H * a.T * p.chunks;
    const long long grid = (threads + 255) / 256;
    if (grid > 0x7fffffffLL) return KVQ_ELIMIT;
    if (a.bits == 8) kivi_quantize_kernel<8><<<(unsigned)grid, 256, 0, st>>>(p);
    else kivi_quantize_kernel<4><<<(unsigned)grid, 256, 0, st>>>(p);
    return check_launch();
}

extern "C" int kvq_kivi_dequantize(const KvqKiviArgs* args, kvq_stream_t stream) {
    using namespace kvq;
    if (!args) return KVQ_EINVAL;
    KiviParams p;
    int rc = kivi_check(*args, p);
    if (rc) return rc;
    const KvqKiviArgs& a = *args;
    if (a.B == 0 || a.T == 0) return KVQ_OK;
    if (!a.k_out) return KVQ_EINVAL;
    if (((uintptr_t)a.k_out & 15) || (a.v_out && ((uintptr_t)a.v_out & 15)) || (a.out_stride_b & 7) || (a.out_stride_h & 7) ||
        (a.out_stride_s & 7))
        return KVQ_EINVAL;
    const long long threads = (a.v_out ? 2LL : 1LL) * a.B * a.H * a.T * p.chunks;
    const long long grid = (threads + 255) / 256;
    if (grid > 0x7fffffffLL) return KVQ_ELIMIT;
    cudaStream_t st = (cudaStream_t)stream;
    if (a.bits == 8) kivi_dequantize_kernel<8><<<(unsigned)grid, 256, 0, st>>>(p);
    else kivi_dequantize_kernel<4><<<(unsigned)grid, 256, 0, st>>>(p);
    return check_launch();
}
