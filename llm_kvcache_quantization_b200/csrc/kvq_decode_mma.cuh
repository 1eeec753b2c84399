// Tensor-core split-K decode-attention kernel for sm_100a: INT8 and unquantised fp16 caches.
// (The nibble-packed INT4 cache has its own kernel, kvq_decode_int4.cuh, which shares the helpers below.)
//
// Shapes: head_dim 128; INT8 payload with one fp16 scale per group of 16 / 32 / 64 / 128 channels per
// token, optional fp16 zero-points (one group per token), optional fp16 outlier side channels; or an
// unquantised fp16 cache.  <= 8 query heads per KV head per CTA.  Everything else goes to the generic kernel.
//
// Structure
//  * grid = (KV split, kv head [x head chunk], batch row); 4 warps per CTA.  Every warp
//    owns a private ring of NSTAGE shared-memory stages of TS = 32 tokens and walks
//    the stages i = warp, warp + 4, ... of the CTA's token range.  There is no
//    producer warp and no CTA-wide barrier inside the loop.
//  * Payload tiles (TS rows x 128 B or 64 B) are fetched by TMA
//    (cp.async.bulk.tensor.4d, one elected lane, completion on the stage's mbarrier)
//    with the 128 B / 64 B shared-memory swizzle, so that both the row-wise K reads
//    (ld.shared.v4) and the transposing V reads (ldmatrix.trans) are bank-conflict free.
//    Rows past the end of the cache view are zero-filled by TMA.  Per-token fp16 scales
//    (and zero-points) are fetched with 16-byte cp.async on the same mbarrier.
//  * q.K and P.V run on the tensor cores (mma.sync m16n8k16, f16 in, f32 accumulate):
//    tokens on M and the <= 8 grouped query heads on N for q.K; head_dim on M, heads
//    on N, tokens on K for P.V.  A dot product does not depend on the order of its
//    terms, so head_dim (for q.K) and the token axis (for P.V) are permuted such that
//    every thread dequantises a CONTIGUOUS slice it loaded itself:
//      q.K  thread (g = lane/4, t = lane%4) owns channels [32t, 32t+32) of token rows
//           g and g+8  -> exactly one quantisation group, one scale per row;
//      P.V  ldmatrix.trans hands thread (g, t) the bytes of tokens {2t, 2t+1} (and
//           {2t+8, 2t+9}) for a 2- or 4-channel slice, already paired per token as
//           the A fragment wants them.
//    P is rounded to fp16 and transposed across the warp with movmatrix.
//  * Dequantisation reproduces the reference bit for bit: the integer code becomes an
//    exact fp16 through the 0x6400 magic-number trick, then ONE fp16 multiply by the
//    fp16 scale (and ONE fp16 add of the zero-point), i.e. RN16(RN16(c * s) + z)
//    (src/engine/patch_model.py:355-362, src/quant/asymmetric_quant.py:193-196).
//  * Every wait on an mbarrier is bounded; on expiry the warp raises a device error flag
//    and leaves the loop, so a lost copy cannot hang the GPU.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "kvq_decode_generic.cuh"
#include "kvq_internal.h"

// Profiling builds only (build.py -DKVQ_ABLATE=bits --out ...): leave one phase of the loop out so that its share of
// the kernel time can be read from CUDA-event timings.  1: no scale / zero-point arithmetic, 2: no softmax
// (probabilities = logits), 4: no P.V product, 8: no q.K product, 16: scales and zero-points are not fetched, 32 (packed-INT4 kernel): no copies
// and no waits at all - the arithmetic alone, on whatever the slots hold, 64 (packed-INT4 kernel without outliers): the
// slot protocol (barriers, release counters) without the copies.  The results of such a build are meaningless.
#ifndef KVQ_ABLATE
#define KVQ_ABLATE 0
#endif

namespace kvq {

constexpr int kMmaWarps = 4;
constexpr int kTS = 32;              // tokens per stage (two 16-token mma tiles)
constexpr int kWaitLimit = 1 << 22;  // bounded mbarrier polling

__device__ int g_kvq_error_flag = 0;  // 1: an mbarrier wait expired

struct MmaParams {
    AttnParams p;
    int nstage;
    int warp_smem_bytes;     // nstage * bytes of one stage: the private ring of one warp
};

// Bytes of one pipeline stage: K tile, V tile (each TS rows), then 2 (4 with zero-points)
// scale tiles of TS x 8 B.  Rounded so that every payload tile stays aligned to the swizzle
// period (1024 B for 128-byte rows, 512 B for 64-byte rows).
constexpr int kMaxOut = 4;           // fp16 outlier channels per kv head the tensor-core kernel handles
__host__ __device__ constexpr int mma_stage_bytes(int fmt, bool asym, bool outl, int gs) {
    // K tile, V tile, then 2 (4 with zero-points) scale tiles of TS x (128/gs) fp16, then, with outliers,
    // K and V side tiles of TS x kMaxOut fp16 (256 B each); rounded up to the swizzle period
    // (fp16 cache: K and V tiles of TS x 256 B, each as two 128-byte-wide halves; no scales)
    if (fmt == KVQ_FMT_FP16) return 2 * kTS * 256;
    const int payload = 2 * kTS * (fmt == KVQ_FMT_INT8 ? 128 : 64);
    const int scb = kTS * (128 / gs) * 2;
    const int raw = payload + (asym ? 4 : 2) * scb + (outl ? 512 : 0);
    const int al = 1024;      // the 128-byte swizzle repeats every 1024 bytes
    return (raw + al - 1) / al * al;
}

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// try_wait that lets the hardware park the thread for up to `hint_ns` before it reports "not yet"
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void lds128(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lds64(uint32_t addr, uint32_t (&r)[2]) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
template <int LUT>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(d) : "r"(a), "r"(b), "r"(c), "n"(LUT));
    return d;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) { return h2_as_u32(__hmul2_rn(u32_as_h2(a), u32_as_h2(b))); }
__device__ __forceinline__ uint32_t hadd2_u(uint32_t a, uint32_t b) { return h2_as_u32(__hadd2_rn(u32_as_h2(a), u32_as_h2(b))); }
__device__ __forceinline__ uint32_t hsub2_u(uint32_t a, uint32_t b) { return h2_as_u32(__hsub2_rn(u32_as_h2(a), u32_as_h2(b))); }
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
    return h2_as_u32(__hfma2(u32_as_h2(a), u32_as_h2(b), u32_as_h2(c)));
}
// exp2 on the special-function unit; ex2.approx(-inf) = +0
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    return h2_as_u32(__floats2half2_rn(lo, hi));
}

// fp16 scales of the token pair (tok, tok+1), `NG` groups each, re-paired per group:
// out[G] = half2(s[tok][G], s[tok+1][G]); `addr` = shared address of s[tok][0]
template <int NG>
__device__ __forceinline__ void load_scale_pairs(uint32_t addr, uint32_t (&out)[NG], uint32_t mask) {
    if (NG == 1) {
        uint32_t w;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(addr));
        out[0] = w & mask;
    } else if (NG == 2) {
        uint32_t r[2];
        lds64(addr, r);
        out[0] = prmt(r[0], r[1], 0x5410u) & mask;
        out[NG - 1] = prmt(r[0], r[1], 0x7632u) & mask;
    } else if (NG == 4) {
        uint32_t r[4];
        lds128(addr, r);
        out[0] = prmt(r[0], r[2], 0x5410u) & mask; out[1 % NG] = prmt(r[0], r[2], 0x7632u) & mask;
        out[2 % NG] = prmt(r[1], r[3], 0x5410u) & mask; out[3 % NG] = prmt(r[1], r[3], 0x7632u) & mask;
    } else {
        uint32_t ra[4], rb[4];
        lds128(addr, ra);
        lds128(addr + 16, rb);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            out[(2 * w) % NG] = prmt(ra[w], rb[w], 0x5410u) & mask;
            out[(2 * w + 1) % NG] = prmt(ra[w], rb[w], 0x7632u) & mask;
        }
    }
}
// the NG fp16 values of one token row as floats; `addr` = shared address of s[row][0]
template <int NG>
__device__ __forceinline__ void load_row_floats(uint32_t addr, float (&f)[NG]) {
    if (NG == 1) {
        unsigned short u;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u) : "r"(addr));
        f[0] = __half2float(__ushort_as_half(u));
    } else if (NG == 2) {
        uint32_t w;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(addr));
        const float2 v = __half22float2(u32_as_h2(w));
        f[0] = v.x; f[NG - 1] = v.y;
    } else {
        uint32_t r[2];
        lds64(addr, r);
        const float2 a = __half22float2(u32_as_h2(r[0])), b = __half22float2(u32_as_h2(r[1]));
        f[0] = a.x; f[1 % NG] = a.y; f[2 % NG] = b.x; f[3 % NG] = b.y;
    }
}

// Byte offset of 16-byte chunk `c` (0..3) of token row `r` (0..31) inside a packed-INT4 payload tile.
// Narrow tile: 32 rows of 64 bytes, 64-byte swizzle.  Wide tile: the same 2 KB fetched as 16 rows of 128 bytes
// (tokens 2i, 2i+1 side by side), 128-byte swizzle - twice the bytes per copy-engine request.  In both layouts the
// eight rows of an 8x8 ldmatrix tile and the lanes of a row-wise 16-byte load fall into distinct banks.
__device__ __forceinline__ uint32_t int4_tile_off(bool wide, int r, int c) {
    return wide ? (uint32_t)((r >> 1) * 128 + (((((r & 1) << 2) | c) ^ ((r >> 1) & 7)) << 4))
                : (uint32_t)(r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
}

constexpr uint32_t kMagic = 0x64006400u;     // half2(1024, 1024)
constexpr uint32_t kH1152 = 0x64806480u;     // half2(1152, 1152)
constexpr uint32_t kH1032 = 0x64086408u;     // half2(1032, 1032)
constexpr uint32_t kHsixteenth = 0x2c002c00u;  // half2(1/16, 1/16)
constexpr uint32_t kHm72 = 0xd480d480u;      // half2(-72, -72)

// int8 pair -> exact fp16 pair.  `w` already has its sign bits flipped (w ^ 0x80808080), so
// a byte b holds code + 128 and 0x6400 | b is the fp16 number 1152 + code.
__device__ __forceinline__ uint32_t i8pair_to_h2(uint32_t w, uint32_t sel) {
    return hsub2_u(prmt(w, 0x64646464u, sel), kH1152);
}
// two nibbles (bits 0-3 of each 16-bit half) -> exact fp16 (nibble - 8)
__device__ __forceinline__ uint32_t nib_lo_to_h2(uint32_t w) {
    return hsub2_u(lop3<0xEA>(w, 0x000F000Fu, kMagic), kH1032);            // (w & m) | magic
}
// two nibbles in bits 4-7 of each half: (1024 + 16 n) / 16 - 72 = n - 8, exact in one fma
__device__ __forceinline__ uint32_t nib_hi_to_h2(uint32_t w) {
    return hfma2_u(lop3<0xEA>(w, 0x00F000F0u, kMagic), kHsixteenth, kHm72);
}
template <bool ASYM>
__device__ __forceinline__ uint32_t apply_scale(uint32_t c, uint32_t s2, uint32_t z2) {
    if (KVQ_ABLATE & 1) return c;
    uint32_t v = hmul2_u(c, s2);
    if (ASYM) v = hadd2_u(v, z2);
    return v;
}

// ---------------------------------------------------------------- the kernel
// Per-warp shared memory stage layout (bytes):
//   [0, TS*RB)            K payload tile   (TMA, swizzled)
//   [TS*RB, 2*TS*RB)      V payload tile   (TMA, swizzled)
//   then K scales [TS][4] fp16, V scales, (K zero-points, V zero-points)   256 B each
//
// GS = quantisation group size (16 / 32 / 64 / 128 channels), NG = 128 / GS scales per token.
template <int FMT, bool ASYM, bool OUTL, int GS>
__global__ void __launch_bounds__(kMmaWarps * 32, 1)
decode_split_mma_kernel(const MmaParams mp, const __grid_constant__ CUtensorMap kmap,
                        const __grid_constant__ CUtensorMap vmap) {
    constexpr bool F16 = FMT == KVQ_FMT_FP16;                 // unquantised cache: no scales, no dequantisation
    constexpr int RB = F16 ? 256 : 128;                       // payload bytes per token row
    constexpr int D = 128;
    constexpr int NG = 128 / GS;                              // scale groups per token
    constexpr int SCB = kTS * NG * 2;                         // bytes of one scale tile
    constexpr int STAGE_BYTES = mma_stage_bytes(FMT, ASYM, OUTL, GS);
    static_assert(GS == 16 || GS == 32 || GS == 64 || GS == 128, "group size");
    static_assert(FMT == KVQ_FMT_FP16 || FMT == KVQ_FMT_INT8, "packed INT4 is served by kvq_decode_int4.cuh");
    static_assert(!(ASYM && OUTL), "outlier side buffer is defined for symmetric formats");
    static_assert(!F16 || (!ASYM && !OUTL && GS == 128), "the fp16 cache has neither scales nor side channels");
    const AttnParams& p = mp.p;
    const KvqAttnArgs& a = p.a;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, b = blockIdx.z;
    const int kvh = blockIdx.y / p.rep_chunks, rc = blockIdx.y % p.rep_chunks;
    const int h0 = kvh * p.n_rep + rc * kHeadsPerCta;
    const int nh = min(kHeadsPerCta, p.n_rep - rc * kHeadsPerCta);
    const int nstage = mp.nstage;

    extern __shared__ unsigned char smem_dyn[];
    // stage buffers, 1024-byte aligned by hand: the TMA swizzle pattern is a function of the
    // shared-memory address bits, and the read side recomputes it from row indices
    unsigned char* smem_raw = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    const uint32_t wbase_u = smem_u32(smem_raw) + (uint32_t)warp * mp.warp_smem_bytes;
    __shared__ __align__(8) unsigned long long bars[kMmaWarps][8];
    __shared__ float red_ml[kMmaWarps][kHeadsPerCta][2];

    const uint32_t bar0 = smem_u32(&bars[warp][0]);
    if (lane == 0) {
        for (int s = 0; s < nstage; ++s) mbar_init(bar0 + 8 * s, 33);   // 1 expect_tx arrive + 32 cp.async arrives
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    // Nothing above touched global memory.  From here on the kernel reads q and the cache, which the
    // previous kernel in the stream (the append of the new token) may still be writing.
    pdl_wait();

    int ctx = a.context_lens ? a.context_lens[b] : a.max_ctx;
    ctx = max(0, min(ctx, a.max_ctx) - a.tail_tokens);      // the tail belongs to the combine stage
    int s0, s1;
    split_range(ctx, p.splits, split, kTS, s0, s1);

    // ---- Q fragments: thread (g = head, t) holds q[head g][32t .. 32t+32) in the channel
    // order of the K fragments.
    uint32_t qf[16];
    if (F16) {
        // natural B-fragment order: k-chunk j <-> channels 16j + {2t, 2t+1} and 16j + 8 + {2t, 2t+1}
        const bool hv = g < nh;
        const uint32_t* q32 = reinterpret_cast<const uint32_t*>(
            (const __half*)a.q + (long long)b * a.q_stride_b + (long long)(h0 + (hv ? g : 0)) * a.q_stride_h);
        const __half tau = (a.inv_tau && hv) ? __float2half_rn(a.inv_tau[h0 + g]) : __float2half(1.0f);
        const __half2 tau2 = __half2half2(tau);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t w0 = q32[8 * j + t], w1 = q32[8 * j + 4 + t];
            if (!hv) w0 = w1 = 0u;
            if (a.inv_tau) { w0 = hmul2_u(w0, h2_as_u32(tau2)); w1 = hmul2_u(w1, h2_as_u32(tau2)); }
            qf[2 * j] = w0;
            qf[2 * j + 1] = w1;
        }
    } else {
        const bool hv = g < nh;
        const __half* qp = (const __half*)a.q + (long long)b * a.q_stride_b + (long long)(h0 + (hv ? g : 0)) * a.q_stride_h +
                           32 * t;
        __half qv[32];
        const __half tau = (a.inv_tau && hv) ? __float2half_rn(a.inv_tau[h0 + g]) : __float2half(1.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 v = *(const uint4*)(qp + 8 * i);               // channels 32 t + 8 i .. + 7
            *(uint4*)(qv + 8 * i) = v;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            qv[i] = hv ? qv[i] : __float2half(0.f);
            if (a.inv_tau) qv[i] = __hmul(qv[i], tau);
        }
        if (a.q_chan_scale) {
            // per-channel factor of this kv head; element i of the slice is channel 32 t + i
            const float* cs = a.q_chan_scale + (long long)b * a.qcs_stride_b + (long long)kvh * a.qcs_stride_h;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int ch = 32 * t + i;
                qv[i] = __float2half_rn(__half2float(qv[i]) * cs[ch]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {                           // k-chunk j <-> channels 4j..4j+3
            qf[2 * j] = h2_as_u32(__halves2half2(qv[4 * j], qv[4 * j + 1]));
            qf[2 * j + 1] = h2_as_u32(__halves2half2(qv[4 * j + 2], qv[4 * j + 3]));
        }
    }

    // outlier channels: q values of heads 2t, 2t+1 at the listed channels, and fp32 side accumulators
    const int n_out = OUTL ? a.n_out : 0;
    float qo[2][kMaxOut], oo[2][kMaxOut];
    int och[kMaxOut];
    if (OUTL) {
#pragma unroll
        for (int j = 0; j < kMaxOut; ++j) {
            och[j] = (j < n_out) ? (int)a.outlier_idx[kvh * n_out + j] : 0;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int hd = 2 * t + e;
                float v = 0.f;
                if (j < n_out && hd < nh) {
                    __half qv = ((const __half*)a.q)[(long long)b * a.q_stride_b + (long long)(h0 + hd) * a.q_stride_h + och[j]];
                    if (a.inv_tau) qv = __hmul(qv, __float2half_rn(a.inv_tau[h0 + hd]));
                    v = __half2float(qv);
                }
                qo[e][j] = v;
                oo[e][j] = 0.f;
            }
        }
    }

    const float qk_scale = a.sm_scale * kLog2e;
    float m_run[2] = {-INFINITY, -INFINITY};   // running max (log2 domain) of heads 2t, 2t+1
    float l_run[2] = {0.f, 0.f};               // this thread's share of the softmax denominator
    float o[8][4];                             // O^T fragments: 8 m-blocks of 16 channels x 8 heads
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

    // ---- stage bookkeeping
    const int n_tiles_cta = (s1 - s0 + kTS - 1) / kTS;
    const int n_my = (n_tiles_cta > warp) ? (n_tiles_cta - warp + kMmaWarps - 1) / kMmaWarps : 0;
    const __half* ks_row = (const __half*)a.k.scale + (long long)b * a.k.sc_stride_b + (long long)kvh * a.k.sc_stride_h;
    const __half* vs_row = (const __half*)a.v.scale + (long long)b * a.v.sc_stride_b + (long long)kvh * a.v.sc_stride_h;
    const __half* kz_row = ASYM ? (const __half*)a.k.zp + (long long)b * a.k.sc_stride_b + (long long)kvh * a.k.sc_stride_h : nullptr;
    const __half* vz_row = ASYM ? (const __half*)a.v.zp + (long long)b * a.v.sc_stride_b + (long long)kvh * a.v.sc_stride_h : nullptr;

    const __half* kside_row = OUTL ? (const __half*)a.k.side + (long long)b * a.k.side_stride_b + (long long)kvh * a.k.side_stride_h : nullptr;
    const __half* vside_row = OUTL ? (const __half*)a.v.side + (long long)b * a.v.side_stride_b + (long long)kvh * a.v.side_stride_h : nullptr;

    auto issue = [&](int k) {
        const int st = k % nstage;
        const int tok0 = s0 + (warp + k * kMmaWarps) * kTS;
        const uint32_t sb = wbase_u + st * STAGE_BYTES;
        const uint32_t bar = bar0 + 8 * st;
        if (lane == 0) {
            mbar_expect_tx(bar, 2 * kTS * RB);
            if (F16) {   // a 256-byte row travels as two 128-byte-wide boxes (the widest swizzle span)
                tma_load_4d(sb, &kmap, bar, 0, tok0, kvh, b);
                tma_load_4d(sb + kTS * 128, &kmap, bar, 128, tok0, kvh, b);
                tma_load_4d(sb + kTS * RB, &vmap, bar, 0, tok0, kvh, b);
                tma_load_4d(sb + kTS * RB + kTS * 128, &vmap, bar, 128, tok0, kvh, b);
            } else {
                tma_load_4d(sb, &kmap, bar, 0, tok0, kvh, b);
                tma_load_4d(sb + kTS * RB, &vmap, bar, 0, tok0, kvh, b);
            }
        }
        // scale-like tiles: TS tokens x NG fp16 = 4*NG chunks of 16 bytes per tile; 2 (or 4) tiles.
        // Only bytes of tokens inside the cache view are read; the rest is zero-filled.
        if (!F16 && lane < 4 * NG && !(KVQ_ABLATE & 16)) {
            const int tok = tok0 + lane * 8 / NG;                  // first token of this 16-byte chunk
            const int nbytes = max(0, min(16, (a.max_ctx - tok) * 2 * NG));
            const long long off = nbytes ? (long long)tok * NG : 0;
            const uint32_t dst = sb + 2 * kTS * RB + lane * 16;
            cp_async16(dst, ks_row + off, nbytes);
            cp_async16(dst + SCB, vs_row + off, nbytes);
            if (ASYM) {
                cp_async16(dst + 2 * SCB, kz_row + off, nbytes);
                cp_async16(dst + 3 * SCB, vz_row + off, nbytes);
            }
        }
        if (OUTL) {
            // side tiles: TS tokens x n_out fp16, contiguous; 4*n_out 16-byte chunks per side
            const int nchunk = 4 * n_out;
            const int which = lane >= nchunk;
            const int c = lane - (which ? nchunk : 0);
            if (c < nchunk) {
                const int valid = max(0, min(kTS, a.max_ctx - tok0)) * n_out * 2;   // bytes inside the view
                const int nbytes = max(0, min(16, valid - 16 * c));
                const __half* src = (which ? vside_row : kside_row) + (nbytes ? (long long)tok0 * n_out + 8 * c : 0);
                cp_async16(sb + 2 * kTS * RB + 2 * SCB + which * 256 + 16 * c, src, nbytes);
            }
        }
        cp_async_mbar_arrive(bar);
    };

    bool failed = false;
    const int prolog = min(nstage - 1, n_my);
    for (int k = 0; k < prolog; ++k) issue(k);

    for (int k = 0; k < n_my; ++k) {
        __syncwarp();                                   // every lane has finished reading stage (k-1)
        if (k + nstage - 1 < n_my) issue(k + nstage - 1);
        const int st = k % nstage;
        const uint32_t parity = (uint32_t)((k / nstage) & 1);
        bool ok = mbar_wait_bounded(bar0 + 8 * st, parity);
        if (!__all_sync(0xffffffffu, ok)) {
            failed = true;
            break;
        }
        const int tok0 = s0 + (warp + k * kMmaWarps) * kTS;
        const bool partial = tok0 + kTS > s1;
        const uint32_t kb = wbase_u + st * STAGE_BYTES;
        const uint32_t vb = kb + kTS * RB;
        const uint32_t ksb = kb + 2 * kTS * RB;
        const uint32_t vsb = ksb + SCB;
        const uint32_t kzb = ksb + 2 * SCB;
        const uint32_t vzb = ksb + 3 * SCB;
        const uint32_t kob = ksb + 2 * SCB;                // outlier side tiles share the zero-point slots
        const uint32_t vob = kob + 256;

        // ================= q.K : logits for 2 sub-tiles of 16 tokens =================
        float sacc[2][4];
        constexpr bool NO_QK = (KVQ_ABLATE & 8) != 0, NO_PV = (KVQ_ABLATE & 4) != 0, NO_SOFTMAX = (KVQ_ABLATE & 2) != 0;
        if (NO_QK) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub)
#pragma unroll
                for (int j = 0; j < 4; ++j) sacc[sub][j] = 0.f;
        }
        if (F16 && !NO_QK) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
                for (int j = 0; j < 4; ++j) sacc[sub][j] = 0.f;
                // ldmatrix row of this lane: matrix (lane>>3): bit 0 = token half, bit 1 = second 8-channel chunk
                const int lrow = 16 * sub + ((lane >> 3) & 1) * 8 + (lane & 7);
                const uint32_t rowb = kb + lrow * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j) {                   // k-chunk j: channels 16j .. 16j+15
                    uint32_t r[4];
                    ldmatrix_x4(rowb + (j >> 2) * (kTS * 128) + (((2 * (j & 3) + (lane >> 4)) ^ (lrow & 7)) << 4), r);
                    mma16816(sacc[sub], r[0], r[1], r[2], r[3], qf[2 * j], qf[2 * j + 1]);
                }
            }
        }
#pragma unroll
        for (int sub = 0; sub < ((F16 || NO_QK) ? 0 : 2); ++sub) {
#pragma unroll
            for (int j = 0; j < 4; ++j) sacc[sub][j] = 0.f;
            const int r0 = 16 * sub + g, r1 = r0 + 8;
            // one group (= one scale) per thread per row
            // the thread's 32 channels [32t, 32t+32) lie in one group (GS >= 32) or in the two groups
            // 2t, 2t+1 (GS == 16): s2[row][half], half = which 16-channel half of the slice
            uint32_t s2[2][2], z2[2][2] = {{0u, 0u}, {0u, 0u}};
            {
                const int gidx = (32 * t) / GS;                  // first group of the slice
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int r = rr ? r1 : r0;
                    if (GS == 16) {
                        uint32_t w;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(ksb + (r * NG + gidx) * 2));
                        s2[rr][0] = prmt(w, 0u, 0x1010u);
                        s2[rr][1] = prmt(w, 0u, 0x3232u);
                        if (ASYM) {
                            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(kzb + (r * NG + gidx) * 2));
                            z2[rr][0] = prmt(w, 0u, 0x1010u);
                            z2[rr][1] = prmt(w, 0u, 0x3232u);
                        }
                    } else {
                        unsigned short u;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u) : "r"(ksb + (r * NG + gidx) * 2));
                        s2[rr][0] = s2[rr][1] = prmt((uint32_t)u, 0u, 0x1010u);
                        if (ASYM) {
                            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u) : "r"(kzb + (r * NG + gidx) * 2));
                            z2[rr][0] = z2[rr][1] = prmt((uint32_t)u, 0u, 0x1010u);
                        }
                    }
                }
            }
            uint32_t w[2][8];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int r = rr ? r1 : r0;
                uint32_t x[4], y[4];
                lds128(kb + r * 128 + (((2 * t) ^ (r & 7)) << 4), x);
                lds128(kb + r * 128 + (((2 * t + 1) ^ (r & 7)) << 4), y);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    w[rr][i] = x[i] ^ 0x80808080u;
                    w[rr][4 + i] = y[i] ^ 0x80808080u;
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int hh = j >> 2;                           // channels 4j.. lie in half j / 4 of the slice
                uint32_t a0 = apply_scale<ASYM>(i8pair_to_h2(w[0][j], 0x5140u), s2[0][hh], z2[0][hh]);
                uint32_t a1 = apply_scale<ASYM>(i8pair_to_h2(w[1][j], 0x5140u), s2[1][hh], z2[1][hh]);
                uint32_t a2 = apply_scale<ASYM>(i8pair_to_h2(w[0][j], 0x5342u), s2[0][hh], z2[0][hh]);
                uint32_t a3 = apply_scale<ASYM>(i8pair_to_h2(w[1][j], 0x5342u), s2[1][hh], z2[1][hh]);
                mma16816(sacc[sub], a0, a1, a2, a3, qf[2 * j], qf[2 * j + 1]);
            }
        }

        if (OUTL) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                const int r0 = 16 * sub + g, r1 = r0 + 8;
#pragma unroll
                for (int j = 0; j < kMaxOut; ++j) {
                    if (j < n_out) {
                        unsigned short u0, u1;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u0) : "r"(kob + (r0 * n_out + j) * 2));
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u1) : "r"(kob + (r1 * n_out + j) * 2));
                        const float k0 = __half2float(__ushort_as_half(u0)), k1 = __half2float(__ushort_as_half(u1));
                        sacc[sub][0] = fmaf(qo[0][j], k0, sacc[sub][0]);
                        sacc[sub][1] = fmaf(qo[1][j], k0, sacc[sub][1]);
                        sacc[sub][2] = fmaf(qo[0][j], k1, sacc[sub][2]);
                        sacc[sub][3] = fmaf(qo[1][j], k1, sacc[sub][3]);
                    }
                }
            }
        }

        // ================= online softmax over the 32 tokens of the stage =================
        if (partial) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                const int ta = tok0 + 16 * sub + g;
                if (ta >= s1) { sacc[sub][0] = -INFINITY; sacc[sub][1] = -INFINITY; }
                if (ta + 8 >= s1) { sacc[sub][2] = -INFINITY; sacc[sub][3] = -INFINITY; }
            }
        }
        float mx[2];
        mx[0] = fmaxf(fmaxf(sacc[0][0], sacc[0][2]), fmaxf(sacc[1][0], sacc[1][2]));
        mx[1] = fmaxf(fmaxf(sacc[0][1], sacc[0][3]), fmaxf(sacc[1][1], sacc[1][3]));
#pragma unroll
        for (int off = 4; off <= (NO_SOFTMAX ? 0 : 16); off <<= 1) {
            mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], off));
            mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], off));
        }
        float corr[2], mneg[2];
        bool changed = false;
        if (NO_SOFTMAX) { corr[0] = corr[1] = 1.f; mneg[0] = mneg[1] = 0.f; m_run[0] = m_run[1] = 0.f; }
#pragma unroll
        for (int e = 0; e < (NO_SOFTMAX ? 0 : 2); ++e) {
            const float m_new = fmaxf(m_run[e], mx[e] * qk_scale);   // finite: the stage has a valid token
            changed |= (m_new != m_run[e]);
            corr[e] = fast_exp2(m_run[e] - m_new);                       // exp2(-inf) = 0 on the first stage
            m_run[e] = m_new;
            mneg[e] = -m_new;
        }
        float psum[2] = {0.f, 0.f};
        uint32_t pb[2][2];                                           // P^T B fragments per sub-tile
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
            float p0, p1, p2, p3;
            if (NO_SOFTMAX) {
                p0 = sacc[sub][0] * 1e-4f; p1 = sacc[sub][1] * 1e-4f; p2 = sacc[sub][2] * 1e-4f; p3 = sacc[sub][3] * 1e-4f;
            } else {
                p0 = fast_exp2(fmaf(sacc[sub][0], qk_scale, mneg[0]));
                p1 = fast_exp2(fmaf(sacc[sub][1], qk_scale, mneg[1]));
                p2 = fast_exp2(fmaf(sacc[sub][2], qk_scale, mneg[0]));
                p3 = fast_exp2(fmaf(sacc[sub][3], qk_scale, mneg[1]));
            }
            psum[0] += p0 + p2;
            psum[1] += p1 + p3;
            if (OUTL) {
                const int r0 = 16 * sub + g, r1 = r0 + 8;
                const bool ok0 = !partial || tok0 + r0 < s1, ok1 = !partial || tok0 + r1 < s1;
#pragma unroll
                for (int j = 0; j < kMaxOut; ++j) {
                    if (j < n_out) {
                        unsigned short u0, u1;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u0) : "r"(vob + (r0 * n_out + j) * 2));
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u1) : "r"(vob + (r1 * n_out + j) * 2));
                        const float v0 = ok0 ? __half2float(__ushort_as_half(u0)) : 0.f;
                        const float v1 = ok1 ? __half2float(__ushort_as_half(u1)) : 0.f;
                        if (sub == 0) { oo[0][j] *= corr[0]; oo[1][j] *= corr[1]; }
                        oo[0][j] = fmaf(p0, v0, fmaf(p2, v1, oo[0][j]));
                        oo[1][j] = fmaf(p1, v0, fmaf(p3, v1, oo[1][j]));
                    }
                }
            }
            pb[sub][0] = movmatrix_trans(pack_h2(p0, p1));           // tokens 2t,2t+1   of head g
            pb[sub][1] = movmatrix_trans(pack_h2(p2, p3));           // tokens 2t+8,2t+9 of head g
        }
        l_run[0] = fmaf(l_run[0], corr[0], psum[0]);
        l_run[1] = fmaf(l_run[1], corr[1], psum[1]);
        if (__any_sync(0xffffffffu, changed)) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[1]; o[i][2] *= corr[0]; o[i][3] *= corr[1];
            }
        }

        // ================= P.V =================
        if (F16 && !NO_PV) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                uint32_t mxm = 0xffffffffu, mym = 0xffffffffu;
                if (partial) {   // rows past the range may hold anything (even NaN): zero them, P is 0 there
                    const int tg = tok0 + 16 * sub + 2 * t;
                    mxm = (tg < s1 ? 0x0000ffffu : 0u) | (tg + 1 < s1 ? 0xffff0000u : 0u);
                    mym = (tg + 8 < s1 ? 0x0000ffffu : 0u) | (tg + 9 < s1 ? 0xffff0000u : 0u);
                }
                // transposing load: matrix (lane>>3): bit 0 = second 8-channel chunk, bit 1 = token half
                const int vrow = 16 * sub + (lane >> 4) * 8 + (lane & 7);
                const uint32_t rowb = vb + vrow * 128;
#pragma unroll
                for (int i = 0; i < 8; ++i) {                   // m-block i: channels 16i .. 16i+15
                    uint32_t r[4];
                    ldmatrix_x4_trans(rowb + (i >> 2) * (kTS * 128) + (((2 * (i & 3) + ((lane >> 3) & 1)) ^ (vrow & 7)) << 4), r);
                    mma16816(o[i], r[0] & mxm, r[1] & mxm, r[2] & mym, r[3] & mym, pb[sub][0], pb[sub][1]);
                }
            }
        }
#pragma unroll
        for (int sub = 0; sub < ((F16 || NO_PV) ? 0 : 2); ++sub) {
            // scales of tokens (2t, 2t+1) and (2t+8, 2t+9), paired per group
            uint32_t sx[NG], sy[NG], zx[NG], zy[NG];
            {
                const int ta = 16 * sub + 2 * t;
                uint32_t mxm = 0xffffffffu, mym = 0xffffffffu;
                if (partial) {
                    // tokens past the range may hold anything (even NaN scales): force them to 0 * 0
                    const int tg = tok0 + ta;
                    mxm = (tg < s1 ? 0x0000ffffu : 0u) | (tg + 1 < s1 ? 0xffff0000u : 0u);
                    mym = (tg + 8 < s1 ? 0x0000ffffu : 0u) | (tg + 9 < s1 ? 0xffff0000u : 0u);
                }
                load_scale_pairs<NG>(vsb + ta * 2 * NG, sx, mxm);
                load_scale_pairs<NG>(vsb + (ta + 8) * 2 * NG, sy, mym);
                if (ASYM) {
                    load_scale_pairs<NG>(vzb + ta * 2 * NG, zx, mxm);
                    load_scale_pairs<NG>(vzb + (ta + 8) * 2 * NG, zy, mym);
                } else {
#pragma unroll
                    for (int G = 0; G < NG; ++G) zx[G] = zy[G] = 0u;
                }
            }
            // ldmatrix source row for this lane: matrix (lane>>3): bit0 = token half, bit1 = chunk + 1
            const int lrow = 16 * sub + ((lane >> 3) & 1) * 8 + (lane & 7);
            const int lchunk = lane >> 4;
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                uint32_t r[4];
                ldmatrix_x4_trans(vb + lrow * 128 + (((i + lchunk) ^ (lrow & 7)) << 4), r);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t X = r[2 * e] ^ 0x80808080u, Y = r[2 * e + 1] ^ 0x80808080u;
                    const int grp = (16 * (i + e)) / GS;             // channels 16(i+e) .. +15
                    uint32_t a0 = apply_scale<ASYM>(i8pair_to_h2(X, 0x5240u), sx[grp], zx[grp]);
                    uint32_t a1 = apply_scale<ASYM>(i8pair_to_h2(X, 0x5341u), sx[grp], zx[grp]);
                    uint32_t a2 = apply_scale<ASYM>(i8pair_to_h2(Y, 0x5240u), sy[grp], zy[grp]);
                    uint32_t a3 = apply_scale<ASYM>(i8pair_to_h2(Y, 0x5341u), sy[grp], zy[grp]);
                    mma16816(o[i + e], a0, a1, a2, a3, pb[sub][0], pb[sub][1]);
                }
            }
        }
    }
    if (failed && lane == 0) atomicExch(&g_kvq_error_flag, 1);
    pdl_launch_dependents();      // the combine kernel may be scheduled while this CTA merges its warps

    // ---- epilogue: warp totals, then merge the 4 warps through shared memory.
    // The stage buffers are reused as [warp][head][channel] fp32; all copies have landed
    // (every issued stage was waited for, unless the bounded wait expired).
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], off);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], off);
    }
    __syncthreads();
    float* red_acc = reinterpret_cast<float*>(smem_raw);          // [kMmaWarps][8][D]
    if (g == 0) {
        red_ml[warp][2 * t][0] = m_run[0]; red_ml[warp][2 * t][1] = l_run[0];
        red_ml[warp][2 * t + 1][0] = m_run[1]; red_ml[warp][2 * t + 1][1] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int d0, d1;                                               // channels of fragment rows g, g+8
        if (F16) { d0 = 16 * i + g; d1 = d0 + 8; }
        else { d0 = 16 * i + 2 * g; d1 = d0 + 1; }
        float* ra = red_acc + (size_t)warp * kHeadsPerCta * D;
        ra[(2 * t) * D + d0] = o[i][0];
        ra[(2 * t + 1) * D + d0] = o[i][1];
        ra[(2 * t) * D + d1] = o[i][2];
        ra[(2 * t + 1) * D + d1] = o[i][3];
    }
    if (OUTL) {
#pragma unroll
        for (int j = 0; j < kMaxOut; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e)
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1) oo[e][j] += __shfl_xor_sync(0xffffffffu, oo[e][j], off);
        __syncwarp();
        if (g == 0) {
            float* ra = red_acc + (size_t)warp * kHeadsPerCta * D;
#pragma unroll
            for (int j = 0; j < kMaxOut; ++j) {      // the payload holds code 0 there, so this is the whole value
                if (j < n_out) {
                    ra[(2 * t) * D + och[j]] += oo[0][j];
                    ra[(2 * t + 1) * D + och[j]] += oo[1][j];
                }
            }
        }
    }
    __syncthreads();
    // per (warp, head) merge weight, per head total: computed once, not once per channel
    __shared__ float mrg_w[kMmaWarps][kHeadsPerCta];
    __shared__ float mrg_ml[kHeadsPerCta][2];
    if (threadIdx.x < kHeadsPerCta) {
        const int h = threadIdx.x;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) M = fmaxf(M, red_ml[w][h][0]);
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) {
            const float mw = red_ml[w][h][0];
            const float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
            mrg_w[w][h] = wgt;
            L += red_ml[w][h][1] * wgt;
        }
        mrg_ml[h][0] = M;
        mrg_ml[h][1] = L;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nh * D; i += kMmaWarps * 32) {
        const int h = i / D, d = i % D;
        float ov = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) ov += red_acc[((size_t)w * kHeadsPerCta + h) * D + d] * mrg_w[w][h];
        const long long row = ((long long)b * a.Hq + (h0 + h)) * p.splits + split;
        p.ws_o[row * D + d] = ov;
        if (d == 0) { p.ws_ml[row * 2] = mrg_ml[h][0]; p.ws_ml[row * 2 + 1] = mrg_ml[h][1]; }
    }
}

}  // namespace kvq
