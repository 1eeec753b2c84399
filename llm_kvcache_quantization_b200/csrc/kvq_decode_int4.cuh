// Split-K decode-attention kernel for the nibble-packed INT4 cache on sm_100a.
//
// head_dim 128, one fp16 scale per group of 16 / 32 / 64 / 128 channels per token, optional fp16
// zero-points, optional fp16 outlier side channels (group 32), <= 8 query heads per KV head per CTA.
//
// Why a kernel of its own (the INT8 / fp16 kernel of kvq_decode_mma.cuh keeps a private ring per warp):
// a packed row is only 64 bytes, so a warp-private stage of 32 tokens is a 2 KB copy per tensor plus
// 16-byte pieces of scales.  Timed with the arithmetic compiled out, that skeleton moved 4.3 - 5.0 TB/s
// where the 128-byte-row INT8 form reaches 6 TB/s: the copy engine is paced by requests, not bytes.
// Here ONE stage serves the whole CTA:
//  * stage = 128 tokens (32 per warp): K and V payload tiles of 8 KB each, fetched as 64 rows of 128 bytes
//    (two tokens per row, 128-byte swizzle) by one cp.async.bulk.tensor each, and the fp16 scale /
//    zero-point tiles (128 tokens x G values) by one 3-D tensor copy each - 4 to 6 copies of 1 - 8 KB per
//    stage, all completing on the stage's mbarrier; rows past the view are zero-filled by the copy engine;
//  * a stage slot is refilled by whichever warp finishes reading it last (shared-memory arrival counter with
//    acquire/release), so there is no producer warp and no warp ever waits for a free slot;
//  * every mbarrier wait is bounded (device error flag, bit 0 of kvq_debug_error_flag).
//
// Arithmetic.  q.K and P.V run on mma.sync m16n8k16 with fp32 accumulation, as in the INT8 kernel.
//  FAST = true (default for groups of >= 32 channels): the scales stay OUTSIDE the integer products -
//    q.K keeps one fp32 accumulator per quantisation group over exact integer codes and combines them with
//    the fp32 values of the token's fp16 scales; the K zero-point term sum_G z[t,G] * sum_{d in G} q_d is one
//    more mma over a (hi, lo) fp16 split of the per-group query sums; P.V folds the V scale of (token, group)
//    into the fp16 probabilities, and accumulates the V zero-point term in fp32.
//    This is the arithmetic of the reference's fused kernel, which multiplies fp32 codes by fp32 scales
//    (src/kernels/triton_decode_attn_int8.py:239, 277).
//  FAST = false: every element is dequantised as RN16(RN16(code * scale) + zero_point) before the product -
//    bit for bit the fp16 values of the reference's torch path (src/engine/patch_model.py:355-362,
//    src/quant/asymmetric_quant.py:193-196).  About 1.7x the instructions; opt-in.
#pragma once

#include "kvq_decode_mma.cuh"

// resident CTAs per SM this kernel is compiled for (register cap = 65536 / (128 * this))
#ifndef KVQ_I4_MIN_CTAS
#define KVQ_I4_MIN_CTAS 4
#endif

namespace kvq {

constexpr int kI4Tok = 128;          // tokens per stage: 32 per warp
constexpr int kI4MaxStages = 4;

struct Int4Params {
    AttnParams p;
    int nstage;
    int wide_rows;           // payload maps built over 128-byte rows of two tokens
    int prefetch_stages;     // stages a CTA requests into L2 before it waits for the previous kernel (0 = none)
    int l2_ahead;            // in the loop: stages beyond the one being copied that are requested into L2 (0 = none)
};

// K tile, V tile (128 x 64 B each), 2 (4 with zero-points) tiles of 128 x G fp16, with outliers two side
// tiles of 128 x kMaxOut fp16; rounded to the swizzle period.
__host__ __device__ constexpr int int4_stage_bytes(bool asym, bool outl, int gs) {
    const int raw = 2 * kI4Tok * 64 + (asym ? 4 : 2) * kI4Tok * (128 / gs) * 2 + (outl ? 2 * kI4Tok * kMaxOut * 2 : 0);
    return (raw + 1023) / 1024 * 1024;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// Ask the memory system to bring one box of a tensor map into L2; nothing is written to shared memory and nothing
// completes on a barrier.
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ uint32_t atom_add_acq_rel_shared(uint32_t addr, uint32_t v) {
    uint32_t old;
    asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}
// d = a * b with a fresh accumulator (the zero operand costs no register)
__device__ __forceinline__ void mma16816_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t w;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(addr));
    return w;
}

template <bool ASYM, int NOUT, bool FAST, int GS>
__global__ void __launch_bounds__(kMmaWarps * 32, KVQ_I4_MIN_CTAS)
decode_split_int4_kernel(const Int4Params ip, const __grid_constant__ CUtensorMap kmap,
                         const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap ksmap,
                         const __grid_constant__ CUtensorMap vsmap, const __grid_constant__ CUtensorMap kzmap,
                         const __grid_constant__ CUtensorMap vzmap) {
    constexpr int D = 128;
    constexpr bool OUTL = NOUT > 0;                           // NOUT fp16 outlier channels per kv head (compile time)
    constexpr int NG = 128 / GS;                              // scale groups per token
    constexpr int SCB = kI4Tok * NG * 2;                      // bytes of one scale tile
    constexpr int TILE = kI4Tok * 64;                         // bytes of one payload tile
    constexpr int STAGE_BYTES = int4_stage_bytes(ASYM, OUTL, GS);
    constexpr int EPT = (NG * 2 > 8) ? 2 : 1;                 // 8-byte elements per token in the scale maps (GS 16)
    constexpr bool NO_QK = (KVQ_ABLATE & 8) != 0, NO_PV = (KVQ_ABLATE & 4) != 0, NO_SOFTMAX = (KVQ_ABLATE & 2) != 0;
    static_assert(GS == 16 || GS == 32 || GS == 64 || GS == 128, "group size");
    static_assert(!FAST || GS >= 32, "the factored path needs whole 32-channel chunks inside one group");
    static_assert(!(ASYM && OUTL), "outlier side buffer is defined for symmetric formats");
    static_assert(!OUTL || GS == 32, "outlier side buffer: groups of 32");
    const AttnParams& p = ip.p;
    const KvqAttnArgs& a = p.a;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, b = blockIdx.z;
    int kvh = blockIdx.y, rc = 0;
    if (p.rep_chunks > 1) { kvh = blockIdx.y / p.rep_chunks; rc = blockIdx.y % p.rep_chunks; }   // > 8 heads per kv head
    const int h0 = kvh * p.n_rep + rc * kHeadsPerCta;
    const int nh = min(kHeadsPerCta, p.n_rep - rc * kHeadsPerCta);
    const int nstage = ip.nstage;
    const bool wide = ip.wide_rows != 0;

    extern __shared__ unsigned char smem_dyn[];
    // 1024-byte aligned by hand: the swizzle pattern is a function of the shared-memory address bits
    unsigned char* smem_raw = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem_raw);
    __shared__ __align__(8) unsigned long long bars[kI4MaxStages];
    __shared__ uint32_t done_cnt[kI4MaxStages];                // warps that finished reading the slot, ever
    __shared__ float red_ml[kMmaWarps][kHeadsPerCta][2];


    const uint32_t bar0 = smem_u32(&bars[0]);
    const uint32_t done0 = smem_u32(&done_cnt[0]);
    if (threadIdx.x == 0) {
        // 1 arrival with the byte count by the issuing lane (+ 32 cp.async arrivals of its warp for the side tiles)
        for (int s = 0; s < nstage; ++s) { mbar_init(bar0 + 8 * s, OUTL ? 33 : 1); done_cnt[s] = 0u; }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        prefetch_tensormap(&kmap); prefetch_tensormap(&vmap); prefetch_tensormap(&ksmap); prefetch_tensormap(&vsmap);
        if (ASYM) { prefetch_tensormap(&kzmap); prefetch_tensormap(&vzmap); }
        // While the previous kernel of the stream is still running (programmatic dependent launch), start moving this
        // CTA's first stages from HBM into L2.  A prefetch consumes nothing, so it may run before the dependency is
        // resolved; the range assumes the longest context (max_ctx) - for a shorter row it fetches bytes nobody
        // reads, bounded by `prefetch_stages`.
        if (ip.prefetch_stages > 0) {
            int a0, a1;
            split_range(max(0, a.max_ctx - a.tail_tokens), p.splits, split, kI4Tok, a0, a1);
            const int n = min(ip.prefetch_stages, (a1 - a0 + kI4Tok - 1) / kI4Tok);
            for (int k = 0; k < n; ++k) {
                const int tok0 = a0 + k * kI4Tok;
                tma_prefetch_4d(&kmap, 0, wide ? (tok0 >> 1) : tok0, kvh, b);
                tma_prefetch_4d(&vmap, 0, wide ? (tok0 >> 1) : tok0, kvh, b);
                tma_prefetch_3d(&ksmap, tok0 * EPT, kvh, b);
                tma_prefetch_3d(&vsmap, tok0 * EPT, kvh, b);
                if (ASYM) { tma_prefetch_3d(&kzmap, tok0 * EPT, kvh, b); tma_prefetch_3d(&vzmap, tok0 * EPT, kvh, b); }
            }
        }
    }
    __syncthreads();

    // Nothing above touched global memory.  From here on the kernel reads q and the cache, which the
    // previous kernel in the stream may still be writing.
    pdl_wait();

    int ctx = a.context_lens ? a.context_lens[b] : a.max_ctx;
    // the query rows are requested before the first stages so that they do not queue behind those copies
    const bool hv = g < nh;
    const __half* qp = (const __half*)a.q + (long long)b * a.q_stride_b + (long long)(h0 + (hv ? g : 0)) * a.q_stride_h +
                       (FAST ? 8 * t : 32 * t);
    uint4 qraw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)   // FAST: channels 32 i + 8 t .. + 7 (8 channels of every chunk); else 32 t + 8 i .. + 7
        qraw[i] = *(const uint4*)(qp + (FAST ? 32 : 8) * i);
    const float tau_f = (a.inv_tau && hv) ? a.inv_tau[h0 + g] : 1.0f;

    ctx = max(0, min(ctx, a.max_ctx) - a.tail_tokens);      // the tail belongs to the combine stage
    int s0, s1;
    split_range(ctx, p.splits, split, kI4Tok, s0, s1);
    const int n_st = (s1 - s0 + kI4Tok - 1) / kI4Tok;         // stages of this CTA

    constexpr int n_out = NOUT;
    const __half* kside_row = OUTL ? (const __half*)a.k.side + (long long)b * a.k.side_stride_b + (long long)kvh * a.k.side_stride_h : nullptr;
    const __half* vside_row = OUTL ? (const __half*)a.v.side + (long long)b * a.v.side_stride_b + (long long)kvh * a.v.side_stride_h : nullptr;

    // Called by ALL lanes of one warp: lane 0 arms the barrier and starts the tensor copies.
    auto issue = [&](int k, int st) {        // stage k of the CTA into slot st = k mod nstage
        if (KVQ_ABLATE & 32) return;         // timing experiment: arithmetic on whatever the slots hold, no copies
        const int tok0 = s0 + k * kI4Tok;
        const uint32_t sb = sbase + st * STAGE_BYTES;
        const uint32_t bar = bar0 + 8 * st;
        if ((KVQ_ABLATE & 64) && !OUTL) {    // timing experiment: the slot protocol without the copies (barrier completes at once)
            if (lane == 0) mbar_expect_tx(bar, 0);
            return;
        }
        if (lane == 0) {
            mbar_expect_tx(bar, 2 * TILE + ((KVQ_ABLATE & 16) ? 0 : (ASYM ? 4 : 2) * SCB));
            tma_load_4d(sb, &kmap, bar, 0, wide ? (tok0 >> 1) : tok0, kvh, b);
            tma_load_4d(sb + TILE, &vmap, bar, 0, wide ? (tok0 >> 1) : tok0, kvh, b);
            if (!(KVQ_ABLATE & 16)) {
                tma_load_3d(sb + 2 * TILE, &ksmap, bar, tok0 * EPT, kvh, b);
                tma_load_3d(sb + 2 * TILE + SCB, &vsmap, bar, tok0 * EPT, kvh, b);
                if (ASYM) {
                    tma_load_3d(sb + 2 * TILE + 2 * SCB, &kzmap, bar, tok0 * EPT, kvh, b);
                    tma_load_3d(sb + 2 * TILE + 3 * SCB, &vzmap, bar, tok0 * EPT, kvh, b);
                }
            }
            // The ring is only `nstage` deep (shared memory), the way from HBM is longer than one stage of arithmetic:
            // ask for the stage `l2_ahead` further on to be brought into L2 now, so that its copy into shared memory,
            // issued when a slot frees up, is served from L2.
            if (ip.l2_ahead > 0 && k + ip.l2_ahead < n_st) {
                const int tp = tok0 + ip.l2_ahead * kI4Tok;
                tma_prefetch_4d(&kmap, 0, wide ? (tp >> 1) : tp, kvh, b);
                tma_prefetch_4d(&vmap, 0, wide ? (tp >> 1) : tp, kvh, b);
                if (!(KVQ_ABLATE & 16)) {
                    tma_prefetch_3d(&ksmap, tp * EPT, kvh, b);
                    tma_prefetch_3d(&vsmap, tp * EPT, kvh, b);
                    if (ASYM) { tma_prefetch_3d(&kzmap, tp * EPT, kvh, b); tma_prefetch_3d(&vzmap, tp * EPT, kvh, b); }
                }
            }
        }
        if (OUTL) {
            // side tiles: 128 tokens x n_out fp16, contiguous: 16 n_out chunks of 16 bytes per side; only bytes of
            // tokens inside the cache view are read, the rest is zero-filled
            const int nchunk = 16 * n_out;
            const int valid = max(0, min(kI4Tok, a.max_ctx - tok0)) * n_out * 2;
            for (int c = lane; c < 2 * nchunk; c += 32) {
                const int which = c >= nchunk;
                const int cc = c - (which ? nchunk : 0);
                const int nbytes = max(0, min(16, valid - 16 * cc));
                const __half* src = (which ? vside_row : kside_row) + (nbytes ? (long long)tok0 * n_out + 8 * cc : 0);
                cp_async16(sb + 2 * TILE + 2 * SCB + which * (kI4Tok * kMaxOut * 2) + 16 * cc, src, nbytes);
            }
            cp_async_mbar_arrive(bar);
        }
    };
    // Only the first stage is requested here; the other slots are filled when it has landed (below).  A launch of
    // this kernel is one wave of CTAs that all start together: with every CTA asking for two stages at once, half of a
    // short context's bytes queue at the memory in the first microsecond and everybody's first stage arrives late.
    if (warp == 0 && n_st > 0) issue(0, 0);               // an empty range issues nothing (its start need not even be aligned)
    pdl_launch_dependents();      // the combine kernel may take free SM resources; it waits for this grid itself

    // ---- Q fragments: thread (g = head, t) holds 32 channels of q[head g] in the channel order of the K fragments
    // (nibble order d1,d5 | d0,d4 | d3,d7 | d2,d6 inside every 8 channels).
    uint32_t qf[16];
    uint32_t zq_b0 = 0u;                 // FAST with zero-points: B fragment of the (hi, lo) split of the group sums of q
    float oz[NG][2];                     // FAST with zero-points: sum_t p * zero_point per group, heads 2t, 2t+1
#pragma unroll
    for (int G = 0; G < NG; ++G) oz[G][0] = oz[G][1] = 0.f;
    {
        uint32_t qw[16];                 // word 4 i + j = elements 8 i + 2 j, 8 i + 2 j + 1 of the slice
#pragma unroll
        for (int i = 0; i < 4; ++i) { qw[4 * i] = qraw[i].x; qw[4 * i + 1] = qraw[i].y; qw[4 * i + 2] = qraw[i].z; qw[4 * i + 3] = qraw[i].w; }
        const uint32_t tau2 = h2_as_u32(__half2half2(__float2half_rn(tau_f)));
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            qw[i] = hv ? qw[i] : 0u;
            if (a.inv_tau) qw[i] = hmul2_u(qw[i], tau2);          // RN16(q * RN16(inv_tau)) per element
        }
        if (a.q_chan_scale) {
            // per-channel factor of this kv head; element e of the slice is channel 32 (e / 8) + 8 t + e % 8 in the
            // factored layout, 32 t + e otherwise
            const float* cs = a.q_chan_scale + (long long)b * a.qcs_stride_b + (long long)kvh * a.qcs_stride_h;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int e = 2 * i;
                const int ch = FAST ? 32 * (e >> 3) + 8 * t + (e & 7) : 32 * t + e;
                const float2 f = __half22float2(u32_as_h2(qw[i]));
                qw[i] = pack_h2(f.x * cs[ch], f.y * cs[ch + 1]);
            }
        }
        if (FAST && ASYM) {
            float gsum[NG];
#pragma unroll
            for (int G = 0; G < NG; ++G) gsum[G] = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {                       // 32-channel chunk c lies in group (32 c) / GS
                float acc = 0.f;                                // this thread: 8 channels of chunk c of head g
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(u32_as_h2(qw[4 * c + j]));
                    acc += f.x + f.y;
                }
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                acc += __shfl_xor_sync(0xffffffffu, acc, 2);    // every lane of the quad: whole chunk of head g
                gsum[(32 * c) / GS] += acc;
            }
            // k slots of the zero-point mma: [hi(G = 0..NG-1), lo(G = 0..NG-1), 0 ...]; this thread supplies
            // slots 2t and 2t+1 of column (head) g
            float e0 = 0.f, e1 = 0.f;
#pragma unroll
            for (int G = 0; G < NG; ++G) {
                const float hi = __half2float(__float2half_rn(gsum[G]));
                const float lo = gsum[G] - hi;
                if (2 * t == G) e0 = hi;
                if (2 * t + 1 == G) e1 = hi;
                if (2 * t == NG + G) e0 = lo;
                if (2 * t + 1 == NG + G) e1 = lo;
            }
            zq_b0 = pack_h2(e0, e1);
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) {                           // words 4w..4w+3 <-> channels 8w..8w+7 of the slice
            qf[4 * w + 0] = prmt(qw[4 * w], qw[4 * w + 2], 0x7632u);      // (e1, e5)
            qf[4 * w + 1] = prmt(qw[4 * w], qw[4 * w + 2], 0x5410u);      // (e0, e4)
            qf[4 * w + 2] = prmt(qw[4 * w + 1], qw[4 * w + 3], 0x7632u);  // (e3, e7)
            qf[4 * w + 3] = prmt(qw[4 * w + 1], qw[4 * w + 3], 0x5410u);  // (e2, e6)
        }
    }

    // Outlier channels.  q.K: one more k-slice on the tensor cores (k slots = outlier channels, NOUT of the 16 used):
    // logits += Kside[token][j] * q[head][channel_j], A = side tile rows, B = q_out_b0 (this lane: head g, slots 2t,
    // 2t+1) - exact, fp16 products summed in fp32.  P.V: fp32 FMAs on the unrounded probabilities (side values are
    // large by construction; the fp16 rounding of P that the quantized channels tolerate would show on them).
    uint32_t q_out_b0 = 0u;
    float oo[2][NOUT > 0 ? NOUT : 1];        // heads 2t, 2t+1 x outlier j: this lane's tokens
    if (OUTL) {
        const __half* qrow = (const __half*)a.q + (long long)b * a.q_stride_b + (long long)(h0 + (hv ? g : 0)) * a.q_stride_h;
        __half e[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int j = 2 * t + x;
            __half v = __float2half(0.f);
            if (j < NOUT && hv) {
                v = qrow[a.outlier_idx[kvh * NOUT + j]];
                if (a.inv_tau) v = __hmul(v, __float2half_rn(tau_f));
            }
            e[x] = v;
        }
        q_out_b0 = h2_as_u32(__halves2half2(e[0], e[1]));
#pragma unroll
        for (int j = 0; j < NOUT; ++j) oo[0][j] = oo[1][j] = 0.f;
    }

    const float qk_scale = a.sm_scale * kLog2e;
    float m_run[2] = {-INFINITY, -INFINITY};   // reference max (log2 domain) of heads 2t, 2t+1; see the softmax below
    float l_run[2] = {0.f, 0.f};               // this thread's share of the softmax denominator
    float o[8][4];                             // O^T fragments: 8 m-blocks of 16 channels x 8 heads
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

    // Lane-dependent byte offsets inside a stage, computed once; everything else below is a compile-time offset
    // from one of them.
    //  L_ld[gp]  ldmatrix row of this lane in the warp's quarter of the K tile (V tile: + TILE; sub-tile 1: + 1024):
    //            matrix (lane >> 3): bit 0 = token half, bit 1 = second 16-byte chunk of the pair `gp`
    //  L_kr[rr]  bit-faithful q.K: 16-byte chunk t of token row g + 8 rr
    //  L_row     K scale row of token g (rows g + 8, sub-tile 1, the other tiles: constants away)
    //  L_pair    V scale rows of the token pair (2t, 2t+1)
    //  L_kz      K zero-point words of the zero-point mma (slots 2t, 2t+1 of row g)
    uint32_t L_ld[2], L_kr[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int lrow = ((lane >> 3) & 1) * 8 + (lane & 7);
        L_ld[x] = warp * (32 * 64) + int4_tile_off(wide, lrow, 2 * x + (lane >> 4));
        L_kr[x] = warp * (32 * 64) + int4_tile_off(wide, g + 8 * x, t);
    }
    const uint32_t L_row = 2 * TILE + warp * (32 * NG * 2) + g * (2 * NG);
    const uint32_t L_pair = 2 * TILE + SCB + warp * (32 * NG * 2) + (2 * t) * (2 * NG);
    const uint32_t L_kz = L_row + 2 * SCB + ((NG >= 2) ? ((2 * t) % NG) * 2 : 0);
    const uint32_t L_side = g * (NOUT * 2);                        // row g of a side tile
    constexpr int ROWB = 2 * NG;                                   // bytes of one scale row
    constexpr int SIDE = kI4Tok * kMaxOut * 2;                     // bytes of one outlier side tile

    bool failed = false;
    int st = 0;
    uint32_t parity = 0u;
    for (int k = 0; k < n_st; ++k) {
        const bool ok = (KVQ_ABLATE & 32) ? true : mbar_wait_bounded(bar0 + 8 * st, parity);
        if (!__all_sync(0xffffffffu, ok)) {
            failed = true;
            break;
        }
        if (k == 0 && warp == 0) {                              // the first stage is here: request the rest of the ring
            const int first = min(nstage, n_st);
            for (int kk = 1; kk < first; ++kk) issue(kk, kk);
        }
        const int tok0 = s0 + k * kI4Tok + warp * 32;           // first token of this warp's quarter
        const uint32_t sb = sbase + st * STAGE_BYTES;
        if (tok0 < s1 && !(KVQ_ABLATE == 30 || KVQ_ABLATE == 14)) {
        const uint32_t A_ld0 = sb + L_ld[0], A_ld1 = sb + L_ld[1];
        const uint32_t A_row = sb + L_row, A_pair = sb + L_pair;
        const uint32_t kob = sb + 2 * TILE + 2 * SCB + warp * (32 * n_out * 2);   // outlier side tiles (K; V: + SIDE)
        const int nvalid = s1 - tok0;                               // tokens of the quarter inside the range
        if (nvalid < 32) {
            // Rows past the range hold whatever the cache holds there (even NaN).  Their logits are forced to -inf
            // below, so P is exactly 0; their V scales, zero-points and side values are overwritten with zeros here so
            // that 0 * garbage cannot reach the accumulators.  One lane per row; the tile is private to this warp
            // until the slot is released.
            if (lane >= nvalid) {
                const uint32_t vrow = sb + 2 * TILE + SCB + warp * (32 * ROWB) + lane * ROWB;
#pragma unroll
                for (int j = 0; j < NG; ++j) {
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(vrow + 2 * j), "h"((unsigned short)0) : "memory");
                    if (ASYM) asm volatile("st.shared.u16 [%0], %1;" ::"r"(vrow + 2 * SCB + 2 * j), "h"((unsigned short)0) : "memory");
                }
                if (OUTL)
#pragma unroll
                    for (int j = 0; j < NOUT; ++j)
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(kob + SIDE + (lane * NOUT + j) * 2), "h"((unsigned short)0) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // ordered before the slot's next copy
            __syncwarp();
        }

        // ================= q.K : logits for 2 sub-tiles of 16 tokens =================
        float sacc[2][4];
        if (NO_QK) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub)
#pragma unroll
                for (int j = 0; j < 4; ++j) sacc[sub][j] = 0.f;
        }
        if (FAST && !NO_QK) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                float sg[NG][4];                                 // per-group integer dot products
#pragma unroll
                for (int gp = 0; gp < 2; ++gp) {
                    uint32_t r[4];                               // rows g | g+8 of chunk 2gp, then of chunk 2gp+1
                    ldmatrix_x4((gp ? A_ld1 : A_ld0) + sub * 1024, r);
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int c = 2 * gp + e;                // 32-channel chunk; its group:
                        const int G = (32 * c) / GS;
                        const uint32_t w0 = r[2 * e], w1 = r[2 * e + 1];
                        const uint32_t* qc = qf + 4 * c;
                        if ((32 * c) % GS == 0)
                            mma16816_zero(sg[G], nib_lo_to_h2(w0), nib_lo_to_h2(w1), nib_hi_to_h2(w0), nib_hi_to_h2(w1),
                                          qc[0], qc[1]);
                        else
                            mma16816(sg[G], nib_lo_to_h2(w0), nib_lo_to_h2(w1), nib_hi_to_h2(w0), nib_hi_to_h2(w1),
                                     qc[0], qc[1]);
                        const uint32_t x0 = w0 >> 8, x1 = w1 >> 8;
                        mma16816(sg[G], nib_lo_to_h2(x0), nib_lo_to_h2(x1), nib_hi_to_h2(x0), nib_hi_to_h2(x1),
                                 qc[2], qc[3]);
                    }
                }
                float sa[NG], sb2[NG];                           // K scales of rows 16 sub + g, + 8
                load_row_floats<NG>(A_row + (16 * sub) * ROWB, sa);
                load_row_floats<NG>(A_row + (16 * sub + 8) * ROWB, sb2);
                if (ASYM) {
                    // zero-point term: rows (tokens) x k slots [z_0..z_{NG-1}, z_0..z_{NG-1}, 0..] times the (hi, lo)
                    // split of the query group sums; this lane supplies slots 2t, 2t+1 of both rows
                    const uint32_t A_kz = sb + L_kz;
                    uint32_t za = 0u, zb = 0u;
                    if (NG >= 2) {
                        if (2 * t < 2 * NG) {
                            za = lds32(A_kz + (16 * sub) * ROWB);
                            zb = lds32(A_kz + (16 * sub + 8) * ROWB);
                        }
                    } else if (t == 0) {
                        unsigned short u0, u1;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u0) : "r"(A_kz + (16 * sub) * ROWB));
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u1) : "r"(A_kz + (16 * sub + 8) * ROWB));
                        za = prmt((uint32_t)u0, 0u, 0x1010u);
                        zb = prmt((uint32_t)u1, 0u, 0x1010u);
                    }
                    mma16816_zero(sacc[sub], za, zb, 0u, 0u, zq_b0, 0u);
                } else {
                    sacc[sub][0] = sacc[sub][1] = sacc[sub][2] = sacc[sub][3] = 0.f;
                }
#pragma unroll
                for (int G = 0; G < NG; ++G) {
                    sacc[sub][0] = fmaf(sa[G], sg[G][0], sacc[sub][0]);
                    sacc[sub][1] = fmaf(sa[G], sg[G][1], sacc[sub][1]);
                    sacc[sub][2] = fmaf(sb2[G], sg[G][2], sacc[sub][2]);
                    sacc[sub][3] = fmaf(sb2[G], sg[G][3], sacc[sub][3]);
                }
            }
        }
#pragma unroll
        for (int sub = 0; sub < ((FAST || NO_QK) ? 0 : 2); ++sub) {
#pragma unroll
            for (int j = 0; j < 4; ++j) sacc[sub][j] = 0.f;
            // the thread's 32 channels [32t, 32t+32) lie in one group (GS >= 32) or in the two groups
            // 2t, 2t+1 (GS == 16): s2[row][half], half = which 16-channel half of the slice
            uint32_t s2[2][2], z2[2][2] = {{0u, 0u}, {0u, 0u}};
            {
                const int gidx = (32 * t) / GS;                  // first group of the slice
                const uint32_t A_g = A_row + gidx * 2;
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int roff = (16 * sub + 8 * rr) * ROWB;
                    if (GS == 16) {
                        uint32_t w = lds32(A_g + roff);
                        s2[rr][0] = prmt(w, 0u, 0x1010u);
                        s2[rr][1] = prmt(w, 0u, 0x3232u);
                        if (ASYM) {
                            w = lds32(A_g + 2 * SCB + roff);
                            z2[rr][0] = prmt(w, 0u, 0x1010u);
                            z2[rr][1] = prmt(w, 0u, 0x3232u);
                        }
                    } else {
                        unsigned short u;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u) : "r"(A_g + roff));
                        s2[rr][0] = s2[rr][1] = prmt((uint32_t)u, 0u, 0x1010u);
                        if (ASYM) {
                            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u) : "r"(A_g + 2 * SCB + roff));
                            z2[rr][0] = z2[rr][1] = prmt((uint32_t)u, 0u, 0x1010u);
                        }
                    }
                }
            }
            uint32_t w[2][4];
            lds128(sb + L_kr[0] + sub * 1024, w[0]);
            lds128(sb + L_kr[1] + sub * 1024, w[1]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int hh = i >> 1;                           // channels 8i.. lie in half i / 2 of the slice
                uint32_t lo0 = apply_scale<ASYM>(nib_lo_to_h2(w[0][i]), s2[0][hh], z2[0][hh]);
                uint32_t lo1 = apply_scale<ASYM>(nib_lo_to_h2(w[1][i]), s2[1][hh], z2[1][hh]);
                uint32_t hi0 = apply_scale<ASYM>(nib_hi_to_h2(w[0][i]), s2[0][hh], z2[0][hh]);
                uint32_t hi1 = apply_scale<ASYM>(nib_hi_to_h2(w[1][i]), s2[1][hh], z2[1][hh]);
                mma16816(sacc[sub], lo0, lo1, hi0, hi1, qf[4 * i], qf[4 * i + 1]);
                const uint32_t w0 = w[0][i] >> 8, w1 = w[1][i] >> 8;
                lo0 = apply_scale<ASYM>(nib_lo_to_h2(w0), s2[0][hh], z2[0][hh]);
                lo1 = apply_scale<ASYM>(nib_lo_to_h2(w1), s2[1][hh], z2[1][hh]);
                hi0 = apply_scale<ASYM>(nib_hi_to_h2(w0), s2[0][hh], z2[0][hh]);
                hi1 = apply_scale<ASYM>(nib_hi_to_h2(w1), s2[1][hh], z2[1][hh]);
                mma16816(sacc[sub], lo0, lo1, hi0, hi1, qf[4 * i + 2], qf[4 * i + 3]);
            }
        }

        if (OUTL) {
            // lanes t = 0 (slots 0, 1) and t = 1 (slots 2, 3) supply the side values of rows g and g + 8
            const bool c0 = 2 * t < NOUT, c1 = 2 * t + 1 < NOUT;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                uint32_t a0 = 0u, a1 = 0u;
                if (c0) {
                    const uint32_t ad = kob + ((16 * sub) * NOUT) * 2 + L_side + 4 * t;
                    unsigned short u00, u01 = 0, u10, u11 = 0;
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u00) : "r"(ad));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u10) : "r"(ad + 8 * NOUT * 2));
                    if (c1) {
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u01) : "r"(ad + 2));
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u11) : "r"(ad + 8 * NOUT * 2 + 2));
                    }
                    a0 = (uint32_t)u00 | ((uint32_t)u01 << 16);
                    a1 = (uint32_t)u10 | ((uint32_t)u11 << 16);
                }
                mma16816(sacc[sub], a0, a1, 0u, 0u, q_out_b0, 0u);
            }
        }

        // ================= online softmax over the 32 tokens of the quarter =================
        if (nvalid < 32) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                if (16 * sub + g >= nvalid) { sacc[sub][0] = -INFINITY; sacc[sub][1] = -INFINITY; }
                if (16 * sub + g + 8 >= nvalid) { sacc[sub][2] = -INFINITY; sacc[sub][3] = -INFINITY; }
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
        // The reference max m_run only moves when a tile's max exceeds it by more than 2^kMaxLag: probabilities are
        // then at most 2^kMaxLag (exact in the fp32 sums, 11 significant bits in the fp16 product as always) and the
        // accumulators are rescaled a handful of times per CTA instead of once per tile.
        constexpr float kMaxLag = 8.f;
        if (NO_SOFTMAX) { m_run[0] = m_run[1] = 0.f; }
        const float mt0 = mx[0] * qk_scale, mt1 = mx[1] * qk_scale;           // finite: the quarter has a valid token
        if (!NO_SOFTMAX && __any_sync(0xffffffffu, mt0 > m_run[0] + kMaxLag || mt1 > m_run[1] + kMaxLag)) {
            const float n0 = fmaxf(m_run[0], mt0), n1 = fmaxf(m_run[1], mt1);
            const float c0 = fast_exp2(m_run[0] - n0), c1 = fast_exp2(m_run[1] - n1);   // exp2(-inf) = 0 the first time
            m_run[0] = n0; m_run[1] = n1;
            l_run[0] *= c0; l_run[1] *= c1;
#pragma unroll
            for (int i = 0; i < 8; ++i) { o[i][0] *= c0; o[i][1] *= c1; o[i][2] *= c0; o[i][3] *= c1; }
            if (FAST && ASYM) {
#pragma unroll
                for (int G = 0; G < NG; ++G) { oz[G][0] *= c0; oz[G][1] *= c1; }
            }
            if (OUTL) {
#pragma unroll
                for (int j = 0; j < NOUT; ++j) { oo[0][j] *= c0; oo[1][j] *= c1; }
            }
        }
        const float mneg0 = -m_run[0], mneg1 = -m_run[1];
        float pf[2][4];                                              // fp32 probabilities
        uint32_t pb[2][2];                                           // P^T B fragments per sub-tile
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
            float p0, p1, p2, p3;
            if (NO_SOFTMAX) {
                p0 = sacc[sub][0] * 1e-4f; p1 = sacc[sub][1] * 1e-4f; p2 = sacc[sub][2] * 1e-4f; p3 = sacc[sub][3] * 1e-4f;
            } else {
                p0 = fast_exp2(fmaf(sacc[sub][0], qk_scale, mneg0));
                p1 = fast_exp2(fmaf(sacc[sub][1], qk_scale, mneg1));
                p2 = fast_exp2(fmaf(sacc[sub][2], qk_scale, mneg0));
                p3 = fast_exp2(fmaf(sacc[sub][3], qk_scale, mneg1));
            }
            l_run[0] += p0 + p2;
            l_run[1] += p1 + p3;
            pf[sub][0] = p0; pf[sub][1] = p1; pf[sub][2] = p2; pf[sub][3] = p3;
            pb[sub][0] = movmatrix_trans(pack_h2(p0, p1));           // tokens 2t,2t+1   of head g
            pb[sub][1] = movmatrix_trans(pack_h2(p2, p3));           // tokens 2t+8,2t+9 of head g
            if (OUTL) {
                const uint32_t ad = kob + SIDE + ((16 * sub) * NOUT) * 2 + L_side;      // row 16 sub + g of the V side tile
#pragma unroll
                for (int j = 0; j < NOUT; ++j) {
                    unsigned short u0, u1;
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u0) : "r"(ad + 2 * j));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u1) : "r"(ad + 8 * NOUT * 2 + 2 * j));
                    const float v0 = __half2float(__ushort_as_half(u0)), v1 = __half2float(__ushort_as_half(u1));
                    oo[0][j] = fmaf(p0, v0, fmaf(p2, v1, oo[0][j]));
                    oo[1][j] = fmaf(p1, v0, fmaf(p3, v1, oo[1][j]));
                }
            }
        }

        // ================= P.V =================
        if (FAST && !NO_PV) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                // fold the V scale of (token, group) into P: B fragments per group
                uint32_t px[NG], py[NG];
                load_scale_pairs<NG>(A_pair + (16 * sub) * ROWB, px, 0xffffffffu);
                load_scale_pairs<NG>(A_pair + (16 * sub + 8) * ROWB, py, 0xffffffffu);
#pragma unroll
                for (int G = 0; G < NG; ++G) {
                    px[G] = hmul2_u(pb[sub][0], px[G]);
                    py[G] = hmul2_u(pb[sub][1], py[G]);
                }
#pragma unroll
                for (int gp = 0; gp < 2; ++gp) {
                    uint32_t r[4];
                    ldmatrix_x4_trans((gp ? A_ld1 : A_ld0) + TILE + sub * 1024, r);
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int c = 2 * gp + e;                // 32-channel chunk c, group (32 c) / GS
                        const int G = (32 * c) / GS;
                        const uint32_t X = r[2 * e], Y = r[2 * e + 1];
                        mma16816(o[2 * c], nib_lo_to_h2(X), nib_hi_to_h2(X), nib_lo_to_h2(Y), nib_hi_to_h2(Y), px[G], py[G]);
                        const uint32_t X8 = X >> 8, Y8 = Y >> 8;
                        mma16816(o[2 * c + 1], nib_lo_to_h2(X8), nib_hi_to_h2(X8), nib_lo_to_h2(Y8), nib_hi_to_h2(Y8),
                                 px[G], py[G]);
                    }
                }
                if (ASYM) {
                    float y[NG], z[NG];                          // V zero-points of rows 16 sub + g, + 8
                    load_row_floats<NG>(A_row + 3 * SCB + (16 * sub) * ROWB, y);
                    load_row_floats<NG>(A_row + 3 * SCB + (16 * sub + 8) * ROWB, z);
#pragma unroll
                    for (int G = 0; G < NG; ++G) {
                        oz[G][0] = fmaf(pf[sub][0], y[G], fmaf(pf[sub][2], z[G], oz[G][0]));
                        oz[G][1] = fmaf(pf[sub][1], y[G], fmaf(pf[sub][3], z[G], oz[G][1]));
                    }
                }
            }
        }
#pragma unroll
        for (int sub = 0; sub < ((FAST || NO_PV) ? 0 : 2); ++sub) {
            // scales of tokens (2t, 2t+1) and (2t+8, 2t+9), paired per group
            uint32_t sx[NG], sy[NG], zx[NG], zy[NG];
            load_scale_pairs<NG>(A_pair + (16 * sub) * ROWB, sx, 0xffffffffu);
            load_scale_pairs<NG>(A_pair + (16 * sub + 8) * ROWB, sy, 0xffffffffu);
            if (ASYM) {
                load_scale_pairs<NG>(A_pair + 2 * SCB + (16 * sub) * ROWB, zx, 0xffffffffu);
                load_scale_pairs<NG>(A_pair + 2 * SCB + (16 * sub + 8) * ROWB, zy, 0xffffffffu);
            } else {
#pragma unroll
                for (int G = 0; G < NG; ++G) zx[G] = zy[G] = 0u;
            }
#pragma unroll
            for (int gp = 0; gp < 2; ++gp) {
                uint32_t r[4];
                ldmatrix_x4_trans((gp ? A_ld1 : A_ld0) + TILE + sub * 1024, r);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t X = r[2 * e], Y = r[2 * e + 1];
                    const int c = 2 * gp + e;                        // 32-channel chunk; this thread's 4 channels
                    // 32c + 4g .. +3 lie in group 2c + (g >> 2) when GS == 16, else in (32 c) / GS
                    uint32_t ux, uy, vx, vy;
                    if (GS == 16) {
                        const bool up = (g >> 2) != 0;
                        ux = up ? sx[(2 * c + 1) % NG] : sx[(2 * c) % NG]; uy = up ? sy[(2 * c + 1) % NG] : sy[(2 * c) % NG];
                        vx = up ? zx[(2 * c + 1) % NG] : zx[(2 * c) % NG]; vy = up ? zy[(2 * c + 1) % NG] : zy[(2 * c) % NG];
                    } else {
                        ux = sx[(32 * c) / GS]; uy = sy[(32 * c) / GS]; vx = zx[(32 * c) / GS]; vy = zy[(32 * c) / GS];
                    }
                    uint32_t a0 = apply_scale<ASYM>(nib_lo_to_h2(X), ux, vx);
                    uint32_t a1 = apply_scale<ASYM>(nib_hi_to_h2(X), ux, vx);
                    uint32_t a2 = apply_scale<ASYM>(nib_lo_to_h2(Y), uy, vy);
                    uint32_t a3 = apply_scale<ASYM>(nib_hi_to_h2(Y), uy, vy);
                    mma16816(o[2 * c], a0, a1, a2, a3, pb[sub][0], pb[sub][1]);
                    const uint32_t X8 = X >> 8, Y8 = Y >> 8;
                    a0 = apply_scale<ASYM>(nib_lo_to_h2(X8), ux, vx);
                    a1 = apply_scale<ASYM>(nib_hi_to_h2(X8), ux, vx);
                    a2 = apply_scale<ASYM>(nib_lo_to_h2(Y8), uy, vy);
                    a3 = apply_scale<ASYM>(nib_hi_to_h2(Y8), uy, vy);
                    mma16816(o[2 * c + 1], a0, a1, a2, a3, pb[sub][0], pb[sub][1]);
                }
            }
        }
        }   // this warp's quarter holds tokens of the range

        // ---- release the slot; the warp that releases it last refills it
        __syncwarp();
        uint32_t prev = 0u;
        if (lane == 0) prev = atom_add_acq_rel_shared(done0 + 4 * st, 1u);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if ((prev & (kMmaWarps - 1)) == kMmaWarps - 1 && k + nstage < n_st) issue(k + nstage, st);
        if (++st == nstage) { st = 0; parity ^= 1u; }
    }
    if (failed && lane == 0) atomicExch(&g_kvq_error_flag, 1);

    // ---- epilogue: warp totals, then merge the 4 warps through shared memory.
    // The stage buffers are reused as [warp][head][channel] fp32; all copies have landed
    // (every issued stage was waited for by every warp, unless the bounded wait expired).
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], off);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], off);
    }
    if (FAST && ASYM) {
        // oz[G][e]: this lane's share of sum_t p * zero-point for group G, head 2t+e.  Summed over the lanes that hold
        // other tokens (same t), it belongs to every channel of the group: o[i] covers chunk i / 2 of heads 2t, 2t+1.
#pragma unroll
        for (int G = 0; G < NG; ++G)
#pragma unroll
            for (int e = 0; e < 2; ++e)
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1) oz[G][e] += __shfl_xor_sync(0xffffffffu, oz[G][e], off);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int G = (32 * (i >> 1)) / GS;
            o[i][0] += oz[G][0]; o[i][1] += oz[G][1]; o[i][2] += oz[G][0]; o[i][3] += oz[G][1];
        }
    }
    __syncthreads();
    // [warp][head][HS] fp32 over the stage buffers; HS = D + 4 keeps the 16-byte stores of a quarter-warp
    // (2 values of g x 4 values of t) in distinct banks
    constexpr int HS = D + 4;
    float* red_acc = reinterpret_cast<float*>(smem_raw);
    if (g == 0) {
        red_ml[warp][2 * t][0] = m_run[0]; red_ml[warp][2 * t][1] = l_run[0];
        red_ml[warp][2 * t + 1][0] = m_run[1]; red_ml[warp][2 * t + 1][1] = l_run[1];
    }
    float* ra = red_acc + (size_t)warp * kHeadsPerCta * HS;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        // fragment rows g, g+8 of m-blocks 2c, 2c+1 are channels 32c + 4g + {1, 0, 3, 2}
        *reinterpret_cast<float4*>(ra + (2 * t) * HS + 32 * c + 4 * g) =
            make_float4(o[2 * c][2], o[2 * c][0], o[2 * c + 1][2], o[2 * c + 1][0]);
        *reinterpret_cast<float4*>(ra + (2 * t + 1) * HS + 32 * c + 4 * g) =
            make_float4(o[2 * c][3], o[2 * c][1], o[2 * c + 1][3], o[2 * c + 1][1]);
    }
    if (OUTL) {
#pragma unroll
        for (int j = 0; j < NOUT; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e)
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1) oo[e][j] += __shfl_xor_sync(0xffffffffu, oo[e][j], off);
        __syncwarp();
        if (g == 0) {
#pragma unroll
            for (int j = 0; j < NOUT; ++j) {      // the payload holds code 0 there, so this is the whole value
                const int ch = (int)a.outlier_idx[kvh * NOUT + j];
                ra[(2 * t) * HS + ch] += oo[0][j];
                ra[(2 * t + 1) * HS + ch] += oo[1][j];
            }
        }
    }
    __syncthreads();
    // thread -> (head, 8 consecutive channels): merge the 4 warps' partials and store the CTA's partial of the split
    {
        const int h = threadIdx.x >> 4, d8 = (threadIdx.x & 15) * 8;
        float mw[kMmaWarps], lw[kMmaWarps];
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) { mw[w] = red_ml[w][h][0]; lw[w] = red_ml[w][h][1]; M = fmaxf(M, mw[w]); }
        float L = 0.f, acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) {
            const float wgt = (mw[w] == -INFINITY) ? 0.f : fast_exp2(mw[w] - M);
            L = fmaf(lw[w], wgt, L);
            const float4 x = *reinterpret_cast<const float4*>(red_acc + ((size_t)w * kHeadsPerCta + h) * HS + d8);
            const float4 y = *reinterpret_cast<const float4*>(red_acc + ((size_t)w * kHeadsPerCta + h) * HS + d8 + 4);
            acc[0] = fmaf(x.x, wgt, acc[0]); acc[1] = fmaf(x.y, wgt, acc[1]); acc[2] = fmaf(x.z, wgt, acc[2]); acc[3] = fmaf(x.w, wgt, acc[3]);
            acc[4] = fmaf(y.x, wgt, acc[4]); acc[5] = fmaf(y.y, wgt, acc[5]); acc[6] = fmaf(y.z, wgt, acc[6]); acc[7] = fmaf(y.w, wgt, acc[7]);
        }
        if (h < nh) {
            const long long row = ((long long)b * a.Hq + (h0 + h)) * p.splits + split;
            float4* dst = reinterpret_cast<float4*>(p.ws_o + row * D + d8);
            dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
            if (d8 == 0) *reinterpret_cast<float2*>(p.ws_ml + row * 2) = make_float2(M, L);
        }
    }
}

}  // namespace kvq
