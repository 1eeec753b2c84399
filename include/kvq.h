/*
 * kvq.h - C ABI of libkvq: quantize-on-append and q_len==1 fused decode
 * attention over a quantized KV cache, for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *  - every pointer is a DEVICE pointer owned by the caller unless stated;
 *  - every entry point returns 0 (KVQ_OK) or a negative KVQ_E* code, never
 *    throws, never traps; kvq_strerror() gives the text;
 *  - `stream` is a cudaStream_t passed as void*; work is enqueued, not waited for;
 *  - cache layout is the reference project's: payload [B, Hkv, S, Dp] with the
 *    last dimension contiguous (Dp = D for fp16/int8, D/2 for packed int4),
 *    scales / zero-points [B, Hkv, S, G] fp16, G = D / group_size
 *    (reference: src/cache/int8_cache.py:101-106, src/cache/int4_cache.py:651-673).
 *    All strides are given explicitly so that views into larger preallocated
 *    buffers (capacity > S) can be passed without copies.
 *
 * Each declaration cites the reference interface it stands in for
 * (paths relative to the reference project root).
 */
#ifndef KVQ_H_
#define KVQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVQ_ABI_VERSION 5

#if defined(__GNUC__)
#define KVQ_API __attribute__((visibility("default")))
#else
#define KVQ_API
#endif

/* status codes */
#define KVQ_OK            0
#define KVQ_EINVAL       -1  /* bad argument (shape, stride, alignment, NULL) */
#define KVQ_EUNSUPPORTED -2  /* valid request this build has no kernel for */
#define KVQ_ECUDA        -3  /* a CUDA runtime call failed; see kvq_last_cuda_error() */
#define KVQ_EWORKSPACE   -4  /* workspace too small */
#define KVQ_ELIMIT       -5  /* request exceeds a fixed limit of the entry point */

/* payload formats */
#define KVQ_FMT_FP16  0      /* fp16 [.., D]                                   */
#define KVQ_FMT_INT8  1      /* int8 codes [.., D] (also unpacked int4 codes)  */
#define KVQ_FMT_INT4  2      /* two codes per byte [.., D/2]:
                                byte i = ((c[2i]+8) << 4) | (c[2i+1]+8)
                                (reference: src/quant/int4_basic.py:260-272)   */

/* how the group scale is obtained when appending */
#define KVQ_SCALE_STATIC      0  /* calibrated [Hkv, G] table (+ flags below)    */
#define KVQ_SCALE_DYNAMIC_PCT 1  /* per token-group percentile of |x|            */
#define KVQ_SCALE_ASYM_MINMAX 2  /* per token-group min/max, scale + zero-point  */

/* flags for KVQ_SCALE_STATIC */
#define KVQ_F_ADAPTIVE     1  /* s = max(static*margin, absmax/qmax)  (int8_cache.py:392-402, int4_cache.py:451-455) */
#define KVQ_F_ADAPT_SKIP_K 16  /* with KVQ_F_ADAPTIVE: the K side keeps its plain static scale (adaptive_static_k=False) */
#define KVQ_F_ADAPT_SKIP_V 32  /* with KVQ_F_ADAPTIVE: the V side keeps its plain static scale (adaptive_static_v=False);
                                  the reference applies the rule to K and V independently (int8_cache.py:394, :427) */
#define KVQ_F_MIXED_RESCUE 2  /* s = max(s, absmax/7)                 (int4_cache.py:456-459)                        */
#define KVQ_F_RESCUE_THR   4  /* s = dyn >= *thr ? max(s,dyn) : s     (int4_cache.py:360-390)                        */
#define KVQ_F_UNPACKED     8  /* KVQ_FMT_INT4 only: store one code per byte ([.., D] int8 in [-8, 7]) instead of
                                 two nibbles per byte: INT4KVCache(bit_packed=False), int4_cache.py:520-560; the
                                 attention kernels read such a payload as KVQ_FMT_INT8                          */

typedef void* kvq_stream_t;

/* One side (K or V) of an append. */
typedef struct KvqAppendSide {
    const void* src;          /* fp16 new tokens [B, Hkv, T, D], D contiguous             */
    int64_t src_stride_b, src_stride_h, src_stride_t;   /* in elements                  */
    void*   payload;          /* cache payload base (token 0), see formats above          */
    int64_t pay_stride_b, pay_stride_h, pay_stride_s;   /* in BYTES                     */
    void*   scale;            /* fp16 [B,Hkv,cap,G]; NULL for KVQ_FMT_FP16                */
    void*   zp;               /* fp16 zero-points, same strides; KVQ_SCALE_ASYM_MINMAX only */
    float*  scale_f32;        /* optional fp32 copy of the scale (same strides) or NULL   */
    int64_t sc_stride_b, sc_stride_h, sc_stride_s;      /* in elements                  */
    void*   side;             /* fp16 outlier side buffer [B,Hkv,cap,n_out] or NULL       */
    int64_t side_stride_b, side_stride_h, side_stride_s; /* in elements                 */
    const void*  static_scale;      /* [Hkv, G] contiguous; KVQ_SCALE_STATIC              */
    int32_t      static_scale_is_f32; /* 0: fp16 table, 1: fp32 table                     */
    const float* rescue_threshold;  /* device scalar, KVQ_F_RESCUE_THR                    */
} KvqAppendSide;

typedef struct KvqAppendArgs {
    int32_t format;           /* KVQ_FMT_*                                                */
    int32_t policy;           /* KVQ_SCALE_*                                              */
    int32_t flags;            /* KVQ_F_*                                                  */
    int32_t B, Hkv, T, D;
    int32_t group_size;       /* divides D; 8..D                                          */
    float   adaptive_margin;
    float   quantile;         /* percentile/100 as fp32, KVQ_SCALE_DYNAMIC_PCT; >=1 means absmax */
    int32_t n_out;            /* fp16 outlier channels per KV head (0 = none)             */
    const int16_t* outlier_idx;   /* [Hkv, n_out] sorted channel indices                  */
    int64_t write_pos;        /* first cache slot to write                                */
    const int32_t* write_pos_dev; /* if not NULL the slot is read on the device instead   */
    int64_t max_slots;        /* token slots of the destination buffers (their capacity).  > 0: a host
                                 write_pos with write_pos + T > max_slots is refused (KVQ_ELIMIT); with a
                                 device-side position the kernel stores nothing for a token whose slot is
                                 >= max_slots and raises bit 1 of kvq_debug_error_flag.  0: unchecked    */
    KvqAppendSide k, v;
    /* Optional rotary embedding fused in front of the quantizer (rope_cos == NULL: off).  K is rotated
     * before it is quantized, V is not; with q_src the query rows are rotated by the same launch and
     * written to q_out (the attention kernel's q).  Rotate-half convention with fp16 arithmetic rounded
     * per operation, RN16(RN16(x cos) + RN16(rot(x) sin)), as _apply_rope does
     * (src/engine/patch_model.py:223-278); channels >= rotary_dim pass through. */
    const void* rope_cos;     /* fp16 [B or 1, T, rotary_dim]                             */
    const void* rope_sin;
    int64_t rope_stride_b, rope_stride_t;               /* elements; stride_b 0 = shared by the batch */
    int32_t rotary_dim;       /* even, <= D                                               */
    int32_t Hq;               /* query heads in q_src                                     */
    const void* q_src;        /* fp16 [B, Hq, T, D] before rotation, or NULL              */
    int64_t q_stride_b, q_stride_h, q_stride_t;         /* elements                      */
    void*   q_out;            /* fp16 [B, Hq, T, D] after rotation                        */
    int64_t qo_stride_b, qo_stride_h, qo_stride_t;      /* elements                      */
} KvqAppendArgs;

/*
 * Quantize T new tokens of K and V and write payload, scales (zero-points,
 * outlier side buffer) at cache slots [write_pos, write_pos + T): ONE launch for
 * both tensors (v.src == NULL quantizes the K side only).
 * Stands in for INT8KVCache.append / INT4KVCache.append / FP16KVCache.append
 * (src/cache/int8_cache.py:350-488, src/cache/int4_cache.py:392-589,
 *  src/cache/fp16_cache.py) and the quantizers they call
 * (src/quant/int8_basic.py:18-164, src/quant/int4_basic.py:24-159, :230-272,
 *  src/quant/asymmetric_quant.py:24-141 applied group-wise).
 * Codes, packed bytes and fp16 scales are bit-identical to those functions.
 */
KVQ_API int kvq_quantize_append(const KvqAppendArgs* args, kvq_stream_t stream);

/* One side (K or V) of the cache as the attention kernel reads it. */
typedef struct KvqCacheSide {
    const void* payload;
    int64_t pay_stride_b, pay_stride_h, pay_stride_s;   /* BYTES                         */
    const void* scale;        /* fp16; strides may be 0 to broadcast a static table       */
    const void* zp;           /* fp16 or NULL                                             */
    int64_t sc_stride_b, sc_stride_h, sc_stride_s;      /* elements                      */
    const void* side;         /* fp16 outlier values [B,Hkv,S,n_out] or NULL              */
    int64_t side_stride_b, side_stride_h, side_stride_s; /* elements                     */
} KvqCacheSide;

typedef struct KvqAttnArgs {
    int32_t format;           /* KVQ_FMT_*                                                */
    int32_t B, Hq, Hkv, D;
    int32_t group_size;
    int32_t max_ctx;          /* upper bound of context_lens (the S extent of the views)  */
    const void* q;            /* fp16 [B, Hq, D], D contiguous                            */
    int64_t q_stride_b, q_stride_h;                     /* elements                      */
    const float* inv_tau;     /* fp32 [Hq] or NULL: q <- RN16(q * RN16(inv_tau[h]))       */
    float   sm_scale;
    KvqCacheSide k, v;
    int32_t n_out;
    const int16_t* outlier_idx;  /* [Hkv, n_out]                                          */
    const int32_t* context_lens; /* int32 [B], clamped to [0, max_ctx]; NULL = every row has max_ctx tokens */
    int32_t splits;           /* KV splits per (batch, kv head); 0 = library heuristic    */
    int32_t stages;           /* 0 = split kernel + combine; 1 = split kernel only; 2 = combine only
                                 (for profiling one stage; the workspace carries the partials) */
    int32_t fast_dequant;     /* packed INT4 with groups of >= 32 channels on the tensor-core kernel; ignored elsewhere.
                                 0: library default = 1 (KVQ_INT4_EXACT=1 in the environment makes it 2).
                                 1: factored scales - integer code products per group, scales applied outside, fp32
                                    accumulation: the arithmetic of the reference's fused kernel, which multiplies fp32
                                    codes by fp32 scales (src/kernels/triton_decode_attn_int8.py:239, 277).
                                 2: bit-faithful - every element is RN16(RN16(code * scale) + zero_point) before the
                                    product, the fp16 values of the reference's torch path
                                    (src/engine/patch_model.py:355-362); about 1.6x the instructions.
                                 Both meet |a-b| <= 2e-3 + 1e-2 |b| against the torch path on the benchmark
                                 configurations; they differ from each other by the fp16 granularity of code * scale
                                 (2^-11 of its magnitude per unit of probability), which shows only on data whose
                                 dequantised magnitudes reach the tens (unquantised outlier channels).             */
    int32_t tail_tokens;      /* 0 or 1.  1: the LAST token of every row's context is not read by the split
                                 kernel (stage 1) but by the combine (stage 2), straight from the cache.  The
                                 split kernel then does not depend on the kernel that appends that token: a
                                 caller may run stage 1 and kvq_quantize_append concurrently (two streams) and
                                 stage 2 after both.  Same result up to summation order.                       */
    void*   workspace;        /* >= kvq_decode_workspace_bytes(...)                       */
    size_t  workspace_bytes;
    void*   out;              /* fp16 [B, Hq, D] or NULL                                  */
    int64_t out_stride_b, out_stride_h;                 /* elements                      */
    /* optional normalised partial for a cross-GPU merge (all three or none):            */
    const float* q_chan_scale; /* fp32 [B, Hkv, D] or NULL: q[b, h, d] <- RN16(q[b, h, d] * q_chan_scale[b, h / n_rep, d])
                                  after inv_tau - a per-channel K scale carried by the query (KIVI-format caches,
                                  whose K tiles then hold scale 1)                                                  */
    int64_t qcs_stride_b, qcs_stride_h;                 /* elements                      */
    float*  part_o;           /* fp32 [B, Hq, D]  o = sum p v / l                         */
    float*  part_m;           /* fp32 [B, Hq]     running max of scaled logits (-inf if empty) */
    float*  part_l;           /* fp32 [B, Hq]     sum exp(logit - m)  (0 if empty)        */
    int64_t part_o_stride;    /* elements between consecutive (b, h) rows of part_o; 0 = D        */
    int64_t part_ml_stride;   /* elements between consecutive (b, h) entries of part_m / part_l; 0 = 1
                                 (lets o, m, l share one packed [B, Hq, D+2] send buffer)          */
} KvqAttnArgs;

/*
 * out[b,h,:] = softmax(sm_scale * q[b,h] . Khat[b, h / n_rep, :ctx_b]^T) Vhat,
 * Khat = RN16(fp16(code) * scale) (+ zero-point, outlier side values), split-K
 * flash-decoding over the KV axis followed by a log-sum-exp combine.
 * Rows with context 0 give zeros (never NaN).
 * Stands in for decode_attn_int8 / decode_attn_int4
 * (src/kernels/triton_decode_attn_int8.py:306-519,
 *  src/kernels/triton_decode_attn_int4.py:62-121) and matches
 * _decode_attn_int8_torch_ref (src/engine/patch_model.py:281-377) within
 * |a-b| <= 2e-3 + 1e-2 |b|.
 */
KVQ_API int kvq_decode_attn(const KvqAttnArgs* args, kvq_stream_t stream);

/*
 * kvq_decode_attn for callers that cannot allocate device memory.  (No counterpart in the
 * reference: its Triton wrapper allocates freely through torch.)
 *
 * Who needs it: a host that has handed all of HBM to its own pool and must not call cudaMalloc
 * any more, or one that calls this library from a place where no allocator may run.  Such a
 * caller has nowhere to get the split-K scratch buffer from, so this variant keeps the partials
 * in a fixed KVQ_STATIC_WORKSPACE_BYTES array that is part of the library image (every GPU that
 * loads the library holds that much until the process exits).
 *
 * Same arguments and result as kvq_decode_attn; `workspace` / `workspace_bytes` are ignored.
 * It calls no cudaMalloc, cudaFree or other allocating routine.
 *  - Limit: B * Hq * splits * (D + 2) * 4 bytes must fit the array.  With `splits == 0` the
 *    library lowers its own split choice until it fits; if even one split does not fit, or an
 *    explicit `splits` is too large, the call returns KVQ_ELIMIT and launches nothing.
 *    On a 148-SM part the library's own choice stays near 3 MB (<= 8 heads x resident CTAs x 520 bytes), so the
 *    lowering is a guard for other parts; KVQ_STATIC_WS_LIMIT=<bytes> in the environment (read once) makes the
 *    entry point use less of the array.
 *  - The first call on each device looks up the array's device address (with that device
 *    current) and caches it; make that first call outside any stream capture.  First calls from several
 *    host threads at once are fine (they resolve and cache the same address).
 *  - All calls on a device share the one array and it keeps the previous call's partials.
 *    Nothing in it has to start at zero (every slot a call reads it has written first), but two
 *    calls that overlap on the GPU - different streams, or graphs replayed concurrently - race
 *    on it.  Serialise them on one stream.
 */
#define KVQ_STATIC_WORKSPACE_BYTES (8u << 20)
KVQ_API int kvq_decode_attn_static(const KvqAttnArgs* args, kvq_stream_t stream);

/* Host-side query, no launch: 1 if kvq_decode_attn would take the tensor-core TMA kernel for these
 * arguments (head_dim 128, group 16/32/64/128, int8 / packed int4, 16-byte aligned rows), 0 for the generic kernel. */
KVQ_API int kvq_decode_kernel_kind(const KvqAttnArgs* args);

KVQ_API size_t kvq_decode_workspace_bytes(int32_t B, int32_t Hq, int32_t D, int32_t splits);
/* Split count the library would choose for these arguments on the current device (host-side query,
 * no launch): the count that minimises waves x (tokens per split rounded to 128, plus a fixed
 * per-CTA cost of 128 tokens), where a wave is the resident CTAs per SM of the kernel that would
 * run times the SM count. */
KVQ_API int32_t kvq_decode_pick_splits(const KvqAttnArgs* args);

typedef struct KvqCombineArgs {
    int32_t P, B, Hq, D;      /* P partials (e.g. one per GPU)                            */
    const float* part_o;      /* fp32 [P, B, Hq, D] normalised partial outputs            */
    const float* part_m;      /* fp32 [P, B, Hq]                                          */
    const float* part_l;      /* fp32 [P, B, Hq]                                          */
    void*   out;              /* fp16 [B, Hq, D]                                          */
    int64_t out_stride_b, out_stride_h;
    int64_t part_o_stride;    /* elements between (b, h) rows of part_o; 0 = D                    */
    int64_t part_ml_stride;   /* elements between (b, h) entries of part_m / part_l; 0 = 1        */
    int64_t part_o_stride_p;  /* elements between partials p of part_o; 0 = B*Hq*part_o_stride    */
    int64_t part_ml_stride_p; /* elements between partials p of part_m / part_l; 0 = B*Hq*part_ml_stride */
} KvqCombineArgs;

/*
 * Merge P normalised partials: M = max m_p,
 * out = sum_p o_p l_p e^(m_p - M) / sum_p l_p e^(m_p - M); all-empty rows give 0.
 * No counterpart in the reference (it has no sequence sharding); the math is the
 * online-softmax merge of src/kernels/triton_decode_attn_int8.py:247-283.
 */
KVQ_API int kvq_lse_combine(const KvqCombineArgs* args, kvq_stream_t stream);

/*
 * KIVI-format cache (src/cache/kivi_style_cache.py): K asymmetric per channel with parameters fixed by the
 * first append of a layer, V asymmetric per token; fp32 scale and float zero-point; INT8 codes or
 * nibble-packed INT4.  kvq_kivi_append stands in for KIVIStyleKVCache.append (:296-600) with
 * quantize_asymmetric_per_channel / _per_token (src/quant/asymmetric_quant.py:199-289) at percentile 100;
 * kvq_kivi_dequantize for get_kv (:602-650) with dequantize_asymmetric (:144-196).  Bit-exact codes,
 * parameters and dequantised values.  In kvq_kivi_dequantize, T is the number of cached tokens to convert.
 */
typedef struct KvqKiviArgs {
    int32_t bits;                /* 4 (packed, payload [.., D/2]) or 8 (payload [.., D])      */
    int32_t B, H, T, D;          /* D in {64, 128, 256}                                       */
    int32_t init_k_params;       /* append: 1 = compute k_scale / k_zp from these T tokens    */
    const void* k_src;           /* fp16 [B, H, T, D] new tokens (append)                     */
    const void* v_src;
    int64_t src_stride_b, src_stride_h, src_stride_t;   /* elements, multiples of 8      */
    void* k_payload;             /* int8 cache [B, H, cap, D or D/2]                          */
    void* v_payload;
    int64_t pay_stride_b, pay_stride_h, pay_stride_s;   /* BYTES                         */
    float* k_scale;              /* fp32 [B, H, D] contiguous, 16-byte aligned                */
    float* k_zp;
    float* v_scale;              /* fp32 [B, H, cap], token-contiguous                        */
    float* v_zp;
    int64_t vs_stride_b, vs_stride_h;                   /* elements                      */
    int64_t write_pos;           /* append: first slot written                                */
    const int32_t* write_pos_dev;/* if not NULL the slot is read on the device                */
    int64_t max_slots;           /* append: capacity of the destination buffers in tokens; same rule as
                                    KvqAppendArgs.max_slots (bit 2 of kvq_debug_error_flag); 0: unchecked */
    void* k_out;                 /* dequantize: fp16 [B, H, T, D]                             */
    void* v_out;                 /* or NULL                                                   */
    int64_t out_stride_b, out_stride_h, out_stride_s;   /* elements, multiples of 8      */
    void* v_scale_h;             /* append, optional: fp16 copies RN16(v_scale), RN16(v_zp), laid out like the fp32  */
    void* v_zp_h;                /* buffers - the per-token tiles the fused decode kernel reads                      */
    /* append, optional clipping bounds (percentiles below 100, src/quant/asymmetric_quant.py:98-104): the range of a
     * channel / token is [lo, hi] instead of its minimum and maximum; values outside are clipped by the code range.
     * Both pointers of a pair or neither.  kvq_sorted_quantile computes them from sorted values.              */
    const float* k_lo;           /* fp32 [B, H, D] contiguous, used when init_k_params = 1                     */
    const float* k_hi;
    const float* v_lo;           /* fp32 [B, H, T] contiguous                                                   */
    const float* v_hi;
} KvqKiviArgs;

KVQ_API int kvq_kivi_append(const KvqKiviArgs* args, kvq_stream_t stream);
KVQ_API int kvq_kivi_dequantize(const KvqKiviArgs* args, kvq_stream_t stream);

/*
 * Two quantiles of every row of a row-sorted matrix, as torch.quantile(x, q, dim=-1) (linear interpolation) gives
 * them: rank = q * (n - 1) in fp32, w = rank - floor(rank), value = w < 0.5 ? fma(w, hi - lo, lo) :
 * fma(w - 1, hi - lo, hi).  `sorted` is fp32 [rows, n], contiguous, ascending in every row (the caller sorts: a sort
 * has no rounding).  Used for the clipping bounds of the KIVI-format cache
 * (src/quant/asymmetric_quant.py:98-104 calls torch.quantile twice, with q = 1 - p and p).
 */
typedef struct KvqQuantileArgs {
    const float* sorted;
    int64_t rows;
    int32_t n;
    float   q_lo, q_hi;
    float*  out_lo;              /* fp32 [rows] */
    float*  out_hi;
} KvqQuantileArgs;

KVQ_API int kvq_sorted_quantile(const KvqQuantileArgs* args, kvq_stream_t stream);

/*
 * Calibration statistic: out[h, g] = max(out[h, g], max over batch rows, tokens and the channels of group g
 * of |x[b, h, s, d]|).  Stands in for compute_absmax_per_group (scripts/calibrate_behavior.py:228-260), the
 * collection half of static-scale calibration; `out` (fp32 [H, G]) is zero-filled by the caller once and
 * accumulates over calls.  Bit-identical to the reference's abs().amax() (a maximum has no rounding).
 */
typedef struct KvqAbsmaxArgs {
    int32_t B, H, S, D;
    int32_t group_size;          /* channels per group; -1 = D                               */
    const void* x;               /* fp16 [B, H, S, D], D contiguous, 16-byte aligned rows    */
    int64_t stride_b, stride_h, stride_s;               /* elements, multiples of 8      */
    float*  out;                 /* fp32 [H, D / group_size]                                 */
} KvqAbsmaxArgs;

KVQ_API int kvq_group_absmax(const KvqAbsmaxArgs* args, kvq_stream_t stream);

/*
 * Sequence-sharded decode, fused exchange: merge this rank's KV splits (the partials that
 * kvq_decode_attn with stages = 1 left in `workspace`), store the normalised partial of every
 * (batch, head) row into every rank's receive buffer with plain 8-byte peer stores over NVLink
 * (value + epoch stamp in one store: no fence, no separate flag), wait (bounded) for the other
 * ranks' rows, and merge the `world` partials into `out` - one launch in
 * place of combine + all-gather + kvq_lse_combine.  No counterpart in the reference (single GPU).
 *
 * Every rank owns one receive buffer of kvq_exchange_bytes(...) bytes, zero-filled before the first
 * use and mapped into every peer (`peer_base[q]` = rank q's buffer as seen from this process; CUDA
 * IPC / symmetric memory; peer_base[rank] is the local buffer).  `slots` independent exchanges
 * (e.g. one per layer) share the buffer; `*epoch` must be >= 1, equal on all ranks, and advance by
 * one between two uses of the same slot.  Ranks must launch the same sequence of exchanges.
 * One process per GPU: a rank never waits for work of its own GPU.
 */
#define KVQ_MAX_PEERS 16
typedef struct KvqExchangeArgs {
    int32_t B, Hq, D, splits;
    const void* workspace;       /* split-K partials of this rank                            */
    size_t  workspace_bytes;
    int32_t rank, world;         /* world <= KVQ_MAX_PEERS                                   */
    void* const* peer_base;      /* HOST array [world] of device pointers                    */
    int32_t slot, slots;
    const int32_t* epoch;        /* device int32                                             */
    uint64_t wait_ns;            /* bound of the wait for peers; 0 = one second              */
    int32_t* status;             /* device int32 or NULL: set to 1 when a wait expired       */
    void*   out;                 /* fp16 [B, Hq, D]                                          */
    int64_t out_stride_b, out_stride_h;                 /* elements                      */
    const KvqAttnArgs* tail_attn; /* HOST pointer or NULL.  The arguments of the stage-1 call when that call ran with
                                     tail_tokens = 1: this rank's last token is then attended here, from the cache,
                                     before the partial is sent (the rank that appended the new token).            */
} KvqExchangeArgs;

/* Bytes of one rank's receive buffer: 2 x slots x world x B x Hq x (D + 2) words of 8 bytes
 * (fp32 value + epoch stamp), rounded up to 256. */
KVQ_API size_t kvq_exchange_bytes(int32_t B, int32_t Hq, int32_t D, int32_t slots, int32_t world);
KVQ_API int kvq_combine_exchange(const KvqExchangeArgs* args, kvq_stream_t stream);

/*
 * Dequantise a cache (or a slice of one) back to fp16 [B, Hkv, S, D].
 * Stands in for INT8KVCache.get_kv (src/cache/int8_cache.py:490-542), INT4KVCache.get_kv and
 * to_tuple, i.e. dequantize_symmetric_int8 / dequantize_symmetric_int4
 * (src/quant/int8_basic.py:167-246, src/quant/int4_basic.py:162-227, after unpack_int4
 * src/quant/int4_basic.py:275-303) and dequantize_asymmetric (src/quant/asymmetric_quant.py:144-196):
 *   value = RN16(fp16(code) * scale)  [ + zero_point, rounded again ];  outlier channels take the
 *   fp16 side value.  K and V are converted in one launch; v.payload == NULL converts K only.
 */
typedef struct KvqDequantArgs {
    int32_t format;              /* KVQ_FMT_INT8 or KVQ_FMT_INT4 (nibble-packed)             */
    int32_t B, Hkv, S, D;
    int32_t group_size;          /* channels per scale; -1 = D                               */
    int32_t n_out;
    const int16_t* outlier_idx;  /* [Hkv, n_out] or NULL                                     */
    KvqCacheSide k, v;
    void* k_out;                 /* fp16, 16-byte aligned                                    */
    void* v_out;
    int64_t out_stride_b, out_stride_h, out_stride_s;   /* elements, multiples of 8; D contiguous */
} KvqDequantArgs;

KVQ_API int kvq_dequantize(const KvqDequantArgs* args, kvq_stream_t stream);

/*
 * Device-side error flags (synchronises the device): 0 = clean.  Bit 0 (1): a bounded wait on a
 * copy-completion barrier expired inside the tensor-core decode kernel (results of that launch
 * are invalid).  Bit 1 (2): kvq_quantize_append met a device-side position at or beyond
 * max_slots and skipped the stores of that token.  Bit 2 (4): the same for kvq_kivi_append.
 * `reset` != 0 clears them.  Negative = KVQ_E*.  No reference counterpart.
 */
KVQ_API int kvq_debug_error_flag(int reset);

/*
 * Self-test of the quantizer's division: the kernels divide every element by a scale that is fixed per group and do
 * it as reciprocal + one residual correction instead of an IEEE division; this runs both on the device over a
 * family of (dividend, divisor) pairs and counts the pairs whose quotients differ as numbers (NaN equals NaN, -0 equals
 * +0: the integer code that follows has no signed zero).  The
 * reference divides with torch's IEEE division (src/quant/int8_basic.py:155-161, int4_basic.py:150-156,
 * asymmetric_quant.py), so the count must be 0.
 *   mode 0: dividends = all 65 536 fp16 values (zeros, subnormals, infinities and NaNs included) x divisors = every
 *           `stride`-th of the 2^23 significands in [1, 2), then the same dividends x the binades 2^-17 .. 2^16 with
 *           a coarse significand sweep, inf and NaN; then every fp32 dividend significand over the constant divisors
 *           7, 15, 127 and 255 (amax / 7, range / 15, ...).  stride 1 covers every quotient the symmetric quantizers
 *           can form (no exponent of theirs under- or overflows).
 *   mode 1: dividends = every `stride`-th fp32 significand in [1, 2) x divisors = all 2^23 significands in [1, 2):
 *           with stride 1 every pair of fp32 significands, which settles every normal fp32 pair whose quotient and
 *           residual stay normal (scaling by powers of two is exact) - the asymmetric quantizer's x - zero_point.
 * Allocates one counter for the duration of the call and synchronises the device.  No reference counterpart.
 */
KVQ_API int kvq_selftest_division(int mode, uint32_t stride, uint64_t* mismatches, uint64_t* pairs);

KVQ_API const char* kvq_strerror(int code);
KVQ_API int  kvq_last_cuda_error(void);     /* cudaError_t of the last KVQ_ECUDA on this thread */
KVQ_API int  kvq_abi_version(void);
/* sizeof of an argument struct as this library was compiled, for binders that mirror the structs by hand
 * (ctypes, cgo): 0 KvqAppendSide, 1 KvqAppendArgs, 2 KvqCacheSide, 3 KvqAttnArgs, 4 KvqCombineArgs,
 * 5 KvqDequantArgs, 6 KvqKiviArgs, 7 KvqAbsmaxArgs, 8 KvqExchangeArgs, 9 KvqQuantileArgs; 0 for any other id.  No reference counterpart. */
KVQ_API size_t kvq_struct_size(int which);

#ifdef __cplusplus
}
#endif
#endif /* KVQ_H_ */
