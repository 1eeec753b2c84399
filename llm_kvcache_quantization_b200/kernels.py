"""Fused q_len==1 decode attention entry points.

`decode_attn_int8` and `decode_attn_int4` keep the signatures, argument
meaning and error behaviour of the reference's Triton wrappers
(src/kernels/triton_decode_attn_int8.py:306-519,
 src/kernels/triton_decode_attn_int4.py:62-121); the work is done by the
sm_100a split-K kernel in libkvq.so.  Differences, all deliberate:

* INT4 caches are read packed; nothing is unpacked or materialised.
* `block_size` is accepted and validated but only recorded: tiling is fixed
  inside the kernel.
* The two `.item()` syncs the reference performs on `context_lens` are replaced
  by one (`KVQ_SKIP_CONTEXT_CHECK=1` removes it; the kernel clamps lengths to
  `[0, S]` and zero-length rows yield zeros either way).

The remaining entry points (`decode_attn_fp16`, `decode_attn_int4_asym`,
`decode_attn_int4_outlier`) cover formats the reference has no fused kernel for.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import ops
from ._lib import FMT_FP16, FMT_INT4, FMT_INT8

_BLOCK_SIZES = (32, 64, 128, 256)


def _resolve_block_size(block_size: Optional[int], max_ctx: int) -> int:
    if block_size is None:
        env_block_size = os.environ.get("KV_TRITON_BLOCK_SIZE")
        if env_block_size:
            try:
                block_size = int(env_block_size)
            except ValueError as exc:
                raise ValueError(
                    f"KV_TRITON_BLOCK_SIZE must be an integer, got {env_block_size!r}") from exc
        else:
            block_size = 128 if max_ctx >= 8192 else 64
    if block_size not in _BLOCK_SIZES:
        raise ValueError(f"Unsupported block_size={block_size}. Choose from [32, 64, 128, 256].")
    return block_size


def _validate_common(q, k_cache, v_cache, k_scale, v_scale, context_lens, payload_dim, what):
    if q.ndim != 3:
        raise ValueError(f"q must have shape [B, Hq, D], got {tuple(q.shape)}")
    if k_cache.ndim != 4 or v_cache.ndim != 4:
        raise ValueError(
            f"k_cache/v_cache must have shape [B, Hkv, S, D], got {tuple(k_cache.shape)} / {tuple(v_cache.shape)}")
    if k_scale.ndim != 4 or v_scale.ndim != 4:
        raise ValueError(
            f"k_scale/v_scale must have shape [B, Hkv, S, G], got {tuple(k_scale.shape)} / {tuple(v_scale.shape)}")
    if context_lens.ndim != 1:
        raise ValueError(f"context_lens must be 1D, got {tuple(context_lens.shape)}")
    if not q.is_cuda:
        raise ValueError(f"{what} requires CUDA tensors.")
    if k_cache.dtype != torch.int8:
        raise ValueError(f"k_cache must be torch.int8, got {k_cache.dtype}")
    if v_cache.dtype != torch.int8:
        raise ValueError(f"v_cache must be torch.int8, got {v_cache.dtype}")
    if k_scale.dtype != torch.float16:
        raise ValueError(
            f"k_scale must be torch.float16 for the fused kernel, got {k_scale.dtype}. "
            "Cast with k_scale.to(torch.float16) before calling.")
    if v_scale.dtype != torch.float16:
        raise ValueError(
            f"v_scale must be torch.float16 for the fused kernel, got {v_scale.dtype}. "
            "Cast with v_scale.to(torch.float16) before calling.")
    if k_cache.stride(-1) != 1:
        raise ValueError(
            f"k_cache inner dim must be contiguous (stride=1), got stride={k_cache.stride(-1)}. "
            "Use .contiguous() before passing to kernel.")
    if v_cache.stride(-1) != 1:
        raise ValueError(f"v_cache inner dim must be contiguous (stride=1), got stride={v_cache.stride(-1)}.")
    batch, q_heads, head_dim = q.shape
    if head_dim == 0 or (head_dim & (head_dim - 1)) != 0:
        raise ValueError(f"HEAD_DIM must be a power of 2, got {head_dim}.")
    if k_cache.shape[0] != batch or v_cache.shape[0] != batch:
        raise ValueError(f"Batch mismatch: q={batch}, k={k_cache.shape[0]}, v={v_cache.shape[0]}")
    if k_cache.shape[-1] != payload_dim or v_cache.shape[-1] != payload_dim:
        raise ValueError(
            f"Head dim mismatch: q={head_dim}, k={k_cache.shape[-1]}, v={v_cache.shape[-1]}")
    if k_cache.shape[:3] != v_cache.shape[:3]:
        raise ValueError(f"k/v cache shape mismatch: {tuple(k_cache.shape)} vs {tuple(v_cache.shape)}")
    if k_scale.shape[:3] != k_cache.shape[:3] or v_scale.shape[:3] != v_cache.shape[:3]:
        raise ValueError(
            "Scale and cache shapes mismatch: "
            f"k_scale={tuple(k_scale.shape)}, v_scale={tuple(v_scale.shape)}, "
            f"k={tuple(k_cache.shape)}, v={tuple(v_cache.shape)}")
    if k_scale.shape[-1] != v_scale.shape[-1]:
        raise ValueError(
            f"k_scale/v_scale num_groups mismatch: k={k_scale.shape[-1]} vs v={v_scale.shape[-1]}.")
    if context_lens.shape[0] != batch:
        raise ValueError(f"context_lens batch mismatch: expected {batch}, got {context_lens.shape[0]}")
    kv_heads = k_cache.shape[1]
    if q_heads % kv_heads != 0:
        raise ValueError(f"GQA head mismatch: q_heads={q_heads} must be a multiple of kv_heads={kv_heads}")
    num_groups = k_scale.shape[-1]
    if num_groups <= 0:
        raise ValueError(f"num_groups must be > 0, got {num_groups}")
    if head_dim % num_groups != 0:
        raise ValueError(f"head_dim {head_dim} must be divisible by num_groups {num_groups}")


def _check_context_range(context_lens: torch.Tensor, max_seq: int):
    """Returns (min, max) of context_lens, or (None, None) when the check is disabled."""
    if os.environ.get("KVQ_SKIP_CONTEXT_CHECK", "0") == "1" or context_lens.numel() == 0:
        return None, None
    lo, hi = torch.aminmax(context_lens)
    lo_hi = torch.stack((lo, hi)).tolist()        # one host sync
    mn, mx = int(lo_hi[0]), int(lo_hi[1])
    if mn < 0:
        raise ValueError(f"context_lens must be >= 0, got min={mn}")
    if mx > max_seq:
        raise ValueError(f"context_lens max ({mx}) exceeds cache seq dim ({max_seq})")
    return mn, mx


def _record_stats(debug_stats, layer_idx, block_size):
    if isinstance(debug_stats, dict):
        debug_stats["triton_kernel_calls"] = int(debug_stats.get("triton_kernel_calls", 0)) + 1
        debug_stats["triton_block_size"] = int(block_size)
        if layer_idx is not None:
            hits = debug_stats.setdefault("triton_layer_hits", {})
            key = str(layer_idx)
            hits[key] = int(hits.get(key, 0)) + 1


def _run(fmt, q, k_cache, v_cache, k_scale, v_scale, context_lens, sm_scale, head_dim,
         debug_stats, layer_idx, block_size, **extra):
    if sm_scale is None:
        sm_scale = 1.0 / (q.shape[-1] ** 0.5)
    max_seq = int(k_cache.shape[2])
    mn, mx = _check_context_range(context_lens, max_seq)
    if mx == 0 or max_seq == 0 or q.shape[0] == 0:
        return torch.zeros_like(q)
    block_size = _resolve_block_size(block_size, mx if mx is not None else max_seq)
    original_dtype = q.dtype
    if original_dtype != torch.float16:
        q = q.to(torch.float16)
    _record_stats(debug_stats, layer_idx, block_size)
    out = ops.decode_attn(fmt, q, k_cache, v_cache, k_scale, v_scale, context_lens, float(sm_scale),
                          head_dim=head_dim, max_ctx=mx, **extra)
    if original_dtype != torch.float16:
        out = out.to(original_dtype)
    return out


def decode_attn_int8(q, k_cache, v_cache, k_scale, v_scale, context_lens, sm_scale=None,
                     debug_stats: Optional[dict] = None, layer_idx: Optional[int] = None,
                     block_size: Optional[int] = None, *, inv_tau: Optional[torch.Tensor] = None):
    """q [B,Hq,D]; k_cache/v_cache int8 [B,Hkv,S,D]; k_scale/v_scale fp16 [B,Hkv,S,G];
    context_lens int32 [B] -> [B,Hq,D] in q's dtype.
    `inv_tau` (fp32 [Hq], optional, not in the reference signature) multiplies q in
    fp16 inside the kernel, as the reference's patched forward does before the call."""
    _validate_common(q, k_cache, v_cache, k_scale, v_scale, context_lens, q.shape[-1], "decode_attn_int8")
    return _run(FMT_INT8, q, k_cache, v_cache, k_scale, v_scale, context_lens, sm_scale, q.shape[-1],
                debug_stats, layer_idx, block_size, inv_tau=inv_tau)


def decode_attn_int4(q, k_cache_int4, v_cache_int4, k_scale, v_scale, context_lens,
                     sm_scale: Optional[float] = None, *, bit_packed: bool = True,
                     head_dim: Optional[int] = None, debug_stats: Optional[dict] = None,
                     layer_idx: Optional[int] = None, block_size: Optional[int] = None,
                     inv_tau: Optional[torch.Tensor] = None):
    """INT4 cache, packed ([B,Hkv,S,D/2]) or unpacked ([B,Hkv,S,D] int8 codes in [-8,7])."""
    if q.ndim != 3:
        raise ValueError(f"q must have shape [B, Hq, D], got {tuple(q.shape)}")
    if head_dim is not None:
        d = int(head_dim)
        if d <= 0:
            raise ValueError(f"head_dim must be positive, got {d}")
    else:
        d = q.shape[-1]
    if not bit_packed:
        if k_cache_int4.shape[-1] != d or v_cache_int4.shape[-1] != d:
            raise ValueError(
                f"Unpacked INT4 cache last dim mismatch: got {k_cache_int4.shape[-1]}, expected {d}")
        for c in (k_cache_int4, v_cache_int4):
            if c.stride(-1) != 1:
                raise ValueError(
                    f"Unpacked INT4 cache inner dim must be contiguous (stride=1), got stride={c.stride(-1)}. "
                    "Use .contiguous().")
            if c.dtype != torch.int8:
                raise ValueError(f"Unpacked INT4 cache must be int8, got {c.dtype}.")
        return decode_attn_int8(q, k_cache_int4, v_cache_int4, k_scale, v_scale, context_lens, sm_scale,
                                debug_stats=debug_stats, layer_idx=layer_idx, block_size=block_size,
                                inv_tau=inv_tau)
    if k_cache_int4.shape[-1] * 2 != d or v_cache_int4.shape[-1] * 2 != d:
        raise ValueError(
            f"Packed INT4 cache last dim mismatch: got {k_cache_int4.shape[-1]}, expected {d // 2}")
    if q.shape[-1] != d:
        raise ValueError(f"Head dim mismatch: q={q.shape[-1]}, head_dim={d}")
    _validate_common(q, k_cache_int4, v_cache_int4, k_scale, v_scale, context_lens, d // 2, "decode_attn_int4")
    return _run(FMT_INT4, q, k_cache_int4, v_cache_int4, k_scale, v_scale, context_lens, sm_scale, d,
                debug_stats, layer_idx, block_size, inv_tau=inv_tau)


def decode_attn_int4_asym(q, k_cache_int4, v_cache_int4, k_scale, k_zp, v_scale, v_zp, context_lens,
                          sm_scale: Optional[float] = None, *, debug_stats=None, layer_idx=None,
                          inv_tau: Optional[torch.Tensor] = None):
    """Group-wise asymmetric INT4 (fp16 scale and zero-point per token group), packed nibbles.
    Dequantisation is RN16(RN16(code * scale) + zp), the fp16 arithmetic of
    dequantize_asymmetric (src/quant/asymmetric_quant.py:193-196)."""
    d = q.shape[-1]
    _validate_common(q, k_cache_int4, v_cache_int4, k_scale, v_scale, context_lens, d // 2,
                     "decode_attn_int4_asym")
    for z, s in ((k_zp, k_scale), (v_zp, v_scale)):
        if z.dtype != torch.float16 or z.shape != s.shape:
            raise ValueError("zero-points must be fp16 with the shape of the scales")
    return _run(FMT_INT4, q, k_cache_int4, v_cache_int4, k_scale, v_scale, context_lens, sm_scale, d,
                debug_stats, layer_idx, None, inv_tau=inv_tau, k_zp=k_zp, v_zp=v_zp)


def decode_attn_int4_outlier(q, k_cache_int4, v_cache_int4, k_scale, v_scale, k_side, v_side, outlier_idx,
                             context_lens, sm_scale: Optional[float] = None, *, debug_stats=None,
                             layer_idx=None, inv_tau: Optional[torch.Tensor] = None):
    """Symmetric INT4 plus an fp16 side buffer for `outlier_idx` ([Hkv, n_out] int16) channels:
    those channels carry code 0 in the payload and their fp16 values in
    k_side / v_side [B,Hkv,S,n_out]; the gather is fused into the dequant loop."""
    d = q.shape[-1]
    _validate_common(q, k_cache_int4, v_cache_int4, k_scale, v_scale, context_lens, d // 2,
                     "decode_attn_int4_outlier")
    if outlier_idx.dtype != torch.int16 or outlier_idx.ndim != 2 or outlier_idx.shape[0] != k_cache_int4.shape[1]:
        raise ValueError("outlier_idx must be int16 [Hkv, n_out]")
    for sd in (k_side, v_side):
        if sd.dtype != torch.float16 or sd.shape[:3] != k_cache_int4.shape[:3] or sd.shape[-1] != outlier_idx.shape[1]:
            raise ValueError("outlier side buffers must be fp16 [B, Hkv, S, n_out]")
    return _run(FMT_INT4, q, k_cache_int4, v_cache_int4, k_scale, v_scale, context_lens, sm_scale, d,
                debug_stats, layer_idx, None, inv_tau=inv_tau, outlier_idx=outlier_idx.contiguous(),
                k_side=k_side, v_side=v_side)


def decode_attn_fp16(q, k_cache, v_cache, context_lens, sm_scale: Optional[float] = None, *,
                     debug_stats=None, layer_idx=None, inv_tau: Optional[torch.Tensor] = None):
    """Unquantized fp16 cache [B,Hkv,S,D] through the same split-K kernel."""
    if q.ndim != 3 or k_cache.ndim != 4 or v_cache.ndim != 4:
        raise ValueError("expected q [B,Hq,D] and k/v [B,Hkv,S,D]")
    if not q.is_cuda:
        raise ValueError("decode_attn_fp16 requires CUDA tensors.")
    if k_cache.dtype != torch.float16 or v_cache.dtype != torch.float16:
        raise ValueError("fp16 cache expected")
    if k_cache.shape != v_cache.shape or k_cache.shape[-1] != q.shape[-1] or k_cache.shape[0] != q.shape[0]:
        raise ValueError("q / k / v shape mismatch")
    if q.shape[1] % k_cache.shape[1] != 0:
        raise ValueError("GQA head mismatch")
    return _run(FMT_FP16, q, k_cache, v_cache, None, None, context_lens, sm_scale, q.shape[-1],
                debug_stats, layer_idx, None, inv_tau=inv_tau)
