"""Functional quantizers with the reference's names and return conventions
(src/quant/__init__.py:17-55), executed by the CUDA quantize-append kernel.

Inputs must be fp16 CUDA tensors [B, H, S, D]; outputs are bit-identical to the
reference's torch implementations on the same inputs.  Dequantizers are the
element-wise inverse used by the non-fused `get_kv` path.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import ops
from ._lib import (FMT_INT4, FMT_INT8, SCALE_ASYM_MINMAX, SCALE_DYNAMIC_PCT, SCALE_STATIC)


def _check_quantize_input(tensor: Tensor, func_name: str = "quantize") -> None:
    """NaN/Inf guard of src/quant/_common.py:13-20 (costs one host sync)."""
    if tensor.numel() == 0:
        return
    if not bool(torch.isfinite(tensor).all()):
        if bool(torch.isnan(tensor).any()):
            raise ValueError(f"{func_name}: input contains NaN — refusing to quantize corrupt data")
        raise ValueError(f"{func_name}: input contains Inf — refusing to quantize corrupt data")


def _prep(tensor: Tensor, group_size: int, name: str, need_4d: bool = True):
    if not tensor.is_floating_point():
        raise ValueError(f"Input tensor must be float, got {tensor.dtype}")
    _check_quantize_input(tensor, name)
    if tensor.ndim != 4:
        raise ValueError(f"{name} expects 4D tensor [B,H,S,D], got ndim={tensor.ndim}")
    if not tensor.is_cuda:
        raise ValueError(f"{name} requires a CUDA tensor (no CPU path)")
    if tensor.dtype != torch.float16:
        raise ValueError(f"{name}: the CUDA quantizer is implemented for float16 inputs, got {tensor.dtype}")
    head_dim = tensor.shape[-1]
    if group_size == -1:
        group_size = head_dim
    if group_size <= 0 or head_dim % group_size != 0:
        raise ValueError(f"head_dim {head_dim} must be divisible by group_size {group_size}")
    if tensor.stride(-1) != 1:
        tensor = tensor.contiguous()
    return tensor, group_size, head_dim // group_size


def normalize_static_scale(scale: Tensor, batch: int, heads: int, seq_len: int, num_groups: int) -> Tensor:
    """Accepted static-scale layouts -> a view broadcastable to [B,H,S,G]
    (src/quant/_common.py:37-135): [H,G]; [B|1,H,G]; [H,1,G]; [H,G,1]; [1,H,1,G]; [B,H,S,G]; [B,H,S,G,1]."""
    if scale.ndim == 5:
        if scale.shape[-1] != 1:
            raise ValueError(f"Unsupported scale shape {tuple(scale.shape)}")
        scale = scale[..., 0]
    inferred = None
    if scale.ndim == 2:
        inferred = int(scale.shape[0])
    elif scale.ndim == 4:
        inferred = int(scale.shape[1])
    if inferred is not None and inferred != heads:
        raise ValueError(
            "_normalize_static_scale: calibration vs model heads mismatch "
            "(fail-fast; wrong calibration file was loaded).\n"
            f"  expected heads: {heads} (from model/cache config)\n"
            f"  scale heads:    {inferred} (from scale.shape={tuple(scale.shape)})\n"
            f"  num_groups:     {num_groups}")
    if scale.ndim == 2:
        view = scale[None, :, None, :]
    elif scale.ndim == 4:
        view = scale
    elif scale.ndim == 3:
        d0, d1, d2 = scale.shape
        if d2 == num_groups and d0 == heads and d1 == 1:
            view = scale[:, 0, :][None, :, None, :]
        elif d1 == num_groups and d0 == heads and d2 == 1:
            view = scale[..., 0][None, :, None, :]
        elif d2 == num_groups and d0 == 1 and d1 == heads:
            view = scale[:, :, None, :]
        elif d2 == num_groups and d0 == batch and d1 == heads:
            view = scale[:, :, None, :]
        else:
            raise ValueError(
                f"Unsupported 3D scale shape: {scale.shape} for batch={batch}, heads={heads}, "
                f"num_groups={num_groups}")
    else:
        raise ValueError(f"Unsupported scale ndim={scale.ndim}, shape={tuple(scale.shape)}")
    return view.expand(batch, heads, seq_len, num_groups)


def _alloc(tensor: Tensor, fmt: int, G: int, want_f32: bool, want_zp: bool):
    B, H, S, D = tensor.shape
    dp = D if fmt == FMT_INT8 else D // 2
    dev = tensor.device
    pay = torch.empty((B, H, S, dp), dtype=torch.int8, device=dev)
    sc = torch.empty((B, H, S, G), dtype=torch.float16, device=dev)
    sc32 = torch.empty((B, H, S, G), dtype=torch.float32, device=dev) if want_f32 else None
    zp = torch.empty((B, H, S, G), dtype=torch.float16, device=dev) if want_zp else None
    return pay, sc, sc32, zp


def _run_single(fmt, policy, tensor, group_size, G, *, static=None, quantile=1.0, want_f32=False,
                want_zp=False):
    """Quantize one tensor through the K side of the append kernel into fresh buffers."""
    pay, sc, sc32, zp = _alloc(tensor, fmt, G, want_f32, want_zp)
    ops.quantize_append(fmt, policy, tensor, None, pay, None, sc, None, 0, group_size,
                        k_zp=zp, k_scale_f32=sc32, k_static=static, quantile=quantile)
    return pay, sc, sc32, zp


def _static_rows(tensor: Tensor, scale: Tensor, G: int):
    """Static scales of any accepted layout as a per-row table: view the tensor as
    [1, B*H*S, 1, D] with a [B*H*S, G] table when the layout is not plain [H, G]."""
    B, H, S, D = tensor.shape
    if scale.device != tensor.device:
        raise ValueError(
            f"scale device ({scale.device}) != tensor device ({tensor.device}). "
            "Move scale to the same device before quantization.")
    if scale.ndim == 2 and scale.shape == (H, G):
        return tensor, scale.contiguous(), None
    full = normalize_static_scale(scale, B, H, S, G).reshape(B * H * S, G).contiguous()
    flat = tensor.contiguous().view(1, B * H * S, 1, D)
    return flat, full, (B, H, S)


def quantize_symmetric_int8(tensor: Tensor, percentile: float = 99.9, group_size: int = 128
                            ) -> Tuple[Tensor, Tensor]:
    """src/quant/int8_basic.py:18-108 -> (int8 [B,H,S,D], fp16 scale [B,H,S,G])."""
    tensor, gs, G = _prep(tensor, group_size, "quantize_symmetric_int8")
    q = max(min(percentile / 100.0, 1.0), 0.0) if percentile < 100.0 else 1.0
    pay, sc, _, _ = _run_single(FMT_INT8, SCALE_DYNAMIC_PCT, tensor, gs, G, quantile=q)
    return pay, sc


def quantize_symmetric_int8_with_scale(tensor: Tensor, scale: Tensor, group_size: int
                                       ) -> Tuple[Tensor, Tensor]:
    """src/quant/int8_basic.py:111-164."""
    tensor, gs, G = _prep(tensor, group_size, "quantize_symmetric_int8_with_scale")
    if scale.dtype not in (torch.float16, torch.float32):
        scale = scale.float()
    flat, table, shape = _static_rows(tensor, scale, G)
    pay, sc, _, _ = _run_single(FMT_INT8, SCALE_STATIC, flat, gs, G, static=table)
    if shape is not None:
        B, H, S = shape
        pay, sc = pay.view(B, H, S, -1), sc.view(B, H, S, G)
    return pay, sc


def quantize_symmetric_int4(tensor: Tensor, percentile: float = 99.9, group_size: int = 32
                            ) -> Tuple[Tensor, Tensor]:
    """src/quant/int4_basic.py:24-112 -> (int8 codes in [-7,7] [B,H,S,D], fp32 scale)."""
    tensor, gs, G = _prep(tensor, group_size, "quantize_symmetric_int4")
    q = max(min(percentile / 100.0, 1.0), 0.0) if percentile < 100.0 else 1.0
    pay, _, sc32, _ = _run_single(FMT_INT4, SCALE_DYNAMIC_PCT, tensor, gs, G, quantile=q, want_f32=True)
    return unpack_int4(pay), sc32


def quantize_symmetric_int4_with_scale(tensor: Tensor, scale: Tensor, group_size: int
                                       ) -> Tuple[Tensor, Tensor]:
    """src/quant/int4_basic.py:115-159."""
    tensor, gs, G = _prep(tensor, group_size, "quantize_symmetric_int4_with_scale")
    flat, table, shape = _static_rows(tensor, scale.float() if scale.dtype != torch.float16 else scale, G)
    pay, _, sc32, _ = _run_single(FMT_INT4, SCALE_STATIC, flat, gs, G, static=table, want_f32=True)
    codes = unpack_int4(pay)
    if shape is not None:
        B, H, S = shape
        codes, sc32 = codes.view(B, H, S, -1), sc32.view(B, H, S, G)
    return codes, sc32


def quantize_asymmetric_groupwise(tensor: Tensor, group_size: int = 32, quant_bits: int = 4):
    """Group-wise asymmetric quantization: the reference's `quantize_asymmetric`
    (src/quant/asymmetric_quant.py:24-141) on a [B,H,S,G,gs] view with axis=-1.
    Returns (payload, scale fp32 [B,H,S,G], zero_point fp32-valued fp16 pair is not
    kept: scale/zp are returned as the fp16 values the decode kernel reads, plus the fp32 scale)."""
    tensor, gs, G = _prep(tensor, group_size, "quantize_asymmetric_groupwise")
    if quant_bits not in (4, 8):
        raise ValueError(f"quant_bits must be 4 or 8, got {quant_bits}")
    fmt = FMT_INT4 if quant_bits == 4 else FMT_INT8
    pay, sc, sc32, zp = _run_single(fmt, SCALE_ASYM_MINMAX, tensor, gs, G, want_f32=True, want_zp=True)
    return pay, sc, zp, sc32


# ------------------------------------------------------------------ pack / unpack
def pack_int4(tensor: Tensor) -> Tensor:
    """src/quant/int4_basic.py:230-272 (integer reshuffle; torch ops on the tensor's device)."""
    if tensor.dtype != torch.int8:
        raise ValueError(f"pack_int4 expects int8 input, got {tensor.dtype}")
    if tensor.shape[-1] % 2 != 0:
        raise ValueError("Last dimension must be even for packing")
    if os.environ.get("KV_PACK_VALIDATE", "0") == "1" and tensor.numel() > 0:
        lo, hi = int(tensor.min().item()), int(tensor.max().item())
        if lo < -8 or hi > 7:
            raise ValueError(f"pack_int4 expects values in [-8, 7], got min={lo}, max={hi}")
    u = (tensor.to(torch.int16) + 8).to(torch.uint8)
    u = u.view(*tensor.shape[:-1], tensor.shape[-1] // 2, 2)
    return ((u[..., 0] << 4) | u[..., 1]).to(torch.int8)


def unpack_int4(packed: Tensor) -> Tensor:
    """src/quant/int4_basic.py:275-303."""
    if packed.dtype != torch.int8:
        raise ValueError(f"unpack_int4 expects int8 packed input, got {packed.dtype}")
    u = packed.view(torch.uint8)
    out = torch.stack(((u >> 4) & 0x0F, u & 0x0F), dim=-1).view(*packed.shape[:-1], packed.shape[-1] * 2)
    return (out.to(torch.int16) - 8).to(torch.int8)


# ------------------------------------------------------------------ dequantizers
def _dequant(quantized: Tensor, scale: Tensor, zp: Optional[Tensor], name: str) -> Tensor:
    if quantized.dtype != torch.int8:
        raise ValueError(f"quantized must be torch.int8, got {quantized.dtype}")
    if not scale.is_floating_point():
        raise ValueError(f"scale must be floating point, got {scale.dtype}")
    if scale.ndim == quantized.ndim + 1:
        scale = scale.squeeze(-1)
        if zp is not None:
            zp = zp.squeeze(-1)
    if scale.ndim != quantized.ndim:
        raise ValueError(
            f"Unsupported scale rank for {name}: quantized.ndim={quantized.ndim}, scale.ndim={scale.ndim}")
    B, H, S, D = quantized.shape
    G = scale.shape[-1]
    if G <= 0 or D % G != 0:
        raise ValueError(
            f"Invalid scale shape for group-wise dequantization: quantized={tuple(quantized.shape)}, "
            f"scale={tuple(scale.shape)}")
    x = quantized.view(B, H, S, G, D // G).to(scale.dtype) * scale.unsqueeze(-1)
    if zp is not None:
        x = x + zp.unsqueeze(-1)
    return x.view(B, H, S, D)


def dequantize_symmetric_int8(quantized: Tensor, scale: Tensor) -> Tensor:
    """src/quant/int8_basic.py:167-246."""
    return _dequant(quantized, scale, None, "dequantize_symmetric_int8")


def dequantize_symmetric_int4(quantized: Tensor, scale: Tensor) -> Tensor:
    """src/quant/int4_basic.py:162-227."""
    return _dequant(quantized, scale, None, "dequantize_symmetric_int4")


def dequantize_asymmetric_groupwise(quantized: Tensor, scale: Tensor, zero_point: Tensor) -> Tensor:
    """codes * scale + zero_point in the scale's dtype (src/quant/asymmetric_quant.py:144-196)."""
    return _dequant(quantized, scale, zero_point, "dequantize_asymmetric_groupwise")
