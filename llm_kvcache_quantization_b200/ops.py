"""Thin tensor-level wrappers over the C ABI (pointers, strides, stream, workspace).

torch is used for device memory, streams and dtype bookkeeping only; all
arithmetic happens in libkvq.so.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import (FMT_FP16, FMT_INT4, FMT_INT8, F_ADAPTIVE, F_MIXED_RESCUE, F_RESCUE_THR,
                   SCALE_ASYM_MINMAX, SCALE_DYNAMIC_PCT, SCALE_STATIC)

_WORKSPACES = {}


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("libkvq requires CUDA tensors (there is no CPU path).")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"device mismatch: {t.device} vs {dev}")
    return dev


_RETIRED = []      # outgrown workspaces: a CUDA graph captured earlier may still hold their addresses


def get_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Per-(device, stream) scratch buffer for split-K partials; grows, never shrinks.  A buffer that has been handed
    out is never returned to the allocator while the process lives (unless `release_workspaces` is called): a CUDA
    graph captured around an earlier call replays with the old address, which must stay ours."""
    key = (device.index, _stream_ptr(device))
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _RETIRED.append(buf)
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buf
    return buf


def release_workspaces() -> None:
    """Drop every scratch buffer.  Only when no captured graph that used them will be replayed again."""
    _WORKSPACES.clear()
    _RETIRED.clear()


_LAST_SPLITS = 0


def last_splits() -> int:
    """KV split count used by the most recent decode_attn call (diagnostics)."""
    return _LAST_SPLITS


# --------------------------------------------------------------------------- append
def _append_side(src, payload, scale, zp, scale_f32, side, static_scale, rescue_thr) -> _lib.KvqAppendSide:
    s = _lib.KvqAppendSide()
    if src.stride(-1) != 1:
        raise ValueError("new K/V tokens must be contiguous in head_dim")
    s.src = src.data_ptr()
    s.src_stride_b, s.src_stride_h, s.src_stride_t = src.stride(0), src.stride(1), src.stride(2)
    es = payload.element_size()
    if payload.stride(-1) != 1:
        raise ValueError("cache payload must be contiguous in its last dimension")
    s.payload = payload.data_ptr()
    s.pay_stride_b, s.pay_stride_h, s.pay_stride_s = (payload.stride(0) * es, payload.stride(1) * es,
                                                      payload.stride(2) * es)
    if scale is not None:
        if scale.dtype != torch.float16 or scale.stride(-1) != 1:
            raise ValueError("cache scale buffer must be fp16, contiguous in groups")
        s.scale = scale.data_ptr()
        s.sc_stride_b, s.sc_stride_h, s.sc_stride_s = scale.stride(0), scale.stride(1), scale.stride(2)
    if zp is not None:
        if zp.dtype != torch.float16 or zp.stride() != scale.stride():
            raise ValueError("zero-point buffer must be fp16 with the strides of the scale buffer")
        s.zp = zp.data_ptr()
    if scale_f32 is not None:
        if scale_f32.dtype != torch.float32 or scale_f32.stride() != scale.stride():
            raise ValueError("fp32 scale copy must share the strides of the fp16 scale buffer")
        s.scale_f32 = scale_f32.data_ptr()
    if side is not None:
        if side.dtype != torch.float16 or side.stride(-1) != 1:
            raise ValueError("outlier side buffer must be fp16, contiguous in its last dimension")
        s.side = side.data_ptr()
        s.side_stride_b, s.side_stride_h, s.side_stride_s = side.stride(0), side.stride(1), side.stride(2)
    if static_scale is not None:
        if static_scale.dtype not in (torch.float16, torch.float32) or not static_scale.is_contiguous():
            raise ValueError("static scale table must be a contiguous fp16/fp32 [Hkv, G] tensor")
        s.static_scale = static_scale.data_ptr()
        s.static_scale_is_f32 = 1 if static_scale.dtype == torch.float32 else 0
    if rescue_thr is not None:
        s.rescue_threshold = rescue_thr.data_ptr()
    return s


def quantize_append(fmt: int, policy: int, k_new: torch.Tensor, v_new: torch.Tensor,
                    k_payload: torch.Tensor, v_payload: torch.Tensor,
                    k_scale: Optional[torch.Tensor], v_scale: Optional[torch.Tensor],
                    write_pos, group_size: int, *,
                    k_zp=None, v_zp=None, k_scale_f32=None, v_scale_f32=None,
                    k_static=None, v_static=None, flags: int = 0, adaptive_margin: float = 1.0,
                    quantile: float = 1.0, k_rescue_thr=None, v_rescue_thr=None,
                    outlier_idx=None, k_side=None, v_side=None,
                    rope_cos: Optional[torch.Tensor] = None, rope_sin: Optional[torch.Tensor] = None,
                    q: Optional[torch.Tensor] = None, q_out: Optional[torch.Tensor] = None):
    """Quantize `k_new`, `v_new` ([B,Hkv,T,D] fp16) into cache slots
    [write_pos, write_pos+T) of the given payload / scale buffers in one launch (`v_new=None`: K side only).
    `write_pos` is an int or an int32 device tensor (read on the device).

    With `rope_cos` / `rope_sin` (fp16 [B or 1, T, rotary_dim]) the same launch applies rotate-half
    RoPE to K before quantizing it and, when `q` ([B,Hq,T,D] fp16, before rotation) is given, to the
    query; the rotated query is returned (`q_out` or a new tensor)."""
    dev = _require_cuda(k_new, v_new, k_payload, v_payload, k_scale, v_scale)
    if k_new.dtype != torch.float16 or (v_new is not None and v_new.dtype != torch.float16):
        raise ValueError("quantize_append expects fp16 K/V")
    if k_new.ndim != 4 or (v_new is not None and k_new.shape != v_new.shape):
        raise ValueError(f"k/v shape mismatch or not 4D: {tuple(k_new.shape)}")
    B, H, T, D = k_new.shape
    a = _lib.KvqAppendArgs()
    a.format, a.policy, a.flags = fmt, policy, flags
    a.B, a.Hkv, a.T, a.D = B, H, T, D
    a.group_size = group_size
    a.adaptive_margin = float(adaptive_margin)
    a.quantile = float(quantile)
    if outlier_idx is not None:
        if outlier_idx.dtype != torch.int16 or not outlier_idx.is_contiguous() or outlier_idx.shape[0] != H:
            raise ValueError("outlier_idx must be a contiguous int16 [Hkv, n_out] tensor")
        a.n_out = outlier_idx.shape[1]
        a.outlier_idx = outlier_idx.data_ptr()
    # the kernel itself refuses slots at or beyond the smallest destination buffer (a device-side position that ran
    # past the capacity stores nothing and raises bit 1 of kvq_debug_error_flag)
    cap = k_payload.shape[2] if v_payload is None or v_new is None else min(k_payload.shape[2], v_payload.shape[2])
    a.max_slots = cap
    if isinstance(write_pos, torch.Tensor):
        if write_pos.dtype != torch.int32 or not write_pos.is_cuda:
            raise ValueError("device write_pos must be an int32 CUDA tensor")
        a.write_pos_dev = write_pos.data_ptr()
    else:
        a.write_pos = int(write_pos)
        if a.write_pos < 0 or a.write_pos + T > cap:
            raise ValueError(f"append of {T} tokens at {a.write_pos} exceeds capacity {cap}")
    a.k = _append_side(k_new, k_payload, k_scale, k_zp, k_scale_f32, k_side, k_static, k_rescue_thr)
    if v_new is not None:
        a.v = _append_side(v_new, v_payload, v_scale, v_zp, v_scale_f32, v_side, v_static, v_rescue_thr)
    if (rope_cos is None) != (rope_sin is None):
        raise ValueError("rope_cos and rope_sin go together")
    if q is not None and rope_cos is None:
        raise ValueError("a query is only taken together with rope_cos / rope_sin")
    if rope_cos is not None:
        for name, t in (("rope_cos", rope_cos), ("rope_sin", rope_sin)):
            if t.dtype != torch.float16 or t.ndim != 3 or t.stride(-1) != 1 or t.shape[1] != T or \
                    t.shape[0] not in (1, B) or not t.is_cuda:
                raise ValueError(f"{name} must be an fp16 CUDA tensor [B or 1, T, rotary_dim]")
        if rope_cos.shape != rope_sin.shape or rope_cos.stride() != rope_sin.stride():
            raise ValueError("rope_cos / rope_sin must share shape and strides")
        rd = rope_cos.shape[-1]
        if rd % 2 or rd > D:
            raise ValueError(f"RoPE dim {rd} must be even and <= head_dim {D}")
        a.rope_cos, a.rope_sin = rope_cos.data_ptr(), rope_sin.data_ptr()
        a.rope_stride_b = 0 if rope_cos.shape[0] == 1 else rope_cos.stride(0)
        a.rope_stride_t = rope_cos.stride(1)
        a.rotary_dim = rd
        if q is not None:
            if q.dtype != torch.float16 or q.ndim != 4 or q.shape[0] != B or q.shape[2] != T or q.shape[3] != D or \
                    q.stride(-1) != 1:
                raise ValueError("q must be fp16 [B, Hq, T, D], contiguous in head_dim")
            if q_out is None:
                q_out = torch.empty((B, q.shape[1], T, D), dtype=torch.float16, device=dev)
            elif q_out.shape != q.shape or q_out.dtype != torch.float16 or q_out.stride(-1) != 1:
                raise ValueError("q_out must match q")
            a.Hq = q.shape[1]
            a.q_src = q.data_ptr()
            a.q_stride_b, a.q_stride_h, a.q_stride_t = q.stride(0), q.stride(1), q.stride(2)
            a.q_out = q_out.data_ptr()
            a.qo_stride_b, a.qo_stride_h, a.qo_stride_t = q_out.stride(0), q_out.stride(1), q_out.stride(2)
    with torch.cuda.device(dev):
        rc = _lib.load().kvq_quantize_append(C.byref(a), _stream_ptr(dev))
    _lib.check("kvq_quantize_append", rc)
    return q_out


# --------------------------------------------------------------------------- attention
def _cache_side(payload, scale, zp, side) -> _lib.KvqCacheSide:
    s = _lib.KvqCacheSide()
    es = payload.element_size()
    s.payload = payload.data_ptr()
    s.pay_stride_b, s.pay_stride_h, s.pay_stride_s = (payload.stride(0) * es, payload.stride(1) * es,
                                                      payload.stride(2) * es)
    if scale is not None:
        s.scale = scale.data_ptr()
        s.sc_stride_b, s.sc_stride_h, s.sc_stride_s = scale.stride(0), scale.stride(1), scale.stride(2)
    if zp is not None:
        if zp.stride() != scale.stride():
            raise ValueError("zero-points must share the strides of the scales")
        s.zp = zp.data_ptr()
    if side is not None:
        s.side = side.data_ptr()
        s.side_stride_b, s.side_stride_h, s.side_stride_s = side.stride(0), side.stride(1), side.stride(2)
    return s


def decode_attn(fmt: int, q: torch.Tensor, k_payload: torch.Tensor, v_payload: torch.Tensor,
                k_scale: Optional[torch.Tensor], v_scale: Optional[torch.Tensor],
                context_lens: Optional[torch.Tensor], sm_scale: float, *, head_dim: int,
                k_zp=None, v_zp=None, inv_tau: Optional[torch.Tensor] = None,
                outlier_idx=None, k_side=None, v_side=None,
                splits: int = 0, out: Optional[torch.Tensor] = None,
                return_partial: bool = False, max_ctx: Optional[int] = None, stages: int = 0,
                packed_partial: Optional[torch.Tensor] = None, fast_dequant: Optional[bool] = None,
                tail_tokens: int = 0, exchange: Optional[dict] = None,
                q_chan_scale: Optional[torch.Tensor] = None):
    """Fused q_len==1 attention over a (quantized) cache.  q fp16 [B,Hq,D].

    Returns `out` fp16 [B,Hq,D]; with `return_partial` also the normalised
    partial `(o fp32 [B,Hq,D], m fp32 [B,Hq], l fp32 [B,Hq])` used by the
    sequence-sharded merge.  `packed_partial` (fp32 [B,Hq,D+2], contiguous) receives the
    same partial as one buffer `[o (D) | m | l]` per (b, h) - the send buffer of the
    sequence-sharded all-gather.  No host synchronisation happens here.

    `exchange` (sequence sharding, see `parallel.PeerExchange`): the combine stage becomes the fused
    combine / peer-store exchange / merge kernel, and `out` receives the attention over ALL ranks' tokens.
    """
    dev = _require_cuda(q, k_payload, v_payload, k_scale, v_scale, context_lens)
    if q.dtype != torch.float16:
        raise ValueError("decode_attn expects an fp16 query")
    B, Hq, D = q.shape
    if D != head_dim:
        raise ValueError(f"Head dim mismatch: q={D}, expected {head_dim}")
    Hkv = k_payload.shape[1]
    S = k_payload.shape[2]
    a = _lib.KvqAttnArgs()
    a.format = fmt
    a.B, a.Hq, a.Hkv, a.D = B, Hq, Hkv, D
    G = 1 if k_scale is None else k_scale.shape[-1]
    a.group_size = D // G
    a.max_ctx = S if max_ctx is None else min(int(max_ctx), S)
    if q.stride(-1) != 1:
        q = q.contiguous()
    a.q = q.data_ptr()
    a.q_stride_b, a.q_stride_h = q.stride(0), q.stride(1)
    if inv_tau is not None:
        if inv_tau.dtype != torch.float32 or not inv_tau.is_contiguous() or inv_tau.numel() != Hq:
            raise ValueError("inv_tau must be a contiguous fp32 [Hq] tensor")
        a.inv_tau = inv_tau.data_ptr()
    a.sm_scale = float(sm_scale)
    a.stages = int(stages)
    # packed INT4, groups of >= 32 channels: 0 = library default (factored scales), 1 = factored scales, 2 = bit-faithful
    # fp16 dequantisation; KVQ_INT4_FAST=1 / 0 picks one for calls that do not say
    if fast_dequant is None:
        env = os.environ.get("KVQ_INT4_FAST")
        a.fast_dequant = 0 if env is None else (1 if env == "1" else 2)
    else:
        a.fast_dequant = 1 if fast_dequant else 2
    if q_chan_scale is not None:       # fp32 [B, Hkv, D]: per-channel factor applied to the query inside the kernel
        if q_chan_scale.dtype != torch.float32 or tuple(q_chan_scale.shape) != (B, Hkv, D) or q_chan_scale.stride(-1) != 1:
            raise ValueError("q_chan_scale must be an fp32 [B, Hkv, D] tensor, contiguous in head_dim")
        a.q_chan_scale = q_chan_scale.data_ptr()
        a.qcs_stride_b, a.qcs_stride_h = q_chan_scale.stride(0), q_chan_scale.stride(1)
    a.tail_tokens = int(tail_tokens)   # 1: the last token of each row is attended by the combine stage (see kvq.h)
    a.k = _cache_side(k_payload, k_scale, k_zp, k_side)
    a.v = _cache_side(v_payload, v_scale, v_zp, v_side)
    if outlier_idx is not None:
        a.n_out = outlier_idx.shape[1]
        a.outlier_idx = outlier_idx.data_ptr()
    if context_lens is not None:        # None: every row attends over all max_ctx tokens of the view
        if context_lens.dtype != torch.int32 or not context_lens.is_contiguous():
            context_lens = context_lens.to(torch.int32).contiguous()
        a.context_lens = context_lens.data_ptr()
    lib = _lib.load()
    with torch.cuda.device(dev):
        a.splits = int(splits) if splits else int(lib.kvq_decode_pick_splits(C.byref(a)))
        global _LAST_SPLITS
        _LAST_SPLITS = a.splits
        need = int(lib.kvq_decode_workspace_bytes(B, Hq, D, a.splits))
        ws = get_workspace(dev, need)
        a.workspace = ws.data_ptr()
        a.workspace_bytes = ws.numel()
        if out is None:
            out = torch.empty((B, Hq, D), dtype=torch.float16, device=dev)
        a.out = out.data_ptr()
        a.out_stride_b, a.out_stride_h = out.stride(0), out.stride(1)
        part = None
        if return_partial:
            po = torch.empty((B, Hq, D), dtype=torch.float32, device=dev)
            pm = torch.empty((B, Hq), dtype=torch.float32, device=dev)
            pl = torch.empty((B, Hq), dtype=torch.float32, device=dev)
            a.part_o, a.part_m, a.part_l = po.data_ptr(), pm.data_ptr(), pl.data_ptr()
            part = (po, pm, pl)
        elif packed_partial is not None:
            pp = packed_partial
            if pp.dtype != torch.float32 or not pp.is_contiguous() or tuple(pp.shape) != (B, Hq, D + 2):
                raise ValueError("packed_partial must be a contiguous fp32 [B, Hq, D+2] tensor")
            a.part_o, a.part_m, a.part_l = pp.data_ptr(), pp.data_ptr() + 4 * D, pp.data_ptr() + 4 * (D + 1)
            a.part_o_stride = a.part_ml_stride = D + 2
            part = (pp[..., :D], pp[..., D], pp[..., D + 1])
        if exchange is not None:
            if return_partial or packed_partial is not None or not (B > 0 and a.max_ctx > 0):
                raise ValueError("exchange needs a non-empty local chunk and no partial outputs")
            rc = 0
            if a.stages != 2:
                a.stages = 1
                rc = lib.kvq_decode_attn(C.byref(a), _stream_ptr(dev))
            if rc == 0 and int(stages) != 1:
                combine_exchange(exchange["peer_ptrs"], exchange["rank"], exchange["slot"], exchange["slots"],
                                 exchange["epoch"], out, splits=a.splits, status=exchange.get("status"),
                                 wait_ns=exchange.get("wait_ns", 0), tail_attn=a if a.tail_tokens else None)
        elif B > 0 and a.max_ctx > 0:
            rc = lib.kvq_decode_attn(C.byref(a), _stream_ptr(dev))
        else:
            # nothing cached (an empty sequence shard): zeros, and the neutral partial (l = 0, m = -inf)
            rc = 0
            out.zero_()
            if part is not None:
                part[0].zero_(); part[1].fill_(float("-inf")); part[2].zero_()
    _lib.check("kvq_decode_attn", rc)
    if return_partial:
        return out, part
    return out


def group_absmax(x: torch.Tensor, group_size: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 [H, G] table of max |x| per (head, channel group) over batch rows and tokens of `x`
    ([B,H,S,D] or [H,S,D] fp16); max-accumulates into `out` when given (zero-filled by the caller)."""
    dev = _require_cuda(x)
    if x.dtype != torch.float16:
        raise ValueError("group_absmax expects an fp16 tensor")
    if x.ndim == 3:
        x = x[None]
    if x.ndim != 4 or x.stride(-1) != 1:
        raise ValueError("expected [B,H,S,D] (or [H,S,D]) with a contiguous last dimension")
    B, H, S, D = x.shape
    gs = D if group_size == -1 else int(group_size)
    if gs <= 0 or D % gs != 0:
        raise ValueError(f"head_dim ({D}) must be divisible by group_size ({group_size})")
    if out is None:
        out = torch.zeros((H, D // gs), dtype=torch.float32, device=dev)
    elif out.dtype != torch.float32 or tuple(out.shape) != (H, D // gs) or not out.is_contiguous():
        raise ValueError("out must be a contiguous fp32 [H, G] tensor")
    a = _lib.KvqAbsmaxArgs()
    a.B, a.H, a.S, a.D, a.group_size = B, H, S, D, gs
    a.x = x.data_ptr()
    a.stride_b, a.stride_h, a.stride_s = x.stride(0), x.stride(1), x.stride(2)
    a.out = out.data_ptr()
    with torch.cuda.device(dev):
        rc = _lib.load().kvq_group_absmax(C.byref(a), _stream_ptr(dev))
    _lib.check("kvq_group_absmax", rc)
    return out


def neutral_partial(B: int, Hq: int, D: int, dev) -> None:
    """Fill the split-K workspace with ONE empty split per (batch, head) row (o = 0, m = -inf, l = 0):
    what a rank without cached tokens hands to `combine_exchange`."""
    need = int(_lib.load().kvq_decode_workspace_bytes(B, Hq, D, 1))
    ws = get_workspace(torch.device(dev), need)
    o_bytes = (B * Hq * D * 4 + 255) & ~255
    ws[:o_bytes].zero_()
    ml = ws[o_bytes:o_bytes + B * Hq * 8].view(torch.float32).view(B * Hq, 2)
    ml[:, 0] = float("-inf")
    ml[:, 1] = 0.0


def exchange_bytes(B: int, Hq: int, D: int, slots: int, world: int) -> int:
    """Bytes of one rank's receive buffer of the fused exchange."""
    return int(_lib.load().kvq_exchange_bytes(B, Hq, D, slots, world))


def combine_exchange(peer_ptrs, rank: int, slot: int, slots: int, epoch: torch.Tensor, out: torch.Tensor, *,
                     splits: int, status: Optional[torch.Tensor] = None, wait_ns: int = 0,
                     tail_attn=None) -> torch.Tensor:
    """Second half of a sequence-sharded decode_attn(..., stages=1) call on this rank: merge the KV
    splits left in the workspace, exchange the normalised partial with every peer by direct stores
    into their receive buffers (`peer_ptrs[q]` = rank q's buffer mapped into this process), wait for
    theirs and write the merged fp16 `out` [B,Hq,D].  One launch; `epoch` is a device int32 >= 1."""
    dev = _require_cuda(out, epoch)
    B, Hq, D = out.shape
    world = len(peer_ptrs)
    if out.dtype != torch.float16 or out.stride(-1) != 1:
        raise ValueError("out must be an fp16 [B,Hq,D] tensor, contiguous in head_dim")
    if epoch.dtype != torch.int32 or (status is not None and status.dtype != torch.int32):
        raise ValueError("epoch / status must be int32 device tensors")
    x = _lib.KvqExchangeArgs()
    x.B, x.Hq, x.D, x.splits = B, Hq, D, int(splits)
    need = int(_lib.load().kvq_decode_workspace_bytes(B, Hq, D, x.splits))
    ws = get_workspace(dev, need)
    x.workspace, x.workspace_bytes = ws.data_ptr(), ws.numel()
    x.rank, x.world = int(rank), world
    arr = (C.c_void_p * world)(*[int(p) for p in peer_ptrs])
    x.peer_base = C.cast(arr, C.POINTER(C.c_void_p))
    x.slot, x.slots = int(slot), int(slots)
    x.epoch = epoch.data_ptr()
    x.wait_ns = int(wait_ns)
    x.status = status.data_ptr() if status is not None else None
    x.out = out.data_ptr()
    x.out_stride_b, x.out_stride_h = out.stride(0), out.stride(1)
    if tail_attn is not None:          # the KvqAttnArgs of the stage-1 call (tail_tokens = 1)
        x.tail_attn = C.pointer(tail_attn)
    with torch.cuda.device(dev):
        rc = _lib.load().kvq_combine_exchange(C.byref(x), _stream_ptr(dev))
    _lib.check("kvq_combine_exchange", rc)
    return out


def dequantize(fmt: int, k_payload: torch.Tensor, v_payload: Optional[torch.Tensor], k_scale: torch.Tensor,
               v_scale: Optional[torch.Tensor], *, k_zp=None, v_zp=None, outlier_idx=None, k_side=None, v_side=None):
    """Quantized cache views -> fp16 [B,Hkv,S,D] (K and V in one launch; V optional).
    Values are RN16(code * scale) (+ zero-point, rounded again); outlier channels take the side value."""
    dev = _require_cuda(k_payload, v_payload, k_scale, v_scale)
    if k_payload.dtype != torch.int8 or k_scale.dtype != torch.float16:
        raise ValueError("dequantize expects an int8 payload and fp16 scales")
    B, H, S, Dp = k_payload.shape
    D = Dp * 2 if fmt == _lib.FMT_INT4 else Dp
    a = _lib.KvqDequantArgs()
    a.format, a.B, a.Hkv, a.S, a.D = fmt, B, H, S, D
    a.group_size = D // k_scale.shape[-1]
    if k_payload.stride(-1) != 1 or (v_payload is not None and v_payload.stride(-1) != 1):
        raise ValueError("payload last dimension must be contiguous")
    a.k = _cache_side(k_payload, k_scale, k_zp, k_side)
    k_out = torch.empty((B, H, S, D), dtype=torch.float16, device=dev)
    a.k_out = k_out.data_ptr()
    v_out = None
    if v_payload is not None:
        if v_payload.shape != k_payload.shape:
            raise ValueError("k / v payload shapes differ")
        a.v = _cache_side(v_payload, v_scale, v_zp, v_side)
        v_out = torch.empty_like(k_out)
        a.v_out = v_out.data_ptr()
    a.out_stride_b, a.out_stride_h, a.out_stride_s = k_out.stride(0), k_out.stride(1), k_out.stride(2)
    if outlier_idx is not None:
        if outlier_idx.dtype != torch.int16 or not outlier_idx.is_contiguous() or outlier_idx.shape[0] != H:
            raise ValueError("outlier_idx must be a contiguous int16 [Hkv, n_out] tensor")
        a.n_out = outlier_idx.shape[1]
        a.outlier_idx = outlier_idx.data_ptr()
    with torch.cuda.device(dev):
        rc = _lib.load().kvq_dequantize(C.byref(a), _stream_ptr(dev))
    _lib.check("kvq_dequantize", rc)
    return k_out, v_out


def decode_kernel_kind(fmt: int, q, k_payload, v_payload, k_scale, v_scale, *, k_zp=None, v_zp=None,
                       n_out: int = 0) -> int:
    """Which kernel kvq_decode_attn would launch for these tensors: 1 = tensor-core TMA kernel,
    0 = generic kernel.  Pure host-side query (no launch)."""
    a = _lib.KvqAttnArgs()
    B, Hq, D = q.shape
    a.format, a.B, a.Hq, a.Hkv, a.D = fmt, B, Hq, k_payload.shape[1], D
    a.group_size = D // (1 if k_scale is None else k_scale.shape[-1])
    a.max_ctx = k_payload.shape[2]
    a.q, a.q_stride_b, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    a.k = _cache_side(k_payload, k_scale, k_zp, None)
    a.v = _cache_side(v_payload, v_scale, v_zp, None)
    a.n_out = n_out
    return int(_lib.load().kvq_decode_kernel_kind(C.byref(a)))


def lse_combine(part_o: torch.Tensor, part_m: torch.Tensor, part_l: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Merge P normalised partials ([P,B,Hq,D], [P,B,Hq], [P,B,Hq] fp32) -> fp16 [B,Hq,D]."""
    dev = _require_cuda(part_o, part_m, part_l)
    P, B, Hq, D = part_o.shape
    for t in (part_o, part_m, part_l):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError("partials must be contiguous fp32 tensors")
    if out is None:
        out = torch.empty((B, Hq, D), dtype=torch.float16, device=dev)
    c = _lib.KvqCombineArgs()
    c.P, c.B, c.Hq, c.D = P, B, Hq, D
    c.part_o, c.part_m, c.part_l = part_o.data_ptr(), part_m.data_ptr(), part_l.data_ptr()
    c.out = out.data_ptr()
    c.out_stride_b, c.out_stride_h = out.stride(0), out.stride(1)
    with torch.cuda.device(dev):
        rc = _lib.load().kvq_lse_combine(C.byref(c), _stream_ptr(dev))
    _lib.check("kvq_lse_combine", rc)
    return out


def lse_combine_packed(packed: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Merge P packed partials (fp32 [P,B,Hq,D+2], rows `[o (D) | m | l]`, e.g. the receive buffer
    of an all-gather) -> fp16 [B,Hq,D]."""
    dev = _require_cuda(packed)
    if packed.dtype != torch.float32 or not packed.is_contiguous() or packed.ndim != 4:
        raise ValueError("packed partials must be a contiguous fp32 [P, B, Hq, D+2] tensor")
    P, B, Hq, W = packed.shape
    D = W - 2
    if out is None:
        out = torch.empty((B, Hq, D), dtype=torch.float16, device=dev)
    c = _lib.KvqCombineArgs()
    c.P, c.B, c.Hq, c.D = P, B, Hq, D
    base = packed.data_ptr()
    c.part_o, c.part_m, c.part_l = base, base + 4 * D, base + 4 * (D + 1)
    c.part_o_stride = c.part_ml_stride = W
    c.part_o_stride_p = c.part_ml_stride_p = B * Hq * W
    c.out = out.data_ptr()
    c.out_stride_b, c.out_stride_h = out.stride(0), out.stride(1)
    with torch.cuda.device(dev):
        rc = _lib.load().kvq_lse_combine(C.byref(c), _stream_ptr(dev))
    _lib.check("kvq_lse_combine", rc)
    return out


def decode_attn_static(fmt: int, q: torch.Tensor, k_payload: torch.Tensor, v_payload: torch.Tensor,
                       k_scale: Optional[torch.Tensor], v_scale: Optional[torch.Tensor],
                       context_lens: Optional[torch.Tensor], sm_scale: float, out: torch.Tensor, *,
                       k_zp=None, v_zp=None, inv_tau: Optional[torch.Tensor] = None,
                       outlier_idx=None, k_side=None, v_side=None, splits: int = 0) -> torch.Tensor:
    """Fused decode attention through `kvq_decode_attn_static`, the entry point for hosts that are
    not allowed to allocate GPU memory at call time (for instance a serving process whose memory
    pool already owns all of HBM).  The split-K partials go to an 8 MiB array inside the library
    instead of a torch-allocated workspace, and this wrapper allocates nothing either: the caller
    passes `out` (fp16 [B,Hq,D]).

    Raises `KvqError` with code `KVQ_ELIMIT` when B*Hq*splits*(D+2)*4 bytes exceed the array.
    Calls on one device share that array: keep them on one stream (overlapping calls race).
    The first call per device resolves the array's address; do it before capturing a CUDA graph.
    """
    dev = _require_cuda(q, k_payload, v_payload, k_scale, v_scale, context_lens, out)
    if q.dtype != torch.float16 or out.dtype != torch.float16:
        raise ValueError("decode_attn_static expects fp16 q and out")
    if q.stride(-1) != 1 or out.stride(-1) != 1:
        raise ValueError("q and out must be contiguous in head_dim")
    B, Hq, D = q.shape
    a = _lib.KvqAttnArgs()
    a.format = fmt
    a.B, a.Hq, a.Hkv, a.D = B, Hq, k_payload.shape[1], D
    a.group_size = D // (1 if k_scale is None else k_scale.shape[-1])
    a.max_ctx = k_payload.shape[2]
    a.q, a.q_stride_b, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    if inv_tau is not None:
        a.inv_tau = inv_tau.data_ptr()
    a.sm_scale = float(sm_scale)
    a.k = _cache_side(k_payload, k_scale, k_zp, k_side)
    a.v = _cache_side(v_payload, v_scale, v_zp, v_side)
    if outlier_idx is not None:
        a.n_out = outlier_idx.shape[1]
        a.outlier_idx = outlier_idx.data_ptr()
    if context_lens is not None:
        if context_lens.dtype != torch.int32 or not context_lens.is_contiguous():
            raise ValueError("context_lens must be a contiguous int32 tensor (no conversion is done here)")
        a.context_lens = context_lens.data_ptr()
    a.splits = int(splits)
    a.out, a.out_stride_b, a.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    with torch.cuda.device(dev):
        rc = _lib.load().kvq_decode_attn_static(C.byref(a), _stream_ptr(dev))
    _lib.check("kvq_decode_attn_static", rc)
    return out
