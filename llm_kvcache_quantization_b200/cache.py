"""KV caches with quantize-on-append, API-compatible with the reference's
`INT8KVCache`, `INT4KVCache` and `FP16KVCache`
(src/cache/int8_cache.py:29-682, src/cache/int4_cache.py:32-773,
 src/cache/fp16_cache.py:26-370, src/cache/protocol.py:30-63).

What is the same: constructor arguments, `append / get_kv / get_int8_tensors /
get_int4_tensors / get_seq_len / clear / release / get_memory_mb / to_tuple /
from_tuple`, the decode-stat counters, the growth policy (first allocation
`max(target, 256)`, then doubling, capped by `max_seq_len`), the exceptions, and
the stored codes / packed bytes, which are bit-identical.

What is different, on purpose:
* `append` is ONE kernel launch for K and V (scale policy, quantization, nibble
  packing and the slot write fused) instead of ~30 eager ops and host syncs.
* Scales are stored in fp16 - the value the decode kernel and the torch reference
  consume (`scale.to(float16)`, src/engine/patch_model.py:909-917, 927-933) - so
  the per-call cast disappears and scale traffic halves.  `keep_fp32_scales=True`
  keeps the reference's fp32 copy as well (`get_fp32_scales`).
* The clip-ratio warnings (ENG-040 / KVC-021) and the NaN/Inf guard each need a
  host sync per append; they run only with `validate_inputs=True` (or `KVQ_VALIDATE=1`).
* Two formats the reference lacks: group-wise asymmetric INT4 (`asymmetric=True`)
  and an fp16 outlier-channel side buffer (`outlier_idx=`).
"""
from __future__ import annotations

import logging
import os
import warnings
from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor

from . import ops, quant
from ._lib import (FMT_FP16, FMT_INT4, FMT_INT8, F_ADAPTIVE, F_ADAPT_SKIP_K, F_ADAPT_SKIP_V, F_MIXED_RESCUE, F_RESCUE_THR,
                   F_UNPACKED,
                   SCALE_ASYM_MINMAX, SCALE_DYNAMIC_PCT, SCALE_STATIC)

logger = logging.getLogger(__name__)
_CLIP_WARN_THRESHOLD = 0.01


def _new_stats() -> Dict[str, object]:
    return {"fused_decode_calls": 0, "triton_kernel_calls": 0, "triton_decode_calls": 0,
            "torch_ref_calls": 0, "layer_hits": {}, "triton_layer_hits": {}}


class _CacheBase:
    """Storage, growth and bookkeeping shared by the three caches."""

    _fmt = FMT_INT8
    _qmax = 127.0

    def __init__(self, num_layers: int, device="cuda", dtype: torch.dtype = torch.float16,
                 max_seq_len: Optional[int] = None):
        if num_layers <= 0:
            raise ValueError(f"num_layers must be > 0, got {num_layers}")
        self.num_layers = num_layers
        self.device = device
        self.dtype = dtype
        self.max_seq_len = int(max_seq_len) if max_seq_len is not None else None
        if self.max_seq_len is not None and self.max_seq_len <= 0:
            raise ValueError(f"max_seq_len must be > 0, got {self.max_seq_len}")
        self._min_capacity = 256
        self._bufs: List[Optional[Dict[str, Tensor]]] = [None] * num_layers
        self._layer_seq_lens: List[int] = [0] * num_layers
        self._dev_positions = None
        self._layer_capacity: List[int] = [0] * num_layers
        self._seq_len = 0
        self.decode_stats: Dict[str, object] = _new_stats()

    # ---- decode statistics (key names are read by the reference's callers/tests)
    def _bump_counter(self, key: str, delta: int = 1) -> None:
        self.decode_stats[key] = int(self.decode_stats.get(key, 0)) + int(delta)

    def record_fused_decode(self, layer_id: int, decode_impl: str) -> None:
        self._bump_counter("fused_decode_calls", 1)
        if decode_impl == "triton_fused":
            self._bump_counter("triton_decode_calls", 1)
        elif decode_impl == "torch_ref":
            self._bump_counter("torch_ref_calls", 1)
        hits = self.decode_stats.setdefault("layer_hits", {})
        hits[str(layer_id)] = int(hits.get(str(layer_id), 0)) + 1

    def record_triton_kernel_call(self, layer_id: Optional[int] = None) -> None:
        self._bump_counter("triton_kernel_calls", 1)
        if layer_id is None:
            return
        hits = self.decode_stats.setdefault("triton_layer_hits", {})
        hits[str(layer_id)] = int(hits.get(str(layer_id), 0)) + 1

    def reset_decode_stats(self) -> None:
        self.decode_stats = _new_stats()

    def get_decode_stats(self) -> Dict[str, object]:
        s = self.decode_stats
        return {k: (dict(s.get(k, {})) if k.endswith("hits") else int(s.get(k, 0))) for k in _new_stats()}

    # ---- storage
    def _buffer_specs(self, batch, heads, head_dim) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        raise NotImplementedError

    def _alloc(self, specs, capacity) -> Dict[str, Tensor]:
        out = {}
        for name, (tail, dt) in specs.items():
            b, h, w = tail
            out[name] = torch.empty((b, h, capacity, w), device=self.device, dtype=dt)
        return out

    def _ensure_capacity(self, layer_id: int, batch: int, heads: int, head_dim: int, target_len: int) -> None:
        if self.max_seq_len is not None and target_len > self.max_seq_len:
            raise ValueError(
                f"target_len {target_len} exceeds max_seq_len {self.max_seq_len} for layer {layer_id}")
        specs = self._buffer_specs(batch, heads, head_dim)
        bufs = self._bufs[layer_id]
        capacity = self._layer_capacity[layer_id]
        if bufs is not None:
            for name, (tail, _) in specs.items():
                t = bufs[name]
                if (t.shape[0], t.shape[1], t.shape[3]) != tail:
                    raise ValueError(
                        f"Inconsistent KV shape for layer {layer_id}: existing {name}={tuple(t.shape)}, "
                        f"incoming=({batch}, {heads}, *, {head_dim})")
            if target_len <= capacity:
                return
            new_capacity = max(target_len, capacity * 2)
        else:
            new_capacity = max(target_len, self._min_capacity)
        if self.max_seq_len is not None:
            new_capacity = min(new_capacity, self.max_seq_len)
            if new_capacity < target_len:
                raise ValueError(
                    f"target_len {target_len} exceeds capped capacity {new_capacity} for layer {layer_id}")
        # physical slots are rounded up to 32 tokens so that every (batch, head) row of every
        # buffer starts 16-byte aligned (the tensor-core decode kernel copies 16-byte units)
        new = self._alloc(specs, (new_capacity + 31) // 32 * 32)     # an OOM here leaves the layer untouched
        old_len = self._layer_seq_lens[layer_id]
        if bufs is not None and old_len > 0:
            for name in new:
                new[name][:, :, :old_len] = bufs[name][:, :, :old_len]
        self._bufs[layer_id] = new
        self._layer_capacity[layer_id] = new_capacity

    def reserve(self, layer_id: int, batch: int, heads: int, head_dim: int, capacity: int) -> None:
        """Preallocate `capacity` slots so that later appends never reallocate
        (views handed to the decode kernel stay valid; required for CUDA graphs)."""
        self._ensure_capacity(layer_id, batch, heads, head_dim, capacity)

    def _check_append(self, layer_id: int, k: Tensor, v: Tensor) -> None:
        if layer_id < 0 or layer_id >= self.num_layers:
            raise ValueError(f"layer_id {layer_id} out of range")
        if k.ndim != 4:
            raise ValueError(f"k must be 4D [B,H,S,D], got ndim={k.ndim}")
        if v.ndim != 4:
            raise ValueError(f"v must be 4D [B,H,S,D], got ndim={v.ndim}")
        if tuple(k.shape) != tuple(v.shape):
            raise ValueError(f"k/v shape mismatch: k={tuple(k.shape)} vs v={tuple(v.shape)}")
        target = torch.device(self.device)
        if k.device.type != target.type or v.device.type != target.type:
            raise ValueError(f"Device mismatch: cache_device={target}, k.device={k.device}, v.device={v.device}")
        if not k.is_cuda:
            raise ValueError("this cache quantizes with a CUDA kernel; CPU tensors are not supported")

    def _layer_view(self, layer_id: int, names) -> Tuple[Tensor, ...]:
        if layer_id < 0 or layer_id >= self.num_layers:
            raise ValueError(f"layer_id {layer_id} out of range [0, {self.num_layers})")
        bufs = self._bufs[layer_id]
        if bufs is None:
            raise ValueError(f"Cache for layer {layer_id} is empty")
        n = self._layer_seq_lens[layer_id] if self._dev_positions is None else self._dev_positions[2]
        return tuple(bufs[name][:, :, :n] for name in names)

    def _finish_append(self, layer_id: int, target_len: int) -> None:
        if self._dev_positions is not None:
            return                                   # lengths live on the device; advance_host_lengths() follows
        self._layer_seq_lens[layer_id] = target_len
        if layer_id == 0:
            self._seq_len = target_len

    # ---- device-side positions: what a captured (CUDA-graph) decode step needs.  While this mode is on,
    # single-token appends write at `*pos` (int32 device scalar), fused_decode attends over `ctx` (int32 [B]
    # device tensor) inside views of the first `capacity` slots, and nothing here touches host-side lengths.
    def use_device_positions(self, pos: Tensor, ctx: Tensor, capacity: int) -> None:
        if pos.dtype != torch.int32 or ctx.dtype != torch.int32 or not pos.is_cuda or not ctx.is_cuda:
            raise ValueError("pos / ctx must be int32 CUDA tensors")
        for l in range(self.num_layers):
            if self._bufs[l] is None or self._bufs[l]["k"].shape[2] < capacity:
                raise ValueError(f"reserve at least {capacity} slots in layer {l} before switching to device positions")
        self._dev_positions = (pos, ctx, int(capacity))

    def use_host_positions(self) -> None:
        self._dev_positions = None

    def advance_host_lengths(self, tokens: int = 1) -> None:
        """Bring the host-side lengths in line after `tokens` replays of a captured step."""
        for l in range(self.num_layers):
            self._layer_seq_lens[l] += tokens
        self._seq_len = self._layer_seq_lens[0]

    def _write_slot(self, layer_id: int, batch: int, heads: int, head_dim: int, tokens: int):
        """(first slot to write - an int, or the device scalar -, host length before the append)."""
        old = self._layer_seq_lens[layer_id]
        if self._dev_positions is None:
            self._ensure_capacity(layer_id, batch, heads, head_dim, old + tokens)
            return old, old
        if tokens != 1:
            raise ValueError("device-side positions serve single-token appends")
        return self._dev_positions[0], old

    @staticmethod
    def _rope_tables(cos: Tensor, sin: Tensor, batch: int, tokens: int, device):
        """cos / sin of rank 2-4 (as HF hands them to the attention module) -> fp16 [B or 1, T, rotary_dim]."""
        out = []
        for t in (cos, sin):
            if t.ndim > 4:
                raise ValueError(f"Unexpected cos/sin rank {t.ndim}; expected 2-4.")
            if t.ndim == 4:
                t = t[:, 0]
            if t.ndim == 2:
                t = t[None]
            if t.shape[0] not in (1, batch) or t.shape[1] != tokens:
                raise ValueError(f"cos/sin shape {tuple(t.shape)} does not match batch {batch}, tokens {tokens}")
            out.append(t.to(device=device, dtype=torch.float16).contiguous())
        return out[0], out[1]

    def supports_fused_rope(self) -> bool:
        """True when append_rotary can rotate inside the quantizer launch."""
        return True

    def append_rotary(self, layer_id: int, q: Tensor, k: Tensor, v: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        """Rotate q and k (rotate-half RoPE, the arithmetic of src/engine/patch_model.py:223-278),
        append k (rotated) and v, all in ONE launch; returns the rotated q [B,Hq,T,D] fp16."""
        raise NotImplementedError

    def get_seq_len(self) -> int:
        return self._seq_len

    def clear(self) -> None:
        """Reset lengths, keep the buffers."""
        self._layer_seq_lens = [0] * self.num_layers
        self._seq_len = 0

    def release(self) -> None:
        self._bufs = [None] * self.num_layers
        self._layer_seq_lens = [0] * self.num_layers
        self._layer_capacity = [0] * self.num_layers
        self._seq_len = 0

    def get_memory_mb(self) -> float:
        total = 0
        for bufs in self._bufs:
            if bufs is not None:
                total += sum(t.numel() * t.element_size() for t in bufs.values())
        return total / (1024 * 1024)

    def to_tuple(self) -> Tuple[Tuple[Tensor, Tensor], ...]:
        out = []
        for i in range(self.num_layers):
            if self._bufs[i] is None:
                raise ValueError(f"Layer {i} cache is empty")
            out.append(self.get_kv(i))
        return tuple(out)

    def __repr__(self) -> str:
        return (f"{type(self).__name__}(num_layers={self.num_layers}, seq_len={self._seq_len}, "
                f"memory={self.get_memory_mb():.2f}MB)")


class FP16KVCache(_CacheBase):
    """Unquantized cache (src/cache/fp16_cache.py:26-370) with the same slot-write kernel."""

    _fmt = FMT_FP16

    def __init__(self, num_layers: int, device="cuda", dtype: torch.dtype = torch.float16,
                 max_seq_len: Optional[int] = None):
        super().__init__(num_layers, device, dtype, max_seq_len)

    def _buffer_specs(self, batch, heads, head_dim):
        return {"k": ((batch, heads, head_dim), torch.float16), "v": ((batch, heads, head_dim), torch.float16)}

    def append(self, layer_id: int, k: Tensor, v: Tensor) -> None:
        self._check_append(layer_id, k, v)
        B, H, T, D = k.shape
        slot, old = self._write_slot(layer_id, B, H, D, T)
        bufs = self._bufs[layer_id]
        ops.quantize_append(FMT_FP16, SCALE_STATIC, k.to(torch.float16), v.to(torch.float16),
                            bufs["k"], bufs["v"], None, None, slot, D)
        self._finish_append(layer_id, old + T)

    def append_rotary(self, layer_id: int, q: Tensor, k: Tensor, v: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        self._check_append(layer_id, k, v)
        B, H, T, D = k.shape
        slot, old = self._write_slot(layer_id, B, H, D, T)
        bufs = self._bufs[layer_id]
        c16, s16 = self._rope_tables(cos, sin, B, T, k.device)
        q_rot = ops.quantize_append(FMT_FP16, SCALE_STATIC, k.to(torch.float16), v.to(torch.float16),
                                    bufs["k"], bufs["v"], None, None, slot, D, rope_cos=c16, rope_sin=s16,
                                    q=q.to(torch.float16))
        self._finish_append(layer_id, old + T)
        return q_rot

    def get_kv(self, layer_id: int) -> Tuple[Tensor, Tensor]:
        k, v = self._layer_view(layer_id, ("k", "v"))
        return k.to(self.dtype), v.to(self.dtype)

    def get_fp16_tensors(self, layer_id: int) -> Tuple[Tensor, Tensor]:
        return self._layer_view(layer_id, ("k", "v"))

    def fused_decode(self, layer_id: int, q: Tensor, sm_scale: float, inv_tau: Optional[Tensor] = None,
                     out: Optional[Tensor] = None) -> Tensor:
        """q_len==1 attention over the cached fp16 K/V of this layer through the split-K kernel."""
        k, v = self.get_fp16_tensors(layer_id)
        original = q.dtype
        if original != torch.float16:
            q = q.to(torch.float16)
        ctx = None if self._dev_positions is None else self._dev_positions[1]
        res = ops.decode_attn(FMT_FP16, q, k, v, None, None, ctx, float(sm_scale), head_dim=q.shape[-1],
                              inv_tau=None if inv_tau is None else inv_tau.float(), out=out)
        return res if original == torch.float16 else res.to(original)

    @classmethod
    def from_tuple(cls, past_key_values, device="cuda") -> "FP16KVCache":
        cache = cls(num_layers=len(past_key_values), device=device)
        for i, item in enumerate(past_key_values):
            cache.append(i, item[0].to(device), item[1].to(device))
        return cache


class _QuantCache(_CacheBase):
    """Common part of the INT8 and INT4 caches: scale policy selection and the fused append."""

    def __init__(self, num_layers, device, clip_percentile, group_size, dtype, max_seq_len,
                 decode_attn_impl, static_k_scale, static_v_scale, inv_tau, use_attn_temperature,
                 adaptive_static_scales, adaptive_static_margin, adaptive_static_k, adaptive_static_v,
                 keep_fp32_scales, validate_inputs):
        super().__init__(num_layers, device, dtype, max_seq_len)
        if adaptive_static_margin <= 0:
            raise ValueError(f"adaptive_static_margin must be > 0, got {adaptive_static_margin}")
        self.clip_percentile = clip_percentile
        self.group_size = group_size
        self.decode_attn_impl = decode_attn_impl
        self.static_k_scale = static_k_scale
        self.static_v_scale = static_v_scale
        self.inv_tau = inv_tau
        self.use_attn_temperature = use_attn_temperature
        self.adaptive_static_scales = adaptive_static_scales
        self.adaptive_static_margin = adaptive_static_margin
        self.adaptive_static_k = adaptive_static_k
        self.adaptive_static_v = adaptive_static_v
        self.keep_fp32_scales = bool(keep_fp32_scales)
        self.validate_inputs = bool(validate_inputs) or os.environ.get("KVQ_VALIDATE", "0") == "1"
        self.asymmetric = False
        self.outlier_idx = None          # int16 [L, Hkv, n_out] or None
        self._scale_dtype = torch.float16
        self._static_tables: Dict[Tuple[str, int], Tensor] = {}

    # payload width in bytes for head_dim D
    def _payload_dim(self, head_dim: int) -> int:
        return head_dim

    def _num_groups(self, head_dim: int) -> int:
        gs = head_dim if self.group_size == -1 else self.group_size
        if gs <= 0 or head_dim % gs != 0:
            raise ValueError(f"head_dim {head_dim} must be divisible by group_size {self.group_size}")
        return head_dim // gs

    def _buffer_specs(self, batch, heads, head_dim):
        G = self._num_groups(head_dim)
        dp = self._payload_dim(head_dim)
        specs = {"k": ((batch, heads, dp), torch.int8), "v": ((batch, heads, dp), torch.int8),
                 "ks": ((batch, heads, G), torch.float16), "vs": ((batch, heads, G), torch.float16)}
        if self.keep_fp32_scales:
            specs["ks32"] = ((batch, heads, G), torch.float32)
            specs["vs32"] = ((batch, heads, G), torch.float32)
        if self.asymmetric:
            specs["kz"] = ((batch, heads, G), torch.float16)
            specs["vz"] = ((batch, heads, G), torch.float16)
        if self.outlier_idx is not None:
            n_out = int(self.outlier_idx.shape[-1])
            specs["kside"] = ((batch, heads, n_out), torch.float16)
            specs["vside"] = ((batch, heads, n_out), torch.float16)
        return specs

    def _static_table(self, which: str, layer_id: int, heads: int, G: int, device) -> Tensor:
        """The calibrated [Hkv, G] table of one layer on the right device, validated once."""
        key = (which, layer_id)
        tab = self._static_tables.get(key)
        if tab is None:
            src = self.static_k_scale if which == "k" else self.static_v_scale
            tab = src[layer_id]
            if not isinstance(tab, Tensor):
                tab = torch.as_tensor(tab)
            if tab.ndim == 5 and tab.shape[-1] == 1:
                tab = tab[..., 0]
            if tab.ndim == 3 and tab.shape[1] == 1:          # legacy [H,1,G]
                tab = tab[:, 0, :]
            elif tab.ndim == 3 and tab.shape[2] == 1:        # legacy [H,G,1]
                tab = tab[..., 0]
            elif tab.ndim == 3 and tab.shape[0] == 1:        # [1,H,G]
                tab = tab[0]
            elif tab.ndim == 4 and tab.shape[0] == 1 and tab.shape[2] == 1:   # [1,H,1,G]
                tab = tab[0, :, 0, :]
            if tab.ndim != 2:
                raise ValueError(f"Unsupported static scale shape: {tuple(tab.shape)}")
            if tab.shape[0] != heads:
                raise ValueError(
                    "_normalize_static_scale: calibration vs model heads mismatch "
                    "(fail-fast; wrong calibration file was loaded).\n"
                    f"  expected heads: {heads} (from model/cache config)\n"
                    f"  scale heads:    {tab.shape[0]} (from scale.shape={tuple(tab.shape)})\n"
                    f"  num_groups:     {G}\n  layer_id:       {layer_id}")
            if tab.shape[1] != G:
                raise ValueError(
                    f"static scale has {tab.shape[1]} groups but head_dim/group_size gives {G}")
            if tab.dtype not in (torch.float16, torch.float32):
                tab = tab.float()
            tab = tab.to(device).contiguous()
            self._static_tables[key] = tab
        return tab

    def _rescue_threshold(self, x: Tensor, G: int) -> Optional[Tensor]:
        return None

    def _append_impl(self, layer_id: int, k: Tensor, v: Tensor, extra_flags: int = 0, rope=None):
        """`rope = (q, cos, sin)`: rotate q and k inside the launch; returns the rotated q."""
        self._check_append(layer_id, k, v)
        for nm, sc in (("static_k_scale", self.static_k_scale), ("static_v_scale", self.static_v_scale)):
            if sc is not None and layer_id >= len(sc):
                raise IndexError(f"layer_id {layer_id} exceeds calibration layers {len(sc)} for {nm}")
        if (self.static_k_scale is None) != (self.static_v_scale is None) and not self.asymmetric:
            raise ValueError("static_k_scale and static_v_scale must be given together "
                             "(K and V are quantized by one fused launch)")
        if k.dtype != torch.float16:
            k, v = k.to(torch.float16), v.to(torch.float16)
        if self.validate_inputs:
            quant._check_quantize_input(k, "append(k)")
            quant._check_quantize_input(v, "append(v)")
        B, H, T, D = k.shape
        if rope is not None:
            if extra_flags & F_RESCUE_THR:
                raise ValueError("outlier_rescue_ratio in (0,1) needs a quantile of the rotated keys before the "
                                 "launch; rotate in torch and call append() instead")
            c16, s16 = self._rope_tables(rope[1], rope[2], B, T, k.device)
        G = self._num_groups(D)
        gs = D // G
        slot, old = self._write_slot(layer_id, B, H, D, T)
        bufs = self._bufs[layer_id]
        kw = dict(k_scale_f32=bufs.get("ks32"), v_scale_f32=bufs.get("vs32"))
        oidx = None
        if self.outlier_idx is not None:
            oidx = self.outlier_idx[layer_id].to(device=k.device, dtype=torch.int16).contiguous()
            kw.update(outlier_idx=oidx, k_side=bufs["kside"], v_side=bufs["vside"])
        flags = extra_flags & F_UNPACKED
        if self.asymmetric:
            policy = SCALE_ASYM_MINMAX
            kw.update(k_zp=bufs["kz"], v_zp=bufs["vz"])
        elif self.static_k_scale is not None:
            policy = SCALE_STATIC
            kw.update(k_static=self._static_table("k", layer_id, H, G, k.device),
                      v_static=self._static_table("v", layer_id, H, G, k.device))
            if self.adaptive_static_scales and (self.adaptive_static_k or self.adaptive_static_v):
                # the rule applies to K and V independently (src/cache/int8_cache.py:394, :427)
                flags |= F_ADAPTIVE
                if not self.adaptive_static_k:
                    flags |= F_ADAPT_SKIP_K
                if not self.adaptive_static_v:
                    flags |= F_ADAPT_SKIP_V
            flags |= extra_flags
            if flags & F_RESCUE_THR:
                kw.update(k_rescue_thr=self._rescue_threshold(k, G), v_rescue_thr=self._rescue_threshold(v, G))
        else:
            policy = SCALE_DYNAMIC_PCT
            p = float(self.clip_percentile)
            kw.update(quantile=(max(min(p / 100.0, 1.0), 0.0) if p < 100.0 else 1.0))
        if rope is not None:
            kw.update(rope_cos=c16, rope_sin=s16, q=rope[0].to(torch.float16))
        q_rot = ops.quantize_append(self._fmt, policy, k, v, bufs["k"], bufs["v"], bufs["ks"], bufs["vs"], slot, gs,
                                    flags=flags, adaptive_margin=float(self.adaptive_static_margin), **kw)
        self._finish_append(layer_id, old + T)
        if self.validate_inputs and policy == SCALE_STATIC and rope is None and self._dev_positions is None:
            self._warn_if_clipped(layer_id, k, v, old, T)
        return q_rot

    def _warn_if_clipped(self, layer_id, k, v, old, T) -> None:
        bufs = self._bufs[layer_id]
        for nm, x, code, sc in (("K", k, bufs["k"], bufs["ks"]), ("V", v, bufs["v"], bufs["vs"])):
            B, H, _, D = x.shape
            G = sc.shape[-1]
            bound = (sc[:, :, old:old + T].float() * self._qmax).unsqueeze(-1)
            ratio = float((x.float().view(B, H, T, G, D // G).abs() > bound * (1 + 2 ** -10)).float().mean())
            if ratio > _CLIP_WARN_THRESHOLD:
                warnings.warn(
                    f"Static {nm} scale overflow at layer {layer_id}: {ratio:.1%} of values exceed scale "
                    f"capacity (threshold={_CLIP_WARN_THRESHOLD:.0%}). Consider re-calibrating or enabling "
                    "adaptive_static_scales.", RuntimeWarning)

    def get_fp32_scales(self, layer_id: int) -> Tuple[Tensor, Tensor]:
        if not self.keep_fp32_scales:
            raise ValueError("construct the cache with keep_fp32_scales=True to keep fp32 scale copies")
        return self._layer_view(layer_id, ("ks32", "vs32"))

    def get_decode_tensors(self, layer_id: int) -> Dict[str, Optional[Tensor]]:
        """Everything the fused decode kernel reads for this layer, as views."""
        names = ["k", "v", "ks", "vs"]
        if self.asymmetric:
            names += ["kz", "vz"]
        if self.outlier_idx is not None:
            names += ["kside", "vside"]
        vals = dict(zip(names, self._layer_view(layer_id, names)))
        vals["outlier_idx"] = None if self.outlier_idx is None else self.outlier_idx[layer_id]
        return vals

    def fused_decode(self, layer_id: int, q: Tensor, sm_scale: float, inv_tau: Optional[Tensor] = None,
                     out: Optional[Tensor] = None) -> Tensor:
        """q_len==1 attention of `q` [B,Hq,D] over everything cached for this layer, in one fused
        call (format, zero-points, outlier side buffer and per-head `inv_tau` handled by the
        kernel).  All rows attend over the layer's full length (no host sync, no length tensor)."""
        t = self.get_decode_tensors(layer_id)
        original = q.dtype
        if original != torch.float16:
            q = q.to(torch.float16)
        extra = {}
        if self.asymmetric:
            extra.update(k_zp=t["kz"], v_zp=t["vz"])
        if self.outlier_idx is not None:
            extra.update(outlier_idx=t["outlier_idx"].to(q.device).contiguous(), k_side=t["kside"], v_side=t["vside"])
        if inv_tau is not None and inv_tau.dtype != torch.float32:
            inv_tau = inv_tau.float()
        ctx = None if self._dev_positions is None else self._dev_positions[1]
        res = ops.decode_attn(getattr(self, "_decode_fmt", self._fmt), q, t["k"], t["v"], t["ks"], t["vs"], ctx, float(sm_scale),
                              head_dim=q.shape[-1], inv_tau=inv_tau, out=out, **extra)
        return res if original == torch.float16 else res.to(original)

    def release(self) -> None:
        super().release()
        self.static_k_scale = None
        self.static_v_scale = None
        self.inv_tau = None
        self._static_tables.clear()


class INT8KVCache(_QuantCache):
    """INT8 symmetric group-wise cache (src/cache/int8_cache.py:29-682)."""

    _fmt = FMT_INT8
    _qmax = 127.0

    def __init__(self, num_layers: int, device="cuda", clip_percentile: float = 99.9, group_size: int = 128,
                 dtype: torch.dtype = torch.float16, max_seq_len: Optional[int] = None,
                 decode_attn_impl: str = "triton_fused", static_k_scale=None, static_v_scale=None,
                 inv_tau: Optional[Tensor] = None, use_attn_temperature: bool = True,
                 adaptive_static_scales: bool = False, adaptive_static_margin: float = 1.0,
                 adaptive_static_k: bool = True, adaptive_static_v: bool = True, *,
                 keep_fp32_scales: bool = False, validate_inputs: bool = False):
        super().__init__(num_layers, device, clip_percentile, group_size, dtype, max_seq_len, decode_attn_impl,
                         static_k_scale, static_v_scale, inv_tau, use_attn_temperature, adaptive_static_scales,
                         adaptive_static_margin, adaptive_static_k, adaptive_static_v, keep_fp32_scales,
                         validate_inputs)

    def append(self, layer_id: int, k: Tensor, v: Tensor) -> None:
        """Quantize and append (src/cache/int8_cache.py:350-488)."""
        self._append_impl(layer_id, k, v)

    def append_rotary(self, layer_id: int, q: Tensor, k: Tensor, v: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        return self._append_impl(layer_id, k, v, rope=(q, cos, sin))

    def get_int8_tensors(self, layer_id: int) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
        """(k_int8, v_int8, k_scale, v_scale) views of the valid tokens; scales are fp16."""
        return self._layer_view(layer_id, ("k", "v", "ks", "vs"))

    def get_kv(self, layer_id: int) -> Tuple[Tensor, Tensor]:
        k, v, ks, vs = self.get_int8_tensors(layer_id)
        if k.shape[2] == 0:
            logger.warning("get_kv(layer_id=%d) returning zero-length tensors.", layer_id)
        # one rounding of the exact product code * scale, as the reference's dequant (int8_cache.py:536-542)
        kd, vd = ops.dequantize(FMT_INT8, k, v, ks, vs)
        return kd.to(self.dtype), vd.to(self.dtype)

    @classmethod
    def from_tuple(cls, past_key_values, device="cuda", clip_percentile: float = 99.9,
                   group_size: int = 128) -> "INT8KVCache":
        cache = cls(num_layers=len(past_key_values), device=device, clip_percentile=clip_percentile,
                    group_size=group_size)
        for i, item in enumerate(past_key_values):
            cache.append(i, item[0].to(device), item[1].to(device))
        return cache


class INT4KVCache(_QuantCache):
    """INT4 group-wise cache, nibble-packed by default (src/cache/int4_cache.py:32-773).

    `mixed_rescue` / `outlier_rescue_ratio` keep the reference's meaning (scale
    adjustments).  `asymmetric=True` stores group-wise min/max quantization with
    fp16 scale + zero-point; `outlier_idx` (int16 [L, Hkv, n_out]) keeps the listed
    channels in an fp16 side buffer - both are extensions."""

    _fmt = FMT_INT4
    _qmax = 7.0

    def __init__(self, num_layers: int, device="cuda", clip_percentile: float = 99.9, group_size: int = 32,
                 dtype: torch.dtype = torch.float16, max_seq_len: Optional[int] = None,
                 decode_attn_impl: str = "triton_fused", static_k_scale=None, static_v_scale=None,
                 inv_tau: Optional[Tensor] = None, use_attn_temperature: bool = True,
                 adaptive_static_scales: bool = False, adaptive_static_margin: float = 1.0,
                 adaptive_static_k: bool = True, adaptive_static_v: bool = True,
                 bit_packed: bool = True, outlier_rescue_ratio: float = 0.0, mixed_rescue: bool = False, *,
                 asymmetric: bool = False, outlier_idx: Optional[Tensor] = None,
                 keep_fp32_scales: bool = False, validate_inputs: bool = False):
        super().__init__(num_layers, device, clip_percentile, group_size, dtype, max_seq_len, decode_attn_impl,
                         static_k_scale, static_v_scale, inv_tau, use_attn_temperature, adaptive_static_scales,
                         adaptive_static_margin, adaptive_static_k, adaptive_static_v, keep_fp32_scales,
                         validate_inputs)
        if outlier_rescue_ratio < 0:
            raise ValueError(f"outlier_rescue_ratio must be >= 0, got {outlier_rescue_ratio}")
        # bit_packed=False keeps one INT4 code per byte (src/cache/int4_cache.py:520-560): same quantizer,
        # payload [B,H,S,D]; the attention kernels read it as INT8 codes with the same scales
        self.bit_packed = bool(bit_packed)
        self.outlier_rescue_ratio = float(outlier_rescue_ratio)
        self.mixed_rescue = bool(mixed_rescue)
        self.asymmetric = bool(asymmetric)
        if outlier_idx is not None:
            if asymmetric:
                raise ValueError("outlier side buffer is defined for symmetric INT4 only")
            outlier_idx = torch.as_tensor(outlier_idx).to(torch.int16)
            if outlier_idx.ndim != 3 or outlier_idx.shape[0] != num_layers:
                raise ValueError("outlier_idx must be [num_layers, Hkv, n_out]")
            outlier_idx, _ = torch.sort(outlier_idx, dim=-1)
        self.outlier_idx = outlier_idx

    def _payload_dim(self, head_dim: int) -> int:
        if not self.bit_packed:
            return head_dim
        if head_dim % 2 != 0:
            raise ValueError(f"INT4 bit packing requires even head_dim, got {head_dim}")
        return head_dim // 2

    @property
    def _decode_fmt(self) -> int:
        return FMT_INT4 if self.bit_packed else FMT_INT8

    def _rescue_threshold(self, x: Tensor, G: int) -> Tensor:
        """Global quantile of the per-group absmax/7 over the whole appended tensor
        (src/cache/int4_cache.py:360-390).  The order statistic is taken with
        torch.quantile on the device; no host sync."""
        B, H, T, D = x.shape
        dyn = x.reshape(B, H, T, G, D // G).abs().amax(dim=-1).float().clamp(min=1e-5) / 7.0
        q = max(0.0, min(1.0, 1.0 - self.outlier_rescue_ratio))
        return torch.quantile(dyn.reshape(-1), q).reshape(1).contiguous()

    def append(self, layer_id: int, k: Tensor, v: Tensor) -> None:
        """Quantize, pack and append (src/cache/int4_cache.py:392-589)."""
        if self.static_k_scale is None and not self.asymmetric:
            if self.outlier_rescue_ratio > 0:
                warnings.warn(
                    f"KVC-031: outlier_rescue_ratio={self.outlier_rescue_ratio} has no effect at layer "
                    f"{layer_id} because no static scale is provided.", RuntimeWarning)
            if self.mixed_rescue:
                warnings.warn(
                    f"KVC-031: mixed_rescue=True has no effect at layer {layer_id} because no static "
                    "scale is provided.", RuntimeWarning)
        self._append_impl(layer_id, k, v, extra_flags=self._rescue_flags())

    def _rescue_flags(self) -> int:
        flags = 0 if self.bit_packed else F_UNPACKED
        if self.mixed_rescue:
            flags |= F_MIXED_RESCUE
        if self.outlier_rescue_ratio >= 1.0:
            flags |= F_MIXED_RESCUE          # max(static, dynamic) everywhere (int4_cache.py:380-381)
        elif self.outlier_rescue_ratio > 0.0:
            flags |= F_RESCUE_THR
        return flags

    def supports_fused_rope(self) -> bool:
        return not (self._rescue_flags() & F_RESCUE_THR)

    def append_rotary(self, layer_id: int, q: Tensor, k: Tensor, v: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        return self._append_impl(layer_id, k, v, extra_flags=self._rescue_flags(), rope=(q, cos, sin))

    def get_int4_tensors(self, layer_id: int) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
        """(k_packed, v_packed, k_scale, v_scale) views; payload [B,Hkv,S,D/2], scales fp16."""
        return self._layer_view(layer_id, ("k", "v", "ks", "vs"))

    def get_kv(self, layer_id: int) -> Tuple[Tensor, Tensor]:
        t = self.get_decode_tensors(layer_id)
        if t["k"].shape[2] == 0:
            logger.warning("get_kv(layer_id=%d) returning zero-length tensors.", layer_id)
        oidx = t.get("outlier_idx")
        if oidx is not None:
            oidx = oidx.to(device=t["k"].device, dtype=torch.int16).contiguous()
        kd, vd = ops.dequantize(self._decode_fmt, t["k"], t["v"], t["ks"], t["vs"], k_zp=t.get("kz"), v_zp=t.get("vz"),
                                outlier_idx=oidx, k_side=t.get("kside"), v_side=t.get("vside"))
        return kd.to(self.dtype), vd.to(self.dtype)

    @classmethod
    def from_tuple(cls, past_key_values, device="cuda", clip_percentile: float = 99.9,
                   group_size: int = 32) -> "INT4KVCache":
        cache = cls(num_layers=len(past_key_values), device=device, clip_percentile=clip_percentile,
                    group_size=group_size)
        for i, item in enumerate(past_key_values):
            cache.append(i, item[0].to(device), item[1].to(device))
        return cache
