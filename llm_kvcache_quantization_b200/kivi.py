"""KIVI-format KV cache: K quantized per channel (parameters fixed by the prompt), V per token, both
asymmetric with fp32 scale and float zero-point, INT8 codes or nibble-packed INT4.

Mirror of the reference's `KIVIStyleKVCache` (src/cache/kivi_style_cache.py:34-895) on the CUDA kernels of
csrc/kvq_kivi.cu: `append` (one launch for K and V; three small launches more on the first append of a
layer, which derives the per-channel K parameters), `get_kv` (bit-exact dequantisation) and a decode call
over the quantized cache (one fused kernel at head_dim 128; dequantise-then-attend otherwise, which is how
the reference decodes this cache, `decode_attn_impl = "torch_ref"`).  With `residual_length > 0` the newest
decode tokens stay in an fp16 window and are quantized as they leave it (:363-405); attention then merges the
partial over the quantized tokens with the partial over the window.  Clipping percentiles below 100
(src/quant/asymmetric_quant.py:98-104: two-sided torch.quantile bounds, over the prompt's tokens for K and over the
head dimension of each token for V) sort on the device (torch.sort: no rounding) and interpolate in
kvq_sorted_quantile; the append kernel takes the bounds in place of the minimum and maximum.
`RoleAwareAsymKVCache` (src/cache/role_aware_asym_cache.py:27-83) is the same cache carrying the metadata of the
calibrated-percentile family.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor

from . import _lib, ops
from .cache import _new_stats


def _clip_bounds(x: Tensor, percentile: float) -> Tuple[Tensor, Tensor]:
    """(quantile(1 - p), quantile(p)) over the last axis of an fp32 tensor, the clipping range of the reference's
    asymmetric quantizer below percentile 100 (src/quant/asymmetric_quant.py:98-104)."""
    srt = torch.sort(x.contiguous(), dim=-1).values
    rows, n = srt.numel() // srt.shape[-1], srt.shape[-1]
    lo = torch.empty(srt.shape[:-1], dtype=torch.float32, device=x.device)
    hi = torch.empty_like(lo)
    q = _lib.KvqQuantileArgs()
    q.sorted, q.rows, q.n = srt.data_ptr(), rows, n
    q.q_lo = max(0.0, min((100.0 - percentile) / 100.0, 1.0))
    q.q_hi = max(0.0, min(percentile / 100.0, 1.0))
    q.out_lo, q.out_hi = lo.data_ptr(), hi.data_ptr()
    with torch.cuda.device(x.device):
        rc = _lib.load().kvq_sorted_quantile(C.byref(q), ops._stream_ptr(x.device))
    _lib.check("kvq_sorted_quantile", rc)
    return lo, hi


class KIVIStyleKVCache:
    def __init__(self, num_layers: int, device: str = "cuda", dtype: torch.dtype = torch.float16,
                 max_seq_len: Optional[int] = None, quant_bits: int = 8, k_percentile: float = 100.0,
                 v_percentile: float = 100.0, inv_tau: Optional[Tensor] = None, use_attn_temperature: bool = False,
                 residual_length: int = 0):
        if num_layers <= 0:
            raise ValueError(f"num_layers must be > 0, got {num_layers}")
        if quant_bits not in (4, 8):
            raise ValueError(f"quant_bits must be 4 or 8, got {quant_bits}")
        for nm, pct in (("k_percentile", k_percentile), ("v_percentile", v_percentile)):
            if not (50.0 < float(pct) <= 100.0):      # the quantizer's own check (src/quant/asymmetric_quant.py:64-68)
                raise ValueError(f"percentile must be in (50.0, 100.0], got {pct} for {nm}. "
                                 "Values <= 50 invert min/max and produce silent errors.")
        self.num_layers = num_layers
        self.device = device
        self.dtype = dtype
        self.max_seq_len = int(max_seq_len) if max_seq_len is not None else None
        self.quant_bits = quant_bits
        self.k_percentile, self.v_percentile = float(k_percentile), float(v_percentile)
        self.bit_packed = bool(quant_bits == 4)
        self.decode_attn_impl = "torch_ref"
        self.inv_tau = inv_tau
        self.use_attn_temperature = use_attn_temperature
        self.residual_length = max(0, int(residual_length))
        self._fp16_k_recent: List[Optional[Tensor]] = [None] * num_layers    # [B, H, residual_length, D]
        self._fp16_v_recent: List[Optional[Tensor]] = [None] * num_layers
        self._residual_lens: List[int] = [0] * num_layers
        self._min_capacity = 256
        self._k_cache: List[Optional[Tensor]] = [None] * num_layers
        self._v_cache: List[Optional[Tensor]] = [None] * num_layers
        self._k_scale: List[Optional[Tensor]] = [None] * num_layers     # fp32 [B, H, D]
        self._k_zp: List[Optional[Tensor]] = [None] * num_layers
        self._v_scale: List[Optional[Tensor]] = [None] * num_layers     # fp32 [B, H, capacity]
        self._v_zp: List[Optional[Tensor]] = [None] * num_layers
        # fp16 per-token tiles for the fused decode kernel (INT4): copies of the V parameters, and the
        # constant K tiles (scale 1, zero-point 0: the per-channel K scale travels inside the query)
        self._v_scale16: List[Optional[Tensor]] = [None] * num_layers
        self._v_zp16: List[Optional[Tensor]] = [None] * num_layers
        self._k_ones: List[Optional[Tensor]] = [None] * num_layers
        self._k_zeros: List[Optional[Tensor]] = [None] * num_layers
        self._k_scale_initialized: List[bool] = [False] * num_layers
        self._layer_seq_lens: List[int] = [0] * num_layers
        self._layer_capacity: List[int] = [0] * num_layers
        self._seq_len = 0
        self.decode_stats: Dict[str, object] = _new_stats()

    # ------------------------------------------------------------------ storage
    def _ensure_capacity(self, layer_id: int, batch: int, heads: int, head_dim: int, target_len: int) -> None:
        if self.max_seq_len is not None and target_len > self.max_seq_len:
            raise ValueError(f"target_len {target_len} exceeds max_seq_len {self.max_seq_len} for layer {layer_id}")
        pd = head_dim // 2 if self.bit_packed else head_dim
        kb = self._k_cache[layer_id]
        if kb is not None:
            if kb.shape[0] != batch or kb.shape[1] != heads or kb.shape[3] != pd:
                raise ValueError(f"Inconsistent shape for layer {layer_id}: existing K={tuple(kb.shape)}, "
                                 f"incoming=({batch}, {heads}, *, {head_dim})")
            if target_len <= self._layer_capacity[layer_id]:
                return
            new_cap = max(target_len, self._layer_capacity[layer_id] * 2)
        else:
            new_cap = max(target_len, self._min_capacity)
        if self.max_seq_len is not None:
            new_cap = min(new_cap, self.max_seq_len)
            if new_cap < target_len:
                raise ValueError(f"target_len {target_len} exceeds capped capacity {new_cap} for layer {layer_id}")
        phys = (new_cap + 31) // 32 * 32
        dev = self.device
        new = (torch.empty((batch, heads, phys, pd), device=dev, dtype=torch.int8),
               torch.empty((batch, heads, phys, pd), device=dev, dtype=torch.int8),
               torch.empty((batch, heads, phys), device=dev, dtype=torch.float32),
               torch.empty((batch, heads, phys), device=dev, dtype=torch.float32))
        old = self._layer_seq_lens[layer_id]
        if kb is not None and old > 0:
            for dst, src in zip(new, (self._k_cache[layer_id], self._v_cache[layer_id], self._v_scale[layer_id],
                                      self._v_zp[layer_id])):
                dst[:, :, :old] = src[:, :, :old]
        self._k_cache[layer_id], self._v_cache[layer_id], self._v_scale[layer_id], self._v_zp[layer_id] = new
        self._layer_capacity[layer_id] = new_cap
        if head_dim == 128:
            h16 = [torch.empty((batch, heads, phys, 1), device=dev, dtype=torch.float16) for _ in range(2)]
            if self._v_scale16[layer_id] is not None and old > 0:
                h16[0][:, :, :old] = self._v_scale16[layer_id][:, :, :old]
                h16[1][:, :, :old] = self._v_zp16[layer_id][:, :, :old]
            self._v_scale16[layer_id], self._v_zp16[layer_id] = h16
            self._k_ones[layer_id] = torch.ones((batch, heads, phys, 1), device=dev, dtype=torch.float16)
            self._k_zeros[layer_id] = torch.zeros((batch, heads, phys, 1), device=dev, dtype=torch.float16)
        if self._k_scale[layer_id] is None:
            self._k_scale[layer_id] = torch.empty((batch, heads, head_dim), device=dev, dtype=torch.float32)
            self._k_zp[layer_id] = torch.empty((batch, heads, head_dim), device=dev, dtype=torch.float32)

    def _args(self, layer_id: int, T: int, D: int) -> "_lib.KvqKiviArgs":
        a = _lib.KvqKiviArgs()
        kc, vc = self._k_cache[layer_id], self._v_cache[layer_id]
        a.bits = self.quant_bits
        a.B, a.H, a.T, a.D = kc.shape[0], kc.shape[1], T, D
        a.k_payload, a.v_payload = kc.data_ptr(), vc.data_ptr()
        a.pay_stride_b, a.pay_stride_h, a.pay_stride_s = kc.stride(0), kc.stride(1), kc.stride(2)
        a.max_slots = min(kc.shape[2], vc.shape[2], self._v_scale[layer_id].shape[-1])   # appends beyond it store nothing
        a.k_scale, a.k_zp = self._k_scale[layer_id].data_ptr(), self._k_zp[layer_id].data_ptr()
        vs = self._v_scale[layer_id]
        a.v_scale, a.v_zp = vs.data_ptr(), self._v_zp[layer_id].data_ptr()
        a.vs_stride_b, a.vs_stride_h = vs.stride(0), vs.stride(1)
        if self._v_scale16[layer_id] is not None:
            a.v_scale_h, a.v_zp_h = self._v_scale16[layer_id].data_ptr(), self._v_zp16[layer_id].data_ptr()
        return a

    # ------------------------------------------------------------------ append / read back
    def append(self, layer_id: int, k: Tensor, v: Tensor) -> None:
        """Quantize and append (src/cache/kivi_style_cache.py:296-600): the first append of a layer fixes the
        per-channel K parameters from its tokens; V is quantized per token."""
        if layer_id < 0 or layer_id >= self.num_layers:
            raise ValueError(f"layer_id {layer_id} out of range [0, {self.num_layers})")
        if not isinstance(k, torch.Tensor) or not isinstance(v, torch.Tensor):
            raise TypeError(f"k and v must be tensors, got {type(k)} / {type(v)}")
        if k.ndim != 4 or v.ndim != 4:
            raise ValueError(f"k/v must be 4D tensors [B,H,S,D], got k={tuple(k.shape)} v={tuple(v.shape)}")
        if tuple(k.shape) != tuple(v.shape):
            raise ValueError(f"k/v shape mismatch: k={tuple(k.shape)} vs v={tuple(v.shape)}")
        if not k.is_floating_point() or not v.is_floating_point():
            raise ValueError(f"k/v must be floating point, got {k.dtype} / {v.dtype}")
        if not k.is_cuda or not v.is_cuda:
            raise ValueError("this cache quantizes with a CUDA kernel; CPU tensors are not supported")
        B, H, T, D = k.shape
        if B <= 0 or H <= 0 or T <= 0 or D <= 0:
            raise ValueError(f"Invalid k/v shape values: heads={H}, new_seq_len={T}, head_dim={D}")
        if self.bit_packed and D % 2 != 0:
            raise ValueError(f"KIVI INT4 bit packing requires even head_dim, got {D}")
        if self.residual_length > 0 and T == 1 and self._k_scale_initialized[layer_id]:
            # the token enters the fp16 window; the oldest one leaves it for the quantized cache once it is full
            if self._fp16_k_recent[layer_id] is None:
                self._fp16_k_recent[layer_id] = torch.zeros(B, H, self.residual_length, D, device=k.device, dtype=self.dtype)
                self._fp16_v_recent[layer_id] = torch.zeros(B, H, self.residual_length, D, device=k.device, dtype=self.dtype)
            kr, vr = self._fp16_k_recent[layer_id], self._fp16_v_recent[layer_id]
            rlen = self._residual_lens[layer_id]
            if rlen < self.residual_length:
                kr[:, :, rlen:rlen + 1] = k.to(self.dtype)
                vr[:, :, rlen:rlen + 1] = v.to(self.dtype)
                self._residual_lens[layer_id] = rlen + 1
                if layer_id == 0:
                    self._seq_len = self._layer_seq_lens[0] + self._residual_lens[0]
                return
            evict_k, evict_v = kr[:, :, 0:1].clone(), vr[:, :, 0:1].clone()
            kr[:, :, :-1] = kr[:, :, 1:].clone()
            vr[:, :, :-1] = vr[:, :, 1:].clone()
            kr[:, :, -1:] = k.to(self.dtype)
            vr[:, :, -1:] = v.to(self.dtype)
            k, v = evict_k, evict_v
        k16 = k if k.dtype == torch.float16 else k.to(torch.float16)
        v16 = v if v.dtype == torch.float16 else v.to(torch.float16)
        if k16.stride(-1) != 1:
            k16 = k16.contiguous()
        if v16.stride() != k16.stride():
            k16, v16 = k16.contiguous(), v16.contiguous()
        old = self._layer_seq_lens[layer_id]
        self._ensure_capacity(layer_id, B, H, D, old + T)
        a = self._args(layer_id, T, D)
        a.init_k_params = 0 if self._k_scale_initialized[layer_id] else 1
        a.k_src, a.v_src = k16.data_ptr(), v16.data_ptr()
        a.src_stride_b, a.src_stride_h, a.src_stride_t = k16.stride(0), k16.stride(1), k16.stride(2)
        a.write_pos = old
        dev = k16.device
        keep = []                                     # bounds tensors stay alive until the launch is enqueued
        if a.init_k_params and self.k_percentile < 100.0:
            # per channel over the prompt's tokens: sorted along the token axis
            lo, hi = _clip_bounds(k16.float().transpose(2, 3), self.k_percentile)           # [B, H, D]
            a.k_lo, a.k_hi = lo.data_ptr(), hi.data_ptr()
            keep += [lo, hi]
        if self.v_percentile < 100.0:
            lo, hi = _clip_bounds(v16.float(), self.v_percentile)                           # [B, H, T]
            a.v_lo, a.v_hi = lo.data_ptr(), hi.data_ptr()
            keep += [lo, hi]
        with torch.cuda.device(dev):
            rc = _lib.load().kvq_kivi_append(C.byref(a), ops._stream_ptr(dev))
        _lib.check("kvq_kivi_append", rc)
        del keep
        self._k_scale_initialized[layer_id] = True
        self._layer_seq_lens[layer_id] = old + T
        self._seq_len = max(self._layer_seq_lens) + (max(self._residual_lens) if self.residual_length > 0 else 0)

    def get_kv(self, layer_id: int) -> Tuple[Tensor, Tensor]:
        """Dequantised (k, v) in `self.dtype` (src/cache/kivi_style_cache.py:602-650)."""
        if layer_id < 0 or layer_id >= self.num_layers:
            raise ValueError(f"layer_id {layer_id} out of range [0, {self.num_layers})")
        if self._k_cache[layer_id] is None:
            raise ValueError(f"Cache for layer {layer_id} is empty")
        S = self._layer_seq_lens[layer_id]
        if S <= 0:
            raise ValueError(f"Cache for layer {layer_id} has no tokens")
        kc = self._k_cache[layer_id]
        B, H = kc.shape[0], kc.shape[1]
        D = kc.shape[3] * (2 if self.bit_packed else 1)
        a = self._args(layer_id, S, D)
        k_out = torch.empty((B, H, S, D), dtype=torch.float16, device=kc.device)
        v_out = torch.empty_like(k_out)
        a.k_out, a.v_out = k_out.data_ptr(), v_out.data_ptr()
        a.out_stride_b, a.out_stride_h, a.out_stride_s = k_out.stride(0), k_out.stride(1), k_out.stride(2)
        with torch.cuda.device(kc.device):
            rc = _lib.load().kvq_kivi_dequantize(C.byref(a), ops._stream_ptr(kc.device))
        _lib.check("kvq_kivi_dequantize", rc)
        k_out, v_out = k_out.to(self.dtype), v_out.to(self.dtype)
        rlen = self._residual_lens[layer_id]
        if self.residual_length > 0 and rlen > 0 and self._fp16_k_recent[layer_id] is not None:
            k_out = torch.cat([k_out, self._fp16_k_recent[layer_id][:, :, :rlen]], dim=2)
            v_out = torch.cat([v_out, self._fp16_v_recent[layer_id][:, :, :rlen]], dim=2)
        return k_out, v_out

    def get_int4_asym_tensors(self, layer_id: int):
        """(k_packed, v_packed, k_scale, k_zp, v_scale, v_zp) views (src/cache/kivi_style_cache.py:668-700)."""
        if not self.bit_packed:
            raise ValueError("get_int4_asym_tensors requires quant_bits=4")
        S = self._layer_seq_lens[layer_id]
        return (self._k_cache[layer_id][:, :, :S], self._v_cache[layer_id][:, :, :S], self._k_scale[layer_id],
                self._k_zp[layer_id], self._v_scale[layer_id][:, :, :S], self._v_zp[layer_id][:, :, :S])

    def fused_decode(self, layer_id: int, q: Tensor, sm_scale: float, inv_tau: Optional[Tensor] = None,
                     out: Optional[Tensor] = None) -> Tensor:
        """q_len == 1 attention over this layer.

        head_dim 128: ONE fused kernel over the quantized cache (INT4: the factored-scale path; INT8: per-element
        fp16 scale and zero-point with one group per token).  The per-channel K scale is
        multiplied into the query inside the kernel (`q_chan_scale`; logit = sum_d (q_d s_d) code_d; the K zero-points add the same constant to
        every logit of a head and cancel in the softmax), the per-token V scale is folded into the
        probabilities and the V zero-points enter as sum_t p_t z_t - the factored-scale path of the decode
        kernel with one group per token.  The V parameters are read as fp16 (RN16 of the fp32 ones).
        Otherwise: dequantise, then the tensor-core fp16 attention kernel."""
        original = q.dtype
        if original != torch.float16:
            q = q.to(torch.float16)
        S = self._layer_seq_lens[layer_id]
        kc = self._k_cache[layer_id]
        rlen = self._residual_lens[layer_id] if self.residual_length > 0 else 0
        tau = None if inv_tau is None else inv_tau.float()
        if q.shape[-1] == 128 and kc is not None and S > 0 and self._v_scale16[layer_id] is not None:
            B, Hq, D = q.shape
            H = kc.shape[1]
            fmt = _lib.FMT_INT4 if self.bit_packed else _lib.FMT_INT8
            res = ops.decode_attn(fmt, q, kc[:, :, :S], self._v_cache[layer_id][:, :, :S],
                                  self._k_ones[layer_id][:, :, :S], self._v_scale16[layer_id][:, :, :S], None,
                                  float(sm_scale), head_dim=D, k_zp=self._k_zeros[layer_id][:, :, :S],
                                  v_zp=self._v_zp16[layer_id][:, :, :S], inv_tau=tau, out=out,
                                  fast_dequant=self.bit_packed, return_partial=rlen > 0,
                                  q_chan_scale=self._k_scale[layer_id])
            if rlen > 0:
                # merge with the fp16 window.  The fused kernel's logits lack the constant sum_d q_d zp_d of
                # the K zero-points (it cancels inside one softmax, not across two): add it to that partial's max
                _, (po, pm, pl) = res
                qt = q if tau is None else (q * tau.to(torch.float16).view(1, -1, 1))
                const = (qt.float().view(B, H, Hq // H, D) * self._k_zp[layer_id][:, :, None, :]).sum(-1).view(B, Hq)
                pm = pm + float(sm_scale) * const
                _, (wo, wm, wl) = ops.decode_attn(_lib.FMT_FP16, q, self._fp16_k_recent[layer_id][:, :, :rlen].to(torch.float16),
                                                  self._fp16_v_recent[layer_id][:, :, :rlen].to(torch.float16), None, None,
                                                  None, float(sm_scale), head_dim=D, inv_tau=tau, return_partial=True)
                res = ops.lse_combine(torch.stack([po, wo]), torch.stack([pm, wm]), torch.stack([pl, wl]), out=out)
            return res if original == torch.float16 else res.to(original)
        k, v = self.get_kv(layer_id)
        res = ops.decode_attn(_lib.FMT_FP16, q, k.to(torch.float16), v.to(torch.float16), None, None, None,
                              float(sm_scale), head_dim=q.shape[-1], inv_tau=tau, out=out)
        return res if original == torch.float16 else res.to(original)

    # ------------------------------------------------------------------ bookkeeping (reference surface)
    def get_seq_len(self) -> int:
        return self._seq_len

    def clear(self) -> None:
        self._layer_seq_lens = [0] * self.num_layers
        self._k_scale_initialized = [False] * self.num_layers
        self._residual_lens = [0] * self.num_layers
        self._seq_len = 0

    def release(self) -> None:
        n = self.num_layers
        self._k_cache, self._v_cache = [None] * n, [None] * n
        self._k_scale, self._k_zp, self._v_scale, self._v_zp = [None] * n, [None] * n, [None] * n, [None] * n
        self._v_scale16, self._v_zp16, self._k_ones, self._k_zeros = [None] * n, [None] * n, [None] * n, [None] * n
        self._layer_capacity = [0] * n
        self._fp16_k_recent, self._fp16_v_recent = [None] * n, [None] * n
        self.clear()

    def get_memory_mb(self) -> float:
        total = 0
        for group in (self._k_cache, self._v_cache, self._k_scale, self._k_zp, self._v_scale, self._v_zp):
            for t in group:
                if t is not None:
                    total += t.numel() * t.element_size()
        return total / (1024 * 1024)

    def record_fused_decode(self, layer_id: int, decode_impl: str) -> None:
        self.decode_stats["fused_decode_calls"] = int(self.decode_stats.get("fused_decode_calls", 0)) + 1
        hits = self.decode_stats.setdefault("layer_hits", {})
        hits[layer_id] = hits.get(layer_id, 0) + 1
        if decode_impl == "torch_ref":
            self.decode_stats["torch_ref_calls"] = int(self.decode_stats.get("torch_ref_calls", 0)) + 1

    def record_triton_kernel_call(self, layer_id: Optional[int] = None) -> None:
        self.decode_stats["triton_kernel_calls"] = int(self.decode_stats.get("triton_kernel_calls", 0)) + 1

    def reset_decode_stats(self) -> None:
        self.decode_stats = _new_stats()

    def get_decode_stats(self) -> Dict[str, object]:
        return dict(self.decode_stats)

    def __repr__(self) -> str:
        return (f"KIVIStyleKVCache(num_layers={self.num_layers}, quant_bits={self.quant_bits}, "
                f"seq_len={self._seq_len}, memory={self.get_memory_mb():.1f}MB)")


class RoleAwareAsymKVCache(KIVIStyleKVCache):
    """The KIVI-format cache under the name of the calibrated-percentile family
    (src/cache/role_aware_asym_cache.py:27-83): same storage and quantization, INT4 by default, plus the
    `framework` tag and `ba_calibrated` (either percentile differs from 100) that the reference's routing and
    experiment tracking read."""

    def __init__(self, num_layers: int, device: str = "cuda", dtype: torch.dtype = torch.float16,
                 max_seq_len: Optional[int] = None, quant_bits: int = 4, k_percentile: float = 100.0,
                 v_percentile: float = 100.0, inv_tau: Optional[Tensor] = None, use_attn_temperature: bool = False,
                 framework: str = "ours_asym", residual_length: int = 0):
        super().__init__(num_layers=num_layers, device=device, dtype=dtype, max_seq_len=max_seq_len,
                         quant_bits=quant_bits, k_percentile=k_percentile, v_percentile=v_percentile, inv_tau=inv_tau,
                         use_attn_temperature=use_attn_temperature, residual_length=residual_length)
        self.framework = framework
        self.ba_calibrated = (k_percentile != 100.0) or (v_percentile != 100.0)
