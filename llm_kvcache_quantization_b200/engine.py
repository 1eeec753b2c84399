"""Patched HuggingFace attention forward, HF-cache-shaped wrappers and the decode loop.

Mirrors the reference's `src/engine/patch_model.py` (`apply_int8_fused_patch`,
`remove_int8_fused_patch`, `INT8CacheWrapper`, `INT8CacheWrapperContainer`,
`_fused_forward_impl`, `_decode_attn_int8_torch_ref`) and the part of
`src/engine/generate_loop.py` that drives them (`generate_from_ids`).

One decode step of one layer = q/k/v projections and RoPE (torch), then exactly two
launches of the CUDA library for the KV path: the fused quantize-append of the new
token and the fused decode attention (which applies the per-head `inv_tau`), with no
host synchronisation in between.  The reference's order is kept: append first, then
attend over S+1 tokens including the just-quantized one (src/engine/patch_model.py:755-804).
"""
from __future__ import annotations

import inspect
import json
import logging
import os
import time
import warnings
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from .cache import FP16KVCache, INT4KVCache, INT8KVCache
from .kernels import decode_attn_int4, decode_attn_int8
from .quant import unpack_int4

logger = logging.getLogger(__name__)
_patched_classes = set()
_FUSED_DUMP_WRITTEN = set()        # (directory, layer, step) already dumped by this process
_FUSED_DEBUG_LOGGED = set()        # (layer, implementation) already logged once


def _reset_fused_state() -> None:
    """Forget what was dumped / logged (tests; src/engine/patch_model.py:31-50)."""
    _FUSED_DUMP_WRITTEN.clear()
    _FUSED_DEBUG_LOGGED.clear()

FUSED_KV_MODES = frozenset({"fp16", "int8_baseline", "int8_fused", "int8_ours", "int4_baseline", "int4_fused",
                            "int4_ours", "int4_ours_mixed", "kivi_style", "int4_kivi_aligned", "int4_ours_asym",
                            "int4_ours_asym_ba"})
# modes stored in the KIVI format (per-channel K, per-token V, asymmetric)
KIVI_FORMAT_MODES = frozenset({"kivi_style", "int4_kivi_aligned", "int4_ours_asym", "int4_ours_asym_ba"})


# --------------------------------------------------------------------------- HF cache shims
class INT8CacheWrapper:
    """Per-layer view of a cache engine with the HF cache surface the attention layer uses
    (src/engine/patch_model.py:99-133)."""

    def __init__(self, cache_engine, layer_idx):
        self.engine = cache_engine
        self.layer_idx = layer_idx

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        self.engine.append(layer_idx, key_states, value_states)
        return self.engine.get_kv(layer_idx)

    def get_seq_length(self, layer_idx=0):
        return self.engine.get_seq_len()

    def __getitem__(self, idx):
        return self.engine.get_kv(idx)

    def __iter__(self):
        for i in range(self.engine.num_layers):
            yield self.engine.get_kv(i)

    def __len__(self):
        return self.engine.num_layers


class INT8CacheWrapperContainer:
    """What the model receives as `past_key_values` (src/engine/patch_model.py:135-214)."""

    def __init__(self, cache_engine, num_layers):
        if not any(hasattr(cache_engine, n) for n in
                   ("get_int8_tensors", "get_int4_tensors", "get_int4_asym_tensors", "fused_decode")):
            raise TypeError(
                "INT8CacheWrapperContainer requires an INT8/INT4 fused cache engine. "
                f"Got {type(cache_engine).__name__}. "
                "If you are using kivi_style or fp16, route through the non-fused decode path.")
        self.engine = cache_engine
        self.num_layers = num_layers
        self._layer_wrappers = [INT8CacheWrapper(cache_engine, i) for i in range(num_layers)]

    def get_seq_length(self, layer_idx=0):
        return self.engine.get_seq_len()

    def get_max_cache_shape(self):
        return None

    def __getitem__(self, layer_idx):
        return self._layer_wrappers[layer_idx]

    def __iter__(self):
        return iter(self._layer_wrappers)

    def __len__(self):
        return self.num_layers

    def to_legacy_cache(self):
        return tuple(self.engine.get_kv(i) for i in range(self.num_layers))

    def get_mask_sizes(self, cache_position, layer_idx):
        cached = int(self.engine.get_seq_len())
        current = 0
        if cache_position is not None:
            try:
                current = int(cache_position.shape[0])
            except Exception:
                current = int(getattr(cache_position, "numel", lambda: 0)())
        return cached + current, 0

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        self.engine.append(layer_idx, key_states, value_states)
        return self.engine.get_kv(layer_idx)


# --------------------------------------------------------------------------- RoPE
def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def _apply_rope(query_states, key_states, cos, sin):
    """Rotate-half RoPE on [B,H,S,D] with cos/sin of rank 2-4 and rotary_dim <= D
    (src/engine/patch_model.py:223-278)."""
    bsz, _, _, head_dim = query_states.shape
    cos = cos.to(device=query_states.device, dtype=query_states.dtype)
    sin = sin.to(device=query_states.device, dtype=query_states.dtype)
    if cos.ndim > 4:
        raise ValueError(f"Unexpected cos/sin rank {cos.ndim} in _apply_rope; expected 2-4.")
    if cos.ndim == 2:
        cos, sin = cos[None], sin[None]
    if cos.ndim == 3:
        cos, sin = cos[:, None], sin[:, None]
    elif cos.shape[1] != 1:
        cos, sin = cos[:, :1], sin[:, :1]
    if cos.shape[0] == 1 and bsz > 1:
        cos, sin = cos.expand(bsz, -1, -1, -1), sin.expand(bsz, -1, -1, -1)
    rd = cos.shape[-1]
    if rd > head_dim:
        raise ValueError(f"RoPE dim {rd} > head_dim {head_dim}")
    q_rot, q_pass = query_states[..., :rd], query_states[..., rd:]
    k_rot, k_pass = key_states[..., :rd], key_states[..., rd:]
    q_emb = q_rot * cos + _rotate_half(q_rot) * sin
    k_emb = k_rot * cos + _rotate_half(k_rot) * sin
    if q_pass.numel() == 0:
        return q_emb, k_emb
    return torch.cat([q_emb, q_pass], dim=-1), torch.cat([k_emb, k_pass], dim=-1)


def _get_rope_cos_sin(attn_module, value_states, position_ids, position_embeddings):
    if position_embeddings is not None:
        try:
            cos, sin = position_embeddings
            return cos, sin
        except (TypeError, ValueError) as exc:
            warnings.warn(f"_get_rope_cos_sin: position_embeddings unpack failed ({type(exc).__name__}: {exc}); "
                          "falling back to rotary_emb.", RuntimeWarning)
    rotary = getattr(attn_module, "rotary_emb", None)
    if rotary is None or position_ids is None:
        return None, None
    for call in (lambda: rotary(value_states, position_ids), lambda: rotary(value_states, position_ids=position_ids),
                 lambda: rotary(position_ids)):
        try:
            out = call()
        except (AttributeError, KeyError, TypeError):
            continue
        if isinstance(out, (tuple, list)) and len(out) == 2:
            return out[0], out[1]
    return None, None


def _infer_heads_from_proj(attn_module, proj_name: str, head_dim: int) -> Optional[int]:
    proj = getattr(attn_module, proj_name, None)
    if proj is None:
        return None
    out_features = getattr(proj, "out_features", None)
    if out_features is None and hasattr(proj, "weight"):
        out_features = int(proj.weight.shape[0])
    if out_features is None:
        return None
    if int(out_features) % int(head_dim) != 0:
        raise ValueError(f"{proj_name}.out_features={out_features} is not divisible by head_dim={head_dim}")
    return int(out_features) // int(head_dim)


def _resolve_attn_shape_meta(attn_module) -> Tuple[int, int, int]:
    head_dim = getattr(attn_module, "head_dim", None)
    if head_dim is None:
        raise ValueError("Attention module is missing head_dim.")
    head_dim = int(head_dim)
    q_heads = getattr(attn_module, "_kv_num_attention_heads", None) or getattr(attn_module, "num_heads", None)
    kv_heads = getattr(attn_module, "_kv_num_key_value_heads", None) or getattr(attn_module, "num_key_value_heads", None)
    if q_heads is None:
        q_heads = _infer_heads_from_proj(attn_module, "q_proj", head_dim)
    if kv_heads is None:
        kv_heads = _infer_heads_from_proj(attn_module, "k_proj", head_dim)
    if q_heads is None or kv_heads is None:
        raise ValueError("Unable to resolve attention head metadata for fused decode.")
    q_heads, kv_heads = int(q_heads), int(kv_heads)
    if q_heads <= 0 or kv_heads <= 0:
        raise ValueError(f"Invalid heads: q_heads={q_heads}, kv_heads={kv_heads}")
    if q_heads % kv_heads != 0:
        raise ValueError(f"Invalid GQA mapping for fused decode: q_heads={q_heads}, kv_heads={kv_heads}")
    return q_heads, kv_heads, head_dim


# --------------------------------------------------------------------------- torch ablation path
def _decode_attn_int8_torch_ref(q, k_int8, v_int8, k_scale, v_scale, context_lens, sm_scale):
    """`decode_attn_impl="torch_ref"`: dequantize in fp16, attention in fp32, on the tensors' device
    (the ablation / audit path of src/engine/patch_model.py:281-377; never the default)."""
    if q.ndim != 3:
        raise ValueError(f"Expected q [B, H, D], got {q.shape}")
    if k_int8.ndim != 4 or v_int8.ndim != 4:
        raise ValueError(f"Expected k/v [B, H, S, D], got {k_int8.shape} / {v_int8.shape}")
    if k_scale.ndim != 4 or v_scale.ndim != 4:
        raise ValueError(f"Expected k/v scale [B, H, S, G], got {k_scale.shape} / {v_scale.shape}")
    bsz, q_heads, head_dim = q.shape
    kv_heads = k_int8.shape[1]
    if k_int8.shape[-1] != head_dim:
        raise ValueError(f"Head dim mismatch: q D={head_dim}, kv D={k_int8.shape[-1]}")
    if q_heads % kv_heads != 0:
        raise ValueError(f"GQA unsupported: q_heads={q_heads} not divisible by kv_heads={kv_heads}")
    groups = int(k_scale.shape[-1])
    if groups <= 0 or head_dim % groups != 0:
        raise ValueError(f"Invalid scale groups: D={head_dim} groups={groups}")
    n_rep = q_heads // kv_heads
    lens = [int(x) for x in context_lens.tolist()]
    outs = []
    for b in range(bsz):
        n = lens[b]
        if n <= 0:
            outs.append(torch.zeros((q_heads, head_dim), device=q.device, dtype=q.dtype))
            continue

        def deq(codes, scale):
            c = codes[b, :, :n].reshape(kv_heads, n, groups, head_dim // groups).to(torch.float16)
            return (c * scale[b, :, :n].to(torch.float16).unsqueeze(-1)).reshape(kv_heads, n, head_dim).float()

        kf, vf = deq(k_int8, k_scale), deq(v_int8, v_scale)
        qf = q[b].float().reshape(kv_heads, n_rep, head_dim)
        scores = torch.einsum("hrd,hsd->hrs", qf, kf) * sm_scale
        probs = torch.softmax(scores, dim=-1)
        outs.append(torch.einsum("hrs,hsd->hrd", probs, vf).reshape(q_heads, head_dim).to(q.dtype))
    return torch.stack(outs, dim=0)


# --------------------------------------------------------------------------- fused forward
def _layer_inv_tau(engine, layer_idx: int, q_heads: int, device):
    inv_tau = getattr(engine, "inv_tau", None)
    if inv_tau is None or not getattr(engine, "use_attn_temperature", True):
        return None
    if layer_idx >= inv_tau.shape[0]:
        raise ValueError(f"inv_tau has {inv_tau.shape[0]} layers but fused decode got layer_idx={layer_idx}.")
    row = inv_tau[layer_idx]
    if row.ndim != 1:
        raise ValueError(f"inv_tau[{layer_idx}] must be a 1D tensor [num_heads], got shape {tuple(row.shape)}. "
                         "Check calibration file format.")
    if row.shape[0] != q_heads:
        raise ValueError(f"inv_tau[{layer_idx}] has {row.shape[0]} elements but q_heads={q_heads}. "
                         "inv_tau must be calibrated per query head.")
    return row.to(device=device, dtype=torch.float32).contiguous()



def _optional_int_env(name: str) -> Optional[int]:
    raw = os.environ.get(name, "").strip()
    if not raw:
        return None
    try:
        return int(raw)
    except ValueError:
        logger.warning("Ignoring %s=%r: not an integer.", name, raw)
        return None


def _top_values(t: torch.Tensor, k: int = 5):
    flat = t.detach().float().reshape(-1)
    k = min(k, flat.numel())
    vals, idx = torch.topk(flat, k)
    return [{"index": int(i), "value": float(v)} for v, i in zip(vals, idx)]


def _maybe_dump_fused_decode(engine, layer_idx: int, decode_impl: str, q_kernel: torch.Tensor, inv_tau, sm_scale: float,
                             fused_out: torch.Tensor) -> None:
    """Audit dump of one fused decode call (src/engine/patch_model.py:380-496, called at :970-982).

    KV_FUSED_DUMP_DIR enables it; KV_FUSED_DUMP_LAYER / KV_FUSED_DUMP_STEP (cache length after the append) select
    one call.  Writes `<stem>.pt` (query as the kernel saw it, integer codes, fp16 scales, the fused output, and the
    torch dequantize-then-attention output on the same tensors) and `<stem>.json` (max / mean |difference|, the
    largest entries of both outputs).  Once per (directory, layer, step) and process."""
    dump_dir = os.environ.get("KV_FUSED_DUMP_DIR", "").strip()
    if not dump_dir:
        return
    step = int(engine.get_seq_len()) if hasattr(engine, "get_seq_len") else -1
    want_layer, want_step = _optional_int_env("KV_FUSED_DUMP_LAYER"), _optional_int_env("KV_FUSED_DUMP_STEP")
    if (want_layer is not None and want_layer != layer_idx) or (want_step is not None and want_step != step):
        return
    key = (dump_dir, int(layer_idx), step)
    if key in _FUSED_DUMP_WRITTEN:
        return
    if hasattr(engine, "get_int8_tensors"):
        k, v, ks, vs = engine.get_int8_tensors(layer_idx)
    elif hasattr(engine, "get_int4_tensors"):
        k, v, ks, vs = engine.get_int4_tensors(layer_idx)
        if getattr(engine, "bit_packed", True):
            k, v = unpack_int4(k), unpack_int4(v)          # codes in [-8, 7] stored as int8
    else:
        logger.debug("Skipping fused decode dump at layer %s: the engine exposes no integer tensors.", layer_idx)
        return
    q_eff = q_kernel if inv_tau is None else q_kernel * inv_tau.to(q_kernel.dtype).view(1, -1, 1)
    ctx = torch.full((q_kernel.shape[0],), int(k.shape[2]), dtype=torch.int32, device=q_kernel.device)
    ks16, vs16 = ks.to(torch.float16), vs.to(torch.float16)
    ref_out = _decode_attn_int8_torch_ref(q_eff, k, v, ks16, vs16, ctx, sm_scale)
    diff = (fused_out.float() - ref_out.float()).abs()
    os.makedirs(dump_dir, exist_ok=True)
    stem = f"fused_layer{int(layer_idx):02d}_step{step:05d}_pid{os.getpid()}"
    tensor_path = os.path.join(dump_dir, stem + ".pt")
    torch.save({"layer_idx": int(layer_idx), "step": step, "decode_impl": decode_impl, "sm_scale": float(sm_scale),
                "context_len": int(k.shape[2]), "q": q_eff.detach().cpu(), "k_int8": k.detach().cpu(),
                "v_int8": v.detach().cpu(), "k_scale": ks16.detach().cpu(), "v_scale": vs16.detach().cpu(),
                "fused_out": fused_out.detach().cpu(), "ref_out": ref_out.detach().cpu()}, tensor_path)
    with open(os.path.join(dump_dir, stem + ".json"), "w") as f:
        json.dump({"layer_idx": int(layer_idx), "step": step, "decode_impl": decode_impl, "sm_scale": float(sm_scale),
                   "context_len": int(k.shape[2]), "tensor_path": tensor_path, "max_abs_diff": float(diff.max()),
                   "mean_abs_diff": float(diff.mean()), "logits_topk_fused": _top_values(fused_out),
                   "logits_topk_ref": _top_values(ref_out)}, f, indent=2)
    _FUSED_DUMP_WRITTEN.add(key)
    logger.info("Wrote fused decode dump: layer=%s step=%s -> %s", layer_idx, step, tensor_path)


def _maybe_log_fused_debug(engine, layer_idx: int, decode_impl: str, q_kernel: torch.Tensor) -> None:
    """KV_FUSED_DEBUG=1: one log line per (layer, implementation) with the shapes the kernel got
    (src/engine/patch_model.py:993-1004)."""
    if os.environ.get("KV_FUSED_DEBUG", "0") != "1":
        return
    key = (int(layer_idx), decode_impl)
    if key in _FUSED_DEBUG_LOGGED:
        return
    _FUSED_DEBUG_LOGGED.add(key)
    logger.warning("[KV_FUSED_DEBUG] layer=%d impl=%s q=%s dtype=%s cache=%s seq_len=%s", layer_idx, decode_impl,
                   tuple(q_kernel.shape), q_kernel.dtype, type(engine).__name__,
                   engine.get_seq_len() if hasattr(engine, "get_seq_len") else "?")


def _fused_forward_impl(self, hidden_states, cache_wrapper, attention_mask=None, position_ids=None,
                        position_embeddings=None, cache_position=None, return_cache=False, **kwargs):
    """Decode-only (q_len == 1) attention forward (src/engine/patch_model.py:645-1008)."""
    if attention_mask is not None:
        warnings.warn("Fused INT8/INT4 decode path received a non-None attention_mask, which will be silently "
                      "ignored. The fused kernel handles causality via context lengths.", UserWarning, stacklevel=3)
    layer_idx = getattr(cache_wrapper, "layer_idx", getattr(self, "layer_idx", 0))
    bsz, q_len, _ = hidden_states.shape
    if q_len != 1:
        raise ValueError(f"Fused decode expects q_len==1, got {q_len}")
    q_heads, kv_heads, head_dim = _resolve_attn_shape_meta(self)
    engine = cache_wrapper.engine

    query_states = self.q_proj(hidden_states).view(bsz, 1, q_heads, head_dim).transpose(1, 2)
    key_states = self.k_proj(hidden_states).view(bsz, 1, kv_heads, head_dim).transpose(1, 2)
    value_states = self.v_proj(hidden_states).view(bsz, 1, kv_heads, head_dim).transpose(1, 2)
    if getattr(self, "q_norm", None) is not None:
        query_states = self.q_norm(query_states)
    if getattr(self, "k_norm", None) is not None:
        key_states = self.k_norm(key_states)
    cos, sin = _get_rope_cos_sin(self, value_states, position_ids, position_embeddings)
    if cos is None or sin is None:
        raise RuntimeError("Failed to obtain RoPE cos/sin for fused decode. "
                           "Check transformers version/model API (position_ids/position_embeddings).")
    inv_tau = _layer_inv_tau(engine, layer_idx, q_heads, query_states.device)
    fused_rope = (getattr(engine, "supports_fused_rope", None) is not None and engine.supports_fused_rope()
                  and query_states.dtype == torch.float16 and os.environ.get("KVQ_NO_FUSED_ROPE", "0") != "1")
    if fused_rope:
        # RoPE of q and k, quantization of k and v and the cache write: one launch
        query_states = engine.append_rotary(layer_idx, query_states, key_states, value_states, cos, sin)
    else:
        query_states, key_states = _apply_rope(query_states, key_states, cos, sin)
        engine.append(layer_idx, key_states, value_states)

    q_kernel = query_states.squeeze(2)
    sm_scale = float(getattr(self, "scaling", 1.0 / (head_dim ** 0.5)))
    decode_impl = getattr(engine, "decode_attn_impl", "triton_fused")
    if hasattr(engine, "record_fused_decode"):
        engine.record_fused_decode(layer_idx, decode_impl)
    try:
        if decode_impl == "triton_fused":
            if hasattr(engine, "fused_decode"):
                attn_output = engine.fused_decode(layer_idx, q_kernel, sm_scale, inv_tau=inv_tau)
                if hasattr(engine, "record_triton_kernel_call"):
                    engine.record_triton_kernel_call(layer_idx)
            else:
                attn_output = _dispatch_tensor_api(engine, layer_idx, q_kernel, sm_scale, inv_tau, False)
        elif decode_impl == "torch_ref":
            if not (hasattr(engine, "get_int8_tensors") or hasattr(engine, "get_int4_tensors")) and \
                    hasattr(engine, "fused_decode"):
                # a dequantise-then-attend engine (KIVI format): its own decode call is that path
                attn_output = engine.fused_decode(layer_idx, q_kernel, sm_scale, inv_tau=inv_tau)
            else:
                attn_output = _dispatch_tensor_api(engine, layer_idx, q_kernel, sm_scale, inv_tau, True)
        else:
            raise ValueError(f"Unknown decode_attn_impl={decode_impl!r}; expected 'triton_fused' or 'torch_ref'.")
    except Exception:
        warnings.warn(f"Fused decode failed at layer {layer_idx} after the cache append; the cache now holds one "
                      "more token than outputs were produced for.", RuntimeWarning)
        raise
    if os.environ.get("KV_FUSED_DUMP_DIR") or os.environ.get("KV_FUSED_DEBUG") == "1":
        _maybe_dump_fused_decode(engine, layer_idx, decode_impl, q_kernel, inv_tau, sm_scale, attn_output)
        _maybe_log_fused_debug(engine, layer_idx, decode_impl, q_kernel)
    attn_output = attn_output.to(hidden_states.dtype).reshape(bsz, 1, q_heads * head_dim)
    attn_output = self.o_proj(attn_output)
    if return_cache:
        return attn_output, None, cache_wrapper
    return attn_output, None


def _dispatch_tensor_api(engine, layer_idx, q_kernel, sm_scale, inv_tau, torch_ref: bool):
    """The reference's tensor-level dispatch (src/engine/patch_model.py:837-957) for engines that
    only expose get_int8_tensors / get_int4_tensors, and the torch_ref ablation."""
    if inv_tau is not None:
        q_kernel = q_kernel * inv_tau.to(q_kernel.dtype).view(1, -1, 1)
    if hasattr(engine, "get_int8_tensors"):
        k, v, ks, vs = engine.get_int8_tensors(layer_idx)
        packed = False
    elif hasattr(engine, "get_int4_tensors"):
        k, v, ks, vs = engine.get_int4_tensors(layer_idx)
        packed = bool(getattr(engine, "bit_packed", True))
    else:
        raise RuntimeError("Fused path requires cache engine to provide get_int8_tensors or get_int4_tensors.")
    if k.device != q_kernel.device:
        raise RuntimeError(f"ENG-105: Device mismatch — cache k_quant is on {k.device} but hidden_states is on "
                           f"{q_kernel.device}.")
    bsz, seq_len = q_kernel.shape[0], int(k.shape[2])
    ctx = torch.full((bsz,), seq_len, dtype=torch.int32, device=q_kernel.device)
    ks, vs = ks.to(torch.float16), vs.to(torch.float16)
    if torch_ref:
        if hasattr(engine, "get_int4_tensors") and packed:
            k, v = unpack_int4(k), unpack_int4(v)
        return _decode_attn_int8_torch_ref(q_kernel, k, v, ks, vs, ctx, sm_scale)
    stats = getattr(engine, "decode_stats", None)
    if hasattr(engine, "get_int8_tensors"):
        return decode_attn_int8(q_kernel, k, v, ks, vs, ctx, sm_scale, debug_stats=stats, layer_idx=layer_idx)
    return decode_attn_int4(q_kernel, k, v, ks, vs, ctx, sm_scale, bit_packed=packed, head_dim=q_kernel.shape[-1],
                            debug_stats=stats, layer_idx=layer_idx)


# --------------------------------------------------------------------------- patch / unpatch
def apply_int8_fused_patch(model):
    """Class-level monkey patch of the model's attention forward; idempotent
    (src/engine/patch_model.py:1011-1211)."""
    try:
        layers = model.model.layers
    except Exception:
        layers = None
    if layers is None:
        raise ValueError("Cannot detect model layers (model.model.layers). "
                         "apply_int8_fused_patch requires a standard HF decoder model.")
    cfg = getattr(model, "config", None)
    cfg_q = getattr(cfg, "num_attention_heads", None)
    cfg_kv = getattr(cfg, "num_key_value_heads", cfg_q)
    for idx, layer in enumerate(layers):
        attn = getattr(layer, "self_attn", None)
        if attn is None:
            continue
        if not hasattr(attn, "layer_idx"):
            attn.layer_idx = idx
        head_dim = getattr(attn, "head_dim", None)
        if head_dim is None:
            continue
        q_heads = cfg_q if cfg_q is not None else _infer_heads_from_proj(attn, "q_proj", int(head_dim))
        kv_heads = cfg_kv if cfg_kv is not None else _infer_heads_from_proj(attn, "k_proj", int(head_dim))
        if kv_heads is None:
            logger.warning("Could not infer kv_heads for layer %d; falling back to q_heads=%s.", idx, q_heads)
            kv_heads = q_heads
        if q_heads is not None:
            attn._kv_num_attention_heads = int(q_heads)
        if kv_heads is not None:
            attn._kv_num_key_value_heads = int(kv_heads)

    AttnClass = model.model.layers[0].self_attn.__class__
    if hasattr(AttnClass, "_original_forward"):
        apply_int8_fused_patch._patched_class = AttnClass
        _patched_classes.add(AttnClass)
        return
    AttnClass._original_forward = AttnClass.forward
    sig = inspect.signature(AttnClass._original_forward)
    has_pkv, has_pkvs, has_use_cache = ("past_key_value" in sig.parameters, "past_key_values" in sig.parameters,
                                        "use_cache" in sig.parameters)
    accepts_var_kw = any(p.kind is inspect.Parameter.VAR_KEYWORD for p in sig.parameters.values())

    def forward_proxy(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                      past_key_values=None, output_attentions=False, use_cache=False, **kwargs):
        if past_key_value is None:
            past_key_value = past_key_values
        wrapper = None
        if isinstance(past_key_value, INT8CacheWrapper):
            wrapper = past_key_value
        elif isinstance(past_key_value, INT8CacheWrapperContainer):
            wrapper = past_key_value[getattr(self, "layer_idx", 0)]
        elif hasattr(past_key_value, "__getitem__") and hasattr(past_key_value, "engine"):
            try:
                cand = past_key_value[getattr(self, "layer_idx", 0)]
                if isinstance(cand, INT8CacheWrapper):
                    wrapper = cand
            except Exception:
                wrapper = None
        if hidden_states is not None and hidden_states.shape[1] == 1 and wrapper is not None:
            if output_attentions:
                warnings.warn("output_attentions=True was requested but the fused decode path does not compute "
                              "attention weights. Attention weights will be None.", UserWarning, stacklevel=2)
            return _fused_forward_impl(self, hidden_states, wrapper, attention_mask=attention_mask,
                                       position_ids=position_ids,
                                       position_embeddings=kwargs.pop("position_embeddings", None),
                                       cache_position=kwargs.pop("cache_position", None),
                                       return_cache=use_cache if has_use_cache else False)
        fwd = dict(attention_mask=attention_mask, position_ids=position_ids, output_attentions=output_attentions,
                   use_cache=use_cache, **kwargs)
        if not accepts_var_kw:
            fwd = {k: v for k, v in fwd.items() if k in sig.parameters}
        if past_key_value is not None:
            if has_pkv:
                fwd["past_key_value"] = past_key_value
            elif has_pkvs:
                fwd["past_key_values"] = past_key_value
        return AttnClass._original_forward(self, hidden_states, **fwd)

    AttnClass.forward = forward_proxy
    apply_int8_fused_patch._patched_class = AttnClass
    _patched_classes.add(AttnClass)


def _remove_patch_from_class(AttnClass) -> bool:
    if AttnClass is None:
        return False
    original = AttnClass.__dict__.get("_original_forward")
    if original is None:
        return False
    AttnClass.forward = original
    del AttnClass._original_forward
    _patched_classes.discard(AttnClass)
    if getattr(apply_int8_fused_patch, "_patched_class", None) is AttnClass:
        apply_int8_fused_patch._patched_class = None
    return True


def remove_int8_fused_patch(model=None) -> bool:
    """Restore the original forward of one model's attention class, or of every patched class
    (src/engine/patch_model.py:1214-1298)."""
    if model is not None:
        try:
            cls = model.model.layers[0].self_attn.__class__
        except Exception:
            cls = getattr(apply_int8_fused_patch, "_patched_class", None)
        return _remove_patch_from_class(cls)
    removed = False
    for cls in list(_patched_classes):
        removed |= _remove_patch_from_class(cls)
    legacy = getattr(apply_int8_fused_patch, "_patched_class", None)
    if legacy is not None:
        removed |= _remove_patch_from_class(legacy)
    if not removed:
        logger.warning("remove_int8_fused_patch: no patched class found.")
    return removed


# --------------------------------------------------------------------------- decode loop
@dataclass
class GenerationOutput:
    """Result of `generate` (src/engine/generate_loop.py:151-165)."""
    text: str
    tokens: List[int]
    ttft_ms: float
    tpot_ms: float
    tok_per_s: float
    gpu_mem_peak_mb: float
    prompt_len: int
    gen_len: int
    tok_per_s_per_seq: float = 0.0
    kv_cache_mem_mb: float = 0.0
    kv_cache_seq_len: int = 0


@dataclass
class GenerationBatchOutput:
    """Result of `generate_from_ids` (src/engine/generate_loop.py:168-182), plus this package's extras."""
    generated_ids: torch.Tensor                 # [B, gen_len]
    ttft_ms: float = 0.0
    tpot_ms: float = 0.0
    tok_per_s: float = 0.0
    tok_per_s_per_seq: float = 0.0
    gpu_mem_peak_mb: float = 0.0
    prompt_len: int = 0
    gen_len: int = 0
    batch: int = 0
    kv_cache_mem_mb: float = 0.0
    kv_cache_seq_len: int = 0
    # not in the reference's dataclass:
    kv_mode: str = "fp16"
    decode_stats: dict = field(default_factory=dict)
    step_ms: List[float] = field(default_factory=list)


def load_calibration(calib_file: str, kv_mode: str, device, *, use_static_scales=True, use_attn_temperature=True):
    """Reads the reference's calibration JSON (k_scale / v_scale [L,Hkv,G], inv_tau [L,Hq], group and
    clip settings, int4_outlier_ratio, int4_mixed_rescue; src/engine/generate_loop.py:764-856).
    Static scales are fp16 for INT8 modes and fp32 for INT4 modes, as in the reference."""
    with open(calib_file, "r") as f:
        calib = json.load(f)
    if calib.get("version", 0) < 2:
        warnings.warn(f"Calibration file '{calib_file}' has version={calib.get('version', 0)} (expected >=2).",
                      UserWarning)
    out = {"group_size": calib.get("group_size_k", calib.get("group_size")),
           "clip_percentile": calib.get("clip_percentile_k", calib.get("clip_percentile")),
           "static_k_scale": None, "static_v_scale": None, "inv_tau": None,
           "outlier_rescue_ratio": float(calib.get("int4_outlier_ratio", 0.0) or 0.0),
           "mixed_rescue": bool(calib.get("int4_mixed_rescue", False)) or kv_mode == "int4_ours_mixed"}
    gk, gv = calib.get("group_size_k"), calib.get("group_size_v")
    if gk and gv and gk != gv:
        warnings.warn(f"CAL-022: Calibration group_size_k ({gk}) != group_size_v ({gv}); group_size_k is used "
                      "for both.", UserWarning)
    sdt = torch.float32 if kv_mode.startswith("int4") else torch.float16
    if use_static_scales:
        if "k_scale" in calib:
            out["static_k_scale"] = torch.tensor(calib["k_scale"], dtype=sdt, device=device)
        if "v_scale" in calib:
            out["static_v_scale"] = torch.tensor(calib["v_scale"], dtype=sdt, device=device)
        if ("k_scale" in calib) != ("v_scale" in calib):
            warnings.warn("ENG-048: Calibration file has only one of 'k_scale' / 'v_scale'.", UserWarning)
    if use_attn_temperature and "inv_tau" in calib:
        out["inv_tau"] = torch.tensor(calib["inv_tau"], dtype=torch.float32, device=device)
    return out


def load_role_aware_calibration(calib_file: Optional[str], kv_mode: str, device) -> dict:
    """Percentiles and temperature of the KIVI-format modes that read a calibration file
    (src/engine/generate_loop.py:951-994 for int4_kivi_aligned, :995-1043 for int4_ours_asym / int4_ours_asym_ba):
    `role_aware` section first, the `k_calibration` / `v_calibration` schema as the fallback (with the reference's
    warning); inv_tau only for the modes that use it.  A path that does not exist raises, as in the reference."""
    out = {"k_percentile": 100.0, "v_percentile": 100.0, "inv_tau": None}
    if calib_file is None:
        return out
    if not os.path.exists(calib_file):
        raise FileNotFoundError(f"{kv_mode}: calib_file={calib_file!r} not found. Use an absolute path or run from "
                                "the project root.")
    with open(calib_file, "r") as f:
        data = json.load(f)

    def tau(raw):
        return torch.tensor(raw, dtype=torch.float32, device=device)

    if kv_mode == "int4_kivi_aligned":
        if "k_calibration" in data and "inv_tau" in data["k_calibration"]:
            out["inv_tau"] = tau(data["k_calibration"]["inv_tau"])
        elif "inv_tau" in data:
            out["inv_tau"] = tau(data["inv_tau"])
        if "v_calibration" in data and "v_percentile" in data["v_calibration"]:
            out["v_percentile"] = float(data["v_calibration"]["v_percentile"])
        return out
    if "role_aware" in data:
        ra = data["role_aware"]
        out["k_percentile"] = float(ra.get("k_percentile", 100.0))
        out["v_percentile"] = float(ra.get("v_percentile", 100.0))
    elif "k_calibration" in data:
        warnings.warn(f"RoleAlign mode '{kv_mode}' using k_calibration fallback schema; consider re-generating "
                      "calibration with role_aware schema.", UserWarning)
        out["k_percentile"] = float(data["k_calibration"].get("k_percentile", data.get("k_percentile", 100.0)))
        if "v_calibration" in data:
            out["v_percentile"] = float(data["v_calibration"].get("v_percentile", 100.0))
    if kv_mode == "int4_ours_asym_ba":
        if "role_aware" in data and "inv_tau" in data["role_aware"]:
            out["inv_tau"] = tau(data["role_aware"]["inv_tau"])
        elif "k_calibration" in data and "inv_tau" in data["k_calibration"]:
            out["inv_tau"] = tau(data["k_calibration"]["inv_tau"])
        elif "inv_tau" in data:
            out["inv_tau"] = tau(data["inv_tau"])
    return out


def build_cache(kv_mode: str, num_layers: int, device, *, group_size=128, clip_percentile=99.9, max_seq_len=None,
                calib: Optional[dict] = None, decode_attn_impl="triton_fused", use_attn_temperature=True,
                quant_bits: int = 8, residual_length: int = 0, adaptive_static_scales: bool = False,
                adaptive_static_margin: float = 1.0, adaptive_static_k: bool = True, adaptive_static_v: bool = True):
    """Cache engine for a kv_mode (src/engine/generate_loop.py:891-938)."""
    if kv_mode not in FUSED_KV_MODES:
        raise ValueError(f"kv_mode={kv_mode!r} is not supported here; choose one of {sorted(FUSED_KV_MODES)}")
    if kv_mode == "fp16":
        return FP16KVCache(num_layers, device=device, max_seq_len=max_seq_len)
    if kv_mode == "kivi_style":        # per-channel K / per-token V asymmetric (src/engine/generate_loop.py:939-950)
        from .kivi import KIVIStyleKVCache
        return KIVIStyleKVCache(num_layers, device=device, max_seq_len=max_seq_len, quant_bits=quant_bits,
                                residual_length=residual_length)
    if kv_mode == "int4_kivi_aligned":  # KIVI INT4 with a calibrated temperature and V percentile (:951-994)
        from .kivi import KIVIStyleKVCache
        ra = calib or {}
        return KIVIStyleKVCache(num_layers, device=device, max_seq_len=max_seq_len, quant_bits=4,
                                v_percentile=ra.get("v_percentile", 100.0), inv_tau=ra.get("inv_tau"),
                                use_attn_temperature=use_attn_temperature, residual_length=residual_length)
    if kv_mode in ("int4_ours_asym", "int4_ours_asym_ba"):   # calibrated percentiles (+ temperature for _ba) (:995-1060)
        from .kivi import RoleAwareAsymKVCache
        ra = calib or {}
        ba = kv_mode == "int4_ours_asym_ba"
        cache = RoleAwareAsymKVCache(num_layers, device=device, max_seq_len=max_seq_len, quant_bits=4,
                                     k_percentile=ra.get("k_percentile", 100.0), v_percentile=ra.get("v_percentile", 100.0),
                                     inv_tau=ra.get("inv_tau"), use_attn_temperature=use_attn_temperature and ba,
                                     framework="ours_asym_ba" if ba else "ours_asym")
        cache.decode_attn_impl = decode_attn_impl
        return cache
    calib = calib or {}
    gs = calib.get("group_size") or group_size
    cp = calib.get("clip_percentile") or clip_percentile
    common = dict(device=device, clip_percentile=cp, group_size=gs, max_seq_len=max_seq_len,
                  decode_attn_impl=decode_attn_impl, use_attn_temperature=use_attn_temperature,
                  # passed to every quantized mode, as the reference does (src/engine/generate_loop.py:913-916, 932-935);
                  # the caches apply them only when static scales are present
                  adaptive_static_scales=adaptive_static_scales, adaptive_static_margin=adaptive_static_margin,
                  adaptive_static_k=adaptive_static_k, adaptive_static_v=adaptive_static_v)
    calibrated = kv_mode in ("int8_ours", "int4_ours", "int4_ours_mixed", "int4_fused")
    if calibrated:
        common.update(static_k_scale=calib.get("static_k_scale"), static_v_scale=calib.get("static_v_scale"),
                      inv_tau=calib.get("inv_tau"))
    if kv_mode.startswith("int8"):
        return INT8KVCache(num_layers, **common)
    extra = {}
    if calibrated:
        extra = dict(outlier_rescue_ratio=calib.get("outlier_rescue_ratio", 0.0),
                     mixed_rescue=calib.get("mixed_rescue", False) or kv_mode == "int4_ours_mixed")
    return INT4KVCache(num_layers, **common, **extra)



def _register_prefill_temperature_hooks(model, inv_tau: torch.Tensor):
    """Per-head temperature during PREFILL: scale the query states by `inv_tau[layer]` whenever more than one
    position is processed (src/engine/generate_loop.py:276-390, registered at :1210).  The decode step (one
    position) is left alone - the fused forward applies `inv_tau` itself.  With a `q_norm` module the scale goes on
    its output (either [B,H,S,D] or [B,S,H,D]; the former wins a tie), otherwise on the `q_proj` output.
    Returns the hook handles; the caller removes them."""
    handles = []
    layers = getattr(getattr(model, "model", None), "layers", None)
    if layers is None:
        warnings.warn("Cannot register prefill temperature hooks: model.model.layers not found. "
                      "Per-head temperature scaling will NOT be applied during prefill.", UserWarning)
        return handles
    if not isinstance(inv_tau, torch.Tensor) or inv_tau.ndim != 2:
        raise ValueError(f"inv_tau must be a 2D tensor [layers, heads], got {type(inv_tau)} "
                         f"{getattr(inv_tau, 'shape', None)}")
    cfg_heads = getattr(getattr(model, "config", None), "num_attention_heads", None)
    for layer_idx, layer in enumerate(layers):
        attn = getattr(layer, "self_attn", None)
        if attn is None:
            continue
        heads = next((x for x in (getattr(attn, "num_heads", None), getattr(attn, "_kv_num_attention_heads", None),
                                  cfg_heads) if x is not None), None)
        head_dim = getattr(attn, "head_dim", None)
        if heads is None or head_dim is None:
            continue
        heads, head_dim = int(heads), int(head_dim)
        if layer_idx >= inv_tau.shape[0]:
            raise ValueError(f"inv_tau has {inv_tau.shape[0]} layers but model has layer_idx={layer_idx}.")
        if inv_tau.shape[1] != heads:
            raise ValueError(f"inv_tau head count mismatch at layer {layer_idx}: "
                             f"inv_tau.shape[1]={inv_tau.shape[1]} vs model.num_heads={heads}.")
        row = inv_tau[layer_idx]
        if getattr(attn, "q_norm", None) is not None:
            def after_q_norm(module, inputs, output, row=row, heads=heads):
                if not isinstance(output, torch.Tensor) or output.ndim != 4:
                    return output
                for head_axis, seq_axis in ((1, 2), (2, 1)):
                    if output.shape[head_axis] == heads:
                        if output.shape[seq_axis] <= 1:
                            return output
                        shape = [1, 1, 1, 1]
                        shape[head_axis] = heads
                        return output * row.to(device=output.device, dtype=output.dtype).view(shape)
                return output
            handles.append(attn.q_norm.register_forward_hook(after_q_norm))
        elif getattr(attn, "q_proj", None) is not None:
            def after_q_proj(module, inputs, output, row=row, heads=heads, head_dim=head_dim):
                if not isinstance(output, torch.Tensor) or output.ndim != 3:
                    return output
                if output.shape[1] <= 1 or output.shape[2] != heads * head_dim:
                    return output
                b, s_len, _ = output.shape
                scaled = output.view(b, s_len, heads, head_dim) * row.to(device=output.device, dtype=output.dtype).view(1, 1, -1, 1)
                return scaled.view(b, s_len, heads * head_dim)
            handles.append(attn.q_proj.register_forward_hook(after_q_proj))
    return handles


def _prefill_into_cache(model, cache, input_ids, attention_mask):
    """Plain HF prefill, then bulk quantize-append of every layer's K/V
    (src/engine/generate_loop.py:1228-1256).  HF cache items may be 2- or 3-tuples."""
    out = model(input_ids=input_ids, attention_mask=attention_mask, use_cache=True)
    pkv = out.past_key_values
    layers = getattr(pkv, "layers", None)
    for i in range(cache.num_layers):
        if layers is not None:
            k, v = layers[i].keys, layers[i].values
        else:
            item = pkv[i]
            k, v = item[0], item[1]
        cache.append(i, k, v)
    return out.logits[:, -1, :]


@torch.no_grad()
def generate_from_ids(model, tokenizer, input_ids, attention_mask=None, max_new_tokens=128, kv_mode="fp16",
                      group_size=128, clip_percentile=99.9, seed=1234, calib_file=None, use_attn_temperature=True,
                      use_static_scales=True, adaptive_static_scales=False, adaptive_static_margin=1.0,
                      adaptive_static_k=True, adaptive_static_v=True, decode_attn_impl="triton_fused",
                      allow_missing_calib=False, stop_on_eos=True, quant_bits=8, k_bits=None, v_bits=None,
                      residual_length=0, policy_json=None) -> GenerationBatchOutput:
    """Greedy generation with a quantized KV cache and the fused decode path
    (src/engine/generate_loop.py:393-1581, the fused modes and fp16; same parameters).  Requires CUDA.
    `k_bits` / `v_bits` / `policy_json` belong to the reference's mixed-bit modes, which this package does not
    build: anything but None raises."""
    if kv_mode not in FUSED_KV_MODES:
        raise ValueError(f"kv_mode={kv_mode!r} is not supported here; choose one of {sorted(FUSED_KV_MODES)}")
    for name, val in (("k_bits", k_bits), ("v_bits", v_bits), ("policy_json", policy_json)):
        if val is not None:
            raise ValueError(f"{name}={val!r} selects a mixed-bit cache (kv_mode int4_mixed_kv / kivi policies), "
                             "which this package does not provide; leave it None.")
    if decode_attn_impl not in ("triton_fused", "torch_ref"):
        raise ValueError(f"Unknown decode_attn_impl={decode_attn_impl!r}")
    device = next(model.parameters()).device
    if device.type != "cuda":
        raise RuntimeError("generate_from_ids requires the model on a CUDA device.")
    input_ids = input_ids.to(device)
    bsz, prompt_len = input_ids.shape
    if attention_mask is None:
        attention_mask = torch.ones_like(input_ids)
    elif bsz > 1 and not bool((attention_mask == 1).all()):
        raise ValueError("batch > 1 requires an all-ones attention_mask (no padding) on the fused path.")
    torch.manual_seed(seed)
    calib = None
    if kv_mode in ("int8_ours", "int4_ours", "int4_ours_mixed", "int4_fused"):
        if calib_file is not None and os.path.exists(calib_file):
            calib = load_calibration(calib_file, kv_mode, device, use_static_scales=use_static_scales,
                                     use_attn_temperature=use_attn_temperature)
        elif not allow_missing_calib:
            raise FileNotFoundError(f"kv_mode={kv_mode!r} needs a calibration file (got {calib_file!r}); "
                                    "pass allow_missing_calib=True to fall back to dynamic scales.")
    if kv_mode in ("int4_kivi_aligned", "int4_ours_asym", "int4_ours_asym_ba"):
        calib = load_role_aware_calibration(calib_file, kv_mode, device)
    num_layers = len(model.model.layers)
    max_pos = getattr(model.config, "max_position_embeddings", None)
    max_seq = prompt_len + max_new_tokens if max_pos is None else min(max_pos, prompt_len + max_new_tokens)
    cache = build_cache(kv_mode, num_layers, device, group_size=group_size, clip_percentile=clip_percentile,
                        max_seq_len=max_seq, calib=calib, decode_attn_impl=decode_attn_impl,
                        use_attn_temperature=use_attn_temperature, quant_bits=quant_bits,
                        residual_length=residual_length, adaptive_static_scales=adaptive_static_scales,
                        adaptive_static_margin=adaptive_static_margin, adaptive_static_k=adaptive_static_k,
                        adaptive_static_v=adaptive_static_v)
    eos = getattr(tokenizer, "eos_token_id", None)
    if isinstance(eos, (list, tuple)):
        eos = eos[0] if eos else None
    apply_int8_fused_patch(model)
    hook_handles = []
    inv_tau = (calib or {}).get("inv_tau")
    if kv_mode in ("int8_ours", "int4_ours", "int4_ours_mixed", "int4_fused") and use_attn_temperature and inv_tau is not None:
        # fused modes: the prompt is attended with the calibrated per-head temperature as well
        hook_handles = _register_prefill_temperature_hooks(model, inv_tau)
    torch.cuda.reset_peak_memory_stats(device)
    try:
        t0 = time.perf_counter()
        logits = _prefill_into_cache(model, cache, input_ids, attention_mask)
        next_tok = logits.argmax(dim=-1, keepdim=True)
        torch.cuda.synchronize(device)
        ttft = (time.perf_counter() - t0) * 1e3
        generated = [next_tok]
        finished = torch.zeros(bsz, dtype=torch.bool, device=device)
        step_ms = []
        container = INT8CacheWrapperContainer(cache, num_layers)
        for step in range(1, max_new_tokens):
            if prompt_len + step > max_seq:
                break
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            pos = torch.full((bsz, 1), prompt_len + step - 1, dtype=torch.long, device=device)
            out = model(input_ids=next_tok, position_ids=pos, past_key_values=container, use_cache=True)
            next_tok = out.logits[:, -1, :].argmax(dim=-1, keepdim=True)
            e1.record()
            generated.append(next_tok)
            if stop_on_eos and eos is not None:
                finished |= next_tok.squeeze(1) == eos
                if bool(finished.all()):
                    e1.synchronize()
                    step_ms.append(e0.elapsed_time(e1))
                    break
            e1.synchronize()
            step_ms.append(e0.elapsed_time(e1))
        ids = torch.cat(generated, dim=1)
        tpot = sum(step_ms) / len(step_ms) if step_ms else 0.0
        tps = (bsz * len(step_ms) / (sum(step_ms) * 1e-3)) if step_ms else 0.0
        return GenerationBatchOutput(
            generated_ids=ids, ttft_ms=ttft, tpot_ms=tpot, tok_per_s=tps, tok_per_s_per_seq=tps / max(bsz, 1),
            gpu_mem_peak_mb=torch.cuda.max_memory_allocated(device) / 2 ** 20, prompt_len=int(prompt_len),
            gen_len=int(ids.shape[1]), batch=int(bsz),
            kv_cache_mem_mb=cache.get_memory_mb(), kv_cache_seq_len=cache.get_seq_len(), kv_mode=kv_mode,
            decode_stats=cache.get_decode_stats() if hasattr(cache, "get_decode_stats") else {}, step_ms=step_ms)
    finally:
        for h in hook_handles:
            h.remove()
        remove_int8_fused_patch(model)


@torch.no_grad()
def generate(model, tokenizer, prompt: str, max_new_tokens=128, kv_mode="fp16", group_size=128, clip_percentile=99.9,
             seed=1234, calib_file=None, use_attn_temperature=True, use_static_scales=True,
             adaptive_static_scales=False, adaptive_static_margin=1.0, adaptive_static_k=True, adaptive_static_v=True,
             decode_attn_impl="triton_fused", allow_missing_calib=False, stop_on_eos=True, quant_bits=8, k_bits=None,
             v_bits=None, policy_json=None) -> GenerationOutput:
    """Single-prompt front end of `generate_from_ids` (src/engine/generate_loop.py:1584): tokenize, generate
    greedily, decode the new tokens."""
    enc = tokenizer(prompt, return_tensors="pt")
    device = next(model.parameters()).device
    ids = enc["input_ids"].to(device)
    mask = enc.get("attention_mask")
    out = generate_from_ids(model, tokenizer, ids, attention_mask=None if mask is None else mask.to(device),
                            max_new_tokens=max_new_tokens, kv_mode=kv_mode, group_size=group_size,
                            clip_percentile=clip_percentile, seed=seed, calib_file=calib_file,
                            use_attn_temperature=use_attn_temperature, use_static_scales=use_static_scales,
                            adaptive_static_scales=adaptive_static_scales, adaptive_static_margin=adaptive_static_margin,
                            adaptive_static_k=adaptive_static_k, adaptive_static_v=adaptive_static_v,
                            decode_attn_impl=decode_attn_impl, allow_missing_calib=allow_missing_calib,
                            stop_on_eos=stop_on_eos, quant_bits=quant_bits, k_bits=k_bits, v_bits=v_bits,
                            policy_json=policy_json)
    toks = out.generated_ids[0].tolist()
    eos = getattr(tokenizer, "eos_token_id", None)
    if stop_on_eos and eos is not None and eos in toks:
        toks = toks[:toks.index(eos) + 1]
    return GenerationOutput(text=tokenizer.decode(toks, skip_special_tokens=True), tokens=toks, ttft_ms=out.ttft_ms,
                            tpot_ms=out.tpot_ms, tok_per_s=out.tok_per_s, gpu_mem_peak_mb=out.gpu_mem_peak_mb,
                            prompt_len=out.prompt_len, gen_len=len(toks), tok_per_s_per_seq=out.tok_per_s_per_seq,
                            kv_cache_mem_mb=out.kv_cache_mem_mb, kv_cache_seq_len=out.kv_cache_seq_len)
