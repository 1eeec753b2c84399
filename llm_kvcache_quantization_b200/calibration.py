"""Static-scale calibration artefacts: the collection half of the reference's calibration script and the
JSON file the decode loop reads.

* `compute_absmax_per_group`, `collect_absmax_samples`, `scales_from_absmax_samples` keep the names and
  meaning of scripts/calibrate_behavior.py:228-260, 764-812; the per-(head, group) maximum over a sample's
  sequence is a CUDA reduction (`kvq_group_absmax`) instead of `view().abs().amax().amax()`.
* `save_calibration` writes the version-2 schema that `engine.load_calibration` (and the reference's
  src/engine/generate_loop.py:764-856) reads: k_scale / v_scale [L, Hkv, G], inv_tau [L, Hq],
  group_size_{k,v}, clip_percentile_{k,v}, int4_outlier_ratio, int4_mixed_rescue, version.

The search for inv_tau and for the clipping percentile (the KL-divergence loop of the reference script) is
not part of this module.
"""
from __future__ import annotations

import json
from typing import List, Optional, Sequence

import torch

from . import ops


def compute_absmax_per_group(tensor: torch.Tensor, group_size: int) -> torch.Tensor:
    """[heads, seq, head_dim] (fp16/fp32, CUDA) -> fp32 [heads, num_groups]: max |x| over the sequence and
    the channels of each group."""
    if tensor.ndim != 3:
        raise ValueError(f"expected [heads, seq, head_dim], got {tuple(tensor.shape)}")
    heads, seq_len, head_dim = tensor.shape
    if group_size <= 0 or head_dim % group_size != 0:
        raise ValueError(f"head_dim ({head_dim}) must be divisible by group_size ({group_size})")
    if not tensor.is_cuda:
        raise ValueError("compute_absmax_per_group runs a CUDA reduction; CPU tensors are not supported")
    if tensor.dtype != torch.float16:
        # |x| of a wider type has no exact fp16 image: reduce it with torch, it is still one pass
        return tensor.float().view(heads, seq_len, head_dim // group_size, group_size).abs().amax(dim=3).amax(dim=1)
    return ops.group_absmax(tensor if tensor.stride(-1) == 1 else tensor.contiguous(), group_size)


def collect_absmax_samples(kv_samples: Sequence[Sequence[torch.Tensor]], group_size: int) -> List[List[torch.Tensor]]:
    """list over samples -> list over layers -> [kv_heads, seq, head_dim]  =>
    list over layers -> list over samples -> [kv_heads, num_groups]."""
    if not kv_samples:
        return []
    num_layers = len(kv_samples[0])
    out: List[List[torch.Tensor]] = [[] for _ in range(num_layers)]
    for sample in kv_samples:
        for layer_idx in range(num_layers):
            out[layer_idx].append(compute_absmax_per_group(sample[layer_idx], group_size))
    return out


def scales_from_absmax_samples(absmax_samples: Sequence[Sequence[torch.Tensor]], clip_percentile: float,
                               qmax: int) -> List[torch.Tensor]:
    """Per-layer static scales: percentile over the samples of the per-sample absmax, / qmax, >= 1e-5 / qmax."""
    scales: List[torch.Tensor] = []
    for layer_idx, per_layer in enumerate(absmax_samples):
        if not per_layer:
            raise ValueError(f"absmax_samples[{layer_idx}] is empty - no calibration samples collected for layer "
                             f"{layer_idx}. Check that num_layers matches the model.")
        stack = torch.stack(list(per_layer), dim=0).float()
        absmax = torch.quantile(stack, clip_percentile / 100.0, dim=0)
        scales.append(absmax.clamp(min=1e-5) / float(qmax))
    return scales


def save_calibration(path: str, k_scale: Sequence[torch.Tensor], v_scale: Sequence[torch.Tensor], *, group_size: int,
                     clip_percentile: float, inv_tau: Optional[torch.Tensor] = None, int4_outlier_ratio: float = 0.0,
                     int4_mixed_rescue: bool = False, extra: Optional[dict] = None) -> dict:
    """Write the version-2 calibration JSON; returns the dictionary written."""
    if len(k_scale) != len(v_scale):
        raise ValueError("k_scale and v_scale must cover the same layers")
    doc = {
        "version": 2,
        "group_size_k": int(group_size), "group_size_v": int(group_size),
        "clip_percentile_k": float(clip_percentile), "clip_percentile_v": float(clip_percentile),
        "k_scale": [t.detach().float().cpu().tolist() for t in k_scale],
        "v_scale": [t.detach().float().cpu().tolist() for t in v_scale],
        "int4_outlier_ratio": float(int4_outlier_ratio), "int4_mixed_rescue": bool(int4_mixed_rescue),
    }
    if inv_tau is not None:
        doc["inv_tau"] = inv_tau.detach().float().cpu().tolist()
    if extra:
        doc.update(extra)
    with open(path, "w") as f:
        json.dump(doc, f)
    return doc
