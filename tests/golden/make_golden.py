#!/usr/bin/env python3
"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE.

Usage (only where the reference checkout is available):

    python tests/golden/make_golden.py --reference /path/to/LLM_KVCache_Quantization

The reference's own classes and functions are imported unmodified
(`INT8KVCache`, `INT4KVCache`, `quantize_asymmetric`, `pack_int4`,
`_decode_attn_int8_torch_ref`, `_apply_rope`, `KIVIStyleKVCache`, `apply_int8_fused_patch`,
`INT8CacheWrapperContainer`, `_register_prefill_temperature_hooks`) and driven on seeded inputs on CPU; inputs and
outputs are stored as small `.npz` files.  The fixtures travel with the
repository, the reference does not.
"""
import argparse
import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    return t.detach().cpu().numpy()


def gen_kv(gen, b, h, s, d, outlier_ch=0, outlier_mag=20.0, chan_std=False):
    x = torch.randn(b, h, s, d, generator=gen)
    if chan_std:
        std = torch.exp(torch.empty(1, h, 1, d).uniform_(np.log(0.3), np.log(3.0), generator=gen))
        x = x * std
    if outlier_ch:
        for hh in range(h):
            ch = torch.randperm(d, generator=gen)[:outlier_ch]
            x[:, hh, :, ch] *= outlier_mag
    return x.to(torch.float16)


def make_rope():
    """Rotate-half RoPE of the patched forward (src/engine/patch_model.py:223-278) in fp16 on CPU:
    full and partial rotary dims, cos/sin of rank 2, 3 and 4, batch-shared and per-row tables."""
    from src.engine.patch_model import _apply_rope
    gen = torch.Generator().manual_seed(20261126)
    out = {}
    cases = (("full_r3", 2, 12, 2, 3, 128, 128, 3), ("partial_r3", 2, 6, 2, 1, 128, 64, 3),
             ("shared_r2", 1, 4, 4, 5, 128, 128, 2), ("decode_r4", 3, 14, 2, 1, 128, 128, 4),
             ("d64_r3", 2, 4, 2, 2, 64, 64, 3))
    for name, b, hq, hkv, t, d, rd, rank in cases:
        q = (torch.randn(b, hq, t, d, generator=gen) * 2).half()
        k = (torch.randn(b, hkv, t, d, generator=gen) * 2).half()
        pos = torch.randint(0, 4096, (b, t), generator=gen).float()
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, rd, 2).float() / rd))
        ang = pos[..., None] * inv_freq                       # [b, t, rd/2]
        emb = torch.cat([ang, ang], dim=-1)
        cos, sin = emb.cos().half(), emb.sin().half()         # [b, t, rd]
        if rank == 2:
            cos_in, sin_in = cos[0], sin[0]                   # [t, rd], shared by the batch (b == 1)
        elif rank == 4:
            cos_in, sin_in = cos[:, None], sin[:, None]
        else:
            cos_in, sin_in = cos, sin
        q_emb, k_emb = _apply_rope(q, k, cos_in, sin_in)
        out[f"{name}_q"] = _np(q); out[f"{name}_k"] = _np(k)
        out[f"{name}_cos"] = _np(cos_in); out[f"{name}_sin"] = _np(sin_in)
        out[f"{name}_q_out"] = _np(q_emb); out[f"{name}_k_out"] = _np(k_emb)
    np.savez_compressed(os.path.join(HERE, "rope.npz"), **out)
    print("rope.npz", os.path.getsize(os.path.join(HERE, "rope.npz")) // 1024, "KiB")


def make_kivi():
    """KIVIStyleKVCache (src/cache/kivi_style_cache.py) on CPU: a prompt, then single-token appends; INT4 and
    INT8; payloads, per-channel K and per-token V parameters, and get_kv."""
    from src.cache.kivi_style_cache import KIVIStyleKVCache
    gen = torch.Generator().manual_seed(20261127)
    out = {}
    B, H, P, N, D = 2, 2, 37, 3, 128
    k = gen_kv(gen, B, H, P + N, D, outlier_ch=2)
    v = gen_kv(gen, B, H, P + N, D, chan_std=True)
    k[:, :, P + 1] *= 3.0                        # a decode token outside the prompt's range: clipped codes
    out["k"], out["v"], out["prompt"] = _np(k), _np(v), np.array(P)
    for bits in (4, 8):
        c = KIVIStyleKVCache(num_layers=1, device="cpu", quant_bits=bits)
        c.append(0, k[:, :, :P], v[:, :, :P])
        for t in range(P, P + N):
            c.append(0, k[:, :, t:t + 1], v[:, :, t:t + 1])
        S = P + N
        out[f"b{bits}_k_payload"] = _np(c._k_cache[0][:, :, :S])
        out[f"b{bits}_v_payload"] = _np(c._v_cache[0][:, :, :S])
        out[f"b{bits}_k_scale"], out[f"b{bits}_k_zp"] = _np(c._k_scale[0]), _np(c._k_zp[0])
        out[f"b{bits}_v_scale"], out[f"b{bits}_v_zp"] = _np(c._v_scale[0][:, :, :S]), _np(c._v_zp[0][:, :, :S])
        kd, vd = c.get_kv(0)
        out[f"b{bits}_k_deq"], out[f"b{bits}_v_deq"] = _np(kd), _np(vd)
    # fp16 residual window: the newest `residual_length` decode tokens stay unquantized, older ones are
    # quantized as they leave the window
    R, N2 = 4, 7
    k2 = gen_kv(gen, B, H, P + N2, D, outlier_ch=2)
    v2 = gen_kv(gen, B, H, P + N2, D)
    out["res_k"], out["res_v"], out["res_len"] = _np(k2), _np(v2), np.array(R)
    c = KIVIStyleKVCache(num_layers=1, device="cpu", quant_bits=4, residual_length=R)
    c.append(0, k2[:, :, :P], v2[:, :, :P])
    for t in range(P, P + N2):
        c.append(0, k2[:, :, t:t + 1], v2[:, :, t:t + 1])
    nq = c._layer_seq_lens[0]
    out["res_quantized_len"], out["res_seq_len"] = np.array(nq), np.array(c.get_seq_len())
    out["res_k_payload"], out["res_v_payload"] = _np(c._k_cache[0][:, :, :nq]), _np(c._v_cache[0][:, :, :nq])
    kd, vd = c.get_kv(0)
    out["res_k_deq"], out["res_v_deq"] = _np(kd), _np(vd)
    np.savez_compressed(os.path.join(HERE, "kivi.npz"), **out)
    print("kivi.npz", os.path.getsize(os.path.join(HERE, "kivi.npz")) // 1024, "KiB")


def make_kivi_percentile():
    """KIVIStyleKVCache and RoleAwareAsymKVCache (src/cache/role_aware_asym_cache.py) with clipping percentiles
    below 100 on CPU: K bounds = torch.quantile over the prompt's tokens, V bounds = torch.quantile over the head
    dimension of every token (src/quant/asymmetric_quant.py:98-106); a prompt, then single-token appends."""
    from src.cache.kivi_style_cache import KIVIStyleKVCache
    from src.cache.role_aware_asym_cache import RoleAwareAsymKVCache
    gen = torch.Generator().manual_seed(20261128)
    out = {}
    B, H, P, N, D = 2, 2, 45, 3, 128
    k = gen_kv(gen, B, H, P + N, D, outlier_ch=2)
    v = gen_kv(gen, B, H, P + N, D, chan_std=True)
    out["k"], out["v"], out["prompt"] = _np(k), _np(v), np.array(P)
    cases = (("kivi", KIVIStyleKVCache, 4, 99.0, 99.9), ("kivi", KIVIStyleKVCache, 8, 97.5, 90.0),
             ("role", RoleAwareAsymKVCache, 4, 99.5, 98.5))
    out["cases"] = np.array([[bits, kp, vp] for _, _, bits, kp, vp in cases], dtype=np.float64)
    for i, (_, cls, bits, kp, vp) in enumerate(cases):
        c = cls(num_layers=1, device="cpu", quant_bits=bits, k_percentile=kp, v_percentile=vp)
        c.append(0, k[:, :, :P], v[:, :, :P])
        for t in range(P, P + N):
            c.append(0, k[:, :, t:t + 1], v[:, :, t:t + 1])
        S = P + N
        out[f"c{i}_k_payload"] = _np(c._k_cache[0][:, :, :S])
        out[f"c{i}_v_payload"] = _np(c._v_cache[0][:, :, :S])
        out[f"c{i}_k_scale"], out[f"c{i}_k_zp"] = _np(c._k_scale[0]), _np(c._k_zp[0])
        out[f"c{i}_v_scale"], out[f"c{i}_v_zp"] = _np(c._v_scale[0][:, :, :S]), _np(c._v_zp[0][:, :, :S])
        kd, vd = c.get_kv(0)
        out[f"c{i}_k_deq"], out[f"c{i}_v_deq"] = _np(kd), _np(vd)
        if cls is RoleAwareAsymKVCache:
            out["role_framework"] = np.array(c.framework)
            out["role_ba_calibrated"] = np.array(bool(c.ba_calibrated))
    np.savez_compressed(os.path.join(HERE, "kivi_pct.npz"), **out)
    print("kivi_pct.npz", os.path.getsize(os.path.join(HERE, "kivi_pct.npz")) // 1024, "KiB")


def make_calibration(reference_root):
    """Two fixtures of the calibration row:
    calib_absmax.npz - `compute_absmax_per_group` (scripts/calibrate_behavior.py:228-260) on seeded K tensors, per
    sample and as the running maximum over samples that the collection loop keeps;
    calib_schema.json - the schema of the calibration file the reference ships (artifacts/kv_calib_mse_1p5b_int8.json):
    every key, with the per-layer tables cut to the first two layers, so that the loader is tested on the real layout."""
    import json
    import types
    for name in ("matplotlib", "matplotlib.pyplot", "datasets"):      # plotting / dataset imports of the script's CLI
        if name not in sys.modules:
            try:
                __import__(name)
            except Exception:
                sys.modules[name] = types.ModuleType(name)
    from scripts.calibrate_behavior import compute_absmax_per_group
    gen = torch.Generator().manual_seed(20261129)
    H, S, D, n = 2, 67, 128, 2
    xs = [(torch.randn(H, S, D, generator=gen) * torch.exp(torch.randn(H, 1, D, generator=gen))).half() for _ in range(n)]
    out = {"x": np.stack([_np(x) for x in xs])}
    for gs in (16, 32, 128):
        per = [compute_absmax_per_group(x, gs).float() for x in xs]
        out[f"g{gs}_per_sample"] = np.stack([_np(p) for p in per])
        out[f"g{gs}_running_max"] = _np(torch.stack(per).amax(0))
    np.savez_compressed(os.path.join(HERE, "calib_absmax.npz"), **out)
    print("calib_absmax.npz", os.path.getsize(os.path.join(HERE, "calib_absmax.npz")) // 1024, "KiB")
    with open(os.path.join(reference_root, "artifacts", "kv_calib_mse_1p5b_int8.json")) as f:
        full = json.load(f)
    keep = 2
    cut = {}
    for key, val in full.items():
        if key in ("k_scale", "v_scale", "inv_tau"):
            cut[key] = val[:keep]
        elif key == "selection":
            cut[key] = {k2: (v2 if not isinstance(v2, (list, dict)) else type(v2)()) for k2, v2 in val.items()}
        else:
            cut[key] = val
    cut["num_layers_in_shipped_file"] = full["num_layers"]
    cut["shapes_in_shipped_file"] = {k2: list(np.asarray(full[k2]).shape) for k2 in ("k_scale", "v_scale", "inv_tau")}
    with open(os.path.join(HERE, "calib_schema.json"), "w") as f:
        json.dump(cut, f)
    print("calib_schema.json", os.path.getsize(os.path.join(HERE, "calib_schema.json")) // 1024, "KiB")


ENGINE_GEOMETRY = dict(vocab_size=48, hidden_size=256, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=128, max_position_embeddings=64, rope_theta=10000.0,
                       tie_word_embeddings=False)


def tiny_qwen2(seed=1234):
    """The seeded random-init Qwen2 of the engine fixture (CPU, fp16): 2 layers, 2 query heads over 1 KV head of
    128 channels.  Deterministic for a given torch build; the fixture stores a checksum of the weights."""
    import transformers
    cfg = transformers.Qwen2Config(**ENGINE_GEOMETRY)
    torch.manual_seed(seed)
    model = transformers.Qwen2ForCausalLM(cfg).eval()
    # spread the logits: the default init (std 0.02) gives near-uniform attention, a weak test of the temperature
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if "q_proj" in name or "k_proj" in name:
                prm.mul_(6.0)
    return model.half()


def weights_checksum(model):
    return float(sum(p.detach().double().abs().sum() for p in model.parameters()))


def make_engine():
    """The reference's patched attention forward end to end on CPU (src/engine/patch_model.py:645-1211 through
    apply_int8_fused_patch + INT8CacheWrapperContainer, caches with decode_attn_impl="torch_ref", prefill with
    _register_prefill_temperature_hooks, src/engine/generate_loop.py:276-390): prompt of 7 tokens x batch 2, three
    greedy decode steps, static scales and per-head inverse temperatures of a calibration file's shape.  Stored:
    the prompt, the calibration, the prefill K/V the reference's model produced, the logits of the prefill and of
    every decode step, and the final cache tensors.  `generate_from_ids` itself refuses to run without CUDA
    (src/engine/generate_loop.py:600-603), so the loop is driven here as it drives it."""
    from src.cache.int8_cache import INT8KVCache
    from src.cache.int4_cache import INT4KVCache
    from src.engine.patch_model import (INT8CacheWrapperContainer, apply_int8_fused_patch, remove_int8_fused_patch)
    from src.engine.generate_loop import _register_prefill_temperature_hooks
    gen = torch.Generator().manual_seed(20261127)
    L, Hq, Hkv, D, gs = 2, 2, 1, 128, 32
    G = D // gs
    out = {"weights_checksum": np.array(0.0)}
    prompt = torch.randint(0, ENGINE_GEOMETRY["vocab_size"], (2, 7), generator=gen)
    out["prompt"] = _np(prompt)
    inv_tau = torch.empty(L, Hq).uniform_(0.7, 1.3, generator=gen)
    out["inv_tau"] = _np(inv_tau)
    for mode in ("int8_ours", "int4_ours", "int4_ours_mixed"):
        model = tiny_qwen2()
        out["weights_checksum"] = np.array(weights_checksum(model))
        qmax = 127.0 if mode.startswith("int8") else 7.0
        sdt = torch.float16 if mode.startswith("int8") else torch.float32      # generate_loop.py:816-820
        ks = (torch.empty(L, Hkv, G).uniform_(1.5, 4.0, generator=gen) / qmax).to(sdt)
        vs = (torch.empty(L, Hkv, G).uniform_(0.05, 0.2, generator=gen) / qmax).to(sdt)
        out[f"{mode}_k_scale"], out[f"{mode}_v_scale"] = _np(ks.float()), _np(vs.float())
        common = dict(device="cpu", group_size=gs, decode_attn_impl="torch_ref", static_k_scale=ks, static_v_scale=vs,
                      inv_tau=inv_tau, use_attn_temperature=True)
        if mode.startswith("int8"):
            cache = INT8KVCache(L, **common)
        else:
            cache = INT4KVCache(L, mixed_rescue=(mode == "int4_ours_mixed"), **common)
        handles = _register_prefill_temperature_hooks(model, inv_tau)
        apply_int8_fused_patch(model)
        try:
            with torch.no_grad():
                o = model(input_ids=prompt, attention_mask=torch.ones_like(prompt), use_cache=True)
                pk, pv = [], []
                for i, item in enumerate(o.past_key_values):
                    k, v = item[0], item[1]
                    pk.append(k); pv.append(v)
                    cache.append(i, k, v)
                out[f"{mode}_prefill_k"] = _np(torch.stack(pk)); out[f"{mode}_prefill_v"] = _np(torch.stack(pv))
                out[f"{mode}_prefill_logits"] = _np(o.logits[:, -1].float())
                tok = o.logits[:, -1].argmax(-1, keepdim=True)
                toks, step_logits = [tok], []
                container = INT8CacheWrapperContainer(cache, L)
                for step in range(3):
                    pos = torch.full((2, 1), prompt.shape[1] + step, dtype=torch.long)
                    o = model(input_ids=tok, position_ids=pos, past_key_values=container, use_cache=True)
                    step_logits.append(o.logits[:, -1].float())
                    tok = o.logits[:, -1].argmax(-1, keepdim=True)
                    toks.append(tok)
                out[f"{mode}_tokens"] = _np(torch.cat(toks, 1)); out[f"{mode}_step_logits"] = _np(torch.stack(step_logits))
                for i in range(L):
                    t = cache.get_int8_tensors(i) if mode.startswith("int8") else cache.get_int4_tensors(i)
                    for name, x in zip(("qk", "qv", "sk", "sv"), t):
                        out[f"{mode}_l{i}_{name}"] = _np(x)
        finally:
            for h in handles:
                h.remove()
            remove_int8_fused_patch(model)
    np.savez_compressed(os.path.join(HERE, "engine.npz"), **out)
    print("engine.npz", os.path.getsize(os.path.join(HERE, "engine.npz")) // 1024, "KiB")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--only", default="", help="'rope' / 'kivi' / 'kivi_pct' / 'calib' / 'engine': regenerate that fixture alone")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    warnings.simplefilter("ignore")
    if args.only == "rope":
        make_rope()
        return
    if args.only == "kivi_pct":
        make_kivi_percentile()
        return
    if args.only == "calib":
        make_calibration(args.reference)
        return
    if args.only == "kivi":
        make_kivi()
        return
    if args.only == "engine":
        make_engine()
        return

    from src.cache.int8_cache import INT8KVCache
    from src.cache.int4_cache import INT4KVCache
    from src.quant.asymmetric_quant import quantize_asymmetric, dequantize_asymmetric
    from src.quant.int4_basic import pack_int4, unpack_int4
    from src.engine.patch_model import _decode_attn_int8_torch_ref

    torch.manual_seed(0)
    gen = torch.Generator().manual_seed(20261125)

    # ------------------------------------------------------------------ quantizers
    out = {}
    B, H, S, D = 2, 2, 37, 128
    for gs in (16, 32, 64, 128):
        G = D // gs
        k = gen_kv(gen, B, H, S, D, outlier_ch=4)
        v = gen_kv(gen, B, H, S, D, chan_std=True)
        # make some exact ties / clamp cases / tiny values
        k[0, 0, 0, :8] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, 1e-4, 6e-8, 0.0]).half()
        calib_k = gen_kv(gen, 4, H, 64, D, outlier_ch=0).float().abs().view(4, H, 64, G, gs).amax(dim=(0, 2, 4))
        calib_v = gen_kv(gen, 4, H, 64, D, chan_std=True).float().abs().view(4, H, 64, G, gs).amax(dim=(0, 2, 4))
        out[f"g{gs}_k"] = _np(k)
        out[f"g{gs}_v"] = _np(v)
        # --- INT8 static, fp16 calibration scales (generate_loop.py:816-817)
        ks8 = (calib_k / 127.0).to(torch.float16)
        vs8 = (calib_v / 127.0).to(torch.float16)
        ks8[0, 0] = 0.0  # exercises the 1e-5 clamp
        out[f"g{gs}_int8_static_ks_in"] = _np(ks8)
        out[f"g{gs}_int8_static_vs_in"] = _np(vs8)
        c = INT8KVCache(1, device="cpu", group_size=gs, static_k_scale=ks8[None], static_v_scale=vs8[None])
        c.append(0, k, v)
        qk, qv, sk, sv = c.get_int8_tensors(0)
        out[f"g{gs}_int8_static_qk"] = _np(qk); out[f"g{gs}_int8_static_qv"] = _np(qv)
        out[f"g{gs}_int8_static_sk"] = _np(sk); out[f"g{gs}_int8_static_sv"] = _np(sv)
        # --- INT8 adaptive static
        c = INT8KVCache(1, device="cpu", group_size=gs, static_k_scale=ks8[None], static_v_scale=vs8[None],
                        adaptive_static_scales=True, adaptive_static_margin=0.9)
        c.append(0, k, v)
        qk, qv, sk, sv = c.get_int8_tensors(0)
        out[f"g{gs}_int8_adapt_qk"] = _np(qk); out[f"g{gs}_int8_adapt_qv"] = _np(qv)
        out[f"g{gs}_int8_adapt_sk"] = _np(sk); out[f"g{gs}_int8_adapt_sv"] = _np(sv)
        # --- INT8 dynamic
        for p in (99.9, 100.0, 95.0):
            c = INT8KVCache(1, device="cpu", group_size=gs, clip_percentile=p)
            c.append(0, k, v)
            qk, qv, sk, sv = c.get_int8_tensors(0)
            out[f"g{gs}_int8_dyn{p}_qk"] = _np(qk); out[f"g{gs}_int8_dyn{p}_qv"] = _np(qv)
            out[f"g{gs}_int8_dyn{p}_sk"] = _np(sk); out[f"g{gs}_int8_dyn{p}_sv"] = _np(sv)
        # --- INT4 static (fp32 calibration scales, generate_loop.py:818-820)
        ks4 = (calib_k / 7.0).float()
        vs4 = (calib_v / 7.0).float()
        ks4[0, 0] = 0.0
        out[f"g{gs}_int4_static_ks_in"] = _np(ks4)
        out[f"g{gs}_int4_static_vs_in"] = _np(vs4)
        variants = {
            "static": dict(),
            "mixed": dict(mixed_rescue=True),
            "rescue": dict(outlier_rescue_ratio=0.05),
            "rescue1": dict(outlier_rescue_ratio=1.0),
            "adapt": dict(adaptive_static_scales=True, adaptive_static_margin=1.1),
        }
        for name, kw in variants.items():
            c = INT4KVCache(1, device="cpu", group_size=gs, static_k_scale=ks4[None], static_v_scale=vs4[None], **kw)
            c.append(0, k, v)
            qk, qv, sk, sv = c.get_int4_tensors(0)
            out[f"g{gs}_int4_{name}_qk"] = _np(qk); out[f"g{gs}_int4_{name}_qv"] = _np(qv)
            out[f"g{gs}_int4_{name}_sk"] = _np(sk); out[f"g{gs}_int4_{name}_sv"] = _np(sv)
        for p in (99.9, 100.0):
            c = INT4KVCache(1, device="cpu", group_size=gs, clip_percentile=p)
            c.append(0, k, v)
            qk, qv, sk, sv = c.get_int4_tensors(0)
            out[f"g{gs}_int4_dyn{p}_qk"] = _np(qk); out[f"g{gs}_int4_dyn{p}_qv"] = _np(qv)
            out[f"g{gs}_int4_dyn{p}_sk"] = _np(sk); out[f"g{gs}_int4_dyn{p}_sv"] = _np(sv)
        # --- group-wise asymmetric INT4 = generic quantize_asymmetric on a grouped view
        for nm, t in (("k", k), ("v", v)):
            q, s, z = quantize_asymmetric(t.view(B, H, S, G, gs), axis=-1, quant_bits=4)
            out[f"g{gs}_asym_q{nm}"] = _np(pack_int4(q.view(B, H, S, D)))
            out[f"g{gs}_asym_s{nm}"] = _np(s); out[f"g{gs}_asym_z{nm}"] = _np(z)
            deq = dequantize_asymmetric(q, s.half(), z.half(), axis=-1).view(B, H, S, D)
            out[f"g{gs}_asym_deq{nm}"] = _np(deq)
    np.savez_compressed(os.path.join(HERE, "quantizers.npz"), **out)

    # ------------------------------------------------------------------ pack / unpack
    allv = torch.arange(-8, 8, dtype=torch.int8)
    pairs = torch.stack(torch.meshgrid(allv, allv, indexing="ij"), -1).reshape(1, 1, 16, 32)
    packed = pack_int4(pairs)
    np.savez_compressed(os.path.join(HERE, "pack_int4.npz"), codes=_np(pairs), packed=_np(packed),
                        unpacked=_np(unpack_int4(packed)))

    # ------------------------------------------------------------------ attention
    att = {}
    cases = {
        # name: (B, Hq, Hkv, S, gs, kind, outlier_ch, ctx)
        "c1_small": (1, 12, 2, 300, 32, "int8", 4, [300]),
        "gqa7_ragged": (3, 28, 4, 129, 32, "int8", 0, [129, 1, 64]),
        "zero_ctx": (2, 8, 2, 40, 64, "int8", 0, [0, 40]),
        "int4_g32": (2, 12, 2, 200, 32, "int4", 0, [200, 77]),
        "int4_g16": (1, 40, 8, 96, 16, "int4", 0, [96]),
        "mha_g128": (2, 4, 4, 65, 128, "int8", 0, [65, 33]),
    }
    for name, (b, hq, hkv, s, gs, kind, och, ctx) in cases.items():
        d = 128
        q = torch.randn(b, hq, d, generator=gen).half()
        k = gen_kv(gen, b, hkv, s, d, outlier_ch=och)
        v = gen_kv(gen, b, hkv, s, d, outlier_ch=och)
        inv_tau = torch.empty(hq).uniform_(0.8, 1.2, generator=gen)
        g = d // gs
        if kind == "int8":
            sc_k = (k.float().abs().view(b, hkv, s, g, gs).amax(dim=(0, 2, 4)) / 127.0).half()
            sc_v = (v.float().abs().view(b, hkv, s, g, gs).amax(dim=(0, 2, 4)) / 127.0).half()
            c = INT8KVCache(1, device="cpu", group_size=gs, static_k_scale=sc_k[None], static_v_scale=sc_v[None])
            c.append(0, k, v)
            qk, qv, sk, sv = c.get_int8_tensors(0)
            k8, v8 = qk, qv
        else:
            sc_k = (k.float().abs().view(b, hkv, s, g, gs).amax(dim=(0, 2, 4)) / 7.0).float()
            sc_v = (v.float().abs().view(b, hkv, s, g, gs).amax(dim=(0, 2, 4)) / 7.0).float()
            c = INT4KVCache(1, device="cpu", group_size=gs, static_k_scale=sc_k[None], static_v_scale=sc_v[None])
            c.append(0, k, v)
            qk, qv, sk, sv = c.get_int4_tensors(0)
            k8, v8 = unpack_int4(qk), unpack_int4(qv)
        # inv_tau applied in fp16 before the kernel (patch_model.py:712-746)
        q_scaled = q * inv_tau.to(torch.float16).view(1, -1, 1)
        ctx_t = torch.tensor(ctx, dtype=torch.int32)
        sm = 1.0 / (d ** 0.5)
        ref = _decode_attn_int8_torch_ref(q_scaled, k8, v8, sk.half(), sv.half(), ctx_t, sm)
        att[f"{name}_q"] = _np(q); att[f"{name}_inv_tau"] = _np(inv_tau)
        att[f"{name}_k"] = _np(qk); att[f"{name}_v"] = _np(qv)
        att[f"{name}_ks"] = _np(sk.half()); att[f"{name}_vs"] = _np(sv.half())
        att[f"{name}_ctx"] = _np(ctx_t); att[f"{name}_out"] = _np(ref)
        att[f"{name}_meta"] = np.array([b, hq, hkv, s, gs, 1 if kind == "int4" else 0])
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **att)
    for f in ("quantizers.npz", "pack_int4.npz", "attention.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")
    make_rope()
    make_kivi()
    make_kivi_percentile()
    make_calibration(args.reference)
    make_engine()


if __name__ == "__main__":
    main()
