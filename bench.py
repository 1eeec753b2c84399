#!/usr/bin/env python3
"""Benchmark of the quantized-KV decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2]

One "step" = one decode step over the whole KV stack of the workload: for every
layer, quantize-on-append of the new token (one launch for K and V) followed by
the fused decode attention (split-K kernel + combine) over the cached context.
Default workload is configuration 2 of the benchmark definition (Qwen2.5-1.5B geometry, 28
layers, batch 16, context 8192, INT4 asymmetric group-32 with fp16 scale and
zero-point).  With N > 1 the batch is sharded by sequence: every rank owns its own
batch of sequences and its own cache, no collective on the data path (weak scaling).
The single-sequence workload c5 with N > 1 shards the KV sequence instead: every rank
scans its contiguous chunk, the packed partials cross NVLink in one NCCL all-gather per
layer and are merged on every rank (strong scaling: the total work is fixed).

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: layers, B, Hq, Hkv, S, kind, n_out
    "c1": dict(layers=1, B=1, Hq=12, Hkv=2, S=4096, kind="int8_static", n_out=0,
               desc="C1: 1 layer, Qwen2.5-1.5B geometry, batch 1, ctx 4096, INT8 static group-32"),
    "c2": dict(layers=28, B=16, Hq=12, Hkv=2, S=8192, kind="int4_asym", n_out=0,
               desc="C2: 28-layer KV stack, Qwen2.5-1.5B geometry (12q/2kv heads, d128), batch 16, ctx 8192, "
                    "INT4 asymmetric group-32 (fp16 scale+zero-point), decode step incl. quantize-on-append"),
    "c3": dict(layers=28, B=32, Hq=12, Hkv=2, S=16384, kind="int4_outlier", n_out=3,
               desc="C3: 28-layer KV stack, Qwen2.5-1.5B geometry, batch 32, ctx 16384, INT4 group-32 + 3 fp16 outlier "
                    "channels"),
    "c4": dict(layers=28, B=64, Hq=28, Hkv=4, S=32768, kind="int8_dyn", n_out=0,
               desc="C4: 28-layer KV stack (64 GB), Qwen2.5-7B geometry, batch 64, ctx 32768, INT8 group-32"),
    "c2_fp16": dict(layers=28, B=16, Hq=12, Hkv=2, S=8192, kind="fp16", n_out=0,
                    desc="config-2 shape with an UNQUANTISED fp16 cache (comparison point): 28-layer KV stack, batch 16, "
                         "ctx 8192"),
    "c2_kivi4": dict(layers=28, B=16, Hq=12, Hkv=2, S=8192, kind="kivi4", n_out=0,
                     desc="config-2 shape with the KIVI-format cache: per-channel K / per-token V asymmetric INT4, "
                          "28-layer KV stack, batch 16, ctx 8192"),
    "c5": dict(layers=48, B=1, Hq=40, Hkv=8, S=131072, kind="int4_outlier", n_out=1,
               desc="C5: 48-layer KV stack, Qwen2.5-14B geometry, batch 1, ctx 131072, INT4 group-32 + 1 fp16 outlier "
                    "channel"),
}
D = 128
GS = 32
G = D // GS


# DRAM traffic / algorithmic bytes of the split-K scan, from the ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch of the same kernel, scaled by token-heads)
NCU_TRAFFIC_RATIO = {"kivi4": 1.0, "fp16": 1.0, "int4_asym": 1.003, "int8_dyn": 1.004, "int8_static": 1.004, "int4_outlier": 1.028}


def bytes_per_token_head(kind: str, n_out: int) -> int:
    """Algorithmic HBM bytes per cached token per KV head (K and V): payload + per-token
    fp16 scales (+ zero-points) (+ fp16 outlier side values), each counted once."""
    if kind == "fp16":
        return 2 * 2 * D
    if kind == "kivi4":               # packed K and V rows + the four fp16 per-token tiles the fused kernel reads
        return 2 * (D // 2) + 4 * 2
    if kind in ("int8_static", "int8_dyn"):
        return 2 * (D + 2 * G)
    if kind == "int4_asym":
        return 2 * (D // 2 + 2 * G + 2 * G)
    if kind == "int4_outlier":
        return 2 * (D // 2 + 2 * G + 2 * n_out)
    raise ValueError(kind)


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- workload
def build_workload(wl: dict, dev, seed: int, extra_slots: int):
    """Synthetic KV of the configuration's shape and value distribution, generated on the
    GPU layer by layer and quantized with the library's own quantizer into a preallocated cache."""
    import numpy as np
    import torch
    import llm_kvcache_quantization_b200 as kvq

    L, B, Hq, Hkv, S, kind, n_out = (wl[k] for k in ("layers", "B", "Hq", "Hkv", "S", "kind", "n_out"))
    gen = torch.Generator(device=dev).manual_seed(seed)
    cap = S + extra_slots
    kw = dict(device=dev, group_size=GS, max_seq_len=cap)
    outlier_idx = None
    if kind == "fp16":
        cache = kvq.FP16KVCache(L, device=dev, max_seq_len=cap)
    elif kind == "kivi4":
        cache = kvq.KIVIStyleKVCache(L, device=dev, quant_bits=4, max_seq_len=cap)
    elif kind == "int8_static":
        tab = torch.full((L, Hkv, G), 4.5 / 127, dtype=torch.float16, device=dev)
        cache = kvq.INT8KVCache(L, static_k_scale=tab, static_v_scale=tab, **kw)
    elif kind == "int8_dyn":
        cache = kvq.INT8KVCache(L, clip_percentile=100.0, **kw)
    elif kind == "int4_asym":
        cache = kvq.INT4KVCache(L, asymmetric=True, **kw)
    else:
        cpu_gen = torch.Generator().manual_seed(seed)
        outlier_idx = torch.stack([torch.stack([torch.randperm(D, generator=cpu_gen)[:n_out].sort().values
                                                for _ in range(Hkv)]) for _ in range(L)]).to(torch.int16)
        tab = torch.full((L, Hkv, G), 4.5 / 7, dtype=torch.float32, device=dev)
        cache = kvq.INT4KVCache(L, static_k_scale=tab, static_v_scale=tab, outlier_idx=outlier_idx.to(dev), **kw)
    chunk = max(1, min(S, (1 << 26) // (B * Hkv * D)))       # <= 128 MB fp16 per generated chunk
    for l in range(L):
        if kind == "kivi4":
            cache._ensure_capacity(l, B, Hkv, D, cap)
        else:
            cache.reserve(l, B, Hkv, D, cap)
        if kind == "int4_asym":
            std = torch.exp(torch.empty(1, Hkv, 1, D, device=dev).uniform_(np.log(0.3), np.log(3.0), generator=gen))
        else:
            std = torch.ones(1, Hkv, 1, D, device=dev)
            if outlier_idx is not None:
                for h in range(Hkv):
                    std[0, h, 0, outlier_idx[l, h].long().to(dev)] = 30.0
        for s0 in range(0, S, chunk):
            n = min(chunk, S - s0)
            k = (torch.randn(B, Hkv, n, D, device=dev, generator=gen) * std).half()
            v = (torch.randn(B, Hkv, n, D, device=dev, generator=gen) * std).half()
            cache.append(l, k, v)
            del k, v
    q = torch.randn(L, B, Hq, D, device=dev, generator=gen).half()
    k_new = torch.randn(L, B, Hkv, 1, D, device=dev, generator=gen).half()
    v_new = torch.randn(L, B, Hkv, 1, D, device=dev, generator=gen).half()
    inv_tau = torch.empty(L, Hq, device=dev).uniform_(0.8, 1.2, generator=gen)
    return cache, q, k_new, v_new, inv_tau


def make_kivi_step(wl, cache, q, k_new, v_new, inv_tau, out, stages=0, with_append=True):
    """Decode step over the KIVI-format cache: per layer the single-token append (slot S every step) and the
    fused decode (per-channel K scale applied to the query inside the kernel, factored-scale path over the
    packed cache)."""
    import torch
    from llm_kvcache_quantization_b200 import ops, _lib
    L, B, Hq, Hkv, S = wl["layers"], wl["B"], wl["Hq"], wl["Hkv"], wl["S"]
    n = S + 1

    def step():
        for l in range(L):
            if with_append:
                cache._layer_seq_lens[l] = S
                cache.append(l, k_new[l], v_new[l])
            ops.decode_attn(_lib.FMT_INT4, q[l], cache._k_cache[l][:, :, :n], cache._v_cache[l][:, :, :n],
                            cache._k_ones[l][:, :, :n], cache._v_scale16[l][:, :, :n], None, 1.0 / D ** 0.5, head_dim=D,
                            k_zp=cache._k_zeros[l][:, :, :n], v_zp=cache._v_zp16[l][:, :, :n], inv_tau=inv_tau[l],
                            out=out[l], fast_dequant=True, stages=stages, q_chan_scale=cache._k_scale[l])
    return step, (lambda: ops.last_splits())


def make_step(wl, cache, q, k_new, v_new, inv_tau, out, stages=0, with_append=True):
    """Returns a callable running one decode step with device-resident inputs.  The new
    token is written at slot S every step (steady state at the nominal context)."""
    import torch
    from llm_kvcache_quantization_b200 import ops, _lib

    if wl["kind"] == "kivi4":
        return make_kivi_step(wl, cache, q, k_new, v_new, inv_tau, out, stages, with_append)
    L, B, Hkv, S, kind = wl["layers"], wl["B"], wl["Hkv"], wl["S"], wl["kind"]
    dev = q.device
    ctx = torch.full((B,), S + 1, dtype=torch.int32, device=dev)
    fmt = _lib.FMT_FP16 if kind == "fp16" else _lib.FMT_INT8 if kind.startswith("int8") else _lib.FMT_INT4
    splits = int(os.environ.get("KVQ_BENCH_SPLITS", "0"))
    layers = []
    for l in range(L):
        b = cache._bufs[l]
        view = {n: t[:, :, :S + 1] for n, t in b.items()}
        app = dict(k_zp=b.get("kz"), v_zp=b.get("vz"))
        if kind == "int4_asym":
            policy = _lib.SCALE_ASYM_MINMAX
        elif kind == "int8_dyn":
            policy = _lib.SCALE_DYNAMIC_PCT
            app.update(quantile=1.0)
        elif kind == "fp16":
            policy = _lib.SCALE_STATIC
        else:
            policy = _lib.SCALE_STATIC
            app.update(k_static=cache._static_table("k", l, Hkv, G, dev), v_static=cache._static_table("v", l, Hkv, G, dev))
        att = dict(k_zp=view.get("kz"), v_zp=view.get("vz"))
        if kind == "int4_outlier":
            oidx = cache.outlier_idx[l].contiguous()
            app.update(outlier_idx=oidx, k_side=b["kside"], v_side=b["vside"])
            att.update(outlier_idx=oidx, k_side=view["kside"], v_side=view["vside"])
        layers.append((b, view, policy, app, att))
    gsz = D if kind == "fp16" else GS

    # The append of a layer runs on a second stream, concurrently with the split-K scan of the old tokens
    # (tail_tokens = 1); the combine stage waits for both and attends the new token from the cache.
    overlap = with_append and stages == 0 and os.environ.get("KVQ_BENCH_NO_OVERLAP", "0") != "1"
    side = torch.cuda.Stream(device=dev) if overlap else None

    def attend(l, view, att, **kw):
        ops.decode_attn(fmt, q[l], view["k"], view["v"], view.get("ks"), view.get("vs"), ctx, 1.0 / D ** 0.5,
                        head_dim=D, inv_tau=inv_tau[l], splits=splits, out=out[l], max_ctx=S + 1, **att, **kw)

    def step():
        for l, (b, view, policy, app, att) in enumerate(layers):
            if overlap:
                main = torch.cuda.current_stream(dev)
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    ops.quantize_append(fmt, policy, k_new[l], v_new[l], b["k"], b["v"], b.get("ks"), b.get("vs"), S, gsz, **app)
                attend(l, view, att, stages=1, tail_tokens=1)
                main.wait_stream(side)
                attend(l, view, att, stages=2, tail_tokens=1)
                continue
            if with_append:
                ops.quantize_append(fmt, policy, k_new[l], v_new[l], b["k"], b["v"], b.get("ks"), b.get("vs"), S, gsz, **app)
            # scan-only timing: the same scan as the overlapped step (the newest token belongs to the combine stage)
            attend(l, view, att, stages=stages, tail_tokens=1 if (stages == 1 and not with_append) else 0)
    return step, (lambda: ops.last_splits())


MODEL_GEOMETRY = {   # (Hq, Hkv) -> hidden, intermediate size, vocabulary of the Qwen2.5 member with that attention shape
    (12, 2): (1536, 8960, 151936), (28, 4): (3584, 18944, 152064), (40, 8): (5120, 13824, 152064),
}


def time_model_step(wl, cache, dev, steps=5):
    """One decode step of a random-init Qwen2 model with the workload's geometry (model-card sizes, weights drawn
    on the GPU) through the patched attention forward: HF embedding / norms / projections / MLP / lm_head in eager
    PyTorch, RoPE + quantize-append + fused decode attention per layer from this library, over the synthetic cache
    already built.  The model has as many layers as the cache.  Times `steps` steps with CUDA events."""
    import torch
    import transformers
    from llm_kvcache_quantization_b200 import engine as E
    L, B, Hq, Hkv, S = wl["layers"], wl["B"], wl["Hq"], wl["Hkv"], wl["S"]
    hidden, inter, vocab = MODEL_GEOMETRY[(Hq, Hkv)]
    cfg = transformers.Qwen2Config(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=L,
                                   num_attention_heads=Hq, num_key_value_heads=Hkv, head_dim=D,
                                   max_position_embeddings=S + 4096, rope_theta=1e6, tie_word_embeddings=False)
    torch.manual_seed(0)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.float16)
    try:
        with torch.device(dev):
            model = transformers.Qwen2ForCausalLM(cfg)
    finally:
        torch.set_default_dtype(prev)
    model = model.eval()
    n_params = sum(p.numel() for p in model.parameters())
    start = cache.get_seq_len()
    tok = torch.randint(0, vocab, (B, 1), device=dev)
    E.apply_int8_fused_patch(model)
    try:
        wrapper = E.INT8CacheWrapperContainer(cache, L)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        times = []
        with torch.no_grad():
            for i in range(steps + 2):
                pos = torch.full((B, 1), cache.get_seq_len(), dtype=torch.long, device=dev)
                torch.cuda.synchronize()
                e0.record()
                out = model(input_ids=tok, position_ids=pos, past_key_values=wrapper, use_cache=True)
                tok = out.logits[:, -1].argmax(-1, keepdim=True)
                e1.record()
                torch.cuda.synchronize()
                if i >= 2:
                    times.append(e0.elapsed_time(e1))
        assert bool(torch.isfinite(out.logits.float()).all())
    finally:
        E.remove_int8_fused_patch(model)
    ms = statistics.median(times)
    # the same step as ONE CUDA graph (device-side positions, greedy token fed back on the device)
    from llm_kvcache_quantization_b200.runtime import GraphedModelStep
    graphed = None
    st = GraphedModelStep(model, cache, B)
    try:
        with torch.no_grad():
            st.capture(tok)
            for _ in range(2):
                st.step()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(steps):
                st.step()
            e1.record()
            torch.cuda.synchronize()
        gms = e0.elapsed_time(e1) / steps
        graphed = {"ms_per_step": gms, "tokens_per_s": B / (gms * 1e-3),
                   "what": "runtime.GraphedModelStep: the whole model step (embedding .. argmax, token feedback) "
                           "captured once and replayed"}
    finally:
        st.close()
    return {"ms_per_step": ms, "tokens_per_s": B / (ms * 1e-3), "graphed": graphed, "layers": L, "parameters": n_params,
            "context_start": start, "steps": steps,
            "what": "eager HF Qwen2 forward (random-init weights of the model-card sizes) with the library's patched "
                    "attention: fused RoPE + quantize-append, fused decode attention; argmax of the logits read back"}


def time_aux(wl, cache, dev, iters=10):
    """The kernels either side of the decode path, at this workload's shape, one layer per call, CUDA events:
    `get_kv` (kvq_dequantize of a whole layer) and a bulk prefill append of S tokens (quantize, pack, store)."""
    import torch
    B, Hkv, S, kind, n_out = wl["B"], wl["Hkv"], wl["S"], wl["kind"], wl["n_out"]
    L = wl["layers"]
    res = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    read_b = B * Hkv * S * bytes_per_token_head(kind, n_out)
    for _ in range(2):
        for l in range(min(L, 2)):
            cache.get_kv(l)
    torch.cuda.synchronize()
    e0.record()
    for i in range(iters):
        kv = cache.get_kv(i % L)
    e1.record(); torch.cuda.synchronize()
    del kv
    us = e0.elapsed_time(e1) * 1e3 / iters
    res["get_kv"] = {"us_per_layer": us, "GBps": (read_b + 2 * B * Hkv * S * D * 2) / us / 1e3,
                     "bytes": "payload + scales read, 2 x fp16 [B,Hkv,S,D] written"}
    gen = torch.Generator(device=dev).manual_seed(7)
    chunk = max(1, min(S, (1 << 25) // (B * Hkv * D)))
    k = torch.randn(B, Hkv, chunk, D, device=dev, generator=gen).half()
    v = torch.randn(B, Hkv, chunk, D, device=dev, generator=gen).half()
    old = list(cache._layer_seq_lens)

    def refill(l):
        cache._layer_seq_lens[l] = 0
        for s0 in range(0, S - chunk + 1, chunk):
            cache.append(l, k, v)
    refill(0)
    torch.cuda.synchronize()
    e0.record()
    for i in range(iters):
        refill(i % L)
    e1.record(); torch.cuda.synchronize()
    n_tok = (S // chunk) * chunk
    for l in range(L):                       # restore the nominal lengths (contents are synthetic either way)
        cache._layer_seq_lens[l] = old[l]
    us = e0.elapsed_time(e1) * 1e3 / iters
    res["prefill_append"] = {"us_per_layer": us, "tokens": n_tok,
                             "GBps": (2 * B * Hkv * n_tok * D * 2 + B * Hkv * n_tok * bytes_per_token_head(kind, n_out)) / us / 1e3,
                             "bytes": "fp16 K and V read, payload + scales written"}
    return res


def capture(step):
    import torch
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        step()                      # warm (workspace allocation happens outside capture)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    return g


def time_graph(g, iters, dist=None):
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    return e0.elapsed_time(e1)


# --------------------------------------------------------------------------- CPU baseline / reference arm
def cpu_sample(wl, seed=1234, target_s=12.0, max_rows=4):
    """Times the CPU oracle (C restatement, OpenMP, all host threads) on a bounded sample of
    the workload: ONE layer, `rows` batch rows at the full context, quantize-on-append of the
    new token plus decode attention.  Returns (seconds per sample pass, rows, threads)."""
    import numpy as np
    from oracle import c_oracle as CO
    from oracle import kvq_oracle as O

    Hq, Hkv, S, kind, n_out = wl["Hq"], wl["Hkv"], wl["S"], wl["kind"], wl["n_out"]
    rows = min(max_rows, wl["B"])
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((rows, Hkv, S + 1, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((rows, Hkv, S + 1, D), dtype=np.float32).astype(np.float16)
    q = rng.standard_normal((rows, Hq, D), dtype=np.float32).astype(np.float16)
    tau = rng.uniform(0.8, 1.2, Hq).astype(np.float32)
    ctx = np.full(rows, S + 1, np.int32)
    sm = 1.0 / np.sqrt(D)
    extra = {}
    if kind == "int4_asym":
        pk, sk, zk = CO.quant_int4_asym(k, GS)
        pv, sv, zv = CO.quant_int4_asym(v, GS)
        fmt, extra = 2, dict(kz=zk, vz=zv)
        append = lambda: (CO.quant_int4_asym(k[:, :, -1:], GS), CO.quant_int4_asym(v[:, :, -1:], GS))
    elif kind.startswith("int8"):
        tab = np.full((Hkv, G), 4.5 / 127, np.float16)
        pk, sk = CO.quant_int8_static(k, tab, GS)
        pv, sv = CO.quant_int8_static(v, tab, GS)
        fmt = 1
        append = lambda: (CO.quant_int8_static(k[:, :, -1:], tab, GS), CO.quant_int8_static(v[:, :, -1:], tab, GS))
    else:
        idx = np.stack([np.sort(rng.permutation(D)[:n_out]) for _ in range(Hkv)]).astype(np.int16)
        tab = np.full((Hkv, G), 4.5 / 7, np.float32)
        bk, sidek = O.split_outliers(k, idx)
        bv, sidev = O.split_outliers(v, idx)
        pk, sk = CO.quant_int4_static(bk, tab, GS)
        pv, sv = CO.quant_int4_static(bv, tab, GS)
        fmt, extra = 2, dict(kside=sidek, vside=sidev, outlier_idx=idx)
        append = lambda: (CO.quant_int4_static(bk[:, :, -1:], tab, GS), CO.quant_int4_static(bv[:, :, -1:], tab, GS))

    def one_pass():
        append()
        return CO.decode_attn(fmt, q, pk, pv, sk, sv, ctx, sm, inv_tau=tau, **extra)

    one_pass()
    t0 = time.perf_counter()
    n = 0
    while True:
        one_pass()
        n += 1
        el = time.perf_counter() - t0
        if el >= target_s or n >= 50:
            break
    return el / n, rows, CO.num_threads()


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # the multi-process launcher pins every rank to one OpenMP thread; this arm runs on rank 0 alone and
        # uses the host's cores (the setting is read when the OpenMP runtime of the C oracle starts)
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    per_pass, rows, threads = cpu_sample(wl, target_s=2.0)          # warm-up + calibration
    times = []
    for _ in range(max(args.warmup, 0)):
        cpu_sample(wl, target_s=0.0)
    for _ in range(args.steps):
        t, rows, threads = cpu_sample(wl, target_s=0.0)
        times.append(t)
    per_pass = statistics.mean(times) if times else per_pass
    # extrapolate the sample (1 layer x rows sequences) linearly to the full step
    step_s = per_pass * wl["layers"] * (wl["B"] / rows)
    value = wl["B"] * args.gpus / step_s if False else wl["B"] / step_s
    sample = (f"1 of {wl['layers']} layers x {rows} of {wl['B']} sequences at full context, "
              f"quantize-append + decode attention; extrapolated linearly to the full step")
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": workload_config(wl, args.workload),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(wl, name):
    return {"workload": wl["desc"], "name": name, "layers": wl["layers"], "batch_per_gpu": wl["B"],
            "context": wl["S"], "group_size": GS, "l2": "inputs larger than L2 (KV stack cycles through all layers)"
            if wl["layers"] * wl["B"] * wl["Hkv"] * wl["S"] * bytes_per_token_head(wl["kind"], wl["n_out"]) > 126e6
            else "L2 flushed between timed iterations by a 256 MB write"}



# --------------------------------------------------------------------------- sequence sharding (one long sequence)
def run_sequence_sharded(args, wl, dev, dist, rank, world):
    """KV-sequence sharding of a single long sequence over `world` GPUs: rank r owns a contiguous
    chunk of tokens, the owner of position S appends the new token, every rank runs the fused
    decode over its chunk into a packed normalised partial, ONE NCCL all-gather per layer moves the
    partials, and every rank merges them.  The whole step (kernels and collectives) is one CUDA graph."""
    import torch
    from llm_kvcache_quantization_b200 import ops, _lib, parallel as P

    L, B, Hq, Hkv, S, kind, n_out = (wl[k] for k in ("layers", "B", "Hq", "Hkv", "S", "kind", "n_out"))
    sh = P.SequenceSharding(world=world, max_seq_len=S + 1)
    lo, hi = sh.token_range(rank)
    n_old = sh.local_len(rank, S)                    # cached tokens of this rank before the step
    owner = sh.owner_of(S) == rank                   # this rank stores the new token
    n_att = n_old + (1 if owner else 0)
    local = dict(wl, S=n_old)
    # same seed on every rank for q / k_new / v_new would need a shared generator; the inputs of a step are
    # replicated in a real deployment, here rank 0's are broadcast
    cache, q, k_new, v_new, inv_tau = build_workload(local, dev, seed=1234 + rank, extra_slots=8)
    for t in (q, k_new, v_new, inv_tau):
        dist.broadcast(t, src=0)
    fmt = _lib.FMT_INT8 if kind.startswith("int8") else _lib.FMT_INT4
    out = torch.empty(L, B, Hq, D, dtype=torch.float16, device=dev)
    send = torch.empty(B, Hq, D + 2, dtype=torch.float32, device=dev)
    recv = torch.empty(world, B, Hq, D + 2, dtype=torch.float32, device=dev)
    P.check_partial_shapes(send.shape)
    fused = args.collective == "fused"
    xchg = P.PeerExchange(B, Hq, D, slots=L) if fused else None
    layers = []
    for l in range(L):
        b = cache._bufs[l]
        tens = dict(b)
        tens["outlier_idx"] = None if cache.outlier_idx is None else cache.outlier_idx[l].contiguous()
        app = dict(k_zp=b.get("kz"), v_zp=b.get("vz"))
        if kind == "int4_asym":
            policy = _lib.SCALE_ASYM_MINMAX
        elif kind == "int8_dyn":
            policy = _lib.SCALE_DYNAMIC_PCT
            app.update(quantile=1.0)
        else:
            policy = _lib.SCALE_STATIC
            app.update(k_static=cache._static_table("k", l, Hkv, G, dev), v_static=cache._static_table("v", l, Hkv, G, dev))
        if tens["outlier_idx"] is not None:
            app.update(outlier_idx=tens["outlier_idx"], k_side=b["kside"], v_side=b["vside"])
        layers.append((b, tens, policy, app))

    def step(scan_only=False):
        if fused and not scan_only:
            xchg.advance()
        for l, (b, tens, policy, app) in enumerate(layers):
            if scan_only:
                extra = {}
                if tens.get("kz") is not None:
                    extra.update(k_zp=tens["kz"][:, :, :n_att], v_zp=tens["vz"][:, :, :n_att])
                if tens["outlier_idx"] is not None:
                    extra.update(outlier_idx=tens["outlier_idx"], k_side=tens["kside"][:, :, :n_att],
                                 v_side=tens["vside"][:, :, :n_att])
                ops.decode_attn(fmt, q[l], tens["k"][:, :, :n_att], tens["v"][:, :, :n_att], tens["ks"][:, :, :n_att],
                                tens["vs"][:, :, :n_att], None, 1.0 / D ** 0.5, head_dim=D, inv_tau=inv_tau[l],
                                out=out[l], stages=1, **extra)
                continue
            do_append = None
            if owner:
                do_append = (lambda l=l, b=b, policy=policy, app=app: ops.quantize_append(
                    fmt, policy, k_new[l], v_new[l], b["k"], b["v"], b["ks"], b["vs"], n_old, GS, **app))
            if fused:
                # on the owner the append runs beside the scan; the exchange kernel attends the new token
                xchg.decode(fmt, q[l], tens, n_att, 1.0 / D ** 0.5, slot=l, out=out[l], inv_tau=inv_tau[l],
                            append=do_append)
            else:
                if owner:
                    do_append()
                P.sharded_decode(fmt, q[l], tens, n_att, 1.0 / D ** 0.5, send=send, recv=recv, inv_tau=inv_tau[l],
                                 out=out[l])

    g_step = capture(step)
    splits = ops.last_splits()
    g_scan = capture(lambda: step(scan_only=True))
    time_graph(g_step, args.warmup, dist)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    ms = time_graph(g_step, args.steps, dist)
    time_graph(g_scan, 3, dist)
    ms_scan = time_graph(g_scan, args.steps, dist)
    t_end = time.time() + 0.4                   # keep the scans running while the clock sampler is still on
    while time.time() < t_end:
        for _ in range(5):
            g_scan.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["window"] = "timed region + 0.4 s of split-K scans"

    # end to end with host buffers: upload q / k / v of the token, replay, download the merged output
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k_new, v_new))
    hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def host_step():
        q.copy_(hq, non_blocking=True); k_new.copy_(hk, non_blocking=True); v_new.copy_(hv, non_blocking=True)
        g_step.replay()
        hout.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    for _ in range(3):
        host_step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier(); torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        host_step()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([ms, ms_scan, e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_scan, ems = (float(x) for x in t)
    ms_per_step = ms / args.steps

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    alg_bytes = B * Hkv * sh.chunk * bytes_per_token_head(kind, n_out)       # the largest shard
    scan_us = ms_scan / (args.steps * L) * 1e3
    achieved = alg_bytes / (scan_us * 1e-6) / 1e9
    if rank == 0:
        line = {
            "metric": "decode_tokens_per_s", "value": B / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": dict(workload_config(wl, args.workload), parallelism=f"sequence-sharded x{world}",
                           chunk_tokens=sh.chunk, splits=splits,
                           collective=("fused kernel: combine + peer stores of [B,Hq,D+2] fp32 over NVLink + merge, "
                                       "one launch per layer" if fused else
                                       "one NCCL all-gather of [B,Hq,D+2] fp32 per layer"),
                           step=(f"CUDA graph of {L}x(append on the owner, split-K scan, fused combine/exchange/merge)"
                                 if fused else
                                 f"CUDA graph (kernels + NCCL all-gather) of {L}x(append on the owner, split-K scan, "
                                 "combine, all-gather, merge)"),
                           exchange_status=(int(xchg.status.item()) if fused else None)),
            "us_per_layer": ms_per_step * 1e3 / L,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": alg_bytes * NCU_TRAFFIC_RATIO.get(kind, 1.0),
                         "traffic_source": "ncu capture of the same kernel (profiles/), scaled by token-heads",
                         "peak_source": peak_src, "kernel": "decode split-K scan (largest shard, per GPU)",
                         "us_per_launch": scan_us, "algorithmic_bytes_per_launch": alg_bytes,
                         "frac_of_8TBps": achieved / 8000.0},
            "cpu_baseline": None,
            "e2e": {"value": B / (ems / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": (q.numel() + k_new.numel() + v_new.numel()) * 2,
                    "d2h_bytes_per_step": out.numel() * 2, "ms_per_step": ems / args.steps,
                    "api": "pinned H2D of q/k/v on every rank, one CUDA graph (sharded_decode per layer), pinned D2H"},
            "gpu_launches": args.steps * L * (3 if fused else 4), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    # Tearing the process group down while captured graphs still hold its collectives did not return in a
    # two-GPU run: drain, agree that every rank is done, drop the graphs, and leave without the teardown.
    torch.cuda.synchronize()
    dist.barrier()
    del g_step, g_scan
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


# --------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling captures only)")
    ap.add_argument("--aux", action="store_true",
                    help="also time the neighbouring kernels at this workload's shape: bulk prefill quantize-append "
                         "(T = context) and the dequantising get_kv, one layer each")
    ap.add_argument("--model-step", action="store_true",
                    help="also time one decode step of a random-init Qwen2 model of the workload's geometry through "
                         "the patched attention forward over the same synthetic cache (weights, MLP, eager Python "
                         "included); reported under model_step")
    ap.add_argument("--collective", default="fused", choices=("fused", "nccl"),
                    help="sequence-sharded mode: the library's fused combine/peer-store/merge kernel, or "
                         "combine + NCCL all-gather + merge")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.layers > 0:
        wl["layers"] = args.layers
        wl["desc"] += f" [layers overridden to {args.layers}]"
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args, wl)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # the fused exchange uses plain peer stores; symmetric-memory buffers are not bound to an NVLink multicast object
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch
    import llm_kvcache_quantization_b200 as kvq
    from llm_kvcache_quantization_b200 import ops
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        # a collective that a peer never joins ends with an error after two minutes instead of waiting forever
        dist_mod.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
        dist = dist_mod

    if world > 1 and wl["B"] == 1:
        run_sequence_sharded(args, wl, dev, dist, rank, world)
        return

    L, B, Hq, Hkv, S = wl["layers"], wl["B"], wl["Hq"], wl["Hkv"], wl["S"]
    e2e_slots = args.steps + args.warmup + 8 + (64 if args.model_step else 0)
    cache, q, k_new, v_new, inv_tau = build_workload(wl, dev, seed=1234 + rank, extra_slots=e2e_slots)
    out = torch.empty(L, B, Hq, D, dtype=torch.float16, device=dev)
    small = L * B * Hkv * S * bytes_per_token_head(wl["kind"], wl["n_out"]) <= 126e6
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None

    step, splits_fn = make_step(wl, cache, q, k_new, v_new, inv_tau, out)
    g_step = capture(step)
    splits = splits_fn()
    split_only, _ = make_step(wl, cache, q, k_new, v_new, inv_tau, out, stages=1, with_append=False)
    g_split = capture(split_only)

    def timed(graph, iters):
        if flush is None:
            return time_graph(graph, iters, dist)
        tot = 0.0
        for _ in range(iters):
            flush.fill_(1)
            tot += time_graph(graph, 1, dist)
        return tot

    timed(g_step, args.warmup)
    sampler = ClockSampler(local)
    sampler.start()
    ms = timed(g_step, args.steps)
    # dominant kernel alone (split-K scan), same clocks window
    timed(g_split, 3)
    ms_split = timed(g_split, args.steps)
    # the timed region lasts a few milliseconds - shorter than the sampling period of nvidia-smi - so the same
    # step keeps running for another 0.4 s (untimed) while the clock sampler is still on
    t_end = time.time() + 0.4
    while time.time() < t_end:
        for _ in range(20):
            g_step.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["window"] = "timed region + 0.4 s of the same step"
    if dist is not None:
        t = torch.tensor([ms, ms_split], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_split = float(t[0]), float(t[1])
    ms_per_step = ms / args.steps
    value = world * B / (ms_per_step * 1e-3)

    # roofline of the dominant kernel
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    alg_bytes = B * Hkv * (S + 1) * bytes_per_token_head(wl["kind"], wl["n_out"])
    split_us = ms_split / (args.steps * L) * 1e3
    achieved = alg_bytes / (split_us * 1e-6) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": alg_bytes * NCU_TRAFFIC_RATIO.get(wl["kind"], 1.0),
                "traffic_source": "ncu capture of the same kernel on this shape (profiles/), scaled by token-heads",
                "peak_source": peak_src, "kernel": "decode split-K scan",
                "us_per_launch": split_us, "algorithmic_bytes_per_launch": alg_bytes,
                "frac_of_8TBps": achieved / 8000.0}

    # end to end through the public API with HOST buffers: every step uploads this token's q / k / v
    # for all layers from pinned memory, replays the captured whole-stack step (append + attention per
    # layer, device-side position counter, the cache grows by one token) and downloads the outputs
    e2e = None
    if not args.no_e2e and wl["kind"] != "kivi4":      # the host-buffer stepper serves the group-wise caches
        from llm_kvcache_quantization_b200.runtime import GraphedKVStackStep
        stepper = GraphedKVStackStep(cache, Hq, 1.0 / D ** 0.5, inv_tau=inv_tau)
        stepper.capture()
        stepper.host_q.copy_(q.cpu()); stepper.host_k.copy_(k_new.cpu()); stepper.host_v.copy_(v_new.cpu())
        for _ in range(3):
            stepper.step(stepper.host_q, stepper.host_k, stepper.host_v)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            res = stepper.step(stepper.host_q, stepper.host_k, stepper.host_v)
        e1.record()
        torch.cuda.synchronize()
        ems = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ems], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t[0])
        assert bool(torch.isfinite(res.float()).all())
        e2e = {"value": world * B / (ems / args.steps * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": stepper.h2d_bytes_per_step, "d2h_bytes_per_step": stepper.d2h_bytes_per_step,
               "ms_per_step": ems / args.steps,
               "api": "GraphedKVStackStep.step(host_q, host_k, host_v) -> host_out: one CUDA graph launch holding the "
                      "pinned H2D copies of q/k/v (first layers, then the rest beside their kernels), append + attention "
                      "for every layer, and the pinned D2H of the outputs (all but the last layers beside the last "
                      "layers' kernels, then the tail); stream sync"}

    aux = None
    if args.aux and wl["kind"] not in ("fp16", "kivi4"):
        aux = time_aux(wl, cache, dev)

    model_step = None
    if args.model_step and world == 1:
        model_step = time_model_step(wl, cache, dev, steps=max(3, min(args.steps, 10)))

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and wl["kind"] not in ("fp16", "kivi4"):
        per_pass, rows, threads = cpu_sample(wl, target_s=12.0)
        step_s = per_pass * L * (B / rows)
        cpu = {"value": B / step_s, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"1 of {L} layers x {rows} of {B} sequences at full context (C oracle, OpenMP), "
                         f"{per_pass * 1e3:.1f} ms per pass, extrapolated linearly"}

    if rank == 0:
        line = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": dict(workload_config(wl, args.workload), parallelism=f"batch-sharded x{world}", splits=splits,
                           step=f"CUDA graph of {L}x(quantize-append || split-K scan of the old tokens, then combine "
                                "incl. the new token)"),
            "us_per_layer": ms_per_step * 1e3 / L,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": args.steps * L * 3, "clocks": clocks,
        }
        if aux is not None:
            line["aux"] = aux
        if model_step is not None:
            line["model_step"] = model_step
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
