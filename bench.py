#!/usr/bin/env python3
"""Benchmark of the quantized-KV decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c4]

One "step" = one decode step over the whole KV stack of a workload: for every layer, quantize-on-append
of the new token (one launch for K and V) and the fused decode attention (split-K scan + combine) over the
cached context, captured as one CUDA graph - with the append either on a second stream beside the scan or in
stream order, whichever a short trial of both finds faster for the shape (`step`, `step_form_trial_ms`).

Headline workload = configuration 4 of the benchmark definition, the largest one that fits a single GPU
(Qwen2.5-7B geometry, 28 layers, batch 64, context 32768, INT8 group-32: 64 GB of cache).  The other
configurations (c1, c2, c3, c5 and the KIVI-format variant of c2) are measured in the same run and
reported under `extra.workloads`, each with its own step time, scan roofline, end-to-end number and
clocks; packed-INT4 workloads report both dequantisation arithmetics.

With N > 1 (one process per GPU) the FIXED batch of 64 sequences of configuration 4 is sharded by sequence
(`parallel.batch_shard`: 64 / N rows per GPU, no collective on the data path; strong scaling), and the
single-sequence configuration 5 is sharded by KV-sequence chunks with its partials exchanged once per layer
(`extra.sequence_sharded`: the library's fused combine / peer-store / merge kernel, and the NCCL all-gather form).

Every timed region is a repetition of blocks of exactly K steps (barrier + device synchronisation on both
sides of a block, CUDA events, maximum over ranks) until at least `--min-seconds` have been timed; the
median over blocks is reported, the minimum beside it.

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
NCU_TRAFFIC_RATIO = {"kivi4": 1.0, "fp16": 1.0, "int4_asym": 1.002, "int8_dyn": 1.004, "int8_static": 1.004, "int4_outlier": 1.022}


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
    """The kernels either side of the decode path, at this workload's shape, one layer per call: `get_kv`
    (kvq_dequantize of a whole layer) and a bulk prefill append of S tokens (quantize, pack, store).  Each call is
    captured in a CUDA graph (the Python around one call costs more than the kernel) and replayed over the layers'
    worth of distinct buffers it touches; CUDA events."""
    import torch
    B, Hkv, S, kind, n_out = wl["B"], wl["Hkv"], wl["S"], wl["kind"], wl["n_out"]
    res = {}
    read_b = B * Hkv * S * bytes_per_token_head(kind, n_out)
    holder = {}

    def read_back():
        holder["kv"] = cache.get_kv(0)
    g = capture(read_back)
    time_graph(g, 3)
    us = min(time_graph(g, iters) for _ in range(3)) * 1e3 / iters
    holder.clear()
    del g
    res["get_kv"] = {"us_per_layer": us, "GBps": (read_b + 2 * B * Hkv * S * D * 2) / us / 1e3,
                     "frac_of_measured_hbm": (read_b + 2 * B * Hkv * S * D * 2) / us / 1e3 / hbm_peak()[0],
                     "bytes": "payload + scales read, 2 x fp16 [B,Hkv,S,D] written"}
    gen = torch.Generator(device=dev).manual_seed(7)
    chunk = max(1, min(S, (1 << 25) // (B * Hkv * D)))
    k = torch.randn(B, Hkv, chunk, D, device=dev, generator=gen).half()
    v = torch.randn(B, Hkv, chunk, D, device=dev, generator=gen).half()
    old = list(cache._layer_seq_lens)

    def refill():
        cache._layer_seq_lens[0] = 0
        for s0 in range(0, S - chunk + 1, chunk):
            cache.append(0, k, v)
    g = capture(refill)
    time_graph(g, 3)
    us = min(time_graph(g, iters) for _ in range(3)) * 1e3 / iters
    del g
    n_tok = (S // chunk) * chunk
    cache._layer_seq_lens[0] = old[0]        # the nominal length again (contents are synthetic either way)
    moved = 2 * B * Hkv * n_tok * D * 2 + B * Hkv * n_tok * bytes_per_token_head(kind, n_out)
    res["prefill_append"] = {"us_per_layer": us, "tokens": n_tok, "GBps": moved / us / 1e3,
                             "frac_of_measured_hbm": moved / us / 1e3 / hbm_peak()[0],
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


# --------------------------------------------------------------------------- timing
def timed_blocks(run_block, steps, min_seconds, dist=None, dev=None, max_blocks=2000):
    """Repeats `run_block(steps)` (which returns the elapsed milliseconds of exactly `steps` steps, measured between
    its own synchronisation points) until at least `min_seconds` have been timed.  Returns ms per step of every block.
    With several ranks every block's time is the maximum over ranks, so that all ranks time the same number of blocks."""
    per_step, total = [], 0.0
    while True:
        ms = run_block(steps)
        if dist is not None:
            ms, = allreduce_max([ms], dev, dist)
        per_step.append(ms / steps)
        total += ms
        if total >= min_seconds * 1e3 or len(per_step) >= max_blocks:
            return per_step


def block_stats(per_step):
    return {"median": statistics.median(per_step), "min": min(per_step), "blocks": len(per_step)}


def allreduce_max(vals, dev, dist):
    import torch
    if dist is None:
        return [float(v) for v in vals]
    t = torch.tensor(list(vals), dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


# --------------------------------------------------------------------------- CPU baseline / reference arm
def cpu_inputs(wl, rows, layers, seed=1234):
    """Host-side inputs of the CPU oracle for `layers` layers x `rows` batch rows at the full context: random
    payload bytes, fp16 scales (zero-points, side values) and queries of the workload's shapes and dtypes.  The
    oracle's run time does not depend on the values, so nothing is quantized here; generated ONCE, outside any
    timed pass."""
    import numpy as np
    Hq, Hkv, S, kind, n_out = wl["Hq"], wl["Hkv"], wl["S"], wl["kind"], wl["n_out"]
    rng = np.random.default_rng(seed)
    n = S + 1
    per_layer = []
    for _ in range(layers):
        d = {}
        if kind == "fp16":
            d["fmt"] = 0
            d["k"] = rng.standard_normal((rows, Hkv, n, D), dtype=np.float32).astype(np.float16)
            d["v"] = rng.standard_normal((rows, Hkv, n, D), dtype=np.float32).astype(np.float16)
            d["ks"] = d["vs"] = None
        else:
            int8 = kind.startswith("int8")
            d["fmt"] = 1 if int8 else 2
            dp = D if int8 else D // 2
            d["k"] = rng.integers(-127, 128, (rows, Hkv, n, dp), dtype=np.int8)
            d["v"] = rng.integers(-127, 128, (rows, Hkv, n, dp), dtype=np.int8)
            d["ks"] = rng.uniform(0.01, 0.1, (rows, Hkv, n, G)).astype(np.float16)
            d["vs"] = rng.uniform(0.01, 0.1, (rows, Hkv, n, G)).astype(np.float16)
            if kind in ("int4_asym", "kivi4"):
                d["kz"] = rng.uniform(-0.5, 0.5, (rows, Hkv, n, G)).astype(np.float16)
                d["vz"] = rng.uniform(-0.5, 0.5, (rows, Hkv, n, G)).astype(np.float16)
            if kind == "int4_outlier":
                d["outlier_idx"] = np.stack([np.sort(rng.permutation(D)[:n_out]) for _ in range(Hkv)]).astype(np.int16)
                d["kside"] = rng.standard_normal((rows, Hkv, n, n_out), dtype=np.float32).astype(np.float16)
                d["vside"] = rng.standard_normal((rows, Hkv, n, n_out), dtype=np.float32).astype(np.float16)
        d["q"] = rng.standard_normal((rows, Hq, D), dtype=np.float32).astype(np.float16)
        d["k_new"] = rng.standard_normal((rows, Hkv, 1, D), dtype=np.float32).astype(np.float16)
        d["v_new"] = rng.standard_normal((rows, Hkv, 1, D), dtype=np.float32).astype(np.float16)
        per_layer.append(d)
    tau = rng.uniform(0.8, 1.2, Hq).astype(np.float32)
    return per_layer, tau


def cpu_pass(wl, per_layer, tau):
    """One pass of the CPU oracle (C restatement, OpenMP) over the given layers: quantize-on-append of the new token
    and decode attention over the full context.  Returns the seconds it took."""
    import numpy as np
    from oracle import c_oracle as CO
    kind = wl["kind"]
    rows = per_layer[0]["q"].shape[0]
    ctx = np.full(rows, wl["S"] + 1, np.int32)
    sm = 1.0 / np.sqrt(D)
    tab8 = np.full((wl["Hkv"], G), 4.5 / 127, np.float16)
    tab4 = np.full((wl["Hkv"], G), 4.5 / 7, np.float32)
    t0 = time.perf_counter()
    for d in per_layer:
        if kind.startswith("int8"):
            CO.quant_int8_static(d["k_new"], tab8, GS); CO.quant_int8_static(d["v_new"], tab8, GS)
        elif kind in ("int4_asym", "kivi4"):
            CO.quant_int4_asym(d["k_new"], GS); CO.quant_int4_asym(d["v_new"], GS)
        elif kind == "int4_outlier":
            CO.quant_int4_static(d["k_new"], tab4, GS); CO.quant_int4_static(d["v_new"], tab4, GS)
        extra = {k: d[k] for k in ("kz", "vz", "kside", "vside", "outlier_idx") if k in d}
        CO.decode_attn(d["fmt"], d["q"], d["k"], d["v"], d["ks"], d["vs"], ctx, sm, inv_tau=tau, **extra)
    return time.perf_counter() - t0


def cpu_plan(wl):
    """How much of the workload one CPU pass covers: whole layers with all batch rows; as many layers as keep the
    host arrays under ~3 GB (every layer of a small stack, one layer of the 64 GB one).  Returns (layers, factor):
    step time = pass time x factor."""
    per_layer_bytes = wl["B"] * wl["Hkv"] * (wl["S"] + 1) * bytes_per_token_head(wl["kind"], wl["n_out"])
    layers = max(1, min(wl["layers"], int(3e9 // max(per_layer_bytes, 1))))
    return layers, wl["layers"] / layers


def cpu_baseline(wl, passes=3, budget_s=25.0):
    """`cpu_baseline` object of the JSON line: the CPU oracle on whole layers of this workload (all batch rows, full
    context), inputs built once, `passes` timed passes (fewer if the budget runs out), scaled by layers only."""
    from oracle import c_oracle as CO
    layers, factor = cpu_plan(wl)
    per_layer, tau = cpu_inputs(wl, wl["B"], layers)
    cpu_pass(wl, per_layer[:1], tau)                                   # load the library, touch the pages
    times, t_start = [], time.perf_counter()
    for _ in range(passes):
        times.append(cpu_pass(wl, per_layer, tau))
        if time.perf_counter() - t_start > budget_s:
            break
    step_s = statistics.median(times) * factor
    return {"value": wl["B"] / step_s, "unit": "tokens/s", "cores": CO.num_threads(), "kind": "port",
            "ms_per_step": step_s * 1e3,
            "sample": (f"C restatement of the reference's torch decode path (OpenMP): {layers} of {wl['layers']} layers, "
                       f"all {wl['B']} sequences at the full context, quantize-append + decode attention, "
                       f"{len(times)} passes of {statistics.median(times) * 1e3:.0f} ms, inputs built once outside them; "
                       + ("the whole step, no extrapolation" if layers == wl["layers"]
                          else f"step = pass x {factor:g} (layers only)"))}


def workload_config(wl, name, n_gpus=1):
    """The `config` object; identical for both arms of a run (repo and reference)."""
    big = wl["layers"] * wl["B"] * wl["Hkv"] * wl["S"] * bytes_per_token_head(wl["kind"], wl["n_out"]) > 126e6
    par = ("single GPU" if n_gpus == 1 else
           f"one long sequence sharded by KV chunks x{n_gpus}" if wl["B"] == 1 else
           f"fixed batch of {wl['B']} sharded by sequence x{n_gpus}")
    return {"workload": wl["desc"], "name": name, "layers": wl["layers"], "batch": wl["B"], "context": wl["S"],
            "group_size": GS, "parallelism": par,
            "l2": "inputs larger than L2 (the KV stack cycles through all layers)" if big
            else "L2 flushed between timed iterations by a 256 MB write"}


def run_reference_arm(args, name, wl):
    """`--impl reference`: the reference's CPU path (C restatement of its torch dequantize-then-attention decode, all
    host threads) on the repo arm's workload.  Rank 0 alone runs it; every step is one pass over whole layers."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # the multi-process launcher pins every rank to one OpenMP thread; this arm runs on rank 0 alone and
        # uses the host's cores (the setting is read when the OpenMP runtime of the C oracle starts)
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from oracle import c_oracle as CO
    layers, factor = cpu_plan(wl)
    per_layer, tau = cpu_inputs(wl, wl["B"], layers)
    cpu_pass(wl, per_layer[:1], tau)
    for _ in range(max(args.warmup, 0)):
        cpu_pass(wl, per_layer, tau)
    times = [cpu_pass(wl, per_layer, tau) for _ in range(max(args.steps, 1))]
    step_s = statistics.mean(times) * factor
    value = wl["B"] / step_s
    sample = (f"{layers} of {wl['layers']} layers, all {wl['B']} sequences at the full context per step, quantize-append "
              f"+ decode attention, inputs built once outside the timed passes; "
              + ("the whole decode step, no extrapolation" if layers == wl["layers"]
                 else f"ms_per_step = pass x {factor:g} (layers only; the 64 GB stack does not fit the host arrays)"))
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": workload_config(wl, name, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": CO.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "pass_ms": [t * 1e3 for t in times],
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- one workload on this rank's GPU
def hbm_peak():
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        return float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback"


PROFILE_OF = {"int8_dyn": "profiles/decode_split_mma_int8_c4.md", "int8_static": "profiles/decode_split_mma_int8_c4.md",
              "int4_asym": "profiles/decode_split_int4_c2.md", "int4_outlier": "profiles/decode_split_int4_c3_c5.md",
              "fp16": "profiles/decode_split_mma_fp16_c2shape.md", "kivi4": "profiles/decode_split_int4_c2.md"}


def parity_check(wl, cache, q, inv_tau, out0, rows):
    """Layer 0 of the step that was just timed against the CPU oracle on the batch rows `rows` (context S + 1)."""
    import numpy as np
    import torch
    from oracle import c_oracle as CO
    S, kind = wl["S"], wl["kind"]
    b = cache._bufs[0]
    idx = torch.as_tensor(rows, device=q.device)

    def host(name):
        t = b.get(name)
        return None if t is None else t[idx, :, :S + 1].contiguous().cpu().numpy()
    fmt = 0 if kind == "fp16" else 1 if kind.startswith("int8") else 2
    extra = {}
    if kind == "int4_asym":
        extra = dict(kz=host("kz"), vz=host("vz"))
    elif kind == "int4_outlier":
        extra = dict(kside=host("kside"), vside=host("vside"), outlier_idx=cache.outlier_idx[0].cpu().numpy())
    ref = CO.decode_attn(fmt, q[0][idx].cpu().numpy(), host("k"), host("v"), host("ks"), host("vs"),
                         np.full(len(rows), S + 1, np.int32), 1.0 / np.sqrt(D), inv_tau=inv_tau[0].cpu().numpy(),
                         **extra).astype(np.float32)
    got = out0[idx].float().cpu().numpy()
    err = np.abs(got - ref)
    ok = bool(np.isfinite(got).all() and (err <= 2e-3 + 1e-2 * np.abs(ref)).all())
    return {"max_abs": float(err.max()), "ok": ok, "rows": [int(r) for r in rows], "layer": 0,
            "tolerance": "|a-b| <= 2e-3 + 1e-2 |b| against the CPU restatement of the reference's torch path"}


def measure_workload(name, wl, args, dev, dist, rank, world, *, e2e=True, cpu=False, parity=True):
    """Builds this rank's share of the workload and measures it: the decode step (graph), the split-K scan alone
    (graph; both dequantisation arithmetics for packed INT4), the host-buffer end-to-end step, clocks, parity."""
    import torch
    from llm_kvcache_quantization_b200 import ops
    from llm_kvcache_quantization_b200.parallel import batch_shard
    wl = dict(wl)
    B_total = wl["B"]
    if world > 1:
        lo, hi = batch_shard(B_total, rank, world)
        wl["B"] = hi - lo
    L, B, Hq, Hkv, S, kind, n_out = (wl[k] for k in ("layers", "B", "Hq", "Hkv", "S", "kind", "n_out"))
    res = {"name": name, "config": workload_config(dict(wl, B=B_total), name, world), "batch_per_gpu": B}
    free, _ = torch.cuda.mem_get_info()
    need = L * B * Hkv * (S + 64) * bytes_per_token_head(kind, n_out) * (1.1 if kind != "kivi4" else 1.6) + (3 << 30)
    short, = allreduce_max([1.0 if free < need else 0.0], dev, dist)      # every rank takes the same branch
    if short:
        res["skipped"] = f"needs {need / 2**30:.0f} GiB of device memory, {free / 2**30:.0f} GiB free"
        return res
    cache, q, k_new, v_new, inv_tau = build_workload(wl, dev, seed=1234 + rank, extra_slots=64)
    out = torch.empty(L, B, Hq, D, dtype=torch.float16, device=dev)
    small = L * B * Hkv * S * bytes_per_token_head(kind, n_out) <= 126e6
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None

    # Two forms of the same step: the append on a second stream beside the scan of the old tokens (the combine then
    # attends the new token), or append, scan, combine in stream order.  Which is faster depends on the shape (the
    # fork and join of the second stream cost about as much as a small append hides): both are captured, timed for a
    # few steps, and the faster one is measured; every rank takes the same one.
    forms = {}
    for form, env in (("append beside the scan", None), ("append in stream order", "1")):
        old = os.environ.get("KVQ_BENCH_NO_OVERLAP")
        forced = old is not None
        if env is not None and not forced:
            os.environ["KVQ_BENCH_NO_OVERLAP"] = env
        try:
            fn, splits_fn = make_step(wl, cache, q, k_new, v_new, inv_tau, out)
            forms[form] = (capture(fn), splits_fn())
        finally:
            if env is not None and not forced:
                os.environ.pop("KVQ_BENCH_NO_OVERLAP", None)
        if forced:
            forms = {("append in stream order" if old == "1" else "append beside the scan"): forms[form]}
            break
    trial = {}
    for form, (gph, _) in forms.items():
        time_graph(gph, 3, dist)
        trial[form], = allreduce_max([min(time_graph(gph, max(args.steps, 5), dist) for _ in range(2))], dev, dist)
    step_form = min(trial, key=trial.get)
    g_step, splits = forms[step_form]
    forms.clear()
    int4 = kind in ("int4_asym", "int4_outlier")
    scans = {}
    for arm, env in (("default", None), ("bit_faithful", "0")) if int4 else (("default", None),):
        old = os.environ.get("KVQ_INT4_FAST")
        if env is not None:
            os.environ["KVQ_INT4_FAST"] = env
        try:
            fn, _ = make_step(wl, cache, q, k_new, v_new, inv_tau, out, stages=1, with_append=False)
            scans[arm] = capture(fn)
        finally:
            if env is not None:
                if old is None:
                    os.environ.pop("KVQ_INT4_FAST", None)
                else:
                    os.environ["KVQ_INT4_FAST"] = old

    def run_block(graph):
        def block(steps):
            if flush is None:
                return time_graph(graph, steps, dist)
            tot = 0.0
            for _ in range(steps):
                flush.fill_(1)
                tot += time_graph(graph, 1, dist)
            return tot
        return block

    for gph in [g_step] + list(scans.values()):
        run_block(gph)(args.warmup)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    step_ms = timed_blocks(run_block(g_step), args.steps, args.min_seconds, dist, dev)
    scan_ms = {arm: timed_blocks(run_block(gph), args.steps, args.min_seconds, dist, dev) for arm, gph in scans.items()}
    clocks = sampler.stop()
    clocks["window"] = "the timed regions of the decode step and of the split-K scans"
    n_steps_timed = len(step_ms) * args.steps
    med, mn = allreduce_max([statistics.median(step_ms), min(step_ms)], dev, dist)
    res.update(ms_per_step=med, ms_per_step_min=mn, blocks=len(step_ms), us_per_layer=med * 1e3 / L,
               value=B_total / (med * 1e-3), unit="tokens/s", splits=splits, clocks=clocks,
               gpu_launches=n_steps_timed * L * 3,
               step=(f"CUDA graph of {L}x(quantize-append || split-K scan of the old tokens, then combine incl. the new token)"
                     if step_form == "append beside the scan" else
                     f"CUDA graph of {L}x(quantize-append, split-K scan, combine) in stream order"),
               step_form_trial_ms={k: v / max(args.steps, 5) for k, v in trial.items()})

    peak, peak_src = hbm_peak()
    alg_bytes = B * Hkv * (S + 1) * bytes_per_token_head(kind, n_out)

    def roof(ms_list, what):
        m, lo_ = allreduce_max([statistics.median(ms_list), min(ms_list)], dev, dist)
        us = m * 1e3 / L
        ach = alg_bytes / (us * 1e-6) / 1e9
        return {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                "traffic": alg_bytes * NCU_TRAFFIC_RATIO.get(kind, 1.0),
                "traffic_source": f"algorithmic bytes x {NCU_TRAFFIC_RATIO.get(kind, 1.0)}: a stored constant, the ratio "
                                  f"dram bytes / algorithmic bytes of one ncu capture of this kernel ({PROFILE_OF.get(kind)}), "
                                  "not a measurement of this run",
                "peak_source": peak_src, "kernel": what, "us_per_launch": us, "us_per_launch_min": lo_ * 1e3 / L,
                "algorithmic_bytes_per_launch": alg_bytes, "frac_of_8TBps": ach / 8000.0,
                "timed": f"{len(ms_list)} blocks of {args.steps} graph replays of the {L} scans, CUDA events, per GPU"}
    res["roofline"] = roof(scan_ms["default"], "decode split-K scan" + (" (packed INT4, factored scales: library default)" if int4 else ""))
    if "bit_faithful" in scan_ms:
        res["roofline_bit_faithful"] = roof(scan_ms["bit_faithful"],
                                            "decode split-K scan (packed INT4, fp16 dequantisation bit for bit as the reference's torch path)")

    if parity and kind != "kivi4":
        g_step.replay()
        torch.cuda.synchronize()
        rows = sorted({0, B - 1})
        try:
            res["parity_check"] = parity_check(wl, cache, q, inv_tau, out[0], rows)
        except Exception as e:      # the oracle library is test infrastructure: its absence must not hide the numbers
            res["parity_check"] = {"ok": None, "error": repr(e)[:200]}

    # end to end through the public API with HOST buffers: every step uploads this token's q / k / v
    # for all layers from pinned memory, replays the captured whole-stack step (append + attention per
    # layer, device-side position counter, the cache grows by one token) and downloads the outputs
    if e2e and kind != "kivi4":
        from llm_kvcache_quantization_b200.runtime import GraphedKVStackStep
        stepper = GraphedKVStackStep(cache, Hq, 1.0 / D ** 0.5, inv_tau=inv_tau,
                                     overlap_append=step_form == "append beside the scan")
        stepper.capture()
        stepper.host_q.copy_(q.cpu()); stepper.host_k.copy_(k_new.cpu()); stepper.host_v.copy_(v_new.cpu())
        room = stepper.capacity - stepper._len - 1
        for _ in range(3):
            stepper.step(stepper.host_q, stepper.host_k, stepper.host_v)
        room -= 3
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def e2e_block(steps):
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(steps):
                r = stepper.step(stepper.host_q, stepper.host_k, stepper.host_v)
            e1.record()
            torch.cuda.synchronize()
            assert bool(torch.isfinite(r.float()).all())
            return e0.elapsed_time(e1)
        # the cache grows by one token per step: as many blocks as the reserved slots allow, at least one
        nb = max(1, min(int(room // max(args.steps, 1)), 200))
        ems, tot = [], 0.0
        for _ in range(nb):
            ms, = allreduce_max([e2e_block(args.steps)], dev, dist)
            ems.append(ms / args.steps)
            tot += ms
            if tot >= args.min_seconds * 1e3:
                break
        em, = allreduce_max([statistics.median(ems)], dev, dist)
        res["e2e"] = {"value": B_total / (em * 1e-3), "unit": "tokens/s",
                      "h2d_bytes_per_step": stepper.h2d_bytes_per_step * world,
                      "d2h_bytes_per_step": stepper.d2h_bytes_per_step * world, "ms_per_step": em, "blocks": len(ems),
                      "api": "GraphedKVStackStep.step(host_q, host_k, host_v) -> host_out: one CUDA graph launch holding the "
                             "pinned H2D copies of q/k/v, append + attention for every layer, and the pinned D2H of the "
                             "outputs; stream sync"}
        del stepper

    if args.decompose and world == 1 and kind != "kivi4":
        # where a layer's time goes: graphs of the scan alone, scan + combine, and the two forms of the whole step
        # (L2 is not flushed between replays here: meaningful for stacks larger than L2 or read as a warm-cache figure)
        dec = {}
        for label, kw, env in (("scan", dict(stages=1, with_append=False), None),
                               ("scan_combine", dict(stages=0, with_append=False), None),
                               ("step_append_in_order", dict(), "1"), ("step_append_beside", dict(), "0")):
            old = os.environ.get("KVQ_BENCH_NO_OVERLAP")
            if env is not None:
                os.environ["KVQ_BENCH_NO_OVERLAP"] = env
            try:
                fn, _ = make_step(wl, cache, q, k_new, v_new, inv_tau, out, **kw)
                gph = capture(fn)
            finally:
                if env is not None:
                    if old is None:
                        os.environ.pop("KVQ_BENCH_NO_OVERLAP", None)
                    else:
                        os.environ["KVQ_BENCH_NO_OVERLAP"] = old
            time_graph(gph, 5)
            dec[label] = min(time_graph(gph, 30) for _ in range(5)) / 30 / L * 1e3
            del gph
        res["decomposition_us_per_layer"] = dec

    # the callers either side of the decode path (dequantising read-back, bulk prefill append): always for configuration 2
    if (args.aux or name == "c2") and kind not in ("fp16", "kivi4") and world == 1:
        res["aux"] = time_aux(wl, cache, dev)
    if args.model_step and world == 1 and (Hq, Hkv) in MODEL_GEOMETRY:
        try:
            res["model_step"] = time_model_step(wl, cache, dev, steps=max(3, min(args.steps, 10)))
        except Exception as e:
            res["model_step"] = {"error": repr(e)[:300]}
    if cpu and rank == 0 and kind not in ("fp16", "kivi4"):
        try:
            res["cpu_baseline"] = cpu_baseline(dict(wl, B=B_total))
        except Exception as e:
            res["cpu_baseline"] = {"error": repr(e)[:300]}
    del g_step, scans, cache, q, k_new, v_new, out, flush
    ops.release_workspaces()
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------- sequence sharding (one long sequence)
def run_sequence_sharded(args, wl, dev, dist, rank, world, collective):
    """KV-sequence sharding of a single long sequence over `world` GPUs: rank r owns a contiguous
    chunk of tokens, the owner of position S appends the new token, every rank runs the fused
    decode over its chunk into a packed normalised partial, the partials cross NVLink once per layer
    (the library's fused combine / peer-store / merge kernel, or ONE NCCL all-gather), and every rank merges
    them.  The whole step (kernels and collectives) is one CUDA graph.  Returns the result object (rank 0)."""
    import torch
    from llm_kvcache_quantization_b200 import ops, _lib, parallel as P

    L, B, Hq, Hkv, S, kind, n_out = (wl[k] for k in ("layers", "B", "Hq", "Hkv", "S", "kind", "n_out"))
    sh = P.SequenceSharding(world=world, max_seq_len=S + 1, align=128)
    n_old = sh.local_len(rank, S)                    # cached tokens of this rank before the step
    owner = sh.owner_of(S) == rank                   # this rank stores the new token
    n_att = n_old + (1 if owner else 0)
    local = dict(wl, S=n_old)
    # the inputs of a step are replicated in a real deployment; here rank 0's are broadcast
    cache, q, k_new, v_new, inv_tau = build_workload(local, dev, seed=1234 + rank, extra_slots=8)
    for t in (q, k_new, v_new, inv_tau):
        dist.broadcast(t, src=0)
    fmt = _lib.FMT_INT8 if kind.startswith("int8") else _lib.FMT_INT4
    out = torch.empty(L, B, Hq, D, dtype=torch.float16, device=dev)
    send = torch.empty(B, Hq, D + 2, dtype=torch.float32, device=dev)
    recv = torch.empty(world, B, Hq, D + 2, dtype=torch.float32, device=dev)
    P.check_partial_shapes(send.shape)
    fused = collective == "fused"
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
                                out=out[l], stages=1, tail_tokens=1, **extra)
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
    time_graph(g_scan, args.warmup, dist)
    step_ms = timed_blocks(lambda n: time_graph(g_step, n, dist), args.steps, args.min_seconds, dist, dev)
    scan_ms = timed_blocks(lambda n: time_graph(g_scan, n, dist), args.steps, args.min_seconds, dist, dev)
    ms, ms_min, sc = allreduce_max([statistics.median(step_ms), min(step_ms), statistics.median(scan_ms)], dev, dist)
    peak, peak_src = hbm_peak()
    alg_bytes = B * Hkv * sh.chunk * bytes_per_token_head(kind, n_out)       # the largest shard
    scan_us = sc * 1e3 / L
    achieved = alg_bytes / (scan_us * 1e-6) / 1e9
    status = int(xchg.status.item()) if fused else None
    res = {"collective": ("fused kernel: combine + peer stores of [B,Hq,D+2] fp32 over NVLink + merge, one launch per layer"
                          if fused else "one NCCL all-gather of [B,Hq,D+2] fp32 per layer, then the merge kernel"),
           "ms_per_step": ms, "ms_per_step_min": ms_min, "blocks": len(step_ms), "us_per_layer": ms * 1e3 / L,
           "tokens_per_s": B / (ms * 1e-3), "chunk_tokens": sh.chunk, "splits": splits, "exchange_status": status,
           "scan_us_per_layer": scan_us, "scan_frac_of_measured_hbm": achieved / peak, "peak_source": peak_src,
           "gpu_launches": len(step_ms) * args.steps * L * (3 if fused else 4)}
    del g_step, g_scan, xchg, cache
    ops.release_workspaces()
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------- main
EXTRA_WORKLOADS = ("c1", "c2", "c3", "c5", "c2_kivi4")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS),
                    help="headline workload (default: configuration 4, the largest that fits one GPU)")
    ap.add_argument("--min-seconds", type=float, default=0.5, help="minimum length of every timed region")
    ap.add_argument("--no-extras", action="store_true", help="measure the headline workload only")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling captures only)")
    ap.add_argument("--decompose", action="store_true",
                    help="also time graphs of the scan alone, scan + combine and both forms of the step (us per layer)")
    ap.add_argument("--aux", action="store_true",
                    help="also time the neighbouring kernels at the headline shape: bulk prefill quantize-append "
                         "(T = context) and the dequantising get_kv, one layer each")
    ap.add_argument("--model-step", action="store_true",
                    help="also time one decode step of a random-init Qwen2 model of the headline geometry through "
                         "the patched attention forward over the same synthetic cache (weights, MLP, eager Python "
                         "included); reported under model_step")
    ap.add_argument("--collective", default="both", choices=("both", "fused", "nccl"),
                    help="sequence-sharded sub-result: the library's fused combine/peer-store/merge kernel, "
                         "combine + NCCL all-gather + merge, or both")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.layers > 0:
        wl["layers"] = args.layers
        wl["desc"] += f" [layers overridden to {args.layers}]"
        args.no_extras = True
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args, args.workload, wl)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # the fused exchange uses plain peer stores; symmetric-memory buffers are never bound to an NVLink multicast object
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    import torch
    import llm_kvcache_quantization_b200 as kvq  # noqa: F401
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
    t_start = time.time()

    head = measure_workload(args.workload, wl, args, dev, dist, rank, world, e2e=not args.no_e2e,
                            cpu=not args.no_cpu_baseline and world == 1)
    if "skipped" in head and args.workload == "c4":
        # a GPU with less free memory than the 64 GB stack needs: fall back to the next largest configuration
        note = head["skipped"]
        args.workload, wl = "c3", dict(WORKLOADS["c3"])
        head = measure_workload("c3", wl, args, dev, dist, rank, world, e2e=not args.no_e2e,
                                cpu=not args.no_cpu_baseline and world == 1)
        head["headline_fallback"] = f"configuration 4 skipped ({note})"

    extra = {}
    if world == 1 and not args.no_extras:
        if args.workload == "c4" and not args.model_step and (wl["Hq"], wl["Hkv"]) in MODEL_GEOMETRY:
            pass    # the random-init 7B model step of configuration 4 is opt-in (--model-step): it adds ~1 minute
        items = []
        for name in EXTRA_WORKLOADS:
            if name == args.workload:
                continue
            try:
                r = measure_workload(name, dict(WORKLOADS[name]), args, dev, None, 0, 1, e2e=not args.no_e2e,
                                     cpu=(name == "c2" and not args.no_cpu_baseline))
            except Exception as e:
                r = {"name": name, "error": repr(e)[:300]}
            items.append(r)
        extra["workloads"] = items
    if world > 1 and not args.no_extras:
        # configuration 5, one sequence of 131072 tokens: KV-sequence sharding over the same N GPUs, and the same step
        # on one GPU (rank 0, the others wait) for the speed-up
        c5 = dict(WORKLOADS["c5"])
        seq = {"config": workload_config(c5, "c5", world)}
        which = ("fused", "nccl") if args.collective == "both" else (args.collective,)
        for coll in which:
            # every rank runs the same calls; a failure on one rank surfaces on all through the collective's timeout
            try:
                seq[coll] = run_sequence_sharded(args, c5, dev, dist, rank, world, coll)
            except Exception as e:
                import traceback
                traceback.print_exc()
                seq[coll] = {"error": repr(e)[:300]}
        if rank == 0:
            try:
                one = measure_workload("c5", c5, args, dev, None, 0, 1, e2e=False, parity=False)
                seq["single_gpu_us_per_layer"] = one.get("us_per_layer")
                for coll in which:
                    if one.get("us_per_layer") and seq[coll].get("us_per_layer"):
                        seq[coll]["speedup_over_one_gpu"] = one["us_per_layer"] / seq[coll]["us_per_layer"]
            except Exception as e:
                import traceback
                traceback.print_exc()
                seq["single_gpu_error"] = repr(e)[:300]
        extra["sequence_sharded"] = seq

    if rank == 0:
        line = {
            "metric": "decode_tokens_per_s", "value": head.get("value"), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head.get("ms_per_step"),
            "ms_per_step_min": head.get("ms_per_step_min"), "timed_blocks": head.get("blocks"),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": head["config"], "batch_per_gpu": head.get("batch_per_gpu"), "splits": head.get("splits"),
            "step": head.get("step"), "us_per_layer": head.get("us_per_layer"),
            "roofline": head.get("roofline"), "cpu_baseline": head.get("cpu_baseline"), "e2e": head.get("e2e"),
            "gpu_launches": head.get("gpu_launches"), "clocks": head.get("clocks"),
            "parity_check": head.get("parity_check"),
        }
        for k in ("roofline_bit_faithful", "aux", "model_step", "headline_fallback", "skipped", "step_form_trial_ms",
                  "decomposition_us_per_layer"):
            if k in head:
                line[k] = head[k]
        if extra:
            line["extra"] = extra
        line["bench_seconds"] = time.time() - t_start
        print(json.dumps(line), flush=True)
    if dist is not None:
        # Tearing the process group down while captured graphs still hold its collectives did not return in a
        # two-GPU run: drain, agree that every rank is done, and leave without the teardown.
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
