"""Whole-stack decode step as ONE CUDA graph.

`GraphedKVStackStep` runs, for every layer of a KV cache, the fused quantize-append of the new
token followed by the fused decode attention - the two library calls the patched attention
forward makes per layer - as a single captured graph with a device-resident position counter,
so that one host call (three pinned-memory uploads, one graph launch, one download) advances the
whole stack by one token.  It replaces ~25 eager launches and several host syncs per layer in
the reference's decode loop (src/engine/generate_loop.py:1320-1498, src/cache/int8_cache.py:350-488).

The cache must be preallocated (`cache.reserve`) because graph replay needs stable addresses;
lengths live on the device (`write_pos_dev`, `context_lens`) and are advanced inside the graph.

With `overlap_append` the append of a layer runs on a second stream concurrently with the split-K scan
of the same layer: the scan skips the new token (`tail_tokens = 1`) and the combine stage, which waits
for both, attends it straight from the cache.  The append leaves the critical path, the fork and join of
the second stream enter it: measured, that pays for layers of hundreds of megabytes (1 % at 2.3 GB per
layer) and costs 1-2 us per layer on small ones, so the default (`None`) turns it on from 512 MB of cached
bytes per layer.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib, ops
from .cache import FP16KVCache, INT4KVCache, INT8KVCache


class GraphedKVStackStep:
    def __init__(self, cache, num_q_heads: int, sm_scale: float, inv_tau: Optional[torch.Tensor] = None,
                 capacity: Optional[int] = None, overlap_append: Optional[bool] = None):
        if not isinstance(cache, (INT8KVCache, INT4KVCache, FP16KVCache)):
            raise TypeError("GraphedKVStackStep needs one of this package's caches")
        self.cache = cache
        L = cache.num_layers
        b0 = cache._bufs[0]
        if b0 is None:
            raise ValueError("preallocate the cache (append a prompt or call reserve) before building the step")
        B, Hkv, cap_phys = b0["k"].shape[0], b0["k"].shape[1], b0["k"].shape[2]
        packed = cache._fmt == _lib.FMT_INT4 and getattr(cache, "bit_packed", True)
        D = b0["k"].shape[3] * (2 if packed else 1)
        self.L, self.B, self.Hq, self.Hkv, self.D = L, B, num_q_heads, Hkv, D
        self.capacity = min(cap_phys, capacity or cache._layer_capacity[0])
        dev = b0["k"].device
        self.device = dev
        self.sm_scale = float(sm_scale)
        self.inv_tau = None if inv_tau is None else inv_tau.to(device=dev, dtype=torch.float32).contiguous()
        lens = set(cache._layer_seq_lens)
        if len(lens) != 1:
            raise ValueError("all layers must hold the same number of tokens")
        self._len = lens.pop()
        # device state advanced inside the graph
        self.pos = torch.full((1,), self._len, dtype=torch.int32, device=dev)
        self.ctx = torch.full((B,), self._len + 1, dtype=torch.int32, device=dev)
        # device staging + pinned host mirrors.  q | k | v of one layer are contiguous (one upload per layer);
        # the public tensors are views into the staging rows
        nq, nk = B * num_q_heads * D, B * Hkv * D
        self._stage = torch.empty(L, nq + 2 * nk, dtype=torch.float16, device=dev)
        self._host_stage = torch.empty(L, nq + 2 * nk, dtype=torch.float16).pin_memory()

        def views(t):
            return (t[:, :nq].view(L, B, num_q_heads, D), t[:, nq:nq + nk].view(L, B, Hkv, 1, D),
                    t[:, nq + nk:].view(L, B, Hkv, 1, D))
        self.q, self.k_new, self.v_new = views(self._stage)
        self.host_q, self.host_k, self.host_v = views(self._host_stage)
        self.out = torch.empty(L, B, num_q_heads, D, dtype=torch.float16, device=dev)
        self.host_out = torch.empty(self.out.shape, dtype=torch.float16).pin_memory()
        self.graph = None
        self.graph_host = None
        self.launches_per_step = 0
        if overlap_append is None:
            layer_bytes = sum(t[:, :, :self.capacity].numel() * t.element_size() for t in b0.values())
            overlap_append = layer_bytes >= (512 << 20)
        self.overlap_append = bool(overlap_append)
        self._side = torch.cuda.Stream(device=dev) if self.overlap_append else None

    def _append_then_attend(self, append, attend) -> None:
        """`append()` launches the quantize-append, `attend(**kw)` the decode attention."""
        if not self.overlap_append:
            append()
            attend()
            return
        main = torch.cuda.current_stream(self.device)
        self._side.wait_stream(main)                  # this token's k / v and the position counter are ready
        with torch.cuda.stream(self._side):
            append()
        attend(stages=1, tail_tokens=1)               # scan of the old tokens, independent of the append
        main.wait_stream(self._side)
        attend(stages=2, tail_tokens=1)               # combine + the new token

    # one layer: append at the device-side position, then attend over pos+1 tokens
    def _layer(self, l: int) -> None:
        c = self.cache
        b = c._bufs[l]
        cap = self.capacity
        view = {n: t[:, :, :cap] for n, t in b.items()}
        fmt = c._fmt
        if fmt == _lib.FMT_FP16:
            self._append_then_attend(
                lambda: ops.quantize_append(fmt, _lib.SCALE_STATIC, self.k_new[l], self.v_new[l], b["k"], b["v"],
                                            None, None, self.pos, self.D),
                lambda **kw: ops.decode_attn(fmt, self.q[l], view["k"], view["v"], None, None, self.ctx, self.sm_scale,
                                             head_dim=self.D, inv_tau=None if self.inv_tau is None else self.inv_tau[l],
                                             out=self.out[l], max_ctx=cap, **kw))
            return
        G = b["ks"].shape[-1]
        gs = self.D // G
        app, att = {}, {}
        flags = 0
        dfmt = fmt                                     # unpacked INT4 codes are read by the kernels as INT8
        if fmt == _lib.FMT_INT4 and not getattr(c, "bit_packed", True):
            flags |= _lib.F_UNPACKED
            dfmt = _lib.FMT_INT8
        if getattr(c, "asymmetric", False):
            policy = _lib.SCALE_ASYM_MINMAX
            app.update(k_zp=b["kz"], v_zp=b["vz"])
            att.update(k_zp=view["kz"], v_zp=view["vz"])
        elif c.static_k_scale is not None:
            policy = _lib.SCALE_STATIC
            app.update(k_static=c._static_table("k", l, self.Hkv, G, self.device),
                       v_static=c._static_table("v", l, self.Hkv, G, self.device))
            if c.adaptive_static_scales and (c.adaptive_static_k or c.adaptive_static_v):
                flags |= _lib.F_ADAPTIVE
                if not c.adaptive_static_k:
                    flags |= _lib.F_ADAPT_SKIP_K
                if not c.adaptive_static_v:
                    flags |= _lib.F_ADAPT_SKIP_V
            if getattr(c, "mixed_rescue", False) or getattr(c, "outlier_rescue_ratio", 0.0) >= 1.0:
                flags |= _lib.F_MIXED_RESCUE
            elif getattr(c, "outlier_rescue_ratio", 0.0) > 0.0:
                raise ValueError("outlier_rescue_ratio in (0,1) needs a per-append quantile and is not graph-capturable")
        else:
            policy = _lib.SCALE_DYNAMIC_PCT
            p = float(c.clip_percentile)
            app.update(quantile=(max(min(p / 100.0, 1.0), 0.0) if p < 100.0 else 1.0))
        if c.outlier_idx is not None:
            oidx = c.outlier_idx[l].to(self.device).contiguous()
            app.update(outlier_idx=oidx, k_side=b["kside"], v_side=b["vside"])
            att.update(outlier_idx=oidx, k_side=view["kside"], v_side=view["vside"])
        self._append_then_attend(
            lambda: ops.quantize_append(fmt, policy, self.k_new[l], self.v_new[l], b["k"], b["v"], b["ks"], b["vs"],
                                        self.pos, gs, flags=flags, adaptive_margin=float(c.adaptive_static_margin),
                                        k_scale_f32=b.get("ks32"), v_scale_f32=b.get("vs32"), **app),
            lambda **kw: ops.decode_attn(dfmt, self.q[l], view["k"], view["v"], view["ks"], view["vs"], self.ctx,
                                         self.sm_scale, head_dim=self.D,
                                         inv_tau=None if self.inv_tau is None else self.inv_tau[l], out=self.out[l],
                                         max_ctx=cap, **att, **kw))

    def _body(self) -> None:
        for l in range(self.L):
            self._layer(l)
        self.pos.add_(1)
        self.ctx.add_(1)

    def capture(self) -> None:
        """Warm up once eagerly on a side stream (first-use set-up, workspace growth), rewind the
        device counters, then capture the step."""
        if self._len + 1 > self.capacity:              # the warm-up below appends at slot `_len`
            raise ValueError(f"cache capacity {self.capacity} exhausted: nothing left to capture a step into")
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self._body()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        self.pos.fill_(self._len)
        self.ctx.fill_(self._len + 1)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._body()
        self.pos.fill_(self._len)
        self.ctx.fill_(self._len + 1)
        self.graph = g
        self.launches_per_step = self.L * 3
        # The host-buffer form: uploads, the step and the downloads as ONE graph launch.  The copies run on
        # their own streams in two pieces each: the first layers' inputs (small, exposed), then the rest while
        # those layers compute; all outputs but the last layers' while the last layers compute, then the tail
        # (small, exposed).  Two extra cross-stream edges in all, so the kernels of the other layers keep their
        # programmatic launch overlap.
        L = self.L
        head = min(2, L)
        tail = min(2, L - head) if L > head else 0
        up, down = torch.cuda.Stream(device=self.device), torch.cuda.Stream(device=self.device)
        gh = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gh):
            main = torch.cuda.current_stream(self.device)
            up.wait_stream(main)
            down.wait_stream(main)
            with torch.cuda.stream(up):
                self._stage[:head].copy_(self._host_stage[:head], non_blocking=True)
                first = torch.cuda.Event()
                first.record(up)
                if L > head:
                    self._stage[head:].copy_(self._host_stage[head:], non_blocking=True)
            main.wait_event(first)
            for l in range(L):
                if l == head:
                    main.wait_stream(up)
                self._layer(l)
                if tail and l == L - tail - 1:
                    down.wait_stream(main)
                    with torch.cuda.stream(down):
                        self.host_out[:L - tail].copy_(self.out[:L - tail], non_blocking=True)
            self.pos.add_(1)
            self.ctx.add_(1)
            main.wait_stream(up)
            main.wait_stream(down)
            done = L - tail if tail else 0             # layers whose output went out with the early download
            self.host_out[done:].copy_(self.out[done:], non_blocking=True)
        self.pos.fill_(self._len)
        self.ctx.fill_(self._len + 1)
        self.graph_host = gh

    def step_device(self) -> torch.Tensor:
        """Advance by one token with inputs already in `self.q / self.k_new / self.v_new`."""
        if self.graph is None:
            self.capture()
        if self._len + 1 > self.capacity:
            raise ValueError(f"cache capacity {self.capacity} exhausted")
        self.graph.replay()
        self._len += 1
        for i in range(self.L):
            self.cache._layer_seq_lens[i] = self._len
        self.cache._seq_len = self._len
        return self.out

    def step(self, host_q: torch.Tensor, host_k: torch.Tensor, host_v: torch.Tensor) -> torch.Tensor:
        """Host-to-host step: upload this token's q / k / v for all layers (pinned memory, one copy
        each), replay the graph, download the attention outputs.  Returns the pinned output buffer
        (valid until the next call) after synchronising the stream."""
        if self.graph is None:
            self.capture()
        if self._len + 1 > self.capacity:
            raise ValueError(f"cache capacity {self.capacity} exhausted")
        if host_q is not self.host_q:
            self.host_q.copy_(host_q)
            self.host_k.copy_(host_k)
            self.host_v.copy_(host_v)
        self.graph_host.replay()                       # pinned uploads, every layer, pinned downloads
        self._len += 1
        for i in range(self.L):
            self.cache._layer_seq_lens[i] = self._len
        self.cache._seq_len = self._len
        torch.cuda.current_stream(self.device).synchronize()
        return self.host_out

    @property
    def h2d_bytes_per_step(self) -> int:
        return (self.q.numel() + self.k_new.numel() + self.v_new.numel()) * 2

    @property
    def d2h_bytes_per_step(self) -> int:
        return self.out.numel() * 2


class GraphedModelStep:
    """One greedy decode step of a HuggingFace causal LM as ONE CUDA graph: embedding, every layer (norms,
    projections, the patched attention with fused RoPE + quantize-append + fused decode attention, MLP),
    final norm, lm_head, argmax - and the feedback of the chosen token into the next step's input.  The
    per-step host work of the reference's decode loop (src/engine/generate_loop.py:1320-1498: Python
    dispatch of every op, position tensors, cache bookkeeping) shrinks to one graph launch.

    The cache must hold the prompt already and have `capacity` slots reserved in every layer; positions
    live on the device and advance inside the graph.  The attention-forward patch of `engine` is applied
    for the lifetime of this object (`close()` removes it).
    """

    def __init__(self, model, cache, batch: int, capacity: Optional[int] = None):
        from . import engine as E
        self.model, self.cache = model, cache
        self.L = cache.num_layers
        lens = set(cache._layer_seq_lens)
        if len(lens) != 1:
            raise ValueError("all layers must hold the same number of tokens")
        self._len = lens.pop()
        b0 = cache._bufs[0]
        if b0 is None:
            raise ValueError("prefill the cache (and reserve room for the new tokens) first")
        self.capacity = min(b0["k"].shape[2], capacity or cache._layer_capacity[0])
        dev = b0["k"].device
        self.device, self.B = dev, batch
        self.pos = torch.full((1,), self._len, dtype=torch.int32, device=dev)
        self.ctx = torch.full((batch,), self._len + 1, dtype=torch.int32, device=dev)
        self.pos_ids = torch.full((batch, 1), self._len, dtype=torch.long, device=dev)
        self.tok = torch.zeros((batch, 1), dtype=torch.long, device=dev)
        self.next_tok = torch.zeros((batch, 1), dtype=torch.long, device=dev)
        self.logits = None
        self.graph = None
        self._E = E
        E.apply_int8_fused_patch(model)
        self.wrapper = E.INT8CacheWrapperContainer(cache, self.L)

    def _body(self) -> None:
        out = self.model(input_ids=self.tok, position_ids=self.pos_ids, past_key_values=self.wrapper, use_cache=True)
        self.logits = out.logits
        self.next_tok.copy_(out.logits[:, -1].argmax(-1, keepdim=True))
        self.tok.copy_(self.next_tok)                 # greedy feedback: the next replay consumes it
        self.pos.add_(1)
        self.ctx.add_(1)
        self.pos_ids.add_(1)

    def _rewind(self) -> None:
        self.pos.fill_(self._len)
        self.ctx.fill_(self._len + 1)
        self.pos_ids.fill_(self._len)

    def capture(self, first_token: torch.Tensor) -> None:
        """`first_token` [B,1]: the token the prompt's last logits chose."""
        if self._len + 1 > self.capacity:              # the warm-up below appends at slot `_len`
            raise ValueError(f"cache capacity {self.capacity} exhausted: nothing left to capture a step into")
        self.cache.use_device_positions(self.pos, self.ctx, self.capacity)
        keep = first_token.to(self.device).clone()
        with torch.no_grad():
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                self.tok.copy_(keep)
                self._body()                          # warm-up: lazy initialisation, workspaces, autotuned GEMMs
            torch.cuda.current_stream(self.device).wait_stream(s)
            torch.cuda.synchronize(self.device)
            self._rewind()
            self.tok.copy_(keep)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._body()
            self._rewind()
            self.tok.copy_(keep)
        self.graph = g

    def step(self) -> torch.Tensor:
        """Advance by one token; returns the device tensor [B,1] of the tokens just chosen (valid until the
        next call; no host synchronisation)."""
        if self.graph is None:
            raise RuntimeError("capture(first_token) first")
        if self._len + 1 > self.capacity:
            raise ValueError(f"cache capacity {self.capacity} exhausted")
        self.graph.replay()
        self._len += 1
        self.cache.advance_host_lengths(1)
        return self.next_tok

    def close(self) -> None:
        self.cache.use_host_positions()
        self._E.remove_int8_fused_patch(self.model)
