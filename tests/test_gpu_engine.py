"""End-to-end decode of a small random-init Qwen2 model through the patched forward, the cache
shims and the fused kernels, compared with plain HuggingFace decoding on the same weights."""
import os

import numpy as np
import pytest
import torch

import llm_kvcache_quantization_b200 as kvq
from llm_kvcache_quantization_b200 import engine as E
from oracle import kvq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def tiny_model():
    transformers = pytest.importorskip("transformers")
    cfg = transformers.Qwen2Config(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=3,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=1024,
                                   rope_theta=10000.0, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = transformers.Qwen2ForCausalLM(cfg).to(DEV).half().eval()
    assert model.model.layers[0].self_attn.head_dim == 128
    return model


class _Tok:
    eos_token_id = None


@torch.no_grad()
def _hf_greedy(model, ids, n):
    out = model(input_ids=ids, use_cache=True)
    pkv, tok = out.past_key_values, out.logits[:, -1].argmax(-1, keepdim=True)
    toks, logits = [tok], [out.logits[:, -1].float()]
    for _ in range(n - 1):
        out = model(input_ids=tok, past_key_values=pkv, use_cache=True)
        pkv, tok = out.past_key_values, out.logits[:, -1].argmax(-1, keepdim=True)
        toks.append(tok); logits.append(out.logits[:, -1].float())
    return torch.cat(toks, 1), torch.stack(logits, 1)


def test_fp16_mode_matches_hf_greedy(tiny_model):
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 512, (2, 40), generator=g).to(DEV)
    ref, _ = _hf_greedy(tiny_model, ids, 8)
    out = E.generate_from_ids(tiny_model, _Tok(), ids, max_new_tokens=8, kv_mode="fp16", stop_on_eos=False)
    assert out.generated_ids.shape == (2, 8) and out.kv_cache_seq_len == 47
    assert (out.generated_ids == ref).float().mean() >= 0.8      # random-init logits are nearly flat: allow ties
    assert torch.equal(out.generated_ids[:, 0], ref[:, 0])
    assert not hasattr(type(tiny_model.model.layers[0].self_attn), "_original_forward")   # unpatched in finally


@pytest.mark.parametrize("mode", ("int8_baseline", "int4_baseline"))
def test_quantized_modes_track_fp16_logits(tiny_model, mode):
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 512, (2, 64), generator=g).to(DEV)
    model = tiny_model
    _, ref_logits = _hf_greedy(model, ids, 2)
    cache = E.build_cache(mode, 3, DEV, group_size=32, clip_percentile=100.0, max_seq_len=128)
    E.apply_int8_fused_patch(model)
    try:
        with torch.no_grad():
            first = E._prefill_into_cache(model, cache, ids, torch.ones_like(ids))
            tok = first.argmax(-1, keepdim=True)
            pos = torch.full((2, 1), 64, dtype=torch.long, device=DEV)
            out = model(input_ids=tok, position_ids=pos, past_key_values=E.INT8CacheWrapperContainer(cache, 3),
                        use_cache=True)
    finally:
        E.remove_int8_fused_patch(model)
    got = out.logits[:, -1].float()
    err = (got - ref_logits[:, 1]).abs().max().item()
    scale = ref_logits[:, 1].abs().max().item()
    assert err < (0.02 if mode.startswith("int8") else 0.25) * max(scale, 1.0), (err, scale)
    st = cache.get_decode_stats()
    assert st["fused_decode_calls"] == 3 and st["triton_kernel_calls"] == 3 and cache.get_seq_len() == 65


def test_torch_ref_impl_agrees_with_fused(tiny_model):
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 512, (1, 50), generator=g).to(DEV)
    outs = {}
    for impl in ("triton_fused", "torch_ref"):
        cache = E.build_cache("int8_baseline", 3, DEV, group_size=32, clip_percentile=100.0, max_seq_len=64)
        cache.decode_attn_impl = impl
        E.apply_int8_fused_patch(tiny_model)
        try:
            with torch.no_grad():
                first = E._prefill_into_cache(tiny_model, cache, ids, torch.ones_like(ids))
                tok = first.argmax(-1, keepdim=True)
                pos = torch.full((1, 1), 50, dtype=torch.long, device=DEV)
                outs[impl] = tiny_model(input_ids=tok, position_ids=pos,
                                        past_key_values=E.INT8CacheWrapperContainer(cache, 3)).logits.float()
        finally:
            E.remove_int8_fused_patch(tiny_model)
        assert cache.get_decode_stats()["torch_ref_calls" if impl == "torch_ref" else "triton_decode_calls"] == 3
    assert torch.allclose(outs["triton_fused"], outs["torch_ref"], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("overlap,L", ((False, 3), (True, 3), (True, 1), (True, 7)))
def test_graphed_stack_step_equals_eager_layer_calls(overlap, L):
    """The captured whole-stack step (device-side position, cache growing inside the graph) against eager
    per-layer append + fused decode, over several steps: bit-identical caches always; outputs within the attention
    tolerance (the two forms may hand the newest token to different stages - the combine stage attends it when the
    append runs beside the scan, and whenever a packed-INT4 view has an odd length - i.e. another summation order)."""
    import llm_kvcache_quantization_b200 as kvq
    from llm_kvcache_quantization_b200.runtime import GraphedKVStackStep
    g = torch.Generator().manual_seed(5)
    B, Hq, Hkv, S, D, steps = 2, 12, 2, 200, 128, 4         # L = 1 / 3 / 7: every shape of the two-piece copy pipeline
    for make in (lambda: kvq.INT4KVCache(L, device=DEV, group_size=32, asymmetric=True, max_seq_len=S + 8),
                 lambda: kvq.INT8KVCache(L, device=DEV, group_size=32, clip_percentile=100.0, max_seq_len=S + 8),
                 lambda: kvq.FP16KVCache(L, device=DEV, max_seq_len=S + 8)):
        ca, cb = make(), make()
        for l in range(L):
            k = torch.randn(B, Hkv, S, D, generator=g).half().to(DEV)
            v = torch.randn(B, Hkv, S, D, generator=g).half().to(DEV)
            for c in (ca, cb):
                c.reserve(l, B, Hkv, D, S + 8)
                c.append(l, k, v)
        tau = torch.empty(L, Hq).uniform_(0.8, 1.2, generator=g).to(DEV)
        st = GraphedKVStackStep(ca, Hq, 0.088, inv_tau=tau, overlap_append=overlap)
        for _ in range(steps):
            hq = torch.randn(L, B, Hq, D, generator=g).half()
            hk = torch.randn(L, B, Hkv, 1, D, generator=g).half()
            hv = torch.randn(L, B, Hkv, 1, D, generator=g).half()
            got = st.step(hq, hk, hv).clone()
            for l in range(L):
                cb.append(l, hk[l].to(DEV), hv[l].to(DEV))
                ref = cb.fused_decode(l, hq[l].to(DEV), 0.088, inv_tau=tau[l])
                err = (got[l].to(DEV).float() - ref.float()).abs()
                assert bool((err <= 2e-3 + 1e-2 * ref.float().abs()).all()), (l, float(err.max()))
        assert ca.get_seq_len() == cb.get_seq_len() == S + steps
        for l in range(L):
            if isinstance(ca, kvq.FP16KVCache):
                for x, y in zip(ca.get_kv(l), cb.get_kv(l)):
                    assert torch.equal(x, y)
                continue
            ta, tb = ca.get_decode_tensors(l), cb.get_decode_tensors(l)
            for n in ("k", "v", "ks", "vs"):
                assert torch.equal(ta[n], tb[n])


def test_graphed_model_step_matches_the_eager_patched_loop(tiny_model):
    """Whole-model greedy decode as one CUDA graph per token (device-side positions, token fed back on
    the device) against the eager patched forward on a second cache with the same prompt."""
    import llm_kvcache_quantization_b200 as kvq
    from llm_kvcache_quantization_b200.runtime import GraphedModelStep
    g = torch.Generator().manual_seed(11)
    B, P, N = 2, 48, 6
    ids = torch.randint(0, 512, (B, P), generator=g).to(DEV)
    model = tiny_model

    def fresh():
        c = E.build_cache("int8_baseline", 3, DEV, group_size=32, clip_percentile=100.0, max_seq_len=P + N + 8)
        with torch.no_grad():
            first = E._prefill_into_cache(model, c, ids, torch.ones_like(ids))
        for l in range(3):
            c.reserve(l, B, 2, 128, P + N + 8)
        return c, first.argmax(-1, keepdim=True)

    ca, tok0 = fresh()
    cb, _ = fresh()
    # eager reference: patched forward, host-side positions
    E.apply_int8_fused_patch(model)
    try:
        ref, tok = [], tok0
        with torch.no_grad():
            for i in range(N):
                pos = torch.full((B, 1), P + i, dtype=torch.long, device=DEV)
                out = model(input_ids=tok, position_ids=pos, past_key_values=E.INT8CacheWrapperContainer(cb, 3),
                            use_cache=True)
                tok = out.logits[:, -1].argmax(-1, keepdim=True)
                ref.append(tok)
    finally:
        E.remove_int8_fused_patch(model)
    st = GraphedModelStep(model, ca, B)
    try:
        st.capture(tok0)
        got = [st.step().clone() for _ in range(N)]
    finally:
        st.close()
    assert ca.get_seq_len() == cb.get_seq_len() == P + N
    assert torch.equal(torch.cat(got, 1), torch.cat(ref, 1))
    for l in range(3):
        for a, b in zip(ca.get_int8_tensors(l), cb.get_int8_tensors(l)):
            assert torch.equal(a, b)
    assert not hasattr(type(model.model.layers[0].self_attn), "_original_forward")


@pytest.mark.parametrize("bits", (8, 4))
def test_kivi_style_mode_generates(tiny_model, bits):
    """kv_mode="kivi_style": prompt K/V quantized per channel / per token, decode through the patched forward
    (dequantise + tensor-core fp16 attention); INT8 tracks plain HF greedy decoding on the first tokens."""
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, 512, (2, 40), generator=g).to(DEV)
    ref, _ = _hf_greedy(tiny_model, ids, 6)
    out = E.generate_from_ids(tiny_model, _Tok(), ids, max_new_tokens=6, kv_mode="kivi_style", quant_bits=bits,
                              residual_length=4 if bits == 4 else 0, stop_on_eos=False)
    assert out.generated_ids.shape == (2, 6) and out.kv_cache_seq_len == 45
    assert torch.equal(out.generated_ids[:, 0], ref[:, 0])          # the first token comes from the fp16 prefill
    if bits == 8:
        assert (out.generated_ids == ref).float().mean() >= 0.6


@pytest.mark.parametrize("mode", ("int4_ours_asym", "int4_ours_asym_ba", "int4_kivi_aligned"))
def test_role_aware_modes_generate(tiny_model, mode, tmp_path):
    """The KIVI-format modes that read a calibration file (src/engine/generate_loop.py:951-1060): the percentiles reach
    the cache, inv_tau only where the mode uses it, generation runs through the fused decode of the KIVI cache and
    equals a KIVIStyleKVCache run with the same settings."""
    import json
    cfg = tiny_model.config
    L, Hq = cfg.num_hidden_layers, cfg.num_attention_heads
    tau = [[1.0 + 0.01 * (l + h) for h in range(Hq)] for l in range(L)]
    f = tmp_path / "ra.json"
    f.write_text(json.dumps({"role_aware": {"k_percentile": 99.5, "v_percentile": 99.0, "inv_tau": tau},
                             "k_calibration": {"inv_tau": tau}, "v_calibration": {"v_percentile": 99.0}}))
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, 512, (2, 33), generator=g).to(DEV)
    seen = {}
    real = E.build_cache

    def spy(*a, **k):
        seen["cache"] = real(*a, **k)
        return seen["cache"]
    E.build_cache = spy
    try:
        out = E.generate_from_ids(tiny_model, _Tok(), ids, max_new_tokens=5, kv_mode=mode, calib_file=str(f), stop_on_eos=False)
    finally:
        E.build_cache = real
    c = seen["cache"]
    assert out.generated_ids.shape == (2, 5) and out.kv_cache_seq_len == 37
    assert c.quant_bits == 4 and c.v_percentile == 99.0
    if mode == "int4_kivi_aligned":
        assert type(c) is kvq.KIVIStyleKVCache and c.k_percentile == 100.0 and c.inv_tau is not None
    else:
        assert type(c) is kvq.RoleAwareAsymKVCache and c.k_percentile == 99.5 and c.ba_calibrated
        assert c.framework == ("ours_asym_ba" if mode.endswith("_ba") else "ours_asym")
        assert (c.inv_tau is not None) == mode.endswith("_ba") and c.use_attn_temperature == mode.endswith("_ba")
    ref, _ = _hf_greedy(tiny_model, ids, 5)
    assert torch.equal(out.generated_ids[:, 0], ref[:, 0])          # the first token comes from the fp16 prefill


# --------------------------------------------------------------------------- pinned to the reference's patched forward
def _fixture_model_and_data(golden_dir):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(golden_dir, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    fx = np.load(os.path.join(golden_dir, "engine.npz"))
    model = mg.tiny_qwen2()
    if abs(mg.weights_checksum(model) - float(fx["weights_checksum"])) > 1e-6 * float(fx["weights_checksum"]):
        pytest.skip("this torch build initialises the seeded model differently from the one that made the fixture")
    return model, fx


@pytest.mark.parametrize("mode", ("int8_ours", "int4_ours", "int4_ours_mixed"))
def test_patched_forward_matches_the_reference_run(golden_dir, mode):
    """tests/golden/engine.npz holds a run of the REFERENCE's patched forward on CPU (apply_int8_fused_patch +
    INT8CacheWrapperContainer + caches with decode_attn_impl="torch_ref", prefill temperature hooks, calibration
    with static scales and inv_tau) on a seeded tiny Qwen2.  Same weights, this package's engine on the GPU:
      1. the reference's own prefill K/V through this package's cache: cache bytes and scales bit-equal;
      2. the whole loop on the GPU (its own prefill with the temperature hooks, three decode steps, the reference's
         tokens fed back): logits within fp16 tolerance of the reference's, and the cache rows it wrote equal to
         the reference's up to the few codes that sit on a rounding boundary of the CPU / GPU projections."""
    from llm_kvcache_quantization_b200 import engine as E
    model, fx = _fixture_model_and_data(golden_dir)
    L, gs = 2, 32
    int8 = mode.startswith("int8")
    sdt = torch.float16 if int8 else torch.float32
    calib = dict(group_size=gs, clip_percentile=99.9, inv_tau=torch.from_numpy(fx["inv_tau"]).to(DEV),
                 static_k_scale=torch.from_numpy(fx[f"{mode}_k_scale"]).to(sdt).to(DEV),
                 static_v_scale=torch.from_numpy(fx[f"{mode}_v_scale"]).to(sdt).to(DEV),
                 outlier_rescue_ratio=0.0, mixed_rescue=(mode == "int4_ours_mixed"))

    def tensors(cache, l):
        return cache.get_int8_tensors(l) if int8 else cache.get_int4_tensors(l)

    # 1. quantize-on-append of the reference's prefill tensors
    c1 = E.build_cache(mode, L, DEV, group_size=gs, calib=calib, max_seq_len=16)
    for l in range(L):
        c1.append(l, torch.from_numpy(fx[f"{mode}_prefill_k"][l]).to(DEV), torch.from_numpy(fx[f"{mode}_prefill_v"][l]).to(DEV))
        for name, got in zip(("qk", "qv", "sk", "sv"), tensors(c1, l)):
            want = fx[f"{mode}_l{l}_{name}"][:, :, :7]
            got = got.cpu().numpy()
            if name in ("sk", "sv"):
                assert np.array_equal(got.astype(np.float16).view(np.uint16), want.astype(np.float16).view(np.uint16)), (l, name)
            else:
                assert np.array_equal(got, want), (l, name)

    # 2. the loop on the GPU
    model = model.to(DEV)
    prompt = torch.from_numpy(fx["prompt"]).to(DEV)
    cache = E.build_cache(mode, L, DEV, group_size=gs, calib=calib, max_seq_len=16)
    handles = E._register_prefill_temperature_hooks(model, calib["inv_tau"])
    E.apply_int8_fused_patch(model)
    try:
        with torch.no_grad():
            logits = E._prefill_into_cache(model, cache, prompt, torch.ones_like(prompt))
            worst = float((logits.float().cpu() - torch.from_numpy(fx[f"{mode}_prefill_logits"])).abs().max())
            container = E.INT8CacheWrapperContainer(cache, L)
            toks = torch.from_numpy(fx[f"{mode}_tokens"]).to(DEV)
            for step in range(3):
                pos = torch.full((2, 1), 7 + step, dtype=torch.long, device=DEV)
                out = model(input_ids=toks[:, step:step + 1], position_ids=pos, past_key_values=container, use_cache=True)
                d = (out.logits[:, -1].float().cpu() - torch.from_numpy(fx[f"{mode}_step_logits"][step])).abs().max()
                worst = max(worst, float(d))
    finally:
        for h in handles:
            h.remove()
        E.remove_int8_fused_patch(model)
    # logits are O(1); the reference ran its projections in fp16 on the CPU, this run on the GPU
    assert worst <= (3e-2 if int8 else 1e-1), worst
    off = tot = 0
    for l in range(L):
        for name, got in zip(("qk", "qv"), tensors(cache, l)[:2]):
            want = fx[f"{mode}_l{l}_{name}"]
            got = got.cpu().numpy()
            if not int8:                                   # compare codes, not packed bytes
                got, want = O.unpack_int4(got), O.unpack_int4(want)
            diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
            assert diff.max() <= 1, (l, name, int(diff.max()))
            off += int((diff != 0).sum()); tot += diff.size
    assert off <= 0.02 * tot, (off, tot)
