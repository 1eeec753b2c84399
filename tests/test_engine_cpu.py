"""Host logic of the patched forward: HF-cache shims, RoPE helper, patch / unpatch / routing,
the torch ablation path's closed-form answers (style of the reference's tests/test_patch_model.py)."""
import math

import pytest
import torch

from llm_kvcache_quantization_b200 import engine as E


class _FakeEngine:
    num_layers = 2

    def __init__(self):
        self.appended = []
        self.seq = 5

    def get_int8_tensors(self, i):
        raise NotImplementedError

    def append(self, i, k, v):
        self.appended.append(i)

    def get_kv(self, i):
        return torch.full((1, 1, self.seq, 2), float(i)), torch.full((1, 1, self.seq, 2), float(i) + 0.5)

    def get_seq_len(self):
        return self.seq


def test_container_surface():
    eng = _FakeEngine()
    c = E.INT8CacheWrapperContainer(eng, 2)
    assert len(c) == 2 and c.get_seq_length() == 5 and c.get_max_cache_shape() is None
    assert isinstance(c[1], E.INT8CacheWrapper) and c[1].layer_idx == 1
    assert [w.layer_idx for w in c] == [0, 1]
    assert c.get_mask_sizes(torch.arange(3), 0) == (8, 0) and c.get_mask_sizes(None, 0) == (5, 0)
    k, v = c.update(torch.zeros(1), torch.zeros(1), 1)
    assert eng.appended == [1] and float(k[0, 0, 0, 0]) == 1.0
    legacy = c.to_legacy_cache()
    assert len(legacy) == 2 and float(legacy[1][1][0, 0, 0, 0]) == 1.5
    with pytest.raises(TypeError, match="fused cache engine"):
        E.INT8CacheWrapperContainer(object(), 2)


def test_rotate_half_and_rope_known_values():
    x = torch.tensor([[[[1.0, 2.0, 3.0, 4.0]]]])
    assert torch.equal(E._rotate_half(x), torch.tensor([[[[-3.0, -4.0, 1.0, 2.0]]]]))
    cos, sin = torch.zeros(1, 1, 4), torch.ones(1, 1, 4)           # 90 degree rotation
    q, k = E._apply_rope(x, 2 * x, cos, sin)
    assert torch.equal(q, E._rotate_half(x)) and torch.equal(k, 2 * E._rotate_half(x))
    q2, _ = E._apply_rope(x, x, torch.ones(1, 2), torch.zeros(1, 2))   # partial rotary, rank-2 tables
    assert torch.equal(q2, x)
    with pytest.raises(ValueError, match="RoPE dim"):
        E._apply_rope(x, x, torch.ones(1, 1, 8), torch.ones(1, 1, 8))


def test_torch_ref_known_answers():
    q = torch.zeros(1, 1, 4); q[0, 0, 0] = 1.0
    k = torch.zeros(1, 1, 2, 4, dtype=torch.int8); k[0, 0, 0, 0] = 1
    v = torch.zeros(1, 1, 2, 4, dtype=torch.int8); v[0, 0, 0, 0] = 1; v[0, 0, 1, 1] = 1
    one = torch.ones(1, 1, 2, 1, dtype=torch.float16)
    out = E._decode_attn_int8_torch_ref(q, k, v, one, one, torch.tensor([2]), 1.0)
    e = math.e
    assert abs(float(out[0, 0, 0]) - e / (e + 1)) < 1e-3 and abs(float(out[0, 0, 1]) - 1 / (e + 1)) < 1e-3
    out1 = E._decode_attn_int8_torch_ref(q, k, v, one, one, torch.tensor([1]), 1.0)
    assert torch.equal(out1[0, 0], v[0, 0, 0].float())              # single token -> V
    out0 = E._decode_attn_int8_torch_ref(q, k, v, one, one, torch.tensor([0]), 1.0)
    assert float(out0.abs().max()) == 0.0
    with pytest.raises(ValueError, match="GQA unsupported"):
        E._decode_attn_int8_torch_ref(torch.zeros(1, 3, 4), k.expand(1, 2, 2, 4), v.expand(1, 2, 2, 4),
                                      one.expand(1, 2, 2, 1), one.expand(1, 2, 2, 1), torch.tensor([1]), 1.0)


class _Attn(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.head_dim = 4
        self.q_proj = torch.nn.Linear(8, 8, bias=False)
        self.k_proj = torch.nn.Linear(8, 4, bias=False)

    def forward(self, hidden_states, attention_mask=None, past_key_values=None):
        return "original", past_key_values


class _Model:
    def __init__(self):
        layer = type("L", (), {})()
        layer.self_attn = _Attn()
        self.model = type("M", (), {})()
        self.model.layers = [layer]
        self.config = type("C", (), {"num_attention_heads": 2, "num_key_value_heads": 1})()


def test_patch_unpatch_and_routing(monkeypatch):
    m = _Model()
    attn = m.model.layers[0].self_attn
    original = _Attn.forward
    E.apply_int8_fused_patch(m)
    assert _Attn.forward is not original and _Attn._original_forward is original
    assert attn.layer_idx == 0 and attn._kv_num_attention_heads == 2 and attn._kv_num_key_value_heads == 1
    E.apply_int8_fused_patch(m)                                   # idempotent
    assert _Attn._original_forward is original
    # q_len > 1 or no wrapper -> original forward, extra kwargs filtered to its signature
    assert attn(torch.zeros(1, 3, 8), position_ids=None, use_cache=True)[0] == "original"
    cont = E.INT8CacheWrapperContainer(_FakeEngine(), 1)
    res = attn(torch.zeros(1, 3, 8), past_key_values=cont)
    assert res[0] == "original" and res[1] is cont
    called = {}

    def fake_fused(self, hidden_states, cache_wrapper, **kw):
        called["wrapper"] = cache_wrapper
        return "fused", None
    monkeypatch.setattr(E, "_fused_forward_impl", fake_fused)
    assert attn(torch.zeros(1, 1, 8), past_key_values=cont)[0] == "fused"
    assert isinstance(called["wrapper"], E.INT8CacheWrapper) and called["wrapper"].layer_idx == 0
    assert E.remove_int8_fused_patch(m) is True
    assert _Attn.forward is original and not hasattr(_Attn, "_original_forward")
    assert E.remove_int8_fused_patch(m) is False
    with pytest.raises(ValueError, match="Cannot detect model layers"):
        E.apply_int8_fused_patch(object())


def test_shape_meta_and_inv_tau_validation():
    a = _Attn()
    assert E._resolve_attn_shape_meta(a) == (2, 1, 4)
    a._kv_num_attention_heads, a._kv_num_key_value_heads = 3, 2
    with pytest.raises(ValueError, match="Invalid GQA"):
        E._resolve_attn_shape_meta(a)
    eng = type("Eng", (), {"inv_tau": torch.ones(2, 4), "use_attn_temperature": True})()
    assert E._layer_inv_tau(eng, 1, 4, "cpu").shape == (4,)
    with pytest.raises(ValueError, match="layers"):
        E._layer_inv_tau(eng, 2, 4, "cpu")
    with pytest.raises(ValueError, match="q_heads"):
        E._layer_inv_tau(eng, 0, 8, "cpu")
    eng.use_attn_temperature = False
    assert E._layer_inv_tau(eng, 0, 4, "cpu") is None


def test_build_cache_modes(tmp_path):
    import json
    assert type(E.build_cache("fp16", 2, "cpu")).__name__ == "FP16KVCache"
    assert type(E.build_cache("int8_baseline", 2, "cpu", group_size=32)).__name__ == "INT8KVCache"
    kivi = E.build_cache("kivi_style", 2, "cpu", quant_bits=4)
    assert type(kivi).__name__ == "KIVIStyleKVCache" and kivi.bit_packed and kivi.decode_attn_impl == "torch_ref"
    with pytest.raises(ValueError, match="not supported"):
        E.build_cache("int4_mixed_kv", 2, "cpu")
    f = tmp_path / "calib.json"
    f.write_text(json.dumps({"version": 2, "group_size_k": 32, "group_size_v": 32, "clip_percentile_k": 99.5,
                             "k_scale": [[[0.1] * 4]], "v_scale": [[[0.2] * 4]], "inv_tau": [[1.0, 1.1]],
                             "int4_outlier_ratio": 0.01}))
    cal = E.load_calibration(str(f), "int4_ours_mixed", "cpu")
    assert cal["static_k_scale"].dtype == torch.float32 and cal["mixed_rescue"] is True and cal["group_size"] == 32
    c = E.build_cache("int4_ours_mixed", 1, "cpu", calib=cal)
    assert c.mixed_rescue and c.group_size == 32 and abs(c.outlier_rescue_ratio - 0.01) < 1e-9 and c.inv_tau is not None
    cal8 = E.load_calibration(str(f), "int8_ours", "cpu")
    assert cal8["static_k_scale"].dtype == torch.float16


def test_save_calibration_writes_the_schema_load_calibration_reads(tmp_path):
    """calibration.save_calibration -> engine.load_calibration on CPU tensors (no kernel involved)."""
    import json
    import torch
    from llm_kvcache_quantization_b200 import calibration as C, engine as E
    ks = [torch.full((2, 4), 0.01 * (l + 1)) for l in range(3)]
    path = str(tmp_path / "c.json")
    doc = C.save_calibration(path, ks, ks, group_size=32, clip_percentile=99.5, inv_tau=torch.ones(3, 12),
                             int4_outlier_ratio=0.02, int4_mixed_rescue=True)
    assert json.load(open(path)) == doc and doc["version"] == 2
    out = E.load_calibration(path, "int4_ours", "cpu")
    assert out["group_size"] == 32 and out["clip_percentile"] == 99.5 and out["mixed_rescue"] is True
    assert out["outlier_rescue_ratio"] == 0.02 and out["static_k_scale"].dtype == torch.float32
    assert tuple(out["static_k_scale"].shape) == (3, 2, 4) and tuple(out["inv_tau"].shape) == (3, 12)
    with __import__("pytest").raises(ValueError):
        C.compute_absmax_per_group(torch.zeros(2, 5, 128), 48)


# --------------------------------------------------------------------------- prefill temperature hooks, decode-loop arguments
class _TinyAttn(torch.nn.Module):
    def __init__(self, heads, head_dim, with_norm):
        super().__init__()
        self.num_heads, self.head_dim = heads, head_dim
        self.q_proj = torch.nn.Linear(heads * head_dim, heads * head_dim, bias=False)
        if with_norm:
            self.q_norm = torch.nn.Identity()


class _TinyModel(torch.nn.Module):
    def __init__(self, layers, heads, head_dim, with_norm=False):
        super().__init__()
        self.model = torch.nn.Module()
        self.model.layers = torch.nn.ModuleList()
        for _ in range(layers):
            layer = torch.nn.Module()
            layer.self_attn = _TinyAttn(heads, head_dim, with_norm)
            self.model.layers.append(layer)


def test_prefill_temperature_hooks_scale_queries_of_prompts_only():
    """src/engine/generate_loop.py:276-390: per-head scale on q_proj's output when more than one position is
    processed; a single position (decode) passes through; the handles remove the hooks."""
    torch.manual_seed(0)
    heads, hd = 2, 4
    m = _TinyModel(2, heads, hd)
    inv_tau = torch.tensor([[0.5, 2.0], [1.5, 0.25]])
    x_prompt, x_step = torch.randn(3, 5, heads * hd), torch.randn(3, 1, heads * hd)
    plain = [l.self_attn.q_proj(x_prompt) for l in m.model.layers]
    plain_step = m.model.layers[0].self_attn.q_proj(x_step)
    handles = E._register_prefill_temperature_hooks(m, inv_tau)
    assert len(handles) == 2
    for l, layer in enumerate(m.model.layers):
        got = layer.self_attn.q_proj(x_prompt).view(3, 5, heads, hd)
        assert torch.allclose(got, plain[l].view(3, 5, heads, hd) * inv_tau[l].view(1, 1, -1, 1))
    assert torch.equal(m.model.layers[0].self_attn.q_proj(x_step), plain_step)
    for h in handles:
        h.remove()
    assert torch.equal(m.model.layers[1].self_attn.q_proj(x_prompt), plain[1])
    # with a q_norm module the scale goes on ITS output, in either layout
    n = _TinyModel(1, heads, hd, with_norm=True)
    handles = E._register_prefill_temperature_hooks(n, inv_tau[:1])
    qn = n.model.layers[0].self_attn.q_norm
    bhsd, bshd = torch.randn(2, heads, 6, hd), torch.randn(2, 6, heads, hd)
    assert torch.allclose(qn(bhsd), bhsd * inv_tau[0].view(1, -1, 1, 1))
    assert torch.allclose(qn(bshd), bshd * inv_tau[0].view(1, 1, -1, 1))
    one = torch.randn(2, heads, 1, hd)
    assert torch.equal(qn(one), one)
    # shape errors of the calibration tensor
    with pytest.raises(ValueError, match="2D tensor"):
        E._register_prefill_temperature_hooks(m, torch.ones(2))
    with pytest.raises(ValueError, match="head count mismatch"):
        E._register_prefill_temperature_hooks(m, torch.ones(2, 3))
    with pytest.raises(ValueError, match="layers but model"):
        E._register_prefill_temperature_hooks(m, torch.ones(1, 2))
    with pytest.warns(UserWarning, match="model.model.layers not found"):
        assert E._register_prefill_temperature_hooks(torch.nn.Linear(2, 2), inv_tau) == []


def test_generate_from_ids_refuses_what_it_does_not_build():
    ids = torch.zeros(1, 3, dtype=torch.long)
    for kw in (dict(k_bits=4), dict(v_bits=8), dict(policy_json="p.json")):
        with pytest.raises(ValueError, match="mixed-bit"):
            E.generate_from_ids(None, None, ids, kv_mode="int8_ours", **kw)
    with pytest.raises(ValueError, match="not supported"):
        E.generate_from_ids(None, None, ids, kv_mode="int4_mixed_kv")
    import inspect
    names = list(inspect.signature(E.generate_from_ids).parameters)
    # the reference's parameter list, in its order (src/engine/generate_loop.py:393-418)
    assert names == ["model", "tokenizer", "input_ids", "attention_mask", "max_new_tokens", "kv_mode", "group_size",
                     "clip_percentile", "seed", "calib_file", "use_attn_temperature", "use_static_scales",
                     "adaptive_static_scales", "adaptive_static_margin", "adaptive_static_k", "adaptive_static_v",
                     "decode_attn_impl", "allow_missing_calib", "stop_on_eos", "quant_bits", "k_bits", "v_bits",
                     "residual_length", "policy_json"]
    fields = {f for f in E.GenerationBatchOutput.__dataclass_fields__}
    assert {"generated_ids", "ttft_ms", "tpot_ms", "tok_per_s", "tok_per_s_per_seq", "gpu_mem_peak_mb", "prompt_len",
            "gen_len", "batch", "kv_cache_mem_mb", "kv_cache_seq_len"} <= fields


def test_fused_decode_dump_writes_tensors_and_summary(tmp_path, monkeypatch):
    """KV_FUSED_DUMP_DIR / _LAYER / _STEP (src/engine/patch_model.py:380-496): one dump per (directory, layer, step)."""
    import json
    import os

    class Eng:
        def __init__(self):
            g = torch.Generator().manual_seed(1)
            self.k = torch.randint(-127, 128, (1, 1, 6, 8), generator=g, dtype=torch.int8)
            self.v = torch.randint(-127, 128, (1, 1, 6, 8), generator=g, dtype=torch.int8)
            self.s = torch.full((1, 1, 6, 1), 0.01)

        def get_int8_tensors(self, i):
            return self.k, self.v, self.s, self.s

        def get_seq_len(self):
            return 6
    E._reset_fused_state()
    eng, q = Eng(), torch.randn(1, 2, 8).half()
    ctx = torch.full((1,), 6, dtype=torch.int32)
    fused = E._decode_attn_int8_torch_ref(q, eng.k, eng.v, eng.s.half(), eng.s.half(), ctx, 0.3)
    monkeypatch.setenv("KV_FUSED_DUMP_DIR", str(tmp_path))
    monkeypatch.setenv("KV_FUSED_DUMP_LAYER", "1")
    E._maybe_dump_fused_decode(eng, 0, "triton_fused", q, None, 0.3, fused)          # filtered out: layer 0
    assert os.listdir(tmp_path) == []
    E._maybe_dump_fused_decode(eng, 1, "triton_fused", q, None, 0.3, fused)
    E._maybe_dump_fused_decode(eng, 1, "triton_fused", q, None, 0.3, fused)          # second call: already written
    files = sorted(os.listdir(tmp_path))
    assert len(files) == 2 and files[0].startswith("fused_layer01_step00006_pid") and files[0].endswith(".json")
    summary = json.load(open(os.path.join(tmp_path, files[0])))
    assert summary["max_abs_diff"] == 0.0 and summary["context_len"] == 6 and len(summary["logits_topk_ref"]) == 5
    blob = torch.load(os.path.join(tmp_path, files[1]))
    assert set(blob) >= {"q", "k_int8", "v_int8", "k_scale", "v_scale", "fused_out", "ref_out", "sm_scale"}
    monkeypatch.setenv("KV_FUSED_DUMP_STEP", "7")
    E._reset_fused_state()
    E._maybe_dump_fused_decode(eng, 1, "triton_fused", q, None, 0.3, fused)          # filtered out: step 6
    assert len(os.listdir(tmp_path)) == 2


def test_role_aware_calibration_schemas(tmp_path):
    """The calibration reader of the KIVI-format modes (src/engine/generate_loop.py:951-1043): `role_aware` section,
    the k_calibration / v_calibration fallback with its warning, inv_tau only where the mode uses it, a missing file
    raises."""
    import json
    import warnings as W
    from llm_kvcache_quantization_b200 import engine as E
    f1 = tmp_path / "ra.json"
    f1.write_text(json.dumps({"role_aware": {"k_percentile": 99.5, "v_percentile": 99.9, "inv_tau": [[1.0, 1.1]]}, "inv_tau": [[2.0, 2.0]]}))
    a = E.load_role_aware_calibration(str(f1), "int4_ours_asym", "cpu")
    assert (a["k_percentile"], a["v_percentile"], a["inv_tau"]) == (99.5, 99.9, None)
    b = E.load_role_aware_calibration(str(f1), "int4_ours_asym_ba", "cpu")
    assert b["inv_tau"].dtype == torch.float32 and b["inv_tau"].tolist() == [[1.0, pytest.approx(1.1)]]
    f2 = tmp_path / "v3.json"
    f2.write_text(json.dumps({"k_calibration": {"k_percentile": 99.0, "inv_tau": [[0.9, 0.8]]}, "v_calibration": {"v_percentile": 98.0}}))
    with pytest.warns(UserWarning, match="k_calibration fallback schema"):
        c = E.load_role_aware_calibration(str(f2), "int4_ours_asym_ba", "cpu")
    assert (c["k_percentile"], c["v_percentile"]) == (99.0, 98.0) and c["inv_tau"].shape == (1, 2)
    with W.catch_warnings():
        W.simplefilter("error")
        d = E.load_role_aware_calibration(str(f2), "int4_kivi_aligned", "cpu")
    assert (d["k_percentile"], d["v_percentile"]) == (100.0, 98.0) and d["inv_tau"].shape == (1, 2)
    assert E.load_role_aware_calibration(None, "int4_ours_asym", "cpu") == {"k_percentile": 100.0, "v_percentile": 100.0, "inv_tau": None}
    with pytest.raises(FileNotFoundError):
        E.load_role_aware_calibration(str(tmp_path / "missing.json"), "int4_ours_asym", "cpu")
    assert {"int4_kivi_aligned", "int4_ours_asym", "int4_ours_asym_ba"} <= E.FUSED_KV_MODES


def test_load_calibration_reads_the_schema_of_the_shipped_file(golden_dir):
    """tests/golden/calib_schema.json keeps every key of the reference's artifacts/kv_calib_mse_1p5b_int8.json (tables
    cut to two layers).  The loader takes group size and percentile from the *_k keys, gives fp16 static scales to
    INT8 modes and fp32 to INT4 modes, warns about version < 2 as the reference does
    (src/engine/generate_loop.py:764-856)."""
    import json
    import os
    from llm_kvcache_quantization_b200 import engine as E
    path = os.path.join(golden_dir, "calib_schema.json")
    raw = json.load(open(path))
    assert raw["shapes_in_shipped_file"] == {"k_scale": [28, 2, 8], "v_scale": [28, 2, 8], "inv_tau": [28, 12]}
    with pytest.warns(UserWarning, match="version=1"):
        c = E.load_calibration(path, "int8_ours", "cpu")
    assert c["group_size"] == 16 and c["clip_percentile"] == 99.5
    assert c["static_k_scale"].dtype == torch.float16 and tuple(c["static_k_scale"].shape) == (2, 2, 8)
    assert tuple(c["static_v_scale"].shape) == (2, 2, 8) and tuple(c["inv_tau"].shape) == (2, 12)
    assert c["inv_tau"].dtype == torch.float32
    assert torch.equal(c["static_k_scale"], torch.tensor(raw["k_scale"], dtype=torch.float16))
    assert torch.equal(c["inv_tau"], torch.tensor(raw["inv_tau"], dtype=torch.float32))
    assert c["outlier_rescue_ratio"] == 0.0 and c["mixed_rescue"] is False
    with pytest.warns(UserWarning):
        c4 = E.load_calibration(path, "int4_ours", "cpu", use_attn_temperature=False)
    assert c4["static_k_scale"].dtype == torch.float32 and c4["inv_tau"] is None
    with pytest.warns(UserWarning):
        c0 = E.load_calibration(path, "int8_ours", "cpu", use_static_scales=False)
    assert c0["static_k_scale"] is None and c0["static_v_scale"] is None
