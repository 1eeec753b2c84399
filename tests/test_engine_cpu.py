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
