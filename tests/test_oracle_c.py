"""Cross-checks the C restatement of the oracle against the numpy oracle (which is
pinned to the reference's fixtures) and against the attention fixtures directly."""
import os

import numpy as np
import pytest

from oracle import c_oracle as CO
from oracle import kvq_oracle as O


@pytest.fixture(scope="module")
def att(golden_dir):
    return np.load(os.path.join(golden_dir, "attention.npz"))


@pytest.fixture(scope="module")
def qz(golden_dir):
    return np.load(os.path.join(golden_dir, "quantizers.npz"))


@pytest.mark.parametrize("name", ("c1_small", "gqa7_ragged", "zero_ctx", "int4_g32", "int4_g16", "mha_g128"))
def test_c_attention_vs_reference_fixture(att, name):
    b, hq, hkv, s, gs, is4 = att[f"{name}_meta"]
    out = CO.decode_attn(2 if is4 else 1, att[f"{name}_q"], att[f"{name}_k"], att[f"{name}_v"], att[f"{name}_ks"],
                         att[f"{name}_vs"], att[f"{name}_ctx"], 1 / np.sqrt(128.0), inv_tau=att[f"{name}_inv_tau"])
    ref = att[f"{name}_out"].astype(np.float32)
    err = np.abs(out.astype(np.float32) - ref)
    assert np.all(err <= 1e-3 + 2e-3 * np.abs(ref)), float(err.max())


@pytest.mark.parametrize("gs", (16, 32, 64, 128))
def test_c_quantizers_bit_exact(qz, gs):
    for t in ("k", "v"):
        x = qz[f"g{gs}_{t}"]
        c, s = CO.quant_int8_static(x, qz[f"g{gs}_int8_static_{t}s_in"], gs)
        assert np.array_equal(c, qz[f"g{gs}_int8_static_q{t}"])
        assert np.array_equal(s.astype(np.float32), qz[f"g{gs}_int8_static_s{t}"])
        p, s = CO.quant_int4_static(x, qz[f"g{gs}_int4_static_{t}s_in"], gs)
        assert np.array_equal(p, qz[f"g{gs}_int4_static_q{t}"])
        assert np.array_equal(s, qz[f"g{gs}_int4_static_s{t}"].astype(np.float16))
        p, s, z = CO.quant_int4_asym(x, gs)
        assert np.array_equal(p, qz[f"g{gs}_asym_q{t}"])
        assert np.array_equal(s, qz[f"g{gs}_asym_s{t}"].astype(np.float16))
        assert np.array_equal(z, qz[f"g{gs}_asym_z{t}"].astype(np.float16))


def test_c_asym_outlier_fp16_vs_numpy():
    rng = np.random.default_rng(5)
    b, hq, hkv, s, d = 2, 12, 2, 700, 128
    q = rng.standard_normal((b, hq, d)).astype(np.float16)
    k = (rng.standard_normal((b, hkv, s, d)) * 2).astype(np.float16)
    v = rng.standard_normal((b, hkv, s, d)).astype(np.float16)
    ctx = [s, 123]
    ck, sk, zk = O.quantize_asym_group(k, 32)
    cv, sv, zv = O.quantize_asym_group(v, 32)
    a = CO.decode_attn(2, q, O.pack_int4(ck), O.pack_int4(cv), sk.astype(np.float16), sv.astype(np.float16), ctx,
                       0.088, kz=zk.astype(np.float16), vz=zv.astype(np.float16))
    r = O.decode_attn_int4_asym(q, O.pack_int4(ck), O.pack_int4(cv), sk, zk, sv, zv, ctx, 0.088)
    assert np.allclose(a.astype(np.float32), r.astype(np.float32), atol=1e-3, rtol=2e-3)
    idx = np.array([[3, 40, 99], [0, 64, 127]], np.int16)
    body, side_k = O.split_outliers(k, idx)
    bodyv, side_v = O.split_outliers(v, idx)
    tab = np.abs(body.astype(np.float32)).reshape(b, hkv, s, 4, 32).max(axis=(0, 2, 4)) / 7
    ck, sk = O.quantize_int4_static(body, tab, 32)
    cv, sv = O.quantize_int4_static(bodyv, tab, 32)
    a = CO.decode_attn(2, q, O.pack_int4(ck), O.pack_int4(cv), sk.astype(np.float16), sv.astype(np.float16), ctx,
                       0.088, kside=side_k, vside=side_v, outlier_idx=idx)
    r = O.decode_attn_int4_outlier(q, O.pack_int4(ck), O.pack_int4(cv), sk, sv, side_k, side_v, idx, ctx, 0.088)
    assert np.allclose(a.astype(np.float32), r.astype(np.float32), atol=1e-3, rtol=2e-3)
    a = CO.decode_attn(0, q, k, v, None, None, ctx, 0.088)
    r = O.decode_attn_fp16(q, k, v, ctx, 0.088)
    assert np.allclose(a.astype(np.float32), r.astype(np.float32), atol=1e-3, rtol=2e-3)
    assert CO.num_threads() >= 1
