"""Pins the numpy oracle against fixtures produced by running the reference
(`tests/golden/make_golden.py`).  Integer outputs must be bit-exact."""
import os

import numpy as np
import pytest

from oracle import kvq_oracle as O

GS = (16, 32, 64, 128)


@pytest.fixture(scope="module")
def qz(golden_dir):
    return np.load(os.path.join(golden_dir, "quantizers.npz"))


@pytest.fixture(scope="module")
def att(golden_dir):
    return np.load(os.path.join(golden_dir, "attention.npz"))


@pytest.mark.parametrize("gs", GS)
def test_int8_static(qz, gs):
    for t in ("k", "v"):
        codes, s16 = O.quantize_int8_static(qz[f"g{gs}_{t}"], qz[f"g{gs}_int8_static_{t}s_in"], gs)
        assert np.array_equal(codes, qz[f"g{gs}_int8_static_q{t}"])
        ref = qz[f"g{gs}_int8_static_s{t}"]
        assert np.array_equal(s16.astype(np.float32), ref)  # reference keeps an fp32 copy of the fp16 scale


@pytest.mark.parametrize("gs", GS)
def test_int8_adaptive(qz, gs):
    for t in ("k", "v"):
        codes, s16 = O.quantize_int8_static(qz[f"g{gs}_{t}"], qz[f"g{gs}_int8_static_{t}s_in"], gs,
                                            adaptive_margin=0.9)
        assert np.array_equal(codes, qz[f"g{gs}_int8_adapt_q{t}"])
        assert np.array_equal(s16.astype(np.float32), qz[f"g{gs}_int8_adapt_s{t}"])


@pytest.mark.parametrize("gs", GS)
@pytest.mark.parametrize("p", (99.9, 100.0, 95.0))
def test_int8_dynamic(qz, gs, p):
    for t in ("k", "v"):
        codes, s16 = O.quantize_int8_dynamic(qz[f"g{gs}_{t}"], p, gs)
        assert np.array_equal(s16.astype(np.float32), qz[f"g{gs}_int8_dyn{p}_s{t}"])
        assert np.array_equal(codes, qz[f"g{gs}_int8_dyn{p}_q{t}"])


@pytest.mark.parametrize("gs", GS)
@pytest.mark.parametrize("name,kw", [
    ("static", {}), ("mixed", dict(mixed_rescue=True)), ("rescue", dict(outlier_rescue_ratio=0.05)),
    ("rescue1", dict(outlier_rescue_ratio=1.0)), ("adapt", dict(adaptive_margin=1.1))])
def test_int4_static_variants(qz, gs, name, kw):
    for t in ("k", "v"):
        codes, s32 = O.quantize_int4_static(qz[f"g{gs}_{t}"], qz[f"g{gs}_int4_static_{t}s_in"], gs, **kw)
        assert np.array_equal(s32, qz[f"g{gs}_int4_{name}_s{t}"])
        assert np.array_equal(O.pack_int4(codes), qz[f"g{gs}_int4_{name}_q{t}"])


@pytest.mark.parametrize("gs", GS)
@pytest.mark.parametrize("p", (99.9, 100.0))
def test_int4_dynamic(qz, gs, p):
    for t in ("k", "v"):
        codes, s32 = O.quantize_int4_dynamic(qz[f"g{gs}_{t}"], p, gs)
        assert np.array_equal(s32, qz[f"g{gs}_int4_dyn{p}_s{t}"])
        assert np.array_equal(O.pack_int4(codes), qz[f"g{gs}_int4_dyn{p}_q{t}"])


@pytest.mark.parametrize("gs", GS)
def test_asym_group(qz, gs):
    for t in ("k", "v"):
        codes, sc, zp = O.quantize_asym_group(qz[f"g{gs}_{t}"], gs)
        assert np.array_equal(sc, qz[f"g{gs}_asym_s{t}"])
        assert np.array_equal(zp, qz[f"g{gs}_asym_z{t}"])
        assert np.array_equal(O.pack_int4(codes), qz[f"g{gs}_asym_q{t}"])
        deq = O.dequant_asym_fp16(codes, sc, zp)
        assert np.array_equal(deq.view(np.uint16), qz[f"g{gs}_asym_deq{t}"].view(np.uint16))


def test_pack_unpack_full_range(golden_dir):
    z = np.load(os.path.join(golden_dir, "pack_int4.npz"))
    assert np.array_equal(O.pack_int4(z["codes"]), z["packed"])
    assert np.array_equal(O.unpack_int4(z["packed"]), z["unpacked"])
    assert np.array_equal(O.unpack_int4(O.pack_int4(z["codes"])), z["codes"])


ATT_CASES = ("c1_small", "gqa7_ragged", "zero_ctx", "int4_g32", "int4_g16", "mha_g128")


@pytest.mark.parametrize("name", ATT_CASES)
def test_attention_reference(att, name):
    b, hq, hkv, s, gs, is4 = att[f"{name}_meta"]
    fn = O.decode_attn_int4 if is4 else O.decode_attn_int8
    out = fn(att[f"{name}_q"], att[f"{name}_k"], att[f"{name}_v"], att[f"{name}_ks"], att[f"{name}_vs"],
             att[f"{name}_ctx"], 1.0 / np.sqrt(128.0), inv_tau=att[f"{name}_inv_tau"])
    ref = att[f"{name}_out"].astype(np.float32)
    # same arithmetic, different fp32 summation order: one fp16 ulp of slack
    err = np.abs(out.astype(np.float32) - ref)
    assert np.all(err <= 1e-3 + 2e-3 * np.abs(ref)), float(err.max())
    assert not np.isnan(out).any()


# closed-form known answers, as in the reference's tests/test_patch_model.py:280-333
def test_single_token_returns_v():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 4, 128)).astype(np.float16)
    k = rng.integers(-127, 128, (1, 2, 1, 128)).astype(np.int8)
    v = rng.integers(-127, 128, (1, 2, 1, 128)).astype(np.int8)
    ks = np.full((1, 2, 1, 4), 0.01, np.float16)
    vs = np.full((1, 2, 1, 4), 0.02, np.float16)
    out = O.decode_attn_int8(q, k, v, ks, vs, np.array([1]), 0.1)
    vh = O.dequant_sym_fp16(v, vs)
    assert np.array_equal(out[0, 0], vh[0, 0, 0]) and np.array_equal(out[0, 3], vh[0, 1, 0])


def test_two_token_softmax_known_answer():
    q = np.zeros((1, 1, 128), np.float16); q[0, 0, 0] = 1.0
    k = np.zeros((1, 1, 2, 128), np.int8); k[0, 0, 0, 0] = 1
    v = np.zeros((1, 1, 2, 128), np.int8); v[0, 0, 0, 0] = 1; v[0, 0, 1, 1] = 1
    one = np.ones((1, 1, 2, 1), np.float16)
    out = O.decode_attn_int8(q, k, v, one, one, np.array([2]), 1.0).astype(np.float32)
    e = np.e
    assert abs(out[0, 0, 0] - e / (e + 1)) < 1e-3 and abs(out[0, 0, 1] - 1 / (e + 1)) < 1e-3


def test_lse_merge_matches_full():
    rng = np.random.default_rng(1)
    b, hq, hkv, s, d = 2, 6, 2, 96, 128
    q = rng.standard_normal((b, hq, d)).astype(np.float16)
    k = rng.standard_normal((b, hkv, s, d)).astype(np.float16)
    v = rng.standard_normal((b, hkv, s, d)).astype(np.float16)
    full = O.decode_attn_dequantized(q, k, v, [s, 50], 0.088)
    parts = []
    for lo, hi in ((0, 32), (32, 64), (64, 96)):
        ctx = [max(0, min(c, hi) - lo) for c in (s, 50)]
        o, m, l = O.decode_attn_dequantized(q, k[:, :, lo:hi], v[:, :, lo:hi], ctx, 0.088, return_lse=True)
        parts.append((o.astype(np.float32), m, l))
    merged = O.lse_merge([p[0] for p in parts], [p[1] for p in parts], [p[2] for p in parts])
    assert np.allclose(merged.astype(np.float32), full.astype(np.float32), atol=2e-3, rtol=1e-2)


ROPE_CASES = ("full_r3", "partial_r3", "shared_r2", "decode_r4", "d64_r3")


@pytest.mark.parametrize("name", ROPE_CASES)
def test_rope_matches_reference(golden_dir, name):
    """Rotate-half RoPE restated in numpy fp16 == the reference's _apply_rope, bit for bit."""
    z = np.load(os.path.join(golden_dir, "rope.npz"))
    for which in ("q", "k"):
        got = O.apply_rope(z[f"{name}_{which}"], z[f"{name}_cos"], z[f"{name}_sin"])
        ref = z[f"{name}_{which}_out"]
        assert got.dtype == np.float16 and got.shape == ref.shape
        assert np.array_equal(got.view(np.uint16), ref.view(np.uint16)), f"{name} {which}"


@pytest.mark.parametrize("bits", (4, 8))
def test_kivi_format_matches_reference(golden_dir, bits):
    """Per-channel K (parameters from the prompt, later tokens clipped) and per-token V asymmetric
    quantization restated in numpy == the reference's KIVIStyleKVCache on CPU: payloads, fp32
    parameters and dequantised values, bit for bit."""
    z = np.load(os.path.join(golden_dir, "kivi.npz"))
    k, v, P = z["k"], z["v"], int(z["prompt"])
    ck, sk, zk = O.quantize_asym_axis(k[:, :, :P], 2, bits)
    codes_k = np.concatenate([ck, O.quantize_asym_with_params(k[:, :, P:], sk, zk, 2, bits)], axis=2)
    cv, sv, zv = O.quantize_asym_axis(v, 3, bits)
    pk, pv = (O.pack_int4(codes_k), O.pack_int4(cv)) if bits == 4 else (codes_k, cv)
    assert np.array_equal(pk, z[f"b{bits}_k_payload"]) and np.array_equal(pv, z[f"b{bits}_v_payload"])
    for got, name in ((sk, "k_scale"), (zk, "k_zp"), (sv, "v_scale"), (zv, "v_zp")):
        assert got.dtype == np.float32 and np.array_equal(got, z[f"b{bits}_{name}"]), name
    assert np.array_equal(O.dequant_asym_f32(codes_k, sk, zk, 2).view(np.uint16), z[f"b{bits}_k_deq"].view(np.uint16))
    assert np.array_equal(O.dequant_asym_f32(cv, sv, zv, 3).view(np.uint16), z[f"b{bits}_v_deq"].view(np.uint16))


@pytest.mark.parametrize("case", (0, 1, 2))
def test_kivi_format_with_clipping_percentiles_matches_reference(golden_dir, case):
    """Clipping percentiles below 100 (two-sided torch.quantile bounds: over the prompt's tokens for K, over the head
    dimension of each token for V) restated in numpy == the reference's KIVIStyleKVCache / RoleAwareAsymKVCache on
    CPU, bit for bit."""
    z = np.load(os.path.join(golden_dir, "kivi_pct.npz"))
    bits, kp, vp = int(z["cases"][case][0]), float(z["cases"][case][1]), float(z["cases"][case][2])
    k, v, P = z["k"], z["v"], int(z["prompt"])
    ck, sk, zk = O.quantize_asym_axis(k[:, :, :P], 2, bits, percentile=kp)
    codes_k = np.concatenate([ck, O.quantize_asym_with_params(k[:, :, P:], sk, zk, 2, bits)], axis=2)
    cv, sv, zv = O.quantize_asym_axis(v, 3, bits, percentile=vp)
    pk, pv = (O.pack_int4(codes_k), O.pack_int4(cv)) if bits == 4 else (codes_k, cv)
    for got, name in ((sk, "k_scale"), (zk, "k_zp"), (sv, "v_scale"), (zv, "v_zp")):
        assert got.dtype == np.float32 and np.array_equal(got, z[f"c{case}_{name}"]), name
    assert np.array_equal(pk, z[f"c{case}_k_payload"]) and np.array_equal(pv, z[f"c{case}_v_payload"])
    assert np.array_equal(O.dequant_asym_f32(codes_k, sk, zk, 2).view(np.uint16), z[f"c{case}_k_deq"].view(np.uint16))
    assert np.array_equal(O.dequant_asym_f32(cv, sv, zv, 3).view(np.uint16), z[f"c{case}_v_deq"].view(np.uint16))
    assert int((np.abs(codes_k.astype(np.int32)) >= (7 if bits == 4 else 127)).sum()) > 0      # clipping happened
