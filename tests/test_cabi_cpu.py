"""CPU-side checks: the C-ABI library loads, exports every declared symbol, and the
host wrappers reject bad input before any launch."""
import ctypes
import os
import re

import pytest
import torch

import llm_kvcache_quantization_b200 as kvq
from llm_kvcache_quantization_b200 import _lib, build, quant

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_header_symbols_all_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "kvq.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(kvq_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    bound = {name for name, _, _ in _lib.EXPORTS}
    assert declared == bound, declared ^ bound
    for name in declared:
        assert hasattr(lib, name)


def test_abi_version_and_strerror(lib):
    assert lib.kvq_abi_version() == 5 == _lib.ABI_VERSION
    assert lib.kvq_strerror(0) == b"ok"
    assert b"invalid" in lib.kvq_strerror(-1)


def test_workspace_bytes(lib):
    n = lib.kvq_decode_workspace_bytes(2, 12, 128, 8)
    assert n >= 2 * 12 * 8 * (128 + 2) * 4 and n % 256 == 0
    assert lib.kvq_decode_workspace_bytes(0, 12, 128, 8) == 0


def test_null_args_are_rejected_without_launch(lib):
    assert lib.kvq_decode_attn(None, None) == _lib.KVQ_EINVAL
    assert lib.kvq_quantize_append(None, None) == _lib.KVQ_EINVAL
    assert lib.kvq_lse_combine(None, None) == _lib.KVQ_EINVAL
    a = _lib.KvqAttnArgs()
    a.B, a.Hq, a.Hkv, a.D = 1, 12, 5, 128      # Hq not a multiple of Hkv
    assert lib.kvq_decode_attn(ctypes.byref(a), None) == _lib.KVQ_EINVAL


def test_struct_sizes_match_header(lib):
    # all fields are 4- or 8-byte scalars/pointers: natural alignment, no packing pragma
    assert ctypes.sizeof(_lib.KvqCacheSide) == 13 * 8
    assert ctypes.sizeof(_lib.KvqCombineArgs) == 4 * 4 + 10 * 8
    assert ctypes.sizeof(_lib.KvqDequantArgs) == 8 * 4 + 8 + 2 * 13 * 8 + 5 * 8
    assert ctypes.sizeof(_lib.KvqKiviArgs) == 6 * 4 + 30 * 8
    assert ctypes.sizeof(_lib.KvqQuantileArgs) == 8 + 8 + 3 * 4 + 4 + 2 * 8
    assert ctypes.sizeof(_lib.KvqAbsmaxArgs) == 5 * 4 + 4 + 8 + 3 * 8 + 8
    assert ctypes.sizeof(_lib.KvqExchangeArgs) == 4 * 4 + 2 * 8 + 2 * 4 + 8 + 2 * 4 + 7 * 8


def test_binding_structs_match_the_compiled_header(lib):
    for i, st in enumerate(_lib.STRUCTS):
        assert lib.kvq_struct_size(i) == ctypes.sizeof(st), st.__name__
    assert lib.kvq_struct_size(len(_lib.STRUCTS)) == 0


def test_append_beyond_max_slots_is_refused_on_the_host(lib):
    a = _lib.KvqAppendArgs()
    a.format, a.policy = _lib.FMT_INT8, _lib.SCALE_DYNAMIC_PCT
    a.B, a.Hkv, a.T, a.D, a.group_size = 1, 2, 4, 128, 32
    a.write_pos, a.max_slots = 30, 32             # slots 30..33 of a 32-slot cache
    assert lib.kvq_quantize_append(ctypes.byref(a), None) == _lib.KVQ_ELIMIT
    a.max_slots = -1
    assert lib.kvq_quantize_append(ctypes.byref(a), None) == _lib.KVQ_EINVAL
    k = _lib.KvqKiviArgs()
    k.bits, k.B, k.H, k.T, k.D = 4, 1, 2, 4, 128
    k.k_src = k.v_src = 16
    k.write_pos, k.max_slots = 30, 32
    assert lib.kvq_kivi_append(ctypes.byref(k), None) in (_lib.KVQ_ELIMIT, _lib.KVQ_EINVAL)


def test_exchange_buffer_layout(lib):
    total = lib.kvq_exchange_bytes(1, 40, 128, 48, 8)
    rows = 2 * 48 * 8 * 1 * 40
    assert total == (rows * 130 * 8 + 255) // 256 * 256
    assert lib.kvq_exchange_bytes(0, 40, 128, 1, 2) == 0


def test_cpu_tensors_raise_value_error():
    q = torch.zeros(1, 4, 128, dtype=torch.float16)
    k = torch.zeros(1, 2, 8, 128, dtype=torch.int8)
    s = torch.ones(1, 2, 8, 4, dtype=torch.float16)
    ctx = torch.tensor([8], dtype=torch.int32)
    with pytest.raises(ValueError, match="requires CUDA"):
        kvq.decode_attn_int8(q, k, k, s, s, ctx)
    with pytest.raises(ValueError, match="CUDA"):
        kvq.quantize_symmetric_int8(torch.zeros(1, 1, 1, 128, dtype=torch.float16))


def test_wrapper_shape_dtype_errors():
    q = torch.zeros(1, 4, 128, dtype=torch.float16)
    k = torch.zeros(1, 2, 8, 128, dtype=torch.int8)
    s = torch.ones(1, 2, 8, 4, dtype=torch.float16)
    ctx = torch.tensor([8], dtype=torch.int32)
    with pytest.raises(ValueError, match=r"q must have shape"):
        kvq.decode_attn_int8(q[0], k, k, s, s, ctx)
    with pytest.raises(ValueError, match=r"k_cache/v_cache must have shape"):
        kvq.decode_attn_int8(q, k[0], k, s, s, ctx)
    with pytest.raises(ValueError, match=r"context_lens must be 1D"):
        kvq.decode_attn_int8(q, k, k, s, s, ctx[None])
    with pytest.raises(ValueError, match="head_dim must be positive"):
        kvq.decode_attn_int4(q, k, k, s, s, ctx, head_dim=0)


def test_normalize_static_scale_layouts():
    B, H, S, G = 2, 3, 5, 4
    base = torch.arange(H * G, dtype=torch.float32).view(H, G) + 1
    want = base[None, :, None, :].expand(B, H, S, G)
    for layout in (base, base[None], base[:, None, :], base[:, :, None], base[None, :, None, :],
                   want.contiguous(), want.contiguous()[..., None]):
        got = quant.normalize_static_scale(layout, B, H, S, G)
        assert got.shape == (B, H, S, G) and torch.equal(got, want)
    with pytest.raises(ValueError, match="heads mismatch"):
        quant.normalize_static_scale(torch.ones(7, G), B, H, S, G)
    with pytest.raises(ValueError, match="Unsupported 3D"):
        quant.normalize_static_scale(torch.ones(9, 9, 9), B, H, S, G)


def test_pack_unpack_round_trip_cpu(golden_dir):
    import numpy as np
    z = np.load(os.path.join(golden_dir, "pack_int4.npz"))
    codes = torch.from_numpy(z["codes"])
    assert torch.equal(quant.pack_int4(codes), torch.from_numpy(z["packed"]))
    assert torch.equal(quant.unpack_int4(quant.pack_int4(codes)), codes)
    with pytest.raises(ValueError):
        quant.pack_int4(codes.float())


def test_cache_constructor_validation():
    with pytest.raises(ValueError):
        kvq.INT8KVCache(0)
    with pytest.raises(ValueError):
        kvq.INT8KVCache(2, adaptive_static_margin=0.0)
    with pytest.raises(ValueError):
        kvq.INT4KVCache(2, max_seq_len=0)
    c = kvq.INT8KVCache(2, device="cpu")
    assert c.get_seq_len() == 0 and c.get_memory_mb() == 0.0
    with pytest.raises(ValueError, match="is empty"):
        c.get_int8_tensors(0)
    with pytest.raises(ValueError, match="out of range"):
        c.get_int8_tensors(5)
    c.record_fused_decode(1, "triton_fused")
    c.record_triton_kernel_call(1)
    st = c.get_decode_stats()
    assert st["fused_decode_calls"] == 1 and st["triton_decode_calls"] == 1 and st["triton_layer_hits"] == {"1": 1}
    with pytest.raises(ValueError, match="CPU tensors are not supported|CUDA"):
        c.append(0, torch.zeros(1, 2, 1, 128, dtype=torch.float16), torch.zeros(1, 2, 1, 128, dtype=torch.float16))
