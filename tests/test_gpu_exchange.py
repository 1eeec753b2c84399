"""Single-GPU checks of the fused combine-and-exchange kernel: a one-rank exchange equals the plain
combine, and a peer that never arrives ends the bounded wait with a status flag - no hang, and the
context stays usable.  (The real two-rank exchange runs in test_gpu_multi.py on two GPUs; ranks that
wait for one another are never emulated as separate launches on one GPU.)"""
import numpy as np
import pytest
import torch

import llm_kvcache_quantization_b200 as kvq
from llm_kvcache_quantization_b200 import _lib, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(seed=5, B=2, Hq=12, Hkv=2, S=700):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, 128, generator=g).half().to(DEV)
    k = torch.randn(B, Hkv, S, 128, generator=g).half().to(DEV)
    v = torch.randn(B, Hkv, S, 128, generator=g).half().to(DEV)
    c = kvq.INT8KVCache(1, device=DEV, group_size=32, clip_percentile=100.0)
    c.append(0, k, v)
    return q, c.get_int8_tensors(0)


def _same(a, b):
    # the merge renormalises (o / l) * l / l in fp32: equal up to an fp16 rounding flip
    return torch.allclose(a.float(), b.float(), atol=1e-3, rtol=2e-3)


def _buffers(B, Hq, D, slots, world):
    total = ops.exchange_bytes(B, Hq, D, slots, world)
    assert total % 256 == 0 and total >= 2 * slots * world * B * Hq * (D + 2) * 8
    return [torch.zeros(total // 4, dtype=torch.float32, device=DEV) for _ in range(world)]


def test_single_rank_exchange_equals_combine():
    q, (k, v, ks, vs) = _setup()
    B, Hq, D = q.shape
    ref = ops.decode_attn(_lib.FMT_INT8, q, k, v, ks, vs, None, 0.088, head_dim=D, splits=5)
    bufs = _buffers(B, Hq, D, 3, 1)
    epoch = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty_like(ref)
    for step in range(3):                              # both parities, slot 2 of 3
        epoch.add_(1)
        out.zero_()
        ops.decode_attn(_lib.FMT_INT8, q, k, v, ks, vs, None, 0.088, head_dim=D, splits=5, stages=1, out=out)
        ops.combine_exchange([bufs[0].data_ptr()], 0, 2, 3, epoch, out, splits=5, status=status)
        assert _same(out, ref)
    assert int(status.item()) == 0


def test_absent_peer_ends_the_wait_with_a_status():
    q, (k, v, ks, vs) = _setup(seed=6)
    B, Hq, D = q.shape
    ref = ops.decode_attn(_lib.FMT_INT8, q, k, v, ks, vs, None, 0.088, head_dim=D, splits=4)
    bufs = _buffers(B, Hq, D, 1, 2)                    # "rank 1" is a buffer nobody writes
    epoch = torch.ones(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.zeros_like(ref)
    ops.decode_attn(_lib.FMT_INT8, q, k, v, ks, vs, None, 0.088, head_dim=D, splits=4, stages=1, out=out)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    ops.combine_exchange([b.data_ptr() for b in bufs], 0, 0, 1, epoch, out, splits=4, status=status,
                         wait_ns=20_000_000)           # 20 ms
    t1.record()
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert 15.0 < t0.elapsed_time(t1) < 500.0
    assert _same(out, ref)                             # the rank finished with its own partial
    # the context is intact: the next ordinary call works
    again = ops.decode_attn(_lib.FMT_INT8, q, k, v, ks, vs, None, 0.088, head_dim=D, splits=4)
    assert torch.equal(again, ref)
    with pytest.raises(_lib.KvqError):
        ops.combine_exchange([bufs[0].data_ptr()] * 17, 0, 0, 1, epoch, out, splits=4)
