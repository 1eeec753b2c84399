"""Host-side logic of the multi-GPU partitioning, run as world_size-2 gloo ranks on CPU:
token-range ownership, the packed-partial all-gather, shape agreement, and the merge rule
(checked with the oracle's merge; the CUDA merge kernel is covered by the GPU tests)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llm_kvcache_quantization_b200 import parallel as P
from oracle import kvq_oracle as O


def test_batch_shard_covers_batch_once():
    for batch, world in ((64, 8), (10, 4), (3, 8), (16, 1)):
        rows = [P.batch_shard(batch, r, world) for r in range(world)]
        assert rows[0][0] == 0 and rows[-1][1] == batch
        assert all(rows[i][1] == rows[i + 1][0] for i in range(world - 1))
        sizes = [hi - lo for lo, hi in rows]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        P.batch_shard(8, 2, 2)


def test_sequence_sharding_ownership():
    s = P.SequenceSharding(world=8, max_seq_len=131073)
    assert s.chunk % 32 == 0 and s.chunk * 8 >= 131073
    covered = 0
    for r in range(8):
        lo, hi = s.token_range(r)
        assert lo == covered or lo == hi
        covered = hi
    assert covered == 131073
    assert s.owner_of(0) == 0 and s.owner_of(131072) == 7 and s.owner_of(s.chunk) == 1
    assert sum(s.local_len(r, 40000) for r in range(8)) == 40000
    assert s.local_len(7, 100) == 0
    with pytest.raises(ValueError):
        s.owner_of(131073)
    tiny = P.SequenceSharding(world=4, max_seq_len=10)      # fewer tokens than ranks x alignment
    assert [tiny.token_range(r) for r in range(4)] == [(0, 10), (10, 10), (10, 10), (10, 10)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)                       # same data on every rank
        b, hq, hkv, s, d = 2, 6, 2, 150, 128
        q = rng.standard_normal((b, hq, d)).astype(np.float16)
        k = rng.standard_normal((b, hkv, s, d)).astype(np.float16)
        v = rng.standard_normal((b, hkv, s, d)).astype(np.float16)
        total = [s, 70]
        if mode == "mismatch":
            shape = (b, hq, d + 2) if rank == 0 else (b, hq + 1, d + 2)
            try:
                P.check_partial_shapes(shape)
                ret[rank] = "no error"
            except RuntimeError as e:
                ret[rank] = "raised" if "disagree" in str(e) else repr(e)
            return
        sh = P.SequenceSharding(world=world, max_seq_len=s, align=32)
        lo, hi = sh.token_range(rank)
        ctx = [max(0, min(t, hi) - lo) for t in total]
        o, m, l = O.decode_attn_dequantized(q, k[:, :, lo:hi], v[:, :, lo:hi], ctx, 0.088, return_lse=True)
        packed = torch.from_numpy(np.concatenate([o.astype(np.float32), m[..., None], l[..., None]], axis=-1))
        P.check_partial_shapes(packed.shape)
        allp = P.gather_partials(packed).numpy()             # [W, B, Hq, D+2]
        merged = O.lse_merge(allp[..., :d], allp[..., d], allp[..., d + 1])
        full = O.decode_attn_dequantized(q, k, v, total, 0.088)
        err = np.abs(merged.astype(np.float32) - full.astype(np.float32)).max()
        ret[rank] = float(err)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ("merge", "mismatch"))
def test_two_gloo_ranks(mode):
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), mode, ret), nprocs=world, join=True)
    assert len(ret) == world
    if mode == "merge":
        assert all(v < 2e-3 for v in ret.values()), dict(ret)
    else:
        assert all(v == "raised" for v in ret.values()), dict(ret)
