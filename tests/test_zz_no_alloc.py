"""`kvq_decode_attn_static`: decode attention for hosts that may not allocate GPU memory.

Some callers of this library cannot call cudaMalloc when they need attention - a serving
process whose memory pool took all of HBM at start-up, or a plugin invoked where the allocator
is off limits.  For them the library keeps the split-K partials in a fixed array of its own.
This file checks that entry point, through the C ABI, against the regular one: same inputs, two
calls in a row (the array is reused and keeps the first call's contents), plus the size limit.

It is named to be collected last, so that a run that stops at the first failure has already run
every other test; it also passes when run alone in a fresh process.
"""
import numpy as np
import pytest
import torch

import llm_kvcache_quantization_b200 as kvq
from llm_kvcache_quantization_b200 import _lib, ops
from oracle import kvq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
ATOL, RTOL = 2e-3, 1e-2          # the tolerance of the other decode tests


def _case(seed, b, hq, hkv, s, fmt):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, hq, 128, generator=g).half().to(DEV)
    k = torch.randn(b, hkv, s, 128, generator=g).half().to(DEV)
    v = torch.randn(b, hkv, s, 128, generator=g).half().to(DEV)
    cache = (kvq.INT8KVCache if fmt == _lib.FMT_INT8 else kvq.INT4KVCache)(1, device=DEV, group_size=32)
    cache.append(0, k, v)
    t = cache.get_decode_tensors(0)
    ctx = torch.tensor([s] + [max(1, s // 3)] * (b - 1), dtype=torch.int32, device=DEV)
    return q, t, ctx


def _assert_close(got, ref):
    got, ref = got.float().cpu().numpy(), ref.float().cpu().numpy()
    assert not np.isnan(got).any()
    err = np.abs(got - ref)
    assert np.all(err <= ATOL + RTOL * np.abs(ref)), float(err.max())


def test_static_workspace_matches_regular_entry_point_twice_in_a_row():
    sm = 1.0 / np.sqrt(128.0)
    # call 1: INT8, several splits; call 2: INT4 with a different shape - it finds the array
    # full of call 1's partials and must not be disturbed by them
    for seed, (b, hq, hkv, s, fmt) in enumerate(((2, 12, 2, 1500, _lib.FMT_INT8), (3, 28, 4, 700, _lib.FMT_INT4))):
        q, t, ctx = _case(40 + seed, b, hq, hkv, s, fmt)
        ref = ops.decode_attn(fmt, q, t["k"], t["v"], t["ks"], t["vs"], ctx, sm, head_dim=128)
        out = torch.full_like(ref, float("nan"))
        out2 = torch.full_like(ref, float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        ops.decode_attn_static(fmt, q, t["k"], t["v"], t["ks"], t["vs"], ctx, sm, out)
        # and once more on the same inputs: a call right after another one on the same array
        ops.decode_attn_static(fmt, q, t["k"], t["v"], t["ks"], t["vs"], ctx, sm, out2)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, "the entry point (or its wrapper) obtained device memory"
        _assert_close(out, ref)
        assert torch.equal(out, out2)
        # and against the oracle itself, not only against the other entry point
        host = [t[n].cpu().numpy() for n in ("k", "v", "ks", "vs")]
        fn = O.decode_attn_int8 if fmt == _lib.FMT_INT8 else O.decode_attn_int4
        _assert_close(out, torch.from_numpy(fn(q.cpu().numpy(), *host, ctx.cpu().numpy(), sm).astype(np.float32)))
    torch.cuda.synchronize()
    assert _lib.load().kvq_debug_error_flag(0) == 0


def test_static_workspace_lowers_its_own_split_choice_to_fit():
    """With `splits == 0` the entry point lowers the library's split choice until the partials fit.  On this part the
    choice never comes near 8 MiB, so the check runs in a child process with KVQ_STATIC_WS_LIMIT (read once per
    process) set to less than the choice needs."""
    import os
    import subprocess
    import sys
    code = r"""
import numpy as np, torch
import llm_kvcache_quantization_b200 as kvq
from llm_kvcache_quantization_b200 import _lib, ops
g = torch.Generator().manual_seed(3)
b, hq, hkv, s = 1, 12, 2, 6000
q = torch.randn(b, hq, 128, generator=g).half().cuda()
k = torch.randn(b, hkv, s, 128, generator=g).half().cuda()
v = torch.randn(b, hkv, s, 128, generator=g).half().cuda()
c = kvq.INT8KVCache(1, device="cuda", group_size=32); c.append(0, k, v)
t = c.get_decode_tensors(0)
ctx = torch.tensor([s], dtype=torch.int32, device="cuda")
ref = ops.decode_attn(_lib.FMT_INT8, q, t["k"], t["v"], t["ks"], t["vs"], ctx, 0.088, head_dim=128)
auto = ops.last_splits()
need = _lib.load().kvq_decode_workspace_bytes(b, hq, 128, auto)
assert auto >= 4 and need > 16384, (auto, need)            # the limit below is smaller than the automatic choice needs
out = torch.full_like(ref, float("nan"))
ops.decode_attn_static(_lib.FMT_INT8, q, t["k"], t["v"], t["ks"], t["vs"], ctx, 0.088, out)
err = (out.float() - ref.float()).abs()
assert bool((err <= 2e-3 + 1e-2 * ref.float().abs()).all()), float(err.max())
print("ok", auto)
"""
    env = dict(os.environ, KVQ_STATIC_WS_LIMIT="16384")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=root, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().startswith("ok"), r.stdout[-500:] + r.stderr[-2000:]


def test_static_workspace_rejects_requests_beyond_its_size():
    q, t, ctx = _case(50, 2, 12, 2, 4096, _lib.FMT_INT8)
    out = torch.empty(2, 12, 128, dtype=torch.float16, device=DEV)
    limit = 8 << 20
    too_many = limit // (2 * 12 * 130 * 4) + 1          # splits whose partials no longer fit
    with pytest.raises(_lib.KvqError) as ei:
        ops.decode_attn_static(_lib.FMT_INT8, q, t["k"], t["v"], t["ks"], t["vs"], ctx, 0.088, out, splits=too_many)
    assert ei.value.code == _lib.KVQ_ELIMIT and "limit" in str(ei.value)
    # the largest split count that fits is accepted
    ops.decode_attn_static(_lib.FMT_INT8, q, t["k"], t["v"], t["ks"], t["vs"], ctx, 0.088, out, splits=too_many - 2)
    ref = ops.decode_attn(_lib.FMT_INT8, q, t["k"], t["v"], t["ks"], t["vs"], ctx, 0.088, head_dim=128)
    _assert_close(out, ref)
