"""GPU parity at the shapes bench.py times: ONE full-size layer of each benchmark configuration, built by the
bench's own workload builder, stepped by the bench's own step function (quantize-on-append of the new token +
split-K scan with the library's split choice + combine), compared with the C restatement of the reference's
torch dequantize-then-attention path (src/engine/patch_model.py:355-374) on the same cache bytes.
Tolerance (north star): |a-b| <= 2e-3 + 1e-2 |b|."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
import bench  # noqa: E402
from llm_kvcache_quantization_b200 import ops, _lib  # noqa: E402
from oracle import c_oracle as CO  # noqa: E402

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-3, 1e-2


def _oracle_rows(wl, cache, q, inv_tau, rows):
    """C oracle over the batch rows `rows` of layer 0, context S + 1 (the appended token included)."""
    S, kind = wl["S"], wl["kind"]
    b = cache._bufs[0]
    idx = torch.as_tensor(rows, device=q.device)

    def host(name):
        t = b.get(name)
        return None if t is None else t[idx, :, :S + 1].contiguous().cpu().numpy()
    fmt = 0 if kind == "fp16" else 1 if kind.startswith("int8") else 2
    extra = {}
    if kind == "int4_asym":
        extra = dict(kz=host("kz"), vz=host("vz"))
    elif kind == "int4_outlier":
        extra = dict(kside=host("kside"), vside=host("vside"), outlier_idx=cache.outlier_idx[0].cpu().numpy())
    ctx = np.full(len(rows), S + 1, np.int32)
    return CO.decode_attn(fmt, q[0][idx].cpu().numpy(), host("k"), host("v"), host("ks"), host("vs"), ctx,
                          1.0 / np.sqrt(bench.D), inv_tau=inv_tau[0].cpu().numpy(), **extra).astype(np.float32)


def _check(got, ref, what):
    got = got.float().cpu().numpy()
    assert not np.isnan(got).any(), what
    err = np.abs(got - ref)
    bad = err > ATOL + RTOL * np.abs(ref)
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} outside tolerance, max abs err {float(err.max()):.3e}"
    return float(err.max())


CASES = {
    # name: batch rows handed to the oracle (None = all)
    "c2": None,
    "c3": None,
    "c5": None,
    "c4": (0, 1, 31, 32, 56, 57, 62, 63),       # all 64 rows run on the GPU; 8 of them, first to last, are checked
    "c1": None,
}


@pytest.mark.parametrize("name", list(CASES))
def test_one_full_size_layer_matches_the_oracle(name, monkeypatch):
    dev = torch.device("cuda", 0)
    wl = dict(bench.WORKLOADS[name], layers=1)
    free, _ = torch.cuda.mem_get_info()
    need = wl["B"] * wl["Hkv"] * wl["S"] * bench.bytes_per_token_head(wl["kind"], wl["n_out"])
    if free < 3 * need + (2 << 30):
        pytest.skip("not enough free device memory for this layer")
    cache, q, k_new, v_new, inv_tau = bench.build_workload(wl, dev, seed=77, extra_slots=8)
    rows = list(range(wl["B"])) if CASES[name] is None else list(CASES[name])
    out = torch.empty(1, wl["B"], wl["Hq"], bench.D, dtype=torch.float16, device=dev)
    ref = None
    modes = [("0", "0"), ("1", "0")]                   # (KVQ_BENCH_NO_OVERLAP, KVQ_INT4_FAST)
    if wl["kind"].startswith("int4"):
        modes += [("0", "1"), ("1", "1")]
    for no_overlap, fast in modes:
        # tail_tokens = 1 (append beside the scan, the new token attended by the combine stage) and tail_tokens = 0
        monkeypatch.setenv("KVQ_BENCH_NO_OVERLAP", no_overlap)
        monkeypatch.setenv("KVQ_INT4_FAST", fast)
        out.zero_()
        step, splits_fn = bench.make_step(wl, cache, q, k_new, v_new, inv_tau, out)
        step()
        torch.cuda.synchronize()
        if ref is None:                                 # the append wrote slot S: same bytes for every mode
            ref = _oracle_rows(wl, cache, q, inv_tau, rows)
        _check(out[0][torch.as_tensor(rows, device=dev)], ref,
               f"{name} splits={splits_fn()} no_overlap={no_overlap} fast={fast}")
    assert _lib.load().kvq_debug_error_flag(0) == 0
    del cache
    ops.release_workspaces()
    torch.cuda.empty_cache()
