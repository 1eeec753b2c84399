"""Calibration statistics on the GPU: the per-(head, group) absmax reduction is bit-identical to the torch
expression the reference uses (scripts/calibrate_behavior.py:228-260), accumulates over calls, and the
sample -> scale pipeline round-trips through the calibration JSON into a cache."""
import json

import numpy as np
import pytest
import torch

import llm_kvcache_quantization_b200 as kvq
from llm_kvcache_quantization_b200 import calibration as C, engine as E, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(t, gs):
    h, s, d = t.shape
    return t.float().view(h, s, d // gs, gs).abs().amax(dim=3).amax(dim=1)


@pytest.mark.parametrize("gs", (8, 16, 32, 64, 128))
def test_group_absmax_matches_torch(gs):
    g = torch.Generator().manual_seed(gs)
    x = (torch.randn(3, 4, 1000, 128, generator=g) * 3).half().to(DEV)
    x[1, 2, 777, 5] = 123.5                                  # a lone outlier must surface in its group
    got = ops.group_absmax(x, gs)
    want = torch.stack([_ref(x[b], gs) for b in range(3)]).amax(dim=0)
    assert torch.equal(got, want)
    # a strided view (every other head), accumulated over two calls, equals the whole
    part = torch.zeros(2, 128 // gs, device=DEV)
    ops.group_absmax(x[:2, ::2], gs, out=part)
    ops.group_absmax(x[2:, ::2], gs, out=part)
    assert torch.equal(part, want[::2])
    assert torch.equal(C.compute_absmax_per_group(x[0], gs), _ref(x[0], gs))
    assert tuple(ops.group_absmax(x[:, :, :0], gs).shape) == (4, 128 // gs)


def test_calibration_pipeline_round_trip(tmp_path):
    g = torch.Generator().manual_seed(3)
    L, H, D, gs = 2, 2, 128, 32
    samples = [[(torch.randn(H, 50 + 10 * i, D, generator=g) * (1 + l)).half().to(DEV) for l in range(L)] for i in range(5)]
    stats = C.collect_absmax_samples(samples, gs)
    assert len(stats) == L and len(stats[0]) == 5 and tuple(stats[0][0].shape) == (H, D // gs)
    k_scale = C.scales_from_absmax_samples(stats, 99.9, 127)
    want = torch.quantile(torch.stack([_ref(s[1], gs) for s in samples]).float(), 0.999, dim=0).clamp(min=1e-5) / 127.0
    assert torch.equal(k_scale[1], want)
    path = str(tmp_path / "calib.json")
    tau = torch.full((L, 12), 1.1)
    C.save_calibration(path, k_scale, k_scale, group_size=gs, clip_percentile=99.9, inv_tau=tau)
    doc = json.load(open(path))
    assert doc["version"] == 2 and doc["group_size_k"] == gs and len(doc["k_scale"]) == L
    calib = E.load_calibration(path, "int8_ours", DEV)
    assert calib["group_size"] == gs and tuple(calib["static_k_scale"].shape) == (L, H, D // gs)
    assert torch.allclose(calib["static_k_scale"].float().cpu(), torch.stack(k_scale).cpu(), rtol=1e-3)
    cache = E.build_cache("int8_ours", L, DEV, calib=calib, max_seq_len=64)
    k = samples[0][0][None, :, :40]
    cache.append(0, k, k)
    kd, _ = cache.get_kv(0)
    assert float((kd.float() - k.float()).abs().max()) < 0.05 * float(k.float().abs().max())


@pytest.mark.parametrize("gs", (16, 32, 128))
def test_group_absmax_reproduces_the_reference_function(golden_dir, gs):
    """Fixture from the reference's own compute_absmax_per_group (scripts/calibrate_behavior.py:228-260), per sample and
    as the running maximum its collection loop keeps."""
    import os
    z = np.load(os.path.join(golden_dir, "calib_absmax.npz"))
    x = torch.from_numpy(z["x"]).to(DEV)                       # [samples, H, S, D]
    acc = torch.zeros(x.shape[1], x.shape[3] // gs, device=DEV)
    for i in range(x.shape[0]):
        got = C.compute_absmax_per_group(x[i], gs)
        assert np.array_equal(got.float().cpu().numpy(), z[f"g{gs}_per_sample"][i])
        ops.group_absmax(x[i][None], gs, out=acc)
    assert np.array_equal(acc.cpu().numpy(), z[f"g{gs}_running_max"])
