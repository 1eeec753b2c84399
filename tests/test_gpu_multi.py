"""Two-GPU checks (skipped on a single-GPU box): sequence-sharded decode with one NCCL all-gather of
the packed partials per layer, against the same attention computed on one GPU; and the library's
fused combine / peer-store exchange / merge kernel against the NCCL path."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"     # plain peer stores only; nothing is bound to a multicast object
    import torch.distributed as dist
    import llm_kvcache_quantization_b200 as kvq
    from llm_kvcache_quantization_b200 import _lib, ops, parallel as P
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        g = torch.Generator().manual_seed(11)                      # identical data on every rank
        B, Hq, Hkv, S, D = 1, 40, 8, 3000, 128
        q = torch.randn(B, Hq, D, generator=g).half()
        k = torch.randn(B, Hkv, S + 1, D, generator=g).half()
        v = torch.randn(B, Hkv, S + 1, D, generator=g).half()
        tau = torch.empty(Hq).uniform_(0.8, 1.2, generator=g)
        idx = torch.tensor([[7]] * Hkv, dtype=torch.int16)
        tab = torch.full((1, Hkv, 4), 0.6, dtype=torch.float32)
        sh = P.SequenceSharding(world=world, max_seq_len=S + 1)
        lo, hi = sh.token_range(rank)
        local = kvq.INT4KVCache(1, device=dev, group_size=32, static_k_scale=tab.to(dev), static_v_scale=tab.to(dev),
                                outlier_idx=idx[None])
        local.reserve(0, B, Hkv, D, max(32, sh.chunk))
        n_prompt = max(0, min(S, hi) - lo)
        if n_prompt:
            local.append(0, k[:, :, lo:lo + n_prompt].to(dev), v[:, :, lo:lo + n_prompt].to(dev))
        if sh.owner_of(S) == rank:                                  # only the owner appends the new token
            local.append(0, k[:, :, S:S + 1].to(dev), v[:, :, S:S + 1].to(dev))
        n_local = sh.local_len(rank, S + 1)
        assert local._layer_seq_lens[0] == n_local
        send = torch.empty(B, Hq, D + 2, dtype=torch.float32, device=dev)
        recv = torch.empty(world, B, Hq, D + 2, dtype=torch.float32, device=dev)
        P.check_partial_shapes(send.shape)
        t = {n: b for n, b in local._bufs[0].items()}
        t["outlier_idx"] = idx.to(dev)
        out = P.sharded_decode(_lib.FMT_INT4, q.to(dev), t, n_local, 0.088, send=send, recv=recv, inv_tau=tau.to(dev))
        torch.cuda.synchronize()
        if rank == 0:
            full = kvq.INT4KVCache(1, device=dev, group_size=32, static_k_scale=tab.to(dev), static_v_scale=tab.to(dev),
                                   outlier_idx=idx[None])
            full.append(0, k.to(dev), v.to(dev))
            ref = full.fused_decode(0, q.to(dev), 0.088, inv_tau=tau.to(dev))
            err = (out.float() - ref.float()).abs()
            ret["max_err"] = float(err.max())
            ret["ok"] = bool((err <= 2e-3 + 1e-2 * ref.float().abs()).all())
            # and against the oracle itself (the reference's torch path restated), not only the one-GPU kernel
            from oracle import kvq_oracle as O
            ft = full.get_decode_tensors(0)
            want = O.decode_attn_int4_outlier(q.numpy(), *(ft[n].cpu().numpy() for n in ("k", "v", "ks", "vs", "kside", "vside")),
                                              idx.numpy(), [S + 1], 0.088, inv_tau=tau.numpy()).astype(np.float32)
            oerr = np.abs(out.float().cpu().numpy() - want)
            ret["oracle_max_err"] = float(oerr.max())
            ret["oracle_ok"] = bool((oerr <= 2e-3 + 1e-2 * np.abs(want)).all())
        # the library's own exchange: combine + peer stores over NVLink + merge in one launch.  Five
        # steps reuse both parities of the receive buffer; the query changes every step.
        xchg = P.PeerExchange(B, Hq, D, slots=2)
        out2 = torch.empty(2, B, Hq, D, dtype=torch.float16, device=dev)
        worst, good = 0.0, True
        local.reserve(0, B, Hkv, D, sh.chunk + 32)
        t = {n: b for n, b in local._bufs[0].items()}
        t["outlier_idx"] = idx.to(dev)
        is_owner = sh.owner_of(S) == rank
        for step in range(5):
            qs = (q * (1.0 + 0.25 * step)).to(dev)
            # one more token per step, stored by the owner of the sequence end: its append runs beside the
            # scan and the exchange kernel attends the new token from the cache
            kt = torch.randn(B, Hkv, 1, D, generator=g).half().to(dev)
            vt = torch.randn(B, Hkv, 1, D, generator=g).half().to(dev)
            app = None
            if is_owner:
                n_local += 1
                app = lambda: local.append(0, kt, vt)
            xchg.advance()
            for slot in range(2):
                xchg.decode(_lib.FMT_INT4, qs if slot == 0 else -qs, t, n_local, 0.088, slot=slot, out=out2[slot],
                            inv_tau=tau.to(dev), append=app if slot == 0 else None)
            torch.cuda.synchronize()
            for slot in range(2):
                want = P.sharded_decode(_lib.FMT_INT4, qs if slot == 0 else -qs, t, n_local, 0.088, send=send, recv=recv,
                                        inv_tau=tau.to(dev))
                err = (out2[slot].float() - want.float()).abs()
                worst = max(worst, float(err.max()))
                good = good and bool((err <= 1e-3 + 2e-3 * want.float().abs()).all())
        torch.cuda.synchronize()
        ret[f"xchg_ok_{rank}"] = good and int(xchg.status.item()) == 0
        ret[f"xchg_err_{rank}"] = worst
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sequence_sharded_decode_two_gpus():
    import torch.multiprocessing as mp
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert ret.get("ok") is True and ret.get("oracle_ok") is True, dict(ret)
    assert ret.get("xchg_ok_0") is True and ret.get("xchg_ok_1") is True, dict(ret)
