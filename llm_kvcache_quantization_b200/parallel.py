"""Multi-GPU partitioning of the decode path: one process per GPU.

Two ways the path shards (neither exists in the reference, which is single-GPU):

* batch sharding   - sequences are independent; rank r owns batch rows `batch_shard(B, r, W)`,
  its own cache and its own decode calls.  No collective on the data path.
* sequence sharding - one long sequence; rank r owns the contiguous token range
  `SequenceSharding.token_range(r)`, appends a new token only if it owns that position, runs the
  fused decode over its chunk into a packed normalised partial `[o | m | l]`, and the partials are
  merged after ONE all-gather per layer:
      M = max_r m_r;  out = sum_r o_r l_r e^{m_r - M} / sum_r l_r e^{m_r - M}
  Remote partials land in this GPU's own receive buffer before the merge kernel reads them.

The collective goes through `torch.distributed` (NCCL on GPUs; gloo for the host-side tests), or,
with `PeerExchange`, through the library's own fused kernel: combine + peer stores over NVLink +
merge in one launch per layer, no library collective on the data path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


def batch_shard(batch: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [lo, hi) of a batch owned by `rank`: contiguous, sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, rem = divmod(batch, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


@dataclass(frozen=True)
class SequenceSharding:
    """Contiguous token chunks of `chunk` tokens per rank (a multiple of 32 so that every shard
    starts on a tile boundary of the decode kernel)."""
    world: int
    max_seq_len: int
    align: int = 32

    @property
    def chunk(self) -> int:
        per = -(-self.max_seq_len // self.world)
        return -(-per // self.align) * self.align

    def token_range(self, rank: int) -> Tuple[int, int]:
        lo = min(self.max_seq_len, rank * self.chunk)
        return lo, min(self.max_seq_len, lo + self.chunk)

    def owner_of(self, position: int) -> int:
        if position < 0 or position >= self.max_seq_len:
            raise ValueError(f"position {position} outside [0, {self.max_seq_len})")
        return position // self.chunk

    def local_len(self, rank: int, total_len: int) -> int:
        """How many of the first `total_len` tokens of the sequence live on `rank`."""
        lo, hi = self.token_range(rank)
        return max(0, min(total_len, hi) - lo)


def gather_partials(packed: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather the packed partial `[B,Hq,D+2]` of every rank into `[W,B,Hq,D+2]` (one collective).
    Ranks must agree on the shape; a mismatch is detected here, before the collective, through the
    sizes exchanged at group set-up (`check_partial_shapes`)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world,) + tuple(packed.shape), dtype=packed.dtype, device=packed.device)
    elif tuple(out.shape) != (world,) + tuple(packed.shape):
        raise ValueError(f"receive buffer {tuple(out.shape)} does not match {world} x {tuple(packed.shape)}")
    if packed.is_cuda:
        dist.all_gather_into_tensor(out, packed.contiguous(), group=group)      # one NCCL all-gather
    else:
        dist.all_gather(list(out.unbind(0)), packed.contiguous(), group=group)  # gloo (host-side tests)
    return out


def check_partial_shapes(shape, group=None) -> None:
    """Host-side agreement check (run once per configuration, not per step): every rank must use the
    same [B, Hq, D+2]; raises on all ranks if any differs."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    mine = [int(x) for x in shape]
    all_shapes = [None] * world
    dist.all_gather_object(all_shapes, mine, group=group)
    if any(s != mine for s in all_shapes):
        raise RuntimeError(f"sequence-sharded ranks disagree on the partial shape: {all_shapes}")


def sharded_decode(fmt: int, q: torch.Tensor, tensors: dict, local_len: int, sm_scale: float, *,
                   send: torch.Tensor, recv: torch.Tensor, inv_tau=None, out=None, group=None) -> torch.Tensor:
    """One layer of sequence-sharded decode attention on this rank.

    `tensors` is `cache.get_decode_tensors(layer)` of the LOCAL chunk, `local_len` the number of
    valid local tokens (0 is fine: the rank then contributes the neutral partial), `send` a
    persistent fp32 `[B,Hq,D+2]` buffer and `recv` a persistent `[W,B,Hq,D+2]` buffer.
    Returns the merged fp16 `[B,Hq,D]` output (identical on every rank)."""
    from . import ops
    k = tensors["k"][:, :, :local_len]
    v = tensors["v"][:, :, :local_len]
    ks = tensors["ks"][:, :, :local_len]
    vs = tensors["vs"][:, :, :local_len]
    extra = {}
    if tensors.get("kz") is not None:
        extra.update(k_zp=tensors["kz"][:, :, :local_len], v_zp=tensors["vz"][:, :, :local_len])
    if tensors.get("outlier_idx") is not None:
        extra.update(outlier_idx=tensors["outlier_idx"].contiguous(), k_side=tensors["kside"][:, :, :local_len],
                     v_side=tensors["vside"][:, :, :local_len])
    scratch = torch.empty((q.shape[0], q.shape[1], q.shape[2]), dtype=torch.float16, device=q.device) if out is None else out
    ops.decode_attn(fmt, q, k, v, ks, vs, None, sm_scale, head_dim=q.shape[-1], inv_tau=inv_tau,
                    out=scratch, packed_partial=send, **extra)
    gather_partials(send, group=group, out=recv)
    return ops.lse_combine_packed(recv, out=scratch)


class PeerExchange:
    """Receive buffers of the fused combine-and-exchange kernel, one per rank, mapped into every peer
    through torch's symmetric memory (CUDA IPC under the hood; NVLink multicast is not used and its
    binding is switched off).  `slots` independent exchanges per decode step (one per layer).

        xchg = PeerExchange(B, Hq, D, slots=L)          # collective: every rank, same arguments
        per step:   xchg.advance()                       # once, before the first layer
        per layer:  xchg.decode(fmt, q, tensors, local_len, sm_scale, slot=l, out=out[l], ...)

    Every rank must issue the same sequence of calls.  A peer that never arrives makes the kernel give
    up after `wait_ns` (default one second), set `status` to 1 and return; the context stays usable."""

    def __init__(self, B: int, Hq: int, D: int, slots: int, group=None, device=None, wait_ns: int = 0):
        import os
        # The exchange kernel uses plain peer stores.  Symmetric-memory buffers must never be bound to an NVLink
        # multicast object: a rank that leaves while its memory is bound to one disturbs the other ranks' GPUs.
        # The package sets the switch at import; refuse to go on if something turned it back on.
        if os.environ.get("TORCH_SYMM_MEM_DISABLE_MULTICAST") != "1":
            raise RuntimeError("PeerExchange needs TORCH_SYMM_MEM_DISABLE_MULTICAST=1 (set when this package is imported); "
                               "it was changed afterwards")
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        from . import ops
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.B, self.Hq, self.D, self.slots = B, Hq, D, slots
        self.wait_ns = int(wait_ns)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        total = ops.exchange_bytes(B, Hq, D, slots, self.world)
        self.buf = symm.empty(total // 4, dtype=torch.float32, device=dev)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, self.group.group_name)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._side = None
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)             # nobody stores into a buffer that is still being cleared

    def advance(self) -> None:
        """Next decode step (device-side, capturable)."""
        self.epoch.add_(1)

    def decode(self, fmt: int, q: torch.Tensor, tensors: dict, local_len: int, sm_scale: float, *, slot: int,
               out: torch.Tensor, inv_tau=None, append=None) -> torch.Tensor:
        """Sequence-sharded decode attention of one layer: split-K scan of the local chunk, then the
        fused combine / exchange / merge.  Same contract as `sharded_decode`.

        `append` (only on the rank that stores the new token): a callable that launches the
        quantize-append of that token; it then runs on a second stream beside the scan of the older
        tokens, and the exchange kernel attends the new token from the cache (`local_len` counts it)."""
        from . import ops
        n = local_len
        spec = dict(peer_ptrs=self.peer_ptrs, rank=self.rank, slot=slot, slots=self.slots, epoch=self.epoch,
                    status=self.status, wait_ns=self.wait_ns)
        if n <= 0:
            if append is not None:
                raise ValueError("the appending rank holds at least the new token")
            # an empty shard contributes the neutral partial: one split with l = 0
            ops.neutral_partial(q.shape[0], q.shape[1], q.shape[2], q.device)
            return ops.combine_exchange(self.peer_ptrs, self.rank, slot, self.slots, self.epoch, out, splits=1,
                                        status=self.status, wait_ns=self.wait_ns)
        extra = {}
        if tensors.get("kz") is not None:
            extra.update(k_zp=tensors["kz"][:, :, :n], v_zp=tensors["vz"][:, :, :n])
        if tensors.get("outlier_idx") is not None:
            extra.update(outlier_idx=tensors["outlier_idx"].contiguous(), k_side=tensors["kside"][:, :, :n],
                         v_side=tensors["vside"][:, :, :n])
        scale = (None, None) if tensors.get("ks") is None else (tensors["ks"][:, :, :n], tensors["vs"][:, :, :n])

        def attend(**kw):
            return ops.decode_attn(fmt, q, tensors["k"][:, :, :n], tensors["v"][:, :, :n], scale[0], scale[1], None,
                                   sm_scale, head_dim=q.shape[-1], inv_tau=inv_tau, out=out, exchange=spec,
                                   **extra, **kw)
        if append is None:
            return attend()
        if self._side is None:
            self._side = torch.cuda.Stream(device=q.device)
        main = torch.cuda.current_stream(q.device)
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            append()
        attend(stages=1, tail_tokens=1)
        main.wait_stream(self._side)
        return attend(stages=2, tail_tokens=1)
