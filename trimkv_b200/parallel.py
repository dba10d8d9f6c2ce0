"""Batch partition of requests across the GPUs of one box.

Every (request, layer, KV head) segment of the cache is appended to, evicted and attended independently
(the reference's per-head policy is row-wise over ``[B, Hkv]``, src/trimkv/cache_utils.py:190-198), so requests
are split across ranks and each rank runs its own model replica and cache: there is no collective on the cache
path.  The only exchange is the gather of the generated token ids at the end.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import ops


def partition_bounds(num_requests: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous slice ``[lo, hi)`` of the request list owned by ``rank``; sizes differ by at most one."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(num_requests, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_rows(local: torch.Tensor, num_requests: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All ranks' row blocks (rank order = request order) concatenated on every rank.

    ``local`` is ``[n_local, T]`` on any device the backend supports; blocks may have different ``n_local``.
    """
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    width = local.shape[1]
    sizes = [partition_bounds(num_requests, world, r) for r in range(world)]
    biggest = max(hi - lo for lo, hi in sizes)
    padded = local.new_zeros(biggest, width)
    padded[: local.shape[0]] = local
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded, group=group)
    return torch.cat([o[: hi - lo] for o, (lo, hi) in zip(out, sizes)], dim=0)


def generate_partitioned(generate_fn: Callable[[torch.Tensor], torch.Tensor], input_ids: torch.Tensor,
                         group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Runs ``generate_fn`` on this rank's slice of ``input_ids`` ``[N, S]`` and returns all ``[N, S + new]`` rows.

    ``generate_fn`` is e.g. ``lambda ids: model.generate(ids, max_new_tokens=..., past_key_values=TrimKVCache())``.
    Results are identical to a single-rank run request by request, because no state is shared between requests.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    lo, hi = partition_bounds(input_ids.shape[0], world, rank)
    local = generate_fn(input_ids[lo:hi]) if hi > lo else input_ids.new_zeros(0, 0)
    if world == 1:
        return local
    # ranks with no request still have to agree on the row width
    width = torch.tensor([local.shape[1] if hi > lo else 0], dtype=torch.int64, device=input_ids.device)
    dist.all_reduce(width, op=dist.ReduceOp.MAX, group=group)
    if hi == lo:
        local = input_ids.new_zeros(0, int(width.item()))
    return gather_rows(local, input_ids.shape[0], group)


class PeerExchange:
    """Gathered-output buffers of a head-sharded decode step, visible to every rank of one box.

    Every rank allocates one block holding ``nbuf`` buffers ``[batch, width]`` and an ``int32[world]`` flag array in
    its own memory, exports it (CUDA IPC) and maps the peers' blocks into its address space with its own device
    current, which also enables peer access over NVLink.  The attention merge kernel then stores each rank's column
    block into every rank's buffer and raises a flag (``ops.decode_attn_push``), and ``ops.peer_wait`` holds the
    consumer's stream until all blocks have arrived: attention and all-gather in one pass, no library collective in
    the step.  The mapped peer memory is only ever written, never read.
    """

    def __init__(self, batch: int, width: int, dtype: torch.dtype, device, nbuf: int = 3,
                 group: Optional[dist.ProcessGroup] = None):
        import ctypes
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.nbuf, self.width = nbuf, width
        esize = torch.empty((), dtype=dtype).element_size()
        buf_bytes = -(-batch * width * esize // 256) * 256
        flag_off = nbuf * buf_bytes
        # The block gets an allocation of its own (a private pool): the IPC handle exports the whole allocation a
        # pointer lies in, and the peers must be able to write to this block and to nothing else of this process.
        self._device = torch.device(device)
        self._pool = torch.cuda.MemPool()
        with torch.cuda.use_mem_pool(self._pool, device=self._device):
            self._block = torch.zeros(flag_off + 256, dtype=torch.uint8, device=self._device)
        self.buffers = [self._block[i * buf_bytes: i * buf_bytes + batch * width * esize].view(dtype).view(batch, width)
                        for i in range(nbuf)]
        self.flags = self._block[flag_off: flag_off + 4 * self.world].view(torch.int32)
        self.sync = torch.zeros(3, dtype=torch.int32, device=device)   # CTA counter, exchanges sent, received
        torch.cuda.synchronize(device)
        everyone = [None] * self.world
        try:
            mine = ops.ipc_export(self._block)
        except ops._lib.TrimKVNativeError as e:
            raise RuntimeError("the exchange block could not be exported over CUDA IPC (not supported with the "
                               "allocator's expandable_segments setting)") from e
        dist.all_gather_object(everyone, mine, group=group)
        bases, self._imported = [], []
        with torch.cuda.device(self._device):
            for r, (handle, offset) in enumerate(everyone):
                if r == self.rank:
                    bases.append(self._block.data_ptr())
                else:
                    bases.append(ops.ipc_import(handle) + offset)
                    self._imported.append(handle)
        self.out_ptrs = [(ctypes.c_void_p * self.world)(*[b + i * buf_bytes for b in bases]) for i in range(nbuf)]
        self.flag_ptrs = (ctypes.c_void_p * self.world)(*[b + flag_off for b in bases])
        dist.barrier(group=group)   # nobody pushes before every rank has zeroed and mapped its block

    def buffer(self, i: int) -> torch.Tensor:
        return self.buffers[i]

    def close(self) -> None:
        """Unmaps the peers' blocks.  Collective: every rank calls it once no exchange is in flight (the barrier makes
        sure nobody unmaps a block a peer is still writing to)."""
        if getattr(self, "_imported", None) is None:
            return
        torch.cuda.synchronize(self._device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self._device):
            for handle in self._imported:
                ops.ipc_release(handle)
        self._imported = None
