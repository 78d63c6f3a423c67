"""Column-parallel sharding of a dequantize-GEMM over the GPUs of one node.

The reference is a single-GPU kernel compiler and has no counterpart (its only
multi-GPU feature benchmarks autotuner candidates on several devices,
tilelang/autotuner/tuner.py:872-946). The weight of ``C = A @ dequant(W)^T``
shards along N: rank r owns a contiguous block of weight rows with its scales and
zeros (groups run along K, so a shard never splits a group), the activations are
replicated, each rank computes ``C[:, shard]`` with the single-GPU kernel, and the
only exchange step is one all-gather of C -- or none when the consumer is
row-parallel and takes C column-sharded. One process per GPU, ``torch.distributed``
(NCCL on GPUs, gloo in CPU tests) for the plumbing.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    rank: int
    start: int   # first weight row (output column) owned
    stop: int    # one past the last

    @property
    def size(self) -> int:
        return self.stop - self.start


def plan_column_shards(N: int, world_size: int, align: int = 128) -> List[Shard]:
    """Contiguous blocks of output columns, as even as possible in units of ``align``
    rows (the kernel's weight-tile height) so at most the last rank has a ragged tile."""
    if N <= 0 or world_size <= 0:
        raise ValueError("N and world_size must be positive")
    units = (N + align - 1) // align
    base, extra = divmod(units, world_size)
    shards, start = [], 0
    for r in range(world_size):
        n_units = base + (1 if r < extra else 0)
        stop = min(N, start + n_units * align)
        shards.append(Shard(r, start, stop))
        start = stop
    return shards


class ColumnParallelDequantLinear:
    """Holds this rank's shard of a packed weight and runs the sharded GEMM.

    ``pack_fn(rows_slice) -> packed`` builds the rank-local packed weight from a slice of
    weight rows; ``gemm_fn(A, packed) -> C_shard`` is the single-GPU kernel call. Both
    are injected so the host logic runs unchanged on GPUs (``ops.pack_*`` / ``ops.gemm``)
    and in CPU tests.
    """

    def __init__(self, N: int, pack_fn: Callable[[slice], object], gemm_fn: Callable[[torch.Tensor, object], torch.Tensor],
                 group: Optional[dist.ProcessGroup] = None, align: int = 128):
        self.group = group
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N = N
        self.shards = plan_column_shards(N, self.world_size, align)
        self.shard = self.shards[self.rank]
        self.packed = pack_fn(slice(self.shard.start, self.shard.stop)) if self.shard.size > 0 else None
        self.gemm_fn = gemm_fn

    def forward_sharded(self, A: torch.Tensor) -> torch.Tensor:
        """C[:, shard] for this rank (no communication)."""
        if self.shard.size == 0:
            return A.new_zeros((A.shape[0], 0))
        return self.gemm_fn(A, self.packed)

    def forward(self, A: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Full C on every rank: local GEMM, then one all-gather of the column blocks."""
        c_local = self.forward_sharded(A)
        if self.world_size == 1:
            return c_local
        M = A.shape[0]
        sizes = [s.size for s in self.shards]
        if out is None:
            out = c_local.new_empty((M, self.N))
        if len(set(sizes)) == 1:
            # equal blocks: gather into a (world, M, n) buffer, then interleave the blocks
            buf = c_local.new_empty((self.world_size * M, sizes[0]))
            dist.all_gather_into_tensor(buf, c_local.contiguous(), group=self.group)
            out.view(M, self.world_size, sizes[0]).copy_(buf.view(self.world_size, M, sizes[0]).permute(1, 0, 2))
        else:
            # ragged blocks: collectives want equal sizes, so pad to the widest block
            widest = max(sizes)
            padded = c_local.new_zeros((M, widest))
            padded[:, :c_local.shape[1]] = c_local
            buf = c_local.new_empty((self.world_size * M, widest))
            dist.all_gather_into_tensor(buf, padded, group=self.group)
            buf = buf.view(self.world_size, M, widest)
            for s in self.shards:
                out[:, s.start:s.stop] = buf[s.rank, :, :s.size]
        return out


class PeerGatheredOutput:
    """The gathered output of a column-parallel GEMM, filled by the GEMM kernels themselves.

    Every rank allocates one ``(world, M, n_local)`` buffer in symmetric memory (equal shards);
    rank r's kernel stores its ``(M, n_local)`` block to slot r of its own buffer and, through
    peer pointers over NVLink, to slot r of every other rank's buffer, tile by tile from the
    epilogue, so the transfer runs under the rest of the GEMM and there is no separate
    all-gather. ``gemm(A, packed)`` launches the local GEMM; ``wait()`` is the exchange step
    that is left: a barrier after which every slot of ``buffer`` is complete on every rank.
    ``buffer[r]`` is ``C[:, shard r]``; a consumer that wants ``(M, N)`` permutes the view.

    The reference is single-GPU and has no counterpart; this replaces the one
    ``all_gather_into_tensor`` of :class:`ColumnParallelDequantLinear.forward`.
    """

    def __init__(self, M: int, n_local: int, dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("peer stores reach the GPUs of one node (at most 8)")
        self.M, self.n_local = M, n_local
        self.buffer = symm_mem.empty((self.world, M, n_local), dtype=dtype, device=device)
        self._handle = symm_mem.rendezvous(self.buffer, self.group.group_name)
        block_bytes = M * n_local * self.buffer.element_size()
        ptrs = list(self._handle.buffer_ptrs)
        # my block's address inside every other rank's buffer
        self.peer_ptrs = [ptrs[r] + self.rank * block_bytes for r in range(self.world) if r != self.rank]
        self._token = torch.zeros(1, dtype=torch.int32, device=device)

    def gemm(self, A: torch.Tensor, packed, **kwargs) -> torch.Tensor:
        from . import ops
        return ops.gemm(A, packed, out=self.buffer[self.rank], peer_outs=self.peer_ptrs, **kwargs)

    def wait(self) -> torch.Tensor:
        """Every rank's kernel has finished (its peer stores with it): one tiny all-reduce on
        the current stream orders the ranks. Returns the gathered buffer."""
        dist.all_reduce(self._token, group=self.group)
        return self.buffer

