"""A row-partitioned table that every GPU of the node reads in place (CUDA IPC mappings, NVLink / NVSwitch peer loads).

One process per GPU.  Rank g holds rows [g * rows_per_rank, (g + 1) * rows_per_rank) in its own HBM; `PeerTable` exports
that shard once, maps the shards of the other ranks and keeps the `world` base addresses in a small device array, so
`gather(ids, ...)` is one kernel (kge_gather_rows_peers) that copies any rows of the table - local or remote - into a
compact local buffer.  It replaces, for the staging half of a step, the exchange of ids, the gather at each owner and
the all-to-all of rows.

Ordering: a rank's `gather` must run after the owners' last updates of the rows have completed and before their next
ones begin.  `KgeStep` queues a barrier among the ranks behind the updates of a step (`publish`), and an owner's next
update consumes gradients that were computed from the gathered rows, so it cannot start early.

The reference is single-GPU (apps/kge/data/data_init.py:6-15) and has no counterpart.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import DTYPES, check


# A device allocation can be opened once per process: tensors that share one allocation of the caching allocator share
# the mapping.  handle bytes -> [mapped base address, users]
_open_allocations = {}


def _open(handle: bytes) -> int:
    ent = _open_allocations.get(handle)
    if ent is None:
        buf = (C.c_ubyte * 64).from_buffer_copy(handle)
        p = C.c_void_p()
        check(_lib.lib().kge_ipc_open(buf, 0, C.byref(p)))
        ent = _open_allocations[handle] = [p.value, 0]
    ent[1] += 1
    return ent[0]


def _close(handle: bytes) -> None:
    ent = _open_allocations.get(handle)
    if ent is None:
        return
    ent[1] -= 1
    if ent[1] <= 0:
        _lib.lib().kge_ipc_close(ent[0], 0)
        del _open_allocations[handle]


class PeerUnavailable(RuntimeError):
    """Raised on EVERY rank when any rank could not export its tensor or map a peer's (no peer access between two GPUs, memory
    that did not come from cudaMalloc, ...): the callers fall back to collectives together."""


class PeerMap:
    """One tensor per rank, each mapped into every process: `ptrs` is a device array of the `world` base addresses (this
    rank's own tensor included).  Collective: every rank of `group` constructs it at the same point of its program."""

    def __init__(self, local: torch.Tensor, rank: int, world: int, group=None):
        import torch.distributed as dist
        if not local.is_cuda or not local.is_contiguous():
            raise ValueError("expected a contiguous CUDA tensor")
        self.local, self.rank, self.world, self.group = local, int(rank), int(world), group
        L = _lib.lib()
        handle = (C.c_ubyte * 64)()
        off = C.c_uint64(0)
        problem = None
        try:
            check(L.kge_ipc_export(local.data_ptr(), handle, C.byref(off)))
        except Exception as e:                      # still take part in the collectives below
            problem = f"rank {rank}: {e}"
        mine = (bytes(handle), int(off.value), int(local.shape[0]), problem)
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
        self.rows = [rows for _, _, rows, _ in everyone]
        self._opened = []
        ptrs = []
        problem = next((p for _, _, _, p in everyone if p), None)
        if problem is None:
            try:
                for g, (h, o, _, _) in enumerate(everyone):
                    if g == rank:
                        ptrs.append(local.data_ptr())
                        continue
                    ptrs.append(_open(h) + o)
                    self._opened.append(h)
            except Exception as e:
                problem = f"rank {rank}: {e}"
        # every tensor is complete (and mapped everywhere) before anybody reads; the same collective tells every rank
        # whether all of them succeeded
        torch.cuda.synchronize(local.device)
        flag = torch.tensor([0 if problem is None else 1], dtype=torch.int32, device=local.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
        if int(flag.item()) != 0:
            self.close()
            raise PeerUnavailable(problem or "another rank could not map a peer's memory")
        self.ptrs = torch.tensor(ptrs, dtype=torch.int64, device=local.device)

    def close(self) -> None:
        """Unmaps the peers' tensors (nobody may still be reading this rank's)."""
        for h in self._opened:
            _close(h)
        self._opened = []


class PeerTable(PeerMap):
    def __init__(self, ent_local: torch.Tensor, n_ent: int, rank: int, world: int, group=None):
        super().__init__(ent_local, rank, world, group)
        self.ent_local, self.n_ent = ent_local, int(n_ent)
        self.rows_per_rank = (self.n_ent + world - 1) // world
        self.dim = ent_local.shape[1]
        self.dtype = DTYPES[{torch.float32: "f32", torch.bfloat16: "bf16"}[ent_local.dtype]]
        for g, rows in enumerate(self.rows):
            want = max(0, min(self.n_ent, (g + 1) * self.rows_per_rank) - g * self.rows_per_rank)
            if rows != want:
                raise ValueError(f"rank {g} holds {rows} rows, the partition gives it {want}")

    def gather(self, ids: torch.Tensor, n: int, n_dev: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out[i] = row ids[i] of the whole table for i < min(n, *n_dev), on the current stream."""
        if out is None:
            out = torch.empty((max(n, 1), self.dim), dtype=self.ent_local.dtype, device=self.ent_local.device)
        stream = torch.cuda.current_stream().cuda_stream
        check(_lib.lib().kge_gather_rows_peers(self.ptrs.data_ptr(), self.world, self.rows_per_rank, self.n_ent, self.dtype, self.dim,
                                               ids.data_ptr(), int(n), None if n_dev is None else n_dev.data_ptr(), out.data_ptr(), stream))
        return out
