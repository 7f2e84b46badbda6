"""Feature table sharded by node-id range over the GPUs of a job (one process per GPU).

The reference keeps features that do not fit one device off the GPU and fetches remote rows through an MPI RPC
(core/ntsPeerRPC.hpp:44-46).  Here every rank holds the rows of a contiguous id range in its own HBM
(owner = id // shard_rows), maps the other ranks' shards once through CUDA inter-process handles, and the library
reads remote rows with plain loads over NVLink while it stages a batch's uncached rows (nb_gcn_config.d_feat_shards).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _lib


def shard_rows_for(num_vertices: int, num_shards: int) -> int:
    return (int(num_vertices) + num_shards - 1) // num_shards


class ShardedFeatureTable:
    """`table`: int64 device tensor of num_shards row pointers (what d_feat_shards points to); shard k holds the rows
    of vertices [k * shard_rows, (k + 1) * shard_rows) with pitch `ld` floats."""

    def __init__(self, table: torch.Tensor, num_shards: int, shard_rows: int, ld: int, width: int, owned=None,
                 opened: Optional[List[int]] = None, keep=None):
        self.table, self.num_shards, self.shard_rows, self.ld, self.width = table, num_shards, shard_rows, ld, width
        self._owned = owned        # address of the shard this process allocated with nb_shard_alloc, or None
        self._opened = opened or []
        self._keep = keep          # tensors that back the shards of a single-process table

    @classmethod
    def from_local_parts(cls, parts: Sequence[torch.Tensor], shard_rows: int) -> "ShardedFeatureTable":
        """All shards in this process's own memory (tests, and a single GPU that holds the whole table in pieces)."""
        assert all(p.is_cuda and p.dtype == torch.float32 and p.dim() == 2 and p.stride(1) == 1 for p in parts)
        ld = parts[0].stride(0)
        assert all(p.stride(0) == ld for p in parts)
        table = torch.tensor([p.data_ptr() for p in parts], dtype=torch.int64, device=parts[0].device)
        return cls(table, len(parts), int(shard_rows), ld, parts[0].size(1), keep=list(parts))

    @classmethod
    def from_rank_shard(cls, local_rows: torch.Tensor, num_vertices: int, rank: int, world_size: int,
                        device) -> "ShardedFeatureTable":
        """Every rank passes the rows of its own id range (a host or device float32 tensor [rows, F], rows <=
        shard_rows); handles are exchanged with torch.distributed and each peer's shard is mapped once."""
        import torch.distributed as dist
        rows_per = shard_rows_for(num_vertices, world_size)
        F = int(local_rows.size(1))
        assert local_rows.dtype == torch.float32 and local_rows.is_contiguous() and local_rows.size(0) <= rows_per
        own = C.c_void_p()
        _lib.call("nb_shard_alloc", C.byref(own), rows_per * F * 4)
        if local_rows.numel():
            _lib.call("nb_shard_upload", own, C.c_void_p(local_rows.data_ptr()), local_rows.numel() * 4)
        handle = C.create_string_buffer(64)
        _lib.call("nb_shard_export", own, handle)
        mine = torch.tensor(list(handle.raw), dtype=torch.uint8, device=device)
        everyone = [torch.empty(64, dtype=torch.uint8, device=device) for _ in range(world_size)]
        dist.all_gather(everyone, mine)
        pointers, opened = [], []
        for r in range(world_size):
            if r == rank:
                pointers.append(own.value)
                continue
            p = C.c_void_p()
            _lib.call("nb_shard_open", bytes(everyone[r].cpu().tolist()), C.byref(p))
            pointers.append(p.value)
            opened.append(p.value)
        table = torch.tensor(pointers, dtype=torch.int64, device=device)
        dist.barrier()     # every shard is uploaded and mapped before anyone reads
        return cls(table, world_size, rows_per, F, F, owned=own.value, opened=opened)

    def close(self, barrier: bool = True):
        """Unmaps the peers' shards, then (after a barrier, so that no peer still reads it) frees this rank's own."""
        for p in self._opened:
            _lib.call("nb_shard_close", C.c_void_p(p))
        self._opened = []
        if self._owned is not None:
            if barrier:
                import torch.distributed as dist
                if dist.is_initialized():
                    torch.cuda.synchronize()
                    dist.barrier()
            _lib.call("nb_shard_free", C.c_void_p(self._owned))
            self._owned = None
