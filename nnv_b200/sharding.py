"""Generator sharding of one star set over several GPUs (one process per GPU).

Index helpers shared by the host code and the tests, and the all-reduce hook
that ``nnvb_set_shard`` needs: a ctypes callback that sums a device buffer over
the ranks with ``torch.distributed`` (NCCL over NVLink), enqueued on the
engine's stream.

Layout rule (the same in the CUDA engine): predicate ``j`` of a query (0-based
position in its predicate order) lives on rank ``j % world``; the centre is
replicated; the ``c``-th column a ReLU layer appends (numbered over the whole
batch in query order, then ascending neuron index) lives on rank ``c % world``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L


def shard_count(n, rank, world):
    """Number of indices r in [0, n) with r % world == rank."""
    return (n - rank + world - 1) // world if n > rank else 0


def shard_positions(P, rank, world):
    """Predicate positions held by ``rank``."""
    return np.arange(rank, P, world, dtype=np.int64)


def local_new_columns(new_off, q, rank, world):
    """Global numbers c of the new columns of query q that ``rank`` holds, given the
    batch-wide exclusive scan ``new_off`` of the per-query crossing counts."""
    n0, n1 = int(new_off[q]), int(new_off[q + 1])
    first = n0 + ((rank - n0) % world)
    return np.arange(first, n1, world, dtype=np.int64)


class _DevicePtr:
    """Expose a raw device pointer through __cuda_array_interface__ so that torch can wrap it."""

    def __init__(self, ptr, count):
        self.__cuda_array_interface__ = {"shape": (int(count),), "typestr": "<f8", "data": (int(ptr), False),
                                         "version": 2}


def make_allreduce_hook(group=None):
    """Return (callback, keepalive) for nnvb_set_shard: sums the buffer over the ranks of
    ``group`` (default: the world group) on the stream the engine passes in."""
    import torch
    import torch.distributed as dist

    @L.ALLREDUCE_FN
    def hook(user, ptr, count, stream):
        try:
            t = torch.as_tensor(_DevicePtr(ptr, count), device="cuda")
            with torch.cuda.stream(torch.cuda.ExternalStream(int(stream))):
                dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
            return 0
        except Exception as exc:          # never let an exception cross the C boundary
            import sys
            print("nnv_b200 all-reduce hook failed: %r" % (exc,), file=sys.stderr)
            return 1

    return hook
