"""Data-parallel decode across the GPUs of one box: requests are independent, so each rank (one
process per GPU, torch.distributed for rendezvous only) runs its own engine on its shard; the only
exchange is the host-side gather of generated ids."""
from __future__ import annotations

import ctypes

import numpy as np

from . import check, lib


def partition_requests(prompt_lens, decode_steps: int, n_ranks: int):
    """Returns (assignment [n] int32, rank_cost [n_ranks] int64); same result on every rank."""
    lens = np.ascontiguousarray(prompt_lens, dtype=np.int64)
    assign = np.empty(len(lens), dtype=np.int32)
    cost = np.zeros(n_ranks, dtype=np.int64)
    check(lib().gptrs_cuda_partition_requests(lens.ctypes.data if len(lens) else None, len(lens), decode_steps, n_ranks,
                                              assign.ctypes.data if len(lens) else None, cost.ctypes.data))
    return assign, cost


def shard_of(assignment, rank: int):
    """Indices of the requests a rank owns, in request order."""
    return np.nonzero(np.asarray(assignment) == rank)[0]


def gather_generated(local_ids: dict, world_size: int):
    """Gathers {request index: generated ids} from every rank on the host (gloo or nccl group)."""
    import torch.distributed as dist
    if world_size == 1 or not dist.is_initialized():
        return dict(local_ids)
    parts = [None] * world_size
    dist.all_gather_object(parts, local_ids)
    out = {}
    for p in parts:
        out.update(p)
    return out
