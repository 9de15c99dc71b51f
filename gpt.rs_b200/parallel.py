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


def plan_waves(request_ids, prompt_lens, max_batch: int):
    """Cuts one rank's shard into waves of at most `max_batch` requests, longest prompts first, so the KV
    pages a wave needs shrink from wave to wave and the first one shows whether the pool is large enough.
    Every request decodes the same number of steps, so a wave's slots finish together and no slot idles."""
    if max_batch <= 0:
        raise ValueError("max_batch must be positive")
    ids = [int(r) for r in request_ids]
    ids.sort(key=lambda r: (-int(prompt_lens[r]), r))
    return [ids[i:i + max_batch] for i in range(0, len(ids), max_batch)]


def run_requests(model, prompts: dict, decode_steps: int, max_batch: int, prefill_chunk: int | None = None, on_phase=None,
                 generator=None):
    """Serves {request index: prompt ids} on one engine in waves (see plan_waves): prefill every request of a
    wave into its slot, then `decode_steps` greedy steps over the wave's slots. Returns {request index:
    [first id from the prompt's last row, then the decode_steps generated ids]}. `on_phase(name, wave, fn)`,
    when given, runs each phase through the caller (the bench wraps it in timers); `generator` replaces the
    engine's Generator class (host-logic tests pass a stand-in)."""
    if generator is None:
        from .model import Generator as generator
    lens = {r: len(p) for r, p in prompts.items()}
    call = on_phase or (lambda name, wave, fn: fn())
    out = {}
    for wave in plan_waves(prompts.keys(), lens, max_batch):
        first = []

        def prefill():
            for slot in range(len(wave)):
                model.reset_sequence(slot)
            if hasattr(model, "prefill_many"):  # rows of several prompts packed into full passes
                first.extend(model.prefill_many(list(range(len(wave))), [prompts[r] for r in wave], chunk=prefill_chunk))
            else:
                first.extend(model.prefill(slot, prompts[r], chunk=prefill_chunk)[1] for slot, r in enumerate(wave))

        steps = []

        def decode():
            gen = generator(model, first, use_graph=True)
            cur = None
            for _ in range(decode_steps):
                cur = gen.step(tokens_in=cur)
                steps.append(cur)

        call("prefill", wave, prefill)
        call("decode", wave, decode)
        for slot, r in enumerate(wave):
            out[r] = [int(first[slot])] + [int(s[slot]) for s in steps]
    return out
