"""Host logic of the multi-GPU path: the request partitioner, and a world-size-2 run over gloo in
which each rank decodes its own shard and the generated ids are gathered on the host."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:  # spawned workers re-import this module without conftest
    sys.path.insert(0, str(ROOT))
import __graft_entry__ as _entry  # noqa: E402

_entry.load_package()
from gptrs_b200 import parallel  # noqa: E402


def test_partition_covers_every_request_once_and_balances():
    rng = np.random.default_rng(0)
    lens = rng.integers(256, 4097, size=512)
    for ranks in (1, 2, 4, 8):
        assign, cost = parallel.partition_requests(lens, 256, ranks)
        assert assign.min() >= 0 and assign.max() < ranks
        assert sum(len(parallel.shard_of(assign, r)) for r in range(ranks)) == 512
        per = 256 * lens + 256 * 255 // 2 + lens
        assert np.array_equal(cost, [per[assign == r].sum() for r in range(ranks)])
        assert cost.max() - cost.min() <= per.max()  # LPT bound
    a1, _ = parallel.partition_requests(lens, 256, 8)
    a2, _ = parallel.partition_requests(lens, 256, 8)
    assert np.array_equal(a1, a2)


def test_partition_edge_cases():
    a, c = parallel.partition_requests([], 10, 4)
    assert len(a) == 0 and c.tolist() == [0, 0, 0, 0]
    a, c = parallel.partition_requests([5], 0, 3)
    assert a.tolist() == [0]
    a, _ = parallel.partition_requests([7, 7, 7, 7], 1, 2)
    assert sorted(np.bincount(a, minlength=2).tolist()) == [2, 2]


class _FakeEngine:
    """Stand-in for LoadedModel + Generator: the next id is a function of the slot's own history only, as
    in a real engine, so any placement of a request (rank, wave, slot) must give the same ids."""

    def __init__(self):
        self.hist = {}

    def reset_sequence(self, slot):
        self.hist[slot] = []

    def prefill(self, slot, tokens, chunk=None):
        self.hist[slot] = [int(t) for t in tokens]
        return None, self._next(slot)

    def _next(self, slot):
        h = self.hist[slot]
        return (sum(h) * 31 + len(h)) % 1000


class _FakeGenerator:
    def __init__(self, model, first, use_graph=True):
        self.m, self.cur = model, [int(t) for t in first]

    def step(self, tokens_in=None):
        cur = self.cur if tokens_in is None else [int(t) for t in tokens_in]
        out = []
        for slot, t in enumerate(cur):
            self.m.hist[slot].append(t)
            out.append(self.m._next(slot))
        self.cur = out
        return np.array(out, dtype=np.int32)


def _fake_decode(prompt, steps: int):
    eng = _FakeEngine()
    _, first = eng.prefill(0, prompt)
    gen = _FakeGenerator(eng, [first])
    return [first] + [int(gen.step()[0]) for _ in range(steps)]


def _prompts(lens):
    rng = np.random.default_rng(5)
    return {i: rng.integers(0, 1000, size=int(n)).tolist() for i, n in enumerate(lens)}


def test_plan_waves_and_run_requests_on_a_stand_in_engine():
    lens = np.random.default_rng(2).integers(1, 60, size=23)
    waves = parallel.plan_waves(range(23), lens, 5)
    assert [len(w) for w in waves] == [5, 5, 5, 5, 3] and sorted(sum(waves, [])) == list(range(23))
    flat = [int(lens[r]) for w in waves for r in w]
    assert flat == sorted(flat, reverse=True)
    assert parallel.plan_waves([], lens, 4) == []
    with pytest.raises(ValueError):
        parallel.plan_waves([0], lens, 0)
    prompts = _prompts(lens)
    phases = []
    out = parallel.run_requests(_FakeEngine(), prompts, 6, 5, generator=_FakeGenerator,
                                on_phase=lambda name, wave, fn: (phases.append((name, len(wave))), fn()))
    assert phases == [(n, k) for k in (5, 5, 5, 5, 3) for n in ("prefill", "decode")]
    for r, p in prompts.items():
        assert out[r] == _fake_decode(p, 6) and len(out[r]) == 7


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    from gptrs_b200 import parallel as par
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lens = np.random.default_rng(1).integers(16, 200, size=37)
    assign, _ = par.partition_requests(lens, 8, world)
    mine = par.shard_of(assign, rank)
    prompts = _prompts(lens)
    local = par.run_requests(_FakeEngine(), {int(i): prompts[int(i)] for i in mine}, 8, 4, generator=_FakeGenerator)
    merged = par.gather_generated(local, world)
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, sorted(merged.keys()), merged[0], len(mine)))


def test_two_ranks_over_gloo_cover_the_request_set():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, keys, first, n_mine in res:
        assert keys == list(range(37))
        assert first == _fake_decode(_prompts(np.random.default_rng(1).integers(16, 200, size=37))[0], 8)
    assert sum(r[3] for r in res) == 37
