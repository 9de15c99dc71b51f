"""Host logic of the multi-GPU path: the request partitioner, and a world-size-2 run over gloo in
which each rank decodes its own shard and the generated ids are gathered on the host."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
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


def _fake_decode(request_index: int, prompt_len: int, steps: int):
    return [(request_index * 31 + prompt_len + t) % 1000 for t in range(steps)]


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
    local = {int(i): _fake_decode(int(i), int(lens[i]), 8) for i in mine}
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
        assert first == _fake_decode(0, int(np.random.default_rng(1).integers(16, 200, size=37)[0]), 8)
    assert sum(r[3] for r in res) == 37
