"""Tensor-parallel decode (TP = 2) on two GPUs: column-parallel qkv / gate / up / lm_head, row-parallel
w_out / w_down with one all-reduce each — the library's one-shot all-reduce over NVLink peer memory (plain peer
stores, bounded waits, NVLS off) or ncclAllReduce. Every rank must produce the same greedy ids as the
single-GPU oracle, and the logits shards, concatenated, the oracle's logits (f32 mode 1e-4, W4A16 2e-2).
Skipped unless two CUDA devices are visible. Ranks are child processes; the NCCL id travels over gloo."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _worker(rank, world, port, mode, collective, q):
    """A rank that fails tells the parent through the queue and leaves with os._exit, so that the parent can end the
    other rank instead of waiting for a collective that will never complete."""
    try:
        _worker_body(rank, world, port, mode, collective, q)
    except BaseException as e:  # noqa: BLE001
        import traceback
        q.put(("error", rank, "".join(traceback.format_exception(type(e), e, e.__traceback__))))
        q.close()
        q.join_thread()
        os._exit(1)


def _worker_body(rank, world, port, mode, collective, q):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["GPTRS_TP_ALLREDUCE"] = collective
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    from gptrs_b200 import model as gm
    from oracle import models_ref as mr
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = mr.Cfg("ministral", n_layers=2, d_model=256, n_q=4, n_kv=2, hd=128, d_mlp=512, vocab=512, ctx=128, rot=128)
    params = mr.random_params(cfg, seed=11, std=0.05)
    ids = [gm.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    mc = gm.ModelConfig(gm.KIND_MINISTRAL, cfg.n_layers, cfg.d_model, cfg.n_q, cfg.n_kv, cfg.hd, cfg.d_mlp, cfg.vocab, cfg.ctx,
                        cfg.eps, cfg.theta, cfg.rot, weight_mode=mode, max_seqs=2, max_tokens=32, max_logit_rows=2,
                        kv_pages=32, max_pages_per_seq=8, tp_size=world, tp_rank=rank)
    m = gm.LoadedModel(mc, namespace=500 + mode)
    for name, w in params.items():
        m.load_param(name, w)
    m.init_tensor_parallel(ids[0])
    m.finalize()
    kind = m.tp_allreduce_kind()
    prompts = [[5, 17, 300, 41, 8, 99, 250], [77, 3]]
    shards, firsts = [], []
    for s, p in enumerate(prompts):
        lg, tok = m.prefill(s, p, want_logits=True)
        shards.append(lg)
        firsts.append(tok)
    gen = gm.Generator(m, firsts, use_graph=True)
    steps = [gen.step().tolist() for _ in range(5)]
    gathered = [None] * world
    dist.all_gather_object(gathered, (rank, shards, firsts, steps, kind))
    dist.barrier()
    m.close()
    dist.destroy_process_group()
    if rank == 0:
        q.put(gathered)


@pytest.mark.parametrize("collective", ["peer", "nccl"])
@pytest.mark.parametrize("mode", [0, 1], ids=["f32", "w4a16"])
def test_tp2_matches_single_gpu_oracle(mode, collective):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    from oracle import models_ref as mr
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, collective, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        gathered = q.get(timeout=300)
        if gathered and gathered[0] == "error":
            raise AssertionError(f"rank {gathered[1]} failed:\n{gathered[2]}")
        for p in procs:
            p.join(timeout=120)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    finally:
        # never leave a rank behind that spins inside a collective on a shared GPU
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=20)
            if p.is_alive():
                p.kill()
                p.join(timeout=20)
    cfg = mr.Cfg("ministral", n_layers=2, d_model=256, n_q=4, n_kv=2, hd=128, d_mlp=512, vocab=512, ctx=128, rot=128)
    params = mr.random_params(cfg, seed=11, std=0.05)
    if mode == 1:
        params = mr.quantised_params(cfg, params, "w4")
    tol = 1e-4 if mode == 0 else 2e-2
    gathered.sort(key=lambda t: t[0])
    assert gathered[0][2] == gathered[1][2] and gathered[0][3] == gathered[1][3]  # both ranks agree on every id
    want_kind = "nccl" if collective == "nccl" else "peer-store one-shot"
    assert gathered[0][4] == gathered[1][4] == want_kind, (gathered[0][4], gathered[1][4])
    prompts = [[5, 17, 300, 41, 8, 99, 250], [77, 3]]
    refs = [mr.RefModel(cfg, params) for _ in prompts]
    for s, p in enumerate(prompts):
        want = refs[s].forward(p)[-1]
        got = np.concatenate([gathered[r][1][s] for r in range(2)])
        assert np.max(np.abs(got - want)) <= tol
    cur = gathered[0][2]
    for step_ids in gathered[0][3]:
        want = np.stack([refs[s].forward([cur[s]])[-1] for s in range(2)])
        top2 = np.sort(want, axis=1)
        sure = (top2[:, -1] - top2[:, -2]) > 2 * tol
        assert np.array_equal(np.array(step_ids)[sure], np.argmax(want, axis=1)[sure])
        cur = step_ids
