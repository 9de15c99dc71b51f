"""Two host threads drive two models at the same time (the backend trait is Send + Sync): launch options are per thread,
cached state is per device, every model has its own stream. The ids of the concurrent run must equal those of the same
two models run one after the other. Also covers the backend object (create / make_current / destroy)."""
import ctypes
import threading

import numpy as np
import pytest

from gptrs_b200 import check, lib
from gptrs_b200 import model as gm
from oracle import models_ref as mr

pytestmark = pytest.mark.gpu

CFG = mr.Cfg("ministral", n_layers=2, d_model=256, n_q=4, n_kv=2, hd=128, d_mlp=512, vocab=512, ctx=256, rot=128, theta=1e6)
N_SEQ, STEPS = 20, 24   # more than 16 rows: the tensor-core matmuls, decode under a CUDA graph with programmatic launch


def _model(seed, namespace):
    params = mr.random_params(CFG, seed=seed, std=0.05)
    mc = gm.ModelConfig(gm.KIND_MINISTRAL, CFG.n_layers, CFG.d_model, CFG.n_q, CFG.n_kv, CFG.hd, CFG.d_mlp, CFG.vocab, CFG.ctx,
                        CFG.eps, CFG.theta, CFG.rot, weight_mode=gm.MODE_W4A16, max_seqs=N_SEQ, max_tokens=64, max_logit_rows=N_SEQ,
                        kv_pages=N_SEQ * 6 + 4, max_pages_per_seq=6, use_pdl=1)
    m = gm.LoadedModel(mc, namespace=namespace)
    for name, w in params.items():
        m.load_param(name, w)
    m.finalize()
    return m


def _generate(m, seed, out, key, backend=None):
    if backend is not None:
        check(lib().gptrs_cuda_backend_make_current(backend))
    rng = np.random.default_rng(seed)
    first = [m.prefill(s, rng.integers(0, CFG.vocab, size=int(rng.integers(3, 30))).tolist())[1] for s in range(N_SEQ)]
    gen = gm.Generator(m, first, use_graph=True)
    ids = [list(first)]
    for _ in range(STEPS):
        ids.append(gen.step().tolist())
    out[key] = ids


def test_two_threads_two_models(cuda):
    backend = ctypes.c_void_p()
    check(lib().gptrs_cuda_create(0, ctypes.byref(backend)))
    assert lib().gptrs_cuda_backend_device(backend) == 0 and lib().gptrs_cuda_backend_stream(backend)
    serial, parallel = {}, {}
    a, b = _model(21, 9100), _model(22, 9101)
    _generate(a, 1, serial, "a")
    _generate(b, 2, serial, "b")
    a2, b2 = _model(21, 9100), _model(22, 9101)   # same stable ids: the quantised layouts come from the memo
    assert a2.stats()["memo_hits"] > 0
    ta = threading.Thread(target=_generate, args=(a2, 1, parallel, "a", backend))
    tb = threading.Thread(target=_generate, args=(b2, 2, parallel, "b", backend))
    ta.start(); tb.start(); ta.join(); tb.join()
    assert parallel["a"] == serial["a"] and parallel["b"] == serial["b"]
    assert serial["a"] != serial["b"]
    check(lib().gptrs_cuda_destroy(backend))
    bad = ctypes.c_void_p()
    assert lib().gptrs_cuda_create(99, ctypes.byref(bad)) != 0
