"""The failure path of a device-side bounded wait, driven to its limit without faulting anything: a test switch
withholds the first activation tile of the tensor-core matmul, so the waits that depend on it run out after a small
number of polls. The kernel must record its error code, free its tensor memory and return; the host must see the
code (functional level) or an Execution error (engine level); and the next ordinary launch must be correct."""
import numpy as np
import pytest
import torch

from gptrs_b200 import BackendError, check, lib, ops
from gptrs_b200 import model as gm
from oracle import models_ref as mr
from oracle import quant_ref as qr

pytestmark = pytest.mark.gpu


@pytest.fixture
def starved():
    """Switches the starvation on for the body of a test and always off again."""
    def on(limit=2000):
        check(lib().gptrs_cuda_debug_matmul_fault(1, limit))
    yield on
    check(lib().gptrs_cuda_debug_matmul_fault(0, 0))


def test_matmul_wait_runs_out_sets_status_and_recovers(cuda, starved):
    rng = np.random.default_rng(0)
    m, n, k = 64, 512, 1024
    p = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    s = np.exp(rng.normal(-5.0, 0.5, size=(n, k // 128))).astype(np.float16)
    x = qr.to_bf16(rng.normal(0, 1, size=(m, k)).astype(np.float32))
    want = qr.quant_matmul(x, qr.dequant_w4(p, s))
    packed = ops.w4a16_repack(torch.from_numpy(p).to(cuda), torch.from_numpy(s).to(cuda), n, k)
    xd = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
    tol = 4e-3 * max(1.0, float(np.abs(want).max()))
    assert np.abs(ops.quant_matmul_w4a16(xd, packed, m, n, k, out_f32=True).cpu().numpy() - want).max() <= tol
    assert ops.matmul_status() == 0
    starved()
    ops.quant_matmul_w4a16(xd, packed, m, n, k, out_f32=True)   # returns; the result is unspecified
    torch.cuda.synchronize()
    assert ops.matmul_status() == 3          # a bounded wait gave up (reading the word clears it)
    check(lib().gptrs_cuda_debug_matmul_fault(0, 0))
    assert ops.matmul_status() == 0
    assert np.abs(ops.quant_matmul_w4a16(xd, packed, m, n, k, out_f32=True).cpu().numpy() - want).max() <= tol
    assert ops.matmul_status() == 0


def test_engine_reports_a_matmul_wait_that_ran_out(cuda, starved):
    cfg = mr.Cfg("ministral", n_layers=2, d_model=256, n_q=4, n_kv=2, hd=128, d_mlp=512, vocab=512, ctx=256, rot=128, theta=1e6)
    params = mr.random_params(cfg, seed=5, std=0.05)
    n_seq = 20   # more than 16 rows: the tensor-core matmuls
    mc = gm.ModelConfig(gm.KIND_MINISTRAL, cfg.n_layers, cfg.d_model, cfg.n_q, cfg.n_kv, cfg.hd, cfg.d_mlp, cfg.vocab, cfg.ctx,
                        cfg.eps, cfg.theta, cfg.rot, weight_mode=gm.MODE_W4A16, max_seqs=n_seq, max_tokens=64, max_logit_rows=n_seq,
                        kv_pages=n_seq * 4 + 4, max_pages_per_seq=4)
    m = gm.LoadedModel(mc, namespace=8800)
    for name, w in params.items():
        m.load_param(name, w)
    m.finalize()
    rng = np.random.default_rng(6)
    first = [m.prefill(s, rng.integers(0, cfg.vocab, size=5).tolist())[1] for s in range(n_seq)]
    gen = gm.Generator(m, first, use_graph=False)
    good = gen.step()
    assert good.shape == (n_seq,)
    starved()
    with pytest.raises(BackendError) as e:
        gen.step()
    assert e.value.kind == "Execution" and "matmul" in str(e.value)
    check(lib().gptrs_cuda_debug_matmul_fault(0, 0))
    after = gen.step()   # the context is intact: the next step runs and samples ids in range
    assert after.shape == (n_seq,) and int(after.min()) >= 0 and int(after.max()) < cfg.vocab


def test_prefill_attention_wait_runs_out_sets_status_and_recovers(cuda):
    """The tensor-core prefill attention with the K pages of every CTA's first key block withheld: the MMA warp's wait for
    them, then the softmax warps' waits for S and the page warps' waits for a free stage run out after 300 parked polls,
    code 3 lands in the caller's status word, the kernel frees its tensor memory and returns; the next launch is correct."""
    n_q, n_kv, l = 8, 2, 400   # 4 key blocks: every kind of wait is reached
    pages = (l + 15) // 16
    g = torch.Generator(device="cpu").manual_seed(5)
    pool = (torch.randn(pages * n_kv * 2 * 16 * 128, generator=g) * 0.5).to(torch.bfloat16).to(cuda).view(torch.uint8)
    table = torch.arange(pages, dtype=torch.int32, device=cuda).view(1, pages)
    q = torch.randn(l, n_q, 128, generator=g).to(torch.bfloat16).to(cuda)
    slot = torch.zeros(l, dtype=torch.int32, device=cuda)
    ctx = torch.arange(1, l + 1, dtype=torch.int32, device=cuda)
    want, st = ops.paged_attention_decode(q, pool, table, slot, ctx, n_q, n_kv, l)
    good, st0 = ops.paged_attention_decode(q, pool, table, slot, ctx, n_q, n_kv, l, prefill="tc")
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and int(st0.item()) == 0
    check(lib().gptrs_cuda_debug_prefill_tc_fault(1, 300))
    try:
        _, st1 = ops.paged_attention_decode(q, pool, table, slot, ctx, n_q, n_kv, l, prefill="tc")   # returns; the result is unspecified
        torch.cuda.synchronize()
        assert int(st1.item()) == 3
    finally:
        check(lib().gptrs_cuda_debug_prefill_tc_fault(0, 0))
    again, st2 = ops.paged_attention_decode(q, pool, table, slot, ctx, n_q, n_kv, l, prefill="tc")
    torch.cuda.synchronize()
    assert int(st2.item()) == 0
    assert torch.equal(again, good)
    a, b = again.float().cpu().numpy(), want.float().cpu().numpy()
    assert np.all(np.abs(a - b) <= 8e-3 * np.maximum(1.0, np.abs(b)))
