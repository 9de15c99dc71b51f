"""Row-wise functionals (norms, embedding, activations, softmax, sampler, f32 matmul) against
the oracle. Shapes follow the reference's torch-parity catalogue
(crates/gpt-rs-backend-tests/src/torch_parity/functional_ops.rs, matmul.rs, embedding_layer.rs);
tolerance atol 5e-4 / rtol 1e-4 as in torch_parity/common.rs:14-15."""
import numpy as np
import pytest
import torch

from gptrs_b200 import BackendError, ops
from oracle import functional_ref as fr
from oracle import quant_ref as qr

pytestmark = pytest.mark.gpu
ATOL, RTOL = 5e-4, 1e-4


def _d(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("rows,dim,eps", [(6, 4, 1e-5), (3, 1, 1e-5), (5, 13, 1e-3), (2, 3072, 1e-5), (1, 5000, 1e-1), (64, 768, 1e-5)])
def test_layer_norm(cuda, rows, dim, eps):
    rng = np.random.default_rng(rows * dim)
    x = rng.uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    g = rng.uniform(-1, 1, size=dim).astype(np.float32)
    b = rng.uniform(-1, 1, size=dim).astype(np.float32)
    out, mean, inv = ops.add_layer_norm(_d(x, cuda), _d(g, cuda), _d(b, cuda), eps, want_stats=True)
    want, _, wmean, winv = fr.layer_norm(x, g, b, eps)
    assert np.allclose(out.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    assert np.allclose(mean.cpu().numpy(), wmean[:, 0], rtol=RTOL, atol=ATOL)
    assert np.allclose(inv.cpu().numpy(), winv[:, 0], rtol=1e-3, atol=ATOL)


def test_layer_norm_constant_input(cuda):
    x = np.full((2, 16), 3.0, np.float32)
    g, b = np.ones(16, np.float32), np.zeros(16, np.float32)
    out = ops.add_layer_norm(_d(x, cuda), _d(g, cuda), _d(b, cuda), 1e-5)
    assert np.allclose(out.cpu().numpy(), 0.0, atol=ATOL)


@pytest.mark.parametrize("rows,dim", [(6, 4), (64, 3072), (3, 4100), (1, 1)])
def test_rms_norm_and_residual_add(cuda, rows, dim):
    rng = np.random.default_rng(rows + dim)
    x = rng.uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    d = rng.uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    g = rng.uniform(-1, 1, size=dim).astype(np.float32)
    want, _, winv = fr.rms_norm(x + d, g, 1e-5)
    h = _d(x, cuda)
    out, inv = ops.add_rms_norm(h, _d(g, cuda), 1e-5, delta=_d(d, cuda), out_dtype=torch.float32, want_inv_rms=True)
    assert np.allclose(h.cpu().numpy(), x + d)
    assert np.allclose(out.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    assert np.allclose(inv.cpu().numpy(), winv[:, 0], rtol=1e-4)
    # bf16 delta and bf16 output
    h = _d(x, cuda)
    db = qr.to_bf16(d)
    out = ops.add_rms_norm(h, _d(g, cuda), 1e-5, delta=_d(db, cuda).to(torch.bfloat16))
    want, _, _ = fr.rms_norm(x + db, g, 1e-5)
    assert np.allclose(out.float().cpu().numpy(), want, rtol=2 ** -7, atol=1e-3)


@pytest.mark.parametrize("vocab,dim,seq", [(64, 32, 16), (32, 8, 5), (32, 128, 8)])
def test_embedding_lookup_bit_exact(cuda, vocab, dim, seq):
    rng = np.random.default_rng(vocab + seq)
    w = rng.uniform(-1, 1, size=(vocab, dim)).astype(np.float32)
    ids = rng.integers(0, vocab, size=seq).astype(np.int32)
    ids[1] = ids[0]  # duplicates
    out, status = ops.embedding_lookup(_d(w, cuda), _d(ids, cuda))
    assert int(status.item()) == 0
    assert np.array_equal(out.cpu().numpy(), fr.embedding_lookup(w, ids))
    pw = rng.uniform(-1, 1, size=(40, dim)).astype(np.float32)
    pid = np.arange(seq, dtype=np.int32)
    out, _ = ops.embedding_lookup(_d(w, cuda), _d(ids, cuda), _d(pw, cuda), _d(pid, cuda))
    assert np.array_equal(out.cpu().numpy(), fr.embedding_lookup(w, ids) + pw[pid])


def test_embedding_out_of_range_is_flagged(cuda):
    w = np.ones((8, 4), np.float32)
    out, status = ops.embedding_lookup(_d(w, cuda), _d(np.array([1, 8, -1], np.int32), cuda))
    assert int(status.item()) == 2
    assert np.array_equal(out.cpu().numpy()[1:], np.zeros((2, 4), np.float32))


def test_activations_and_bias(cuda):
    rng = np.random.default_rng(7)
    for shape in [(256,), (4, 16), (2, 3, 8)]:
        x = rng.uniform(-1, 1, size=shape).astype(np.float32)
        u = rng.uniform(-1, 1, size=shape).astype(np.float32)
        assert np.allclose(ops.gelu(_d(x, cuda)).cpu().numpy(), fr.gelu(x), rtol=RTOL, atol=ATOL)
        assert np.allclose(ops.silu(_d(x, cuda)).cpu().numpy(), fr.silu(x), rtol=RTOL, atol=ATOL)
        assert np.allclose(ops.swiglu(_d(x, cuda), _d(u, cuda)).cpu().numpy(), fr.swiglu(x, u), rtol=RTOL, atol=ATOL)
    ext = np.array([-100, -20, -5, 0, 5, 20, 100], np.float32)
    assert np.allclose(ops.gelu(_d(ext, cuda)).cpu().numpy(), fr.gelu(ext), rtol=RTOL, atol=ATOL)
    assert np.allclose(ops.silu(_d(ext, cuda)).cpu().numpy(), fr.silu(ext), rtol=RTOL, atol=ATOL)
    x = rng.uniform(-1, 1, size=(2, 5, 8)).astype(np.float32)
    b = rng.uniform(-1, 1, size=8).astype(np.float32)
    assert np.allclose(ops.add_bias(_d(x, cuda), _d(b, cuda)).cpu().numpy(), x + b)


@pytest.mark.parametrize("shape", [(3, 2, 4), (5, 1), (4, 2), (3, 7), (2, 128), (2, 4, 32), (1, 5000)])
def test_softmax(cuda, shape):
    rng = np.random.default_rng(sum(shape))
    x = rng.uniform(-1, 1, size=shape).astype(np.float32)
    assert np.allclose(ops.softmax_last_dim(_d(x, cuda)).cpu().numpy(), fr.softmax_last_dim(x), rtol=RTOL, atol=ATOL)
    c = np.full(shape, 2.5, np.float32)
    assert np.allclose(ops.softmax_last_dim(_d(c, cuda)).cpu().numpy(), 1.0 / shape[-1], rtol=RTOL)
    e = np.array([[1000.0, -1000.0, 0.0, 999.0]], np.float32)
    assert np.allclose(ops.softmax_last_dim(_d(e, cuda)).cpu().numpy(), fr.softmax_last_dim(e), atol=ATOL)


def test_sampler_known_answers(cuda):
    # crates/gpt-rs-backend-triton/tests/decode_sampling.rs:11-20
    logits = _d(np.array([[-1.0, 0.1, 2.5, 0.4]], np.float32), cuda)
    assert ops.sample_decode_token(logits, 0.0) == 2
    # ties -> smallest index (docs/backend.md:270); last row is the one sampled
    l2 = _d(np.array([[9, 0, 0, 0], [1, 7, 7, 3]], np.float32), cuda)
    assert ops.sample_decode_token(l2, 0.0) == 1
    tok = ops.sample_decode_token(logits, 0.8, random_u=0.37)
    assert 0 <= tok < 4
    # a temperature without a draw from the caller is left to the host sampler (runtime/sampling.rs:94-97)
    assert ops.sample_decode_token(logits, 0.8) is None
    assert ops.sample_decode_token(logits, 0.8, random_u=float("nan")) is None
    rng = np.random.default_rng(0)
    big = rng.normal(0, 1, size=(64, 131072)).astype(np.float32)
    got = ops.sample_rows(_d(big, cuda)).cpu().numpy()
    assert np.array_equal(got, np.argmax(big, axis=1))
    lib = __import__("gptrs_b200").lib()
    assert lib.gptrs_cuda_supports_decode_sampling(0.0, 0) == 1
    assert lib.gptrs_cuda_supports_decode_sampling(0.7, 1) == 1


def test_top_k_sampler(cuda):
    """inference/sampler.rs:35-52: logits below the k-th largest are dropped (ties at the threshold stay), the
    draw is from the softmax of the rest. The draw itself is random in the reference, so parity is the kept
    set (exact) and the distribution (statistical)."""
    rng = np.random.default_rng(4)
    big = rng.normal(0, 2, size=(48, 131072)).astype(np.float32)
    big[1] = -np.abs(big[1]) - 5.0          # every logit negative
    big[2] = np.round(big[2])               # heavy ties, also at the threshold
    big[3, :] = 0.0                         # all equal: everything is kept
    big[3, 77] = 1.0
    d = _d(big, cuda)
    for k in (1, 2, 50, 1000):
        for seed in (0, 9):
            got = ops.sample_rows(d, temperature=1.3, seed=seed, top_k=k).cpu().numpy()
            kth = np.partition(big, big.shape[1] - k, axis=1)[:, big.shape[1] - k]
            assert (big[np.arange(48), got] >= kth).all(), (k, seed)
            if k == 1:
                assert np.array_equal(big[np.arange(48), got], big.max(axis=1))
    # k = 0 and k >= vocab filter nothing: the draw of the plain sampler for the same seed
    plain = ops.sample_rows(d, temperature=0.9, seed=5).cpu().numpy()
    for k in (0, 131072, 10 ** 6):
        assert np.array_equal(ops.sample_rows(d, temperature=0.9, seed=5, top_k=k).cpu().numpy(), plain)
    assert np.array_equal(ops.sample_rows(d, temperature=0.0, seed=5, top_k=7).cpu().numpy(), np.argmax(big, axis=1))  # greedy ignores k
    # distribution over the kept set: 8192 rows with the same logits draw independently (the hash mixes the row)
    base = np.array([2.0, -1.0, 0.5, 1.5, 1.5, -3.0, 0.0, 1.0] + [-4.0] * 56, np.float32)
    rows = np.tile(base, (8192, 1))
    temp, k = 0.7, 4
    got = ops.sample_rows(_d(rows, cuda), temperature=temp, seed=123, top_k=k).cpu().numpy()
    keep = base >= np.sort(base)[-k]
    assert keep.sum() == 4 and keep[got].all()
    want = np.where(keep, np.exp((base - base.max()) / temp), 0.0)
    want /= want.sum()
    freq = np.bincount(got, minlength=64) / len(got)
    assert np.abs(freq - want).max() < 0.02, (freq[:8], want[:8])
    tok = ops.sample_decode_token(_d(np.array([[0.0, 5.0, 4.9, -1.0]], np.float32), cuda), 1.0, random_u=0.5, top_k=2)
    assert tok in (1, 2)


MATMUL_SHAPES = [(1, 1, 1), (1, 5, 3), (4, 5, 1), (7, 13, 9), (33, 65, 31), (8, 1, 8), (1, 16, 17), (64, 128, 32),
                 (1, 768, 2304), (1, 3072, 768), (1, 768, 50257), (32, 768, 3072), (3, 100, 257)]


@pytest.mark.parametrize("m,k,n", MATMUL_SHAPES)
def test_matmul_f32(cuda, m, k, n):
    rng = np.random.default_rng(10 + m + k + n)
    a = rng.uniform(-1, 1, size=(m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, size=(k, n)).astype(np.float32)
    got = ops.matmul_f32(_d(a, cuda), _d(b, cuda)).cpu().numpy()
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    assert np.allclose(got, want, rtol=RTOL, atol=ATOL)


def test_matmul_f32_smoke_known_answer(cuda):
    # crates/gpt-rs-backend-tests/src/smoke.rs:12-24
    a = _d(np.array([[1, 2], [3, 4]], np.float32), cuda)
    b = _d(np.array([[5, 6], [7, 8]], np.float32), cuda)
    assert ops.matmul_f32(a, b).cpu().numpy().ravel().tolist() == [19.0, 22.0, 43.0, 50.0]


def test_matmul_f32_epilogue(cuda):
    rng = np.random.default_rng(3)
    m, k, n = 5, 64, 200
    a = rng.uniform(-1, 1, size=(m, k)).astype(np.float32)
    w = rng.uniform(-1, 1, size=(k, n)).astype(np.float32)
    bias = rng.uniform(-1, 1, size=n).astype(np.float32)
    res = rng.uniform(-1, 1, size=(m, n)).astype(np.float32)
    got = ops.matmul_f32(_d(a, cuda), _d(w, cuda), _d(bias, cuda), _d(res, cuda), gelu=True).cpu().numpy()
    want = fr.gelu(fr.linear(a, w, bias)) + res
    assert np.allclose(got, want, rtol=RTOL, atol=ATOL)
