"""Parity of the W4A16 / W8A16 dequant-fused matmul kernels with the CPU oracle (through the
C ABI). Integer unpacking must be bit-exact; outputs are compared at max-abs 2e-2 relative to
the output scale (bf16 output rounding), the tolerance the bf16 decode path is held to."""
import numpy as np
import pytest
import torch

from gptrs_b200 import ops
from oracle import quant_ref as qr

pytestmark = pytest.mark.gpu


def _scales(rng, shape):
    return np.exp(rng.normal(-5.0, 0.5, size=shape)).astype(np.float16)


def _w4_case(rng, n, k):
    q = rng.integers(-8, 8, size=(n, k), dtype=np.int8)
    return qr.pack_int4(q), _scales(rng, (n, k // 128))


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("n,k", [(16, 128), (48, 384), (256, 1024), (3072, 3072)])
def test_w4_repack_unpack_bit_exact(cuda, n, k):
    rng = np.random.default_rng(n + k)
    p, s = _w4_case(rng, n, k)
    for inter in (False, True) if n % 32 == 0 else (False,):
        packed = ops.w4a16_repack(_dev(p, cuda), _dev(s, cuda), n, k, inter)
        for unpack in (ops.w4a16_unpack, ops.w4a16_unpack_rows):  # both layouts held by the buffer
            q2, s2 = unpack(packed, n, k, inter)
            assert np.array_equal(q2.cpu().numpy(), p)
            assert np.array_equal(s2.cpu().numpy().view(np.uint16), s.view(np.uint16))


@pytest.mark.parametrize("n,k", [(16, 128), (48, 384), (3072, 3072)])
def test_w8_repack_unpack_bit_exact(cuda, n, k):
    rng = np.random.default_rng(n * 3 + k)
    q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = _scales(rng, (n,))
    for inter in (False, True) if n % 32 == 0 else (False,):
        packed = ops.w8a16_repack(_dev(q, cuda), _dev(s, cuda), n, k, inter)
        for unpack in (ops.w8a16_unpack, ops.w8a16_unpack_rows):  # both layouts held by the buffer
            q2, s2 = unpack(packed, n, k, inter)
            assert np.array_equal(q2.cpu().numpy(), q)
            assert np.array_equal(s2.cpu().numpy().view(np.uint16), s.view(np.uint16))


@pytest.mark.parametrize("transposed", [False, True])
def test_quantize_kernels_bit_exact(cuda, transposed):
    rng = np.random.default_rng(11)
    n, k = 80, 512
    w_nk = rng.normal(0, 0.02, size=(n, k)).astype(np.float32)
    w_nk[3, 128:256] = 0.0  # an all-zero group
    src = w_nk if transposed else np.ascontiguousarray(w_nk.T)
    q4, s4 = ops.quantize_w4(_dev(src, cuda), transposed)
    p_ref, s_ref = qr.quantize_w4(w_nk)
    assert np.array_equal(s4.cpu().numpy().view(np.uint16), s_ref.view(np.uint16))
    assert np.array_equal(q4.cpu().numpy(), p_ref)
    q8, s8 = ops.quantize_w8(_dev(src, cuda), transposed)
    q_ref, s8_ref = qr.quantize_w8(w_nk)
    assert np.array_equal(s8.cpu().numpy().view(np.uint16), s8_ref.view(np.uint16))
    assert np.array_equal(q8.cpu().numpy(), q_ref)


def _check(got, want, tol=2e-2):
    scale = max(1.0, float(np.max(np.abs(want))))
    err = float(np.max(np.abs(got - want)))
    assert err <= tol * scale, f"max-abs err {err} (scale {scale})"


SHAPES = [
    (1, 16, 128), (1, 3072, 3072), (3, 48, 384), (8, 256, 1024), (9, 144, 640), (16, 3072, 3072),
    (17, 272, 256), (33, 512, 1536), (64, 3072, 3072), (64, 9216, 3072), (1, 9216, 3072),
    (65, 256, 512), (200, 384, 1280), (256, 3072, 3072),
]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_w4a16_matmul_matches_oracle(cuda, m, n, k):
    rng = np.random.default_rng(m * 7 + n + k)
    p, s = _w4_case(rng, n, k)
    x = qr.to_bf16(rng.normal(0, 1, size=(m, k)).astype(np.float32))
    want = qr.quant_matmul(x, qr.dequant_w4(p, s))
    packed = ops.w4a16_repack(_dev(p, cuda), _dev(s, cuda), n, k)
    xd = _dev(x, cuda).to(torch.bfloat16)
    y = ops.quant_matmul_w4a16(xd, packed, m, n, k)
    _check(y.float().cpu().numpy(), qr.to_bf16(want))
    y32 = ops.quant_matmul_w4a16(xd, packed, m, n, k, out_f32=True)
    if m <= 16:
        # exact dequantisation, f32 output: only accumulation-order noise remains
        assert np.allclose(y32.cpu().numpy(), want, rtol=1e-4, atol=1e-4 * max(1.0, np.abs(want).max()))
    else:
        # tensor-core path: weights are rounded to bf16 once (relative 2^-9 per weight)
        assert np.max(np.abs(y32.cpu().numpy() - want)) <= 4e-3 * max(1.0, np.abs(want).max())
    assert ops.matmul_status() == 0


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_w8a16_matmul_matches_oracle(cuda, m, n, k):
    rng = np.random.default_rng(m * 5 + n + k)
    q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = _scales(rng, (n,))
    x = qr.to_bf16(rng.normal(0, 1, size=(m, k)).astype(np.float32))
    want = qr.quant_matmul(x, qr.dequant_w8(q, s))
    packed = ops.w8a16_repack(_dev(q, cuda), _dev(s, cuda), n, k)
    xd = _dev(x, cuda).to(torch.bfloat16)
    y32 = ops.quant_matmul_w8a16(xd, packed, m, n, k, out_f32=True)
    assert np.allclose(y32.cpu().numpy(), want, rtol=1e-4, atol=1e-4 * max(1.0, np.abs(want).max()))
    y = ops.quant_matmul_w8a16(xd, packed, m, n, k)
    _check(y.float().cpu().numpy(), qr.to_bf16(want))


def test_w4a16_epilogues(cuda):
    rng = np.random.default_rng(99)
    m, n, k = 5, 256, 384
    p, s = _w4_case(rng, n, k)
    x = qr.to_bf16(rng.normal(0, 1, size=(m, k)).astype(np.float32))
    base = qr.quant_matmul(x, qr.dequant_w4(p, s))
    xd = _dev(x, cuda).to(torch.bfloat16)
    packed = ops.w4a16_repack(_dev(p, cuda), _dev(s, cuda), n, k)
    bias = rng.normal(0, 1, size=n).astype(np.float32)
    res = rng.normal(0, 1, size=(m, n)).astype(np.float32)
    y = ops.quant_matmul_w4a16(xd, packed, m, n, k, out_f32=True, bias=_dev(bias, cuda), residual=_dev(res, cuda))
    want = base + bias[None, :] + res
    assert np.allclose(y.cpu().numpy(), want, rtol=1e-4, atol=1e-3)
    # SwiGLU: rows [0, n/2) are gate, [n/2, n) are up
    from oracle import functional_ref as fr
    packed_gu = ops.w4a16_repack(_dev(p, cuda), _dev(s, cuda), n, k, True)
    y = ops.quant_matmul_w4a16(xd, packed_gu, m, n, k, out_f32=True, swiglu=True)
    want = fr.swiglu(base[:, : n // 2], base[:, n // 2:])
    assert y.shape == (m, n // 2)
    assert np.allclose(y.cpu().numpy(), want, rtol=1e-3, atol=1e-3 * max(1.0, np.abs(want).max()))
    # same epilogue on the W8 kernel
    q8 = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s8 = _scales(rng, (n,))
    base8 = qr.quant_matmul(x, qr.dequant_w8(q8, s8))
    packed8 = ops.w8a16_repack(_dev(q8, cuda), _dev(s8, cuda), n, k, True)
    y8 = ops.quant_matmul_w8a16(xd, packed8, m, n, k, out_f32=True, swiglu=True)
    want8 = fr.swiglu(base8[:, : n // 2], base8[:, n // 2:])
    assert np.allclose(y8.cpu().numpy(), want8, rtol=1e-3, atol=1e-3 * max(1.0, np.abs(want8).max()))


@pytest.mark.parametrize("m,swiglu", [(40, False), (64, True), (130, False)])
def test_folded_residual_rmsnorm(cuda, m, swiglu):
    """The projection that updates the residual stream also emits bf16(y * gamma) and per-tile sums of y^2; the next
    projection scales its rows by 1 / rms(y). Together they equal matmul -> add -> rms_norm -> matmul."""
    rng = np.random.default_rng(m)
    d, k1, n2, eps = 384, 256, 512, 1e-5
    p1, s1 = _w4_case(rng, d, k1)
    p2, s2 = _w4_case(rng, n2, d)
    x1 = qr.to_bf16(rng.normal(0, 1, size=(m, k1)).astype(np.float32))
    hidden = rng.normal(0, 1, size=(m, d)).astype(np.float32)
    gamma = (1 + 0.1 * rng.normal(size=d)).astype(np.float32)
    w1 = ops.w4a16_repack(_dev(p1, cuda), _dev(s1, cuda), d, k1)
    w2 = ops.w4a16_repack(_dev(p2, cuda), _dev(s2, cuda), n2, d, swiglu)
    hid_d = _dev(hidden, cuda)
    x_next = torch.empty((m, d), dtype=torch.bfloat16, device=cuda)
    sumsq = torch.zeros((d // 128, m), dtype=torch.float32, device=cuda)
    ops.quant_matmul_w4a16(_dev(x1, cuda).to(torch.bfloat16), w1, m, d, k1, out=hid_d, out_f32=True, residual=hid_d,
                           norm_out=(_dev(gamma, cuda), x_next, sumsq))
    y2 = ops.quant_matmul_w4a16(x_next, w2, m, n2, d, out_f32=True, swiglu=swiglu, norm_in=(sumsq, d, eps))
    torch.cuda.synchronize()
    h_gpu = hid_d.cpu().numpy()
    h_ref = hidden + qr.quant_matmul(x1, qr.dequant_w4(p1, s1))
    assert np.allclose(h_gpu, h_ref, rtol=0, atol=4e-3 * np.abs(h_ref).max())
    # by-products are exact functions of the stored residual stream
    assert np.array_equal(x_next.float().cpu().numpy(), qr.to_bf16(h_gpu * gamma))
    assert np.allclose(sumsq.cpu().numpy().sum(axis=0), (h_gpu.astype(np.float64) ** 2).sum(axis=1), rtol=1e-5)
    # the pair against norm-then-matmul on the same residual stream
    rstd = 1.0 / np.sqrt((h_gpu.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + eps)
    xn = qr.to_bf16((h_gpu * rstd * gamma).astype(np.float32))
    want = qr.quant_matmul(xn, qr.dequant_w4(p2, s2))
    if swiglu:
        gate, up = want[:, :n2 // 2], want[:, n2 // 2:]
        want = gate / (1 + np.exp(-gate)) * up
    got = y2.cpu().numpy()
    assert np.allclose(got, want, rtol=0, atol=8e-3 * np.abs(want).max()), np.abs(got - want).max() / np.abs(want).max()


def test_folded_rope_kv_append(cuda):
    """The qkv projection with the RoPE + KV-append epilogue leaves the same rotated Q and the same pool bytes as
    matmul -> gptrs_cuda_rope_kv_append (to one bf16 ulp: the two kernels may contract a*c - b*s differently)."""
    from oracle import functional_ref as fr
    rng = np.random.default_rng(21)
    m, n_q, n_kv, k = 40, 4, 2, 256
    n = (n_q + 2 * n_kv) * 128
    p, s = _w4_case(rng, n, k)
    w = ops.w4a16_repack(_dev(p, cuda), _dev(s, cuda), n, k)
    x = _dev(qr.to_bf16(rng.normal(0, 1, size=(m, k)).astype(np.float32)), cuda).to(torch.bfloat16)
    # two sequences: 25 tokens at positions 3..27 of slot 0 and 15 tokens at positions 0..14 of slot 1
    pos = torch.tensor(list(range(3, 28)) + list(range(15)), dtype=torch.int32, device=cuda)
    slot = torch.tensor([0] * 25 + [1] * 15, dtype=torch.int32, device=cuda)
    table = torch.tensor([[5, 2, 0, 0], [1, 4, 0, 0]], dtype=torch.int32, device=cuda)
    cos, sin = fr.rotary_cos_sin(0, 64, 128, 1e4)
    cos_d, sin_d = _dev(cos, cuda), _dev(sin, cuda)
    pool_a, pool_b = ops.new_kv_pool(6, n_kv, cuda), ops.new_kv_pool(6, n_kv, cuda)
    qkv = ops.quant_matmul_w4a16(x, w, m, n, k)
    q_a = ops.rope_kv_append(qkv, pos, slot, table, cos_d, sin_d, 128, pool_a, n_q, n_kv)
    q_b = torch.zeros((m, n_q, 128), dtype=torch.bfloat16, device=cuda)
    dummy = torch.empty((m, n), dtype=torch.bfloat16, device=cuda)
    ops.quant_matmul_w4a16(x, w, m, n, k, out=dummy, rope=(pos, slot, table, cos_d, sin_d, q_b, pool_b, n_q, n_kv))
    torch.cuda.synchronize()

    def close(a, b):
        a, b = a.float().cpu().numpy(), b.float().cpu().numpy()
        assert np.mean(a == b) > 0.995
        assert np.all(np.abs(a - b) <= 2.0 ** -7 * np.maximum(np.abs(a), 1e-3))

    close(q_a, q_b)
    close(pool_a.view(torch.bfloat16), pool_b.view(torch.bfloat16))
    assert float(q_b.float().abs().sum()) > 0


def test_matmul_rejects_bad_arguments(cuda):
    from gptrs_b200 import BackendError
    x = torch.zeros((1, 100), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(BackendError) as e:
        ops.quant_matmul_w4a16(x, x, 1, 16, 100)
    assert e.value.kind == "SpecViolation"


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m,n,k", [(64, 4096, 512), (33, 1000 * 4, 256), (17, 128, 128)])
def test_greedy_head_candidates_equal_the_argmax_of_the_logits(cuda, bits, m, n, k):
    """The lm_head epilogue that leaves per-tile (max, argmax) candidates, and the pick among them: the ids equal the
    argmax of the kernel's own f32 outputs (ties to the smaller column), with and without the outputs being stored."""
    rng = np.random.default_rng(bits * 1000 + m + n)
    x = torch.from_numpy(rng.normal(0, 1, size=(m, k)).astype(np.float32)).to(cuda).to(torch.bfloat16)
    if bits == 4:
        p = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
        s = (rng.uniform(0.5, 1.5, size=(n, k // 128)) * 0.01).astype(np.float16)
        packed = ops.w4a16_repack(torch.from_numpy(p).to(cuda), torch.from_numpy(s).to(cuda), n, k)
        run = ops.quant_matmul_w4a16
    else:
        q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        s = (rng.uniform(0.5, 1.5, size=(n,)) * 0.01).astype(np.float16)
        packed = ops.w8a16_repack(torch.from_numpy(q).to(cuda), torch.from_numpy(s).to(cuda), n, k)
        run = ops.quant_matmul_w8a16
    tiles = (n + 127) // 128
    logits = run(x, packed, m, n, k, out_f32=True)
    want = torch.argmax(logits, dim=1).to(torch.int32)   # torch returns the first maximum: the smaller column
    for skip in (False, True):
        bv = torch.full((tiles, m), float("nan"), dtype=torch.float32, device=cuda)
        bi = torch.full((tiles, m), -1, dtype=torch.int32, device=cuda)
        out = torch.zeros((m, n), dtype=torch.float32, device=cuda)
        run(x, packed, m, n, k, out=out, out_f32=True, best=(bv, bi, skip))
        got = ops.pick_best(bv, bi)
        assert torch.equal(got, want), skip
        assert torch.equal(out, logits) if not skip else float(out.abs().max()) == 0.0
    assert ops.matmul_status() == 0
