"""CPU checks of the quantisation oracle (formats are this backend's own definition)."""
import numpy as np

from oracle import quant_ref as qr


def test_int4_pack_unpack_bit_exact():
    rng = np.random.default_rng(1)
    q = rng.integers(-8, 8, size=(32, 256), dtype=np.int8)
    p = qr.pack_int4(q)
    assert p.shape == (32, 128)
    # low nibble = even k
    assert (p[0, 0] & 0xF) == (int(q[0, 0]) & 0xF) and (p[0, 0] >> 4) == (int(q[0, 1]) & 0xF)
    assert np.array_equal(qr.unpack_int4(p), q)


def test_bf16_rounding_matches_torch():
    import torch
    rng = np.random.default_rng(2)
    x = rng.normal(0, 3, size=4096).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(qr.to_bf16(x), want)
    assert np.array_equal(qr.bf16_from_bits(qr.bf16_bits(x)), want)


def test_quantize_w4_roundtrip_error_bound():
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, size=(48, 384)).astype(np.float32)
    p, s = qr.quantize_w4(w)
    d = qr.dequant_w4(p, s)
    step = s.astype(np.float32).repeat(128, axis=1)
    assert np.all(np.abs(d - w) <= 0.5 * step * 1.01 + 1e-8)
    q = qr.unpack_int4(p)
    assert q.min() >= -8 and q.max() <= 7


def test_quantize_w8_roundtrip_error_bound():
    rng = np.random.default_rng(4)
    w = rng.normal(0, 0.02, size=(48, 384)).astype(np.float32)
    q, s = qr.quantize_w8(w)
    d = qr.dequant_w8(q, s)
    assert np.all(np.abs(d - w) <= 0.5 * s.astype(np.float32)[:, None] * 1.01 + 1e-8)


def test_gate_up_interleave_is_a_permutation():
    perm = qr.interleave_gate_up_rows(64)
    assert sorted(perm.tolist()) == list(range(64))
    assert perm[:16].tolist() == list(range(8)) + list(range(32, 40))
