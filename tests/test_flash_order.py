"""What the blockwise order of the tensor-core prefill attention costs against the exact softmax of the reference, on the
CPU (oracle/flash_ref.py): random rows, rows whose maximum keeps growing from block to block by less than the lazy
rescale step (the exponentials then reach 2^8 before the accumulator is rescaled), by more than it, and a late outlier."""
import numpy as np
import pytest

from oracle import flash_ref as fl
from oracle import quant_ref as qr


def _case(kind, rng, l=700, hd=128, rows=24):
    q = qr.to_bf16(rng.normal(0, 1, size=(rows, hd)).astype(np.float32))
    k = qr.to_bf16(rng.normal(0, 1, size=(l, hd)).astype(np.float32))
    v = qr.to_bf16(rng.normal(0, 1, size=(l, hd)).astype(np.float32))
    if kind != "random":
        # keys aligned with the first query, growing by `step` (in log2 units of the scaled score) per 128-key block
        step = {"creep": 7.0, "jump": 20.0, "outlier": 0.0}[kind]
        d = q[0] / np.linalg.norm(q[0])
        per_block = step * np.log(2.0) * np.sqrt(hd) / np.linalg.norm(q[0])
        for b in range(l // 128 + 1):
            k[b * 128:(b + 1) * 128] = qr.to_bf16(k[b * 128:(b + 1) * 128] * 0.1 + d * (per_block * b))
        if kind == "outlier":
            k[l - 3] = qr.to_bf16(d * (40.0 * np.log(2.0) * np.sqrt(hd) / np.linalg.norm(q[0])))
    lens = np.concatenate([[l], rng.integers(1, l + 1, size=rows - 1)]).astype(np.int64)
    return q, k, v, lens


@pytest.mark.parametrize("kind", ["random", "creep", "jump", "outlier"])
def test_blockwise_order_matches_the_exact_softmax(kind):
    rng = np.random.default_rng(["random", "creep", "jump", "outlier"].index(kind))
    q, k, v, lens = _case(kind, rng)
    got = fl.causal_rows_blockwise(q, k, v, lens)
    want = fl.causal_rows_exact(q, k, v, lens)
    assert np.isfinite(got).all()
    # P is rounded to bf16 (2^-9 relative per weight) before it meets V: the bar of the GPU parity tests is 2e-2
    assert np.max(np.abs(got - want)) <= 6e-3, np.max(np.abs(got - want))


def test_rows_without_visible_keys_give_zero():
    rng = np.random.default_rng(9)
    q, k, v, lens = _case("random", rng, l=130, rows=4)
    lens[2] = 0
    got = fl.causal_rows_blockwise(q, k, v, lens)
    assert np.all(got[2] == 0) and np.isfinite(got).all()
