"""Paged bf16 decode attention, RoPE + KV append and the f32 dense-cache attention against the
oracle's restatement of functional::attention_decode_cache. bf16 path tolerance: max-abs 2e-2;
f32 path: 1e-4 (the tolerances the decode path is held to)."""
import numpy as np
import pytest
import torch

from gptrs_b200 import ops
from oracle import functional_ref as fr
from oracle import quant_ref as qr

pytestmark = pytest.mark.gpu

HD = 128


def _setup(rng, lens, n_q, n_kv, cuda, extra_pages=3):
    """Random page table (a permutation of the physical pages), one row per sequence."""
    b = len(lens)
    pages_per = [(l + 15) // 16 for l in lens]
    max_pages = max(pages_per) + 1
    total = sum(pages_per) + extra_pages
    perm = rng.permutation(total).astype(np.int32)
    table = np.zeros((b, max_pages), dtype=np.int32)
    o = 0
    for i, n in enumerate(pages_per):
        table[i, :n] = perm[o:o + n]
        o += n
    pool = ops.new_kv_pool(total, n_kv, cuda)
    return table, pool


def _fill(rng, lens, n_q, n_kv, table, pool, cuda, theta=1e6, rope=True):
    """Appends every token of every sequence through the C ABI; returns the oracle's f32 view
    of what was stored (bf16-rounded rotated K, V) per sequence."""
    max_len = max(lens)
    cos, sin = fr.rotary_cos_sin(0, max_len, HD, theta)
    if not rope:
        cos, sin = np.ones_like(cos), np.zeros_like(sin)
    cos_d, sin_d = torch.from_numpy(cos).to(cuda), torch.from_numpy(sin).to(cuda)
    table_d = torch.from_numpy(table).to(cuda)
    width = (n_q + 2 * n_kv) * HD
    stored = []
    last_q = []
    for s, l in enumerate(lens):
        qkv = qr.to_bf16(rng.normal(0, 1, size=(l, width)).astype(np.float32))
        pos = np.arange(l, dtype=np.int32)
        q_rot = ops.rope_kv_append(torch.from_numpy(qkv).to(cuda).to(torch.bfloat16), torch.from_numpy(pos).to(cuda),
                                   torch.full((l,), s, dtype=torch.int32, device=cuda), table_d, cos_d, sin_d, HD,
                                   pool, n_q, n_kv)
        ref = fr.apply_rope_qkv_packed(qkv, cos[:l], sin[:l], n_q, n_kv, HD)
        k_ref = qr.to_bf16(ref[:, n_q * HD:(n_q + n_kv) * HD]).reshape(l, n_kv, HD)
        v_ref = ref[:, (n_q + n_kv) * HD:].reshape(l, n_kv, HD)
        q_ref = qr.to_bf16(ref[:, :n_q * HD]).reshape(l, n_q, HD)
        stored.append((k_ref, v_ref, q_ref))
        last_q.append(q_rot)
    return stored, last_q, table_d


@pytest.mark.parametrize("lens,n_q,n_kv", [([1], 4, 1), ([16, 17, 5], 8, 2), ([100, 33], 32, 8), ([700], 8, 8)])
def test_rope_append_roundtrip(cuda, lens, n_q, n_kv):
    rng = np.random.default_rng(sum(lens) + n_q)
    table, pool = _setup(rng, lens, n_q, n_kv, cuda)
    stored, q_rots, table_d = _fill(rng, lens, n_q, n_kv, table, pool, cuda)
    for s, l in enumerate(lens):
        k, v = ops.kv_gather(pool, table_d[s].contiguous(), l, n_kv)
        k_ref, v_ref, q_ref = stored[s]
        # V is a pure copy: bit-exact. K/Q go through f32 rotation + bf16 rounding: allow 1 bf16 ulp.
        assert np.array_equal(v.float().cpu().numpy(), v_ref)
        assert np.allclose(k.float().cpu().numpy(), k_ref, rtol=2 ** -7, atol=1e-6)
        assert np.allclose(q_rots[s].float().cpu().numpy(), q_ref, rtol=2 ** -7, atol=1e-6)


def _oracle_decode(stored, lens, n_q, n_kv, q_rows):
    """Dense reference per sequence: the reference's attention_decode_cache math on the stored
    (bf16-valued) K/V with capacity = next power of two >= len, query = last token."""
    outs = []
    for s, l in enumerate(lens):
        k_ref, v_ref, _ = stored[s]
        cap = 1 << max(0, (l - 1).bit_length())
        ck = np.zeros((n_kv, cap, HD), np.float32)
        cv = np.zeros((n_kv, cap, HD), np.float32)
        ck[:, :l] = k_ref.transpose(1, 0, 2)
        cv[:, :l] = v_ref.transpose(1, 0, 2)
        row = np.concatenate([q_rows[s].reshape(1, -1), ck[:, l - 1].reshape(1, -1), cv[:, l - 1].reshape(1, -1)], axis=1)
        ctx, _, _ = fr.attention_decode_cache(row, n_q, n_kv, HD, ck, cv, l - 1)
        outs.append(ctx[0])
    return np.stack(outs)


CASES = [
    ([1], 4, 1, None), ([15, 16, 17, 31, 33], 8, 2, None), ([64, 200, 513], 32, 8, None),
    ([1000, 77, 2048], 32, 8, 4), ([300] * 6, 16, 2, 8), ([4099], 8, 8, 16), ([129, 640], 8, 1, None),
]


@pytest.mark.parametrize("lens,n_q,n_kv,chunk", CASES)
def test_paged_attention_matches_oracle(cuda, lens, n_q, n_kv, chunk):
    rng = np.random.default_rng(len(lens) * 1000 + n_q + sum(lens))
    table, pool = _setup(rng, lens, n_q, n_kv, cuda)
    stored, q_rots, table_d = _fill(rng, lens, n_q, n_kv, table, pool, cuda)
    b = len(lens)
    q = torch.stack([q_rots[s][lens[s] - 1] for s in range(b)]).contiguous()
    slot = torch.arange(b, dtype=torch.int32, device=cuda)
    ctx_len = torch.tensor(lens, dtype=torch.int32, device=cuda)
    out, status = ops.paged_attention_decode(q, pool, table_d, slot, ctx_len, n_q, n_kv, max(lens), chunk_pages=chunk)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = _oracle_decode(stored, lens, n_q, n_kv, [q[s].float().cpu().numpy() for s in range(b)])
    got = out.float().cpu().numpy()
    assert np.max(np.abs(got - want)) <= 2e-2, np.max(np.abs(got - want))


def test_prefill_rows_share_one_page_table_row(cuda):
    """Many query tokens of ONE sequence (chunked prefill): token t sees positions 0..t."""
    rng = np.random.default_rng(5)
    l, n_q, n_kv = 90, 8, 2
    table, pool = _setup(rng, [l], n_q, n_kv, cuda)
    stored, q_rots, table_d = _fill(rng, [l], n_q, n_kv, table, pool, cuda)
    slot = torch.zeros(l, dtype=torch.int32, device=cuda)
    ctx_len = torch.arange(1, l + 1, dtype=torch.int32, device=cuda)
    out, status = ops.paged_attention_decode(q_rots[0], pool, table_d, slot, ctx_len, n_q, n_kv, l)
    assert int(status.item()) == 0
    k_ref, v_ref, q_ref = stored[0]
    got = out.float().cpu().numpy()
    for t in (0, 1, 15, 16, 47, 89):
        want = _oracle_decode([(k_ref[:t + 1], v_ref[:t + 1], None)], [t + 1], n_q, n_kv,
                              [q_rots[0][t].float().cpu().numpy()])
        assert np.max(np.abs(got[t] - want[0])) <= 2e-2


def test_attention_rejects_unsupported_geometry(cuda):
    from gptrs_b200 import BackendError
    z = torch.zeros(16, dtype=torch.int32, device=cuda)
    q = torch.zeros((1, 4, 64), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(BackendError):
        ops.paged_attention_decode(q, q, z.view(1, 16), z[:1], z[:1], 4, 1, 16, head_dim=64)


@pytest.mark.parametrize("n_q,n_kv,hd,cap,positions", [(12, 12, 64, 64, [0, 5, 63]), (4, 2, 16, 32, [31]), (8, 1, 128, 128, [7, 100])])
def test_attention_decode_f32_matches_oracle(cuda, n_q, n_kv, hd, cap, positions):
    rng = np.random.default_rng(n_q * 10 + hd)
    n_slots = len(positions)
    width = (n_q + 2 * n_kv) * hd
    ck = rng.normal(0, 1, size=(n_slots, n_kv, cap, hd)).astype(np.float32)
    cv = rng.normal(0, 1, size=(n_slots, n_kv, cap, hd)).astype(np.float32)
    qkv = rng.normal(0, 1, size=(n_slots, width)).astype(np.float32)
    kd, vd = torch.from_numpy(ck).to(cuda), torch.from_numpy(cv).to(cuda)
    pos = torch.tensor(positions, dtype=torch.int32, device=cuda)
    slot = torch.arange(n_slots, dtype=torch.int32, device=cuda)
    qd = torch.from_numpy(qkv).to(cuda)
    ops.kv_append_f32(qd, pos, slot, kd, vd, n_q, n_kv, hd)
    out = ops.attention_decode_f32(qd, kd, vd, pos, slot, n_q, n_kv, hd)
    got = out.cpu().numpy()
    for s, p in enumerate(positions):
        want, k_new, v_new = fr.attention_decode_cache(qkv[s:s + 1], n_q, n_kv, hd, ck[s], cv[s], p)
        assert np.allclose(got[s], want[0], rtol=1e-4, atol=1e-4)
        assert np.array_equal(kd[s].cpu().numpy(), k_new) and np.array_equal(vd[s].cpu().numpy(), v_new)
