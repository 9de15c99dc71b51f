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


@pytest.mark.parametrize("l,n_q,n_kv,chunk", [(90, 8, 2, None), (131, 32, 8, 4), (70, 4, 4, None), (200, 16, 2, 4), (37, 8, 1, None)])
def test_prefill_chunk_entry_point(cuda, l, n_q, n_kv, chunk):
    """gptrs_cuda_paged_attention_prefill streams the pages once per group of 16 / (Hq / Hkv) token rows: same
    results as the one-row-per-CTA entry point and the oracle, for row counts that are not a multiple of the group,
    rows whose visible length ends in different splits (chunk of 4 pages = 64 tokens), and a second sequence whose
    rows start in the middle of the row list at a group boundary."""
    rng = np.random.default_rng(l * 7 + n_q)
    l2 = 21
    table, pool = _setup(rng, [l, l2], n_q, n_kv, cuda)
    stored, q_rots, table_d = _fill(rng, [l, l2], n_q, n_kv, table, pool, cuda)
    tq = 16 // (n_q // n_kv)
    pad = (-l) % tq  # rows of sequence 1 must start a new group: repeat the last row of sequence 0
    q = torch.cat([q_rots[0], q_rots[0][-1:].repeat(pad, 1, 1), q_rots[1]]).contiguous()
    slot = torch.tensor([0] * (l + pad) + [1] * l2, dtype=torch.int32, device=cuda)
    ctx = torch.tensor(list(range(1, l + 1)) + [l] * pad + list(range(1, l2 + 1)), dtype=torch.int32, device=cuda)
    ref, st0 = ops.paged_attention_decode(q, pool, table_d, slot, ctx, n_q, n_kv, l, chunk_pages=chunk)
    out, st1 = ops.paged_attention_decode(q, pool, table_d, slot, ctx, n_q, n_kv, l, chunk_pages=chunk, prefill=True)
    torch.cuda.synchronize()
    assert int(st0.item()) == 0 and int(st1.item()) == 0
    got, base = out.float().cpu().numpy(), ref.float().cpu().numpy()
    assert np.max(np.abs(got - base)) <= 8e-3, np.max(np.abs(got - base))  # both round to bf16 from slightly different sums
    k_ref, v_ref, _ = stored[0]
    for t in sorted({0, 1, tq - 1, tq, 15, 16, 63, 64, 65, l - 2, l - 1} & set(range(l))):
        want = _oracle_decode([(k_ref[:t + 1], v_ref[:t + 1], None)], [t + 1], n_q, n_kv, [q[t].float().cpu().numpy()])
        assert np.max(np.abs(got[t] - want[0])) <= 2e-2, t
    k2, v2, _ = stored[1]
    for t in (0, 5, l2 - 1):
        want = _oracle_decode([(k2[:t + 1], v2[:t + 1], None)], [t + 1], n_q, n_kv, [q[l + pad + t].float().cpu().numpy()])
        assert np.max(np.abs(got[l + pad + t] - want[0])) <= 2e-2, t


def test_prefill_chunk_rejects_odd_group(cuda):
    rng = np.random.default_rng(2)
    table, pool = _setup(rng, [20], 6, 2, cuda)
    stored, q_rots, table_d = _fill(rng, [20], 6, 2, table, pool, cuda)
    from gptrs_b200 import BackendError
    with pytest.raises(BackendError) as e:
        ops.paged_attention_decode(q_rots[0], pool, table_d, torch.zeros(20, dtype=torch.int32, device=cuda),
                                   torch.arange(1, 21, dtype=torch.int32, device=cuda), 6, 2, 20, prefill=True)
    assert e.value.kind == "Unimplemented"


def test_attention_rejects_unsupported_geometry(cuda):
    from gptrs_b200 import BackendError
    z = torch.zeros(16, dtype=torch.int32, device=cuda)
    q = torch.zeros((1, 4, 64), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(BackendError):
        ops.paged_attention_decode(q, q, z.view(1, 16), z[:1], z[:1], 4, 1, 16, head_dim=64)


@pytest.mark.parametrize("n_q,n_kv,hd,cap,positions", [(12, 12, 64, 64, [0, 5, 63]), (4, 2, 16, 32, [31]), (8, 1, 128, 128, [7, 100]),
                                                       (4, 4, 1, 8, [0, 7]), (3, 3, 24, 16, [5, 15]), (2, 1, 6, 300, [299]), (2, 2, 127, 9, [4])])
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
    # the single-launch variant (append inside the attention kernel) leaves the same caches and outputs
    kd2, vd2 = torch.from_numpy(ck).to(cuda), torch.from_numpy(cv).to(cuda)
    out2 = ops.attention_decode_f32(qd, kd2, vd2, pos, slot, n_q, n_kv, hd, append=True)
    assert torch.equal(out2, out) and torch.equal(kd2, kd) and torch.equal(vd2, vd)


def test_context_length_above_the_launch_bound_is_clamped_and_flagged(cuda):
    """A visible length in device memory that exceeds what the launch was sized for must not walk off the page table
    or the split partials: the kernel clamps it and sets code 2 in the status word."""
    rng = np.random.default_rng(12)
    lens, n_q, n_kv = [100, 40], 8, 2
    table, pool = _setup(rng, lens, n_q, n_kv, cuda)
    stored, q_rots, table_d = _fill(rng, lens, n_q, n_kv, table, pool, cuda)
    q = torch.stack([q_rots[s][lens[s] - 1] for s in range(2)]).contiguous()
    slot = torch.arange(2, dtype=torch.int32, device=cuda)
    bad = torch.tensor([100, 5000], dtype=torch.int32, device=cuda)   # second sequence claims 5000 visible tokens
    out, status = ops.paged_attention_decode(q, pool, table_d, slot, bad, n_q, n_kv, 100, chunk_pages=4)
    torch.cuda.synchronize()
    assert int(status.item()) == 2
    want = _oracle_decode(stored[:1], lens[:1], n_q, n_kv, [q[0].float().cpu().numpy()])
    assert np.max(np.abs(out[0].float().cpu().numpy() - want[0])) <= 2e-2   # the well-formed row is unaffected
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("l,n_q,n_kv,chunk", [(90, 8, 2, None), (131, 32, 8, 4), (300, 32, 8, 8), (70, 4, 4, None), (200, 16, 2, 4), (37, 8, 1, None), (16, 32, 8, None)])
def test_prefill_blocks_entry_point(cuda, l, n_q, n_kv, chunk):
    """gptrs_cuda_paged_attention_prefill_blocks: a CTA takes an aligned block of four row groups (16 tokens at a group of
    four) of one sequence and streams the pages once for it. Same results as the one-row-per-CTA entry point and the
    oracle: row counts that are not a multiple of the block, rows whose visible length ends in different splits, more
    pages than the ring has stages, and a second sequence whose rows start at a block boundary."""
    rng = np.random.default_rng(l * 5 + n_q)
    l2 = 21
    table, pool = _setup(rng, [l, l2], n_q, n_kv, cuda)
    stored, q_rots, table_d = _fill(rng, [l, l2], n_q, n_kv, table, pool, cuda)
    blk = 4 * (16 // (n_q // n_kv))
    pad = (-l) % blk  # rows of sequence 1 must start a new block: repeat the last row of sequence 0
    q = torch.cat([q_rots[0], q_rots[0][-1:].repeat(pad, 1, 1), q_rots[1]]).contiguous()
    slot = torch.tensor([0] * (l + pad) + [1] * l2, dtype=torch.int32, device=cuda)
    ctx = torch.tensor(list(range(1, l + 1)) + [l] * pad + list(range(1, l2 + 1)), dtype=torch.int32, device=cuda)
    ref, st0 = ops.paged_attention_decode(q, pool, table_d, slot, ctx, n_q, n_kv, l, chunk_pages=chunk)
    out, st1 = ops.paged_attention_decode(q, pool, table_d, slot, ctx, n_q, n_kv, l, chunk_pages=chunk, prefill="blocks")
    torch.cuda.synchronize()
    assert int(st0.item()) == 0 and int(st1.item()) == 0
    got, base = out.float().cpu().numpy(), ref.float().cpu().numpy()
    assert np.max(np.abs(got - base)) <= 8e-3, np.max(np.abs(got - base))  # both round to bf16 from slightly different sums
    k_ref, v_ref, _ = stored[0]
    for t in sorted({0, 1, 3, 4, 15, 16, 17, 63, 64, 65, l - 2, l - 1} & set(range(l))):
        want = _oracle_decode([(k_ref[:t + 1], v_ref[:t + 1], None)], [t + 1], n_q, n_kv, [q[t].float().cpu().numpy()])
        assert np.max(np.abs(got[t] - want[0])) <= 2e-2, t
    k2, v2, _ = stored[1]
    for t in (0, 5, l2 - 1):
        want = _oracle_decode([(k2[:t + 1], v2[:t + 1], None)], [t + 1], n_q, n_kv, [q[l + pad + t].float().cpu().numpy()])
        assert np.max(np.abs(got[l + pad + t] - want[0])) <= 2e-2, t


@pytest.mark.parametrize("aligned", [True, False])
@pytest.mark.parametrize("l,n_q,n_kv", [(90, 8, 2), (131, 32, 8), (300, 32, 8), (70, 4, 4), (200, 16, 2), (37, 8, 1), (16, 32, 8), (700, 32, 8), (128, 32, 8), (1, 32, 8)])
def test_prefill_tensor_core_entry_point(cuda, l, n_q, n_kv, aligned):
    """gptrs_cuda_paged_attention_prefill_tc (tcgen05 / tensor memory): a CTA takes an aligned tile of 256 / group rows of
    one sequence (two row tiles of 128 that share the K/V blocks) and walks its visible keys in blocks of 128.
    Same results as the one-row-per-CTA entry point and the oracle: row counts that are not a multiple of the tile,
    contexts of one, exactly one and several key blocks, a last block whose tail pages are never loaded, and a second
    sequence whose rows start at a tile boundary (aligned) or in the middle of the first sequence's last tile (a second
    CTA serves them)."""
    rng = np.random.default_rng(l * 7 + n_q)
    l2 = 21
    table, pool = _setup(rng, [l, l2], n_q, n_kv, cuda)
    stored, q_rots, table_d = _fill(rng, [l, l2], n_q, n_kv, table, pool, cuda)
    tile = 256 // (n_q // n_kv)
    pad = (-l) % tile if aligned else 0  # aligned: repeat the last row of sequence 0 up to the tile boundary
    q = torch.cat([q_rots[0], q_rots[0][-1:].repeat(pad, 1, 1), q_rots[1]]).contiguous()
    slot = torch.tensor([0] * (l + pad) + [1] * l2, dtype=torch.int32, device=cuda)
    ctx = torch.tensor(list(range(1, l + 1)) + [l] * pad + list(range(1, l2 + 1)), dtype=torch.int32, device=cuda)
    ref, st0 = ops.paged_attention_decode(q, pool, table_d, slot, ctx, n_q, n_kv, l)
    out, st1 = ops.paged_attention_decode(q, pool, table_d, slot, ctx, n_q, n_kv, l, prefill="tc")
    torch.cuda.synchronize()
    assert int(st0.item()) == 0 and int(st1.item()) == 0
    got, base = out.float().cpu().numpy(), ref.float().cpu().numpy()
    assert np.isfinite(got).all()
    # both round P and the result to bf16 from different sums: one bf16 step (2^-8 relative) at the value's magnitude
    assert np.all(np.abs(got - base) <= 8e-3 * np.maximum(1.0, np.abs(base))), np.max(np.abs(got - base))
    k_ref, v_ref, _ = stored[0]
    for t in sorted({0, 1, 3, 4, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256, l - 2, l - 1} & set(range(l))):
        want = _oracle_decode([(k_ref[:t + 1], v_ref[:t + 1], None)], [t + 1], n_q, n_kv, [q[t].float().cpu().numpy()])
        assert np.max(np.abs(got[t] - want[0])) <= 2e-2, t
    k2, v2, _ = stored[1]
    for t in (0, 5, l2 - 1):
        want = _oracle_decode([(k2[:t + 1], v2[:t + 1], None)], [t + 1], n_q, n_kv, [q[l + pad + t].float().cpu().numpy()])
        assert np.max(np.abs(got[l + pad + t] - want[0])) <= 2e-2, t


def test_prefill_tensor_core_flags_a_tile_of_three_sequences(cuda):
    rng = np.random.default_rng(3)
    n_q, n_kv = 8, 2
    table, pool = _setup(rng, [20, 20, 20], n_q, n_kv, cuda)
    stored, q_rots, table_d = _fill(rng, [20, 20, 20], n_q, n_kv, table, pool, cuda)
    q = torch.cat(q_rots).contiguous()
    slot = torch.tensor([0] * 20 + [1] * 20 + [2] * 20, dtype=torch.int32, device=cuda)   # one 64-row tile, three sequences
    ctx = torch.tensor(list(range(1, 21)) * 3, dtype=torch.int32, device=cuda)
    out, st = ops.paged_attention_decode(q, pool, table_d, slot, ctx, n_q, n_kv, 20, prefill="tc")
    torch.cuda.synchronize()
    assert int(st.item()) == 2
    ref, _ = ops.paged_attention_decode(q, pool, table_d, slot, ctx, n_q, n_kv, 20)
    got, base = out.float().cpu().numpy(), ref.float().cpu().numpy()
    for rows in (slice(0, 20), slice(40, 60)):   # the first and the last sequence of the tile are served all the same
        assert np.all(np.abs(got[rows] - base[rows]) <= 8e-3 * np.maximum(1.0, np.abs(base[rows])))
