"""Allocation-free decode attention entry point (collected last on purpose).

Some callers of this library cannot allocate device memory: a plugin that runs inside a serving
process whose memory pool belongs to the host application, or code that runs at a moment when
cudaMalloc is not permitted. gptrs_cuda_paged_attention_decode_noalloc serves them with a fixed
scratch array inside the library. This test calls it through the C ABI twice in a row (the second
call with other lengths, so stale partials of the first call are in the array) and checks each
result against the regular entry point, which uses a caller-provided scratch buffer. Both run the
same kernels, so the outputs must be bit-identical."""
import numpy as np
import pytest
import torch

import gptrs_b200
from gptrs_b200 import BackendError, ops

pytestmark = pytest.mark.gpu


def _case(cuda, lens, n_q, n_kv, seed):
    g = torch.Generator(device=cuda)
    g.manual_seed(seed)
    pages_per = max((l + 15) // 16 for l in lens) + 1
    total = pages_per * len(lens)
    pool = torch.randn(total * n_kv * 2 * 16 * 128, dtype=torch.bfloat16, device=cuda, generator=g).view(torch.uint8)
    table = torch.randperm(total, device=cuda, generator=g).to(torch.int32).view(len(lens), pages_per).contiguous()
    q = torch.randn((len(lens), n_q, 128), dtype=torch.bfloat16, device=cuda, generator=g)
    slot = torch.arange(len(lens), dtype=torch.int32, device=cuda)
    ctx = torch.tensor(lens, dtype=torch.int32, device=cuda)
    return q, pool, table, slot, ctx


def test_noalloc_entry_matches_regular_entry_twice_in_a_row(cuda):
    lib = gptrs_b200.lib()
    assert lib.gptrs_cuda_paged_attention_noalloc_max_scratch_bytes() == 8 << 20
    n_q, n_kv = 32, 8
    for seed, lens, chunk in [(1, [700, 1300, 64, 2000], 8), (2, [90, 33, 1500], 4)]:
        q, pool, table, slot, ctx = _case(cuda, lens, n_q, n_kv, seed)
        want, st = ops.paged_attention_decode(q, pool, table, slot, ctx, n_q, n_kv, max(lens), chunk_pages=chunk)
        out = torch.full((len(lens), n_q * 128), float("nan"), dtype=torch.bfloat16, device=cuda)
        status = torch.zeros(1, dtype=torch.int32, device=cuda)
        # the first call on a device looks the scratch address up (and may load the module): warm it up, then compare
        # the driver's own free-memory figure around a call. An allocation made inside the library would show there;
        # torch's counter only sees torch's allocator.
        ops.paged_attention_decode_noalloc(q, pool, table, slot, ctx, n_q, n_kv, max(lens), out, status, chunk)
        torch.cuda.synchronize()
        out.fill_(float("nan"))
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()
        ops.paged_attention_decode_noalloc(q, pool, table, slot, ctx, n_q, n_kv, max(lens), out, status, chunk)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_allocated() == before and free_after == free_before  # nothing was allocated by anyone
        assert int(status.item()) == 0 and int(st.item()) == 0
        assert torch.equal(out.view(torch.int16), want.view(torch.int16))
        assert not torch.isnan(out.float()).any()


def test_noalloc_entry_rejects_oversized_launches(cuda):
    q, pool, table, slot, ctx = _case(cuda, [64] * 4, 32, 8, 3)
    out = torch.empty((4, 32 * 128), dtype=torch.bfloat16, device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    big = torch.empty((4096, 32, 128), dtype=torch.bfloat16, device=cuda)  # 4096 tokens x 32 heads x 8 splits
    slot_big = torch.zeros(4096, dtype=torch.int32, device=cuda)
    ctx_big = torch.full((4096,), 64, dtype=torch.int32, device=cuda)
    out_big = torch.empty((4096, 32 * 128), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(BackendError) as e:
        # max_ctx_len 1024 with 8-page chunks = 8 splits -> 4096 * 32 * 8 * 520 B = 545 MB of partials
        table_big = torch.zeros((4, 64), dtype=torch.int32, device=cuda)
        ops.paged_attention_decode_noalloc(big, pool, table_big, slot_big, ctx_big, 32, 8, 1024, out_big, status, 8)
    assert e.value.kind == "SpecViolation" and "8388608" in str(e.value)
    # a launch that fits still works afterwards
    ops.paged_attention_decode_noalloc(q, pool, table, slot, ctx, 32, 8, 64, out, status, 4)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
