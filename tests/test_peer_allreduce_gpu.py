"""The one-shot all-reduce of the tensor-parallel engine (csrc/peer_allreduce.cu), with its ranks emulated on one
device: every rank's receive region and partial tile live in one process, all pushes of a call are launched before the
first wait (so no launch ever polls for a later one), and several calls in a row exercise both receive slots and the
growing flags. The sum is exact here (small integers), every rank must hold the same bits, and the status word stays 0."""
import ctypes

import numpy as np
import pytest
import torch

from gptrs_b200 import check, lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tp,n,calls", [(2, 64 * 3072, 3), (4, 4 * 768, 5), (8, 16 * 3072, 2)])
def test_emulated_ranks_sum_and_repeat(cuda, tp, n, calls):
    L = lib()
    cap = n + 1024
    nbytes = L.gptrs_cuda_peer_region_bytes(tp, cap)
    assert nbytes > 2 * tp * cap * 4
    regions = torch.zeros(tp * nbytes, dtype=torch.uint8, device=cuda)
    rng = np.random.default_rng(tp)
    start = rng.integers(-3, 4, size=(tp, n)).astype(np.float32)
    partials = torch.from_numpy(start).to(cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    check(L.gptrs_cuda_debug_peer_allreduce(regions.data_ptr(), partials.data_ptr(), tp, n, cap, calls, status.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = start.sum(axis=0) * float(tp) ** (calls - 1)   # after the first call every rank holds the sum
    got = partials.cpu().numpy()
    for r in range(tp):
        assert np.array_equal(got[r], want), r


def test_message_must_fit_the_slot(cuda):
    from gptrs_b200 import BackendError
    L = lib()
    regions = torch.zeros(2 * L.gptrs_cuda_peer_region_bytes(2, 1024), dtype=torch.uint8, device=cuda)
    partials = torch.zeros((2, 2048), dtype=torch.float32, device=cuda)
    with pytest.raises(BackendError):
        check(L.gptrs_cuda_debug_peer_allreduce(regions.data_ptr(), partials.data_ptr(), 2, 2048, 1024, 1, None,
                                                torch.cuda.current_stream().cuda_stream))
