"""sy_sort_by_expert_static: the sort for hosts that may not allocate device memory while they
run (all HBM already given to the host's own arena, or allocation calls forbidden on the request
path). Its scratch is an array inside the library image, so the caller passes inputs and
outputs only. Called here through the C ABI; its outputs must equal, bit for bit, those of
sy_sort_by_expert with caller-provided scratch, on two calls in a row (the shared array keeps
whatever the previous call left in it). Collected last on purpose: a run that stops at the first
failure has then already run every other test."""

import ctypes

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def both_sorts(lib, idx, w, E):
    from switchyard_b200 import _lib
    M, k = idx.numel(), idx.shape[1]
    code = _lib.SY_DTYPE_F16 if w.dtype == torch.float16 else _lib.SY_DTYPE_BF16
    stream = torch.cuda.current_stream().cuda_stream
    results = []
    for static in (False, True):
        counts = torch.full((E,), -1, dtype=torch.int32, device=DEV)
        offsets = torch.full((E + 1,), -1, dtype=torch.int32, device=DEV)
        token = torch.full((M,), -1, dtype=torch.int32, device=DEV)
        pos_of = torch.full((M,), -1, dtype=torch.int32, device=DEV)
        wsorted = torch.zeros(M, dtype=w.dtype, device=DEV)
        if static:
            rc = lib.sy_sort_by_expert_static(idx.data_ptr(), w.data_ptr(), M, k, E, code, counts.data_ptr(),
                                              offsets.data_ptr(), token.data_ptr(), wsorted.data_ptr(),
                                              pos_of.data_ptr(), stream)
        else:
            need = lib.sy_sort_scratch_bytes(M, E)
            scratch = torch.empty(max(need, 1), dtype=torch.uint8, device=DEV)
            rc = lib.sy_sort_by_expert(idx.data_ptr(), w.data_ptr(), M, k, E, code, counts.data_ptr(),
                                       offsets.data_ptr(), token.data_ptr(), wsorted.data_ptr(), pos_of.data_ptr(),
                                       scratch.data_ptr(), need, stream)
        assert rc == 0, lib.sy_last_error()
        torch.cuda.synchronize()
        results.append((counts, offsets, token, wsorted, pos_of))
    return results


def test_static_scratch_sort_equals_the_sort_with_caller_scratch():
    from switchyard_b200 import _lib
    lib = _lib.load()
    # two calls in a row on different sizes: several blocks with a large table first, then fewer
    # blocks (stale entries of the first call stay in the array), then a one-block sort
    for (N, E, k, seed, dtype) in [(9000, 64, 8, 21, torch.float16), (3000, 128, 4, 22, torch.bfloat16),
                                   (700, 64, 8, 23, torch.float16)]:
        idx, w = cases.sort_inputs(E, k, N, seed)
        idx, w = idx.to(DEV), w.to(dtype).to(DEV)
        ref, got = both_sorts(lib, idx, w, E)
        for a, b, name in zip(ref, got, ("counts", "offsets", "token", "wsorted", "pos_of")):
            assert torch.equal(a, b), (N, E, name)
        assert int(got[1][-1]) == N * k
    # beyond the stated maximum: a clear error, nothing enqueued
    rc = lib.sy_sort_by_expert_static(None, None, (1 << 20) + 8, 8, 64, 0, ctypes.c_void_p(1), ctypes.c_void_p(1), None,
                                      None, None, None)
    assert rc == -1 and b"at most 1048576 choices" in lib.sy_last_error()
    from switchyard_b200 import kernels
    assert kernels.ext().device_status(DEV) == 0
