"""ms_attention_decode_static, the entry point that allocates nothing, called through its exported C symbol.

It must give what the ordinary entry point gives (same kernel, scratch memory of the library's own), on
two calls in a row of different shapes, so that the second call finds the first one's leftovers in the
shared array.  This file is collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _static(lib):
    fn = lib.ms_attention_decode_static
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P]
    fn.restype = I
    return fn


def test_static_scratch_entry_point_matches_the_ordinary_one():
    import torch

    from machserve_b200 import ops
    from tests.test_kernels_gpu import N, PagedCase, T, dev

    lib = ops.lib()
    fn = _static(lib)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr() if t is not None else 0)
    # two calls in a row: different head counts, splits and row counts, so the counters of the second
    # call lie where the first call left partial results
    for lens, hq, hkv, hd, page, window, splits in [([300, 17, 129], 14, 2, 64, 64, None, 5),
                                                    ([500, 90], 12, 2, 128, 16, 100, 3),
                                                    ([260], 4, 2, 32, 8, None, 1)]:
        case = PagedCase(lens, hq, hkv, hd, page, window, seed=hq)
        rows = [(s, p) for s, n in enumerate(lens) for p in sorted({0, n // 2, n - 1, min(n - 1, 64)})]
        q, want, pos, slot = case.queries(rows, seed=splits)
        q16 = T(q, torch.bfloat16)
        ordinary = torch.empty((len(rows), hq * hd), dtype=torch.bfloat16, device=dev())
        n = ops.attention_decode_scratch_words(len(rows), hq, hkv, hd, splits)
        scratch = torch.zeros((max(n, 1),), dtype=torch.float32, device=dev())
        ops.attention_decode(q16, case.k_pages, case.v_pages, ordinary, scratch, pos, slot, case.table, hq, hkv, hd,
                             window, hd ** -0.5, splits)
        static = torch.full((len(rows), hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]  # the device's own count: a cudaMalloc inside the library would move it
        rc = fn(ptr(q16), ptr(case.k_pages), ptr(case.v_pages), ptr(static), ptr(None), ptr(pos), ptr(slot),
                ptr(case.table), case.table.shape[1], case.k_pages.shape[0], len(rows), hq, hkv, hd, page,
                int(window or 0), hd ** -0.5, splits, stream)
        assert rc == 0, lib.ms_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the entry point changed the device's free memory"
        assert np.abs(N(static) - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
        assert np.abs(N(static) - N(ordinary)).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    import torch

    from machserve_b200 import ops

    lib = ops.lib()
    fn = _static(lib)
    null = ctypes.c_void_p(0)
    # 4096 rows x 32 heads x 16 splits x (128 + 2) words is far more than the array holds: refused before any launch
    rc = fn(null, null, null, null, null, null, null, null, 8, 8, 4096, 32, 8, 128, 16, 0, 1.0, 16,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    msg = lib.ms_last_error().decode()
    assert "words of scratch" in msg and str(1 << 20) in msg
