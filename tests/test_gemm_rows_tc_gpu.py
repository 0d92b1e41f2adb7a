"""The tcgen05 product for up to 64 rows (weights as the 128-row operand) with its epilogues, against float64."""
import numpy as np
import pytest

from tests.test_kernels_gpu import N, T, dev

pytestmark = pytest.mark.gpu

# rows, N, K: N that is no multiple of 128 or 64, K that is no multiple of 64, one block and clusters, every batch width
SHAPES = [(1, 16, 32), (8, 1152, 896), (5, 30, 72), (64, 896, 4864), (17, 400, 200), (33, 7, 8), (9, 1000, 136),
          (64, 9728, 896), (16, 1536, 8960), (40, 130, 64)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_rows_tc(m, n, k):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(m * 1000 + k)
    x, w = T(rng.normal(size=(m, k)), torch.bfloat16), T(rng.normal(size=(n, k)) * 0.5, torch.bfloat16)
    want = N(x) @ N(w).T
    scale = max(1.0, np.abs(want).max())
    out32 = torch.full((m, n), 7.0, dtype=torch.float32, device=dev())
    ops.gemm_rows_tc(x, w, out32)
    assert ops.gemm_tc_status() == 0
    assert np.abs(N(out32) - want).max() <= 2e-5 * scale  # float32 sums of exact bfloat16 products
    out16 = torch.empty((m, n), dtype=torch.bfloat16, device=dev())
    ops.gemm_rows_tc(x, w, out16)
    assert np.abs(N(out16) - want).max() <= 2.0 ** -8 * scale
    # rows with a stride (a view of wider rows) give the same bits, and so does a second run
    wide = torch.zeros((m, k + 24), dtype=torch.bfloat16, device=dev()); wide[:, :k] = x
    again = torch.empty((m, n), dtype=torch.float32, device=dev())
    ops.gemm_rows_tc(wide[:, :k], w, again)
    assert torch.equal(again, out32)
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("m,i,k", [(1, 8, 32), (8, 4864, 896), (7, 200, 96), (64, 136, 72), (20, 8960, 1536), (48, 4864, 896)])
def test_gemm_rows_tc_silu_mul(m, i, k):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(i + k)
    x = T(rng.normal(size=(m, k)), torch.bfloat16)
    wg, wu = T(rng.normal(size=(i, k)) * 0.2, torch.bfloat16), T(rng.normal(size=(i, k)) * 0.2, torch.bfloat16)
    g, u = N(x) @ N(wg).T, N(x) @ N(wu).T
    want = g / (1 + np.exp(-g)) * u
    out = torch.empty((m, i), dtype=torch.bfloat16, device=dev())
    ops.gemm_rows_tc_silu_mul(x, wg, wu, out)
    assert ops.gemm_tc_status() == 0
    assert np.abs(N(out) - want).max() <= 2.0 ** -8 * max(1.0, np.abs(want).max()) + 1e-4


@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (8, 896, 896), (13, 72, 136), (16, 896, 4864), (5, 100, 200), (64, 896, 4864), (37, 1536, 1536)])
def test_gemm_rows_tc_resadd_and_norm(m, n, k):
    """The fused forms: the product added into the float32 residual, with sums of squares per block of 16 columns and
    a rounded copy; and the product of that copy whose rows are divided by their rms made from those sums."""
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(m + n + k)
    x, w = T(rng.normal(size=(m, k)), torch.bfloat16), T(rng.normal(size=(n, k)) * 0.3, torch.bfloat16)
    res0 = rng.normal(size=(m, n)).astype(np.float32) * 3
    res = T(res0)
    nb = ops.gemm_small_m_stats_blocks(n)
    stats = torch.full((m, nb), float("nan"), dtype=torch.float32, device=dev())
    copy = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=dev())
    ops.gemm_rows_tc_resadd(x, w, res, stats, copy)
    assert ops.gemm_tc_status() == 0
    assert torch.equal(copy, res.to(torch.bfloat16))  # the new residual, rounded once
    want = res0.astype(np.float64) + N(x) @ N(w).T
    assert np.abs(N(res) - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    ss = np.stack([(N(res)[:, b * 16 : (b + 1) * 16] ** 2).sum(-1) for b in range(nb)], axis=1)
    assert np.abs(N(stats) - ss).max() <= 1e-5 * max(1.0, ss.max())
    if n % 8:
        return
    eps = 1e-5
    cols = 4864 if n == 896 else 40
    w2, w3 = T(rng.normal(size=(cols, n)) * 0.2, torch.bfloat16), T(rng.normal(size=(cols, n)) * 0.2, torch.bfloat16)
    r = N(res)
    inv = 1.0 / np.sqrt((r * r).mean(-1, keepdims=True) + eps)
    out = torch.empty((m, cols), dtype=torch.bfloat16, device=dev())
    ops.gemm_rows_tc_scaled(copy, stats, nb, eps, w2, None, out)
    want4 = N(copy) @ N(w2).T * inv
    assert np.abs(N(out) - want4).max() <= 2.0 ** -7 * max(1.0, np.abs(want4).max())
    ops.gemm_rows_tc_scaled(copy, stats, nb, eps, w2, w3, out)
    g, u = N(copy) @ N(w2).T * inv, N(copy) @ N(w3).T * inv
    want5 = g / (1 + np.exp(-g)) * u
    assert np.abs(N(out) - want5).max() <= 2.0 ** -7 * max(1.0, np.abs(want5).max()) + 1e-3
    assert ops.gemm_tc_status() == 0


def test_gemm_rows_tc_refuses_what_it_does_not_cover():
    import torch
    from machserve_b200 import ops
    assert not ops.gemm_rows_tc_supports(65, 16, 32) and not ops.gemm_rows_tc_supports(4, 16, 36)
    x, w = torch.zeros((65, 32), dtype=torch.bfloat16, device=dev()), torch.zeros((16, 32), dtype=torch.bfloat16, device=dev())
    with pytest.raises(ops.KernelError, match="M=65"):
        ops.gemm_rows_tc(x, w, torch.empty((65, 16), dtype=torch.float32, device=dev()))
