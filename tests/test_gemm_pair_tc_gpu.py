"""The tcgen05 product for many rows that puts a pair of SMs on every tile (cta_group::2), with its epilogues, against
float64: sizes that are no multiples of the tiles, one tile and many, both tile widths."""
import numpy as np
import pytest

from tests.test_kernels_gpu import N, T, dev

pytestmark = pytest.mark.gpu

# rows, N, K
SHAPES = [(300, 200, 72), (129, 520, 264), (1, 8, 8), (512, 1152, 896), (1000, 4608, 512), (257, 136, 1536)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_pair_tc_plain_and_scaled(m, n, k):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(m + n + k)
    x, w = T(rng.normal(size=(m, k)), torch.bfloat16), T(rng.normal(size=(n, k)) * 0.5, torch.bfloat16)
    want = N(x) @ N(w).T
    out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=dev())
    ops.gemm_pair_tc(x, w, out)
    assert ops.gemm_tc_status() == 0
    assert np.abs(N(out) - want).max() <= 2.0 ** -8 * max(1.0, np.abs(want).max())
    # rows divided by the rms of the rows they were rounded from, given as sums of squares in blocks
    nb = 5
    stats = rng.uniform(0.5, 2.0, size=(m, nb)).astype(np.float32)
    eps = 1e-5
    inv = 1.0 / np.sqrt(stats.astype(np.float64).sum(1) / k + eps)
    ops.gemm_pair_tc(x, w, out, T(stats), nb, eps)
    assert ops.gemm_tc_status() == 0
    assert np.abs(N(out) - want * inv[:, None]).max() <= 2.0 ** -8 * max(1.0, np.abs(want * inv[:, None]).max())


@pytest.mark.parametrize("m,i,k", [(300, 200, 72), (130, 128, 64), (512, 4864, 896), (64, 520, 264)])
def test_gemm_pair_tc_silu_mul(m, i, k):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(i + k)
    x = T(rng.normal(size=(m, k)), torch.bfloat16)
    w = T(rng.normal(size=(2 * i, k)) * 0.2, torch.bfloat16)
    g, u = N(x) @ N(w[:i]).T, N(x) @ N(w[i:]).T
    want = g / (1 + np.exp(-g)) * u
    out = torch.full((m, i), 7.0, dtype=torch.bfloat16, device=dev())
    ops.gemm_pair_tc_silu_mul(x, w, out)
    assert ops.gemm_tc_status() == 0
    assert np.abs(N(out) - want).max() <= 2.0 ** -8 * max(1.0, np.abs(want).max()) + 1e-4


@pytest.mark.parametrize("m,n,k", [(300, 200, 72), (129, 136, 264), (512, 896, 4864), (1000, 1536, 512), (3, 24, 16)])
def test_gemm_pair_tc_resadd(m, n, k):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(m + n + k)
    x, w = T(rng.normal(size=(m, k)), torch.bfloat16), T(rng.normal(size=(n, k)) * 0.3, torch.bfloat16)
    res0 = rng.normal(size=(m, n)).astype(np.float32) * 3
    want = res0.astype(np.float64) + N(x) @ N(w).T
    scale = max(1.0, np.abs(want).max())
    res = T(res0)
    nb = ops.gemm_pair_tc_stats_blocks(m, n)
    stats = torch.full((m, nb), -1.0, dtype=torch.float32, device=dev())
    copy = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=dev())
    ops.gemm_pair_tc_resadd(x, w, res, stats, copy)
    assert ops.gemm_tc_status() == 0
    assert np.abs(N(res) - want).max() <= 2e-5 * scale
    assert np.abs(N(copy) - want).max() <= 2.0 ** -8 * scale
    # the sums of squares: one per row and tile of columns, whatever the tile's width; together the row's
    assert (N(stats) >= 0).all()
    rows = (N(res) ** 2).sum(1)
    assert np.abs(N(stats).sum(1) - rows).max() <= 1e-5 * max(1.0, rows.max())


def test_gemm_pair_tc_refuses_widths_that_are_no_multiple_of_8():
    import torch
    from machserve_b200 import ops
    x, w = torch.zeros((4, 16), dtype=torch.bfloat16, device=dev()), torch.zeros((20, 16), dtype=torch.bfloat16, device=dev())
    with pytest.raises(ops.KernelError, match="multiples? of 8"):
        ops.gemm_pair_tc(x, w, torch.zeros((4, 20), dtype=torch.bfloat16, device=dev()))
