"""Each kernel alone against a plain float64 reference of the same operation, at sizes other than the
engine's tiny models: widths and vocabularies that are no power of two, head sizes in steps of 16,
odd numbers of heads and groups, several page sizes, windows that end inside a page."""
import numpy as np
import pytest

from tests.plain.model import bf16_round

pytestmark = pytest.mark.gpu


def dev():
    import torch
    return torch.device("cuda:0")


def T(a, dtype=None):
    import torch
    t = torch.as_tensor(np.ascontiguousarray(a)).to(dev())
    return t.to(dtype) if dtype is not None else t


def N(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


# ------------------------------------------------------------------ elementwise


@pytest.mark.parametrize("rows,d,vocab", [(1, 7, 11), (33, 896, 1000), (5, 1536, 333)])
def test_embed_gather(rows, d, vocab):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(0)
    table = rng.normal(size=(vocab, d)).astype(np.float32)
    ids = rng.integers(0, vocab, size=rows).astype(np.int32)
    for dt in (torch.float32, torch.bfloat16):
        out = torch.empty((rows, d), dtype=torch.float32, device=dev())
        ops.embed_gather(T(table, dt), T(ids), out)
        assert np.array_equal(N(out), N(T(table, dt))[ids])


@pytest.mark.parametrize("rows,d,eps", [(1, 5, 1e-6), (17, 896, 1e-5), (4, 3584, 1e-6), (3, 4099, 1e-3)])
def test_add_rmsnorm(rows, d, eps):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(1)
    res = rng.normal(size=(rows, d)).astype(np.float32) * 3
    delta = rng.normal(size=(rows, d)).astype(np.float32)
    w = (1 + 0.1 * rng.normal(size=d)).astype(np.float32)

    def ref(x):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w.astype(np.float64)

    # no delta, float32 out
    r = T(res); out = torch.empty_like(r)
    ops.add_rmsnorm(r, None, T(w), out, eps)
    assert np.abs(N(out) - ref(res.astype(np.float64))).max() < 1e-5 and np.array_equal(N(r), res)
    # bfloat16 delta, bfloat16 out, residual updated in float32
    r = T(res); d16 = T(delta, torch.bfloat16); out = torch.empty((rows, d), dtype=torch.bfloat16, device=dev())
    ops.add_rmsnorm(r, d16, T(w), out, eps)
    summed = res.astype(np.float64) + N(d16)
    assert np.abs(N(r) - summed).max() < 1e-6
    assert np.abs(N(out) - ref(summed)).max() < 0.02 * np.abs(ref(summed)).max()
    # picked rows: nothing is written back
    rows_idx = np.array([rows - 1, 0, rows - 1], dtype=np.int32)
    r = T(res); out = torch.empty((3, d), dtype=torch.float32, device=dev())
    ops.add_rmsnorm(r, T(delta), T(w), out, eps, T(rows_idx))
    assert np.array_equal(N(r), res)
    assert np.abs(N(out) - ref(res.astype(np.float64) + delta)[rows_idx]).max() < 1e-5


@pytest.mark.parametrize("rows,inter", [(1, 3), (9, 4864), (130, 200)])
def test_silu_mul(rows, inter):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(2)
    gu = (rng.normal(size=(rows, 2 * inter)) * 4).astype(np.float32)
    g, u = gu[:, :inter].astype(np.float64), gu[:, inter:].astype(np.float64)
    out = torch.empty((rows, inter), dtype=torch.float32, device=dev())
    ops.silu_mul(T(gu), out)
    want = g / (1 + np.exp(-g)) * u
    assert (np.abs(N(out) - want) <= 1e-6 * np.abs(want) + 1e-7).all()  # a few float32 roundings per element
    g16 = T(gu, torch.bfloat16); out = torch.empty((rows, inter), dtype=torch.bfloat16, device=dev())
    ops.silu_mul(g16, out)
    g, u = N(g16)[:, :inter], N(g16)[:, inter:]
    want = g / (1 + np.exp(-g)) * u
    assert np.abs(N(out) - want).max() <= 2.0 ** -8 * np.abs(want).max() + 1e-6


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 67, 33), (64, 64, 16), (70, 130, 200), (3, 1000, 896), (257, 96, 72)])
def test_gemm_f32(m, n, k):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(3)
    x, w, b = rng.normal(size=(m, k)).astype(np.float32), rng.normal(size=(n, k)).astype(np.float32), rng.normal(size=n).astype(np.float32)
    out = torch.empty((m, n), dtype=torch.float32, device=dev())
    ops.gemm_f32(T(x), T(w), T(b), out)
    want = x.astype(np.float64) @ w.astype(np.float64).T + b
    assert np.abs(N(out) - want).max() < 1e-5 * max(1, np.abs(want).max())
    # a row's result does not depend on the rows computed with it
    one = torch.empty((1, n), dtype=torch.float32, device=dev())
    ops.gemm_f32(T(x[m // 2 : m // 2 + 1]), T(w), T(b), one)
    assert torch.equal(one[0], out[m // 2])


@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (8, 1152, 896), (5, 30, 72), (64, 896, 4864), (17, 400, 200),
                                   (3, 151936, 896), (33, 7, 8), (9, 1000, 136), (64, 9728, 896)])
def test_gemm_small_m(m, n, k):
    """The weight-streaming kernel for few rows: any N, K in steps of 8, bfloat16 and float32 out."""
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(m * 1000 + k)
    x, w = T(rng.normal(size=(m, k)), torch.bfloat16), T(rng.normal(size=(n, k)) * 0.5, torch.bfloat16)
    want = N(x) @ N(w).T
    scale = max(1.0, np.abs(want).max())
    out32 = torch.full((m, n), 7.0, dtype=torch.float32, device=dev())
    ops.gemm_small_m(x, w, out32)
    assert np.abs(N(out32) - want).max() <= 2e-5 * scale  # float32 sums of exact bfloat16 products
    out16 = torch.empty((m, n), dtype=torch.bfloat16, device=dev())
    ops.gemm_small_m(x, w, out16)
    assert np.abs(N(out16) - want).max() <= 2.0 ** -8 * scale
    # the same rows alone give the same bits: a row's sum does not depend on the others
    one = torch.empty((1, n), dtype=torch.float32, device=dev())
    ops.gemm_small_m(x[m - 1 :], w, one)
    assert torch.equal(one[0], out32[m - 1])
    # rows with a stride (a slice of a wider buffer)
    wide = torch.zeros((m, k + 24), dtype=torch.bfloat16, device=dev()); wide[:, :k] = x
    out_s = torch.empty((m, n), dtype=torch.float32, device=dev())
    ops.gemm_small_m(wide[:, :k], w, out_s)
    assert torch.equal(out_s, out32)


@pytest.mark.parametrize("m,i,k", [(1, 8, 32), (8, 4864, 896), (7, 200, 96), (64, 136, 72), (20, 8960, 1536)])
def test_gemm_small_m_silu_mul(m, i, k):
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(i + k)
    x = T(rng.normal(size=(m, k)), torch.bfloat16)
    wg, wu = T(rng.normal(size=(i, k)) * 0.2, torch.bfloat16), T(rng.normal(size=(i, k)) * 0.2, torch.bfloat16)
    g, u = N(x) @ N(wg).T, N(x) @ N(wu).T
    want = g / (1 + np.exp(-g)) * u
    out = torch.empty((m, i), dtype=torch.bfloat16, device=dev())
    ops.gemm_small_m_silu_mul(x, wg, wu, out)
    assert np.abs(N(out) - want).max() <= 2.0 ** -8 * max(1.0, np.abs(want).max()) + 1e-4


@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (8, 896, 896), (13, 72, 136), (16, 896, 4864), (5, 100, 200)])
def test_gemm_small_m_resadd_and_norm(m, n, k):
    """The fused forms: the product added into the float32 residual, with per-block sums of squares and a rounded
    copy of the new residual; and the product of that copy whose rows are divided by their rms made from those sums."""
    import torch
    from machserve_b200 import ops
    rng = np.random.default_rng(m + n + k)
    x, w = T(rng.normal(size=(m, k)), torch.bfloat16), T(rng.normal(size=(n, k)) * 0.3, torch.bfloat16)
    res0 = rng.normal(size=(m, n)).astype(np.float32) * 3
    res = T(res0)
    nb = ops.gemm_small_m_stats_blocks(n)
    stats = torch.full((m, nb), float("nan"), dtype=torch.float32, device=dev())
    copy = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=dev())
    ops.gemm_small_m_resadd(x, w, res, stats, copy)
    assert torch.equal(copy, res.to(torch.bfloat16))  # the new residual, rounded once
    want = res0.astype(np.float64) + N(x) @ N(w).T
    assert np.abs(N(res) - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    ss = np.stack([(N(res)[:, b * 16 : (b + 1) * 16] ** 2).sum(-1) for b in range(nb)], axis=1)
    assert np.abs(N(stats) - ss).max() <= 1e-5 * max(1.0, ss.max())
    # the consumer (plain, and gate/up with SiLU)
    eps = 1e-5
    cols = 4864 if (n, k) == (896, 896) else 40  # the wide one: blocks of four warps, every chunk staged
    w2, w3 = T(rng.normal(size=(cols, n)) * 0.2, torch.bfloat16), T(rng.normal(size=(cols, n)) * 0.2, torch.bfloat16)
    r = N(res)
    if n % 8 == 0:
        out = torch.empty((m, cols), dtype=torch.bfloat16, device=dev())
        # the rounded residual times a matrix (that would have the norm's weight folded in), the rows divided by
        # their rms in the epilogue
        inv = 1.0 / np.sqrt((r * r).mean(-1, keepdims=True) + eps)
        ops.gemm_small_m_scaled(copy, stats, nb, eps, w2, None, out)
        want4 = N(copy) @ N(w2).T * inv
        assert np.abs(N(out) - want4).max() <= 2.0 ** -7 * max(1.0, np.abs(want4).max())
        ops.gemm_small_m_scaled(copy, stats, nb, eps, w2, w3, out)
        g, u = N(copy) @ N(w2).T * inv, N(copy) @ N(w3).T * inv
        want5 = g / (1 + np.exp(-g)) * u
        assert np.abs(N(out) - want5).max() <= 2.0 ** -7 * max(1.0, np.abs(want5).max()) + 1e-3


def test_gemm_small_m_refuses_what_it_does_not_cover():
    import torch
    from machserve_b200 import ops
    assert not ops.gemm_small_m_supports(65, 16, 32) and not ops.gemm_small_m_supports(4, 16, 36)
    x, w = torch.zeros((4, 36), dtype=torch.bfloat16, device=dev()), torch.zeros((16, 36), dtype=torch.bfloat16, device=dev())
    with pytest.raises(ops.KernelError, match="K=36"):
        ops.gemm_small_m(x, w, torch.empty((4, 16), dtype=torch.float32, device=dev()))


# ------------------------------------------------------------- cache + attention


class PagedCase:
    """Random sequences laid out in shuffled pages, with the arrays the kernels take."""

    def __init__(self, lens, hq, hkv, hd, page, window=None, seed=0, dtype="bfloat16", extra_pages=3, k_gain=None):
        import torch
        rng = np.random.default_rng(seed)
        self.lens, self.hq, self.hkv, self.hd, self.page, self.window = lens, hq, hkv, hd, page, window
        self.tdtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        rnd = (lambda a: bf16_round(a.astype(np.float32)).astype(np.float64)) if dtype == "bfloat16" else (lambda a: a.astype(np.float32).astype(np.float64))
        self.k = [rnd(rng.normal(size=(n, hkv, hd))) for n in lens]
        if k_gain:  # keys grow with their position, and so does a row's largest score from tile to tile
            self.k = [rnd(k * (1.0 + np.arange(len(k)) / k_gain)[:, None, None]) for k in self.k]
        self.v = [rnd(rng.normal(size=(n, hkv, hd))) for n in lens]
        max_pages = max(-(-n // page) for n in lens) + 1
        total = sum(-(-n // page) for n in lens) + extra_pages
        perm = rng.permutation(total)
        self.num_pages = total
        kp = rng.normal(size=(total, hkv, page, hd)) * 50  # pages no table points to hold garbage
        vp = rng.normal(size=(total, hkv, page, hd)) * 50
        table = -np.ones((len(lens) + 2, max_pages), dtype=np.int32)
        self.slots = list(rng.permutation(len(lens) + 2)[: len(lens)])
        at = 0
        for s, n in enumerate(lens):
            for i in range(-(-n // page)):
                pg = int(perm[at]); at += 1
                table[self.slots[s], i] = pg
                rows = slice(i * page, min((i + 1) * page, n))
                cnt = rows.stop - rows.start
                kp[pg, :, :cnt] = self.k[s][rows].transpose(1, 0, 2)
                vp[pg, :, :cnt] = self.v[s][rows].transpose(1, 0, 2)
        self.k_pages, self.v_pages, self.table = T(kp, self.tdtype), T(vp, self.tdtype), T(table)
        self.rnd = rnd

    def queries(self, rows, seed=1, scale_one=None):
        """rows: list of (sequence, position).  Returns q [T, hq*hd] and the reference output."""
        rng = np.random.default_rng(seed)
        q = self.rnd(rng.normal(size=(len(rows), self.hq, self.hd)))
        for r, h, key in ([] if scale_one is None else scale_one if isinstance(scale_one, list) else [scale_one]):
            s, _ = rows[r]  # make one key stand out for this row and head
            q[r, h] = self.rnd(self.k[s][key, h // (self.hq // self.hkv)] * 4.0)
        want = np.zeros_like(q)
        g = self.hq // self.hkv
        for r, (s, pos) in enumerate(rows):
            lo = max(0, pos - self.window + 1) if self.window else 0
            for h in range(self.hq):
                kk, vv = self.k[s][lo : pos + 1, h // g], self.v[s][lo : pos + 1, h // g]
                sc = kk @ q[r, h] * self.hd ** -0.5
                e = np.exp(sc - sc.max())
                want[r, h] = e @ vv / e.sum()
        pos = np.array([p for _, p in rows], dtype=np.int32)
        slot = np.array([self.slots[s] for s, _ in rows], dtype=np.int32)
        return q.reshape(len(rows), -1), want.reshape(len(rows), -1), T(pos), T(slot)


ATT_CASES = [
    # lens, hq, hkv, hd, page, window
    ([1, 2, 70], 4, 2, 16, 16, None),
    ([300, 17, 64, 65], 14, 2, 64, 64, None),
    ([129, 40], 3, 1, 32, 8, None),
    ([200, 33], 6, 2, 48, 8, 11),
    ([500, 90], 12, 2, 128, 16, 100),
    ([77], 5, 5, 80, 4, 64),
    ([260, 64], 28, 4, 128, 32, None),
    ([150], 16, 1, 96, 16, None),
]


@pytest.mark.parametrize("lens,hq,hkv,hd,page,window", ATT_CASES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_generic(lens, hq, hkv, hd, page, window, dtype):
    import torch
    from machserve_b200 import ops
    case = PagedCase(lens, hq, hkv, hd, page, window, dtype=dtype)
    rows = [(s, p) for s, n in enumerate(lens) for p in sorted({0, n // 2, n - 1, max(0, n - 2)})]
    q, want, pos, slot = case.queries(rows, scale_one=(len(rows) - 1, hq - 1, 0) if not window else None)
    out = torch.empty((len(rows), hq * hd), dtype=case.tdtype, device=dev())
    ops.attention_generic(T(q, case.tdtype), case.k_pages, case.v_pages, out, pos, slot, case.table, hq, hkv, hd, window, hd ** -0.5)
    tol = 2e-6 if dtype == "float32" else 2.0 ** -8
    assert np.abs(N(out) - want).max() <= tol * max(1.0, np.abs(want).max()) + 1e-6


@pytest.mark.parametrize("lens,hq,hkv,hd,page,window", ATT_CASES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_generic_rows_that_share_tiles(lens, hq, hkv, hd, page, window, dtype):
    """Portions of prompts (runs of consecutive rows, cut anywhere, next to single rows of other sequences): eight rows
    a block share the tiles they read, and every row comes out with the same bits as when it is computed alone."""
    import torch
    from machserve_b200 import ops
    case = PagedCase(lens, hq, hkv, hd, page, window, dtype=dtype)
    rows = []
    for s, n in enumerate(lens):
        if s % 3 == 2:
            rows += [(s, n - 1)]                                # a single row
        else:
            a = max(0, n - 45) if s % 2 else 0                  # a portion at the end of a sequence, or from its start
            rows += [(s, p) for p in range(a, min(n, a + 77))]  # (no multiple of eight rows, and across tiles of 32 keys)
    q, want, pos, slot = case.queries(rows)
    alone = torch.empty((len(rows), hq * hd), dtype=case.tdtype, device=dev())
    ops.attention_generic(T(q, case.tdtype), case.k_pages, case.v_pages, alone, pos, slot, case.table, hq, hkv, hd, window, hd ** -0.5)
    shared = torch.full((len(rows), hq * hd), 7.0, dtype=case.tdtype, device=dev())
    ops.attention_generic(T(q, case.tdtype), case.k_pages, case.v_pages, shared, pos, slot, case.table, hq, hkv, hd, window, hd ** -0.5,
                          share_rows=True)
    tol = 2e-6 if dtype == "float32" else 2.0 ** -8
    assert np.abs(N(shared) - want).max() <= tol * max(1.0, np.abs(want).max()) + 1e-6
    assert torch.equal(shared.view(torch.int32 if dtype == "float32" else torch.int16), alone.view(torch.int32 if dtype == "float32" else torch.int16))
    if dtype == "float32" and hd % 4 == 0 and hd <= 128:
        # the float32 decoding form (the warps of a row as the blocks of a cluster), with 1 to 8 heads of a group to a block
        for heads in (1, 2, 4, 8):
            spread = torch.full((len(rows), hq * hd), 7.0, dtype=case.tdtype, device=dev())
            ops.attention_generic(T(q, case.tdtype), case.k_pages, case.v_pages, spread, pos, slot, case.table, hq, hkv, hd, window,
                                  hd ** -0.5, share_rows=-heads)
            assert torch.equal(spread.view(torch.int32), shared.view(torch.int32)), f"{heads} heads a block"


@pytest.mark.parametrize("lens,hq,hkv,hd,page,window", ATT_CASES)
@pytest.mark.parametrize("splits", [1, 2, 5])
def test_attention_decode(lens, hq, hkv, hd, page, window, splits):
    import torch
    from machserve_b200 import ops
    if not ops.attention_decode_supports(hd, hq // hkv):
        pytest.skip("size not covered by the fast kernel (the engine then uses the exact kernel)")
    case = PagedCase(lens, hq, hkv, hd, page, window)
    rows = [(s, p) for s, n in enumerate(lens) for p in sorted({0, n // 2, n - 1, max(0, n - 2), min(n - 1, 63), min(n - 1, 64)})]
    # the last row's last head looks at one far key among hundreds: key 1 of the longest sequence
    far = (len(rows) - 1, hq - 1, max(0, rows[-1][1] - window + 1) if window else 1)
    q, want, pos, slot = case.queries(rows, scale_one=far)
    out = torch.full((len(rows), hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
    n = ops.attention_decode_scratch_words(len(rows), hq, hkv, hd, splits)
    scratch = torch.full((max(n, 1),), float("nan"), dtype=torch.float32, device=dev())
    if splits > 1:
        scratch[n - len(rows) * hkv :] = 0  # the counters start at zero; every launch leaves them so
    ops.attention_decode(T(q, torch.bfloat16), case.k_pages, case.v_pages, out, scratch, pos, slot, case.table, hq, hkv, hd, window, hd ** -0.5, splits)
    # a list of rows: only those are attended, the others keep what they held
    pick = np.array(sorted(set(range(0, len(rows), 2)) | {len(rows) - 1}), dtype=np.int32)
    out2 = torch.full((len(rows), hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
    n = ops.attention_decode_scratch_words(len(pick), hq, hkv, hd, splits)  # the counters' place depends on the row count
    scratch = torch.zeros((max(n, 1),), dtype=torch.float32, device=dev())
    ops.attention_decode(T(q, torch.bfloat16), case.k_pages, case.v_pages, out2, scratch, pos, slot, case.table, hq, hkv, hd, window, hd ** -0.5, splits, rows=T(pick), num_rows=len(pick))
    assert torch.equal(out2[T(pick).long()], out[T(pick).long()])
    rest = np.setdiff1d(np.arange(len(rows)), pick)
    assert (N(out2)[rest] == 7.0).all()
    if splits > 1:
        assert not scratch[n - len(pick) * hkv :].any()
    # probabilities are rounded to bfloat16 before they multiply the values: 2^-8 relative per term
    assert np.abs(N(out) - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("lens,hq,hkv,hd,page,window", ATT_CASES)
@pytest.mark.parametrize("splits,stages,warps,kpw", [(1, 1, 4, 0), (2, 8, 4, 0), (4, 2, 4, 0), (8, 1, 4, 0), (8, 8, 4, 0), (1, 4, 8, 0), (2, 8, 8, 0),
                                                     (8, 5, 8, 0), (2, 2, 4, 16), (4, 1, 4, 32), (1, 3, 4, 64), (8, 4, 4, 16), (2, 4, 8, 16), (1, 8, 4, 64), (1, 2, 4, 16)])
def test_attention_decode_cluster(lens, hq, hkv, hd, page, window, splits, stages, warps, kpw):
    """The cluster variant: splits merged in shared memory, several tiles in flight, the current row copied late;
    four warps with a tile, half or a quarter of a tile each (`kpw`; 0: the kernel's own rule), and eight warps with
    half a tile each."""
    import torch
    from machserve_b200 import ops
    if not ops.attention_decode_supports(hd, hq // hkv):
        pytest.skip("size not covered by the fast kernel (the engine then uses the exact kernel)")
    stages = min(stages, ops.attention_decode_cluster_max_stages(hd))
    case = PagedCase(lens, hq, hkv, hd, page, window, seed=splits)
    rows = [(s, p) for s, n in enumerate(lens) for p in sorted({0, n // 2, n - 1, max(0, n - 2), min(n - 1, 63), min(n - 1, 64)})]
    far = (len(rows) - 1, hq - 1, max(0, rows[-1][1] - window + 1) if window else 1)
    q, want, pos, slot = case.queries(rows, scale_one=far)
    out = torch.full((len(rows) + 1, hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
    q16 = torch.cat([T(q, torch.bfloat16), torch.zeros((1, hq * hd), dtype=torch.bfloat16, device=dev())])
    pos1 = torch.cat([pos, torch.zeros(1, dtype=torch.int32, device=dev())])
    slot1 = torch.cat([slot, torch.full((1,), -1, dtype=torch.int32, device=dev())])  # a padding row at the end
    ops.attention_decode_cluster(q16, case.k_pages, case.v_pages, out, pos1, slot1, case.table, hq, hkv, hd, window,
                                 hd ** -0.5, splits, stages, warps=warps, keys_per_warp=kpw)
    assert np.abs(N(out[:-1]) - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
    assert (N(out[-1]) == 7.0).all()  # nothing is written for the padding row
    pick = np.array(sorted(set(range(0, len(rows), 2)) | {len(rows) - 1}), dtype=np.int32)
    out2 = torch.full((len(rows) + 1, hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
    ops.attention_decode_cluster(q16, case.k_pages, case.v_pages, out2, pos1, slot1, case.table, hq, hkv, hd, window,
                                 hd ** -0.5, splits, stages, rows=T(pick), num_rows=len(pick), warps=warps, keys_per_warp=kpw)
    assert torch.equal(out2[T(pick).long()], out[T(pick).long()])
    assert (N(out2)[np.setdiff1d(np.arange(len(rows)), pick)] == 7.0).all()


@pytest.mark.parametrize("lens,hq,hkv,hd,page,window", ATT_CASES)
@pytest.mark.parametrize("splits,stages,warps,kpw,parts", [(8, 2, 4, 0, 2), (8, 5, 8, 0, 4), (4, 1, 4, 16, 3), (2, 8, 4, 0, 16), (8, 4, 4, 16, 8)])
def test_attention_decode_cluster_in_several_clusters(lens, hq, hkv, hd, page, window, splits, stages, warps, kpw, parts):
    """A row's keys spread over several clusters (few rows with long contexts): each leaves its sums in scratch memory,
    the one that ends last merges them in order.  Against the plain reference, with a far key that stands out, rows
    whose few keys leave most clusters without any, a padding row, a list of rows; launched twice on the same scratch
    and counters (which every launch leaves zero); and the fused form against the two kernels it stands for."""
    import torch
    from machserve_b200 import ops
    from machserve_b200.config import part
    from machserve_b200.parts import Runtime, Workspace
    from machserve_b200.parts.rope import RotaryEncoding
    if not ops.attention_decode_supports(hd, hq // hkv):
        pytest.skip("size not covered by the fast kernel (the engine then uses the exact kernel)")
    stages = min(stages, ops.attention_decode_cluster_max_stages(hd))
    case = PagedCase(lens, hq, hkv, hd, page, window, seed=20 + parts)
    rows = [(s, p) for s, n in enumerate(lens) for p in sorted({0, n // 2, n - 1, max(0, n - 2), min(n - 1, 63), min(n - 1, 64)})]
    far = (len(rows) - 1, hq - 1, max(0, rows[-1][1] - window + 1) if window else 1)
    q, want, pos, slot = case.queries(rows, scale_one=far)
    n = len(rows) + 1
    q16 = torch.cat([T(q, torch.bfloat16), torch.zeros((1, hq * hd), dtype=torch.bfloat16, device=dev())])
    pos1 = torch.cat([pos, torch.zeros(1, dtype=torch.int32, device=dev())])
    slot1 = torch.cat([slot, torch.full((1,), -1, dtype=torch.int32, device=dev())])  # a padding row at the end
    words = ops.attention_decode_cluster_scratch_words(n, hq, hkv, hd, parts)
    scratch = torch.full((words,), float("nan"), dtype=torch.float32, device=dev())
    counters = torch.zeros(n * hkv, dtype=torch.int32, device=dev())
    kw = dict(warps=warps, keys_per_warp=kpw, parts=parts, scratch=scratch, counters=counters)
    if hd not in (64, 128):  # built for the two common head sizes; the others are refused, by name
        with pytest.raises(ops.KernelError, match="head sizes 64 and 128"):
            ops.attention_decode_cluster(q16, case.k_pages, case.v_pages, torch.empty_like(q16), pos1, slot1, case.table, hq, hkv, hd,
                                         window, hd ** -0.5, splits, stages, **kw)
        return
    for _ in range(2):
        out = torch.full((n, hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
        ops.attention_decode_cluster(q16, case.k_pages, case.v_pages, out, pos1, slot1, case.table, hq, hkv, hd, window,
                                     hd ** -0.5, splits, stages, **kw)
        assert np.abs(N(out[:-1]) - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
        assert (N(out[-1]) == 7.0).all()  # nothing is written for the padding row
        assert not counters.any()
    pick = np.array(sorted(set(range(0, len(rows), 2)) | {len(rows) - 1}), dtype=np.int32)
    out2 = torch.full((n, hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
    ops.attention_decode_cluster(q16, case.k_pages, case.v_pages, out2, pos1, slot1, case.table, hq, hkv, hd, window,
                                 hd ** -0.5, splits, stages, rows=T(pick), num_rows=len(pick), **kw)
    assert torch.equal(out2[T(pick).long()], out[T(pick).long()])
    assert (N(out2)[np.setdiff1d(np.arange(len(rows)), pick)] == 7.0).all()
    with pytest.raises(ops.KernelError, match="scratch"):
        ops.attention_decode_cluster(q16, case.k_pages, case.v_pages, out2, pos1, slot1, case.table, hq, hkv, hd, window,
                                     hd ** -0.5, splits, stages, warps=warps, keys_per_warp=kpw, parts=parts, scratch=scratch[:-1],
                                     counters=counters)
    # the fused form: one row per sequence at its end, its key and value written by the block whose run holds the position
    rng = np.random.default_rng(5)
    last = [(s, n_ - 1) for s, n_ in enumerate(lens)]
    pos_l = np.array([p for _, p in last], dtype=np.int32)
    slot_l = np.array([case.slots[s] for s, _ in last], dtype=np.int32)
    pe = RotaryEncoding(part("rope", head_dim=hd, rotary_dim=hd, theta=30000.0, pairing="half"))
    table = pe.rotary_table(Runtime(torch.bfloat16, dev(), Workspace(dev()), max(lens) + 1))
    width = (hq + 2 * hkv) * hd
    qkv = T(rng.normal(size=(len(last), width)), torch.bfloat16)
    bias = T(rng.normal(size=width).astype(np.float32))
    k1, v1 = case.k_pages.clone(), case.v_pages.clone()
    q1 = torch.zeros((len(last), hq * hd), dtype=torch.bfloat16, device=dev())
    ops.rope_kv_store(qkv, bias, T(pos_l), T(slot_l), case.table, table, hd, False, q1, k1, v1, hq, hkv, hd)
    two = torch.empty((len(last), hq * hd), dtype=torch.bfloat16, device=dev())
    ops.attention_decode_cluster(q1, k1, v1, two, T(pos_l), T(slot_l), case.table, hq, hkv, hd, window, hd ** -0.5, splits, stages, **kw)
    k2, v2 = case.k_pages.clone(), case.v_pages.clone()
    one = torch.empty_like(two)
    ops.attention_decode_cluster_rope(qkv, bias, table, True, k2, v2, one, T(pos_l), T(slot_l), case.table, hq, hkv, hd,
                                      window, hd ** -0.5, splits, stages, **kw)
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert np.abs(N(one) - N(two)).max() <= 2.0 ** -8 * max(1.0, np.abs(N(two)).max())
    assert not counters.any()


@pytest.mark.parametrize("lens,hq,hkv,hd,page,window", ATT_CASES)
@pytest.mark.parametrize("splits,stages,store,warps", [(1, 1, True, 4), (2, 8, True, 4), (4, 2, True, 4), (8, 1, True, 4), (8, 8, False, 4),
                                                       (2, 1, False, 4), (1, 4, True, 8), (8, 8, True, 8), (2, 5, False, 8)])
def test_attention_decode_cluster_rope(lens, hq, hkv, hd, page, window, splits, stages, store, warps):
    """The fused form (bias, rotation, cache write and attention in one kernel) against the two kernels it stands
    for, on copies of the same cache: one row per sequence, at the end, at tile and page edges and at position 0,
    with the current position's tile in the first round of a block and in a later one."""
    import torch
    from machserve_b200 import ops
    from machserve_b200.config import part
    from machserve_b200.parts import Runtime, Workspace
    from machserve_b200.parts.rope import RotaryEncoding
    if not ops.attention_decode_supports(hd, hq // hkv):
        pytest.skip("size not covered by the fast kernel (the engine then uses the exact kernel)")
    stages = min(stages, ops.attention_decode_cluster_max_stages(hd))
    case = PagedCase(lens, hq, hkv, hd, page, window, seed=10 + splits)
    rng = np.random.default_rng(3)
    choices = [lambda n: n - 1, lambda n: min(n - 1, 63), lambda n: min(n - 1, 64), lambda n: n // 2, lambda n: 0,
               lambda n: (n - 1) // page * page]
    rows = [(s, choices[s % len(choices)](n)) for s, n in enumerate(lens)]
    pos = np.array([p for _, p in rows] + [0], dtype=np.int32)
    slot = np.array([case.slots[s] for s, _ in rows] + [-1], dtype=np.int32)  # a padding row at the end
    pe = RotaryEncoding(part("rope", head_dim=hd, rotary_dim=hd, theta=30000.0, pairing="half"))
    table = pe.rotary_table(Runtime(torch.bfloat16, dev(), Workspace(dev()), max(lens) + 1))
    width = (hq + (2 * hkv if store else 0)) * hd
    qkv = T(rng.normal(size=(len(rows) + 1, width + 8)), torch.bfloat16)[:, :width]  # a wider row stride
    bias = T(rng.normal(size=width).astype(np.float32))
    scale = hd ** -0.5
    # the two kernels
    k1, v1 = case.k_pages.clone(), case.v_pages.clone()
    q1 = torch.zeros((len(rows) + 1, hq * hd), dtype=torch.bfloat16, device=dev())
    ops.rope_kv_store(qkv, bias, T(pos), T(slot), case.table, table, hd, False, q1, k1 if store else None,
                      v1 if store else None, hq, hkv if store else 0, hd)
    want = torch.full((len(rows) + 1, hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
    ops.attention_decode_cluster(q1, k1, v1, want, T(pos), T(slot), case.table, hq, hkv, hd, window, scale, splits, stages,
                                 warps=warps)
    # the one kernel
    k2, v2 = case.k_pages.clone(), case.v_pages.clone()
    got = torch.full((len(rows) + 1, hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
    ops.attention_decode_cluster_rope(qkv, bias, table, store, k2, v2, got, T(pos), T(slot), case.table, hq, hkv, hd,
                                      window, scale, splits, stages, warps=warps)
    assert torch.equal(k1, k2) and torch.equal(v1, v2)  # same arithmetic, same rounding, same places
    if store:
        assert not torch.equal(k1, case.k_pages)
    assert (N(got[-1]) == 7.0).all()
    assert np.abs(N(got[:-1]) - N(want[:-1])).max() <= 2.0 ** -8 * max(1.0, np.abs(N(want[:-1])).max())
    # and without a bias
    k3, v3 = case.k_pages.clone(), case.v_pages.clone()
    ops.rope_kv_store(qkv, None, T(pos), T(slot), case.table, table, hd, False, q1, k1 if store else None,
                      v1 if store else None, hq, hkv if store else 0, hd)
    ops.attention_decode_cluster(q1, k1, v1, want, T(pos), T(slot), case.table, hq, hkv, hd, window, scale, splits, stages,
                                 warps=warps)
    ops.attention_decode_cluster_rope(qkv, None, table, store, k3, v3, got, T(pos), T(slot), case.table, hq, hkv, hd,
                                      window, scale, splits, stages, warps=warps)
    assert torch.equal(k1, k3) and torch.equal(v1, v3)
    assert np.abs(N(got[:-1]) - N(want[:-1])).max() <= 2.0 ** -8 * max(1.0, np.abs(N(want[:-1])).max())


@pytest.mark.parametrize("lens,hq,hkv,hd,page,window", ATT_CASES)
def test_attention_prefill(lens, hq, hkv, hd, page, window):
    """Portions of sequences in tiles of up to 64 rows: a portion at the start of a sequence, one that
    begins and ends inside pages and tiles, and short ones, each after keys written by earlier steps."""
    import torch
    from machserve_b200 import ops
    if not ops.attention_prefill_supports(hd):
        pytest.skip("size not covered by the fast kernel (the engine then uses the exact kernel)")
    case = PagedCase(lens, hq, hkv, hd, page, window)
    rows, tile0, tilen = [], [], []
    for s, n in enumerate(lens):
        portions = [(0, min(n, 70))] if s % 2 == 0 else [(max(0, n - 37), n)]
        if n > 150:
            portions = [(61, 61 + 131)]
        for a, b in portions:
            for t0 in range(a, b, 64):
                tile0.append(len(rows)); tilen.append(min(64, b - t0))
                rows += [(s, p) for p in range(t0, min(t0 + 64, b))]
    far = (len(rows) - 1, hq - 1, max(0, rows[-1][1] - window + 1) if window else 0)
    q, want, pos, slot = case.queries(rows, scale_one=far)
    out = torch.full((len(rows), hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
    ops.attention_prefill(T(q, torch.bfloat16), case.k_pages, case.v_pages, out, T(np.array(tile0, dtype=np.int32)),
                          T(np.array(tilen, dtype=np.int32)), len(tile0), pos, slot, case.table, hq, hkv, hd, window, hd ** -0.5)
    err = np.abs(N(out) - want).max(axis=1)
    assert err.max() <= 2.0 ** -7 * max(1.0, np.abs(want).max()), f"worst row {int(err.argmax())} of {len(rows)}: {rows[int(err.argmax())]}"


TC_ATT_CASES = [
    # lens, hq, hkv, hd, page, window
    ([300, 17, 64, 65], 14, 2, 64, 64, None),
    ([500, 90], 12, 2, 128, 16, 100),
    ([260, 64], 28, 4, 128, 32, None),
    ([129, 40], 3, 1, 64, 8, None),
    ([700], 4, 2, 64, 128, 200),
    ([1100, 3], 2, 1, 64, 256, None),
]


@pytest.mark.parametrize("splits,alone,run_tiles", [(1, False, 0), (2, False, 0), (3, False, 0), (4, False, 0), (1, True, 0), (3, True, 0),
                                                    (2, False, 2), (4, False, 1), (3, True, 2)])
@pytest.mark.parametrize("lens,hq,hkv,hd,page,window", TC_ATT_CASES)
def test_attention_prefill_tc(lens, hq, hkv, hd, page, window, splits, alone, run_tiles):
    """The tcgen05 kernel for portions of prompts: tiles of up to 128 rows, pages of several sizes, windows; the key
    tiles of every (tile, head) in one run or split over two to four blocks that merge through scratch memory; at
    head size 128 two heads of a group per block, or one (`alone`); every item cut, or only those with more than
    `run_tiles` key tiles.  Run twice on the same scratch memory: a launch
    leaves its counters as it found them."""
    import torch
    from machserve_b200 import ops
    assert ops.attention_prefill_tc_supports(hd, page)
    if alone and hd == 64:
        pytest.skip("at head size 64 a block always takes one head")
    case = PagedCase(lens, hq, hkv, hd, page, window)
    rows, tile0, tilen = [], [], []
    for s, n in enumerate(lens):
        portions = [(0, min(n, 150))] if s % 2 == 0 else [(max(0, n - 37), n)]
        if n > 250:
            portions = [(61, min(n, 61 + 300))]
        for a, b in portions:
            for t0 in range(a, b, 128):
                tile0.append(len(rows)); tilen.append(min(128, b - t0))
                rows += [(s, p) for p in range(t0, min(t0 + 128, b))]
    far = (len(rows) - 1, hq - 1, max(0, rows[-1][1] - window + 1) if window else 0)
    q, want, pos, slot = case.queries(rows, scale_one=far)
    words = ops.attention_prefill_tc_scratch_words(len(tile0), hq, hd, splits)
    assert (words == 0) == (splits == 1)
    # the scratch memory starts as garbage: only the counters have to be zero
    scratch = torch.full((words,), float("nan"), dtype=torch.float32, device=dev()) if words else None
    counters = torch.zeros(len(tile0) * hq, dtype=torch.int32, device=dev()) if words else None
    for again in range(2):
        out = torch.full((len(rows), hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
        ops.attention_prefill_tc(T(q, torch.bfloat16), case.k_pages, case.v_pages, out, T(np.array(tile0, dtype=np.int32)),
                                 T(np.array(tilen, dtype=np.int32)), len(tile0), pos, slot, case.table, hq, hkv, hd, window,
                                 hd ** -0.5, splits, scratch, counters, alone=alone, run_tiles=run_tiles)
        assert ops.gemm_tc_status() == 0
        err = np.abs(N(out) - want).max(axis=1)
        assert err.max() <= 2.0 ** -7 * max(1.0, np.abs(want).max()), f"worst row {int(err.argmax())} of {len(rows)}: {rows[int(err.argmax())]}"
    if scratch is not None:
        assert int(counters.abs().sum()) == 0, "the counters were not left at zero"
        with pytest.raises(ops.KernelError, match="words of scratch"):
            ops.attention_prefill_tc(T(q, torch.bfloat16), case.k_pages, case.v_pages, out, T(np.array(tile0, dtype=np.int32)),
                                     T(np.array(tilen, dtype=np.int32)), len(tile0), pos, slot, case.table, hq, hkv, hd, window,
                                     hd ** -0.5, splits, scratch[:-1], counters)
        with pytest.raises(ops.KernelError, match="counters"):
            ops.attention_prefill_tc(T(q, torch.bfloat16), case.k_pages, case.v_pages, out, T(np.array(tile0, dtype=np.int32)),
                                     T(np.array(tilen, dtype=np.int32)), len(tile0), pos, slot, case.table, hq, hkv, hd, window,
                                     hd ** -0.5, splits, scratch, counters[:-1])


def test_attention_prefill_tc_split_policy():
    """Few tiles of rows against many keys are split; a launch that fills the GPU by itself is not."""
    from machserve_b200 import ops
    assert ops.attention_prefill_tc_plan(64, 14, 2, 64, 8192)[:2] == (1, False)
    assert ops.attention_prefill_tc_plan(4, 14, 2, 64, 2048)[:2] == (4, False)
    assert ops.attention_prefill_tc_plan(16, 14, 2, 64, 2048, 136) == (1, False, 0)  # 224 blocks for 296 places
    # head size 128, by the model of the launch's time
    assert ops.attention_prefill_tc_plan(64, 12, 2, 128, 8192, 2080)[:2] == (1, False)  # a long prompt whole: two heads a block
    assert ops.attention_prefill_tc_plan(16, 12, 2, 128, 2048, 136) == (2, False, 8)    # 96 blocks, the longest of 16 key tiles: those of more than 8 in two runs
    assert ops.attention_prefill_tc_plan(32, 28, 4, 128, 4096)[:2] == (1, False)        # 512 blocks: nothing to gain
    assert ops.attention_prefill_tc_plan(4, 28, 4, 128, 4096, 122)[:2] == (2, False)    # 64 blocks of equal length: 128, not 192
    assert ops.attention_prefill_tc_plan(4, 12, 2, 128, 2048, 58)[:2] == (3, True)      # 24 blocks: 48 of one head, in 3 runs
    assert ops.attention_prefill_tc_plan(4, 12, 2, 128, 512, 10)[:2] == (1, True)       # too few keys to split
    assert ops.attention_prefill_tc_plan(1, 2, 1, 64, 1024)[:2] == (2, False)


@pytest.mark.parametrize("k_gain", [None, 48.0])
def test_attention_prefill_tc_moves_the_reference_of_the_exponents(k_gain):
    """The tcgen05 kernel rescales a row's output only when the row's maximum has grown by more than 8 (in
    powers of two).  Rows whose one large score lies in their first, a middle or their last tile of keys,
    next to rows without one in the same warp; and keys that grow with their position, so that the maximum
    creeps up from tile to tile, sometimes past the threshold and sometimes not."""
    import torch
    from machserve_b200 import ops
    lens, hq, hkv, hd, page = [900, 300], 4, 2, 64, 64
    case = PagedCase(lens, hq, hkv, hd, page, None, seed=5, k_gain=k_gain)
    rows, tile0, tilen = [], [], []
    for s, (a, b) in enumerate([(100, 900), (0, 300)]):
        for t0 in range(a, b, 128):
            tile0.append(len(rows)); tilen.append(min(128, b - t0))
            rows += [(s, p) for p in range(t0, min(t0 + 128, b))]
    rng = np.random.default_rng(11)
    far = []
    if k_gain is None:
        for r in rng.choice(len(rows), size=120, replace=False):
            pos = rows[r][1]
            far.append((int(r), int(rng.integers(hq)), int(rng.integers(0, pos + 1))))
        far += [(len(rows) - 1, 0, rows[-1][1]), (len(rows) - 2, 1, 0), (700, 2, rows[700][1] - 127), (700, 3, rows[700][1] - 128)]
    q, want, pos, slot = case.queries(rows, scale_one=far)
    out = torch.full((len(rows), hq * hd), 7.0, dtype=torch.bfloat16, device=dev())
    ops.attention_prefill_tc(T(q, torch.bfloat16), case.k_pages, case.v_pages, out, T(np.array(tile0, dtype=np.int32)),
                             T(np.array(tilen, dtype=np.int32)), len(tile0), pos, slot, case.table, hq, hkv, hd, None, hd ** -0.5)
    assert ops.gemm_tc_status() == 0
    err = np.abs(N(out) - want).max(axis=1)
    assert err.max() <= 2.0 ** -7 * max(1.0, np.abs(want).max()), f"worst row {int(err.argmax())} of {len(rows)}: {rows[int(err.argmax())]}"


def test_attention_decode_refuses_what_it_does_not_cover():
    import torch
    from machserve_b200 import ops
    assert not ops.attention_decode_supports(24, 2) and not ops.attention_decode_supports(256, 1)
    assert not ops.attention_decode_supports(64, 17)
    case = PagedCase([10], 2, 1, 144, 8)
    q, _, pos, slot = case.queries([(0, 9)])
    out = torch.empty((1, 2 * 144), dtype=torch.bfloat16, device=dev())
    with pytest.raises(ops.KernelError, match="head_dim 144"):
        ops.attention_decode(T(q, torch.bfloat16), case.k_pages, case.v_pages, out, None, pos, slot, case.table, 2, 1, 144, None, 1.0, 1)


@pytest.mark.parametrize("hq,hkv,hd,rot,inter,page", [(4, 2, 16, 16, False, 16), (3, 1, 32, 32, False, 8), (5, 5, 48, 24, True, 4), (14, 2, 64, 64, False, 64), (2, 2, 80, 32, False, 8)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rope_kv_store(hq, hkv, hd, rot, inter, page, dtype):
    """Bias, rotation (both pairings, partial rotary) and the write into shuffled pages."""
    import torch
    from machserve_b200 import ops
    from machserve_b200.config import part
    from machserve_b200.parts import Runtime, Workspace
    from machserve_b200.parts.rope import RotaryEncoding
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    rng = np.random.default_rng(7)
    theta, tokens, max_pos = 50000.0, 23, 200
    pe = RotaryEncoding(part("rope", head_dim=hd, rotary_dim=rot, theta=theta, pairing="interleaved" if inter else "half"))
    table = pe.rotary_table(Runtime(tdt, dev(), Workspace(dev()), max_pos))
    width = (hq + 2 * hkv) * hd
    qkv = T(rng.normal(size=(tokens, width + 5)), tdt)[:, :width]  # a row stride wider than q|k|v
    bias = rng.normal(size=width).astype(np.float32)
    positions = rng.permutation(max_pos)[:tokens].astype(np.int32)
    slots = rng.integers(0, 3, size=tokens).astype(np.int32)
    slots[3] = -1  # a padding row: nothing is written for it
    max_pages = -(-max_pos // page)
    num_pages = 3 * max_pages
    bt = rng.permutation(num_pages).reshape(3, max_pages).astype(np.int32)
    kp = torch.zeros((num_pages, hkv, page, hd), dtype=tdt, device=dev()); vp = torch.zeros_like(kp)
    q_out = torch.zeros((tokens, hq * hd), dtype=tdt, device=dev())
    ops.rope_kv_store(qkv, T(bias), T(positions), T(slots), T(bt), table, rot, inter, q_out, kp, vp, hq, hkv, hd)
    x = N(qkv) + bias
    def rotate(v, pos):  # v [heads, hd]
        out = v.copy()
        j = np.arange(rot // 2)
        ang = pos / theta ** (2.0 * j / rot)
        c, s = np.cos(ang), np.sin(ang)
        a_idx, b_idx = (2 * j, 2 * j + 1) if inter else (j, j + rot // 2)
        out[:, a_idx] = v[:, a_idx] * c - v[:, b_idx] * s
        out[:, b_idx] = v[:, a_idx] * s + v[:, b_idx] * c
        return out
    tol = 1e-5 if dtype == "float32" else 2.0 ** -7
    kpn, vpn = N(kp), N(vp)
    written = np.zeros((num_pages, page), dtype=bool)
    for t in range(tokens):
        if slots[t] < 0:
            assert not N(q_out[t]).any()
            continue
        p = int(positions[t])
        q = rotate(x[t, : hq * hd].reshape(hq, hd), p)
        k = rotate(x[t, hq * hd : (hq + hkv) * hd].reshape(hkv, hd), p)
        v = x[t, (hq + hkv) * hd :].reshape(hkv, hd)
        pg = bt[slots[t], p // page]
        written[pg, p % page] = True
        assert np.abs(N(q_out[t]).reshape(hq, hd) - q).max() <= tol * max(1, np.abs(q).max())
        assert np.abs(kpn[pg, :, p % page] - k).max() <= tol * max(1, np.abs(k).max())
        assert np.abs(vpn[pg, :, p % page] - v).max() <= tol * max(1, np.abs(v).max())
    untouched = ~written  # [pages, slots]; the arrays are [pages, kv heads, slots, head_dim]
    assert not kpn.transpose(0, 2, 1, 3)[untouched].any() and not vpn.transpose(0, 2, 1, 3)[untouched].any()
