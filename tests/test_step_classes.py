"""Steps of any shape share captured graphs by classes of size: the arithmetic of those classes, on the CPU.

`ModelRunner.padded_sizes` pads a step's rows, sequences and wanted rows; `Attention.plan` pads its lists with
entries that do nothing and rounds what its launches depend on.  A graph is captured per distinct combination, so
the steps that a scheduler makes of a serving load must come to few of them.
"""
import collections

import numpy as np

from machserve_b200.cache import CacheManager
from machserve_b200.config import config_from_json
from machserve_b200.engine.runner import ModelRunner
from machserve_b200.engine.scheduler import Scheduler
from machserve_b200.parts.attention import Attention
from machserve_b200.parts.base import PagedKV, StepShape
from machserve_b200.parts.model import DecoderModel
from machserve_b200.sampling.params import SamplingParams
from tests.helpers import TINY


def _attention(name="A"):
    model = DecoderModel(config_from_json(TINY[name]["config"]).model_spec())
    return next(p for p in model.parts() if isinstance(p, Attention))


def test_padded_sizes():
    f = ModelRunner.padded_sizes
    assert f(1, 1, 1) == (16, 16, 16)
    assert f(16, 3, 0) == (16, 16, 0)
    assert f(17, 16, 17) == (32, 16, 32)  # wanted rows never exceed the rows
    assert f(33, 17, 5) == (64, 64, 16)
    assert f(541, 30, 29) == (576, 64, 64) and f(513, 2, 1) == (576, 16, 16)
    assert f(576, 64, 64) == (576, 64, 64) and f(577, 65, 65) == (640, 256, 256)
    assert f(40, 40, 40) == (64, 64, 64)
    for rows in range(1, 700):
        r, s, w = f(rows, min(rows, 64), rows)
        assert r >= rows and w >= min(rows, r) and r - rows < 64 and w <= r


def test_attention_plan_in_classes():
    att = _attention()
    # a portion of 200 rows after 1,000 tokens, three decoding rows, and 53 rows of no sequence at the end (256 in all)
    step = StepShape(256, 16, [0, 1, 201, 202, *[203] * 12], [1, 200, 1, 1, *[0] * 12], [700, 1000, 90, 2047, *[0] * 12], bucketed=True)
    plan = att.plan(step)
    single, t0, tn, b0, bn = (plan.lists[k] for k in ("single_rows", "tile_row0", "tile_rows", "big_tile_row0", "big_tile_rows"))
    assert single[:3] == [0, 201, 202] and len(single) == 16 and set(single[3:]) == {-1}
    many = att.plan(StepShape(64, 64, list(range(20)) + [20] * 44, [1] * 20 + [0] * 44, [5] * 64, bucketed=True)).lists["single_rows"]
    assert many[:20] == list(range(20)) and len(many) == 64 and set(many[20:]) == {-1}
    assert t0[:4] == [1, 65, 129, 193] and tn[:4] == [64, 64, 64, 8] and len(t0) == 4
    assert b0 == [1, 129] and bn == [128, 72]
    # longest decoding context 2,048 -> 4 buckets of 512 -> class 4; the portion ends at 1,200 -> 3 buckets -> class 4;
    # the mean number of key tiles a tile of rows sees is replaced by the bound that this class gives, 16
    assert plan.shape == (4, 4, 16)
    exact = att.plan(StepShape(203, 4, [0, 1, 201, 202], [1, 200, 1, 1], [700, 1000, 90, 2047]))
    assert exact.lists["single_rows"] == [0, 201, 202] and exact.shape == (4, 3, 10)
    # five tiles of 64 rows become eight with three tiles of no rows, three of 128 become four
    plan = att.plan(StepShape(320, 16, [0, *[300] * 15], [300, *[0] * 15], [0] * 16, bucketed=True))
    assert plan.lists["tile_rows"] == [64, 64, 64, 64, 44, 0, 0, 0] and plan.lists["big_tile_rows"] == [128, 128, 44, 0]
    assert plan.lists["single_rows"] == []


def _load(seed, prefill_rows=512, n_req=64, new=256, lo=128, hi=2048, page=64):
    """The steps a scheduler makes of a serving load: [(start, count)] per step, with the engine one step ahead."""
    lengths = [int(x) for x in np.random.default_rng(seed).integers(lo, hi + 1, size=n_req)]
    max_seq = hi + new
    cache = CacheManager([PagedKV(2, 64, None)] * 2, page, n_req * (-(-max_seq // page)), n_req)
    sch = Scheduler(cache, n_req, prefill_rows, max_seq)
    for n in lengths:
        sch.add([1] * n, new, params=SamplingParams())
    steps, inflight = [], None
    while not sch.all_done() or inflight is not None:
        plan = sch.schedule() if not sch.all_done() else None
        if inflight is not None:
            k = sum(1 for e in inflight.entries if e.samples)
            sch.update(inflight, [1] * k, [0.0] * k)
        inflight = plan if plan is not None and plan.entries else None
        if inflight is not None:
            steps.append([(e.start, e.count, e.samples) for e in plan.entries])
    return steps


def _key(att, step):
    counts = [c for _, c, _ in step]
    if all(c == 1 for c in counts):
        return None  # plain decoding: graphs by (batch, context length) of their own
    rows, seqs, wanted = sum(counts), len(step), sum(1 for _, _, w in step if w)
    rows_p, seqs_p, wanted_p = ModelRunner.padded_sizes(rows, seqs, wanted)
    row0 = list(np.cumsum([0] + counts[:-1]))
    empty = seqs_p - seqs
    plan = att.plan(StepShape(rows_p, seqs_p, row0 + [rows] * empty, counts + [0] * empty, [s for s, _, _ in step] + [0] * empty, True))
    return rows_p, seqs_p, wanted_p, tuple(len(v) for v in plan.lists.values()), plan.shape


def test_a_serving_load_comes_to_few_classes():
    att = _attention("D")
    seen = collections.Counter()
    for seed in (11, 12, 13):  # three loads of other prompt lengths first, as a server that has been up for a while
        for step in _load(seed):
            k = _key(att, step)
            if k is not None:
                seen[k] += 1
    captured = {k for k, n in seen.items() if n >= 2}
    steps = [k for k in (_key(att, s) for s in _load(3)) if k is not None]
    hits = sum(1 for k in steps if k in captured)
    assert len(steps) > 100
    assert len(seen) <= ModelRunner.MAX_SHAPE_GRAPHS, f"{len(seen)} classes after three loads"
    assert hits >= 0.8 * len(steps), f"only {hits} of {len(steps)} prompt-bearing steps of a new load fall into a captured class"


def test_decode_attention_launch_rule():
    """The launch shape of the decode attention for the cases it was measured at: (blocks a cluster, tiles held at once,
    warps, keys a warp takes at a time, clusters a row).  Host arithmetic only; it asks the kernel library for two of
    its constants, so it is skipped where the library cannot be built."""
    import types

    import pytest

    from machserve_b200 import ops

    try:
        max_stages = {64: ops.attention_decode_cluster_max_stages(64), 128: ops.attention_decode_cluster_max_stages(128)}
    except Exception as e:  # no compiler here
        pytest.skip(f"the kernel library is not available: {e}")

    def rule(hd, units, tiles):
        att = Attention.__new__(Attention)
        att.rt, att.hd, att.max_stages, att._launch_cache = types.SimpleNamespace(sm_count=148), hd, max_stages[hd], {}
        return att._single_launch(units, tiles)

    # head size 64, two kv heads: batch 8 at 2,048 keys (the benchmark's step): eight blocks a cluster, each holds its run
    assert rule(64, 16, 40) == (8, 5, 8, 0, 1)
    # batch 64: four blocks a cluster (512 blocks, all resident), a ring of two tiles, a quarter of a tile per warp
    assert rule(64, 128, 40) == (4, 2, 4, 16, 1)
    # batch 1 at 32,768 keys: eight clusters a row; at 8,192 keys: four; at 2,048: one
    assert rule(64, 2, 520)[4] == 8 and rule(64, 2, 136)[4] == 4 and rule(64, 2, 40)[4] == 1
    # batch 8: several clusters only from 32,768 keys on (a second block per SM delays the kernels that follow)
    assert rule(64, 16, 264)[4] == 1 and rule(64, 16, 520)[4] == 2
    # never more clusters than 16, never fewer than four tiles a block
    for units in (1, 2, 4, 8, 16, 64):
        for tiles in (8, 40, 136, 520, 2056):
            splits, stages, warps, kpw, parts = rule(128, units, tiles)
            assert 1 <= parts <= 16 and 1 <= stages <= max_stages[128] and warps in (4, 8)
            assert parts == 1 or tiles // (8 * parts) >= 4


def test_few_row_products_stage_their_activations():
    """The few-row products bring their share of the activation rows into shared memory before they multiply; when the
    share does not fit they read it from global memory chunk by chunk after their wait, which costs a decoding step of 9
    to 16 rows at 0.5B sizes about a tenth of its time.  At those sizes every product of up to 16 rows stages them, at
    1.5B sizes every product of up to 8 rows (with more rows, and at larger sizes, the gate/up and down products' shares
    outgrow the 48 KB set aside).  Host arithmetic of the kernel library; skipped where the library cannot be built."""
    import pytest

    from machserve_b200 import ops

    try:
        ops.gemm_small_m_plan(8, 896, 896, sms=148)
    except Exception as e:  # no compiler here
        pytest.skip(f"the kernel library is not available: {e}")
    for name, (hidden, qkv, inter), most in (("0.5b", (896, 1152, 4864), (1, 8, 9, 16)), ("1.5b", (1536, 2048, 8960), (1, 8))):
        for rows in most:
            for what, plan in (("qkv", ops.gemm_small_m_plan(rows, qkv, hidden, sms=148)),
                               ("output", ops.gemm_small_m_plan(rows, hidden, hidden, residual=True, sms=148)),
                               ("gate/up", ops.gemm_small_m_plan(rows, inter, hidden, gated=True, sms=148)),
                               ("down", ops.gemm_small_m_plan(rows, hidden, inter, residual=True, sms=148))):
                assert plan["activation_stride"] > 0, f"{name} {what} at {rows} rows reads its activations from global memory: {plan}"
                assert plan["shared_bytes"] <= 96 * 1024 and plan["cluster"] in (1, 2, 4)
    # what does not fit is read after the wait (the kernel's other path), never staged in part
    assert ops.gemm_small_m_plan(16, 1536, 8960, residual=True, sms=148)["activation_stride"] == 0
