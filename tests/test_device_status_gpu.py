"""A bounded wait that runs out: the kernel gives up, leaves a code, returns, and the host finds it.

The tcgen05 kernels wait on mbarriers with a limit of polls.  Nothing in normal operation makes such a
wait run out, so these tests make one run out in the only form that cannot hang: one thread polls, through
the kernels' own wait helper, a barrier in its own shared memory that nothing arrives on, a thousand times;
no copy and no tensor memory is in flight when it gives up.
"""
import pytest

from tests.helpers import TINY, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kernel,code", [("gemm", 9), ("attention", 19)])
def test_wait_runs_out_and_leaves_its_code(kernel, code):
    import torch

    from machserve_b200 import ops

    assert ops.tc_status_codes() == (0, 0)
    ops.tc_wait_probe(kernel, 1000)
    torch.cuda.synchronize()  # the kernel returned: the context is usable
    assert ops.gemm_tc_status(reset=False) == code
    assert ops.gemm_tc_status() == code
    assert ops.tc_status_codes() == (0, 0), "the status must be clear after it was read with reset"
    x = torch.ones(4, device="cuda")
    assert float((x + 1).sum()) == 8.0


def test_both_codes_are_read_and_cleared_together():
    from machserve_b200 import ops

    ops.tc_wait_probe("gemm")
    ops.tc_wait_probe("attention")
    assert ops.tc_status_codes() == (9, 19)
    assert ops.tc_status_codes() == (0, 0)


def test_runner_and_engine_surface_it(model_root):
    from machserve_b200 import Engine, ops

    d = make_model_dir(model_root, "A")
    eng = Engine(d, "bf16", capacity=2, prefill_rows=8, tpp=8, max_seq=64)
    prompt = random_tokens(TINY["A"]["config"]["vocab_size"], 5, 1)
    assert len(eng.generate([prompt], max_new_tokens=3)[0]) == 3
    ops.tc_wait_probe("attention")
    with pytest.raises(RuntimeError, match="gave up a wait"):
        eng.runner.check_device_status()
    eng.runner.check_device_status()  # cleared by the check that raised
    ops.tc_wait_probe("gemm")
    with pytest.raises(RuntimeError, match="gave up a wait"):
        eng.generate([prompt], max_new_tokens=3)  # the engine checks when it runs empty
    assert ops.tc_status_codes() == (0, 0)


def test_timeline_build_and_reader(model_root):
    """The "timeline" build of the kernels and its reader: a decoding step of a tiny model leaves one record per
    launch of a kernel that carries hooks, five per layer, in order, with the times in order."""
    import json
    import subprocess
    import sys

    from tests.helpers import REPO

    d = make_model_dir(model_root, "D")  # 2 layers
    r = subprocess.run([sys.executable, "-m", "machserve_b200.timeline", "--model", str(d), "--batch", "3", "--context", "40", "--json"],
                       capture_output=True, text=True, timeout=600, cwd=str(REPO))
    assert r.returncode == 0, r.stderr[-2000:]
    recs = [json.loads(line) for line in r.stdout.splitlines() if line.startswith("{")]
    kinds = [x["id"] for x in recs]
    # first layer: plain QKV product after a norm kernel; then per layer attention, output product, gate/up, down product
    assert kinds[:5] == [100, 200, 130, 121, 130] and kinds[5:10] == [101, 200, 130, 121, 130], kinds
    for x in recs:
        assert x["start"] <= x["wait_returned"] <= x["first_end"] <= x["last_end"]
    for a, b in zip(recs, recs[1:]):
        assert b["wait_returned"] >= a["last_end"] - 0.01  # a wait returns when the kernel before has ended
