"""The engine against the plain implementation, in every way of cutting the work.

Each test replays token ids through `ModelRunner.step` (the function generation and
bin/trace_run use) and compares the logits at every position with the plain
whole-sequence implementation, in float32 and in bfloat16.
"""
import numpy as np
import pytest

from tests.helpers import (
    BF16_TOL, F32_TOL, TINY, assert_close, collect_rows, make_model_dir, plain_logits, random_tokens,
    run_trace_cli, trace_portions, trace_tail_decode, trace_whole,
)

pytestmark = pytest.mark.gpu

CASES = [(n, d) for n in TINY for d in ("float32", "bfloat16")]


def _tol(dtype):
    return F32_TOL if dtype == "float32" else BF16_TOL


def _replay(model_dir, dtype, steps, max_tokens, page):
    from machserve_b200.engine.replay import make_replay_runner, replay

    runner = make_replay_runner(model_dir, dtype, max_tokens, page)
    out = replay(runner, steps)
    runner.cache.check()
    assert not runner.cache.requests, "requests still hold cache after the trace ended"
    assert all(g.pool.num_held == 0 for g in runner.cache.groups)
    return out


def _reference(model_dir, dtype, requests):
    return {rid: plain_logits(model_dir, toks, bf16_weights=(dtype == "bfloat16")) for rid, toks in requests.items()}


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole(model_root, name, dtype):
    """Each request alone and whole."""
    d = make_model_dir(model_root, name)
    vocab = TINY[name]["config"]["vocab_size"]
    requests = {f"r{n}": random_tokens(vocab, n, 100 + n) for n in (1, 5, 17, 33, 70)}
    steps = trace_whole(requests)
    got = collect_rows(steps, _replay(d, dtype, steps, 128, TINY[name]["page"]))
    for rid, want in _reference(d, dtype, requests).items():
        assert_close(got[rid], want, _tol(dtype), f"tiny-{name} {dtype} whole {rid}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_tail_decoded(model_root, name, dtype):
    """Most of it in one step and the last 32 tokens one by one."""
    d = make_model_dir(model_root, name)
    toks = random_tokens(TINY[name]["config"]["vocab_size"], 75, 7)
    steps = trace_tail_decode("a", toks, 32)
    got = collect_rows(steps, _replay(d, dtype, steps, 128, TINY[name]["page"]))
    assert_close(got["a"], _reference(d, dtype, {"a": toks})["a"], _tol(dtype), f"tiny-{name} {dtype} tail")


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions(model_root, name, dtype):
    """In portions of changing size, down to two tokens."""
    d = make_model_dir(model_root, name)
    toks = random_tokens(TINY[name]["config"]["vocab_size"], 90, 11)
    steps = trace_portions("a", toks, [7, 2, 13, 3, 2, 16, 5, 9])
    got = collect_rows(steps, _replay(d, dtype, steps, 128, TINY[name]["page"]))
    assert_close(got["a"], _reference(d, dtype, {"a": toks})["a"], _tol(dtype), f"tiny-{name} {dtype} portions")


def mixed_trace(vocab, seed=3):
    """Up to four live requests; portions of some beside decoded tokens of others; with a pool of
    256 tokens the later requests can only run on pages that earlier ones gave back."""
    rng = np.random.default_rng(seed)
    lens = {"a": 60, "b": 41, "c": 23, "d": 50, "e": 37, "f": 64, "g": 30}
    requests = {k: [int(x) for x in rng.integers(0, vocab, size=n)] for k, n in lens.items()}
    pending = list(requests)
    live, at, steps = [], {}, []
    portion = {"a": 9, "b": 7, "c": 5, "d": 11, "e": 2, "f": 13, "g": 6}
    step = 0
    while pending or live:
        while pending and len(live) < 4 and sum((lens[r] + 63) // 64 * 64 for r in live + [pending[0]]) <= 256:
            r = pending.pop(0)
            live.append(r)
            at[r] = 0
        entries, ended = [], []
        for r in list(live):
            if rng.random() < 0.2 and len(live) > 1:
                continue  # left out of this step, goes on later
            remaining = lens[r] - at[r]
            # the first part of a request comes in portions, its last 8 tokens one by one
            n = 1 if remaining <= 8 else min(portion[r], remaining - 8)
            entries.append({"id": r, "tokens": requests[r][at[r] : at[r] + n], "want": list(range(n))})
            at[r] += n
            if at[r] == lens[r]:
                ended.append(r)
                live.remove(r)
        if entries:
            steps.append({"step": step, "entries": entries, "end": ended})
            step += 1
    return requests, steps


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_with_page_reuse(model_root, name, dtype):
    d = make_model_dir(model_root, name)
    requests, steps = mixed_trace(TINY[name]["config"]["vocab_size"])
    assert max(len(s["entries"]) for s in steps) >= 3
    got = collect_rows(steps, _replay(d, dtype, steps, 256, TINY[name]["page"]))
    for rid, want in _reference(d, dtype, requests).items():
        assert_close(got[rid], want, _tol(dtype), f"tiny-{name} {dtype} mixed {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_root, tmp_path, dtype):
    """bin/trace_run itself, as a user drives it: a mixed trace on tiny-B."""
    d = make_model_dir(model_root, "B")
    requests, steps = mixed_trace(TINY["B"]["config"]["vocab_size"], seed=5)
    results = run_trace_cli(d, dtype, steps, 256, tmp_path / "out", page_size=TINY["B"]["page"])
    got = collect_rows(steps, results)
    for rid, want in _reference(d, dtype, requests).items():
        assert_close(got[rid], want, _tol(dtype), f"trace_run {dtype} {rid}")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("C", "float32"), ("C", "bfloat16")])
def test_long_decoding(model_root, name, dtype):
    """A short prompt, then 300 tokens one by one: across many pages and, in tiny-C, far past the window."""
    d = make_model_dir(model_root, name)
    toks = random_tokens(TINY[name]["config"]["vocab_size"], 310, 21)
    steps = trace_tail_decode("a", toks, 300)
    got = collect_rows(steps, _replay(d, dtype, steps, 320, TINY[name]["page"]))
    assert_close(got["a"], _reference(d, dtype, {"a": toks})["a"], _tol(dtype), f"tiny-{name} {dtype} long decoding")


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens(model_root, name, dtype):
    """The first tokens of a sequence: a request that starts with a single token and is decoded from there,
    and requests of two and three tokens, alone and together in one step."""
    d = make_model_dir(model_root, name)
    vocab = TINY[name]["config"]["vocab_size"]
    a, b, c = random_tokens(vocab, 6, 31), random_tokens(vocab, 2, 32), random_tokens(vocab, 3, 33)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:1], "want": [0]}], "end": []}]
    steps += [{"step": i, "entries": [{"id": "a", "tokens": [a[i]], "want": [0]}], "end": []} for i in range(1, 6)]
    steps.append({"step": 6, "entries": [{"id": "b", "tokens": b, "want": [0, 1]}, {"id": "c", "tokens": c, "want": [0, 1, 2]}],
                  "end": ["a", "b", "c"]})
    got = collect_rows(steps, _replay(d, dtype, steps, 192, TINY[name]["page"]))
    for rid, want in _reference(d, dtype, {"a": a, "b": b, "c": c}).items():
        assert_close(got[rid], want, _tol(dtype), f"tiny-{name} {dtype} first tokens {rid}")


def test_decoding_one_request_with_a_long_context(model_root):
    """One request with 4,400 tokens of context, decoded token by token in bfloat16 at head size 64: with so few rows and
    so many keys the attention spreads a row's keys over several clusters, whose sums meet in scratch memory (the test
    checks that this form was chosen).  The logits of the 8 decoded positions are compared with the plain implementation."""
    import torch
    from machserve_b200 import ModelRunner
    from machserve_b200.engine.runner import StepEntry
    from machserve_b200.parts.attention import Attention

    d = make_model_dir(model_root, "D", max_position_embeddings=8192)
    vocab, page = TINY["D"]["config"]["vocab_size"], TINY["D"]["page"]
    toks = random_tokens(vocab, 4408, 77)
    runner = ModelRunner.from_model_dir(d, dtype="bfloat16", page_size=page, num_pages=4608 // page, max_requests=2,
                                        max_step_tokens=1024, max_seq_len=4608)
    at = 0
    while at < 4400:
        n = min(1024, 4400 - at)
        runner.step([StepEntry("a", toks[at : at + n], [])])
        at += n
    rows = []
    for i in range(8):
        rows.append(runner.step([StepEntry("a", [toks[4400 + i]], [0])]).detach().float().cpu().numpy()[0].copy())
    attention = next(p for p in runner.model.parts() if isinstance(p, Attention))
    assert any(choice[4] > 1 for choice in attention._launch_cache.values()), attention._launch_cache
    want = plain_logits(d, toks, bf16_weights=True)[4400:4408]
    assert_close(np.stack(rows), want, BF16_TOL, "tiny-D bfloat16, decoding after 4,400 tokens")
