"""Generation through the Python entry point, compared with the plain implementation."""
import numpy as np
import pytest

from tests.helpers import BF16_TOL, TINY, make_model_dir, random_tokens
from tests.plain import forward_logits, greedy_generate, read_model_dir, sample_token, splitmix64_next

pytestmark = pytest.mark.gpu


def _engine(model_dir, dtype="f32", **kw):
    from machserve_b200 import Engine

    kw.setdefault("capacity", 4)
    kw.setdefault("prefill_rows", 16)
    kw.setdefault("tpp", 8)
    kw.setdefault("max_seq", 128)
    return Engine(model_dir, dtype, **kw)


@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_f32(model_root, name):
    d = make_model_dir(model_root, name)
    cfg, w = read_model_dir(d)
    prompts = [random_tokens(cfg["vocab_size"], n, 50 + n) for n in (5, 17, 33, 1, 24, 40)]
    eng = _engine(d)
    got = eng.generate(prompts, max_new_tokens=8)
    for p, g in zip(prompts, got):
        assert g == greedy_generate(lambda t: forward_logits(w, cfg, t), p, 8)
    eng.runner.cache.check()
    assert not eng.runner.cache.requests


@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_bf16(model_root, name):
    """bfloat16 may break a near tie the other way: every chosen token must be a maximum of the
    plain logits within the bfloat16 tolerance, along the engine's own sequence."""
    d = make_model_dir(model_root, name)
    cfg, w = read_model_dir(d, round_to_bf16=True)
    prompts = [random_tokens(cfg["vocab_size"], n, 60 + n) for n in (9, 30, 2)]
    got = _engine(d, "bf16").generate(prompts, max_new_tokens=8)
    for p, g in zip(prompts, got):
        assert len(g) == 8
        logits = forward_logits(w, cfg, p + g)
        for i, tok in enumerate(g):
            row = logits[len(p) - 1 + i]
            assert row[tok] >= row.max() - 2 * BF16_TOL * max(1.0, np.abs(row).max()), f"token {i} of {g}"


def test_temperature_sampling_follows_the_seeded_draws(model_root):
    """tiny-B at temperature 0.8: with the same SplitMix64 draws the plain sampler picks the same tokens,
    however the prompts are cut (portions of 7 mixed with decoding)."""
    d = make_model_dir(model_root, "B")
    cfg, w = read_model_dir(d)
    prompts = [random_tokens(cfg["vocab_size"], n, 70 + n) for n in (1, 9, 24, 40)]
    from machserve_b200 import SamplingParams

    for rows in (7, 64):
        eng = _engine(d, prefill_rows=rows)
        ids = [eng.add(p, 6, params=SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=1000 + i))
               for i, p in enumerate(prompts)]
        while not eng.all_done():
            eng.step()
        for i, (sid, p) in enumerate(zip(ids, prompts)):
            state, seq, want = 1000 + i, list(p), []
            for _ in range(6):
                u, state = splitmix64_next(state)
                tok, _ = sample_token(forward_logits(w, cfg, seq)[-1], 0.8, 50, 0.95, u)
                want.append(tok); seq.append(tok)
            assert eng.generated(sid) == want, f"prefill_rows={rows} request {i}"
            assert eng.finish_reason(sid) == "length"


def test_eos_stop_sequences_and_penalties(model_root):
    d = make_model_dir(model_root, "A")
    cfg, w = read_model_dir(d)
    p = random_tokens(cfg["vocab_size"], 12, 5)
    base = greedy_generate(lambda t: forward_logits(w, cfg, t), p, 10)
    from machserve_b200 import SamplingParams

    eng = _engine(d)
    a = eng.add(p, 10, eos=base[3])
    b = eng.add(p, 10, stop_seqs=[base[4:6]])
    c = eng.add(p, 10, logit_bias={7: 100.0})
    e = eng.add(p, 10, params=SamplingParams(presence_penalty=0.5, frequency_penalty=0.7))
    while not eng.all_done():
        eng.step()
    first = base.index(base[3])
    assert eng.generated(a) == base[: first + 1] and eng.finish_reason(a) == "stop"
    assert eng.generated(b)[-2:] == base[4:6] and eng.finish_reason(b) == "stop" and len(eng.generated(b)) <= 6
    assert eng.generated(c) == [7] * 10
    seq, counts, want = list(p), {}, []
    for _ in range(10):
        tok, _ = sample_token(forward_logits(w, cfg, seq)[-1], counts=counts, presence_penalty=0.5, frequency_penalty=0.7)
        want.append(tok); seq.append(tok); counts[tok] = counts.get(tok, 0) + 1
    assert eng.generated(e) == want


def test_preemption_on_the_gpu_changes_nothing(model_root):
    """So few pages that decoding requests push the youngest out; recomputed, it ends with the same tokens."""
    d = make_model_dir(model_root, "C")
    cfg, w = read_model_dir(d)
    prompts = [random_tokens(cfg["vocab_size"], n, 80 + n) for n in (20, 18, 22)]
    roomy = _engine(d, num_pages=64).generate(prompts, max_new_tokens=24)
    tight = _engine(d, num_pages=12)  # 96 tokens of cache for three requests that grow to ~44 each
    got = tight.generate(prompts, max_new_tokens=24)
    assert tight.counters["preemptions"] > 0
    assert got == roomy
    for p, g in zip(prompts, got):
        assert g == greedy_generate(lambda t: forward_logits(w, cfg, t), p, 24)


def test_command_line_generate(model_root):
    import json, subprocess, sys
    from tests.helpers import REPO

    d = make_model_dir(model_root, "A")
    cfg, w = read_model_dir(d)
    p = random_tokens(cfg["vocab_size"], 9, 3)
    r = subprocess.run([sys.executable, str(REPO / "bin" / "mach"), "generate", str(d), "--prompt-ids",
                        ",".join(map(str, p)), "--max-new", "5", "--dtype", "f32", "--tpp", "16", "--max-seq", "64",
                        "--capacity", "2"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["tokens"] == greedy_generate(lambda t: forward_logits(w, cfg, t), p, 5)


def test_running_ahead_of_the_host_changes_no_token(model_root):
    """With `run_ahead` a step is launched before the tokens of the one before it are read, and the device
    takes them from the sampler's output.  Same tokens, finish reasons and draws as step by step: greedy and
    seeded temperature sampling, an EOS in the middle (one row in flight is dropped), a length limit, and
    a pool so small that requests wait for one another.  (The preemption test above runs ahead as well.)"""
    from machserve_b200 import SamplingParams

    d = make_model_dir(model_root, "B")
    cfg, w = read_model_dir(d)
    prompts = [random_tokens(cfg["vocab_size"], n, 90 + n) for n in (3, 19, 11, 26)]
    base = greedy_generate(lambda t: forward_logits(w, cfg, t), prompts[1], 12)

    def run(run_ahead, num_pages):
        eng = _engine(d, run_ahead=run_ahead, num_pages=num_pages, prefill_rows=7)
        ids = [
            eng.add(prompts[0], 14, params=SamplingParams(temperature=0.9, top_k=40, top_p=0.9, seed=77)),
            eng.add(prompts[1], 12, eos=base[5]),
            eng.add(prompts[2], 1),
            eng.add(prompts[3], 20),
        ]
        steps = 0
        while not eng.all_done():
            eng.step()
            steps += 1
            assert steps < 2000
        eng.runner.cache.check()
        assert not eng.runner.cache.requests
        return [(eng.generated(i), eng.finish_reason(i)) for i in ids], eng.counters["preemptions"]

    want, _ = run(False, 64)
    assert want[1] == (base[: base.index(base[5]) + 1], "stop") and want[2][1] == "length" and len(want[3][0]) == 20
    got, _ = run(True, 64)
    assert got == want
    tight, _ = run(True, 8)  # 64 tokens of cache for requests that grow to 17, 25, 12 and 46: they take turns
    assert tight == want


def test_top_logprobs_through_the_entry_point(model_root):
    """Beside every generated token the three most probable ones of the plain logits, the generated one first
    when decoding is greedy; requests that did not ask get nothing."""
    from machserve_b200 import SamplingParams

    d = make_model_dir(model_root, "A")
    cfg, w = read_model_dir(d)
    p = random_tokens(cfg["vocab_size"], 9, 123)
    eng = _engine(d)
    a = eng.add(p, 5, params=SamplingParams(top_logprobs=3))
    b = eng.add(p, 5)
    while not eng.all_done():
        eng.step()
    out, tops = eng.generated(a), eng.generated_top_logprobs(a)
    assert eng.generated(b) == out and eng.generated_top_logprobs(b) == []
    assert len(tops) == 5 and all(len(t) == 3 for t in tops)
    logits = forward_logits(w, cfg, p + out)
    from tests.plain import top_logprobs
    for i, tok in enumerate(out):
        want = top_logprobs(logits[len(p) - 1 + i], 0.0, 3)
        assert tops[i][0][0] == tok and [t for t, _ in tops[i]] == [t for t, _ in want]
        assert np.allclose([lp for _, lp in tops[i]], [lp for _, lp in want], atol=1e-3)
        assert abs(eng.generated_logprobs(a)[i] - tops[i][0][1]) < 1e-4


@pytest.mark.parametrize("seed", [0, 1])
def test_random_load_running_ahead_equals_step_by_step(model_root, seed):
    """Thirty requests of random lengths, token limits, EOS tokens and sampling options arrive while others run,
    in a pool small enough to preempt; one is cancelled on the way.  Running one step ahead of the host and
    stepping in lockstep give the same tokens and finish reasons, and nothing is left in the cache."""
    import random

    from machserve_b200 import SamplingParams

    d = make_model_dir(model_root, "C")
    cfg, _ = read_model_dir(d)
    rnd = random.Random(seed)
    jobs = []
    for i in range(30):
        prompt = random_tokens(cfg["vocab_size"], rnd.randint(1, 40), 1000 * seed + i)
        params = SamplingParams() if rnd.random() < 0.5 else SamplingParams(temperature=rnd.choice([0.5, 1.0]), top_k=rnd.choice([0, 20]),
                                                                            top_p=rnd.choice([1.0, 0.9]), seed=100 + i)
        jobs.append((prompt, rnd.randint(1, 25), rnd.choice([None, rnd.randrange(cfg["vocab_size"])]), params, rnd.randint(0, 12)))
    # a random EOS token is rarely met: two greedy requests get one that their own continuation holds
    _, w = read_model_dir(d)
    given = 0
    for k, (prompt, n, eos, params, at) in enumerate(jobs):
        if params.temperature <= 0 and n >= 4 and k != 9 and given < 2:
            jobs[k] = (prompt, n, greedy_generate(lambda t: forward_logits(w, cfg, t), prompt, 3)[2], params, at)
            given += 1

    def run(run_ahead):
        eng = _engine(d, "f32", run_ahead=run_ahead, capacity=4, num_pages=14, prefill_rows=9)
        pending, ids, steps, cancelled = list(jobs), [], 0, None
        while pending or not eng.all_done():
            while pending and pending[0][4] <= steps:
                p, n, eos, params, _ = pending.pop(0)
                ids.append(eng.add(p, n, eos=eos, params=params))
            if len(ids) >= 10 and cancelled is None:
                cancelled = ids[9]
                eng.cancel(cancelled)
            eng.step()
            steps += 1
            assert steps < 5000
        eng.runner.cache.check()
        assert not eng.runner.cache.requests
        return [(eng.generated(i), eng.finish_reason(i)) for i in ids if i != cancelled], eng.counters["preemptions"]

    want, _ = run(False)
    got, preempted = run(True)
    assert got == want
    assert preempted > 0, "the pool was meant to be too small for the load: nothing was preempted"
    assert any(r == "stop" for _, r in want) and any(r == "length" for _, r in want)
    # the greedy requests against the plain implementation (float32 engine: the same tokens)
    kept = [j for k, j in enumerate(jobs) if k != 9]
    checked = 0
    for (prompt, n, eos, params, _), (tokens, reason) in zip(kept, want):
        if params.temperature > 0 or checked >= 6:
            continue
        plain = greedy_generate(lambda t: forward_logits(w, cfg, t), prompt, n)
        if eos is not None and eos in plain:
            plain = plain[: plain.index(eos) + 1]
        assert tokens == plain and reason == ("stop" if eos is not None and plain[-1] == eos else "length")
        checked += 1
    assert checked >= 3


def test_a_pool_that_cannot_fit_is_refused_with_the_numbers(model_root):
    """The memory plan is compared with the device's free memory before anything is allocated."""
    d = make_model_dir(model_root, "A")
    with pytest.raises(RuntimeError, match="does not fit.*GiB are free"):
        _engine(d, num_pages=1 << 30)
