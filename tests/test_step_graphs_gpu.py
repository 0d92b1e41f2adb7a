"""Steps of any shape that share a captured graph.

A step that is no plain decoding is padded to a class of sizes (rows, sequences, wanted rows, the attention's
tile lists and context classes), and steps of one class are replayed from one CUDA graph.  These tests run steps
whose real sizes differ inside one class (portions of prompts of changing length beside a changing number of
decoded tokens), make sure that they were in fact replayed from one graph, and compare every logit with the
plain whole-sequence implementation; in float32 also bit by bit with the same steps run without graphs.
"""
import numpy as np
import pytest

from tests.helpers import BF16_TOL, F32_TOL, TINY, assert_close, make_model_dir, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


def _runner(model_dir, dtype, page, use_graphs=True, max_requests=8):
    from machserve_b200 import ModelRunner

    return ModelRunner.from_model_dir(model_dir, dtype=dtype, page_size=page, num_pages=2048 // page, max_requests=max_requests,
                                      max_step_tokens=256, max_seq_len=512, use_graphs=use_graphs)


def _mixed_steps(vocab, portions, decoders, seed, always=False):
    """One long request fed in portions of the given sizes; beside each portion, the next token of some of the
    `decoders` (requests that have had a prompt of a few tokens in a step of their own before)."""
    rng = np.random.default_rng(seed)
    long = random_tokens(vocab, sum(portions), seed)
    dec = {f"d{i}": random_tokens(vocab, 6 + 3 * i + len(portions), seed + 1 + i) for i in range(decoders)}
    steps = [[(rid, toks[: 6 + 3 * i], list(range(6 + 3 * i)))] for i, (rid, toks) in enumerate(dec.items())]
    fed = {rid: 6 + 3 * i for i, rid in enumerate(dec)}
    at = 0
    for k, n in enumerate(portions):
        entries = [("long", long[at : at + n], list(range(n)))]
        at += n
        for i, rid in enumerate(dec):
            if always or rng.integers(0, 3) or k == 0:  # a changing number of decoding rows
                entries.insert(int(rng.integers(0, len(entries) + 1)), (rid, [dec[rid][fed[rid]]], [0]))
                fed[rid] += 1
        steps.append(entries)
    tokens = {"long": long, **{rid: toks[: fed[rid]] for rid, toks in dec.items()}}
    return steps, tokens


def _run(runner, steps):
    from machserve_b200.engine.runner import StepEntry

    rows = {}
    for entries in steps:
        logits = runner.step([StepEntry(*e) for e in entries]).detach().float().cpu().numpy()
        at = 0
        for rid, toks, want in entries:
            rows.setdefault(rid, []).append(logits[at : at + len(want)].copy())
            at += len(want)
        assert at == logits.shape[0]
    return {rid: np.concatenate(parts) for rid, parts in rows.items()}


CASES = [("A", "float32"), ("C", "float32"), ("D", "float32"), ("A", "bfloat16"), ("B", "bfloat16"), ("D", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_steps_of_like_size_share_one_graph(model_root, name, dtype):
    d = make_model_dir(model_root, name)
    vocab, page = TINY[name]["config"]["vocab_size"], TINY[name]["page"]
    # portions of 20 to 29 rows beside up to 3 decoded tokens: 21 to 32 rows, all padded to 32; one class of contexts
    portions = [23, 29, 20, 27, 22, 28, 21, 26, 25, 24]
    steps, tokens = _mixed_steps(vocab, portions, 3, 11)
    runner = _runner(d, dtype, page)
    assert runner.use_graphs
    got = _run(runner, steps)
    keys = list(runner._shape_graphs)
    replayed = [k for k in keys if k[0] == 32]
    assert len(replayed) == 1, f"the mixed steps were expected to share one graph, got the shapes {keys}"
    seen = runner._shape_seen[replayed[0]]
    assert seen == runner.CAPTURE_AFTER + 1, "later steps of the class must not be counted again: they are replayed"
    tol = F32_TOL if dtype == "float32" else BF16_TOL
    for rid, toks in tokens.items():
        want = plain_logits(d, toks, bf16_weights=(dtype == "bfloat16"))
        assert_close(got[rid], want[: len(got[rid])] if rid == "long" else want, tol, f"tiny-{name} {dtype} shared graph {rid}")
    if dtype == "float32":
        plainly = _run(_runner(d, dtype, page, use_graphs=False), steps)
        for rid in tokens:
            assert np.array_equal(got[rid], plainly[rid]), f"{rid}: a padded, replayed step differs from the step run as it is"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_longer_portions_in_classes_of_64_rows(model_root, dtype):
    """Portions of 70 to 120 rows beside decoded tokens at head size 64 (the tcgen05 kernel for portions in bfloat16): rows
    padded to 128, tile lists padded with tiles of no rows, contexts that cross a class."""
    d = make_model_dir(model_root, "D")
    vocab, page = TINY["D"]["config"]["vocab_size"], TINY["D"]["page"]
    portions = [100, 71, 120, 90, 111, 83, 95, 77, 118]  # 865 tokens: the context classes 512 and 1,024 both occur
    steps, tokens = _mixed_steps(vocab, portions, 2, 5, always=True)
    from machserve_b200 import ModelRunner

    runner = ModelRunner.from_model_dir(d, dtype=dtype, page_size=page, num_pages=2048 // page, max_requests=4,
                                        max_step_tokens=128, max_seq_len=1024)
    got = _run(runner, steps)
    classes = sorted(k[4][0][2] for k in runner._shape_graphs if k[0] == 128)
    # nine steps in two classes of contexts (the portion ends within 512 tokens, or within 1,024)
    assert classes == [(1, 1, 4), (1, 2, 8)], f"the steps of 128 padded rows were to share two graphs: {list(runner._shape_graphs)}"
    tol = F32_TOL if dtype == "float32" else BF16_TOL
    for rid, toks in tokens.items():
        want = plain_logits(d, toks, bf16_weights=(dtype == "bfloat16"))
        assert_close(got[rid], want, tol, f"tiny-D {dtype} portions in classes {rid}")
