"""The engine at the layer widths that are benchmarked, against the plain implementation.

Two layers of the Qwen2.5 0.5B, 1.5B and 7B widths (head sizes 64 and 128, 14/2, 12/2 and 28/4
heads, intermediate sizes 4,864, 8,960 and 18,944), pages of 64 tokens as the engine's default and
the benchmark use, in float32 and in bfloat16.  Each case builds ONE runner whose pool is so small
that every cutting runs on pages an earlier one gave back, and replays through `ModelRunner.step`:

* a request of 1,100 tokens (700 at the 7B widths) whole, with its last 32 tokens one by one, and
  in portions of changing size down to two tokens;
* a prompt of 500 tokens, then one token at a time across the context lengths 512 and 1,024, where
  the decoding step changes its captured graph, its split count and its tile loader;
* a mixed trace shaped like the 7B benchmark step in small: two portions of 130 rows with earlier
  tokens in the cache beside six decoding rows.

Every logit row is compared with the plain float64 implementation on the same weights.  In float32
the logits of different cuttings of one request are also compared with each other bit by bit.
The query and key projections are drawn wider than the other matrices so that the attention is
peaked (scores of a few units): a key that a kernel dropped or misplaced then moves the logits
far more than rounding does.
"""
import numpy as np
import pytest

from tests.helpers import assert_close, collect_rows, trace_portions, trace_tail_decode, trace_whole

pytestmark = pytest.mark.gpu

PAGE = 64
# float32 engine against float64: rounding of float32 sums over up to 18,944 terms
F32_TOL = 3e-5
# bfloat16 engine (activations, cache and products rounded to 8 bits in both layers) against float64 on the
# same bfloat16 weights, relative to the largest logit.  Worst measured on a B200 over all cuttings: 0.034 at the
# 0.5B widths, 0.034 at the 1.5B widths, 0.023 at the 7B widths (float32: 7e-6, 8e-6, 1e-5).  The attention is
# peaked on purpose (scores up to +-12), so a score's rounding of 2^-9 moves a probability by up to 3 %.
BF16_TOL = 4e-2

SIZES = {
    "0.5b": dict(hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64, intermediate_size=4864,
                 vocab_size=2264, tie_word_embeddings=True, long=1100),
    "1.5b": dict(hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, head_dim=128, intermediate_size=8960,
                 vocab_size=1544, tie_word_embeddings=True, long=1100),
    "7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
               vocab_size=1032, tie_word_embeddings=False, long=700),
}
CASES = [(s, d) for s in SIZES for d in ("float32", "bfloat16")]


def _config(size):
    raw = {k: v for k, v in SIZES[size].items() if k != "long"}
    raw.update({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 2,
                "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 4096,
                "use_sliding_window": False, "hidden_act": "silu"})
    return raw


class World:
    """One runner of one size and dtype, the plain implementation on the same weights, and what was computed."""

    def __init__(self, size, dtype):
        import torch

        from machserve_b200 import ModelRunner
        from machserve_b200.config import config_from_json
        from machserve_b200.parts import DecoderModel

        self.size, self.dtype, self.raw = size, dtype, _config(size)
        cfg = config_from_json(self.raw)
        gen = torch.Generator().manual_seed(sum(map(ord, size)))
        hidden = self.raw["hidden_size"]
        tensors = {}
        for d in DecoderModel(cfg.model_spec()).tensors():
            if not d.random:
                continue
            t = torch.randn(d.shape, generator=gen, dtype=torch.float32)
            if d.init == "matrix":
                wide = ".q_proj." in d.name or ".k_proj." in d.name
                t *= 1.8 / hidden ** 0.5 if wide else 0.02
            elif d.init == "bias":
                t *= 0.1
            elif d.init == "scale":
                t = 1.0 + 0.05 * t
            tensors[d.name] = t
        if dtype == "bfloat16":
            tensors = {n: t.to(torch.bfloat16) if t.dim() == 2 else t for n, t in tensors.items()}
        self.weights = {n: t.to(torch.float32).numpy().astype(np.float64) for n, t in tensors.items()}
        self.vocab = self.raw["vocab_size"]
        # the pool holds the longest request and little more: every later cutting runs on pages given back
        self.pool_tokens = 30 * PAGE
        self.runner = ModelRunner(cfg, tensors, dtype=dtype, page_size=PAGE, num_pages=self.pool_tokens // PAGE,
                                  max_requests=8, max_step_tokens=1200, max_seq_len=1152)
        self._plain = {}
        self.worst = 0.0

    def tokens(self, n, seed):
        return [int(x) for x in np.random.default_rng(seed).integers(0, self.vocab, size=n)]

    def plain(self, toks):
        from tests.plain import forward_logits

        key = tuple(toks)
        if key not in self._plain:
            self._plain[key] = forward_logits(self.weights, self.raw, toks)
        return self._plain[key]

    def replay(self, steps):
        from machserve_b200.engine.replay import replay

        out = replay(self.runner, steps)
        self.runner.cache.check()
        assert not self.runner.cache.requests, "requests still hold cache after the trace ended"
        self.runner.check_device_status()
        return collect_rows(steps, out)

    def compare(self, got, toks, what, rows=None):
        want = self.plain(toks)
        if rows is not None:
            want = want[rows]
        tol = F32_TOL if self.dtype == "float32" else BF16_TOL
        assert_close(got, want, tol, f"{self.size} {self.dtype} {what}")
        self.worst = max(self.worst, float(np.abs(got - want).max() / max(1.0, np.abs(want).max())))


@pytest.fixture(scope="module", params=CASES, ids=[f"{s}-{d}" for s, d in CASES])
def world(request):
    w = World(*request.param)
    yield w
    print(f"\n[real sizes] {w.size} {w.dtype}: worst error relative to the largest logit {w.worst:.3g}")
    del w.runner


def test_whole_tail_and_portions(world):
    n = SIZES[world.size]["long"]
    toks = world.tokens(n, 1)
    whole = world.replay(trace_whole({"a": toks}))["a"]
    world.compare(whole, toks, "whole")
    tail = world.replay(trace_tail_decode("a", toks, 32))["a"]
    world.compare(tail, toks, "last 32 tokens one by one")
    sizes = [130, 2, 64, 7, 128, 33, 256, 3, 65, 2, 190]
    portions = world.replay(trace_portions("a", toks, sizes))["a"]
    world.compare(portions, toks, "portions of changing size")
    if world.dtype == "float32":
        # float32: every kernel's arithmetic for a row depends on the row's position alone
        assert np.array_equal(whole, portions), "float32 logits differ between the whole prompt and its portions"
        assert np.array_equal(whole, tail), "float32 logits differ between the whole prompt and the decoded tail"


def test_decoding_across_512_and_1024(world):
    """A prompt of 500 tokens, then one by one: the context passes 512 (and 1,024 where the case is that long)."""
    n = SIZES[world.size]["long"]
    toks = world.tokens(n, 1)  # the tokens of the test before: the plain logits are there already
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:500], "want": [499]}], "end": []}]
    for i in range(500, n):
        steps.append({"step": i - 499, "entries": [{"id": "a", "tokens": [toks[i]], "want": [0]}], "end": []})
    steps[-1]["end"] = ["a"]
    got = world.replay(steps)["a"]
    world.compare(got, toks, "decoding from 500 on", rows=slice(499, n))
    if world.dtype == "float32":
        whole = world.replay(trace_whole({"a": toks}))["a"]
        assert np.array_equal(whole[499:], got), "float32 logits differ between decoding and the whole prompt"


def mixed_trace(world):
    """Six decoding requests beside two prompts that come in portions; step 3 is the benchmark's 7B step in small:
    two portions of 130 rows, each with earlier tokens in the cache, and six single rows."""
    lens = {"d1": 70, "d2": 90, "d3": 140, "d4": 200, "d5": 65, "d6": 129, "p1": 432, "p2": 364}
    req = {r: world.tokens(n + 6, 10 + i) for i, (r, n) in enumerate(lens.items())}
    at = {r: 0 for r in req}

    def take(r, n):
        e = {"id": r, "tokens": req[r][at[r] : at[r] + n], "want": list(range(n))}
        at[r] += n
        return e

    ds = ["d1", "d2", "d3", "d4", "d5", "d6"]
    steps = [
        [take(r, lens[r]) for r in ds[:3]],
        [take(r, lens[r]) for r in ds[3:]],
        [take("p1", 300), take("p2", 170)],
        [take("p1", 130), take("p2", 130)] + [take(r, 1) for r in ds],
        [take("p1", 2), take("p2", 64)] + [take(r, 1) for r in ds],
    ]
    for _ in range(4):
        steps.append([take(r, 1) for r in ["p1", "p2"] + ds])
    out = [{"step": i, "entries": e, "end": []} for i, e in enumerate(steps)]
    out[-1]["end"] = list(req)
    return {r: req[r][: at[r]] for r in req}, out


def test_mixed_portions_beside_decoding_rows(world):
    req, steps = mixed_trace(world)
    assert len(steps[3]["entries"]) == 8 and sum(len(e["tokens"]) for e in steps[3]["entries"]) == 266
    got = world.replay(steps)
    for r, toks in req.items():
        world.compare(got[r], toks, f"mixed {r}")
    if world.dtype == "float32":
        alone = world.replay(trace_whole({"p1": req["p1"]}))["p1"]
        assert np.array_equal(alone, got["p1"]), "float32 logits differ between the mixed trace and the request alone"
