"""Each part alone against its plain counterpart, and a model put together from other parts.

The second half defines, in this file only, a mixer with a state of its own, a routed
feed-forward, a position encoding that is no rotation, and an architecture that mixes them
with attention layers, runs one layer twice and lets a run read another run's cache.  They
are registered, built and stepped without any change to the framework's files, and compared
with a plain computation written here.
"""
import json
from dataclasses import dataclass

import numpy as np
import pytest

from tests.helpers import BF16_TOL, F32_TOL, TINY, assert_close, make_model_dir, random_tokens
from tests.plain import attention_block, decoder_layer, read_model_dir, rms_norm, rope_angles, swiglu
from tests.plain.model import bf16_round

pytestmark = pytest.mark.gpu


def _runner(model_dir, dtype, page=8, tokens=256, **kw):
    from machserve_b200.engine import ModelRunner

    return ModelRunner.from_model_dir(model_dir, dtype=dtype, page_size=page, num_pages=tokens // page, max_requests=4,
                                      max_step_tokens=tokens, max_seq_len=tokens, **kw)


def _step_context(runner, entries):
    """The context the step function would hand to the parts for these entries."""
    from machserve_b200.engine import StepEntry

    entries = [StepEntry(*e) for e in entries]
    runner.reserve(entries)
    runner._upload_tables()
    return runner._stage(entries), entries


def _n(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("name", list(TINY))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parts_alone(model_root, name, dtype):
    """Norm, rotary table, attention mixer, feed-forward, block, embedding and head of a tiny model, one at a time."""
    import torch

    d = make_model_dir(model_root, name)
    bf16 = dtype == "bfloat16"
    cfg, w = read_model_dir(d, round_to_bf16=bf16)
    runner = _runner(d, dtype, page=TINY[name]["page"])
    model, rt = runner.model, runner.rt
    tdt = torch.bfloat16 if bf16 else torch.float32
    tol = BF16_TOL if bf16 else F32_TOL
    hidden, vocab = cfg["hidden_size"], cfg["vocab_size"]
    rng = np.random.default_rng(5)
    # two sequences in one step: 19 and 7 tokens
    toks = [random_tokens(vocab, 19, 1), random_tokens(vocab, 7, 2)]
    ctx, _ = _step_context(runner, [("a", toks[0], [18]), ("b", toks[1], [0, 6])])
    t = 26
    layer = len(model.blocks) - 1  # the last layer: windowed in tiny-C
    block = model.blocks[layer]
    prefix = f"model.layers.{layer}."

    # embedding
    res = torch.empty((t, hidden), dtype=torch.float32, device=rt.device)
    model.embedding.forward(ctx, res)
    want = w["model.embed_tokens.weight"][np.array(toks[0] + toks[1])]
    assert np.array_equal(_n(res), want)

    # norm: adds the delta to the residual first
    x = rng.normal(size=(t, hidden)) * 2
    delta = rng.normal(size=(t, hidden))
    xr = bf16_round(x.astype(np.float32)).astype(np.float64) if bf16 else x.astype(np.float32).astype(np.float64)
    dr = bf16_round(delta.astype(np.float32)).astype(np.float64) if bf16 else delta.astype(np.float32).astype(np.float64)
    res = torch.tensor(x, dtype=torch.float32, device=rt.device)
    out = torch.empty((t, hidden), dtype=tdt, device=rt.device)
    block.mixer_norm.forward(res, torch.tensor(delta, dtype=tdt, device=rt.device), out)
    summed = x.astype(np.float32).astype(np.float64) + dr
    assert_close(_n(res), summed, 1e-6, "residual after the add")
    # In bfloat16 a part that takes its norm into its own kernels has the norm's weight folded into the columns of
    # its first matrix, and the norm keeps a weight of one: norm and part together compute what they always did.
    assert block.fuse_mixer == block.fuse_feed_forward == bf16
    g1 = w[prefix + "input_layernorm.weight"]
    g2 = w[prefix + "post_attention_layernorm.weight"]
    assert_close(_n(out), rms_norm(summed, np.ones_like(g1) if bf16 else g1, cfg["rms_norm_eps"]), tol / 4, "norm")

    # rotary table against the plain angles
    table = block.mixer.position.rotary_table(rt)
    ang = rope_angles(np.arange(table.shape[0]), block.mixer.hd, cfg["rope_theta"])
    assert np.abs(_n(table[..., 0]) - np.cos(ang)).max() < 1e-7 and np.abs(_n(table[..., 1]) - np.sin(ang)).max() < 1e-7

    # attention mixer and feed-forward, given the same normed input
    positions = np.concatenate([np.arange(19), np.arange(7)])
    xn_t = torch.tensor(xr, dtype=tdt, device=rt.device)
    from tests.plain.model import layer_window

    got = _n(block.mixer.forward(ctx, xn_t, runner.bindings[layer]))
    xa, xf = (xr * g1, xr * g2) if bf16 else (xr, xr)  # what the folded matrices stand for
    want = np.concatenate([
        attention_block(xa[:19], w, prefix, cfg, positions[:19], layer_window(cfg, layer)),
        attention_block(xa[19:], w, prefix, cfg, positions[19:], layer_window(cfg, layer)),
    ])
    assert_close(got, want, tol, "attention mixer")
    got = _n(block.feed_forward.forward(ctx, xn_t))
    m = prefix + "mlp."
    assert_close(got, swiglu(xf, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"]), tol, "feed-forward")

    # the block: residual in, residual + both deltas out (the last delta is handed on, not yet added)
    res = torch.tensor(x, dtype=torch.float32, device=rt.device)
    pending = block.forward(ctx, res, None, runner.bindings[layer])
    x32 = x.astype(np.float32).astype(np.float64)
    want = np.concatenate([decoder_layer(x32[:19], w, layer, cfg, positions[:19]), decoder_layer(x32[19:], w, layer, cfg, positions[19:])])
    assert_close(_n(res) + _n(pending), want, tol, "block")

    # final norm on picked rows, and the head
    final = torch.empty((3, hidden), dtype=tdt, device=rt.device)
    res = torch.tensor(x, dtype=torch.float32, device=rt.device)
    model.final_norm.forward(res, None, final, rows=ctx.want_rows)
    rows = np.array([18, 19, 25])
    want_final = rms_norm(x32[rows], w["model.norm.weight"], cfg["rms_norm_eps"])
    assert_close(_n(final), want_final, tol / 4, "final norm of the wanted rows")
    logits = torch.empty((3, vocab), dtype=torch.float32, device=rt.device)
    model.head.forward(ctx, final, logits)
    head_w = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    assert_close(_n(logits), _n(final) @ head_w.T, tol / 4, "head")
    if cfg["tie_word_embeddings"]:
        assert model.head.weight.data_ptr() == model.embedding.table.data_ptr()  # one copy in memory


# =============================================================== parts defined in this test


def _define_toy_parts():
    """Registers the toy parts and the toy architecture.  Everything here uses the public interfaces only."""
    import torch

    from machserve_b200.config import ModelConfig, register_architecture
    from machserve_b200.config.spec import LayerSpec, ModelSpec, RunSpec, part
    from machserve_b200.parts import (
        FeedForward, FixedState, Mixer, PositionEncoding, matrix, register_feed_forward, register_mixer,
        register_position_encoding,
    )
    from machserve_b200.weights import TensorDecl

    @register_mixer("toy_decay")
    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + W_in x_t ; y_t = W_out s_t.  The state s is per request, of fixed size."""

        def __init__(self, spec):
            super().__init__(spec)
            self.prefix, self.hidden, self.state, self.decay = spec["prefix"], spec["hidden_size"], spec["state_size"], spec["decay"]

        def tensors(self):
            return [TensorDecl(self.prefix + "in.weight", (self.state, self.hidden)),
                    TensorDecl(self.prefix + "out.weight", (self.hidden, self.state))]

        def cache_need(self):
            return FixedState((self.state,))

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.w_in = tensors[self.prefix + "in.weight"].to(torch.float32)
            self.w_out = tensors[self.prefix + "out.weight"].to(torch.float32)

        def forward(self, ctx, x, cache, owns_cache=True):
            u = x.float() @ self.w_in.T
            y = torch.empty_like(u)
            for i in range(ctx.num_seqs):  # rows of a sequence are adjacent and in order
                a, b = ctx.host_cu_tokens[i], ctx.host_cu_tokens[i + 1]
                s = cache.state[ctx.host_state_slots[i]].clone()
                for r in range(a, b):
                    s = self.decay * s + u[r]
                    y[r] = s
                if owns_cache:
                    cache.state[ctx.host_state_slots[i]] = s
            return (y @ self.w_out.T).to(self.rt.dtype)

    @register_feed_forward("toy_routed")
    class RoutedFeedForward(FeedForward):
        """Two experts, each a plain matrix; a token goes to the one its router logit prefers, scaled by the margin."""

        def __init__(self, spec):
            super().__init__(spec)
            self.prefix, self.hidden = spec["prefix"], spec["hidden_size"]

        def tensors(self):
            return [TensorDecl(self.prefix + "router.weight", (2, self.hidden)),
                    TensorDecl(self.prefix + "experts.weight", (2, self.hidden, self.hidden))]

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.router = tensors[self.prefix + "router.weight"].to(torch.float32)
            self.experts = tensors[self.prefix + "experts.weight"].to(torch.float32)

        def forward(self, ctx, x):
            xf = x.float()
            logits = xf @ self.router.T  # router logits in float32
            pick = (logits[:, 1] > logits[:, 0]).long()
            gate = torch.sigmoid((logits[:, 1] - logits[:, 0]).abs())
            y = torch.einsum("td,tod->to", xf, self.experts[pick]) * gate[:, None]
            return y.to(self.rt.dtype)

    @register_position_encoding("toy_scale")
    class ScalePositions(PositionEncoding):
        """No rotation: q and k are multiplied by (1 + slope * position).  It has no rotary table, so the
        attention mixer calls apply()."""

        def __init__(self, spec):
            super().__init__(spec)
            self.slope = spec["slope"]

        def apply(self, ctx, q, k):
            f = (1.0 + self.slope * ctx.positions.float())[:, None, None]
            q.copy_((q.float() * f).to(q.dtype))
            if k is not None:
                k.copy_((k.float() * f).to(k.dtype))

    @register_architecture("ToyMixForCausalLM")
    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab_size: int
        hidden_size: int
        state_size: int
        decay: float
        eps: float

        @classmethod
        def from_json(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"], raw["state_size"], raw["decay"], raw["eps"])

        def to_json(self):
            return {"architectures": ["ToyMixForCausalLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "state_size": self.state_size, "decay": self.decay, "eps": self.eps}

        def model_spec(self):
            h = self.hidden_size

            def norm(name):
                return part("rmsnorm", tensor=name, size=h, eps=self.eps)

            def attention(prefix, position):
                return part("attention", prefix=prefix, hidden_size=h, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25,
                            window=None, qkv_bias=False, position=position)

            layers = (
                # layer 0: attention with rotary positions, dense feed-forward
                LayerSpec("prenorm", attention("l0.attn.", part("rope", head_dim=16, rotary_dim=8, theta=100.0, pairing="interleaved")),
                          part("swiglu", prefix="l0.mlp.", hidden_size=h, intermediate_size=40), norm("l0.n1"), norm("l0.n2"), "l0."),
                # layer 1: the mixer with a state of its own, routed feed-forward
                LayerSpec("prenorm", part("toy_decay", prefix="l1.mix.", hidden_size=h, state_size=self.state_size, decay=self.decay),
                          part("toy_routed", prefix="l1.ffn.", hidden_size=h), norm("l1.n1"), norm("l1.n2"), "l1."),
                # layer 2: attention with the toy position encoding
                LayerSpec("prenorm", attention("l2.attn.", part("toy_scale", slope=0.01)),
                          part("swiglu", prefix="l2.mlp.", hidden_size=h, intermediate_size=24), norm("l2.n1"), norm("l2.n2"), "l2."),
            )
            # layer 1 runs twice (each run has a state of its own); the last run is layer 0 again, reading
            # the keys and values that its first run wrote
            order = (RunSpec(0), RunSpec(1), RunSpec(2), RunSpec(1), RunSpec(0, cache_of=0))
            return ModelSpec("ToyMixForCausalLM", h, self.vocab_size,
                             part("embedding", tensor="emb", vocab_size=self.vocab_size, hidden_size=h), layers, order,
                             norm("final"), part("lm_head", tensor="head", tied_to=None, vocab_size=self.vocab_size, hidden_size=h), 512)

    return ToyConfig


def _toy_plain(w, cfg, tokens):
    """The toy model computed plainly: whole sequence, no cache, float64."""
    from tests.plain import causal_attention, linear

    t = len(tokens)
    pos = np.arange(t)
    x = w["emb"][np.array(tokens)]
    eps = cfg["eps"]

    def attn(xn, p, mode, kv=None):
        q = linear(xn, w[p + "q_proj.weight"]).reshape(t, 4, 16)
        if kv is None:
            k = linear(xn, w[p + "k_proj.weight"]).reshape(t, 2, 16)
            v = linear(xn, w[p + "v_proj.weight"]).reshape(t, 2, 16)
        if mode == "rope":  # interleaved pairs (2j, 2j+1) over the first 8 coordinates, theta 100
            ang = pos[:, None] / 100.0 ** (2.0 * np.arange(4) / 8)
            c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]

            def rot(a):
                out = a.copy()
                out[..., 0:8:2] = a[..., 0:8:2] * c - a[..., 1:8:2] * s
                out[..., 1:8:2] = a[..., 0:8:2] * s + a[..., 1:8:2] * c
                return out

            q = rot(q)
            if kv is None:
                k = rot(k)
        else:
            f = (1.0 + 0.01 * pos)[:, None, None]
            q = q * f
            if kv is None:
                k = k * f
        if kv is not None:
            k, v = kv
        a = causal_attention(q * (0.25 / 16 ** -0.5), k, v)  # the mixer's scale is 0.25, the plain function's 1/4 too
        return linear(a.reshape(t, 64), w[p + "o_proj.weight"]), (k, v)

    def decay(xn, p):
        u = linear(xn, w[p + "in.weight"])
        s, ys = np.zeros(cfg["state_size"]), []
        for r in range(t):
            s = cfg["decay"] * s + u[r]
            ys.append(s.copy())
        return linear(np.stack(ys), w[p + "out.weight"])

    def routed(xn, p):
        logits = linear(xn, w[p + "router.weight"])
        pick = (logits[:, 1] > logits[:, 0]).astype(int)
        gate = 1.0 / (1.0 + np.exp(-np.abs(logits[:, 1] - logits[:, 0])))
        return np.einsum("td,tod->to", xn, w[p + "experts.weight"][pick]) * gate[:, None]

    def dense(xn, p):
        return swiglu(xn, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])

    kv0 = None
    for layer, shared in ((0, False), (1, False), (2, False), (1, False), (0, True)):
        p = f"l{layer}."
        xn = rms_norm(x, w[p + "n1"], eps)
        if layer == 0:
            d, kv = attn(xn, p + "attn.", "rope", kv0 if shared else None)
            kv0 = kv0 or kv
        elif layer == 2:
            d, _ = attn(xn, p + "attn.", "scale")
        else:
            d = decay(xn, p + "mix.")
        x = x + d
        xn = rms_norm(x, w[p + "n2"], eps)
        x = x + (routed(xn, p + "ffn.") if layer == 1 else dense(xn, p + "mlp."))
    return linear(rms_norm(x, w["final"], eps), w["head"])


def test_toy_parts_are_registered_built_and_stepped(tmp_path):
    """A mixer with state, a routed feed-forward, another position encoding and a new architecture, all
    defined above: written to a model folder by the random-weights mode, loaded, and replayed whole, in
    portions, token by token and mixed with another request; all against the plain computation."""
    from machserve_b200.config import config_from_json, unregister_architecture
    from machserve_b200.engine.replay import replay
    from machserve_b200.parts import FEED_FORWARDS, MIXERS, POSITION_ENCODINGS
    from machserve_b200.weights import write_random_model
    from tests.helpers import collect_rows, trace_portions, trace_tail_decode, trace_whole

    _define_toy_parts()
    try:
        raw = {"architectures": ["ToyMixForCausalLM"], "vocab_size": 90, "hidden_size": 48, "state_size": 20, "decay": 0.8, "eps": 1e-5}
        cfg = config_from_json(raw)
        d = write_random_model(cfg, tmp_path / "toy", seed=4, weight_std=0.15, norm_std=0.1)
        assert json.loads((d / "config.json").read_text())["architectures"] == ["ToyMixForCausalLM"]
        _, w = read_model_dir(d)
        runner = _runner(d, "float32", page=8, tokens=192)
        assert not runner.use_graphs  # the toy mixer loops on the host: its steps are never captured
        needs = runner.model.cache_needs()
        assert [type(n).__name__ if n else None for n in needs] == ["PagedCache", "FixedState", "PagedCache", "FixedState", None]
        assert len(runner.cache.groups) == 1 and runner.cache.groups[0].runs == [0, 2] and sorted(runner.states) == [1, 3]

        a, b = random_tokens(90, 45, 1), random_tokens(90, 30, 2)
        want = {"a": _toy_plain(w, raw, a), "b": _toy_plain(w, raw, b)}
        for steps in (trace_whole({"a": a, "b": b}), trace_tail_decode("a", a, 20), trace_portions("b", b, [5, 2, 9, 3])):
            got = collect_rows(steps, replay(runner, steps))
            for rid in got:
                assert_close(got[rid], want[rid], F32_TOL, f"toy model {rid}")
            assert not runner.cache.requests
        # both requests live at once, portions of one beside single tokens of the other; slots are reused
        steps, ia, ib, n = [], 0, 0, 0
        while ia < len(a) or ib < len(b):
            entries = []
            if ia < len(a):
                k = 6 if ia < 30 else 1
                entries.append({"id": "a", "tokens": a[ia : ia + k], "want": list(range(len(a[ia : ia + k])))}); ia += k
            if ib < len(b) and n >= 2:
                k = 1 if n % 2 else 4
                entries.append({"id": "b", "tokens": b[ib : ib + k], "want": list(range(len(b[ib : ib + k])))}); ib += k
            steps.append({"step": n, "entries": entries, "end": [r for r, i, s in (("a", ia, a), ("b", ib, b)) if i >= len(s) and any(e["id"] == r for e in entries)]})
            n += 1
        got = collect_rows(steps, replay(runner, steps))
        for rid in ("a", "b"):
            assert_close(got[rid], want[rid], F32_TOL, f"toy model mixed {rid}")
        runner.cache.check()
        assert not runner.cache.requests
    finally:
        unregister_architecture("ToyMixForCausalLM")
        MIXERS.unregister("toy_decay")
        FEED_FORWARDS.unregister("toy_routed")
        POSITION_ENCODINGS.unregister("toy_scale")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_dump_follows_the_plain_layers(model_root, dtype):
    """The step function's tap gives the hidden rows after the embedding and after every layer: a prompt, then a
    decoding step (in bfloat16 the few-row path, whose deltas are added by the products themselves)."""
    from machserve_b200.engine import StepEntry
    from tests.plain import embedding

    d = make_model_dir(model_root, "B")
    bf16 = dtype == "bfloat16"
    cfg, w = read_model_dir(d, round_to_bf16=bf16)
    runner = _runner(d, dtype, page=TINY["B"]["page"])
    toks = random_tokens(cfg["vocab_size"], 12, 9)
    want, x = [], embedding(w["model.embed_tokens.weight"], toks)
    want.append(x)
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, layer, cfg, np.arange(len(toks)))
        want.append(x)
    tol = BF16_TOL if bf16 else F32_TOL
    got = {}
    runner.step([StepEntry("a", toks[:11], [])], tap=lambda i, h: got.__setitem__(i, _n(h)))
    assert sorted(got) == list(range(-1, cfg["num_hidden_layers"]))
    for i in got:
        assert_close(got[i], want[i + 1][:11], tol, f"hidden rows after run {i} of the prompt")
    got.clear()
    runner.step([StepEntry("a", toks[11:], [0])], tap=lambda i, h: got.__setitem__(i, _n(h)))
    for i in got:
        assert_close(got[i], want[i + 1][11:], tol, f"hidden rows after run {i} of the decoded token")
