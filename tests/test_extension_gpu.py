"""What another architecture would add, added here and nowhere else.

Every part below is defined in this file, registered, built from a spec and stepped through
`ModelRunner.step` without a change to the framework's files:

* an embedding that scales its rows and a head with a bias and a soft cap (registries of the two ends);
* a mixer that keeps ONE plane per token of a width of its own in the paged cache and asks for a
  work list of its own with every step (`cache_need`, `plan_key`, `plan`);
* a feed-forward that joins the few-row path of the pre-norm block through the protocol
  (`fuse_norm`, `forward_fused`), checked by the number of launches of the layer;
* a norm and a block of other kinds after built-in layers, in bfloat16 with 1 to 16 rows, where the
  built-in parts hand their successor row statistics instead of a delta;
* two layers whose norms read the same tensor.

Each model is compared with a plain float64 computation written beside it.
"""
from dataclasses import dataclass

import numpy as np
import pytest

from tests.helpers import BF16_TOL, F32_TOL, assert_close, collect_rows, random_tokens, trace_portions, trace_tail_decode, trace_whole
from tests.plain import causal_attention, linear, rms_norm, rope, swiglu
from tests.plain.model import bf16_round

pytestmark = pytest.mark.gpu

H, HEADS, KV, HD, INTER, VOCAB, LATENT = 64, 4, 2, 16, 72, 120, 24
EPS, THETA = 1e-5, 10000.0


def _register():
    """Registers the toy parts and architectures; returns the function that takes them out again."""
    import torch

    from machserve_b200 import ops
    from machserve_b200.config import ModelConfig, register_architecture, unregister_architecture
    from machserve_b200.config.spec import LayerSpec, ModelSpec, RunSpec, part
    from machserve_b200.parts import (
        BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS as HEAD_KINDS, MIXERS, NORMS, Block, CachePlane, FeedForward, Head, Mixer,
        Norm, PagedCache, RowStats, TokenEmbedding, WorkPlan, as_delta, matrix, register_block, register_embedding,
        register_feed_forward, register_head, register_mixer, register_norm, vector_f32,
    )
    from machserve_b200.weights import TensorDecl

    @register_embedding("toy_scaled_embedding")
    class ScaledEmbedding(TokenEmbedding):
        graph_safe = True

        def __init__(self, spec):
            super().__init__(spec)
            self.name, self.vocab, self.hidden, self.scale = spec["tensor"], spec["vocab_size"], spec["hidden_size"], spec["scale"]

        def tensors(self):
            return [TensorDecl(self.name, (self.vocab, self.hidden))]

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.table = matrix(tensors[self.name], rt)

        def forward(self, ctx, out):
            ops.embed_gather(self.table, ctx.token_ids, out)
            return out.mul_(self.scale)

    @register_head("toy_softcap_head")
    class SoftCapHead(Head):
        """logits = cap * tanh((x . W^T + b) / cap): a biased product in the runtime's dtype, then the cap."""

        graph_safe = True

        def __init__(self, spec):
            super().__init__(spec)
            self.name, self.vocab, self.hidden, self.cap = spec["tensor"], spec["vocab_size"], spec["hidden_size"], spec["cap"]

        def tensors(self):
            return [TensorDecl(self.name + ".weight", (self.vocab, self.hidden)), TensorDecl(self.name + ".bias", (self.vocab,), init="bias")]

        def bind(self, tensors, rt, embedding=None):
            super().bind(tensors, rt, embedding)
            self.weight, self.bias = matrix(tensors[self.name + ".weight"], rt), vector_f32(tensors[self.name + ".bias"])

        def forward(self, ctx, x, out):
            ops.linear(x, self.weight, self.bias, out)
            return out.copy_(self.cap * torch.tanh(out / self.cap))

    @register_mixer("toy_latent")
    class LatentMixer(Mixer):
        """c_t = W_c x_t is kept per token in one plane of width `latent`; y_t = W_o mean(c_0 .. c_t).
        It asks for the step's sequences cut into chunks of up to five rows and works through them in order."""

        CHUNK = 5

        def __init__(self, spec):
            super().__init__(spec)
            self.prefix, self.hidden, self.latent = spec["prefix"], spec["hidden_size"], spec["latent"]

        def tensors(self):
            return [TensorDecl(self.prefix + "c.weight", (self.latent, self.hidden)), TensorDecl(self.prefix + "o.weight", (self.hidden, self.latent))]

        def cache_need(self):
            return PagedCache((CachePlane("c", 1, self.latent),), None)

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.w_c, self.w_o = tensors[self.prefix + "c.weight"].float(), tensors[self.prefix + "o.weight"].float()

        def plan_key(self):
            return ("toy_latent", self.CHUNK)

        def plan_words(self, max_rows, max_seqs):
            return 3 * (max_rows // self.CHUNK + max_seqs)

        def plan(self, step):
            row0, rows, seq = [], [], []
            for i, (r, n) in enumerate(zip(step.row0, step.count)):
                for a in range(0, n, self.CHUNK):
                    row0.append(r + a)
                    rows.append(min(self.CHUNK, n - a))
                    seq.append(i)
            return WorkPlan({"chunk_row0": row0, "chunk_rows": rows, "chunk_seq": seq}, (len(row0),))

        def forward(self, ctx, x, cache, owns_cache=True):
            work = ctx.work[self.plan_key()]
            assert work.shape == (work.sizes["chunk_row0"],)
            pages, table = cache.planes["c"], cache.block_table(ctx)  # [num_pages, 1, page, latent]
            page = pages.shape[2]
            c = (x.float() @ self.w_c.T).to(pages.dtype)
            pos, slot = ctx.positions.tolist(), ctx.slot_of_token.tolist()
            table_host = table.tolist()
            out = torch.zeros((x.shape[0], self.latent), dtype=torch.float32, device=x.device)
            chunks = zip(work.lists["chunk_row0"].tolist(), work.lists["chunk_rows"].tolist(), work.lists["chunk_seq"].tolist())
            for r0, n, _ in chunks:  # the lists as they arrived on the device
                for r in range(r0, r0 + n):
                    pages[table_host[slot[r]][pos[r] // page], 0, pos[r] % page] = c[r]
                    held = [pages[table_host[slot[r]][p // page], 0, p % page].float() for p in range(pos[r] + 1)]
                    out[r] = torch.stack(held).mean(0)
            return (out @ self.w_o.T).to(self.rt.dtype)

    @register_feed_forward("toy_linear2")
    class TwoMatrices(FeedForward):
        """delta = W2 (W1 x), with the norm in front and the add behind done by its own products when rows are few."""

        graph_safe = True
        fused_rows = 16

        def __init__(self, spec):
            super().__init__(spec)
            self.prefix, self.hidden, self.inter = spec["prefix"], spec["hidden_size"], spec["intermediate_size"]

        def tensors(self):
            return [TensorDecl(self.prefix + "w1", (self.inter, self.hidden)), TensorDecl(self.prefix + "w2", (self.hidden, self.inter))]

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.w1, self.w2 = matrix(tensors[self.prefix + "w1"], rt), matrix(tensors[self.prefix + "w2"], rt)

        def fuse_norm(self, norm):
            return self.rt.dtype == torch.bfloat16 and norm.fold_into(self.w1)

        def forward_fused(self, ctx, residual, pending, norm, cache=None, owns_cache=True):
            ws, (t, d) = self.rt.workspace, residual.shape
            nb = ops.gemm_small_m_stats_blocks(d)
            h = ws.get("toy.h", (t, self.inter), self.rt.dtype)
            if isinstance(pending, RowStats) and pending.copy is not None:
                ops.gemm_small_m_scaled(pending.copy, pending.stats, pending.blocks, norm.eps, self.w1, None, h)
            else:
                xn = ws.get("toy.xn", (t, d), self.rt.dtype)
                norm.forward(residual, as_delta(pending), xn)
                ops.linear(xn, self.w1, None, h)
            stats, copy = ws.get("toy.stats", (t, nb), torch.float32), ws.get("toy.copy", (t, d), self.rt.dtype)
            ops.gemm_small_m_resadd(h, self.w2, residual, stats, copy)
            return RowStats(stats, nb, copy)

        def forward(self, ctx, x):
            ws, t = self.rt.workspace, x.shape[0]
            h = ops.linear(x, self.w1, None, ws.get("toy.h", (t, self.inter), self.rt.dtype))
            return ops.linear(h, self.w2, None, ws.get("toy.delta", (t, self.hidden), self.rt.dtype))

    @register_norm("toy_centered")
    class CenteredNorm(Norm):
        """y = (x - mean) / sqrt(var + eps) * w; it knows nothing of row statistics and folds into nothing."""

        graph_safe = True

        def __init__(self, spec):
            super().__init__(spec)
            self.name, self.size, self.eps = spec["tensor"], spec["size"], spec["eps"]

        def tensors(self):
            return [TensorDecl(self.name, (self.size,), init="scale")]

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.weight = vector_f32(tensors[self.name])

        def forward(self, residual, delta, out, rows=None):
            assert delta is None or isinstance(delta, torch.Tensor), "a norm is given a delta or None, never row statistics"
            if rows is not None:
                x = residual[rows.long()] + (delta[rows.long()].float() if delta is not None else 0.0)
            else:
                if delta is not None:
                    residual += delta[: residual.shape[0]].float()
                x = residual
            y = (x - x.mean(1, keepdim=True)) / torch.sqrt(x.var(1, unbiased=False, keepdim=True) + self.eps) * self.weight
            return out.copy_(y)

    @register_block("toy_parallel")
    class ParallelBlock(Block):
        """x += mixer(norm(x)) + feed_forward(norm(x)), one norm for both (its second norm is not used)."""

        graph_safe = True

        def forward(self, ctx, residual, pending, cache, owns_cache=True):
            assert pending is None or isinstance(pending, torch.Tensor), "a block of another kind is given a delta or None"
            rt, (t, d) = ctx.rt, residual.shape
            xn = rt.workspace.get("toy.par", (t, d), rt.dtype)
            self.mixer_norm.forward(residual, pending, xn)
            a = self.mixer.forward(ctx, xn, cache, owns_cache).float()
            return (a + self.feed_forward.forward(ctx, xn).float()).to(rt.dtype)

    def rms(name):
        return part("rmsnorm", tensor=name, size=H, eps=EPS)

    def attention(prefix):
        return part("attention", prefix=prefix, hidden_size=H, num_heads=HEADS, num_kv_heads=KV, head_dim=HD, scale=HD ** -0.5,
                    window=None, qkv_bias=True, position=part("rope", head_dim=HD, rotary_dim=HD, theta=THETA, pairing="half"))

    def dense(prefix):
        return part("swiglu", prefix=prefix, hidden_size=H, intermediate_size=INTER)

    def model(name, layers, embedding=None, final=None, head=None, order=None):
        return ModelSpec(
            name, H, VOCAB, embedding or part("embedding", tensor="emb", vocab_size=VOCAB, hidden_size=H), layers,
            order or tuple(RunSpec(i) for i in range(len(layers))), final or rms("final"),
            head or part("lm_head", tensor="head", tied_to=None, vocab_size=VOCAB, hidden_size=H), 512)

    specs = {
        # scaled embedding and capped head around a latent-cache layer between two attention layers
        "ToyEndsForCausalLM": lambda: model("ToyEndsForCausalLM", (
            LayerSpec("prenorm", attention("l0.attn."), dense("l0.mlp."), rms("l0.n1"), rms("l0.n2"), "l0."),
            LayerSpec("prenorm", part("toy_latent", prefix="l1.mix.", hidden_size=H, latent=LATENT), dense("l1.mlp."), rms("l1.n1"), rms("l1.n2"), "l1."),
            LayerSpec("prenorm", attention("l2.attn."), dense("l2.mlp."), rms("l2.n1"), rms("l2.n2"), "l2."),
        ), embedding=part("toy_scaled_embedding", tensor="emb", vocab_size=VOCAB, hidden_size=H, scale=3.0),
            head=part("toy_softcap_head", tensor="head", vocab_size=VOCAB, hidden_size=H, cap=2.0)),
        # built-in layers, then a layer with a norm of another kind, then a block of another kind, a final norm of another kind
        "ToyKindsForCausalLM": lambda: model("ToyKindsForCausalLM", (
            LayerSpec("prenorm", attention("l0.attn."), dense("l0.mlp."), rms("l0.n1"), rms("l0.n2"), "l0."),
            LayerSpec("prenorm", attention("l1.attn."), dense("l1.mlp."),
                      part("toy_centered", tensor="l1.n1", size=H, eps=EPS), part("toy_centered", tensor="l1.n2", size=H, eps=EPS), "l1."),
            LayerSpec("prenorm", attention("l2.attn."), part("toy_linear2", prefix="l2.ffn.", hidden_size=H, intermediate_size=INTER),
                      rms("l2.n1"), rms("l2.n2"), "l2."),
            LayerSpec("toy_parallel", attention("l3.attn."), dense("l3.mlp."), rms("l3.n1"), rms("l3.n2"), "l3."),
        ), final=part("toy_centered", tensor="final", size=H, eps=EPS)),
        # two layers whose norms read the same tensors
        "ToySharedForCausalLM": lambda: model("ToySharedForCausalLM", (
            LayerSpec("prenorm", attention("l0.attn."), dense("l0.mlp."), rms("shared.n1"), rms("shared.n2"), "l0."),
            LayerSpec("prenorm", attention("l1.attn."), dense("l1.mlp."), rms("shared.n1"), rms("shared.n2"), "l1."),
        )),
    }

    for arch, make in specs.items():
        @register_architecture(arch)
        @dataclass(frozen=True)
        class ToyConfig(ModelConfig):
            name: str

            @classmethod
            def from_json(cls, raw):
                return cls(raw["architectures"][0])

            def to_json(self):
                return {"architectures": [self.name]}

            def model_spec(self):
                return specs[self.name]()

    def unregister():
        for arch in specs:
            unregister_architecture(arch)
        EMBEDDINGS.unregister("toy_scaled_embedding")
        HEAD_KINDS.unregister("toy_softcap_head")
        MIXERS.unregister("toy_latent")
        FEED_FORWARDS.unregister("toy_linear2")
        NORMS.unregister("toy_centered")
        BLOCKS.unregister("toy_parallel")

    return unregister


# --------------------------------------------------------------------------------------- plain computations


def _attention(xn, w, p):
    t = xn.shape[0]
    pos = np.arange(t)
    q = rope(linear(xn, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).reshape(t, HEADS, HD), pos, THETA)
    k = rope(linear(xn, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).reshape(t, KV, HD), pos, THETA)
    v = linear(xn, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).reshape(t, KV, HD)
    return linear(causal_attention(q, k, v).reshape(t, HEADS * HD), w[p + "o_proj.weight"])


def _dense(xn, w, p):
    return swiglu(xn, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])


def _centered(x, g):
    return (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + EPS) * g


def _prenorm(x, w, p, mixer, ff, n1=rms_norm, n2=rms_norm, names=None):
    a, b = names or (p + "n1", p + "n2")
    norm = lambda f, x, g: f(x, g, EPS) if f is rms_norm else f(x, g)
    x = x + mixer(norm(n1, x, w[a]))
    return x + ff(norm(n2, x, w[b]))


def plain_ends(w, tokens):
    x = 3.0 * w["emb"][np.array(tokens)]
    x = _prenorm(x, w, "l0.", lambda h: _attention(h, w, "l0.attn."), lambda h: _dense(h, w, "l0.mlp."))

    def latent(h):
        c = linear(h, w["l1.mix.c.weight"])
        return linear(np.cumsum(c, 0) / np.arange(1, len(c) + 1)[:, None], w["l1.mix.o.weight"])

    x = _prenorm(x, w, "l1.", latent, lambda h: _dense(h, w, "l1.mlp."))
    x = _prenorm(x, w, "l2.", lambda h: _attention(h, w, "l2.attn."), lambda h: _dense(h, w, "l2.mlp."))
    return 2.0 * np.tanh(linear(rms_norm(x, w["final"], EPS), w["head.weight"], w["head.bias"]) / 2.0)


def plain_kinds(w, tokens):
    x = w["emb"][np.array(tokens)]
    x = _prenorm(x, w, "l0.", lambda h: _attention(h, w, "l0.attn."), lambda h: _dense(h, w, "l0.mlp."))
    x = _prenorm(x, w, "l1.", lambda h: _attention(h, w, "l1.attn."), lambda h: _dense(h, w, "l1.mlp."), _centered, _centered)
    x = _prenorm(x, w, "l2.", lambda h: _attention(h, w, "l2.attn."), lambda h: linear(linear(h, w["l2.ffn.w1"]), w["l2.ffn.w2"]))
    xn = rms_norm(x, w["l3.n1"], EPS)
    x = x + _attention(xn, w, "l3.attn.") + _dense(xn, w, "l3.mlp.")
    return linear(_centered(x, w["final"]), w["head"])


def plain_shared(w, tokens):
    x = w["emb"][np.array(tokens)]
    for p in ("l0.", "l1."):
        x = _prenorm(x, w, p, lambda h: _attention(h, w, p + "attn."), lambda h: _dense(h, w, p + "mlp."), names=("shared.n1", "shared.n2"))
    return linear(rms_norm(x, w["final"], EPS), w["head"])


def _make(arch, dtype, seed, graphs=True):
    """(runner, float64 weights as the engine holds them) of a toy architecture with random weights."""
    import torch

    from machserve_b200 import ModelRunner
    from machserve_b200.config import config_from_json
    from machserve_b200.parts import DecoderModel
    from machserve_b200.weights import random_tensors

    cfg = config_from_json({"architectures": [arch]})
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = random_tensors(DecoderModel(cfg.model_spec()).tensors(), seed, tdt, weight_std=0.12, bias_std=0.1, norm_std=0.1)
    w = {n: t.float().numpy().astype(np.float64) for n, t in tensors.items()}
    runner = ModelRunner(cfg, tensors, dtype=dtype, page_size=8, num_pages=24, max_requests=4, max_step_tokens=64,
                         max_seq_len=128, use_graphs=graphs)
    return runner, w


def _cuttings(runner, plain, w, tol, what, lengths=(37, 21)):
    from machserve_b200.engine.replay import replay

    a, b = random_tokens(VOCAB, lengths[0], 1), random_tokens(VOCAB, lengths[1], 2)
    want = {"a": plain(w, a), "b": plain(w, b)}
    for steps in (trace_whole({"a": a, "b": b}), trace_tail_decode("a", a, 20), trace_portions("b", b, [5, 2, 9, 3]),
                  trace_tail_decode("b", b, len(b) - 1)):
        got = collect_rows(steps, replay(runner, steps))
        for rid in got:
            assert_close(got[rid], want[rid], tol, f"{what} {rid}")
        runner.cache.check()
        assert not runner.cache.requests


@pytest.fixture()
def toy_kinds():
    unregister = _register()
    yield
    unregister()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_ends_and_a_cache_plane_of_another_width(toy_kinds, dtype):
    runner, w = _make("ToyEndsForCausalLM", dtype, seed=7)
    needs = runner.model.cache_needs()
    assert [n.elements_per_token() for n in needs] == [2 * KV * HD, LATENT, 2 * KV * HD]
    assert len(runner.cache.groups) == 2 and set(runner.pages[1]) == {"c"} and runner.pages[1]["c"].shape[2:] == (1, 8, LATENT)
    assert not runner.use_graphs  # the latent mixer loops on the host
    assert set(runner._planners) == {"attention", ("toy_latent", 5)}
    _cuttings(runner, plain_ends, w, F32_TOL if dtype == "float32" else BF16_TOL, f"ends {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_and_block_of_other_kinds_after_built_in_layers(toy_kinds, dtype):
    """In bfloat16 with up to 16 rows the built-in layers leave row statistics; a norm or a block of another kind that
    follows must see a delta or None (the toy parts assert it) and the logits must still be right."""
    runner, w = _make("ToyKindsForCausalLM", dtype, seed=8)
    assert runner.use_graphs
    blocks = runner.model.blocks
    if dtype == "bfloat16":
        assert blocks[0].fuse_mixer and blocks[0].fuse_feed_forward
        assert not blocks[1].fuse_mixer and not blocks[1].fuse_feed_forward  # its norms fold into nothing
        assert blocks[2].fuse_mixer and blocks[2].fuse_feed_forward  # the toy feed-forward joined the protocol
    _cuttings(runner, plain_kinds, w, F32_TOL if dtype == "float32" else BF16_TOL, f"kinds {dtype}")


def test_a_feed_forward_that_joins_the_few_row_path_costs_two_launches(toy_kinds):
    """A decoding step of the third layer (built-in attention, toy feed-forward, both fused): QKV product, attention,
    output product, and the toy part's two products: five launches, as for the built-in feed-forward."""
    import torch

    from machserve_b200 import StepEntry, ops

    runner, _ = _make("ToyKindsForCausalLM", "bfloat16", seed=8, graphs=False)
    runner.step([StepEntry("a", random_tokens(VOCAB, 9, 3), [])])
    entries = [StepEntry("a", [5], [0])]
    runner.reserve(entries)
    runner._upload_tables()
    ctx = runner._stage(entries)
    residual = torch.randn((1, H), device="cuda")
    pending = runner.model.blocks[0].forward(ctx, residual, None, runner.bindings[0])
    for layer, want in ((0, 5), (2, 5)):
        before = ops.launches()
        pending = runner.model.blocks[layer].forward(ctx, residual, pending, runner.bindings[layer])
        assert ops.launches() - before == want, f"layer {layer}: {ops.launches() - before} launches"
    runner.release("a")


def test_two_layers_share_one_norm_tensor(toy_kinds):
    """Each norm holds a copy of its own: folding one layer's norm into its matrices leaves the other's alone."""
    for dtype in ("float32", "bfloat16"):
        runner, w = _make("ToySharedForCausalLM", dtype, seed=9)
        if dtype == "bfloat16":
            assert all(b.fuse_mixer and b.fuse_feed_forward for b in runner.model.blocks)
        _cuttings(runner, plain_shared, w, F32_TOL if dtype == "float32" else BF16_TOL, f"shared {dtype}")
