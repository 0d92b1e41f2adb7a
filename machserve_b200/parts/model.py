"""A decoder built from a `ModelSpec`: embedding, blocks in their run order, final norm, head.

This is the only model class.  Which parts it holds, with which sizes, and in
which order the layers run is all in the spec; an architecture is a
configuration that produces a spec.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..config.spec import LayerSpec, ModelSpec
from ..weights.loader import TensorDecl
from .base import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, Block, CacheNeed, Part, Runtime, as_delta


def build_block(layer: LayerSpec) -> Block:
    cls = BLOCKS.items.get(layer.block)
    if cls is None:
        raise KeyError(f"no block of kind '{layer.block}' is registered; known: {', '.join(sorted(BLOCKS.items))}")
    return cls(
        layer,
        MIXERS.build(layer.mixer),
        FEED_FORWARDS.build(layer.feed_forward),
        NORMS.build(layer.mixer_norm),
        NORMS.build(layer.feed_forward_norm),
    )


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = EMBEDDINGS.build(spec.embedding)
        self.blocks: List[Block] = [build_block(l) for l in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.head = HEADS.build(spec.head)
        self.rt: Optional[Runtime] = None

    # -- what the model reads and what it needs of the cache ------------------

    def tensors(self) -> List[TensorDecl]:
        out, seen = [], {}
        for part in self.parts():
            for d in part.tensors():
                prev = seen.get(d.name)
                if prev is None:
                    seen[d.name] = d
                    out.append(d)
                elif tuple(prev.shape) != tuple(d.shape):
                    raise ValueError(f"tensor '{d.name}' is declared with shapes {prev.shape} and {d.shape}")
                elif d.required and not prev.required:
                    out[out.index(prev)] = seen[d.name] = d
        return out

    def parts(self) -> List[Part]:
        return [self.embedding, *[p for b in self.blocks for p in b.parts()], self.final_norm, self.head]

    def cache_needs(self) -> List[CacheNeed]:
        """For every entry of the run order: the cache its run owns, or None if it owns none."""
        needs = []
        for run in self.spec.run_order:
            need = self.blocks[run.layer].mixer.cache_need()
            if run.cache_of is not None:
                src = self.blocks[self.spec.run_order[run.cache_of].layer].mixer.cache_need()
                if src != need:
                    raise ValueError(
                        f"run of layer {run.layer} reads the cache of layer {self.spec.run_order[run.cache_of].layer}, "
                        f"but they need different caches: {need} and {src}"
                    )
                need = None
            needs.append(need)
        return needs

    def graph_safe(self) -> bool:
        """Whether a decoding step of this model may be captured in a CUDA graph: every part says so."""
        return all(p.graph_safe for p in self.parts()) and all(getattr(b, "graph_safe", False) for b in self.blocks)

    # -- weights ----------------------------------------------------------------

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.embedding.bind(tensors, rt)
        for b in self.blocks:
            b.bind(tensors, rt)
        self.final_norm.bind(tensors, rt)
        self.head.bind(tensors, rt, self.embedding)

    # -- one step ---------------------------------------------------------------

    def forward(self, ctx, caches: Sequence, tap=None) -> torch.Tensor:
        """Runs the T token rows of `ctx` through the run order and returns float32 logits
        [num_wanted, vocab] for `ctx.want_rows`.  `caches[i]` is the cache binding of run i
        (its own, or the one it reads).  `tap(i, hidden)`, if given, is called after every run with a
        copy of the float32 hidden rows [T, hidden] as they stand after it (and with i = -1 after the
        embedding): what the reference's `set_layer_dump` writes to files
        (crates/mach-model/src/batched.rs:3051-3088 of gqf2008/machserve), for finding the first layer at which two
        implementations part."""
        rt, spec = self.rt, self.spec
        ws = rt.workspace
        t = ctx.token_ids.shape[0]
        residual = ws.get("model.residual", (t, spec.hidden_size), torch.float32)
        self.embedding.forward(ctx, residual)
        if tap is not None:
            tap(-1, residual.clone())
        pending = None
        for i, run in enumerate(spec.run_order):
            block = self.blocks[run.layer]
            if not block.accepts_row_stats:
                pending = as_delta(pending)  # a block of another kind sees a delta or None, as every norm does
            pending = block.forward(ctx, residual, pending, caches[i], run.cache_of is None)
            if tap is not None:  # the delta a block hands on is part of the hidden rows after it
                delta = as_delta(pending)
                tap(i, residual.clone() if delta is None else residual + delta[: residual.shape[0]].float())
        w = ctx.want_rows.shape[0]
        final = ws.get("model.final", (w, spec.hidden_size), rt.dtype)
        self.final_norm.forward(residual, as_delta(pending), final, rows=ctx.want_rows)
        logits = ws.get("model.logits", (w, spec.vocab_size), torch.float32)
        return self.head.forward(ctx, final, logits)


def declared_tensors(spec: ModelSpec) -> List[TensorDecl]:
    return DecoderModel(spec).tensors()
