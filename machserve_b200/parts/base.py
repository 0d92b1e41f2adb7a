"""The interfaces of a model's parts, and the registries that build a part from its spec.

Five kinds of part make a layer: a mixer (attention here), a feed-forward, a
norm, a position encoding, and the block that arranges them.  Each kind has a
registry from the `kind` string of a `PartSpec` to a class.  A part gets all
its sizes and constants from its spec; none of them knows which model it is in.

What every part does:

* `tensors()` lists the tensors it reads (`TensorDecl`), so that the loader and
  the random-weights mode need no knowledge of the model;
* `bind(tensors, runtime)` takes its device tensors and puts them into the form
  its kernels read;
* `forward(...)` runs it on the tokens of one step.

A mixer also says what it needs of the cache (`cache_need()`): pages of one or more
planes per token (`PagedCache`; keys and values are two equal planes, `PagedKV`; all
tokens or a window of them), a fixed-size state per request (`FixedState`), or nothing.

Two optional protocols let a part join the engine's faster paths without the engine
knowing its class: `plan_key`/`plan` (host work lists staged with the step's index
arrays) and `fuse_norm`/`forward_fused` (the norm in front of a part and the add behind
it done by the part's own kernels).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Hashable, List, Optional, Sequence, Tuple, Type, Union

import torch

from ..config.spec import LayerSpec, PartSpec
from ..weights.loader import TensorDecl


# ----------------------------------------------------------------- cache needs


@dataclass(frozen=True)
class CachePlane:
    """One array of a paged cache: per token `heads` vectors of `width` elements of the runtime's dtype.
    Its pages on the device are [num_pages, heads, page_size, width]."""

    name: str
    heads: int
    width: int

    def elements_per_token(self) -> int:
        return self.heads * self.width


@dataclass(frozen=True)
class PagedCache:
    """What a mixer keeps per token, in pages: one or more planes, for every token or for the last `window`
    tokens.  Runs of layers whose needs are equal share a group of pages and one block table per request."""

    planes: Tuple[CachePlane, ...]
    window: Optional[int] = None

    def elements_per_token(self) -> int:
        return sum(p.elements_per_token() for p in self.planes)


def PagedKV(num_kv_heads: int, head_dim: int, window: Optional[int] = None) -> PagedCache:
    """Keys and values of every token (or of the last `window` tokens): two equal planes, "k" and "v"."""
    return PagedCache((CachePlane("k", num_kv_heads, head_dim), CachePlane("v", num_kv_heads, head_dim)), window)


@dataclass(frozen=True)
class FixedState:
    """A state of fixed shape per request, float32, zero when the request starts."""

    shape: Tuple[int, ...]


CacheNeed = Union[PagedCache, FixedState, None]


# --------------------------------------------------------------------- runtime


class Workspace:
    """Named scratch buffers that are reused from step to step.  A buffer that has to grow is
    replaced, and the old one is kept alive: a captured graph that wrote to it still may."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._retired: List[torch.Tensor] = []
        self._zeroed: set = set()  # buffers whose users rely on finding zeros (and leave zeros behind)
        self._views: Dict[tuple, torch.Tensor] = {}  # (name, dtype, shape) -> the view handed out last time

    def get(self, name: str, shape, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A view of the buffer `name`; with `zero`, the buffer is zero-filled when it is made."""
        shape = tuple(shape)
        view = self._views.get((name, dtype, shape))
        if view is not None:
            return view  # asked for with every launch of every step: the same shape gets the same view
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if buf is not None:
                self._retired.append(buf)  # captured graphs may still point into it
            buf = (torch.zeros if zero else torch.empty)(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            if zero:
                self._zeroed.add(key)
            for k in [k for k in self._views if k[0] == name and k[1] == dtype]:
                del self._views[k]  # views of the buffer that was replaced
        view = buf[:n].view(*shape)
        if len(self._views) < 4096:
            self._views[(name, dtype, shape)] = view
        return view

    def rezero(self) -> None:
        """Zeros again what was handed out as zeros: after a kernel gave up half-way and may have left counters behind."""
        for key in self._zeroed:
            self._bufs[key].zero_()

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in [*self._bufs.values(), *self._retired])


@dataclass
class Runtime:
    """What the parts of one engine share: the compute dtype, the device, and scratch memory.

    `dtype` is torch.bfloat16 (bfloat16 weights, activations and cache; float32
    residual stream, norms, softmax, rotation and logits) or torch.float32
    (everything in true float32).
    """

    dtype: torch.dtype
    device: torch.device
    workspace: Workspace
    max_positions: int
    sm_count: int = 148
    _side: Optional["torch.cuda.Stream"] = None

    @property
    def is_f32(self) -> bool:
        return self.dtype == torch.float32

    def side_stream(self) -> "torch.cuda.Stream":
        """A second stream, for two launches of a part that do not depend on each other.  The part orders it behind
        the current stream before and the current stream behind it after; in a captured step that becomes two
        branches of the graph."""
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side


@dataclass
class RowStats:
    """Stands where a block's pending delta would stand when the delta has already been added to the
    residual by the kernel that made it.  `stats[m][b]` is the sum of squares of row m of the residual
    over its b-th block of 16 columns: what an RMS norm needs to skip its own pass over the row."""

    stats: torch.Tensor
    blocks: int
    copy: Optional[torch.Tensor] = None  # the residual rounded to the runtime's dtype, if its producer left one


def as_delta(pending):
    """What a norm adds to the residual before it normalises: a `RowStats` says that the add has been done."""
    return None if isinstance(pending, RowStats) else pending


# ------------------------------------------------------------------- work plans


@dataclass
class StepShape:
    """The rows of one step as the host knows them: what `Part.plan` makes its work lists from.
    Sequence i brings rows [row0[i], row0[i] + count[i]) at positions start[i], start[i] + 1, ...
    A decoding step that is padded to a fixed size ends with sequences of one row that belong to no request.
    `bucketed`: the step is to be replayed from a graph that is shared by all steps of like size.  It may then end
    with sequences of no rows, and `rows` may count rows behind the last sequence's that belong to no sequence (their
    slot and sequence numbers are -1); a plan should pad its lists with entries that do nothing and give its `shape`
    in coarse classes, so that few different (lengths, shape) come out of the many steps of a serving load."""

    rows: int
    seqs: int
    row0: Sequence[int]
    count: Sequence[int]
    start: Sequence[int]
    bucketed: bool = False


@dataclass
class WorkPlan:
    """Host lists of int32 that a part wants on the device for one step (`lists`, by name), and whatever
    else its launches depend on beyond the lengths of those lists (`shape`, hashable): a step is captured in
    a CUDA graph under the lengths and shapes of its plans."""

    lists: Dict[str, Sequence[int]]
    shape: Tuple = ()


@dataclass
class Work:
    """A staged plan: the lists as device tensors, their lengths, and the plan's shape."""

    lists: Dict[str, torch.Tensor]
    sizes: Dict[str, int]
    shape: Tuple = ()


# ------------------------------------------------------------------ interfaces


class Part:
    # True for parts whose forward only launches kernels on the step's device arrays, so that a decoding
    # step may be captured once in a CUDA graph and replayed.  A part that loops on the host over the
    # step's sequences, or reads host-side lists of the context, leaves this False.
    graph_safe = False

    def __init__(self, spec: PartSpec):
        self.spec = spec

    def tensors(self) -> List[TensorDecl]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt

    # -- work lists (optional) -------------------------------------------------------------------------
    # A part whose kernels want lists made on the host (rows sorted by kind, tiles of rows, chunks of a scan)
    # names a key; parts with equal keys share one plan per step.  The step function calls `plan` once per key,
    # stages the lists with the step's index arrays in one transfer, and hands them on as `ctx.work[key]`.

    def plan_key(self) -> Optional[Hashable]:
        return None

    def plan(self, step: StepShape) -> WorkPlan:
        raise NotImplementedError

    def plan_words(self, max_rows: int, max_seqs: int) -> int:
        """The most int32 words the lists of one step can have, for steps of up to `max_rows` rows in `max_seqs` sequences."""
        return 0

    # -- the norm in front and the add behind, inside the part's own kernels (optional) ----------------------
    # Asked once, when the block is bound: a part that can read the residual's rounded copy and its rows' sums
    # of squares (`RowStats`) instead of normed rows takes what it needs of `norm` (see `Norm.fold_into`) and
    # returns True.  `forward_fused` is then used for steps of up to `fused_rows` rows.

    fused_rows = 0

    def fuse_norm(self, norm: "Norm") -> bool:
        return False

    def forward_fused(self, ctx, residual, pending, norm: "Norm", cache=None, owns_cache: bool = True) -> "RowStats":
        """residual += part(norm(residual + pending)); `pending` is a delta, None, or the `RowStats` of a part
        that has already added its delta.  Returns the `RowStats` of the new residual."""
        raise NotImplementedError


class TokenEmbedding(Part):
    """Token ids to the residual stream: forward(ctx, out) writes the float32 rows out[T, hidden] for `ctx.token_ids`."""

    def forward(self, ctx, out):
        raise NotImplementedError


class Head(Part):
    """The final hidden rows to logits: forward(ctx, x, out) with x [W, hidden] in the runtime's dtype (the final
    norm's output for the wanted rows) writes float32 out[W, vocab].  `bind` is also given the model's embedding
    part, for a head that shares its table."""

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime, embedding: Optional[TokenEmbedding] = None) -> None:
        self.rt = rt

    def forward(self, ctx, x, out):
        raise NotImplementedError


class Norm(Part):
    """y = norm(x).  `forward` takes the float32 residual [T, d] and an optional delta to add first.

    forward(residual, delta, out, rows=None) -> out:
      residual += delta (when delta is given and rows is None), out = norm(residual).
      With `rows` (int32 indices), out[i] = norm(residual[rows[i]] + delta[rows[i]]) and nothing is written back.
    """

    def forward(self, residual, delta, out, rows=None):
        raise NotImplementedError

    def fold_into(self, matrix: torch.Tensor) -> bool:
        """For a part that fuses this norm (`Part.fuse_norm`): if the norm is y = x / rms(x, eps) * g, multiply the
        columns of `matrix` [n, size] by g (in float32, rounded once), keep a weight of one from now on, so that
        every path computes with the same matrix, and return True with `self.eps` set.  Any other norm returns False."""
        return False


class PositionEncoding(Part):
    """How positions enter a mixer.

    A rotary encoding returns from `rotary_table(rt)` a float32 table
    [positions, rotary_dim/2, 2] of (cos, sin), with `rotary_dim` and
    `interleaved` attributes; the attention mixer then applies it inside its own
    kernel.  Any other encoding returns None there and implements
    `apply(ctx, q, k)`, which changes q [T, Hq, hd] and k [T, Hkv, hd] in place.
    """

    rotary_dim: int = 0
    interleaved: bool = False

    def rotary_table(self, rt: Runtime) -> Optional[torch.Tensor]:
        return None

    def apply(self, ctx, q: torch.Tensor, k: Optional[torch.Tensor]) -> None:
        raise NotImplementedError


class Mixer(Part):
    """Mixes information between the tokens of a sequence.

    forward(ctx, x, cache) -> delta: x [T, hidden] is the normed input in the
    runtime's dtype, delta [T, hidden] is what the block adds to the residual.
    `cache` is the `CacheBinding` of this run of the layer (None if the mixer
    needs none).  `owns_cache` is False when this run reads a cache another
    run writes.
    """

    def cache_need(self) -> CacheNeed:
        return None

    def forward(self, ctx, x, cache, owns_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    """forward(ctx, x) -> delta, token by token: x [T, hidden] normed input, delta [T, hidden]."""

    def forward(self, ctx, x):
        raise NotImplementedError


class Block:
    """The arrangement of a layer's parts around the residual stream.

    forward(ctx, residual, pending, cache, owns_cache) -> pending: `residual` is
    the float32 stream [T, hidden]; `pending` is a delta not yet added to it
    (or None); the block returns the delta that the next norm adds.  A block that
    sets `accepts_row_stats` may also be given, and may return, a `RowStats` (the
    delta has been added already); other blocks, and every norm, see None in its place.
    """

    accepts_row_stats = False

    def __init__(self, spec: LayerSpec, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ff_norm: Norm):
        self.spec, self.mixer, self.feed_forward, self.mixer_norm, self.ff_norm = spec, mixer, feed_forward, mixer_norm, ff_norm

    def parts(self) -> List[Part]:
        return [self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        for p in self.parts():
            p.bind(tensors, rt)

    def forward(self, ctx, residual, pending, cache, owns_cache=True):
        raise NotImplementedError


# ------------------------------------------------------------------ registries


class _Registry:
    def __init__(self, what: str):
        self.what = what
        self.items: Dict[str, type] = {}

    def register(self, kind: str) -> Callable[[type], type]:
        def deco(cls):
            self.items[kind] = cls
            return cls

        return deco

    def unregister(self, kind: str) -> None:
        self.items.pop(kind, None)

    def build(self, spec: PartSpec, *args):
        if spec.kind not in self.items:
            raise KeyError(f"no {self.what} of kind '{spec.kind}' is registered; known: {', '.join(sorted(self.items))}")
        return self.items[spec.kind](spec, *args)


EMBEDDINGS = _Registry("embedding")
HEADS = _Registry("head")
MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITION_ENCODINGS = _Registry("position encoding")
BLOCKS = _Registry("block")

register_embedding = EMBEDDINGS.register
register_head = HEADS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_block = BLOCKS.register


def vector_f32(t: torch.Tensor) -> torch.Tensor:
    """Norm weights and biases are read as float32 by every kernel, whatever they were stored as.  Always a
    copy of the part's own: a part may rewrite it (a norm whose weight is folded into a matrix)."""
    return t.to(torch.float32).contiguous().clone()


def matrix(t: torch.Tensor, rt: Runtime) -> torch.Tensor:
    """A matrix in the dtype the runtime multiplies with."""
    return t.to(rt.dtype).contiguous()
