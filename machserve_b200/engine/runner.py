"""The step function: one batch of (request, its next tokens) through the model, from the cache.

`ModelRunner` owns the device side of one model: its weights, the page arrays of
every cache group, the per-request state arrays, the per-request block tables
on the device, and the scratch memory.  `step(entries)` runs exactly the tokens
it is given as one batch (portions of prompts beside single decoded tokens, cut
anywhere) and returns float32 logits for the rows that are wanted.

The reference's counterpart is `BatchedModel::decode_step_explicit`
(crates/mach-model/src/batched.rs:4705-4834 of gqf2008/machserve): rows of
(token, position, slot), device block tables that change only when a request's
pages change (`set_block_table`, :889-934), bounds checked on the host before
anything is uploaded (:4716-4737).  Unlike it, logits are computed for the wanted
rows only and sampling is a separate call.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache import CacheManager, OutOfPages
from ..config import ModelConfig, load_config
from ..parts import DecoderModel, FixedState, PagedBinding, PagedKV, Runtime, StateBinding, StepContext, Workspace
from ..weights import load_weights, random_tensors, random_tensors_on_device

_DTYPES = {
    "bfloat16": torch.bfloat16,
    "bf16": torch.bfloat16,
    "float32": torch.float32,
    "f32": torch.float32,
    "fp32": torch.float32,
}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not supported (bfloat16 or float32)")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype '{dtype}' is not supported (bfloat16 or float32)") from None


@dataclass
class StepEntry:
    """A request's next tokens in one step, and the places among them whose logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    # a single token that the host does not know yet: row of the preceding step's sampled tokens (on the device)
    # that holds it; `tokens` then carries any valid id in its place
    from_sampled: Optional[int] = None


class StepError(ValueError):
    """The step as given cannot run (unknown token id, too many tokens, context too long)."""


class ModelRunner:
    def __init__(
        self,
        config: ModelConfig,
        tensors: Dict[str, torch.Tensor],
        dtype=torch.bfloat16,
        page_size: int = 64,
        num_pages: int = 256,
        max_requests: int = 64,
        max_step_tokens: int = 2048,
        max_seq_len: Optional[int] = None,
        device: str = "cuda:0",
        use_graphs: bool = True,
    ):
        if not torch.cuda.is_available():
            raise RuntimeError("machserve_b200 runs on a CUDA device only; none is available")
        self.config = config
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        ops.lib()  # fail now, loudly, if the kernels cannot be built or loaded
        self.spec = config.model_spec()
        self.max_seq_len = int(max_seq_len or min(self.spec.max_positions, page_size * num_pages))
        self.page_size, self.max_requests, self.max_step_tokens = page_size, max_requests, max_step_tokens
        self.rt = Runtime(self.dtype, self.device, Workspace(self.device), self.max_seq_len,
                          torch.cuda.get_device_properties(self.device).multi_processor_count)
        self.model = DecoderModel(self.spec)
        on_device = {n: t.to(self.device) for n, t in tensors.items()}
        self.model.bind(on_device, self.rt)
        del on_device

        self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, max_requests)
        self.max_pages = (self.max_seq_len + page_size - 1) // page_size
        # device side of the cache: pages per group, block tables per group, state per run
        self.pages: List[torch.Tensor] = []
        self.tables: List[torch.Tensor] = []
        for g in self.cache.groups:
            shape = (len(g.runs), 2, g.pool.size, g.need.num_kv_heads, page_size, g.need.head_dim)
            self.pages.append(torch.zeros(shape, dtype=self.dtype, device=self.device))
            self.tables.append(torch.full((max_requests, self.max_pages), -1, dtype=torch.int32, device=self.device))
        self.states: Dict[int, torch.Tensor] = {
            run: torch.zeros((max_requests, *need.shape), dtype=torch.float32, device=self.device)
            for run, need in self.cache.state_runs.items()
        }
        self.bindings = self._make_bindings()
        # staging for one step's index arrays: pinned host buffers in a ring, one device buffer
        self._stage_len = 7 * max_step_tokens + 10 * max_requests + 4 * (max_step_tokens // 64) + 16
        self._pinned = [torch.empty(self._stage_len, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._pinned_events: List[Optional[torch.cuda.Event]] = [None] * len(self._pinned)
        self._turn = 0
        self._device_stage = torch.empty(self._stage_len, dtype=torch.int32, device=self.device)
        self._row_stage = torch.empty((max_requests, self.max_pages), dtype=torch.int32).pin_memory()
        self.steps = 0
        self._sampled: Optional[torch.Tensor] = None
        self.h2d_bytes = 0  # bytes of index arrays and block-table rows copied to the device so far
        # decoding steps are captured once per (padded batch, padded context length) and replayed
        self.use_graphs = use_graphs and self.model.graph_safe()
        self._graphs: Dict[Tuple[int, int], Tuple[torch.cuda.CUDAGraph, torch.Tensor, int]] = {}
        self._shape_graphs: Dict[tuple, Tuple[torch.cuda.CUDAGraph, torch.Tensor, int]] = {}
        self._shape_seen: Dict[tuple, int] = {}

    # ---------------------------------------------------------------- builders

    @classmethod
    def from_model_dir(cls, model_dir, dtype=torch.bfloat16, **kw) -> "ModelRunner":
        config = load_config(model_dir)
        model = DecoderModel(config.model_spec())
        tensors = load_weights(model_dir, model.tensors(), parse_dtype(dtype), "cpu")
        return cls(config, tensors, dtype=dtype, **kw)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int, dtype=torch.bfloat16, on_device: bool = False, **kw) -> "ModelRunner":
        """Random weights in memory.  By default the values are those of `write_random_model` for the same seed
        (made on the host, reproducible anywhere); with `on_device` they are drawn by the device's generator,
        which takes seconds for billions of parameters and is what a benchmark wants."""
        model = DecoderModel(config.model_spec())
        dt = parse_dtype(dtype)
        if on_device:
            device = torch.device(kw.get("device", "cuda:0"))
            return cls(config, random_tensors_on_device(model.tensors(), seed, dt, device), dtype=dt, **kw)
        return cls(config, random_tensors(model.tensors(), seed, dt), dtype=dt, **kw)

    def _make_bindings(self):
        out = []
        for i, run in enumerate(self.spec.run_order):
            owner = i if run.cache_of is None else run.cache_of
            if owner in self.cache.group_of_run:
                g = self.cache.group_of_run[owner]
                j = self.cache.groups[g].runs.index(owner)
                out.append(PagedBinding(g, self.pages[g][j, 0], self.pages[g][j, 1], self.cache.groups[g].need.window))
            elif owner in self.states:
                out.append(StateBinding(self.states[owner]))
            else:
                out.append(None)
        return out

    # -------------------------------------------------------------------- step

    def _check(self, entries: Sequence[StepEntry]) -> None:
        vocab = self.spec.vocab_size
        total = sum(len(e.tokens) for e in entries)
        if total == 0:
            raise StepError("a step without tokens")
        if total > self.max_step_tokens:
            raise StepError(f"{total} tokens in one step, the runner was made for {self.max_step_tokens}")
        if len(entries) > self.max_requests:
            raise StepError(f"{len(entries)} requests in one step, the runner was made for {self.max_requests}")
        seen = set()
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            if e.from_sampled is not None and n != 1:
                raise StepError(f"request {e.request!r}: only a single token can be taken from the sampled tokens")
            if n == 1 and type(e.tokens[0]) is int and 0 <= e.tokens[0] < vocab and (not e.want or list(e.want) == [0]):
                held = self.cache.requests[e.request].num_tokens if e.request in self.cache.requests else 0
                if held + 1 > self.max_seq_len:
                    raise StepError(f"request {e.request!r} would hold {held + 1} tokens, the limit is {self.max_seq_len}")
                continue  # a decoded token: nothing else to check
            ids = np.asarray(e.tokens)
            if ids.ndim != 1 or ids.dtype.kind not in "iu":
                raise StepError(f"request {e.request!r}: tokens must be a flat list of integers")
            if int(ids.min()) < 0 or int(ids.max()) >= vocab:
                bad = int(ids[(ids < 0) | (ids >= vocab)][0])
                raise StepError(f"request {e.request!r}: token id {bad} is outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")
            held = self.cache.num_tokens(e.request) if e.request in self.cache.requests else 0
            if held + n > self.max_seq_len:
                raise StepError(
                    f"request {e.request!r} would hold {held + n} tokens, the limit is {self.max_seq_len}"
                )

    def reserve(self, entries: Sequence[StepEntry]) -> None:
        """Takes slots and pages for a step.  Raises OutOfPages and leaves earlier requests' pages as they were."""
        started = []
        try:
            for e in entries:
                if e.request not in self.cache.requests:
                    self.cache.begin(e.request)
                    started.append(e.request)
                self.cache.reserve(e.request, self.cache.num_tokens(e.request) + len(e.tokens))
        except OutOfPages:
            for r in started:
                self.release(r)
            raise

    def _upload_tables(self) -> None:
        dirty = self.cache.take_dirty()
        if not dirty:
            return
        for g in range(len(self.cache.groups)):
            rows = [r for (r, gg) in dirty if gg == g and r in self.cache.requests]
            if not rows:
                continue
            slots = []
            for i, r in enumerate(rows):
                table = self.cache.block_table(r, g)
                row = self._row_stage[i]
                row.fill_(-1)
                row[: len(table)] = torch.tensor(table, dtype=torch.int32)
                slots.append(self.cache.state_slot(r))
            idx = torch.tensor(slots, dtype=torch.int64, device=self.device)
            self.h2d_bytes += len(rows) * (self.max_pages * 4 + 8)
            self.tables[g].index_copy_(0, idx, self._row_stage[: len(rows)].to(self.device))

    @staticmethod
    def _layout(T: int, S: int, W: int, n_single: int, n_tiles: int, n_big: int = 0):
        """Where each index array of a step lies in the staging buffer: name -> (offset, length)."""
        views, o = {}, 0
        for name, n in (("token_ids", T), ("from_sampled", T), ("positions", T), ("seq_of_token", T), ("slot_of_token", T),
                        ("cu_tokens", S + 1), ("seq_start", S), ("seq_len", S), ("state_slots", S),
                        ("want_rows", W), ("single_rows", n_single), ("tile_row0", n_tiles), ("tile_rows", n_tiles),
                        ("big_tile_row0", n_big), ("big_tile_rows", n_big)):
            views[name] = (o, n)
            o += n
        return views, o

    def _pinned_turn(self):
        turn = self._turn
        self._turn = (turn + 1) % len(self._pinned)
        if self._pinned_events[turn] is not None:
            self._pinned_events[turn].synchronize()
        return turn

    def _send(self, turn: int, length: int, views=None, entries=()) -> None:
        self.h2d_bytes += 4 * length
        self._device_stage[:length].copy_(self._pinned[turn][:length], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._pinned_events[turn] = ev
        if any(e.from_sampled is not None for e in entries):
            if self._sampled is None:
                raise StepError("a token is to be taken from the preceding step's sampled tokens, but none were given")
            (a, n), (b, _) = views["token_ids"], views["from_sampled"]
            ops.take_sampled_tokens(self._device_stage[a : a + n], self._device_stage[b : b + n], self._sampled)

    def _context(self, views, T, S, W, n_single, n_tiles, max_q, max_len, cu=(), start=(), slots=(), n_big=0) -> StepContext:
        dev = self._device_stage
        d = {name: dev[a : a + n] for name, (a, n) in views.items()}
        return StepContext(
            rt=self.rt, num_tokens=T, num_seqs=S, token_ids=d["token_ids"], positions=d["positions"],
            seq_of_token=d["seq_of_token"], slot_of_token=d["slot_of_token"], cu_tokens=d["cu_tokens"],
            seq_start=d["seq_start"], seq_len=d["seq_len"], state_slots=d["state_slots"],
            block_tables={g: self.tables[g] for g in range(len(self.tables))},
            want_rows=d["want_rows"], num_wanted=W, single_rows=d["single_rows"], num_single=n_single,
            tile_row0=d["tile_row0"], tile_rows=d["tile_rows"], num_tiles=n_tiles,
            big_tile_row0=d["big_tile_row0"], big_tile_rows=d["big_tile_rows"], num_big_tiles=n_big,
            host_cu_tokens=[int(x) for x in cu], host_seq_start=[int(x) for x in start],
            host_state_slots=[int(x) for x in slots], max_query_len=max_q, max_seq_len=max_len,
            decode_only=max_q == 1,
        )

    def _stage(self, entries: Sequence[StepEntry]) -> StepContext:
        """Fills one pinned buffer with the step's index arrays and copies it to the device in one transfer."""
        turn = self._pinned_turn()
        host = self._pinned[turn].numpy()
        T = sum(len(e.tokens) for e in entries)
        S = len(entries)
        W = sum(len(e.want) for e in entries)
        n_single = sum(1 for e in entries if len(e.tokens) == 1)
        n_tiles = sum((len(e.tokens) + 63) // 64 for e in entries if len(e.tokens) > 1)
        n_big = sum((len(e.tokens) + 127) // 128 for e in entries if len(e.tokens) > 1)
        views, total = self._layout(T, S, W, n_single, n_tiles, n_big)
        h = {name: host[a : a + n] for name, (a, n) in views.items()}
        big0, bign, bi = h["big_tile_row0"], h["big_tile_rows"], 0
        tok, pos, seq, slot = h["token_ids"], h["positions"], h["seq_of_token"], h["slot_of_token"]
        cu, start, length, slots, want = h["cu_tokens"], h["seq_start"], h["seq_len"], h["state_slots"], h["want_rows"]
        single, tile0, tilen = h["single_rows"], h["tile_row0"], h["tile_rows"]
        si = ti = row = w = 0
        cu[0] = 0
        max_q = max_len = 0
        for i, e in enumerate(entries):
            n = len(e.tokens)
            p0 = self.cache.num_tokens(e.request)
            s = self.cache.state_slot(e.request)
            tok[row : row + n] = e.tokens
            h["from_sampled"][row : row + n] = -1 if e.from_sampled is None else e.from_sampled
            pos[row : row + n] = np.arange(p0, p0 + n, dtype=np.int32)
            seq[row : row + n] = i
            slot[row : row + n] = s
            start[i], length[i], slots[i] = p0, p0 + n, s
            for k in e.want:
                want[w] = row + int(k)
                w += 1
            if n == 1:
                single[si] = row
                si += 1
            else:
                for a in range(0, n, 64):
                    tile0[ti], tilen[ti] = row + a, min(64, n - a)
                    ti += 1
                for a in range(0, n, 128):
                    big0[bi], bign[bi] = row + a, min(128, n - a)
                    bi += 1
            row += n
            cu[i + 1] = row
            max_q, max_len = max(max_q, n), max(max_len, p0 + n)
        self._send(turn, total, views, entries)
        return self._context(views, T, S, W, n_single, n_tiles, max_q, max_len, cu, start, slots, n_big)

    # ------------------------------------------------------- decoding with graphs

    def _graph_shape(self, entries: Sequence[StepEntry]):
        """(padded batch, padded context length) if the step is plain decoding, else None."""
        if not self.use_graphs or any(len(e.tokens) != 1 or list(e.want) != [0] for e in entries):
            return None
        b = 1
        while b < len(entries):
            b *= 2
        longest = max(self.cache.num_tokens(e.request) for e in entries) + 1
        return b, -(-longest // 512) * 512

    def _stage_decode(self, entries: Sequence[StepEntry], b: int):
        """The staging of a decoding step padded to `b` rows: padding rows belong to no request."""
        turn = self._pinned_turn()
        host = self._pinned[turn].numpy()
        s = len(entries)
        views, total = self._layout(b, b, b, b, 0)
        h = {name: host[a : a + n] for name, (a, n) in views.items()}
        p0 = [self.cache.num_tokens(e.request) for e in entries]
        sl = [self.cache.state_slot(e.request) for e in entries]
        for name, vals, pad in (("token_ids", [e.tokens[0] for e in entries], 0),
                                ("from_sampled", [-1 if e.from_sampled is None else e.from_sampled for e in entries], -1),
                                ("positions", p0, 0),
                                ("seq_of_token", range(s), -1), ("slot_of_token", sl, -1), ("seq_start", p0, 0),
                                ("seq_len", [p + 1 for p in p0], 0), ("state_slots", sl, 0)):
            h[name][:s] = vals
            h[name][s:] = pad
        h["cu_tokens"][:] = np.arange(b + 1, dtype=np.int32)
        h["want_rows"][:] = np.arange(b, dtype=np.int32)
        h["single_rows"][:] = np.arange(b, dtype=np.int32)
        self._send(turn, total, views, entries)
        return views

    def _decode_with_graph(self, entries: Sequence[StepEntry], b: int, length: int) -> torch.Tensor:
        views = self._stage_decode(entries, b)
        key = (b, length)
        if key not in self._graphs:
            ctx = self._context(views, b, b, b, b, 0, 1, length)
            self.model.forward(ctx, self.bindings)  # sizes the scratch memory and loads every kernel
            torch.cuda.current_stream().synchronize()
            before = ops.launches()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx, self.bindings)
            self._graphs[key] = (graph, logits, ops.launches() - before)
        graph, logits, launches = self._graphs[key]
        graph.replay()
        ops.count_launches(launches)
        return logits[: len(entries)]

    def step(self, entries: Sequence[StepEntry], reserved: bool = False, sampled: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the entries as one batch.  Returns float32 logits [wanted, vocab] on the device, in the
        order of the entries and of their `want` lists (a view of scratch memory: valid until the next step).
        `sampled`: the int32 device tensor that entries with `from_sampled` take their token from."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._sampled = sampled
        self._check(entries)
        if not reserved:
            self.reserve(entries)
        self._upload_tables()
        fresh = self.cache.take_fresh_slots()
        if fresh and self.states:
            idx = torch.tensor(fresh, dtype=torch.int64, device=self.device)
            for st in self.states.values():
                st.index_fill_(0, idx, 0.0)
        shape = self._graph_shape(entries)
        if shape is not None:
            logits = self._decode_with_graph(entries, *shape)
        else:
            logits = self._step_general(entries)
        for e in entries:
            self.cache.commit(e.request, self.cache.num_tokens(e.request) + len(e.tokens))
        self.steps += 1
        return logits

    MAX_SHAPE_GRAPHS = 24

    def _step_general(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A step of any shape.  A shape that comes a second time (the same numbers of rows, sequences, wanted rows,
        single rows and tiles: a server's steady portions, a benchmark's prompt) is captured in a CUDA graph and
        replayed from then on: the index arrays lie at the same places of the staging buffer, only their
        contents change."""
        ctx = self._stage(entries)
        if not self.use_graphs:
            return self.model.forward(ctx, self.bindings)
        key = (ctx.num_tokens, ctx.num_seqs, ctx.num_wanted, ctx.num_single, ctx.num_tiles, ctx.num_big_tiles,
               -(-ctx.max_seq_len // 512) if ctx.num_single else 0)
        hit = self._shape_graphs.get(key)
        if hit is not None:
            graph, logits, launches = hit
            graph.replay()
            ops.count_launches(launches)
            return logits
        seen = self._shape_seen.get(key, 0)
        self._shape_seen[key] = seen + 1
        if seen == 0 or len(self._shape_graphs) >= self.MAX_SHAPE_GRAPHS:
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            return self.model.forward(ctx, self.bindings)
        # second time: the scratch memory has its size and every kernel has been loaded by the first
        before = ops.launches()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx, self.bindings)
        self._shape_graphs[key] = (graph, logits, ops.launches() - before)
        graph.replay()
        ops.count_launches(ops.launches() - before)
        return logits

    def check_device_status(self) -> None:
        """Raises if a tensor-core kernel gave up one of its bounded waits since the last check (synchronizes)."""
        gemm, attention = ops.tc_status_codes()
        if gemm or attention:
            raise RuntimeError(f"a tcgen05 kernel gave up a wait (product code {gemm}, attention code {attention}); "
                               "the results of recent steps are not valid")

    def release(self, request: Hashable) -> None:
        """The request is finished: its pages and its slot go back."""
        if request in self.cache.requests:
            self.cache.release(request)

    def num_tokens(self, request: Hashable) -> int:
        return self.cache.num_tokens(request) if request in self.cache.requests else 0

    def memory_plan(self) -> Dict[str, int]:
        weights = sum(t.numel() * t.element_size() for t in _unique_tensors(self.model))
        pages = sum(p.numel() * p.element_size() for p in self.pages)
        return {"weights_bytes": weights, "cache_bytes": pages, "workspace_bytes": self.rt.workspace.nbytes()}


def _unique_tensors(model):
    seen, out = set(), []
    parts = [model.embedding, *[p for b in model.blocks for p in b.parts()], model.final_norm, model.head]
    for part in parts:
        for v in vars(part).values():
            if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                seen.add(v.data_ptr())
                out.append(v)
    return out
