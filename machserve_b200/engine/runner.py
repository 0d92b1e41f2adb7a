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
from ..parts import DecoderModel, FixedState, PagedBinding, Runtime, StateBinding, StepContext, Workspace
from ..parts.base import StepShape, Work
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


SCRATCH_MARGIN_BYTES = 256 << 20  # for scratch memory, the library's workspace and the kernels themselves


def estimate_device_bytes(model: DecoderModel, dtype: torch.dtype, page_size: int, num_pages: int, max_requests: int,
                          max_seq_len: int) -> Dict[str, int]:
    """What a runner of this model will hold on the device, from the parts' declarations alone: every tensor once
    (matrices in the runtime's dtype, vectors in float32), the pages of every cache group, the state arrays, the
    block tables, and a margin of 256 MiB (the reference estimates the same before it allocates,
    crates/mach-server/src/startup.rs:344-419 of gqf2008/machserve)."""
    elt = 4 if dtype == torch.float32 else 2
    weights = 0
    for d in model.tensors():
        n = 1
        for s in d.shape:
            n *= int(s)
        if d.random or d.required:  # a tied head's own tensor is absent and costs nothing
            weights += n * (4 if d.init == "table" or len(d.shape) < 2 else elt)
    cache = CacheManager(model.cache_needs(), page_size, num_pages, max_requests)
    pages = sum(len(g.runs) * g.pool.size * page_size * g.need.elements_per_token() * elt for g in cache.groups)
    states = 0
    for need in cache.state_runs.values():
        n = max_requests * 4
        for s in need.shape:
            n *= int(s)
        states += n
    tables = len(cache.groups) * max_requests * (-(-max_seq_len // page_size)) * 4
    total = weights + pages + states + tables + SCRATCH_MARGIN_BYTES
    return {"weights_bytes": weights, "cache_bytes": pages, "state_bytes": states, "table_bytes": tables,
            "margin_bytes": SCRATCH_MARGIN_BYTES, "total_bytes": total}


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
        # before anything is allocated: does it fit?  (weights that are on the device already are not needed twice)
        plan = estimate_device_bytes(self.model, self.dtype, page_size, num_pages, max_requests, self.max_seq_len)
        resident = sum(t.numel() * t.element_size() for t in tensors.values() if t.is_cuda)
        free, total = torch.cuda.mem_get_info(self.device)
        if plan["total_bytes"] - min(resident, plan["weights_bytes"]) > free:
            gib = lambda b: f"{b / 2**30:.2f} GiB"
            raise RuntimeError(
                f"the model does not fit on {self.device}: weights {gib(plan['weights_bytes'])} + cache {gib(plan['cache_bytes'])} "
                f"({num_pages} pages of {page_size} tokens) + states {gib(plan['state_bytes'])} + margin {gib(plan['margin_bytes'])} "
                f"= {gib(plan['total_bytes'])}, of which {gib(resident)} are on the device already; {gib(free)} of {gib(total)} are free. "
                "Use fewer pages (num_pages), a smaller capacity or a shorter max_seq.")
        on_device = {n: t.to(self.device) for n, t in tensors.items()}
        self.model.bind(on_device, self.rt)
        del on_device

        self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, max_requests)
        self.max_pages = (self.max_seq_len + page_size - 1) // page_size
        # device side of the cache: pages per group, block tables per group, state per run
        # (pages[group][plane] : [runs, num_pages, heads, page_size, width])
        self.pages: List[Dict[str, torch.Tensor]] = []
        self.tables: List[torch.Tensor] = []
        for g in self.cache.groups:
            self.pages.append({
                pl.name: torch.zeros((len(g.runs), g.pool.size, pl.heads, page_size, pl.width), dtype=self.dtype, device=self.device)
                for pl in g.need.planes
            })
            self.tables.append(torch.full((max_requests, self.max_pages), -1, dtype=torch.int32, device=self.device))
        self.states: Dict[int, torch.Tensor] = {
            run: torch.zeros((max_requests, *need.shape), dtype=torch.float32, device=self.device)
            for run, need in self.cache.state_runs.items()
        }
        self.bindings = self._make_bindings()
        # the parts that want work lists of their own staged with a step (one per key)
        self._planners: Dict[Hashable, object] = {}
        for part in self.model.parts():
            key = part.plan_key()
            if key is not None and key not in self._planners:
                self._planners[key] = part
        # staging for one step's index arrays: pinned host buffers in a ring, one device buffer.  A decoding step
        # is padded to a power of two of rows, which may exceed max_requests.
        pad = 1
        while pad < max_requests:
            pad *= 2
        # (a step of any shape that is to be replayed from a graph is padded to a multiple of ROW_BUCKET rows and of
        # SEQ_BUCKET sequences)
        rows = max(-(-max_step_tokens // self.ROW_BUCKET) * self.ROW_BUCKET, pad)
        seqs = max(pad, 4 * max_requests + self.SEQ_BUCKET)
        self._stage_len = 6 * rows + 4 * seqs + 1 + sum(p.plan_words(rows, seqs) for p in self._planners.values()) + 16
        self._pinned = [torch.empty(self._stage_len, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._pinned_events: List[Optional[torch.cuda.Event]] = [None] * len(self._pinned)
        self._turn = 0
        self._device_stage = torch.empty(self._stage_len, dtype=torch.int32, device=self.device)
        # changed block-table rows go the same way: per group a region of slots and rows in a pinned ring
        self._row_words = 1 + self.max_pages
        region = max_requests * self._row_words
        self._row_pinned = [torch.empty(max(1, len(self.cache.groups)) * region, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._row_events: List[Optional[torch.cuda.Event]] = [None] * len(self._row_pinned)
        self._row_turn = 0
        self._row_device = torch.empty(max(1, len(self.cache.groups)) * region, dtype=torch.int32, device=self.device)
        self.steps = 0
        self._sampled: Optional[torch.Tensor] = None
        self.h2d_bytes = 0  # bytes of index arrays and block-table rows copied to the device so far
        # decoding steps are captured once per (padded batch, padded context length) and replayed
        self.use_graphs = use_graphs and self.model.graph_safe()
        self._graphs: Dict[Tuple[int, int], Tuple[torch.cuda.CUDAGraph, torch.Tensor, int]] = {}
        self._shape_graphs: Dict[tuple, Tuple[torch.cuda.CUDAGraph, torch.Tensor, int]] = {}
        self._shape_seen: Dict[tuple, int] = {}
        self._decode_plan_cache: Dict[Tuple[int, int], tuple] = {}
        self._capture_stream: Optional[torch.cuda.Stream] = None

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
                out.append(PagedBinding(g, {name: arr[j] for name, arr in self.pages[g].items()}, self.cache.groups[g].need.window))
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
        """Block-table rows that changed go to the device: staged in pinned memory (a ring guarded by events, so the
        host never waits for the device here), copied without blocking, and scattered to their slots."""
        dirty = self.cache.take_dirty()
        if not dirty:
            return
        by_group: Dict[int, list] = {}
        for (r, g) in dirty:
            if r in self.cache.requests:
                by_group.setdefault(g, []).append(r)
        if not by_group:
            return
        turn = self._row_turn
        self._row_turn = (turn + 1) % len(self._row_pinned)
        if self._row_events[turn] is not None:
            self._row_events[turn].synchronize()
        host = self._row_pinned[turn].numpy()
        words, region = self._row_words, self.max_requests * self._row_words
        for g, rows in by_group.items():
            n = len(rows)  # the region of group g: n slots, then n rows
            at = g * region
            slots = host[at : at + n]
            rec = host[at + n : at + n * words].reshape(n, self.max_pages)
            rec[:] = -1
            for i, r in enumerate(rows):
                table = self.cache.block_table(r, g)
                slots[i] = self.cache.state_slot(r)
                rec[i, : len(table)] = table
            dev = self._row_device[at : at + n * words]
            dev.copy_(self._row_pinned[turn][at : at + n * words], non_blocking=True)
            self.tables[g].index_copy_(0, dev[:n].long(), dev[n:].view(n, self.max_pages))
            self.h2d_bytes += 4 * n * words
        ev = torch.cuda.Event()
        ev.record()
        self._row_events[turn] = ev

    @staticmethod
    def _layout(T: int, S: int, W: int, plan_sizes=()):
        """Where each index array of a step lies in the staging buffer: name -> (offset, length).  The parts'
        work lists follow the step's own arrays under the names (key, list name)."""
        views, o = {}, 0
        for name, n in (("token_ids", T), ("from_sampled", T), ("positions", T), ("seq_of_token", T), ("slot_of_token", T),
                        ("cu_tokens", S + 1), ("seq_start", S), ("seq_len", S), ("state_slots", S),
                        ("want_rows", W), *plan_sizes):
            views[name] = (o, n)
            o += n
        return views, o

    def _plans(self, shape: StepShape):
        """Every planner's lists for this step: [(key, WorkPlan)], and their lengths as _layout wants them."""
        plans = [(key, part.plan(shape)) for key, part in self._planners.items()]
        sizes = [((key, name), len(lst)) for key, plan in plans for name, lst in plan.lists.items()]
        return plans, sizes

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

    def _context(self, views, T, S, W, plans, max_q, max_len, cu=(), start=(), slots=()) -> StepContext:
        dev = self._device_stage
        d = {name: dev[a : a + n] for name, (a, n) in views.items()}
        work = {
            key: Work({name: d[(key, name)] for name in plan.lists}, {name: len(lst) for name, lst in plan.lists.items()},
                      tuple(plan.shape))
            for key, plan in plans
        }
        return StepContext(
            rt=self.rt, num_tokens=T, num_seqs=S, token_ids=d["token_ids"], positions=d["positions"],
            seq_of_token=d["seq_of_token"], slot_of_token=d["slot_of_token"], cu_tokens=d["cu_tokens"],
            seq_start=d["seq_start"], seq_len=d["seq_len"], state_slots=d["state_slots"],
            block_tables={g: self.tables[g] for g in range(len(self.tables))},
            want_rows=d["want_rows"], num_wanted=W, work=work,
            host_cu_tokens=[int(x) for x in cu], host_seq_start=[int(x) for x in start],
            host_state_slots=[int(x) for x in slots], max_query_len=max_q, max_seq_len=max_len,
            decode_only=max_q == 1,
        )

    ROW_BUCKET, SEQ_BUCKET, WANT_BUCKET = 64, 16, 16

    @classmethod
    def padded_sizes(cls, rows: int, seqs: int, wanted: int) -> Tuple[int, int, int]:
        """The sizes a step of any shape is padded to when it is to share a captured graph: rows to 16 (the few-row
        kernels' limit), 32 or a multiple of ROW_BUCKET; sequences and wanted rows to SEQ_BUCKET and WANT_BUCKET times
        a power of four (16, 64, 256, ...: what is padded there costs next to nothing, and every class less is a
        graph less), wanted rows never to more than the rows."""
        def coarse(n: int, unit: int) -> int:
            c = unit
            while c < n:
                c *= 4
            return c

        rows_p = 16 if rows <= 16 else 32 if rows <= 32 else -(-rows // cls.ROW_BUCKET) * cls.ROW_BUCKET
        seqs_p = coarse(seqs, cls.SEQ_BUCKET)
        wanted_p = min(coarse(wanted, cls.WANT_BUCKET), rows_p) if wanted else 0
        return rows_p, seqs_p, wanted_p

    def _stage(self, entries: Sequence[StepEntry], bucketed: bool = False) -> StepContext:
        """Fills one pinned buffer with the step's index arrays and copies it to the device in one transfer.
        `bucketed`: the step is padded to 16, 32 or a multiple of ROW_BUCKET rows by rows that belong to no sequence and
        no request (no slot, no pages: every kernel passes them over), its sequences to a multiple of SEQ_BUCKET by
        sequences without rows, its wanted rows to WANT_BUCKET or a power of two by repeats of the last one, and the
        parts pad their lists: steps of like size then have the same lengths everywhere and can share a captured graph."""
        turn = self._pinned_turn()
        host = self._pinned[turn].numpy()
        counts = [len(e.tokens) for e in entries]
        starts = [self.cache.num_tokens(e.request) for e in entries]
        T, S = sum(counts), len(entries)
        W = sum(len(e.want) for e in entries)
        row0, row = [], 0
        for n in counts:
            row0.append(row)
            row += n
        Tp, Sp, Wp = self.padded_sizes(T, S, W) if bucketed else (T, S, W)
        extra, empty = Tp - T, Sp - S
        shape = StepShape(Tp, Sp, row0 + [T] * empty, counts + [0] * empty, starts + [0] * empty, bucketed)
        plans, plan_sizes = self._plans(shape)
        views, total = self._layout(Tp, Sp, Wp, plan_sizes)
        h = {name: host[a : a + n] for name, (a, n) in views.items()}
        tok, pos, seq, slot = h["token_ids"], h["positions"], h["seq_of_token"], h["slot_of_token"]
        cu, start, length, slots, want = h["cu_tokens"], h["seq_start"], h["seq_len"], h["state_slots"], h["want_rows"]
        w = 0
        cu[0] = 0
        for i, e in enumerate(entries):
            n, p0, row = counts[i], starts[i], row0[i]
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
            cu[i + 1] = row + n
        if extra:  # rows of no sequence
            tok[T:], pos[T:], seq[T:], slot[T:] = 0, 0, -1, -1
            h["from_sampled"][T:] = -1
        if empty:  # sequences of no rows
            start[S:], length[S:], slots[S:] = 0, 0, 0
            cu[S + 1 :] = T
        if Wp > W:
            want[W:] = want[W - 1]
        for key, plan in plans:
            for name, lst in plan.lists.items():
                h[(key, name)][:] = lst
        self._send(turn, total, views, entries)
        max_q = max(counts)
        max_len = max(p + n for p, n in zip(starts, counts))
        return self._context(views, Tp, Sp, Wp, plans, max_q, max_len, cu, start, slots)

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

    def _decode_plans(self, b: int, length: int):
        """The parts' plans for a decoding step of `b` rows (padding included) whose longest context is `length`:
        they depend on nothing else, so they are made once per graph."""
        key = (b, length)
        hit = self._decode_plan_cache.get(key)
        if hit is None:
            plans, sizes = self._plans(StepShape(b, b, list(range(b)), [1] * b, [length - 1] * b))
            arrays = [((k, name), np.asarray(lst, dtype=np.int32)) for k, plan in plans for name, lst in plan.lists.items()]
            hit = self._decode_plan_cache[key] = (plans, sizes, arrays)
        return hit

    def _stage_decode(self, entries: Sequence[StepEntry], b: int, length: int):
        """The staging of a decoding step padded to `b` rows: padding rows belong to no request."""
        turn = self._pinned_turn()
        host = self._pinned[turn].numpy()
        s = len(entries)
        plans, plan_sizes, arrays = self._decode_plans(b, length)
        views, total = self._layout(b, b, b, plan_sizes)
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
        for name, arr in arrays:
            h[name][:] = arr
        self._send(turn, total, views, entries)
        return views, plans

    def _capture(self, forward):
        """Records the launches of `forward()` in a CUDA graph (they do not run).  On a stream of its own, ordered after
        and before the current one; without the pause for the collector and the return of cached memory that
        torch.cuda.graph() makes, which cost tens of milliseconds: the scratch memory has its size by now, and what a
        forward pass allocates beside it is small and stays with the graph."""
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.device)
        main, side = torch.cuda.current_stream(), self._capture_stream
        side.wait_stream(main)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            graph.capture_begin()
            try:
                out = forward()
            finally:
                graph.capture_end()
        main.wait_stream(side)
        return graph, out

    def _decode_with_graph(self, entries: Sequence[StepEntry], b: int, length: int) -> torch.Tensor:
        views, plans = self._stage_decode(entries, b, length)
        key = (b, length)
        if key not in self._graphs:
            ctx = self._context(views, b, b, b, plans, 1, length)
            self.model.forward(ctx, self.bindings)  # sizes the scratch memory and loads every kernel
            torch.cuda.current_stream().synchronize()
            before = ops.launches()
            graph, logits = self._capture(lambda: self.model.forward(ctx, self.bindings))
            self._graphs[key] = (graph, logits, ops.launches() - before)
        graph, logits, launches = self._graphs[key]
        graph.replay()
        ops.count_launches(launches)
        return logits[: len(entries)]

    def step(self, entries: Sequence[StepEntry], reserved: bool = False, sampled: Optional[torch.Tensor] = None,
             tap=None) -> torch.Tensor:
        """Runs the entries as one batch.  Returns float32 logits [wanted, vocab] on the device, in the
        order of the entries and of their `want` lists (a view of scratch memory: valid until the next step).
        `sampled`: the int32 device tensor that entries with `from_sampled` take their token from.
        `tap(i, hidden)`: called after the embedding (i = -1) and after every run of a layer with the float32 hidden
        rows [rows of the step, hidden]; such a step is run plainly, never from a captured graph."""
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
        shape = self._graph_shape(entries) if tap is None else None
        if shape is not None:
            logits = self._decode_with_graph(entries, *shape)
        elif tap is not None:
            logits = self.model.forward(self._stage(entries), self.bindings, tap)
        else:
            logits = self._step_general(entries)
        for e in entries:
            self.cache.commit(e.request, self.cache.num_tokens(e.request) + len(e.tokens))
        self.steps += 1
        return logits

    MAX_SHAPE_GRAPHS = 160
    CAPTURE_AFTER = 1  # a capture costs as much as one or two such steps run plainly: a shape that comes again is captured

    def _step_general(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A step of any shape.  With graphs, the step is padded so that steps of like size (rows up to the same
        multiple of ROW_BUCKET, tiles of portions, contexts of the same class) have the same lengths everywhere; such
        a shape is captured in a CUDA graph when it has come CAPTURE_AFTER times and replayed from then on: the index
        arrays lie at the same places of the staging buffer, only their contents change.  A server's steady mix of
        a portion of a prompt beside decoded tokens, and a benchmark's prompt, come to a few dozen shapes."""
        if not self.use_graphs:
            return self.model.forward(self._stage(entries), self.bindings)
        wanted = sum(len(e.want) for e in entries)
        ctx = self._stage(entries, bucketed=True)
        key = (ctx.num_tokens, ctx.num_seqs, ctx.num_wanted, ctx.max_query_len > 1,
               tuple((k, tuple(w.sizes.values()), w.shape) for k, w in ctx.work.items()))
        hit = self._shape_graphs.get(key)
        if hit is not None:
            graph, logits, launches = hit
            graph.replay()
            ops.count_launches(launches)
            return logits[:wanted]
        seen = self._shape_seen.get(key, 0)
        self._shape_seen[key] = seen + 1
        if seen < self.CAPTURE_AFTER or len(self._shape_graphs) >= self.MAX_SHAPE_GRAPHS:
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            return self.model.forward(ctx, self.bindings)[:wanted]
        # the scratch memory has its size and every kernel has been loaded by the runs before
        before = ops.launches()
        graph, logits = self._capture(lambda: self.model.forward(ctx, self.bindings))
        self._shape_graphs[key] = (graph, logits, ops.launches() - before)
        graph.replay()
        ops.count_launches(ops.launches() - before)
        return logits[:wanted]

    def graph_counts(self) -> Dict[str, int]:
        """How many captured graphs the runner holds: of decoding steps, and of steps of other shapes."""
        return {"decode": len(self._graphs), "shapes": len(self._shape_graphs)}

    def check_device_status(self) -> None:
        """Raises if a tensor-core kernel gave up one of its bounded waits since the last check (synchronizes)."""
        gemm, attention = ops.tc_status_codes()
        if gemm or attention:
            self.rt.workspace.rezero()  # a block that gave up may not have counted itself out
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
        pages = sum(p.numel() * p.element_size() for planes in self.pages for p in planes.values())
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
