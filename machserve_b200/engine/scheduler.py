"""The scheduler: which requests run in the next step, with how many tokens each.

Host-side decisions only; it talks to the cache manager and never to the GPU.

The reference (`ContinuousModel`, crates/mach-model/src/continuous.rs of
gqf2008/machserve) visits its slots in order with one row budget, so decoding
requests in higher slots stall behind a long prompt in a lower one (:956-1003);
it reserves a request's whole context at admission and has no answer to a full
pool but to refuse the request (:847-883).  Here:

* waiting requests are admitted first come first served while a slot is free
  and the pages of their whole prompt are free;
* every step, each decoding request gets its one token first; then prompts are
  cut into portions under the budget of `prefill_rows` prompt tokens per step
  (the reference's MACH_PREFILL_ROWS), oldest request first;
* pages are taken as positions are written.  When a decoding request needs a
  page and none is free, the youngest running request is preempted: all it holds
  is given back and it waits again at the head of the queue, to be recomputed
  from its prompt plus what it has generated (its RNG state and its output stay,
  so the tokens that follow are the ones it would have produced);
* a request that could not run even alone in an empty pool is refused at `add`.

A step may be planned before the results of the one before it are known
(`schedule`, `schedule`, `update`, `update`, ...): a request then has `pending`
sampled tokens whose values the host has not seen.  They count as part of the
sequence; the step that reads such a token takes it from the sampler's output
on the device.  What depends on a token's value comes one step late: a request
that ends with EOS or a stop sequence may have one more row in flight, whose
result is dropped; an end by length is foreseen and never overrun.

Finishing follows the reference (:1162-1196, :1266-1272): the EOS token is kept
and ends the output; a stop sequence is matched as a suffix of the generated
ids; `max_new` tokens or the context limit end it with reason "length",
EOS and stop sequences with "stop".
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache import CacheManager, OutOfPages
from ..sampling.params import SamplingParams, advance_seed

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass(eq=False)  # a request is itself: membership tests and removals compare identities, not fields
class Sequence_:
    id: int
    prompt: List[int]
    max_new: int
    eos: Optional[int]
    stop_seqs: List[List[int]]
    logit_bias: Dict[int, float]
    params: SamplingParams
    rng_state: int
    status: str = WAITING
    output: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    top_logprobs: List[list] = field(default_factory=list)  # per generated token: [(token, logprob), ...] if asked for
    finish_reason: Optional[str] = None
    computed: int = 0  # tokens whose keys and values are in the cache, by the steps whose results are known
    planned: int = 0   # the same, by every step planned so far
    pending: int = 0   # sampled tokens of planned steps whose values are not known yet
    preemptions: int = 0
    arrival: int = 0

    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def known(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def total(self) -> int:
        return len(self.prompt) + len(self.output) + self.pending


@dataclass
class PlanEntry:
    seq: Sequence_
    start: int  # position of the first token of this portion
    count: int
    samples: bool  # the portion reaches the sequence's last token: its last row is sampled
    generation: int = 0   # the request's count of preemptions when this was planned
    unknown: bool = False  # the (single) token is a pending one: it is taken from the preceding step's samples


@dataclass
class StepPlan:
    entries: List[PlanEntry]
    preempted: List[int]

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class SchedulerError(ValueError):
    pass


class Scheduler:
    def __init__(self, cache: CacheManager, capacity: int, prefill_rows: int, max_seq_len: int):
        if capacity < 1 or prefill_rows < 1:
            raise ValueError("capacity and prefill_rows must be positive")
        self.cache, self.capacity, self.prefill_rows, self.max_seq_len = cache, capacity, prefill_rows, max_seq_len
        self.waiting: Deque[Sequence_] = deque()
        self.running: List[Sequence_] = []  # in order of admission: the last one is the youngest
        self.seqs: Dict[int, Sequence_] = {}
        self._next_id = 1
        self._clock = 0

    # ------------------------------------------------------------------ requests

    def add(
        self,
        prompt: Sequence[int],
        max_new: int,
        eos: Optional[int] = None,
        stop_seqs: Sequence[Sequence[int]] = (),
        logit_bias: Optional[Dict[int, float]] = None,
        params: SamplingParams = SamplingParams(),
    ) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise SchedulerError("empty prompt")
        if len(prompt) > self.max_seq_len:
            raise SchedulerError(f"prompt of {len(prompt)} tokens is longer than the context limit {self.max_seq_len}")
        if max_new < 1:
            raise SchedulerError("max_new must be at least 1")
        params.check()
        # could it run alone in an empty pool?  Its last step writes position total-1.
        longest = min(len(prompt) + max_new, self.max_seq_len)
        for g in self.cache.groups:
            need = -(-longest // self.cache.page_size)
            if g.need.window is not None:
                need = min(need, -(-(g.need.window + min(self.prefill_rows, longest)) // self.cache.page_size) + 1)
            if need > g.pool.size:
                raise SchedulerError(
                    f"a request of {longest} tokens needs {need} pages of cache group {g.index}, the pool has {g.pool.size}"
                )
        sid = self._next_id
        self._next_id += 1
        seed = params.seed if params.seed != 0 else sid
        seq = Sequence_(sid, prompt, max_new, eos, [list(s) for s in stop_seqs if len(s)], dict(logit_bias or {}),
                        params, seed, arrival=self._clock)
        self._clock += 1
        self.seqs[sid] = seq
        self.waiting.append(seq)
        return sid

    def cancel(self, sid: int) -> bool:
        seq = self.seqs.get(sid)
        if seq is None or seq.status == FINISHED:
            return False
        self._finish(seq, "cancelled")
        return True

    def ack(self, sid: int) -> None:
        """Forgets a finished request's output."""
        if sid in self.seqs and self.seqs[sid].status == FINISHED:
            del self.seqs[sid]

    def all_done(self) -> bool:
        return not self.waiting and not self.running

    # ------------------------------------------------------------------ planning

    def _preempt(self, seq: Sequence_, plan_preempted: List[int]) -> None:
        self.cache.release(seq.id)
        self.running.remove(seq)
        seq.status, seq.computed, seq.planned, seq.pending = WAITING, 0, 0, 0
        seq.preemptions += 1  # results of steps still in flight for it are dropped
        self.waiting.appendleft(seq)
        plan_preempted.append(seq.id)

    def schedule(self) -> StepPlan:
        """The next step.  Pages and slots for it are taken here; `update` must follow the step."""
        preempted: List[int] = []
        while True:
            entries = self._schedule_once(preempted)
            if entries or not self.running or any(s.pending for s in self.running):
                # (requests whose rows are all in flight are no deadlock: their results will move them on)
                self._planned(entries)
                return StepPlan(entries, preempted)
            # every running request is a prompt that waits for pages another one holds:
            # the youngest gives way (a request alone always fits, so this ends)
            self._preempt(self.running[-1], preempted)

    def _schedule_once(self, preempted: List[int]) -> List[PlanEntry]:
        entries: List[PlanEntry] = []
        in_plan = set()  # ids of the requests that have an entry
        # 1. one token for every request that is decoding, oldest first; make room by preempting the youngest
        for seq in list(self.running):
            if seq.status != RUNNING or seq.planned < seq.total - 1:
                continue
            if seq.pending > 1:
                continue  # its next token is not even on the device yet: only the preceding step's samples are
            # never plan past an end that can be foreseen: the tokens in flight may already complete the request
            if len(seq.output) + seq.pending >= seq.max_new or (seq.pending and seq.total >= self.max_seq_len):
                continue
            while not self.cache.can_reserve(seq.id, seq.total):
                victim = self.running[-1]
                if victim.id in in_plan:
                    entries[:] = [e for e in entries if e.seq is not victim]
                    in_plan.discard(victim.id)
                self._preempt(victim, preempted)
                if victim is seq:
                    break
            if seq.status == RUNNING:
                self.cache.reserve(seq.id, seq.total)
                entries.append(PlanEntry(seq, seq.total - 1, 1, True, seq.preemptions, seq.pending > 0))
                in_plan.add(seq.id)
        # 2. portions of prompts under the budget: running requests first, then admissions
        budget = self.prefill_rows
        for seq in list(self.running):
            if budget == 0:
                break
            if seq.planned >= seq.known - 1 or seq.id in in_plan:
                continue
            budget -= self._plan_portion(seq, budget, entries)
        while self.waiting and budget > 0 and len(self.running) < self.capacity:
            seq = self.waiting[0]
            if self.cache.slots.num_free == 0:
                break
            self.cache.begin(seq.id)
            # a request is admitted when the pages of all it has to (re)compute are free now
            if not self.cache.can_reserve(seq.id, seq.total):
                self.cache.release(seq.id)
                break
            self.waiting.popleft()
            seq.status = RUNNING
            self.running.append(seq)
            budget -= self._plan_portion(seq, budget, entries)
        return entries

    def _plan_portion(self, seq: Sequence_, budget: int, entries: List[PlanEntry]) -> int:
        count = min(seq.known - seq.planned, budget)
        # shrink the portion to the pages that are free
        while count > 0 and not self.cache.can_reserve(seq.id, seq.planned + count):
            count = min(count - 1, ((seq.planned + count - 1) // self.cache.page_size) * self.cache.page_size - seq.planned)
        if count <= 0:
            return 0
        self.cache.reserve(seq.id, seq.planned + count)
        entries.append(PlanEntry(seq, seq.planned, count, seq.planned + count == seq.known, seq.preemptions))
        return count

    def _planned(self, entries: List[PlanEntry]) -> None:
        """The plan stands: the requests move on to what follows it."""
        for e in entries:
            e.seq.planned = e.start + e.count
            if e.samples:
                e.seq.pending += 1

    # ------------------------------------------------------------------- results

    def update(self, plan: StepPlan, sampled: Sequence[int], logprobs: Sequence[float], tops: Sequence[list] = ()) -> List[Tuple[int, int]]:
        """Takes the step's sampled tokens (one per entry with `samples`, in plan order), their log-probabilities
        and, for requests that asked, the lists of most probable tokens.  Returns the (request id, token) pairs
        generated in this step."""
        out, k = [], 0
        for e in plan.entries:
            seq = e.seq
            if seq.status != RUNNING or e.generation != seq.preemptions:
                k += e.samples  # cancelled, finished or preempted while the step ran: its result is dropped
                continue
            self.cache.commit(seq.id, e.start + e.count)
            seq.computed = e.start + e.count
            if not e.samples:
                continue
            tok, lp = int(sampled[k]), float(logprobs[k])
            if seq.params.top_logprobs:
                seq.top_logprobs.append(list(tops[k]) if k < len(tops) else [])
            k += 1
            seq.pending -= 1
            seq.rng_state = advance_seed(seq.rng_state)
            seq.output.append(tok)
            seq.logprobs.append(lp)
            out.append((seq.id, tok))
            reason = None
            if seq.eos is not None and tok == seq.eos:
                reason = "stop"
            elif any(len(s) <= len(seq.output) and seq.output[-len(s):] == s for s in seq.stop_seqs):
                reason = "stop"
            elif len(seq.output) >= seq.max_new or seq.known >= self.max_seq_len:
                reason = "length"
            if reason:
                self._finish(seq, reason)
        return out

    def _finish(self, seq: Sequence_, reason: str) -> None:
        if seq.status == RUNNING:
            self.running.remove(seq)
            self.cache.release(seq.id)
        elif seq.status == WAITING:
            self.waiting.remove(seq)
        seq.status, seq.finish_reason = FINISHED, reason

    def penalty_counts(self, seq: Sequence_) -> Dict[int, int]:
        counts: Dict[int, int] = {}
        for t in seq.output:
            counts[t] = counts.get(t, 0) + 1
        return counts
