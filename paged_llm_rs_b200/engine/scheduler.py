"""What runs in the next step: admission, prompts cut into portions under a token
budget, decoding, finishing and freeing.  Pure host logic; no tensor is touched.

The policy is the reference's (crates/pagedllm/src/scheduler.rs):

* With a budget (``chunk``), a step carries every running request's next token
  first, then one portion of one prompt in the room that is left
  (scheduler.rs:388-499).  One prompt is in flight at a time; a new one joins
  only after the residents have their pages (scheduler.rs:436-446).
* Without a budget, a waiting prompt runs whole and alone (scheduler.rs:548-589).
* When the pages run out while decoding, the newest running request other than
  the one that needs the page is preempted: its pages are given back, it goes
  to the front of the queue and is recomputed from its prompt plus what it had
  produced; tokens already returned stay returned (scheduler.rs:645-661, 700-712).
* A prompt that the whole pool could never hold is refused and ends with
  ``Finish.LENGTH`` (scheduler.rs:681-690).  A running request that needs a page
  when nobody is left to evict ends with LENGTH too (the reference idles for good
  in that case, scheduler.rs:647-650, 663-665).
* A step is committed only after it ran: lengths advance, full pages get their
  names, sampled tokens are appended, a stop token ends the request and is not
  returned, ``max_tokens`` ends it with LENGTH (scheduler.rs:717-764).
"""

from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence as Seq, Tuple

from ..cache.manager import CacheManager
from ..errors import ConfigError
from ..sampling.sampler import Rng, SamplingParams
from .step import StepEntry


class Finish(enum.Enum):
    STOP = "stop"      # a stop token came, or the request was cancelled
    LENGTH = "length"  # max_tokens ran out, or the prompt can never fit
    ERROR = "error"    # a step the request was in failed


class Sequence:
    """One request from arrival to its last token (scheduler.rs:34-56)."""

    def __init__(self, id, prompt: Seq[int], sampling: SamplingParams, max_tokens: int,
                 stop_tokens: Seq[int] = (), seed: int = 0):
        if len(prompt) == 0:
            raise ConfigError("cannot generate from an empty prompt")
        self.id = id
        self.history: List[int] = [int(t) for t in prompt]  # prompt, then what was produced
        self.prompt_tokens = len(self.history)
        self.sampling = sampling
        self.max_tokens = int(max_tokens)
        self.stop_tokens = frozenset(int(t) for t in stop_tokens)
        self.rng = Rng(seed)
        self.pending: List[int] = list(self.history)  # fed next: all of history after admission or preemption, else one token
        self.generated = 0
        self.preemptions = 0
        self.prompt_left = 0  # prompt tokens still to run; non-zero only while a prompt runs in portions
        self.finish: Optional[Finish] = None
        self.output: List[int] = []


@dataclass
class Plan:
    kind: str  # "idle", "prefill", "mixed", "decode", "refused" (a waiting prompt), "outgrown" (a running request)
    ids: List[object] = field(default_factory=list)               # requests a token comes back for, in row order
    advanced: List[Tuple[object, int]] = field(default_factory=list)  # (request, tokens it writes)
    entries: List[StepEntry] = field(default_factory=list)
    refused: object = None


@dataclass
class Outcome:
    tokens: List[Tuple[object, int]] = field(default_factory=list)
    finished: List[Tuple[object, Finish]] = field(default_factory=list)


@dataclass
class Metrics:
    """Counters (scheduler.rs:201-250)."""

    steps: int = 0
    prefills: int = 0
    tokens: int = 0
    decode_rows: int = 0
    admission_stalls: int = 0
    preemptions: int = 0
    mixed_steps: int = 0
    decode_steps: int = 0
    recomputed_tokens: int = 0
    cached_tokens: int = 0
    prefilled_tokens: int = 0

    def prefix_hit_rate(self) -> float:
        asked = self.cached_tokens + self.prefilled_tokens
        return self.cached_tokens / asked if asked else 0.0

    def mean_batch(self) -> float:
        return self.decode_rows / self.decode_steps if self.decode_steps else 0.0


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch: int = 16, chunk: Optional[int] = 128,
                 max_positions: Optional[int] = None, max_prefill_seqs: int = 1):
        self.cache = cache
        # Prompts that may share one pass in chunked mode.  1 is the reference's behaviour (one
        # prompt joins per pass, scheduler.rs:388-447, which its README names as what inflates the
        # time to the first token when many requests arrive at once); more lets a prompt that
        # ends inside the budget be followed by the next one's first portion in the same pass.
        self.max_prefill_seqs = max(1, int(max_prefill_seqs))
        self.max_batch = max(1, int(max_batch))
        self.chunk = None if chunk is None else max(1, int(chunk))
        self.max_positions = max_positions
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.metrics = Metrics()

    # -- queueing ----------------------------------------------------------------------
    def submit(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def set_chunk(self, tokens: Optional[int]) -> None:
        self.chunk = None if tokens is None else max(1, int(tokens))

    def running_ids(self):
        return [s.id for s in self.running]

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- planning ----------------------------------------------------------------------
    def plan(self) -> Plan:
        p = self._refuse_unservable()
        if p is not None:
            return p
        if self.chunk is not None:
            p = self._mixed()
            return p if p is not None else self._decode()
        p = self._admit()
        return p if p is not None else self._decode()

    def _refuse_unservable(self) -> Optional[Plan]:
        if not self.waiting:
            return None
        head = self.waiting[0]
        n = len(head.pending)
        too_long = self.max_positions is not None and n > self.max_positions
        if not too_long and self.cache.pages_for(n, self.chunk) <= self.cache.num_pages:
            return None
        self.waiting.popleft()
        head.finish = Finish.LENGTH
        return Plan("refused", refused=head.id)

    def _prompt_in_flight(self, skip=()) -> Optional[int]:
        for i, s in enumerate(self.running):
            if s.prompt_left > 0 and s.finish is None and s.id not in skip:
                return i
        return None

    def _mixed(self) -> Optional[Plan]:
        if not self.waiting and self._prompt_in_flight() is None:
            return None         # no prompt to feed: a plain decode step, planned once (by _decode)
        budget = self.chunk
        ids, advanced, entries = [], [], []
        cap = min(self.max_batch, budget)
        for s in self.running:
            if len(entries) >= cap:
                break
            if s.prompt_left > 0 or s.finish is not None or len(s.pending) != 1:
                continue
            if self.cache.blocks_needed(s.id, 1) > 0 and not self.cache.reserve(s.id, 1):
                # A resident that needs a page from a dry pool is a preemption, and
                # choosing the victim is the plain decode's job (scheduler.rs:413-420).
                return None
            ids.append(s.id)
            advanced.append((s.id, 1))
            entries.append(StepEntry(s.id, [s.pending[0]], [0]))
        decodes = len(entries)
        room = budget - decodes
        if room <= 0:
            return None
        taken = []
        while room > 0 and len(taken) < self.max_prefill_seqs:
            index = self._prompt_in_flight(taken)
            if index is None:
                self._start_next_prompt()
                index = self._prompt_in_flight(taken)
            if index is None:
                break
            s = self.running[index]
            done = len(s.history) - s.prompt_left
            want = min(room, s.prompt_left)
            take = self.cache.reserve_up_to(s.id, want)
            if take <= 0:
                break
            last = take == s.prompt_left
            if last:
                ids.append(s.id)
            advanced.append((s.id, take))
            entries.append(StepEntry(s.id, s.history[done:done + take], [take - 1] if last else []))
            taken.append(s.id)
            room -= take
            if not last:
                break           # a part-run prompt finishes before the next is started
        if not taken:
            return None
        self.metrics.steps += 1
        self.metrics.mixed_steps += 1
        self.metrics.decode_rows += decodes
        if decodes:
            self.metrics.decode_steps += 1
        return Plan("mixed", ids, advanced, entries)

    def _start_next_prompt(self) -> None:
        """Move the first waiting request into the running set without running it,
        so that its prompt can be fed in portions (scheduler.rs:503-539)."""
        if not self.waiting:
            return
        if self.cache.available() == 0 or self.cache.slots_free() == 0:
            self.metrics.admission_stalls += 1
            return
        s = self.waiting.popleft()
        n = len(s.pending)
        self.cache.open(s.id)
        shared = self.cache.claim_prefix(s.id, s.pending)
        if self.cache.blocks_needed(s.id, 1) > 0 and not self.cache.reserve(s.id, 1):
            self.cache.close(s.id)
            s.pending = list(s.history)
            self.waiting.appendleft(s)
            self.metrics.admission_stalls += 1
            return
        self.metrics.cached_tokens += shared
        self.metrics.prefilled_tokens += n - shared
        s.prompt_left = max(1, n - shared)
        s.pending = []
        self.metrics.prefills += 1
        self.running.append(s)

    def _admit(self) -> Optional[Plan]:
        """Whole-prompt admission (scheduler.rs:548-589)."""
        if not self.waiting:
            return None
        n = len(self.waiting[0].pending)
        if self.cache.pages_for(n, None) > self.cache.available() or self.cache.slots_free() == 0:
            self.metrics.admission_stalls += 1
            return None
        s = self.waiting.popleft()
        self.cache.open(s.id)
        shared = self.cache.claim_prefix(s.id, s.pending)
        if not self.cache.reserve(s.id, n - shared):
            self.cache.close(s.id)
            s.pending = list(s.history)
            self.waiting.appendleft(s)
            self.metrics.admission_stalls += 1
            return None
        self.metrics.cached_tokens += shared
        self.metrics.prefilled_tokens += n - shared
        tokens = s.pending[shared:]
        s.pending = []
        self.running.append(s)
        self.metrics.steps += 1
        self.metrics.prefills += 1
        return Plan("prefill", [s.id], [(s.id, len(tokens))], [StepEntry(s.id, tokens, [len(tokens) - 1])])

    def _decode(self) -> Plan:
        """One token for every running request able to take one, preempting where the
        pool cannot give the page one of them needs (scheduler.rs:625-676)."""
        chosen: List[int] = []
        index = 0
        while index < len(self.running) and len(chosen) < self.max_batch:
            s = self.running[index]
            if s.finish is not None or len(s.pending) != 1:
                index += 1
                continue
            if self.cache.blocks_needed(s.id, 1) == 0 or self.cache.reserve(s.id, 1):
                chosen.append(index)
                index += 1
                continue
            victim = self._newest_evictable(index)
            if victim is None:
                index += 1
                continue
            self._preempt(victim)
            chosen = [c - 1 if c > victim else c for c in chosen if c != victim]
            if victim < index:
                index -= 1
        if not chosen:
            # A request that needs a page when nobody is left to evict has outgrown the
            # pool.  The reference idles here for good; this scheduler ends the request
            # with LENGTH, as it does for a prompt the pool can never hold.
            for s in self.running:
                if s.finish is None and len(s.pending) == 1 and self.cache.blocks_needed(s.id, 1) > 0:
                    s.finish = Finish.LENGTH
                    return Plan("outgrown", refused=s.id)
            return Plan("idle")
        seqs = [self.running[i] for i in chosen]
        self.metrics.steps += 1
        self.metrics.decode_steps += 1
        self.metrics.decode_rows += len(seqs)
        return Plan("decode", [s.id for s in seqs], [(s.id, 1) for s in seqs],
                    [StepEntry(s.id, [s.pending[0]], [0]) for s in seqs])

    # -- the decode step after a decode step, planned before that one is committed ----------------------
    def continuation(self, plan: Plan) -> Optional[List[Sequence]]:
        """While the decode step ``plan`` runs: the requests of the decode step after it, if that step
        is sure to be the same rows again provided none of them ends (nobody waits, no prompt is in
        flight, the step holds every running request), with the pages for one more token each reserved.
        None: plan the next step the ordinary way, after this one is committed."""
        if plan.kind != "decode" or self.waiting or len(self.running) != len(plan.ids) or len(plan.ids) > self.max_batch:
            return None
        for s, rid in zip(self.running, plan.ids):
            if s.id != rid or s.finish is not None or s.prompt_left > 0 or len(s.pending) != 1:
                return None
        for s in self.running:
            # (the step in flight is not committed: its token and the next one's both need their page)
            if self.cache.blocks_needed(s.id, 2) > 0 and not self.cache.reserve(s.id, 2):
                return None     # a dry pool: preemption is the ordinary plan's business
        return list(self.running)

    def ends_with(self, s: Sequence, token: int) -> bool:
        """Whether ``commit`` will end request ``s`` when its step brings ``token``."""
        return (s.finish is not None or token in s.stop_tokens or s.generated + 1 >= s.max_tokens
                or (self.max_positions is not None and len(s.history) + 1 >= self.max_positions))

    def count_decode_step(self, rows: int) -> None:
        """The counters of a decode step that was not planned by ``plan`` (see ``continuation``)."""
        self.metrics.steps += 1
        self.metrics.decode_steps += 1
        self.metrics.decode_rows += rows

    def _newest_evictable(self, protect: int) -> Optional[int]:
        for i in range(len(self.running) - 1, -1, -1):
            if i != protect and self.running[i].finish is None:
                return i
        return None

    def _preempt(self, index: int) -> None:
        s = self.running.pop(index)
        self.cache.close(s.id)
        s.pending = list(s.history)
        s.prompt_left = 0
        s.preemptions += 1
        self.metrics.preemptions += 1
        self.metrics.recomputed_tokens += len(s.history)
        self.waiting.appendleft(s)

    # -- committing --------------------------------------------------------------------
    def commit(self, plan: Plan, sampled: Seq[int]) -> Outcome:
        out = Outcome()
        by_id: Dict[object, Sequence] = {s.id: s for s in self.running}
        for rid, written in plan.advanced:
            s = by_id.get(rid)
            if s is None:
                continue
            self.cache.commit(rid, written, s.history)
            s.prompt_left = max(0, s.prompt_left - written)
        for rid, token in zip(plan.ids, sampled):
            s = by_id.get(rid)
            if s is None:
                continue
            token = int(token)
            s.pending = [token]
            s.history.append(token)
            s.generated += 1
            self.metrics.tokens += 1
            if token in s.stop_tokens:
                s.finish = Finish.STOP
            else:
                out.tokens.append((rid, token))
                s.output.append(token)
                if s.generated >= s.max_tokens:
                    s.finish = Finish.LENGTH
                elif self.max_positions is not None and len(s.history) >= self.max_positions:
                    s.finish = Finish.LENGTH  # the next token would sit past the last position
        if plan.kind == "refused":
            out.finished.append((plan.refused, Finish.LENGTH))
        self._retire(out)
        return out

    def fail(self, ids) -> Outcome:
        """A step with these requests failed: each ends with ``Finish.ERROR`` and gives back what it
        holds (pages taken for the step that failed included); nothing of that step is committed
        (crates/pagedllm-server/src/engine.rs:338-348)."""
        ids = set(ids)
        for s in self.running:
            if s.id in ids and s.finish is None:
                s.finish = Finish.ERROR
        out = Outcome()
        self._retire(out)
        return out

    def cancel(self, rid) -> None:
        for s in list(self.waiting):
            if s.id == rid:
                self.waiting.remove(s)
                return
        for s in self.running:
            if s.id == rid:
                s.finish = Finish.STOP
        self._retire(Outcome())

    def _retire(self, out: Outcome) -> None:
        keep = []
        for s in self.running:
            if s.finish is None:
                keep.append(s)
            else:
                self.cache.close(s.id)
                out.finished.append((s.id, s.finish))
        self.running = keep
