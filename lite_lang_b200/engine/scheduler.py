"""The scheduler: admits requests, cuts prompts into portions, decodes, finishes, frees.

In the manner of the reference's scheduler (``litelang/scheduler/scheduler.py:
148-181``, ``req_queue.py:178-261``, ``pause_strategy.py``):

* a waiting queue (first come, first served) and a running list;
* admission by the reference's estimate of the peak number of cached tokens
  (``req_queue.py:219-232``): with the candidates sorted by the tokens they are
  still expected to produce, descending, the peak is
  ``max_k(cumsum(held)[k] + expected[k] * (k + 1))`` and must fit the pool; a
  request is expected to produce ``max_new_tokens`` when the system is busy and
  0.6 of it when it is not, until it outlives that guess (``req_queue.py:59-66``);
  busy means that the tokens held by running and preempted requests exceed
  ``busy_scale`` of the pool (``req_queue.py:194,213-217``);
* when the cache cannot hold the next tokens, requests are taken out of the
  running list in the order of a strategy, their cache is freed, and they go to
  the *front* of the waiting queue to be recomputed from their prompt plus the
  tokens they had produced (``scheduler.py:107-120``, ``req_queue.py:152-165,
  204-207``).  The strategies are the reference's four; its ``LongestFirst`` and
  ``ShortestFirst`` sort the other way round than their names say
  (``pause_strategy.py:24-34``) and are kept here under names that say what they do.

What differs: the reference prefills whole prompts of a new batch in a forward
of their own and looks for new requests every 10 decode steps
(``scheduler.py:42,160-178``).  Here every step is one mixed batch under a token
budget: one token for every request that is decoding, and the rest of the budget
for portions of prompts, running requests first, then newly admitted ones.

What happens when pages run out (decided here, tested in tests/test_scheduler.py):
a decoding request that cannot get its next page makes the strategy's first
victim leave (by default the latest arrival; it may be that request itself); a
prompt portion that cannot get pages shrinks to what fits, or waits while others
are running; if nothing at all can run, the latest arrival leaves; a request
that does not fit even when it is alone finishes with the reason ``cache_full``.
Nothing ever waits for pages that cannot come.
"""

from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.sampler import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass(eq=False)      # a request is itself, not its field values: membership tests stay cheap
class Request:
    id: int
    prompt: List[int]
    params: SamplingParams
    max_new_tokens: int
    eos_ids: Tuple[int, ...] = ()
    output: List[int] = field(default_factory=list)
    status: str = WAITING
    slot: Optional[int] = None
    computed: int = 0                 # tokens whose keys and values are in the cache
    preemptions: int = 0
    finish_reason: Optional[str] = None
    arrival: int = 0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def token_slice(self, start: int, count: int) -> List[int]:
        """tokens[start:start + count] without building the whole list."""
        n = len(self.prompt)
        if start >= n:
            return self.output[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output[:start + count - n]

    @property
    def length(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def decoding(self) -> bool:
        return self.status == RUNNING and self.computed == self.length - 1 and len(self.output) > 0


# ---------------------------------------------------------------- strategies
STRATEGIES: Dict[str, Callable[[List[Request]], List[Request]]] = {}


def register_strategy(name: str):
    def deco(fn):
        STRATEGIES[name] = fn
        return fn
    return deco


@register_strategy("FIFOStrategy")
def _fifo(reqs):          # earliest arrival leaves first (pause_strategy.py:18-21)
    return sorted(reqs, key=lambda r: r.arrival)


@register_strategy("LIFOStrategy")
def _lifo(reqs):          # latest arrival leaves first (pause_strategy.py:36-39)
    return sorted(reqs, key=lambda r: r.arrival, reverse=True)


@register_strategy("ShortestLeavesFirstStrategy")
def _shortest(reqs):      # what the reference calls LongestFirstStrategy does (pause_strategy.py:30-34)
    return sorted(reqs, key=lambda r: (r.length, r.arrival))


@register_strategy("LongestLeavesFirstStrategy")
def _longest(reqs):       # what the reference calls ShortestFirstStrategy does (pause_strategy.py:24-28)
    return sorted(reqs, key=lambda r: (-r.length, r.arrival))


def peak_token_estimate(held_and_expected: Sequence[Tuple[int, int]]) -> int:
    """The reference's estimate of the most tokens the candidates will hold at once."""
    if not held_and_expected:
        return 0
    rows = sorted(held_and_expected, key=lambda he: he[1], reverse=True)
    peak, cum = 0, 0
    for k, (held, expected) in enumerate(rows, start=1):
        cum += held
        peak = max(peak, cum + expected * k)
    return peak


@dataclass
class PlannedEntry:
    request: Request
    start: int            # first token of the portion within request.tokens
    count: int
    samples: bool         # the portion ends the known tokens: its last logits give the next token
    feed: int = -1        # >= 0: planned ahead; the (one) token is the feed-th token sampled by the step before


class Scheduler:
    def __init__(self, manager: CacheManager, max_tokens_per_step: int, max_reqs: int = 1000,
                 busy_scale: float = 0.6, strategy: str = "LIFOStrategy", max_output_length: int = 200):
        if strategy not in STRATEGIES:
            raise ValueError(f"unknown strategy {strategy!r}; known: {sorted(STRATEGIES)}")
        self.manager = manager
        self.budget = int(max_tokens_per_step)
        self.max_reqs = int(max_reqs)
        self.busy_scale = float(busy_scale)
        self.strategy = STRATEGIES[strategy]
        self.max_output_length = int(max_output_length)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self._arrivals = itertools.count()
        self.counters = {"steps": 0, "tokens": 0, "preemptions": 0, "admitted": 0, "finished": 0,
                         "cache_full": 0}

    # ------------------------------------------------------------------
    @property
    def capacity_tokens(self) -> int:
        return self.manager.capacity_tokens()

    def add(self, req: Request) -> bool:
        """Queue a request.  False when the waiting queue is full (``max_reqs``)."""
        if len(self.waiting) >= self.max_reqs:
            return False
        if not req.prompt:
            raise ValueError("a request needs at least one prompt token")
        req.arrival = next(self._arrivals)
        req.status = WAITING
        if len(req.prompt) + 1 > self.manager.max_model_len:
            self._finish(req, "too_long")
            return True
        self.waiting.append(req)
        return True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------
    def _expected_new(self, req: Request, busy: bool) -> int:
        guess = req.max_new_tokens * (1.0 if busy else 0.6)
        if len(req.output) >= guess:
            guess = req.max_new_tokens
        return max(0, int(guess) - len(req.output))

    def _is_busy(self) -> bool:
        held = sum(r.length for r in self.running) + sum(r.length for r in self.waiting if r.preemptions > 0)
        return held > self.capacity_tokens * self.busy_scale

    def _fits(self, candidate: Request) -> bool:
        busy = self._is_busy()
        rows = [(r.length, self._expected_new(r, busy)) for r in self.running + [candidate]]
        return peak_token_estimate(rows) <= self.capacity_tokens

    def _finish(self, req: Request, reason: str) -> None:
        if req.slot is not None:
            self.manager.close(req.slot)
            req.slot = None
        req.status = FINISHED
        req.finish_reason = reason
        if req in self.running:
            self.running.remove(req)
        self.finished.append(req)
        self.counters["finished"] += 1
        if reason == "cache_full":
            self.counters["cache_full"] += 1

    def _preempt(self, req: Request) -> None:
        """Free the request's cache and put it at the front of the waiting queue."""
        self.manager.close(req.slot)
        req.slot = None
        req.computed = 0
        req.status = WAITING
        req.preemptions += 1
        self.running.remove(req)
        self.waiting.appendleft(req)
        self.counters["preemptions"] += 1

    # ------------------------------------------------------------------
    def plan(self) -> List[PlannedEntry]:
        """Decide the next step and reserve its pages.  Empty when there is nothing to run."""
        m = self.manager
        while True:
            plan: List[PlannedEntry] = []
            budget = self.budget
            # 1. one token for every decoding request, in arrival order
            for req in list(self.running):
                if req not in self.running or not req.decoding:
                    continue
                if budget <= 0:
                    break
                while req in self.running and not m.reserve(req.slot, req.computed + 1):
                    planned = {id(p.request) for p in plan}
                    candidates = [r for r in self.running if id(r) not in planned]
                    if len(self.running) == 1:
                        self._finish(req, "cache_full")
                        break
                    victim = self.strategy(candidates)[0] if candidates else req
                    self._preempt(victim)
                if req in self.running:
                    plan.append(PlannedEntry(req, req.computed, 1, True))
                    budget -= 1
            # 2. portions of prompts of requests that already run
            for req in self.running:
                if req.decoding or budget <= 0:
                    continue
                took = self._portion(req, budget)
                if took:
                    plan.append(took)
                    budget -= took.count
            # 3. new requests while the estimate, the slots and the budget allow
            while self.waiting and budget > 0 and m.num_free_slots > 0:
                cand = self.waiting[0]
                if cand.length + 1 > m.max_model_len or not m.can_ever_hold(cand.length):
                    self.waiting.popleft()
                    self._finish(cand, "too_long" if cand.length + 1 > m.max_model_len else "cache_full")
                    continue
                if self.running and not self._fits(cand):
                    break
                slot = m.open()
                if slot is None:
                    break
                cand.slot = slot
                cand.computed = 0
                took = self._portion(cand, budget)
                if took is None:
                    m.close(slot)
                    cand.slot = None
                    break
                self.waiting.popleft()
                cand.status = RUNNING
                self.running.append(cand)
                self.counters["admitted"] += 1
                plan.append(took)
                budget -= took.count
            if plan or not self.running:
                if plan:
                    self.counters["steps"] += 1
                    self.counters["tokens"] += sum(p.count for p in plan)
                return plan
            # nothing can move although requests are running: the latest arrival leaves
            if len(self.running) == 1:
                self._finish(self.running[0], "cache_full")
            else:
                self._preempt(_lifo(self.running)[0])

    def plan_ahead(self, plan: Sequence[PlannedEntry]) -> Optional[List[PlannedEntry]]:
        """The step after ``plan``, decided while ``plan`` still runs and its tokens are unknown.

        Possible when the outcome of ``plan`` cannot change what comes next except by ending a
        request: every running request samples in ``plan`` (so each will simply decode one more
        token), nothing waits for admission, and the pages for one more token can be reserved
        without making anyone leave.  Requests that reach their length limit with ``plan``'s token
        are left out.  A request that ends for a reason only its token shows (an eos id) is in the
        returned plan all the same; ``commit`` ignores it then.  None: decide after the step, as usual.
        """
        if self.waiting or not plan or not all(p.samples for p in plan):
            return None
        live = [(k, p) for k, p in enumerate(plan) if p.request.status == RUNNING]
        if len(live) != len(self.running):
            return None
        m = self.manager
        ahead: List[PlannedEntry] = []
        for k, p in live:
            req = p.request
            # (the token of `plan` is not in req.output yet; one planned ahead before it may not be either)
            known = p.start + p.count + 1 - len(req.prompt)  # output tokens once `plan` is committed
            if known >= req.max_new_tokens or p.start + p.count + 1 >= m.max_model_len:
                continue                  # ends with this step's token
            ahead.append(PlannedEntry(req, p.start + p.count, 1, True, feed=k))
        if not ahead or len(ahead) > self.budget:
            return None
        for q in ahead:
            if not m.reserve(q.request.slot, q.start + 1):
                return None               # pages already taken for others stay theirs and are used next step
        self.counters["steps"] += 1
        self.counters["tokens"] += len(ahead)
        return ahead

    def _portion(self, req: Request, budget: int) -> Optional[PlannedEntry]:
        """The largest next portion of the request that the budget and the free pages allow."""
        m = self.manager
        remaining = req.length - req.computed
        count = min(remaining, budget)
        if count <= 0:
            return None
        if not m.reserve(req.slot, req.computed + count):
            # shrink to what the pools can take now (every cache group is asked)
            count = min(count, m.max_reservable(req.slot) - req.computed)
            if count <= 0 or not m.reserve(req.slot, req.computed + count):
                return None
        return PlannedEntry(req, req.computed, count, req.computed + count == req.length)

    # ------------------------------------------------------------------
    def commit(self, plan: Sequence[PlannedEntry], sampled: Sequence[Optional[int]]) -> List[Request]:
        """Record a finished step.  ``sampled[i]`` is the token drawn for plan[i] (None if it did not
        sample).  The cache manager's lengths were already advanced by the step function.
        Returns the requests that finished."""
        done: List[Request] = []
        for p, tok in zip(plan, sampled):
            req = p.request
            if req.status != RUNNING:
                continue                  # planned ahead, but the request ended with the token before
            req.computed = p.start + p.count
            if not p.samples:
                continue
            if tok is None:
                raise ValueError("a sampling entry came back without a token")
            req.output.append(int(tok))
            reason = None
            if (not req.params.ignore_eos) and int(tok) in req.eos_ids:
                reason = "eos"
            elif len(req.output) >= req.max_new_tokens:
                reason = "length"
            elif req.length >= self.manager.max_model_len:
                reason = "model_len"
            if reason:
                self._finish(req, reason)
                done.append(req)
        return done
