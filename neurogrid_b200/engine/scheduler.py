"""The request scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.  Pure host logic over the cache manager's accounting.

Each step: every running request gets its next tokens (one decode token, or the next portion
of its prompt), in admission order, then waiting requests are admitted first-come
first-served while a slot, budget and pages for all their tokens so far are left.  A portion
is cut to the step's token budget, to ``chunk_size`` and to the pages that are free.

When pages run out for a running request, the most recently admitted running request is
preempted: its pages and slot are given back and it returns to the FRONT of the waiting
queue; when it is admitted again its prompt and the tokens it had generated are recomputed
(its sampled tokens are kept, so its output does not change).  A request that cannot fit
even alone finishes with reason "cache_full".

The reference admits a request only when nothing is decoding, prefills it whole, reserves
all pages of prompt + max_tokens up front, fails the request if they are not free and
ignores a page that is missing in mid-decode
(pkg/inference/batch_scheduler.go:94-246,316,528,560-624).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.sampler import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PLACEHOLDER = -1        # an output token that has been sampled on the device but not read yet


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    key: Optional[int] = None           # number of the request's random stream (default: arrival order)
    output: List[int] = field(default_factory=list)
    fed: int = 0                        # tokens whose keys/values/state are in the cache
    state: str = WAITING
    finish_reason: Optional[str] = None
    preemptions: int = 0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.fed


@dataclass
class PlannedEntry:
    request: Request
    start: int                          # first token index (in prompt + output) of the portion
    count: int
    sample: bool                        # the portion reaches the end: its last logits are sampled
    out_index: int = -1                 # index in request.output that the sampled token fills


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    failed: List[Request] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_tokens_per_step: int, max_requests: int,
                 chunk_size: Optional[int] = None, eos_token_ids: Sequence[int] = ()):
        if max_tokens_per_step < 1:
            raise ValueError("max_tokens_per_step must be >= 1")
        self.cache = cache
        self.max_tokens_per_step = max_tokens_per_step
        self.max_requests = min(max_requests, cache.max_requests)
        self.chunk_size = chunk_size or max_tokens_per_step
        self.eos_token_ids = tuple(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []           # in admission order
        self._next_key = 0
        self.preemptions = 0

    # ------------------------------------------------------------------ queue
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError("a request needs at least one prompt token")
        if req.key is None:
            req.key = self._next_key
        self._next_key += 1
        req.state = WAITING
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _room(self, req: Optional[Request], free: List[int]) -> int:
        """Tokens the request can add with the pages in ``free`` (a new request if ``req`` is
        not live), not counting pages its window lets it give back first."""
        ps = self.cache.page_size
        if req is not None and self.cache.is_live(req.id):
            length = self.cache.length(req.id)
            freed = self.cache.pages_freed_first(req.id)
            have = [len(self.cache.table(req.id, g)) for g in range(len(free))]
        else:
            length, freed, have = 0, [0] * len(free), [0] * len(free)
        room = self.cache.max_seq_len - length
        for g in range(len(free)):
            room = min(room, (have[g] + free[g] + freed[g]) * ps - length)
        return max(0, room)

    def _charge(self, req: Request, n: int, free: List[int]) -> None:
        ps = self.cache.page_size
        if self.cache.is_live(req.id):
            take, freed = self.cache.pages_to_take(req.id, n), self.cache.pages_freed_first(req.id)
        else:
            take, freed = [-(-n // ps)] * len(free), [0] * len(free)
        for g in range(len(free)):
            free[g] -= take[g] - freed[g]

    def plan(self) -> StepPlan:
        """Decide the next step.  Preempted requests have already been released and re-queued,
        failed ones released and marked finished, when this returns."""
        plan = StepPlan()
        while True:
            plan.entries = []
            free = list(self.cache.pages_free())
            budget = self.max_tokens_per_step
            stalled: Optional[Request] = None
            for req in self.running:
                if budget == 0:
                    break
                want = min(req.pending, budget, self.chunk_size)
                if not self.cache.windowed and self.cache.is_live(req.id) and want <= self.cache.slack(req.id):
                    n = want                                 # fits in the pages it holds: nothing to charge
                else:
                    n = min(want, self._room(req, free))
                    if n <= 0:
                        stalled = req
                        break
                    self._charge(req, n, free)
                budget -= n
                plan.entries.append(PlannedEntry(req, req.fed, n, req.fed + n == len(req.prompt) + len(req.output)))
            if stalled is not None:
                victim = self.running[-1]
                if len(self.running) == 1:
                    self._fail(victim, "cache_full")
                    plan.failed.append(victim)
                else:
                    self._preempt(victim)
                    plan.preempted.append(victim)
                continue
            # admit waiting requests, first come first served; none in a step that had to
            # preempt.  A request comes in only if all the tokens it has so far fit in the free
            # pages with one page of headroom for each running request, so that an admission
            # does not at once force a preemption.
            ps = self.cache.page_size
            while self.waiting and budget > 0 and not plan.preempted and len(self.running) < self.max_requests \
                    and self.cache.slots_free() > sum(1 for e in plan.entries if not self.cache.is_live(e.request.id)):
                req = self.waiting[0]
                if req.pending + len(self.running) * ps > self._room(None, free):
                    if not self.running:                     # the whole pool is free and it still does not fit
                        self.waiting.popleft()
                        self._fail(req, "cache_full")
                        plan.failed.append(req)
                        continue
                    break
                n = min(req.pending, budget, self.chunk_size)
                self.waiting.popleft()
                req.state = RUNNING
                self.running.append(req)
                self._charge(req, req.pending, free)         # its later portions are spoken for
                budget -= n
                plan.entries.append(PlannedEntry(req, req.fed, n, req.fed + n == len(req.prompt) + len(req.output)))
            return plan

    def _preempt(self, req: Request) -> None:
        self.running.remove(req)
        if self.cache.is_live(req.id):
            self.cache.release(req.id)
        req.fed = 0
        req.state = WAITING
        req.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(req)

    def _fail(self, req: Request, reason: str) -> None:
        if req in self.running:
            self.running.remove(req)
        if self.cache.is_live(req.id):
            self.cache.release(req.id)
        req.state, req.finish_reason = FINISHED, reason

    # ------------------------------------------------------------------ one step ahead
    def commit_ahead(self, plan: StepPlan) -> None:
        """Record a launched step whose sampled tokens are not known yet: a placeholder stands
        in each sampled request's output until ``finalize`` brings the token."""
        for e in plan.entries:
            req = e.request
            req.fed += e.count
            if e.sample:
                e.out_index = len(req.output)
                req.output.append(PLACEHOLDER)

    def decode_ahead_plan(self) -> Optional[StepPlan]:
        """The step after one that is still in flight, if it can be decided without that
        step's tokens: every running request decodes one token (requests that will reach their
        length limit when the step in flight lands are left out), no request could be admitted,
        and the pages are there.  None otherwise (the caller then waits for the tokens)."""
        if self.waiting and len(self.running) < self.max_requests and self.cache.slots_free() > 0:
            return None
        plan = StepPlan()
        grow = 0
        for req in self.running:
            if req.pending != 1 or not req.output or req.output[-1] != PLACEHOLDER:
                return None
            n_out = len(req.output)
            if n_out >= req.params.max_new_tokens or len(req.prompt) + n_out >= self.cache.max_seq_len:
                continue                                      # finishes by length when its token lands
            if self.cache.windowed:
                return None
            if self.cache.slack(req.id) < 1:
                grow += 1
            plan.entries.append(PlannedEntry(req, req.fed, 1, True))
        if not plan.entries or len(plan.entries) > self.max_tokens_per_step:
            return None
        if grow and any(grow > p.free for p in self.cache.pools):
            return None                                       # would need a preemption: decide it with the tokens in hand
        return plan

    def finalize(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """The tokens of a step recorded by ``commit_ahead`` have arrived.  Requests that stop
        here finish now; if a later step was launched for them meanwhile, its token is dropped
        (their output is cut back to the stopping token)."""
        finished: List[Request] = []
        it = iter(sampled)
        for e in plan.entries:
            if not e.sample:
                continue
            tok = int(next(it))
            req = e.request
            if req.state != RUNNING or e.out_index >= len(req.output) or req.output[e.out_index] != PLACEHOLDER:
                continue                                      # finished or preempted meanwhile
            req.output[e.out_index] = tok
            reason = self._stop_reason(req, tok, e.out_index + 1)
            if reason:
                del req.output[e.out_index + 1:]
                self.running.remove(req)
                if self.cache.is_live(req.id):
                    self.cache.release(req.id)
                req.state, req.finish_reason = FINISHED, reason
                finished.append(req)
        return finished

    # ------------------------------------------------------------------ after the step
    def commit(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """Record the step: ``sampled`` has one token per entry with ``sample`` set, in order.
        Returns the requests that finished (their pages and slots are given back here)."""
        finished: List[Request] = []
        it = iter(sampled)
        for e in plan.entries:
            req = e.request
            req.fed += e.count
            if not e.sample:
                continue
            tok = int(next(it))
            req.output.append(tok)
            reason = self._stop_reason(req, tok)
            if reason:
                self.running.remove(req)
                self.cache.release(req.id)
                req.state, req.finish_reason = FINISHED, reason
                finished.append(req)
        return finished

    def _stop_reason(self, req: Request, tok: int, n_out: Optional[int] = None) -> Optional[str]:
        p = req.params
        n_out = len(req.output) if n_out is None else n_out
        if tok in p.stop_token_ids:
            return "stop"
        if not p.ignore_eos and tok in self.eos_token_ids:
            return "eos"
        if n_out >= p.max_new_tokens:
            return "length"
        if len(req.prompt) + n_out >= self.cache.max_seq_len:
            return "context"
        return None
