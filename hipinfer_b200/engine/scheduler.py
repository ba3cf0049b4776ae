"""The scheduler: it admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees. Host-side decisions only; it looks at the cache manager's free counts and
never touches the device, so its decisions are tested without a GPU.

Each step:
  1. every running request that is decoding gets one row (the token produced last);
  2. what is left of the token budget goes to prompt portions, running requests first, in the
     order they were admitted; a prompt may be cut anywhere, over as many steps as it takes;
  3. waiting requests are admitted, first come first served, while a state slot is free, the
     budget is not spent and the pages for their first portion exist.
A request's tokens are prompt + produced so far; `n_cached` of them are in the cache. The next
token is sampled in the step whose portion reaches the end of the tokens.

When pages run out: the running request admitted LAST is preempted; all its pages and its
state slot are given back and it returns to the FRONT of the waiting queue with nothing
cached, so that prompt and produced tokens are computed again when there is room (its
sampling is keyed by position, so it produces the same tokens). A request that could never fit
(prompt + max_new_tokens beyond the pool or the longest sequence) is refused when it is added,
which is why the oldest running request can always proceed and there is no deadlock.

The reference has no scheduler: the caller prefills slot after slot and decodes slots [0, B) in
lock-step (tests/gate.py:184-187); its only cut is `max_prefill` (src/api.cu:1788).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache import CacheManager
from ..sampling import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


class AdmissionError(ValueError):
    """The request can never run on this engine (too long for the pool or the longest sequence)."""


@dataclass
class Request:
    request_id: object
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    n_cached: int = 0
    status: str = WAITING
    preemptions: int = 0
    finish_reason: Optional[str] = None

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def decoding(self) -> bool:
        return len(self.prompt) + len(self.output) - self.n_cached == 1 and bool(self.output)


@dataclass
class Scheduled:
    request: Request
    start: int       # first token position of the portion
    n: int           # its length
    samples: bool    # the portion reaches the end of the tokens: sample the next token from its last row


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_tokens_per_step: int, max_model_len: int,
                 eos_token_ids: Sequence[int] = ()):
        if max_tokens_per_step < 1 or max_num_seqs < 1:
            raise ValueError("max_tokens_per_step and max_num_seqs must be positive")
        self.cache = cache
        self.max_num_seqs, self.budget, self.max_model_len = max_num_seqs, max_tokens_per_step, max_model_len
        self.eos = tuple(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []   # in admission order
        self.finished: List[Request] = []
        self.n_preemptions = 0
        self._preempted_now: set = set()   # requests preempted by the schedule() call that is running

    # ---------------------------------------------------------------- admission
    def add(self, request: Request) -> None:
        total = len(request.prompt) + request.params.max_new_tokens
        if not request.prompt:
            raise AdmissionError(f"request {request.request_id!r}: empty prompt")
        # the last produced token is never fed, so the cache holds at most total - 1 tokens
        if total - 1 > self.max_model_len:
            raise AdmissionError(f"request {request.request_id!r}: {len(request.prompt)} prompt + "
                                 f"{request.params.max_new_tokens} new tokens exceed the longest sequence "
                                 f"{self.max_model_len}")
        pages = -(-(total - 1) // self.cache.page_size)
        for g, pool in enumerate(self.cache.pools):
            if pages > pool.num_pages:
                raise AdmissionError(f"request {request.request_id!r} needs {pages} pages of cache group "
                                     f"{self.cache.groups[g].name!r}; the pool has {pool.num_pages}")
        request.status = WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- one step's decisions
    def _fits(self, req: Request, n: int, promised: List[int]) -> bool:
        need = self.cache.pages_needed(req.request_id, n)
        return all(nd + pr <= pool.free_count for nd, pr, pool in zip(need, promised, self.cache.pools))

    def _promise(self, req: Request, n: int, promised: List[int]) -> None:
        for g, nd in enumerate(self.cache.pages_needed(req.request_id, n)):
            promised[g] += nd

    def _preempt(self, victim: Request) -> None:
        if self.cache.has_request(victim.request_id):
            self.cache.free_request(victim.request_id)
        self.running.remove(victim)
        victim.n_cached, victim.status = 0, WAITING
        victim.preemptions += 1
        self.n_preemptions += 1
        self._preempted_now.add(victim.request_id)
        self.waiting.appendleft(victim)

    def schedule(self) -> List[Scheduled]:
        out: List[Scheduled] = []
        self._preempted_now = set()
        promised = [0] * len(self.cache.pools)
        budget = self.budget
        order = [r for r in self.running if r.decoding] + [r for r in self.running if not r.decoding]
        for req in order:
            if req.status != RUNNING or budget == 0:
                continue
            n = min(len(req.tokens) - req.n_cached, budget)
            while not self._fits(req, n, promised):
                victim = self.running[-1]
                if victim is req:
                    break
                taken = next((s for s in out if s.request is victim), None)
                if taken is not None:     # give back what this step had promised it
                    out.remove(taken)
                    for g, nd in enumerate(self.cache.pages_needed(victim.request_id, taken.n)):
                        promised[g] -= nd
                    budget += taken.n
                self._preempt(victim)
            if not self._fits(req, n, promised):
                self._preempt(req)        # it is the youngest and there is no room: it waits
                continue
            self._promise(req, n, promised)
            out.append(Scheduled(req, req.n_cached, n, req.n_cached + n == len(req.tokens)))
            budget -= n
        admitted = 0
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs \
                and admitted < self.cache.slots.free_count:
            req = self.waiting[0]
            if req.status != WAITING:     # ended while it waited (finish()): it leaves the queue
                self.waiting.popleft()
                continue
            if req.request_id in self._preempted_now and out:
                break                     # preempted by this very call for lack of room: not in the same step
            n = min(len(req.tokens), budget)
            if not self._fits(req, n, promised):
                break
            self.waiting.popleft()
            req.status = RUNNING
            self.running.append(req)
            self._promise(req, n, promised)
            out.append(Scheduled(req, 0, n, n == len(req.tokens)))
            budget -= n
            admitted += 1
        return out

    def finish(self, req: Request, reason: str) -> None:
        """End a request now, running or waiting (a stop condition noticed outside update): free its cache."""
        req.status, req.finish_reason = FINISHED, reason
        if req in self.running:
            self.running.remove(req)
        if req in self.waiting:           # preempted earlier and still queued: it must not be admitted again
            self.waiting.remove(req)
        if self.cache.has_request(req.request_id):
            self.cache.free_request(req.request_id)
        self.finished.append(req)

    # ---------------------------------------------------------------- after the step
    def update(self, scheduled: Sequence[Scheduled], sampled: Sequence[int]) -> List[Request]:
        """Record a step's result. `sampled` has one token per entry with samples=True, in order.
        Returns the requests that finished (their cache is freed here)."""
        done: List[Request] = []
        it = iter(sampled)
        for s in scheduled:
            req = s.request
            req.n_cached += s.n
            if not s.samples:
                continue
            tok = int(next(it))
            req.output.append(tok)
            reason = None
            if len(req.output) >= req.params.max_new_tokens:
                reason = "length"
            elif tok in req.params.stop_token_ids or (not req.params.ignore_eos and tok in self.eos):
                reason = "stop"
            elif len(req.tokens) > self.max_model_len:
                reason = "max_model_len"
            if reason:
                req.status, req.finish_reason = FINISHED, reason
                self.running.remove(req)
                if self.cache.has_request(req.request_id):
                    self.cache.free_request(req.request_id)
                self.finished.append(req)
                done.append(req)
        return done
