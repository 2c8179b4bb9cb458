"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.  Host-side decisions only; it sees requests, token counts, pages and slots.

Policy (the reference admits first-in first-out into free slots and prefills each prompt whole while
nothing else advances, src/quanta/shim/omlx.py:1449-1510; here prompts are cut so decoding goes on):

1. Every running request whose cache holds all but its newest token decodes one token.  If the
   pages for that are not there, the most recently admitted running request is preempted: its pages
   and slot are given back and it returns to the head of the waiting queue with prompt + generated
   tokens as its new prompt (recomputed later; its draws continue where they stopped).  A request
   that cannot get pages even alone is finished with reason ``out_of_pages``.
2. What is left of the step's token budget goes to prompt portions, in admission order: first the
   running requests that still have prompt to feed, then waiting requests while a state slot is free
   and the pages of their next portion fit.  A portion is at most ``prefill_chunk`` tokens (default 4,096,
   the ``chunk_tokens`` of the reference's chunked prefill, src/quanta/minimax/runtime_m3.py:190-192; a
   step of a model with routed experts reads every expert's weights whatever its size, so up to some
   thousand tokens a larger portion costs no more time than a small one).
3. After the step, a request whose last fed token was the newest one gets a token sampled from that
   position's logits.  It finishes on an eos id (not returned), on ``max_new_tokens`` (``length``) or
   at the position limit (``length``); its pages and slot are freed in the same pass.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager


@dataclass
class SamplingParams:
    """Option names and meanings as in the reference's ``generate`` / engine sampler
    (src/quanta/minimax/generate.py:92-104, src/quanta/shim/omlx.py:1796-1810)."""
    max_new_tokens: int = 16
    temperature: float = 0.0          # <= 0: greedy
    top_k: int = 0                    # 0: off
    top_p: float = 1.0                # outside (0, 1): off
    min_p: float = 0.0                # 0: off
    seed: int = 0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    eos_token_ids: tuple = ()


@dataclass
class Request:
    rid: object
    prompt: list
    params: SamplingParams
    generated: list = field(default_factory=list)
    n_cached: int = 0                 # tokens of prompt + generated whose K/V are in the cache
    status: str = "waiting"           # waiting | running | finished
    finish_reason: str | None = None  # stop | length | out_of_pages
    preemptions: int = 0
    admitted_at: int = -1

    @property
    def tokens(self) -> list:
        return self.prompt + self.generated

    @property
    def n_tokens(self) -> int:
        return len(self.prompt) + len(self.generated)


@dataclass
class PlannedEntry:
    request: Request
    start: int                # first token (index into request.tokens) fed this step
    count: int
    samples: bool             # the last fed token is the newest one: its logits are sampled

    @property
    def tokens(self) -> list:
        return self.request.tokens[self.start: self.start + self.count]


class Scheduler:
    def __init__(self, manager: CacheManager, *, max_step_tokens: int = 4096, prefill_chunk: int = 4096,
                 max_position: int | None = None):
        if max_step_tokens <= 0 or prefill_chunk <= 0:
            raise ValueError("max_step_tokens and prefill_chunk must be positive")
        self.mgr = manager
        self.max_step_tokens = int(max_step_tokens)
        self.prefill_chunk = int(prefill_chunk)
        self.max_position = max_position
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self._clock = 0

    # ---- intake -----------------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError("prompt_ids is empty (need at least one token to prefill)")
        if req.params.max_new_tokens <= 0:
            req.status, req.finish_reason = "finished", "length"
            self.finished.append(req)
            return
        self.waiting.append(req)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- finishing and preempting ---------------------------------------------------------------------
    def _release(self, req: Request) -> None:
        if self.mgr.has(req.rid):
            self.mgr.free(req.rid)
        if req in self.running:
            self.running.remove(req)

    def _finish(self, req: Request, reason: str) -> None:
        self._release(req)
        req.status, req.finish_reason = "finished", reason
        self.finished.append(req)

    def _preempt(self, req: Request) -> None:
        self._release(req)
        req.status, req.n_cached = "waiting", 0
        req.preemptions += 1
        self.mgr.preemptions += 1
        self.waiting.appendleft(req)

    # ---- planning -------------------------------------------------------------------------------------
    def plan(self) -> list[PlannedEntry]:
        """Decide the next step.  May preempt or finish requests as a side effect.  Reserves nothing:
        the step function reserves the pages, which by construction fit.  Returns [] only when no
        request is left."""
        while True:
            entries = self._plan_once()
            if entries or not self.running:
                return entries
            # requests are running but none can move (a prompt portion finds no pages): make room
            self._make_room()

    def _make_room(self) -> None:
        victim = max(self.running, key=lambda r: r.admitted_at)
        if len(self.running) == 1:
            self._finish(victim, "out_of_pages")
        else:
            self._preempt(victim)

    def _plan_once(self) -> list[PlannedEntry]:
        mgr = self.mgr
        budget = self.max_step_tokens
        # 1. decode tokens, preempting from the back until their pages fit
        while True:
            decoders = [r for r in self.running if r.n_cached == r.n_tokens - 1][:budget]
            wants = {r.rid: r.n_cached + 1 for r in decoders}
            if mgr.can_reserve(wants):
                break
            self._make_room()
        entries = [PlannedEntry(r, r.n_cached, 1, True) for r in decoders]
        budget -= len(entries)
        # 2. prompt portions of running requests, in admission order
        for r in sorted(self.running, key=lambda r: r.admitted_at):
            if budget <= 0:
                break
            if r.rid in wants:
                continue
            n = min(self.prefill_chunk, r.n_tokens - r.n_cached, budget)
            trial = dict(wants)
            trial[r.rid] = r.n_cached + n
            if not mgr.can_reserve(trial):
                continue                      # waits for pages that other requests will free
            wants = trial
            entries.append(PlannedEntry(r, r.n_cached, n, r.n_cached + n == r.n_tokens))
            budget -= n
        # 3. admit waiting requests, first in first out
        admitted = 0
        while self.waiting and budget > 0 and admitted < mgr.slots.free_count:
            r = self.waiting[0]
            n = min(self.prefill_chunk, r.n_tokens, budget)
            trial = dict(wants)
            trial[r.rid] = n
            if not mgr.can_reserve(trial):
                if not self.running and not entries:
                    # nothing is running and the head of the queue cannot even start: it never will
                    self.waiting.popleft()
                    self._finish(r, "out_of_pages")
                    continue
                break
            self.waiting.popleft()
            r.status, r.admitted_at = "running", self._clock
            self._clock += 1
            self.running.append(r)
            admitted += 1
            wants = trial
            entries.append(PlannedEntry(r, 0, n, n == r.n_tokens))
            budget -= n
        return entries

    # ---- after the step -----------------------------------------------------------------------------------
    def commit(self, entries: list[PlannedEntry], sampled: dict) -> list[Request]:
        """``sampled``: request id -> token for the entries that sample.  Returns requests that finished."""
        done = []
        for e in entries:
            r = e.request
            r.n_cached = e.start + e.count
            if not e.samples:
                continue
            tok = int(sampled[r.rid])
            if tok in r.params.eos_token_ids:
                self._finish(r, "stop")
                done.append(r)
                continue
            r.generated.append(tok)
            at_limit = self.max_position is not None and r.n_tokens >= self.max_position
            if len(r.generated) >= r.params.max_new_tokens or at_limit:
                self._finish(r, "length")
                done.append(r)
        return done
