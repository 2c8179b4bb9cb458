"""Generation: the scheduler, the step function and the sampler put together, and the entry point.

``generate`` follows the reference's programmatic call (src/quanta/minimax/generate.py:92-148):
``generate(model, prompt_ids, max_new_tokens=..., temperature=..., top_k=..., top_p=..., min_p=...,
eos_id=..., seed=...)`` returns the new token ids; an eos token ends the run and is not returned; an
empty prompt raises.  Unlike the reference, which steps the prompt one token at a time, the prompt is
fed in portions and many requests share each step.
"""

from __future__ import annotations

import time
from pathlib import Path

import torch

from ..sampling.sampler import Sampler
from .model import Model, load_model
from .scheduler import PlannedEntry, Request, SamplingParams, Scheduler
from .step import Engine, StepEntry


def _normalize_eos(eos_id) -> tuple:
    """An int, a collection of ids, or None -> tuple of ints (src/quanta/minimax/generate.py:83-89)."""
    if eos_id is None:
        return ()
    if isinstance(eos_id, (set, frozenset, tuple, list)):
        return tuple(int(s) for s in eos_id if s is not None)
    return (int(eos_id),)


class LLM:
    """A loaded model with its cache, scheduler and sampler.

    ``num_pages`` pages of ``page_size`` tokens are shared by all live requests; ``max_requests`` is the
    number of state slots; a step carries at most ``max_step_tokens`` tokens, a prompt portion at most
    ``prefill_chunk``.
    """

    def __init__(self, model, *, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                 num_pages: int | None = None, max_requests: int = 64, max_step_tokens: int = 4096,
                 prefill_chunk: int = 4096, max_position: int | None = None):
        if isinstance(model, (str, Path)):
            model, cfg = load_model(model, dtype=dtype, device=device)
            self.config = cfg
            if max_position is None:
                max_position = getattr(cfg, "max_position_embeddings", None)
        elif isinstance(model, Model):
            self.config = None
        else:
            raise TypeError("model must be a model folder or a loaded Model")
        if num_pages is None:
            num_pages = max(64, (max_requests * 4096) // page_size)
        self.engine = Engine(model, num_pages=num_pages, page_size=page_size, max_requests=max_requests)
        self.sampler = Sampler(self.engine.device)
        self.sched_opts = dict(max_step_tokens=max_step_tokens, prefill_chunk=prefill_chunk, max_position=max_position)
        self.default_eos = tuple(getattr(self.config, "eos_token_ids", ()) or ())
        self.lookahead = True        # launch decode steps ahead of the host's read of the step before
        self.last_stats: dict = {}
        self.step_log: list = []     # per step of the last run: tokens fed, tokens sampled, bytes copied, host time

    def generate(self, prompts, params=None, **options) -> list:
        """``prompts``: one list of token ids, or a list of such lists.  ``params``: one
        ``SamplingParams`` for all, or one per prompt; or pass its fields as keyword options.
        Returns the generated ids (one list, or a list of lists in the order of the prompts)."""
        single = bool(prompts) and not isinstance(prompts[0], (list, tuple))
        plist = [list(prompts)] if single else [list(p) for p in prompts]
        if params is None:
            if "eos_id" in options:
                options["eos_token_ids"] = _normalize_eos(options.pop("eos_id"))
            options.setdefault("eos_token_ids", self.default_eos)
            params = SamplingParams(**options)
        per = params if isinstance(params, (list, tuple)) else [params] * len(plist)
        if len(per) != len(plist):
            raise ValueError(f"{len(per)} sampling parameter sets for {len(plist)} prompts")
        reqs = [Request(rid=i, prompt=p, params=sp) for i, (p, sp) in enumerate(zip(plist, per))]
        self.run(reqs)
        outs = [r.generated for r in reqs]
        return outs[0] if single else outs

    def _decode_ahead(self, sched: Scheduler, plan: list) -> list | None:
        """The requests of the decode step that follows ``plan`` if that step can be launched before
        ``plan``'s tokens are read: every running request decodes in ``plan``, nothing waits, no request
        needs its earlier tokens on the host (penalties), pages are there without preempting anyone, and
        the step replays a captured graph.  Requests that reach their length with ``plan`` are left out; a
        request that stops on an end token in ``plan`` still runs in the step ahead, and its token there is
        dropped."""
        eng, mgr = self.engine, self.engine.manager
        if not self.lookahead or sched.waiting or len(plan) != len(sched.running):
            return None
        if any(e.count != 1 or not e.samples for e in plan):
            return None
        ahead = []
        for e in plan:
            r, p = e.request, e.request.params
            if p.repetition_penalty != 1.0 or p.frequency_penalty != 0.0 or p.presence_penalty != 0.0:
                return None
            if len(r.generated) + 1 >= p.max_new_tokens:
                continue
            if sched.max_position is not None and r.n_tokens + 1 >= sched.max_position:
                continue
            ahead.append(r)
        if not ahead:
            return None
        wants = {r.rid: mgr.length(r.rid) + 1 for r in ahead}
        if not mgr.can_reserve(wants) or not eng.decode_graph_ready(len(ahead), max(wants.values())):
            return None
        return ahead

    def run(self, requests: list) -> None:
        """Drive the given requests to completion.  While the requests only decode, the next step is
        launched with the ids still on the device, before the host reads them: planning, packing and the
        launch of a step then run while the device works on the step before."""
        eng = self.engine
        sched = Scheduler(eng.manager, **self.sched_opts)
        for r in requests:
            sched.add(r)
        steps = steps_ahead = 0
        self.step_log = []

        def launch(entries, samplers):
            logits = eng.step(entries)
            handle = None
            if samplers:
                handle = self.sampler.sample_async(logits, eng.slots, eng.last_want_slots, samplers, eng.status)
            self.step_log.append({"tokens": sum(len(e.tokens) for e in entries), "sampled": len(samplers),
                                  "h2d_bytes": eng.last_h2d_bytes, "d2h_bytes": 4 * (len(samplers) + 4),
                                  "t_end": None})
            return handle, self.step_log[-1]

        inflight = None           # (plan, requests that sample, handle, log entry) of the step not yet read
        while True:
            if inflight is None:
                plan = sched.plan()
                if not plan:
                    break
                entries = [StepEntry(e.request.rid, e.tokens, (e.count - 1,) if e.samples else ()) for e in plan]
                samplers = [e.request for e in plan if e.samples]
                for r in (e.request for e in plan if not eng.manager.has(e.request.rid)):
                    # the request's record on the device: its options, and where its draws go on (a request
                    # that was preempted comes back with its generated tokens as part of its prompt)
                    eng.admit(r.rid, prompt_len=len(r.prompt), params=r.params, drawn=len(r.generated))
                handle, log = launch(entries, samplers)
                inflight = (plan, samplers, handle, log)
            plan, samplers, handle, log = inflight
            ahead = self._decode_ahead(sched, plan) if handle is not None else None
            nxt = None
            if ahead:
                a_entries = [StepEntry(r.rid, [0], (0,), from_device=True) for r in ahead]
                a_handle, a_log = launch(a_entries, ahead)
                nxt = (ahead, a_handle, a_log)
                steps_ahead += 1
            sampled = {}
            if handle is not None:
                sampled = {r.rid: t for r, t in zip(samplers, handle.read())}
            sched.commit(plan, sampled)
            log["t_end"] = time.perf_counter()
            steps += 1
            inflight = None
            if nxt is not None:
                ahead, a_handle, a_log = nxt
                alive = [r for r in ahead if r.status == "running"]
                if alive:
                    # the step ahead becomes the step in flight, for the requests that are still running
                    a_plan = [PlannedEntry(r, r.n_tokens - 1, 1, True) for r in alive]
                    inflight = (a_plan, ahead, a_handle, a_log)
                else:
                    a_handle.read()                 # nothing of it is kept; wait for it before going on
                    a_log["t_end"] = time.perf_counter()
                    steps += 1
        eng.check()
        self.last_stats = {"steps": steps, "steps_ahead": steps_ahead, "cache": eng.manager.stats(),
                           "finish_reasons": {r.rid: r.finish_reason for r in requests},
                           "preemptions": sum(r.preemptions for r in requests)}


def generate(model, prompt_ids, *, max_new_tokens: int, temperature: float = 0.0, top_k: int = 0,
             top_p: float = 1.0, min_p: float = 0.0, eos_id=None, seed: int = 0,
             repetition_penalty: float = 1.0, frequency_penalty: float = 0.0, presence_penalty: float = 0.0,
             **engine_options):
    """Generate up to ``max_new_tokens`` ids after ``prompt_ids``; stops early on ``eos_id`` (an int
    or a collection; default: the model's own eos ids).  ``model`` is a model folder or an ``LLM``;
    ``prompt_ids`` one prompt or a list of prompts.  ``engine_options`` (dtype, page_size, num_pages,
    max_requests, max_step_tokens, prefill_chunk) apply when ``model`` is a folder."""
    llm = model if isinstance(model, LLM) else LLM(model, **engine_options)
    first = prompt_ids[0] if len(prompt_ids) else None
    if first is None or (isinstance(first, (list, tuple)) and any(len(p) == 0 for p in prompt_ids)):
        raise ValueError("prompt_ids is empty (need at least one token to prefill)")
    eos = llm.default_eos if eos_id is None else _normalize_eos(eos_id)
    params = SamplingParams(max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
                            min_p=min_p, seed=seed, repetition_penalty=repetition_penalty,
                            frequency_penalty=frequency_penalty, presence_penalty=presence_penalty,
                            eos_token_ids=eos)
    return llm.generate(prompt_ids, params)
