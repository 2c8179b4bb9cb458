"""Helpers of the GPU tests: traces (ways of cutting requests into steps), replay through the
engine's step function, and comparison with the plain implementation."""

from __future__ import annotations

import random

import torch

from tests.plain import minimax_m3_plain as P


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# ---- ways of cutting -----------------------------------------------------------------------------
def cut_whole(reqs: dict) -> list[dict]:
    """Each request alone and whole, one step each, every place wanted."""
    steps = []
    for rid, toks in reqs.items():
        steps.append({"entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def cut_tail_decode(reqs: dict, tail: int = 32) -> list[dict]:
    """Most of it in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": toks[i:i + 1], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def cut_portions(reqs: dict, sizes=(7, 2, 13, 3, 5, 2, 29, 4), seed: int = 0) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in reqs.items():
        i, j = 0, seed
        while i < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - i)
            j += 1
            last = i + n == len(toks)
            steps.append({"entries": [{"id": rid, "tokens": toks[i:i + n], "want": list(range(n))}],
                          "end": [rid] if last else []})
            i += n
    return steps


def cut_mixed(reqs: dict, max_live: int = 4, seed: int = 0, prompt_frac: float = 0.6,
              portion_sizes=(2, 3, 5, 8, 17, 40)) -> list[dict]:
    """Up to ``max_live`` live requests; portions of some beside single tokens of others; a request
    is sometimes left out of a step.  The first ``prompt_frac`` of a request goes in portions, the
    rest token by token."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: dict = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, int(len(toks) * prompt_frac))]
        entries, end = [], []
        for rid in list(live):
            toks, done, prompt_len = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                      # left out of this step
            if done < prompt_len:
                n = min(rng.choice(list(portion_sizes)), prompt_len - done)
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[done:done + n], "want": list(range(n))})
            live[rid][1] = done + n
            if done + n == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def tokens_in_flight(steps: list[dict], round_to: int = 64) -> int:
    """Most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


# ---- replay -----------------------------------------------------------------------------------------
def replay(engine, steps: list[dict]) -> dict:
    """Run the steps through ``engine.step``; returns {(request, position): logits row (cpu float32)}."""
    from quanta_b200.engine.step import StepEntry
    got = {}
    pos = {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], tuple(e["want"])) for e in s["entries"]]
        logits = engine.step(entries, end=s["end"])
        engine.check()
        if logits is not None:
            logits = logits.float().cpu()
        row = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = logits[row]
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
    return got


def plain_logits(plain_model, reqs: dict, act=None, schedule=None, windows=None, reads_cache_of=None) -> dict:
    weights, cfg = plain_model
    out = {}
    for rid, toks in reqs.items():
        lg = P.forward_logits(weights, cfg, toks, act=act, compute=torch.float32, schedule=schedule, windows=windows,
                              reads_cache_of=reads_cache_of)
        for i in range(len(toks)):
            out[(rid, i)] = lg[i]
    return out


def worst_error(got: dict, want: dict):
    """(largest absolute difference, where, scale of the logits)."""
    worst, where, scale = 0.0, None, 0.0
    for key, row in got.items():
        ref = want[key]
        d = float((row - ref).abs().max())
        scale = max(scale, float(ref.abs().max()))
        if d > worst or where is None:
            worst, where = max(worst, d), key if d >= worst else where
    return worst, where, scale


def first_wrong(got: dict, want: dict, tol: float):
    bad = sorted((k for k in got if float((got[k] - want[k]).abs().max()) > tol), key=lambda k: (str(k[0]), k[1]))
    return bad[0] if bad else None


def first_wrong_place(err: dict, margins: dict, near_tie: float, tol: float):
    """The first (request, position) whose error exceeds ``tol`` although its router margin is clear."""
    bad = sorted((k for k, e in err.items() if e > tol and margins[k] >= near_tie), key=lambda k: (str(k[0]), k[1]))
    return (bad[0], err[bad[0]], margins[bad[0]]) if bad else None
