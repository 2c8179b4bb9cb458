"""Engine against the plain implementation under every way of cutting requests into steps.

For each tiny configuration, in float32 and in bfloat16: each request alone and whole; most of it in
one step and the last 32 tokens one by one; portions of changing size down to two tokens; and mixed,
up to four live requests with so few pages that freed pages are reused.  Also long decoding, the
first tokens of a sequence, and the replay program itself.

Tolerances.  float32: 2e-5 absolute on logits of magnitude ~0.3 (summation order differs between the
CUDA kernels and the CPU).  bfloat16: the engine may differ from the plain bfloat16 run by at most
twice what bfloat16 rounding itself does to this model, measured as the largest difference between
the plain implementation with and without rounding of activations.
"""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import helpers as H
from tests.conftest import TINY

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
FP32_TOL = 2e-5
LENGTHS = {"A": (5, 11, 16, 75, 50), "B": (7, 23, 64, 33, 97), "C": (2, 49, 80, 17, 65),
           "D": (40, 300, 129, 270, 64)}            # D: several 128-key blocks and 64-key tiles a request


def _requests(name):
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": H.random_tokens(n, vocab, seed=100 * ord(name) + i) for i, n in enumerate(LENGTHS[name])}


_plain_cache = {}


def _plain(plain_models, name, act):
    key = (name, act)
    if key not in _plain_cache:
        _plain_cache[key] = H.plain_logits(plain_models[name], _requests(name), act=act)
    return _plain_cache[key]


def _tolerance(plain_models, name, dtype):
    if dtype == "float32":
        return FP32_TOL
    a, b = _plain(plain_models, name, torch.bfloat16), _plain(plain_models, name, None)
    return 2.0 * max(float((a[k] - b[k]).abs().max()) for k in a)


def _engine(model_dirs, name, dtype, num_pages, page_size):
    from quanta_b200.engine.model import load_model
    from quanta_b200.engine.step import Engine
    model, _ = load_model(model_dirs[name], dtype=dtype)
    return Engine(model, num_pages=num_pages, page_size=page_size, max_requests=8)


def _compare(got, want, tol, what):
    assert set(got) <= set(want)
    bad = H.first_wrong(got, want, tol)
    worst, where, scale = H.worst_error(got, want)
    assert bad is None, (f"{what}: first wrong place {bad} (request, position); worst error {worst:.3e} at "
                         f"{where}, tolerance {tol:.3e}, logits up to {scale:.3f}")
    return worst


CUTS = {
    "whole": lambda reqs: H.cut_whole(reqs),
    "tail_decode": lambda reqs: H.cut_tail_decode(reqs, 32),
    "portions": lambda reqs: H.cut_portions(reqs),
    "mixed": lambda reqs: H.cut_mixed(reqs, max_live=4, seed=3),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_cutting_matches_plain(model_dirs, plain_models, name, dtype):
    reqs = _requests(name)
    act = None if dtype == "float32" else torch.bfloat16
    want = _plain(plain_models, name, act)
    tol = _tolerance(plain_models, name, dtype)
    page_size = {"A": 4, "B": 8, "C": 16, "D": 16}[name]
    results = {}
    for cut, make in CUTS.items():
        steps = make(reqs)
        # exactly as many pages as the live requests need at the worst moment: freed pages are reused
        num_pages = H.tokens_in_flight(steps, page_size) // page_size
        eng = _engine(model_dirs, name, dtype, num_pages, page_size)
        got = H.replay(eng, steps)
        eng.manager.check_invariants()
        assert eng.manager.stats()["live_requests"] == 0
        assert len(got) == sum(len(t) for t in reqs.values())
        if cut == "mixed":
            used = eng.manager.stats()["groups"][0]
            assert used["allocations"] > used["pages"], "the mixed trace did not reuse a page"
        results[cut] = got
        _compare(got, want, tol, f"{name} {dtype} {cut}")
    # the cuttings agree with one another (beyond rounding nothing depends on the cut)
    for cut in ("tail_decode", "portions", "mixed"):
        _compare(results[cut], results["whole"], tol, f"{name} {dtype} {cut} vs whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_dirs, plain_models, dtype):
    """A short prompt and then 150 single-token steps across many page edges."""
    name = "A"
    toks = H.random_tokens(160, TINY[name]["vocab_size"], seed=7)
    reqs = {"long": toks}
    act = None if dtype == "float32" else torch.bfloat16
    want = H.plain_logits(plain_models[name], reqs, act=act)
    tol = FP32_TOL if dtype == "float32" else 2.0 * max(
        float((want[k] - v).abs().max()) for k, v in H.plain_logits(plain_models[name], reqs, act=None).items())
    eng = _engine(model_dirs, name, dtype, num_pages=40, page_size=4)
    got = H.replay(eng, H.cut_tail_decode(reqs, tail=150))
    _compare(got, want, tol, f"long decoding {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_decoding_across_a_graph_bucket_edge(model_dirs, plain_models, name, dtype):
    """A prompt of 500 tokens and then 40 single tokens, from captured graphs: at 512 keys the captured step
    of the first bucket gives way to the one of the next (a wider block table, another cut of the keys over
    the blocks, the same shared graph memory)."""
    toks = H.random_tokens(540, TINY[name]["vocab_size"], seed=21)
    reqs = {"edge": toks}
    act = None if dtype == "float32" else torch.bfloat16
    want = H.plain_logits(plain_models[name], reqs, act=act)
    tol = FP32_TOL if dtype == "float32" else 2.0 * max(
        float((want[k] - v).abs().max()) for k, v in H.plain_logits(plain_models[name], reqs, act=None).items())
    page_size = {"A": 4, "D": 16}[name]
    eng = _engine(model_dirs, name, dtype, num_pages=-(-540 // page_size), page_size=page_size)
    assert eng.use_graphs
    got = H.replay(eng, H.cut_tail_decode(reqs, tail=40))
    _compare(got, want, tol, f"{name} {dtype} across the bucket edge")
    captured = {k for k, g in eng._graphs.items() if g.graph is not None}
    assert captured == {(1, 512), (1, 1024)} and eng.graph_replays == 40 - 2
    assert eng.stats()["graphs"] == 2 and eng.stats()["graph_output_bytes"] > 0


def test_captured_steps_are_dropped_beyond_the_limit(model_dirs, plain_models):
    """Decode batches of 1, 2 and 3 requests with room for two captured steps: the one used longest ago is
    given up, captured again when its shape returns, and the logits stay right throughout."""
    from quanta_b200.engine.model import load_model
    from quanta_b200.engine.step import Engine
    name = "A"
    reqs = {f"g{i}": H.random_tokens(40, TINY[name]["vocab_size"], seed=60 + i) for i in range(3)}
    want = H.plain_logits(plain_models[name], reqs)
    model, _ = load_model(model_dirs[name], dtype="float32")
    eng = Engine(model, num_pages=40, page_size=4, max_requests=4, max_graphs=2)
    rids = list(reqs)
    steps = [{"entries": [{"id": r, "tokens": reqs[r][:10], "want": []} for r in rids], "end": []}]
    batches = [3, 3, 3, 2, 2, 2, 1, 1, 1, 3, 3, 3, 2, 2]        # the live requests of each decode step
    fed = {r: 10 for r in rids}
    for b in batches:
        entries = []
        for r in rids[:b]:
            entries.append({"id": r, "tokens": [reqs[r][fed[r]]], "want": [0]})
            fed[r] += 1
        steps.append({"entries": entries, "end": []})
    steps[-1]["end"] = rids
    got = H.replay(eng, steps)
    _compare(got, want, FP32_TOL, "captured steps dropped and captured again")
    assert eng.stats()["graphs"] == 2 and eng.graph_replays >= 6


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_first_tokens(model_dirs, plain_models, name):
    """Positions 0, 1, 2 of a sequence, fed one at a time and as one portion."""
    toks = H.random_tokens(3, TINY[name]["vocab_size"], seed=11)
    want = H.plain_logits(plain_models[name], {"f": toks})
    eng = _engine(model_dirs, name, "float32", num_pages=4, page_size=4)
    one_by_one = [{"entries": [{"id": "f", "tokens": [t], "want": [0]}], "end": ["f"] if i == 2 else []}
                  for i, t in enumerate(toks)]
    _compare(H.replay(eng, one_by_one), want, FP32_TOL, f"{name} first tokens one by one")
    _compare(H.replay(eng, H.cut_whole({"f": toks})), want, FP32_TOL, f"{name} first tokens whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_dirs, plain_models, tmp_path, dtype):
    """bin/trace_run as a user calls it: steps on stdin, logits files out, 'done <step>' lines."""
    name = "B"
    reqs = {k: v for k, v in list(_requests(name).items())[:3]}
    steps = H.cut_mixed(reqs, max_live=3, seed=5)
    lines = [json.dumps({"step": i, **s}) for i, s in enumerate(steps)]
    out = tmp_path / "logits"
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dirs[name]), "--dtype", dtype,
           "--out", str(out), "--max-tokens", str(H.tokens_in_flight(steps, 64))]
    r = subprocess.run(cmd, input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split() == [w for i in range(len(steps)) for w in ("done", str(i))]
    import numpy as np
    vocab = TINY[name]["vocab_size"]
    act = None if dtype == "float32" else torch.bfloat16
    want = _plain(plain_models, name, act)
    tol = _tolerance(plain_models, name, dtype)
    got, pos = {}, {}
    for i, s in enumerate(steps):
        n_want = sum(len(e["want"]) for e in s["entries"])
        arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(n_want, vocab)
        row = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = torch.from_numpy(arr[row].copy())
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    _compare(got, want, tol, f"trace_run {dtype}")
