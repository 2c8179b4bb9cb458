"""The engine against the plain implementation at the layer widths of the full-size model.

Hidden 3072, 48 q / 8 kv heads of 128, rotary 64, 256 experts of width 1536 with 8 chosen, vocabulary
200064; requests of 1 to 3,072 uniform token ids (seed 7); random weights made on the device from a
seed.  The plain implementation runs on the GPU too, float32 without TF32, one layer's tensors at a time,
drawn by name from the same seeded source the engine's weights came from (a tensor depends on the seed,
its name and the device type only), so the two never hold a second copy of the model.

Cuttings (the list of parity/minimax_m3_prefill_chunked_test.py:100-141, extended): every request whole;
most of it in one step and the last 32 tokens one by one; portions of 512 tokens; mixed, up to four live
requests, portions beside single tokens, with exactly as many pages as the worst moment needs.

What is compared: logits rows at every ``every``-th position and at each request's last, and the experts
every token chose in every layer.

The router is the one discontinuous function of the model.  Two implementations of the same arithmetic
differ by rounding (float32: the order of sums, about 1e-6 of a router score; bfloat16: 1e-3), and a token
whose ``k``-th and ``k+1``-th choice scores are closer than that may choose another expert.  That moves its
own logits by some tenths, and through its keys and values those of every later token of its request a
little, which in turn lets some of them choose differently.  So the comparison has two halves:

* **The choices.**  The engine reports the experts of every token (``--routing`` of ``bin/trace_run``, the
  ``trace`` list of the feed-forward part); the plain implementation reports its own and each token's
  margin (``router_margin``).  A difference is *primary* when no token at or before its position chose
  differently in an earlier layer, that is, when both implementations computed its scores from the same
  inputs up to rounding; every primary difference must lie at a token whose margin is below ``NEAR_TIE``
  (float32) or ``NEAR_TIE_BF16``.  Later differences follow from earlier ones and are free.
* **The arithmetic.**  For requests with a difference the plain implementation runs again, taking the
  engine's choices (``given``) and computing everything else itself.  With the choices equal every
  difference is rounding: float32 rows must agree to ``FP32_TIGHT`` (absolute, on logits of magnitude
  about 6); bfloat16 rows to twice what rounding itself does to this model, measured as the difference
  between the plain implementation with and without rounding of activations under the same choices.

As a program it runs the whole configuration through ``bin/trace_run`` and prints one JSON line a cutting:

    python -m tests.full_width --layers 6 --requests 16 --dtype float32
"""

from __future__ import annotations

import argparse
import json
import random
import subprocess
import sys
import tempfile
from pathlib import Path

import torch

from tests import helpers as H
from tests.plain import minimax_m3_plain as P

ROOT = Path(__file__).resolve().parent.parent
WIDTHS = dict(vocab_size=200064, hidden_size=3072, intermediate_size=1536, num_attention_heads=48,
              num_key_value_heads=8, head_dim=128, rotary_dim=64, rope_theta=5e6, use_qk_norm=True,
              qk_norm_type="per_layer", num_local_experts=256, num_experts_per_tok=8, use_routing_bias=True,
              rms_norm_eps=1e-6, tie_word_embeddings=False, architectures=["MiniMaxM3ForCausalLM"],
              model_type="minimax_m3")
NEAR_TIE = 2e-5        # choice-score margin below which a token may choose differently in float32
NEAR_TIE_BF16 = 1e-2   # the same with activations rounded to bfloat16 (measured: primary differences up to 1.7e-3)
FP32_TIGHT = 1e-4      # absolute, logits of magnitude about 6 (measured: 2.1e-5 at two layers, every cutting)


def raw_config(layers: int, **changes) -> dict:
    return dict(WIDTHS, num_hidden_layers=layers, **changes)


def make_requests(n: int, vocab: int, seed: int = 7, longest: int = 3072) -> dict:
    rng = random.Random(seed)
    lengths = [rng.randint(1, longest) for _ in range(n)]
    return {f"r{i}": H.random_tokens(m, vocab, seed=1000 * seed + i) for i, m in enumerate(lengths)}


def cut_chunks(reqs: dict, chunk: int = 512) -> list[dict]:
    steps = []
    for rid, toks in reqs.items():
        for i in range(0, len(toks), chunk):
            n = min(chunk, len(toks) - i)
            steps.append({"entries": [{"id": rid, "tokens": toks[i:i + n], "want": list(range(n))}],
                          "end": [rid] if i + n == len(toks) else []})
    return steps


def cuttings(reqs: dict) -> dict:
    return {"whole": H.cut_whole(reqs), "tail_decode": H.cut_tail_decode(reqs, 32), "chunks_512": cut_chunks(reqs, 512),
            "mixed": H.cut_mixed(reqs, max_live=4, seed=3, prompt_frac=0.9, portion_sizes=(2, 17, 40, 128, 300))}


def wanted_places(reqs: dict, every: int) -> dict:
    return {rid: sorted(set(range(0, len(t), every)) | {len(t) - 1}) for rid, t in reqs.items()}


def thin(steps: list[dict], places: dict) -> list[dict]:
    """The same steps, asking only for the logits at ``places`` (a row of logits is 800 KB here)."""
    out, seen = [], {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            base, n = seen.get(e["id"], 0), len(e["tokens"])
            keep = set(places[e["id"]])
            entries.append({"id": e["id"], "tokens": e["tokens"], "want": [w for w in range(n) if base + w in keep]})
            seen[e["id"]] = base + n
        out.append({"entries": entries, "end": s["end"]})
    return out


def seeded_weights(cfg, seed: int, device):
    """``name -> tensor`` on ``device``: the tensors ``random_model(cfg, seed)`` gives the engine on the same
    kind of device, drawn again when asked for (weights are data; no model code is shared)."""
    from quanta_b200 import models  # noqa: F401
    from quanta_b200.config.registry import resolve
    from quanta_b200.engine.model import Model
    from quanta_b200.weights.loader import RandomSource
    skeleton = Model(resolve(cfg.to_dict()).build_spec(cfg), dtype=torch.float32, device="cpu")
    src = RandomSource(skeleton.tensor_specs(), seed, matrix_dtype=torch.bfloat16)
    return lambda name: src.read(name, device)


def plain_rows(cfg, seed: int, reqs: dict, places: dict, act, device="cuda:0", given: dict | None = None):
    """The plain implementation on ``device``: ``({(request, position): logits row}, {request: what its router
    did})``; the second holds ``idx`` ``[layers, T, k]`` (experts in ascending order) and ``margin``
    ``[layers, T]``.  ``given[request]`` ``[layers, T, k]``: experts to take instead of the router's choice."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    pcfg = P.normalise_config(cfg.to_dict())
    rids = list(reqs)
    forced = {(j, i): given[rid][i] for j, rid in enumerate(rids) if given and rid in given
              for i in range(given[rid].shape[0])}
    probes = []
    with torch.no_grad():
        out = P.forward_logits_many(seeded_weights(cfg, seed, device), pcfg, [reqs[r] for r in rids],
                                    rows=[places[r] for r in rids], act=act, compute=torch.float32, probes=probes,
                                    given=forced)
    rows = {(rid, p): out[i][j] for i, rid in enumerate(rids) for j, p in enumerate(places[rid])}
    routing = {rid: {"idx": torch.stack([torch.sort(pr["idx"], dim=-1).values for pr in probes[i]]),
                     "margin": torch.stack([pr["margin"] for pr in probes[i]])} for i, rid in enumerate(rids)}
    return rows, routing


def _walk(steps):
    """For each step: its (request, position) keys of the wanted rows, and (request, tokens) of its entries."""
    pos = {}
    for s in steps:
        keys, spans = [], []
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            keys += [(e["id"], base + w) for w in e["want"]]
            spans.append((e["id"], len(e["tokens"])))
            pos[e["id"]] = base + len(e["tokens"])
        yield s, keys, spans


class _Collected:
    """Rows and choices of a replay, as they come step by step."""

    def __init__(self):
        self.rows, self.chunks = {}, {}

    def take(self, keys, spans, logits, chosen):
        for i, key in enumerate(keys):
            self.rows[key] = logits[i].float().clone()
        at = 0
        for rid, n in spans:
            self.chunks.setdefault(rid, []).append(chosen[:, at:at + n])
            at += n

    def choices(self) -> dict:
        return {rid: torch.sort(torch.cat(c, dim=1).long(), dim=-1).values for rid, c in self.chunks.items()}


def trace_routing(model) -> list:
    """Switch the routing trace of every routed feed-forward part on; the parts in the order the layers run."""
    parts = [model.blocks[e.layer].feed_forward for e in model.schedule]
    for p in parts:
        p.trace = []
    return parts


def replay_engine(engine, parts, steps: list[dict]) -> _Collected:
    """The steps through ``engine.step``, with the wanted logits rows and every token's experts."""
    from quanta_b200.engine.step import StepEntry
    got = _Collected()
    for s, keys, spans in _walk(steps):
        logits = engine.step([StepEntry(e["id"], e["tokens"], tuple(e["want"])) for e in s["entries"]], end=s["end"])
        engine.check()
        got.take(keys, spans, logits, torch.stack([p.trace.pop(0) for p in parts]))
    return got


def replay_trace_run(model_dir, dtype: str, seed: int, steps: list[dict], vocab: int, n_layers: int, top_k: int,
                     device="cuda:0") -> _Collected:
    """The same through ``bin/trace_run`` as a child process (weights made there from the seed)."""
    import numpy as np
    got = _Collected()
    with tempfile.TemporaryDirectory() as out:
        cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", out,
               "--max-tokens", str(H.tokens_in_flight(steps, 64)), "--random-weights", str(seed), "--routing"]
        proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        try:
            for i, (s, keys, spans) in enumerate(_walk(steps)):
                proc.stdin.write(json.dumps({"step": i, **s}) + "\n")
                proc.stdin.flush()
                line = proc.stdout.readline().split()
                if line != ["done", str(i)]:
                    raise RuntimeError(f"trace_run answered {line!r} to step {i} (exit code {proc.poll()})")
                logits = None
                if keys:
                    path = Path(out) / f"{i}.f32"
                    logits = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(len(keys), vocab)).to(device)
                    path.unlink()
                path = Path(out) / f"{i}.routing.i32"
                n = sum(m for _, m in spans)
                chosen = torch.from_numpy(np.fromfile(path, dtype="<i4").reshape(n_layers, n, top_k)).to(device)
                path.unlink()
                got.take(keys, spans, logits, chosen)
            proc.stdin.close()
            if proc.wait(timeout=600) != 0:
                raise RuntimeError(f"trace_run exited with {proc.returncode}")
        finally:
            if proc.poll() is None:
                proc.kill()
    return got


def primary_differences(mine: torch.Tensor, theirs: torch.Tensor):
    """``mine``, ``theirs`` ``[layers, T, k]`` sorted choices.  Returns (``differs`` ``[layers, T]`` bool,
    ``primary`` ``[layers, T]`` bool): a difference is primary when no token at or before its position
    differs in an earlier layer."""
    differs = (mine != theirs.to(mine.device)).any(-1)
    upto = torch.cummax(differs.to(torch.int8), dim=1).values.bool()          # some token <= p differs in this layer
    earlier = torch.zeros_like(differs)
    if differs.shape[0] > 1:
        earlier[1:] = torch.cummax(upto[:-1].to(torch.int8), dim=0).values.bool()
    return differs, differs & ~earlier


def quantiles(errors) -> dict:
    t = torch.tensor(sorted(errors), dtype=torch.float64)
    q = lambda f: float(t[min(len(t) - 1, int(f * len(t)))])      # noqa: E731
    return {"median": q(0.5), "p90": q(0.9), "p99": q(0.99), "max": float(t[-1])}


def compare(cfg, seed: int, reqs: dict, places: dict, got: _Collected, free: tuple, act, exact_free: dict | None = None) -> dict:
    """One replay against the plain implementation.  ``free``: ``plain_rows`` of the plain implementation
    left to its own choices (rounded like the engine: ``act``); ``exact_free``: its unrounded rows, for the
    bfloat16 bound.  Returns the figures and ``ok``."""
    rows_free, routing = free
    choices = got.choices()
    near = NEAR_TIE if act is None else NEAR_TIE_BF16
    n_diff = n_primary = 0
    worst_primary_margin = 0.0
    for rid in reqs:
        differs, primary = primary_differences(choices[rid], routing[rid]["idx"])
        n_diff += int(differs.sum())
        n_primary += int(primary.sum())
        if primary.any():
            worst_primary_margin = max(worst_primary_margin, float(routing[rid]["margin"][primary].max()))
    changed = [rid for rid in reqs if not torch.equal(choices[rid], routing[rid]["idx"].to(choices[rid].device))]
    want = dict(rows_free)
    exact = dict(exact_free) if exact_free is not None else None
    if changed:
        sub = {rid: reqs[rid] for rid in changed}
        given = {rid: choices[rid] for rid in changed}
        want.update(plain_rows(cfg, seed, sub, places, act, given=given)[0])
        if exact is not None:
            exact.update(plain_rows(cfg, seed, sub, places, None, given=given)[0])
    err = {k: float((got.rows[k] - want[k]).abs().max()) for k in want}
    res = {"rows": len(err), "token_layers": sum(len(t) for t in reqs.values()) * cfg.num_hidden_layers,
           "choices_differ": n_diff, "primary": n_primary, "largest_primary_margin": worst_primary_margin,
           "requests_rerun": len(changed), "error": quantiles(err.values())}
    ok = worst_primary_margin < near and set(got.rows) == set(want)
    if act is None:
        ok = ok and res["error"]["max"] <= FP32_TIGHT
    else:
        rounding = {k: float((want[k] - exact[k]).abs().max()) for k in want}
        res["rounding"] = quantiles(rounding.values())
        ok = ok and all(res["error"][q] <= 2.0 * res["rounding"][q] for q in res["error"])
    res["ok"] = bool(ok)
    return res


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--every", type=int, default=24, help="logits are compared at every n-th position")
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--seed", type=int, default=0, help="seed of the weights")
    ap.add_argument("--experts", type=int, nargs=2, default=None, metavar=("E", "K"),
                    help="experts and how many are chosen (default: 256 and 8)")
    args = ap.parse_args()
    from quanta_b200.config import MiniMaxM3Config
    changes = {} if args.experts is None else dict(num_local_experts=args.experts[0], num_experts_per_tok=args.experts[1])
    cfg = MiniMaxM3Config.from_dict(raw_config(args.layers, **changes))
    reqs = make_requests(args.requests, cfg.vocab_size)
    places = wanted_places(reqs, args.every)
    act = None if args.dtype == "float32" else torch.bfloat16
    free = plain_rows(cfg, args.seed, reqs, places, act)
    exact_free = plain_rows(cfg, args.seed, reqs, places, None, given={r: v["idx"] for r, v in free[1].items()})[0] \
        if act is not None else None
    scale = max(float(v.abs().max()) for v in free[0].values())
    ok = True
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "config.json").write_text(json.dumps(cfg.to_dict()))
        for cut, steps in cuttings(reqs).items():
            got = replay_trace_run(d, args.dtype, args.seed, thin(steps, places), cfg.vocab_size, cfg.num_hidden_layers,
                                   cfg.num_experts_per_tok)
            res = compare(cfg, args.seed, reqs, places, got, free, act, exact_free)
            ok = ok and res["ok"]
            print(json.dumps({"layers": args.layers, "requests": args.requests, "tokens": sum(map(len, reqs.values())),
                              "dtype": args.dtype, "cutting": cut, "steps": len(steps), "logit_scale": round(scale, 3),
                              **res}), flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
