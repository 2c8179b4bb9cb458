"""Gate: generation through the entry point gives the plain implementation's tokens.

Greedy for three prompts of 5 / 11 / 16 tokens, 8 new tokens, pages of 4 (the first tiny configuration);
temperature 0.8 with a seed for two prompts of 7 / 23 tokens fed in portions of 6 beside decoded tokens,
pages of 8 (the second); an eos id stops a request and is not returned; an empty prompt raises (the
reference's gate of the loop: parity/minimax_generate_test.py:1-17 there)."""
# parity-gate: gpu

from __future__ import annotations

import tempfile

from parity._gates import Checks


def run() -> int:
    from safetensors.torch import load_file

    from quanta_b200 import generate
    from quanta_b200.config import MiniMaxM3Config
    from quanta_b200.engine.generate import LLM
    from quanta_b200.engine.model import write_random_model
    from tests import helpers as H
    from tests.conftest import SEEDS, TINY
    from tests.plain import minimax_m3_plain as P

    c = Checks("minimax_m3_generate_test")
    with tempfile.TemporaryDirectory() as d:
        write_random_model(MiniMaxM3Config.from_dict(TINY["A"]), SEEDS["A"], d)
        weights, cfg = load_file(d + "/model.safetensors"), P.read_config(d)
        llm = LLM(d, dtype="float32", page_size=4, num_pages=40, max_requests=4, max_step_tokens=12, prefill_chunk=6)
        prompts = [H.random_tokens(n, 512, 40 + i) for i, n in enumerate((5, 11, 16))]
        got = generate(llm, prompts, max_new_tokens=8, eos_id=[])
        for p, g in zip(prompts, got):
            c.ok(g == P.generate(weights, cfg, p, max_new_tokens=8), f"greedy tokens of a prompt of {len(p)}")
        stop = got[0][4]
        cut = generate(llm, prompts[0], max_new_tokens=8, eos_id=stop)
        c.ok(cut == got[0][: got[0].index(stop)], "an eos id ends the request and is not returned")
        try:
            generate(llm, [], max_new_tokens=2)
            c.ok(False, "an empty prompt must raise")
        except ValueError:
            c.ok(True, "empty prompt raises")
        c.ok(llm.engine.manager.stats()["live_requests"] == 0, "all slots released")
    with tempfile.TemporaryDirectory() as d:
        write_random_model(MiniMaxM3Config.from_dict(TINY["B"]), SEEDS["B"], d)
        weights, cfg = load_file(d + "/model.safetensors"), P.read_config(d)
        llm = LLM(d, dtype="float32", page_size=8, num_pages=16, max_requests=2, max_step_tokens=8, prefill_chunk=6)
        prompts = [H.random_tokens(7, 1000, 1), H.random_tokens(23, 1000, 2)]
        kw = dict(max_new_tokens=6, temperature=0.8, seed=1234, eos_id=[])
        a, b = generate(llm, prompts, **kw), generate(llm, prompts, **kw)
        c.ok(a == b, "the same seed gives the same tokens")
        c.ok(a != generate(llm, prompts, **{**kw, "seed": 99}), "another seed gives other tokens")
        for p, g in zip(prompts, a):
            c.ok(g == P.generate(weights, cfg, p, max_new_tokens=6, temperature=0.8, seed=1234), f"sampled tokens of a prompt of {len(p)}")
    c.done()
    return 0


if __name__ == "__main__":
    raise SystemExit(run())
