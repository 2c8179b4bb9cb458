"""Gate: float32 logits of the engine equal the plain implementation's under every way of cutting the work.

Two tiny random-weight models that differ in every size and option; each request whole, most of it in one
step and the last 32 tokens one by one, portions of changing size down to two tokens, and up to four live
requests mixed with exactly as many pages as the worst moment needs (the reference's cutting gate:
parity/minimax_m3_prefill_chunked_test.py:100-141 there, which demands bit-equality of its own two paths;
here two implementations are compared, to 2e-5 on logits of magnitude 0.3)."""
# parity-gate: gpu

from __future__ import annotations

import tempfile

from parity._gates import Checks

TOL = 2e-5


def run() -> int:
    import torch
    from safetensors.torch import load_file

    from quanta_b200.config import MiniMaxM3Config
    from quanta_b200.engine.model import load_model, write_random_model
    from quanta_b200.engine.step import Engine
    from tests import helpers as H
    from tests.conftest import SEEDS, TINY
    from tests.plain import minimax_m3_plain as P

    c = Checks("minimax_m3_cuttings_test")
    lengths = {"A": (5, 11, 16, 75, 50), "B": (7, 23, 64, 33, 97)}
    page = {"A": 4, "B": 8}
    for name in ("A", "B"):
        with tempfile.TemporaryDirectory() as d:
            write_random_model(MiniMaxM3Config.from_dict(TINY[name]), SEEDS[name], d)
            plain = (load_file(d + "/model.safetensors"), P.read_config(d))
            model, _ = load_model(d, dtype="float32")
        reqs = {f"r{i}": H.random_tokens(n, TINY[name]["vocab_size"], seed=100 * ord(name) + i) for i, n in enumerate(lengths[name])}
        want = H.plain_logits(plain, reqs)
        cuts = {"whole": H.cut_whole(reqs), "tail": H.cut_tail_decode(reqs, 32), "portions": H.cut_portions(reqs),
                "mixed": H.cut_mixed(reqs, max_live=4, seed=3)}
        for what, steps in cuts.items():
            eng = Engine(model, num_pages=H.tokens_in_flight(steps, page[name]) // page[name], page_size=page[name], max_requests=8)
            got = H.replay(eng, steps)
            worst, where, scale = H.worst_error(got, want)
            c.ok(len(got) == sum(map(len, reqs.values())), f"{name} {what}: every position answered")
            c.ok(H.first_wrong(got, want, TOL) is None, f"{name} {what}: worst error {worst:.2e} at {where} (logits up to {scale:.2f})")
            eng.manager.check_invariants()
            c.ok(eng.manager.stats()["live_requests"] == 0, f"{name} {what}: everything was given back")
        del model
        torch.cuda.empty_cache()
    c.done()
    return 0


if __name__ == "__main__":
    raise SystemExit(run())
