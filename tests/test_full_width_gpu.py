"""The engine at the layer widths of the full-size model against the plain implementation on the GPU:
two layers, six requests of 1 to 3,072 tokens (seed 7), four cuttings, float32 and bfloat16.  What is
compared and the bounds: ``tests/full_width.py``, which also runs the whole configuration (six layers,
sixteen requests) through ``bin/trace_run`` as a program."""

import pytest
import torch

from tests import full_width as F
from tests import helpers as H

pytestmark = pytest.mark.gpu
LAYERS, REQUESTS, EVERY, SEED = 2, 6, 12, 0


def _config(**changes):
    from quanta_b200.config import MiniMaxM3Config
    return MiniMaxM3Config.from_dict(F.raw_config(LAYERS, **changes))


def _replays(cfg, dtype, reqs, places):
    """cutting -> what the engine gave (rows and choices), every cutting with as few pages as it needs."""
    from quanta_b200.engine.model import random_model
    from quanta_b200.engine.step import Engine
    model = random_model(cfg, seed=SEED, dtype=dtype, device="cuda:0")
    parts = F.trace_routing(model)
    out = {}
    for cut, steps in F.cuttings(reqs).items():
        steps = F.thin(steps, places)
        eng = Engine(model, num_pages=H.tokens_in_flight(steps, 16) // 16, page_size=16, max_requests=8)
        out[cut] = F.replay_engine(eng, parts, steps)
        eng.manager.check_invariants()
        if cut == "mixed":
            used = eng.manager.stats()["groups"][0]
            assert used["allocations"] > used["pages"], "the mixed trace did not reuse a page"
        del eng
    del model, parts
    torch.cuda.empty_cache()
    return out


def test_float32_against_plain():
    cfg = _config()
    reqs = F.make_requests(REQUESTS, cfg.vocab_size)
    places = F.wanted_places(reqs, EVERY)
    free = F.plain_rows(cfg, SEED, reqs, places, None)
    scale = max(float(v.abs().max()) for v in free[0].values())
    assert 2.0 < scale < 20.0 and len(free[0]) > 500
    for cut, got in _replays(cfg, "float32", reqs, places).items():
        res = F.compare(cfg, SEED, reqs, places, got, free, None)
        assert res["choices_differ"] < 1e-3 * res["token_layers"], (cut, res)
        assert res["ok"], (cut, res)


def test_bfloat16_against_plain():
    cfg = _config()
    reqs = F.make_requests(REQUESTS, cfg.vocab_size)
    places = F.wanted_places(reqs, EVERY)
    free = F.plain_rows(cfg, SEED, reqs, places, torch.bfloat16)
    exact_free = F.plain_rows(cfg, SEED, reqs, places, None, given={r: v["idx"] for r, v in free[1].items()})[0]
    for cut, got in _replays(cfg, "bfloat16", reqs, places).items():
        res = F.compare(cfg, SEED, reqs, places, got, free, torch.bfloat16, exact_free)
        # measured: 2 % of the tokens choose differently with the same inputs; what follows from them is free
        assert res["primary"] < 0.05 * res["token_layers"], (cut, res)
        assert res["ok"], (cut, res)


def test_bfloat16_with_every_expert_chosen():
    """Eight experts, all eight chosen: no choice can differ, so every difference between the engine and the
    rounded plain run is rounding, and twice the rounding's own effect is a bound of a few hundredths."""
    cfg = _config(num_local_experts=8, num_experts_per_tok=8)
    reqs = dict(list(F.make_requests(REQUESTS, cfg.vocab_size).items())[:4])
    places = F.wanted_places(reqs, EVERY)
    free = F.plain_rows(cfg, SEED, reqs, places, torch.bfloat16)
    exact_free = F.plain_rows(cfg, SEED, reqs, places, None)[0]
    scale = max(float(v.abs().max()) for v in exact_free.values())
    for cut, got in _replays(cfg, "bfloat16", reqs, places).items():
        res = F.compare(cfg, SEED, reqs, places, got, free, torch.bfloat16, exact_free)
        assert res["choices_differ"] == 0 and res["rounding"]["max"] < 0.03 * scale, (cut, res)
        assert res["ok"], (cut, res)
