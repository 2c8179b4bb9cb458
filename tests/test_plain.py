"""The plain implementation itself (CPU): properties of each part, and the comparison with the
outputs of the reference's own oracle functions and config parser stored under tests/golden."""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.conftest import TINY
from tests.golden.make_golden import cases
from tests.plain import minimax_m3_plain as P

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_oracle.json").read_text())


def test_rope_against_reference_oracle():
    cfg, c = cases()
    x = torch.tensor(c["rope_in"][0]).transpose(0, 1)            # [T, heads, hd]
    got = P.partial_rope(x.double(), torch.arange(x.shape[0]), cfg.rotary_dim, cfg.rope_theta)
    want = torch.tensor(GOLDEN["rope"], dtype=torch.float64)[0].transpose(0, 1)
    # angles are a float32 product here, float64 in the oracle
    assert torch.allclose(got, want, atol=2e-6)
    assert torch.equal(got[..., cfg.rotary_dim:], x.double()[..., cfg.rotary_dim:])   # the rest passes unchanged


def test_router_against_reference_oracle():
    cfg, c = cases()
    idx, w = P.router(torch.tensor(c["x"][0]), torch.tensor(c["gate"]), torch.tensor(c["bias"]),
                      cfg.num_experts_per_tok, True, 1.0)
    order = torch.argsort(idx, dim=-1)
    assert torch.gather(idx, 1, order).tolist() == GOLDEN["route_idx"]
    assert torch.allclose(torch.gather(w, 1, order), torch.tensor(GOLDEN["route_w"], dtype=torch.float64), atol=1e-12)


def test_attention_against_reference_oracle():
    cfg, c = cases()
    x = torch.tensor(c["x"][0])
    T = x.shape[0]
    q = (x @ torch.tensor(c["Wq"]).T).reshape(T, 4, 16)
    k = (x @ torch.tensor(c["Wk"]).T).reshape(T, 2, 16)
    v = (x @ torch.tensor(c["Wv"]).T).reshape(T, 2, 16)
    q = P.qk_norm(q, torch.tensor(c["qn"]), 4, 16, "per_head", cfg.norm_eps)
    k = P.qk_norm(k, torch.tensor(c["kn"]), 2, 16, "per_head", cfg.norm_eps)
    pos = torch.arange(T)
    q, k = P.partial_rope(q, pos, 8, 10000.0), P.partial_rope(k, pos, 8, 10000.0)
    out = P.causal_attention(q, k, v, None, torch.float64) @ torch.tensor(c["Wo"]).T
    assert torch.allclose(out, torch.tensor(GOLDEN["attn"], dtype=torch.float64)[0], atol=1e-5)


def test_routed_sum_against_reference_oracle():
    """``_np_moe`` of the reference (parity/minimax_m3_layer_test.py:232-245) with its clamp switched off, its
    shared expert zero and its ``up + 1`` undone through a constant input feature (tests/golden/make_golden.py)
    against the plain routed sum: which matrix gates, which one goes up, the weight after ``down``, the
    sum over the chosen experts and nothing else."""
    from tests.golden.make_golden import with_constant_feature
    cfg, c = cases()
    x1, gate1, w1, w3 = with_constant_feature(c, 0.0)           # this decoder's up projection ignores the feature
    t = lambda a: torch.tensor(a, dtype=torch.float64)          # noqa: E731
    experts = [(t(w1[e]), t(w3[e]), t(c["moe_w2"][e])) for e in range(w1.shape[0])]
    got = P.moe(t(x1[0]), t(gate1), t(c["bias"]), experts, cfg.num_experts_per_tok, True, 1.0, None, torch.float64)
    want = torch.tensor(GOLDEN["moe"], dtype=torch.float64)[0]
    assert want.abs().max() > 0.1 and torch.allclose(got, want, atol=1e-10)


def test_config_reading_against_reference_parser():
    raw, parsed = GOLDEN["config_in"], GOLDEN["config_parsed"]
    c = P.normalise_config(raw)
    assert (c["V"], c["H"], c["I"], c["L"]) == (parsed["vocab_size"], parsed["hidden_size"],
                                                parsed["moe_intermediate_size"], parsed["num_hidden_layers"])
    assert (c["nq"], c["nkv"], c["hd"], c["rd"]) == (parsed["num_attention_heads"], parsed["num_key_value_heads"],
                                                     parsed["head_dim"], parsed["rotary_dim"])
    assert c["theta"] == parsed["rope_theta"] and c["eps"] == parsed["norm_eps"]
    assert c["qk_norm"] == parsed["use_qk_norm"] and c["qk_norm_type"] == parsed["qk_norm_type"]
    assert (c["E"], c["k"], c["bias"], c["renorm"], c["scale"]) == (
        parsed["num_local_experts"], parsed["num_experts_per_tok"], parsed["use_routing_bias"],
        parsed["norm_topk_prob"], parsed["routed_scaling_factor"])
    from quanta_b200.config import MiniMaxM3Config
    ours = MiniMaxM3Config.from_dict(raw)
    assert list(ours.eos_token_ids) == parsed["eos_token_ids"] and ours.attn_type_list == tuple(parsed["attn_type_list"])


def test_router_rules():
    x = torch.zeros(1, 4)
    gate = torch.zeros(6, 4)
    bias = torch.tensor([0.0, 0.3, 0.1, 0.3, -1.0, 0.2])
    idx, w = P.router(x, gate, bias, 3, True, 2.0)
    assert idx.tolist() == [[1, 3, 5]]                          # bias decides; ties go to the lower index
    assert torch.allclose(w, torch.full((1, 3), 2.0 / 3))       # weights are bias-free (all 0.5), renormed, scaled
    _, w2 = P.router(x, gate, bias, 3, False, 1.0)
    assert torch.allclose(w2, torch.full((1, 3), 0.5))


def test_causality_and_grouping(plain_models):
    for name in TINY:
        weights, cfg = plain_models[name]
        ids = [3, 1, 4, 1, 5, 9, 2, 6]
        a = P.forward_logits(weights, cfg, ids)
        b = P.forward_logits(weights, cfg, ids[:5] + [7, 7, 7])
        # a position sees only what came before (the library's products round a row differently in
        # another batch of rows, so equality holds to rounding)
        assert torch.allclose(a[:5], b[:5], atol=1e-6, rtol=0)
        assert not torch.allclose(a[5:], b[5:])
        assert a.shape == (8, cfg["V"])


def test_moe_equals_dense_sum(plain_models):
    weights, cfg = plain_models["A"]
    m = "model.layers.0.block_sparse_moe."
    experts = [tuple(weights[f"{m}experts.{e}.{n}.weight"] for n in ("w1", "w3", "w2")) for e in range(cfg["E"])]
    x = torch.randn(5, cfg["H"])
    gate, bias = weights[m + "gate.weight"], weights[m + "e_score_correction_bias"]
    y = P.moe(x, gate, bias, experts, cfg["k"], True, 1.0, None, torch.float32)
    idx, w = P.router(x, gate, bias, cfg["k"], True, 1.0)
    dense = torch.stack([P.expert_swiglu(x, *experts[e], None, torch.float32) for e in range(cfg["E"])], 1)
    want = sum(w[:, s, None] * dense[torch.arange(5), idx[:, s]] for s in range(cfg["k"]))
    assert torch.allclose(y, want, atol=1e-6)


def test_sampling_rules():
    lg = np.array([1.0, 3.0, 3.0, -2.0, 0.5], dtype=np.float32)
    assert P.sample(lg) == 1                                      # greedy: the first maximum
    kept = P.filter_logits(lg, top_k=2, top_p=1.0, min_p=0.0)
    assert np.isfinite(kept).tolist() == [False, True, True, False, False]
    kept = P.filter_logits(np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32)), 0, 0.7, 0.0)
    assert np.isfinite(kept).tolist() == [True, True, False, False]     # mass before the 2nd is 0.5 < 0.7; before the 3rd 0.8
    kept = P.filter_logits(np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32)), 0, 1.0, 0.35)
    assert np.isfinite(kept).tolist() == [True, True, False, False]     # p < 0.35 * 0.5 dropped
    out = P.apply_penalties(np.array([2.0, -2.0, 1.0], dtype=np.float32), [0, 1, 1], 2.0, 0.5, 0.25)
    assert np.allclose(out, [2.0 / 2 - 0.5 - 0.25, -2.0 * 2 - 1.0 - 0.25, 1.0])
    # same seed and draw: same token; the draws follow the distribution
    p = np.array([0.6, 0.3, 0.1])
    counts = np.zeros(3)
    for d in range(3000):
        counts[P.sample(np.log(p).astype(np.float32), temperature=1.0, seed=5, draw=d)] += 1
    assert np.abs(counts / 3000 - p).max() < 0.03
    assert P.sample(np.log(p).astype(np.float32), temperature=1.0, seed=5, draw=7) == \
        P.sample(np.log(p).astype(np.float32), temperature=1.0, seed=5, draw=7)


def test_philox_known_answers():
    assert [hex(x) for x in P.philox4x32(np.zeros((1, 4)), (0, 0))[0]] == \
        ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    ones = np.full((1, 4), 0xFFFFFFFF, dtype=np.uint64)
    assert [hex(x) for x in P.philox4x32(ones, (0xFFFFFFFF, 0xFFFFFFFF))[0]] == \
        ["0x408f276d", "0x41c83b0e", "0xa20bc7c6", "0x6d5451fd"]


def test_schedule_runs_a_layer_twice(plain_models):
    weights, cfg = plain_models["A"]
    ids = [5, 6, 7, 8]
    a = P.forward_logits(weights, cfg, ids, schedule=[0, 1, 0])
    b = P.forward_logits(weights, cfg, ids)
    assert a.shape == b.shape and not torch.allclose(a, b)
