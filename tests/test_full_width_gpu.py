"""The engine at the layer widths of the full-size model (hidden 3072, 48 q / 8 kv heads of 128, rotary 64,
experts of width 1536, vocabulary 200064), two layers, random weights made on the device.

The plain implementation is too slow at these widths, so the engine is compared with itself: the same
requests whole and mixed (portions beside single tokens, few pages), in float32 and in bfloat16, and
bfloat16 against float32.  Two models:

* eight experts, all eight chosen: routing is continuous, so every difference is rounding and the
  bounds are tight (float32: summation order only; bfloat16: a few hundredths on logits of magnitude 6);
* 256 experts, eight chosen (the real routing): in float32 whole and mixed still agree to 1e-4; in
  bfloat16 a token whose eighth and ninth expert score alike may choose differently after rounding, which
  moves its logits by up to about one, so only the bulk of the rows is bounded.
"""

import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

WIDTHS = dict(vocab_size=200064, hidden_size=3072, intermediate_size=1536, num_hidden_layers=2,
              num_attention_heads=48, num_key_value_heads=8, head_dim=128, rotary_dim=64, rope_theta=5e6,
              use_qk_norm=True, qk_norm_type="per_layer", use_routing_bias=True, rms_norm_eps=1e-6,
              tie_word_embeddings=False, architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3")
LENGTHS = (300, 77, 150, 9)


def _thinned(steps, reqs):
    """Every sixth position and each request's last: a logits row is 800 KB here."""
    out, seen = [], {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            base, n = seen.get(e["id"], 0), len(e["tokens"])
            want = [w for w in range(n) if (base + w) % 6 == 0 or base + w == len(reqs[e["id"]]) - 1]
            entries.append({"id": e["id"], "tokens": e["tokens"], "want": want})
            seen[e["id"]] = base + n
        out.append({"entries": entries, "end": s["end"]})
    return out


def _run(n_experts, top_k):
    from quanta_b200.config import MiniMaxM3Config
    from quanta_b200.engine.model import random_model
    from quanta_b200.engine.step import Engine
    cfg = MiniMaxM3Config.from_dict(dict(WIDTHS, num_local_experts=n_experts, num_experts_per_tok=top_k))
    reqs = {f"r{i}": H.random_tokens(n, cfg.vocab_size, seed=70 + i) for i, n in enumerate(LENGTHS)}
    got = {}
    for dtype in ("float32", "bfloat16"):
        model = random_model(cfg, seed=0, dtype=dtype, device="cuda:0")
        for cut, steps in (("whole", H.cut_whole(reqs)), ("mixed", H.cut_mixed(reqs, 4, seed=3))):
            steps = _thinned(steps, reqs)
            eng = Engine(model, num_pages=H.tokens_in_flight(steps, 16) // 16, page_size=16, max_requests=8)
            got[dtype, cut] = H.replay(eng, steps)
            del eng
        del model
        torch.cuda.empty_cache()
    return got


def _row_errors(a, b):
    assert set(a) == set(b) and len(a) > 80
    return torch.tensor([float((a[k] - b[k]).abs().max()) for k in sorted(a, key=str)])


def test_every_expert_chosen_differences_are_rounding():
    got = _run(8, 8)
    scale = max(float(v.abs().max()) for v in got["float32", "whole"].values())
    assert 2.0 < scale < 20.0
    assert float(_row_errors(got["float32", "whole"], got["float32", "mixed"]).max()) < 1e-4
    assert float(_row_errors(got["bfloat16", "whole"], got["bfloat16", "mixed"]).max()) < 0.02 * scale
    assert float(_row_errors(got["float32", "whole"], got["bfloat16", "whole"]).max()) < 0.02 * scale


def test_real_routing_at_full_width():
    got = _run(256, 8)
    scale = max(float(v.abs().max()) for v in got["float32", "whole"].values())
    assert float(_row_errors(got["float32", "whole"], got["float32", "mixed"]).max()) < 1e-4
    # measured: median 0.009 / largest 0.91 between the cuts, median 0.11 / largest 1.07 between the precisions
    for a, b, mid in ((("bfloat16", "whole"), ("bfloat16", "mixed"), 0.01), (("float32", "whole"), ("bfloat16", "whole"), 0.06)):
        err = _row_errors(got[a], got[b])
        assert torch.isfinite(err).all()
        assert float(err.median()) < mid * scale, (a, b, float(err.median()))
        assert float(err.max()) < 0.5 * scale, (a, b, float(err.max()))
