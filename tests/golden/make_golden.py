"""Anchor the plain implementation on the reference's own code, once, and store small outputs.

The reference's model code (src/quanta/minimax/*.py) imports ``mlx``, which is not installable here,
so it cannot be run.  Two pieces of the reference can: its pure-Python config parser
(src/quanta/minimax/config.py) and the self-contained numpy float64 oracle functions inside
parity/minimax_m3_layer_test.py:162-245 (``_np_rope``, ``_np_route``, ``_np_attn``, ...), which this
script extracts from the file's syntax tree and executes with numpy alone.  It feeds them seeded
inputs, and writes inputs' seeds and the outputs to ``reference_oracle.json`` beside this file;
``tests/test_plain.py`` recomputes the same quantities with the plain implementation and compares.

What this anchors: rotate-half partial rotary, the sigmoid router (selection with bias, bias-free
weights, renormalisation, scaling), the attention core with per-head q/k norm (the oracle applies
``1 + w``, so it is fed ``gain - 1``), and the routed sum of SwiGLU experts (``w1`` gate, ``w3`` up,
``w2`` down, the weight applied after ``down``, no shared term).  The oracle's expert is
``(up + 1) * gate * sigmoid(alpha * gate)`` with both clamped at ``limit``; with ``alpha = 1`` and
``limit = inf`` that is ``(up + 1) * silu(gate)``, and an input feature that is constant 1 whose ``w3``
column is -1 (and whose ``w1`` column is 0) takes the ``+ 1`` away, so ``_np_moe`` computes this
decoder's ``silu(gate) * up``; its shared expert is given zero weights.  What rests on the formulas
alone: q/k norm over the concatenated heads (no code of the reference computes it).

Run:  python tests/golden/make_golden.py /path/to/reference
"""

import ast
import json
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
WANTED = ("_np_sigmoid", "_np_gemma_rms", "_np_rope", "_np_attn", "_np_route", "_np_swigluoai", "_np_moe")


def load_oracle(ref_root: Path) -> dict:
    src = (ref_root / "parity" / "minimax_m3_layer_test.py").read_text()
    tree = ast.parse(src)
    ns = {"np": np}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in WANTED:
            exec(compile(ast.Module([node], []), "oracle", "exec"), ns)
    return ns


def cases():
    """Seeded inputs, small enough to commit the outputs."""
    rng = np.random.default_rng(1234)
    cfg = types.SimpleNamespace(num_attention_heads=4, num_key_value_heads=2, head_dim=16, rotary_dim=8,
                                rope_theta=10000.0, norm_eps=1e-6, attn_scale=16 ** -0.5,
                                num_experts_per_tok=3, norm_topk_prob=True, routed_scaling_factor=1.0)
    T, H = 6, 24
    x = rng.standard_normal((1, T, H))
    Wq = rng.standard_normal((4 * 16, H)) * 0.2
    Wk = rng.standard_normal((2 * 16, H)) * 0.2
    Wv = rng.standard_normal((2 * 16, H)) * 0.2
    Wo = rng.standard_normal((H, 4 * 16)) * 0.2
    qn = 1.0 + rng.uniform(-0.1, 0.1, 16)
    kn = 1.0 + rng.uniform(-0.1, 0.1, 16)
    gate = rng.standard_normal((10, H))
    bias = rng.uniform(-0.05, 0.05, 10)
    rope_in = rng.standard_normal((1, 3, T, 16))
    # routed experts: 10 experts of width 12 over the 24 features plus one that is constant 1
    E, I = 10, 12
    moe_w1 = rng.standard_normal((E, I, H)) * 0.3
    moe_w3 = rng.standard_normal((E, I, H)) * 0.3
    moe_w2 = rng.standard_normal((E, H + 1, I)) * 0.3
    return cfg, dict(x=x, Wq=Wq, Wk=Wk, Wv=Wv, Wo=Wo, qn=qn, kn=kn, gate=gate, bias=bias, rope_in=rope_in,
                     moe_w1=moe_w1, moe_w3=moe_w3, moe_w2=moe_w2)


def with_constant_feature(c, up_column: float):
    """The routed experts' inputs with a feature that is constant 1 appended: ``(x', gate', w1', w3')``.
    The router and ``w1`` ignore the feature (zero columns); ``w3`` weighs it by ``up_column``."""
    x = np.concatenate([c["x"], np.ones(c["x"].shape[:-1] + (1,))], axis=-1)
    pad = lambda w, v: np.concatenate([w, np.full(w.shape[:-1] + (1,), v)], axis=-1)      # noqa: E731
    return x, pad(c["gate"], 0.0), pad(c["moe_w1"], 0.0), pad(c["moe_w3"], up_column)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/the/reference/checkout")
    ref = Path(sys.argv[1])
    ns = load_oracle(ref)
    cfg, c = cases()
    out = {}
    out["rope"] = ns["_np_rope"](c["rope_in"], cfg.rotary_dim, cfg.rope_theta).tolist()
    idx, w = ns["_np_route"](c["x"][0], c["gate"], c["bias"], cfg)
    out["route_idx"] = np.sort(idx, axis=-1).tolist()
    order = np.argsort(idx, axis=-1)
    out["route_w"] = np.take_along_axis(w, order, axis=-1).tolist()
    out["attn"] = ns["_np_attn"](c["x"], c["Wq"], c["Wk"], c["Wv"], c["Wo"], c["qn"] - 1.0, c["kn"] - 1.0, cfg).tolist()
    # routed sum: (up' + 1) * silu(gate) with up' = up - 1 through the constant feature; no clamp; zero shared expert
    x1, gate1, w1, w3 = with_constant_feature(c, -1.0)
    moe_cfg = types.SimpleNamespace(**vars(cfg), swiglu_alpha=1.0, swiglu_limit=np.inf)
    zero = np.zeros((4, x1.shape[-1]))
    out["moe"] = ns["_np_moe"](x1, gate1, c["bias"], w1, c["moe_w2"], w3, zero, zero, np.zeros((x1.shape[-1], 4)),
                               moe_cfg).tolist()
    # the reference's config parser on one of the tiny configurations
    sys.path.insert(0, str(ref / "src"))
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_cfg", ref / "src" / "quanta" / "minimax" / "config.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_cfg"] = mod
    spec.loader.exec_module(mod)
    import tempfile
    raw = dict(vocab_size=512, hidden_size=64, intermediate_size=32, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, rotary_dim=8, rope_theta=10000.0, use_qk_norm=True,
               num_local_experts=8, num_experts_per_tok=2, eos_token_id=[7, 9])
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "config.json").write_text(json.dumps(raw))
        rc = mod.MiniMaxConfig.from_pretrained(d)
    out["config_in"] = raw
    out["config_parsed"] = {k: (list(v) if isinstance(v, tuple) else v) for k, v in vars(rc).items()
                            if isinstance(v, (int, float, str, bool, tuple))}
    (HERE / "reference_oracle.json").write_text(json.dumps(out))
    print("wrote", HERE / "reference_oracle.json", (HERE / "reference_oracle.json").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
