"""Anchor the plain implementation on the reference's own code, once, and store small outputs.

The reference's model code (src/quanta/minimax/*.py) imports ``mlx``, which is not installable here,
so it cannot be run.  Two pieces of the reference can: its pure-Python config parser
(src/quanta/minimax/config.py) and the self-contained numpy float64 oracle functions inside
parity/minimax_m3_layer_test.py:162-245 (``_np_rope``, ``_np_route``, ``_np_attn``, ...), which this
script extracts from the file's syntax tree and executes with numpy alone.  It feeds them seeded
inputs, and writes inputs' seeds and the outputs to ``reference_oracle.json`` beside this file;
``tests/test_plain.py`` recomputes the same quantities with the plain implementation and compares.

What this anchors: rotate-half partial rotary, the sigmoid router (selection with bias, bias-free
weights, renormalisation, scaling), and the attention core with per-head q/k norm (the oracle applies
``1 + w``, so it is fed ``gain - 1``).  What rests on the formulas alone: q/k norm over the
concatenated heads, the SiLU SwiGLU expert (the oracle has only the clamped activation), and the
expert sum without a shared expert.

Run:  python tests/golden/make_golden.py /path/to/reference
"""

import ast
import json
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
WANTED = ("_np_sigmoid", "_np_gemma_rms", "_np_rope", "_np_attn", "_np_route")


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
    return cfg, dict(x=x, Wq=Wq, Wk=Wk, Wv=Wv, Wo=Wo, qn=qn, kn=kn, gate=gate, bias=bias, rope_in=rope_in)


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
