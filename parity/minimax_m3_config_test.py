"""Gate: config.json of the MiniMax-M3 text decoder -> typed configuration.

Required keys, the defaults of the flat and of the nested (``text_config``) parser, the eos fallback
chain, refusals (the reference's gate of the same kind: parity/minimax_m3_config_test.py:122-199 there).
Runs anywhere (no GPU)."""

from __future__ import annotations

from parity._gates import Checks
from quanta_b200.config import ConfigError, MiniMaxM3Config, resolve

BASE = dict(vocab_size=512, hidden_size=64, intermediate_size=32, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, num_local_experts=8, num_experts_per_tok=2)


def _refused(raw, word) -> bool:
    try:
        MiniMaxM3Config.from_dict(raw)
    except ConfigError as e:
        return word in str(e)
    return False


def run() -> int:
    c = Checks("minimax_m3_config_test")
    flat = MiniMaxM3Config.from_dict(BASE)
    c.ok(flat.rotary_dim == 16 and flat.rope_theta == 1e6 and flat.qk_norm_type == "per_layer", "flat defaults")
    c.ok(flat.eos_token_ids == (200020,) and flat.bos_token_id == 200019, "eos / bos fallbacks")
    c.ok(flat.attn_type_list == (1, 1), "attn_type_list default")
    nested = MiniMaxM3Config.from_dict({"text_config": dict(BASE, hidden_act="silu", use_qk_norm=True)})
    c.ok(nested.qk_norm_type == "per_head" and nested.rope_theta == 5e6, "nested defaults")
    gen = MiniMaxM3Config.from_dict(dict(BASE, eos_token_id=5), generation={"eos_token_id": [7, 8]})
    c.ok(gen.eos_token_ids == (7, 8), "generation_config wins")
    c.ok(MiniMaxM3Config.from_dict(dict(BASE, eos_token_id=5)).eos_token_ids == (5,), "config eos")
    for key in BASE:
        c.ok(_refused({k: v for k, v in BASE.items() if k != key}, key), f"missing {key} is refused by name")
    for change, word in (({"attn_type_list": [1]}, "attn_type_list"), ({"attn_type_list": [1, 0]}, "full softmax"),
                         ({"scoring_func": "softmax"}, "scoring_func"), ({"shared_intermediate_size": 8}, "shared"),
                         ({"use_gemma_norm": True}, "use_gemma_norm"), ({"moe_layer_freq": [0, 1]}, "dense feed-forward"),
                         ({"head_dim": 24}, "head_dim"), ({"rotary_dim": 7}, "rotary_dim")):
        c.ok(_refused(dict(BASE, **change), word), f"{change} is refused")
    c.ok(_refused({"text_config": dict(BASE)}, "swigluoai"), "the nested default activation is refused")
    c.ok(MiniMaxM3Config.from_dict(flat.to_dict()) == flat, "round trip")
    c.ok(resolve(dict(BASE, architectures=["MiniMaxM3ForCausalLM"])).name == "MiniMaxM3ForCausalLM", "registry")
    try:
        resolve({"architectures": ["LlamaForCausalLM"]})
        c.ok(False, "an unknown architecture must raise")
    except KeyError as e:
        c.ok("known" in str(e), "unknown architecture lists the known ones")
    c.done()
    return 0


if __name__ == "__main__":
    raise SystemExit(run())
