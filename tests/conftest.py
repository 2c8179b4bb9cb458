"""Shared fixtures: tiny configurations of the architecture and model folders with random weights.

Model folders are written to temporary folders and never committed.  Tests marked ``gpu`` need a
CUDA device and the compiled kernels; everything else runs on the CPU.
"""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the compiled kernels")


# Tiny configurations that differ in every size and option: head counts and groups, sizes that
# are no power of two, layers, vocabulary, eps, rotary share and base, q/k norm (over all heads, per
# head, none), experts, top-k, bias, renormalisation, scale factor, tied head.
TINY = {
    "A": dict(vocab_size=512, hidden_size=64, intermediate_size=32, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, rotary_dim=8, rope_theta=10000.0,
              use_qk_norm=True, qk_norm_type="per_layer", num_local_experts=8, num_experts_per_tok=2,
              use_routing_bias=True, rms_norm_eps=1e-6, tie_word_embeddings=False,
              architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3", eos_token_id=511),
    "B": dict(vocab_size=1000, hidden_size=96, intermediate_size=48, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=1, head_dim=32, rotary_dim=32, rope_theta=5e6,
              use_qk_norm=False, num_local_experts=16, num_experts_per_tok=4, use_routing_bias=False,
              routed_scaling_factor=2.5, rms_norm_eps=1e-5, tie_word_embeddings=True,
              architectures=["MiniMaxM2ForCausalLM"], model_type="minimax_m2", eos_token_id=[998, 999]),
    "C": dict(vocab_size=333, hidden_size=72, intermediate_size=40, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, partial_rotary_factor=0.5,
              rope_theta=25000.0, rope_section=[4, 4, 4], use_qk_norm=True, qk_norm_type="per_head",
              num_local_experts=12, num_experts_per_tok=3, use_routing_bias=True, norm_topk_prob=False,
              routed_scaling_factor=0.5, rms_norm_eps=1e-5, tie_word_embeddings=False,
              architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3", eos_token_id=332),
    # the head size, page size and widths that take the kernels of the full-size model (tcgen05 prefill
    # attention, TMA decode attention, tcgen05 experts, tensor-core router), at a small scale
    "D": dict(vocab_size=777, hidden_size=256, intermediate_size=192, num_hidden_layers=2,
              num_attention_heads=8, num_key_value_heads=2, head_dim=128, rotary_dim=64, rope_theta=5e6,
              use_qk_norm=True, qk_norm_type="per_layer", num_local_experts=16, num_experts_per_tok=4,
              use_routing_bias=True, rms_norm_eps=1e-6, tie_word_embeddings=False,
              architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3", eos_token_id=776),
}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3}


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (random weights, seeded)."""
    from quanta_b200.config import MiniMaxM3Config
    from quanta_b200.engine.model import write_random_model
    out = {}
    for name, raw in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(MiniMaxM3Config.from_dict(raw), SEEDS[name], d)
        out[name] = d
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """name -> (weights by name, normalised config) as the plain implementation reads them."""
    from safetensors.torch import load_file
    from tests.plain import minimax_m3_plain as P
    return {name: (load_file(str(d / "model.safetensors")), P.read_config(d)) for name, d in model_dirs.items()}
