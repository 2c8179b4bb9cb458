"""Configuration and weight loading on the CPU: keys, defaults, refusals, the registry, and the one
error that lists missing and unexpected tensors and wrong shapes."""

import json

import pytest
import torch

from quanta_b200.config import ConfigError, MiniMaxM3Config, known_architectures, load_config, resolve
from quanta_b200.engine.model import Model, write_random_model
from quanta_b200.weights import FolderSource, WeightError, write_safetensors
from quanta_b200.weights.safetensors_io import CheckpointFolder
from tests.conftest import TINY


def test_required_keys_and_defaults():
    raw = dict(vocab_size=10, hidden_size=32, intermediate_size=16, num_hidden_layers=2, num_attention_heads=2,
               num_key_value_heads=1, head_dim=16, num_local_experts=4, num_experts_per_tok=2)
    c = MiniMaxM3Config.from_dict(raw)
    # defaults of the flat parser
    assert c.rotary_dim == 16 and c.rope_theta == 1e6 and not c.use_qk_norm and c.qk_norm_type == "per_layer"
    assert c.use_routing_bias and c.norm_topk_prob and c.routed_scaling_factor == 1.0
    assert c.rms_norm_eps == 1e-6 and not c.tie_word_embeddings and c.attn_type_list == (1, 1)
    assert c.eos_token_ids == (200020,) and c.bos_token_id == 200019
    assert c.q_dim == 32 and c.kv_dim == 16 and c.group_size == 2 and c.attn_scale == 16 ** -0.5
    for k in raw:
        broken = dict(raw)
        del broken[k]
        with pytest.raises(ConfigError, match=k):
            MiniMaxM3Config.from_dict(broken)


def test_nested_text_config_and_generation_config():
    raw = {"architectures": ["MiniMaxM3ForCausalLM"], "text_config": dict(TINY["C"], hidden_act="silu"),
           "eos_token_id": 5}
    c = MiniMaxM3Config.from_dict(raw, generation={"eos_token_id": [7, 8], "bos_token_id": 3})
    assert c.rotary_dim == 24            # round(48 * 0.5)
    assert c.eos_token_ids == (7, 8) and c.bos_token_id == 3
    assert c.rope_section == (4, 4, 4)


def test_nested_defaults_are_the_nested_parsers():
    """Inside ``text_config`` an absent key means what the reference's M3 parser says
    (src/quanta/minimax/config_m3.py:280-303), not what the flat parser says."""
    tc = dict(vocab_size=10, hidden_size=32, intermediate_size=16, num_hidden_layers=2, num_attention_heads=2,
              num_key_value_heads=1, head_dim=16, num_local_experts=4, num_experts_per_tok=2)
    with pytest.raises(ConfigError, match="swigluoai"):         # the nested default activation is not built
        MiniMaxM3Config.from_dict({"text_config": dict(tc)})
    c = MiniMaxM3Config.from_dict({"text_config": dict(tc, hidden_act="silu", use_qk_norm=True)})
    assert c.qk_norm_type == "per_head" and c.rope_theta == 5e6 and c.max_position_embeddings == 1048576
    flat = MiniMaxM3Config.from_dict(dict(tc, use_qk_norm=True))
    assert flat.qk_norm_type == "per_layer" and flat.rope_theta == 1e6 and flat.max_position_embeddings == 204800
    assert MiniMaxM3Config.from_dict(c.to_dict()) == c


@pytest.mark.parametrize("change, word", [
    ({"use_gemma_norm": True}, "use_gemma_norm"), ({"attention_output_gate": True}, "attention_output_gate"),
    ({"moe_layer_freq": [0, 1]}, "dense feed-forward"), ({"moe_layer_freq": [1]}, "moe_layer_freq length"),
    ({"n_shared_experts": 1}, "shared expert"),
    ({"sparse_attention_config": {"use_sparse_attention": True}}, "block-sparse"),
])
def test_options_that_change_the_math_are_refused(change, word):
    """Flat or nested: a key that the M3 checkpoints use to switch the layer math is never ignored."""
    for nested in (False, True):
        body = dict(TINY["A"], hidden_act="silu")
        body.update(change)
        raw = {"architectures": ["MiniMaxM3VLForConditionalGeneration"], "text_config": body} if nested else body
        with pytest.raises(ConfigError, match=word):
            MiniMaxM3Config.from_dict(raw)
    ok = dict(TINY["A"], moe_layer_freq=[1, 1], n_shared_experts=0, use_gemma_norm=False,
              sparse_attention_config={"use_sparse_attention": False})
    c = MiniMaxM3Config.from_dict(ok)
    assert MiniMaxM3Config.from_dict(c.to_dict()) == c


def test_nested_config_matches_reference_m3_parser(tmp_path):
    """Field by field against the reference's nested parser, when its sources are present."""
    import importlib.util
    import os
    import pathlib
    import sys
    root = pathlib.Path(os.environ.get("QUANTA_REFERENCE_DIR") or pathlib.Path(__file__).resolve().parents[2] / "reference")
    ref = root / "src" / "quanta" / "minimax" / "config_m3.py"
    if not ref.exists():
        pytest.skip("reference sources not present")
    spec = importlib.util.spec_from_file_location("ref_minimax_config_m3", ref)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_minimax_config_m3"] = mod
    try:
        spec.loader.exec_module(mod)
    except ImportError as e:
        pytest.skip(f"the reference's nested parser does not import here: {e}")
    tc = dict(vocab_size=300, hidden_size=64, intermediate_size=24, num_hidden_layers=3, num_attention_heads=4,
              num_key_value_heads=2, head_dim=32, partial_rotary_factor=0.5, num_local_experts=6,
              num_experts_per_tok=2, hidden_act="silu", use_qk_norm=True)
    raw = {"architectures": ["MiniMaxM3VLForConditionalGeneration"], "model_type": "minimax_m3_vl", "text_config": tc}
    (tmp_path / "config.json").write_text(json.dumps(raw))
    theirs = mod.MiniMaxM3Config.from_pretrained(tmp_path)
    ours = MiniMaxM3Config.from_dict(raw)
    pairs = [("vocab_size", "vocab_size"), ("hidden_size", "hidden_size"), ("intermediate_size", "moe_intermediate_size"),
             ("num_hidden_layers", "num_hidden_layers"), ("head_dim", "head_dim"), ("rotary_dim", "rotary_dim"),
             ("use_qk_norm", "use_qk_norm"), ("qk_norm_type", "qk_norm_type"), ("rope_theta", "rope_theta"),
             ("use_gemma_norm", "use_gemma_norm"), ("attention_output_gate", "attention_output_gate"),
             ("n_shared_experts", "n_shared_experts"), ("use_sparse_attention", "use_sparse_attention"),
             ("hidden_act", "hidden_act"), ("norm_topk_prob", "norm_topk_prob"), ("use_routing_bias", "use_routing_bias"),
             ("routed_scaling_factor", "routed_scaling_factor"), ("rms_norm_eps", "norm_eps"),
             ("max_position_embeddings", "max_position_embeddings"), ("eos_token_ids", "eos_token_ids"),
             ("tie_word_embeddings", "tie_word_embeddings")]
    for mine, their in pairs:
        assert getattr(ours, mine) == getattr(theirs, their), mine
    assert theirs.moe_layer_freq == (1, 1, 1) and ours.moe_layer_freq == ()     # absent: every layer routed


@pytest.mark.parametrize("change, word", [
    ({"attn_type_list": [1]}, "attn_type_list"), ({"attn_type_list": [1, 0]}, "full softmax"),
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 24}, "head_dim"), ({"rotary_dim": 7}, "rotary_dim"),
    ({"rotary_dim": 32}, "rotary_dim"), ({"rope_section": [1, 2]}, "rope_section"),
    ({"qk_norm_type": "both"}, "qk_norm_type"), ({"scoring_func": "softmax"}, "scoring_func"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"shared_intermediate_size": 8}, "shared"),
    ({"num_experts_per_tok": 9}, "num_experts_per_tok"), ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_refusals(change, word):
    raw = dict(TINY["A"])
    raw.update(change)
    with pytest.raises(ConfigError, match=word):
        MiniMaxM3Config.from_dict(raw)


def test_round_trip_and_registry(tmp_path):
    for name, raw in TINY.items():
        c = MiniMaxM3Config.from_dict(raw)
        assert MiniMaxM3Config.from_dict(c.to_dict()) == c
        assert resolve(raw).name == "MiniMaxM3ForCausalLM"
    assert "minimax_m3" in known_architectures()
    with pytest.raises(KeyError, match="known"):
        resolve({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    (tmp_path / "config.json").write_text(json.dumps(TINY["B"]))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 42}))
    arch, cfg = load_config(tmp_path)
    assert cfg.eos_token_ids == (42,) and cfg.tie_word_embeddings


def test_config_matches_reference_parser(tmp_path):
    """Field by field against the reference's own pure-Python parser, when its sources are present."""
    import importlib.util
    import pathlib
    import os
    # the checkout of the reference: QUANTA_REFERENCE_DIR, or a "reference" folder beside this repository
    root = pathlib.Path(os.environ.get("QUANTA_REFERENCE_DIR") or pathlib.Path(__file__).resolve().parents[2] / "reference")
    ref = root / "src" / "quanta" / "minimax" / "config.py"
    if not ref.exists():
        pytest.skip("reference sources not present")
    spec = importlib.util.spec_from_file_location("ref_minimax_config", ref)
    mod = importlib.util.module_from_spec(spec)
    import sys
    sys.modules["ref_minimax_config"] = mod
    spec.loader.exec_module(mod)
    for name in ("A", "B"):
        raw = dict(TINY[name])
        (tmp_path / "config.json").write_text(json.dumps(raw))
        theirs = mod.MiniMaxConfig.from_pretrained(tmp_path)
        ours = MiniMaxM3Config.from_dict(raw)
        pairs = [("vocab_size", "vocab_size"), ("hidden_size", "hidden_size"), ("intermediate_size", "moe_intermediate_size"),
                 ("num_hidden_layers", "num_hidden_layers"), ("num_attention_heads", "num_attention_heads"),
                 ("num_key_value_heads", "num_key_value_heads"), ("head_dim", "head_dim"), ("rotary_dim", "rotary_dim"),
                 ("use_qk_norm", "use_qk_norm"), ("qk_norm_type", "qk_norm_type"), ("attn_type_list", "attn_type_list"),
                 ("num_local_experts", "num_local_experts"), ("num_experts_per_tok", "num_experts_per_tok"),
                 ("use_routing_bias", "use_routing_bias"), ("norm_topk_prob", "norm_topk_prob"),
                 ("routed_scaling_factor", "routed_scaling_factor"), ("rms_norm_eps", "norm_eps"),
                 ("rope_theta", "rope_theta"), ("tie_word_embeddings", "tie_word_embeddings"),
                 ("eos_token_ids", "eos_token_ids"), ("attn_scale", "attn_scale"), ("q_dim", "q_dim"), ("kv_dim", "kv_dim")]
        for mine, their in pairs:
            assert getattr(ours, mine) == getattr(theirs, their), (name, mine)


# ---- weights ----------------------------------------------------------------------------------------
def _cpu_model(raw):
    from quanta_b200 import models  # noqa: F401
    cfg = MiniMaxM3Config.from_dict(raw)
    return Model(resolve(raw).build_spec(cfg), dtype=torch.float32, device="cpu"), cfg


def test_random_weights_folder_and_own_reader(model_dirs):
    from safetensors.torch import load_file
    for name, d in model_dirs.items():
        assert (d / "config.json").exists() and (d / "model.safetensors").exists()
        theirs = load_file(str(d / "model.safetensors"))         # the library reads what our writer wrote
        ours = CheckpointFolder(d)
        assert set(ours.names()) == set(theirs)
        for n in list(theirs)[:20]:
            assert torch.equal(ours.read(n), theirs[n])
        model, _ = _cpu_model(TINY[name])
        specs = {s.name: s for s in model.tensor_specs()}
        assert set(specs) == set(theirs)
        gate = next(n for n in theirs if n.endswith("gate.weight"))
        assert theirs[gate].dtype == torch.float32                # the router gate is stored in 32-bit
        assert theirs["model.embed_tokens.weight"].dtype == torch.bfloat16
        if TINY[name].get("tie_word_embeddings"):
            assert "lm_head.weight" not in theirs


def test_same_seed_same_weights_any_order(tmp_path):
    from safetensors.torch import load_file
    cfg = MiniMaxM3Config.from_dict(TINY["A"])
    a = load_file(str(write_random_model(cfg, 5, tmp_path / "a") / "model.safetensors"))
    b = load_file(str(write_random_model(cfg, 5, tmp_path / "b") / "model.safetensors"))
    c = load_file(str(write_random_model(cfg, 6, tmp_path / "c") / "model.safetensors"))
    assert all(torch.equal(a[n], b[n]) for n in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    g = a["model.norm.weight"]
    assert float(g.min()) >= 0.9 and float(g.max()) <= 1.1
    bias = a["model.layers.0.block_sparse_moe.e_score_correction_bias"]
    assert float(bias.abs().max()) <= 0.05
    assert abs(float(a["model.embed_tokens.weight"].float().std()) - 0.02) < 0.004


def test_one_error_lists_missing_unexpected_and_wrong_shape(model_dirs, tmp_path):
    from safetensors.torch import load_file
    w = load_file(str(model_dirs["A"] / "model.safetensors"))
    del w["model.layers.1.self_attn.o_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.extra_thing.weight"] = torch.zeros(3)
    w["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16)        # per-head length under per_layer
    w["model.layers.0.block_sparse_moe.experts.3.w2.weight"] = torch.zeros(32, 64, dtype=torch.bfloat16)
    write_safetensors(tmp_path / "model.safetensors", w)
    (tmp_path / "config.json").write_text((model_dirs["A"] / "config.json").read_text())
    model, _ = _cpu_model(TINY["A"])
    with pytest.raises(WeightError) as e:
        model.load(FolderSource(tmp_path))
    msg = str(e.value)
    assert "2 missing" in msg and "model.norm.weight" in msg and "o_proj" in msg
    assert "1 unexpected" in msg and "extra_thing" in msg
    assert "2 tensor(s) of the wrong shape" in msg and "q_norm" in msg and "experts.3.w2" in msg


def test_nested_names_and_other_towers_are_accepted(model_dirs, tmp_path):
    from safetensors.torch import load_file
    w = load_file(str(model_dirs["C"] / "model.safetensors"))
    nested = {"language_model." + n: t for n, t in w.items()}
    nested["vision_tower.blocks.0.weight"] = torch.zeros(4)
    write_safetensors(tmp_path / "model.safetensors", nested)
    (tmp_path / "config.json").write_text((model_dirs["C"] / "config.json").read_text())
    model, _ = _cpu_model(TINY["C"])
    model.load(FolderSource(tmp_path))
    assert model.loaded
    assert model.blocks[0].mixer.w_qkv.shape == ((6 + 2 * 3) * 48, 72)
    assert model.blocks[0].feed_forward.w13.shape == (12, 80, 72)


def test_quantized_checkpoint_is_refused(model_dirs, tmp_path):
    from safetensors.torch import load_file
    w = load_file(str(model_dirs["A"] / "model.safetensors"))
    w["model.layers.0.self_attn.q_proj.weight_scale_inv"] = torch.ones(1, 1)
    write_safetensors(tmp_path / "model.safetensors", w)
    model, _ = _cpu_model(TINY["A"])
    with pytest.raises(WeightError, match="quantized"):
        model.load(FolderSource(tmp_path))


def test_dtypes_kept(model_dirs):
    model, _ = _cpu_model(TINY["A"])
    model.dtype = torch.bfloat16
    model.load(FolderSource(model_dirs["A"]))
    assert model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    assert model.blocks[0].feed_forward.gate_w.dtype == torch.float32      # stored in 32-bit, stays so
    assert model.blocks[0].mixer_norm.weight.dtype == torch.float32


def test_sharded_folder_with_an_index(model_dirs, tmp_path):
    """Two shards and ``model.safetensors.index.json`` (how real checkpoints come,
    src/quanta/minimax/loader.py:96-134) load to the same tensors as the single file; an index that names
    a shard which is not there, or a tensor its shard does not hold, is one clear error."""
    from safetensors.torch import load_file
    src = model_dirs["A"]
    tensors = load_file(str(src / "model.safetensors"))
    names = sorted(tensors)
    halves = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    (tmp_path / "config.json").write_text((src / "config.json").read_text())
    for fn, part in halves.items():
        write_safetensors(tmp_path / fn, {n: tensors[n] for n in part})
    index = {"metadata": {"total_size": 0}, "weight_map": {n: fn for fn, part in halves.items() for n in part}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    folder = CheckpointFolder(tmp_path)
    assert sorted(folder.names()) == names
    folder.close()
    whole, _ = _cpu_model(TINY["A"])
    whole.load(FolderSource(src))
    sharded, _ = _cpu_model(TINY["A"])
    sharded.load(FolderSource(tmp_path))
    a = whole.blocks[1].feed_forward
    b = sharded.blocks[1].feed_forward
    assert torch.equal(a.w13, b.w13) and torch.equal(a.w2, b.w2) and torch.equal(a.gate_w, b.gate_w)
    assert torch.equal(whole.head.weight, sharded.head.weight)
    (tmp_path / "model-00002-of-00002.safetensors").rename(tmp_path / "elsewhere.safetensors")
    with pytest.raises(FileNotFoundError, match="model-00002-of-00002.safetensors"):
        FolderSource(tmp_path)
    (tmp_path / "elsewhere.safetensors").rename(tmp_path / "model-00002-of-00002.safetensors")
    index["weight_map"][names[0]] = "model-00002-of-00002.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    import re
    with pytest.raises(ValueError, match=re.escape(names[0])):
        FolderSource(tmp_path)
