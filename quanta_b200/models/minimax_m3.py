"""MiniMax-M3 text decoder: from its configuration to a model specification.

Every layer is the same arrangement (src/quanta/minimax/model.py:36-73): RMSNorm -> grouped-query
softmax attention with q/k RMSNorm and partial rotary -> RMSNorm -> sigmoid-routed SwiGLU experts.
Checkpoint names follow the flat M2 schema (src/quanta/minimax/loader.py:27-37, 51-53, 188-233); the
nested M3 files carry the same names under ``language_model.`` (src/quanta/minimax/loader_m3.py:23-27)
beside vision tensors that this decoder skips.
"""

from __future__ import annotations

from ..config.minimax_m3 import MiniMaxM3Config
from ..config.registry import register_architecture
from ..parts.spec import ModelSpec


def layer_choice(cfg: MiniMaxM3Config, i: int) -> tuple[str, dict]:
    p = f"model.layers.{i}."
    a, m = p + "self_attn.", p + "block_sparse_moe."
    position = ("partial_rotary", dict(head_dim=cfg.head_dim, rotary_dim=cfg.rotary_dim, theta=cfg.rope_theta,
                                       sections=cfg.rope_section))
    names = {"q": a + "q_proj.weight", "k": a + "k_proj.weight", "v": a + "v_proj.weight",
             "o": a + "o_proj.weight", "q_norm": a + "q_norm.weight", "k_norm": a + "k_norm.weight"}
    mixer = ("gqa_attention", dict(
        hidden_size=cfg.hidden_size, n_q_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim, scale=cfg.attn_scale, position=position,
        qk_norm=cfg.qk_norm_type if cfg.use_qk_norm else None, qk_norm_eps=cfg.rms_norm_eps, names=names))
    ffn = ("sigmoid_topk_experts", dict(
        hidden_size=cfg.hidden_size, expert_size=cfg.intermediate_size, n_experts=cfg.num_local_experts,
        top_k=cfg.num_experts_per_tok, use_bias=cfg.use_routing_bias, renormalize=cfg.norm_topk_prob,
        scaling=cfg.routed_scaling_factor,
        names={"gate": m + "gate.weight", "bias": m + "e_score_correction_bias",
               "w1": m + "experts.{e}.w1.weight", "w2": m + "experts.{e}.w2.weight",
               "w3": m + "experts.{e}.w3.weight"}))
    norm = lambda n: ("rms_norm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps, weight_name=p + n))  # noqa: E731
    return ("pre_norm", dict(hidden_size=cfg.hidden_size, mixer=mixer, feed_forward=ffn,
                             mixer_norm=norm("input_layernorm.weight"),
                             feed_forward_norm=norm("post_attention_layernorm.weight")))


def build_spec(cfg: MiniMaxM3Config) -> ModelSpec:
    return ModelSpec(
        name="MiniMax-M3",
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        embedding_name="model.embed_tokens.weight",
        layers=[layer_choice(cfg, i) for i in range(cfg.num_hidden_layers)],
        final_norm=("rms_norm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps, weight_name="model.norm.weight")),
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        tied_head=cfg.tie_word_embeddings,
        ignored_prefixes=("vision_tower.", "multi_modal_projector.", "patch_merge_mlp.", "mtp.", "model.mtp."),
        name_aliases=(("language_model.", ""),),
    )


ARCHITECTURE = register_architecture(
    ["MiniMaxM3ForCausalLM", "MiniMaxM2ForCausalLM", "MiniMaxM3VLForConditionalGeneration",
     "minimax_m3", "minimax_m2", "minimax_m3_vl", "minimax"],
    MiniMaxM3Config, build_spec)
