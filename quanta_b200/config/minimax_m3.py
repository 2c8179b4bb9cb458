"""Typed configuration of the MiniMax-M3 text decoder (MiniMax-M2-family layer), from config.json.

Key names, defaults and refusals follow the reference's parsers: the flat M2 schema
(src/quanta/minimax/config.py:136-188) and, when ``text_config`` is present, the same names inside
it with the nested parser's own defaults (src/quanta/minimax/config_m3.py:223-315): ``rotary_dim``
falls back to ``round(head_dim * partial_rotary_factor)``, ``rope_theta`` to 5e6, ``qk_norm_type`` to
``"per_head"``, ``hidden_act`` to ``"swigluoai"`` (which this decoder refuses, so a nested config has to
say ``"silu"``), ``max_position_embeddings`` to 1048576.  eos/bos come from ``generation_config.json``
first, then the config, then 200020 / 200019 (config.py:154-155, 183-185).

Keys that change the layer math of the M3 checkpoints and that this decoder does not build are read
and refused, never ignored: ``use_gemma_norm`` (gains applied as 1 + w), ``attention_output_gate``,
dense layers (a 0 in ``moe_layer_freq``), ``n_shared_experts``, block-sparse attention
(``sparse_attention_config.use_sparse_attention``).

Every size and constant the layers use is a field here; no part reads anything else.
"""

from __future__ import annotations

from dataclasses import dataclass, field, asdict

_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "num_key_value_heads", "head_dim", "num_local_experts",
             "num_experts_per_tok")


class ConfigError(ValueError):
    pass


@dataclass(frozen=True)
class MiniMaxM3Config:
    # sizes (required keys)
    vocab_size: int
    hidden_size: int
    intermediate_size: int            # width of one routed expert
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    num_local_experts: int
    num_experts_per_tok: int
    # attention
    rotary_dim: int                   # rotated dims of each head (first rotary_dim dims)
    rope_theta: float = 1e6
    rope_section: tuple[int, ...] | None = None   # pairs per position axis; sum == rotary_dim/2
    use_qk_norm: bool = False
    qk_norm_type: str = "per_layer"   # "per_layer": over the concatenated heads; "per_head"
    attn_type_list: tuple[int, ...] = ()          # 1 = full softmax attention
    # router / experts
    scoring_func: str = "sigmoid"
    use_routing_bias: bool = True
    norm_topk_prob: bool = True
    routed_scaling_factor: float = 1.0
    shared_intermediate_size: int = 0
    hidden_act: str = "silu"
    # options of the M3 checkpoints that change the math and are refused when set
    use_gemma_norm: bool = False
    attention_output_gate: bool = False
    moe_layer_freq: tuple[int, ...] = ()          # 1 = routed experts; () = every layer
    n_shared_experts: int = 0
    use_sparse_attention: bool = False
    # norms / positions / tokens
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 204800
    tie_word_embeddings: bool = False
    bos_token_id: int = 200019
    eos_token_ids: tuple[int, ...] = (200020,)
    torch_dtype: str = "bfloat16"
    model_type: str = "minimax_m3"
    architectures: tuple[str, ...] = ("MiniMaxM3ForCausalLM",)
    extra: dict = field(default_factory=dict, compare=False)   # keys read but unused by the forward

    # ---- derived geometry (src/quanta/minimax/config.py:88-125) ----
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def attn_scale(self) -> float:
        return self.head_dim ** -0.5

    @property
    def eos_token_id(self) -> int:
        return self.eos_token_ids[0]

    # ---- construction ----
    @classmethod
    def from_dict(cls, raw: dict, generation: dict | None = None) -> "MiniMaxM3Config":
        gen = generation or {}
        nested = isinstance(raw.get("text_config"), dict)
        c = raw["text_config"] if nested else raw
        # the two parsers of the reference differ in what an absent key means
        d_theta, d_norm, d_act, d_maxpos = (5e6, "per_head", "swigluoai", 1048576) if nested else \
                                           (1e6, "per_layer", "silu", 204800)
        missing = [k for k in _REQUIRED if k not in c]
        if missing:
            raise ConfigError(f"config.json lacks required key(s): {', '.join(missing)}")
        n_layers = int(c["num_hidden_layers"])
        attn_types = tuple(int(x) for x in c.get("attn_type_list", [1] * n_layers))
        head_dim = int(c["head_dim"])
        if "rotary_dim" in c:
            rotary_dim = int(c["rotary_dim"])
        else:
            rotary_dim = int(round(head_dim * float(c.get("partial_rotary_factor", 1.0))))
        section = c.get("rope_section", c.get("mrope_section"))
        if section is None:
            for holder in ("rope_scaling", "rope_parameters"):
                if isinstance(c.get(holder), dict) and c[holder].get("mrope_section") is not None:
                    section = c[holder]["mrope_section"]
        eos = gen.get("eos_token_id", c.get("eos_token_id", raw.get("eos_token_id", 200020)))
        eos_ids = tuple(int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos]))
        bos = int(gen.get("bos_token_id", c.get("bos_token_id", raw.get("bos_token_id", 200019))))
        archs = tuple(raw.get("architectures") or ("MiniMaxM3ForCausalLM",))
        extra = {k: c[k] for k in ("use_mtp", "num_mtp_modules", "mtp_transformer_layers",
                                   "quantization_config") if k in c}
        sparse = c.get("sparse_attention_config") or {}
        cfg = cls(
            vocab_size=int(c["vocab_size"]), hidden_size=int(c["hidden_size"]),
            intermediate_size=int(c["intermediate_size"]), num_hidden_layers=n_layers,
            num_attention_heads=int(c["num_attention_heads"]),
            num_key_value_heads=int(c["num_key_value_heads"]), head_dim=head_dim,
            num_local_experts=int(c["num_local_experts"]),
            num_experts_per_tok=int(c["num_experts_per_tok"]),
            rotary_dim=rotary_dim, rope_theta=float(c.get("rope_theta", d_theta)),
            rope_section=None if section is None else tuple(int(x) for x in section),
            use_qk_norm=bool(c.get("use_qk_norm", False)),
            qk_norm_type=str(c.get("qk_norm_type", d_norm)),
            attn_type_list=attn_types,
            scoring_func=str(c.get("scoring_func", "sigmoid")),
            use_routing_bias=bool(c.get("use_routing_bias", True)),
            norm_topk_prob=bool(c.get("norm_topk_prob", True)),
            routed_scaling_factor=float(c.get("routed_scaling_factor", 1.0)),
            shared_intermediate_size=int(c.get("shared_intermediate_size", 0)),
            hidden_act=str(c.get("hidden_act", d_act)),
            use_gemma_norm=bool(c.get("use_gemma_norm", False)),
            attention_output_gate=bool(c.get("attention_output_gate", False)),
            moe_layer_freq=tuple(int(x) for x in c.get("moe_layer_freq", ())),
            n_shared_experts=int(c.get("n_shared_experts", 0)),
            use_sparse_attention=bool(sparse.get("use_sparse_attention", False)),
            rms_norm_eps=float(c.get("rms_norm_eps", 1e-6)),
            max_position_embeddings=int(c.get("max_position_embeddings", d_maxpos)),
            tie_word_embeddings=bool(c.get("tie_word_embeddings", raw.get("tie_word_embeddings", False))),
            bos_token_id=bos, eos_token_ids=eos_ids,
            torch_dtype=str(c.get("torch_dtype", raw.get("torch_dtype", "bfloat16"))),
            model_type=str(raw.get("model_type", "minimax_m3")),
            architectures=archs, extra=extra,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        """Refuse what the layers cannot run, before anything is allocated."""
        errs = []
        n = self.num_hidden_layers
        for name in _REQUIRED:
            if getattr(self, name) <= 0:
                errs.append(f"{name} must be positive, got {getattr(self, name)}")
        if len(self.attn_type_list) != n:
            errs.append(f"attn_type_list length {len(self.attn_type_list)} != num_hidden_layers {n}")
        elif any(t != 1 for t in self.attn_type_list):
            bad = [i for i, t in enumerate(self.attn_type_list) if t != 1]
            errs.append(f"attn_type_list marks layers {bad[:8]} as not full softmax attention "
                        f"(only type 1 is implemented)")
        if self.num_key_value_heads > 0 and self.num_attention_heads % self.num_key_value_heads:
            errs.append(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                        f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 16 or self.head_dim > 256:
            errs.append(f"head_dim {self.head_dim} must be a multiple of 16, at most 256")
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            errs.append(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        if self.rope_section is not None and sum(self.rope_section) != self.rotary_dim // 2:
            errs.append(f"rope_section {list(self.rope_section)} sums to {sum(self.rope_section)}, "
                        f"not rotary_dim/2 = {self.rotary_dim // 2}")
        if self.qk_norm_type not in ("per_layer", "per_head"):
            errs.append(f"qk_norm_type {self.qk_norm_type!r} is neither 'per_layer' nor 'per_head'")
        if self.scoring_func != "sigmoid":
            errs.append(f"scoring_func {self.scoring_func!r}: only 'sigmoid' is implemented")
        if self.hidden_act != "silu":
            errs.append(f"hidden_act {self.hidden_act!r}: only 'silu' is implemented")
        if self.shared_intermediate_size != 0:
            errs.append(f"shared_intermediate_size {self.shared_intermediate_size}: this decoder has "
                        f"no shared expert")
        if self.use_gemma_norm:
            errs.append("use_gemma_norm: norms whose gain is stored as w and applied as 1 + w are not implemented")
        if self.attention_output_gate:
            errs.append("attention_output_gate: a gated attention output is not implemented")
        if self.moe_layer_freq and len(self.moe_layer_freq) != n:
            errs.append(f"moe_layer_freq length {len(self.moe_layer_freq)} != num_hidden_layers {n}")
        elif any(f != 1 for f in self.moe_layer_freq):
            bad = [i for i, f in enumerate(self.moe_layer_freq) if f != 1]
            errs.append(f"moe_layer_freq marks layers {bad[:8]} as dense feed-forward layers "
                        f"(only routed-expert layers are implemented)")
        if self.n_shared_experts > 0:
            errs.append(f"n_shared_experts {self.n_shared_experts}: this decoder has no shared expert")
        if self.use_sparse_attention:
            errs.append("sparse_attention_config.use_sparse_attention: block-sparse attention is not implemented")
        if self.num_experts_per_tok > self.num_local_experts:
            errs.append(f"num_experts_per_tok {self.num_experts_per_tok} > num_local_experts "
                        f"{self.num_local_experts}")
        if self.rms_norm_eps <= 0:
            errs.append(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if errs:
            raise ConfigError("invalid MiniMax-M3 configuration: " + "; ".join(errs))

    def to_dict(self) -> dict:
        """The config.json dictionary that ``from_dict`` reads back to an equal configuration."""
        d = asdict(self)
        d.pop("extra")
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = list(eos) if len(eos) > 1 else eos[0]
        d["attn_type_list"] = list(self.attn_type_list)
        d["architectures"] = list(self.architectures)
        for k in ("use_gemma_norm", "attention_output_gate", "n_shared_experts"):
            if not d[k]:
                d.pop(k)
        d.pop("use_sparse_attention")
        if self.use_sparse_attention:
            d["sparse_attention_config"] = {"use_sparse_attention": True}
        if self.moe_layer_freq:
            d["moe_layer_freq"] = list(self.moe_layer_freq)
        else:
            d.pop("moe_layer_freq")
        if self.rope_section is None:
            d.pop("rope_section")
        else:
            d["rope_section"] = list(self.rope_section)
        d.update(self.extra)
        return d
