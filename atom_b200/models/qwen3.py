"""Qwen3 dense (``Qwen3ForCausalLM``): configuration keys and model description.

Structure after atom/models/qwen3.py: decoder layers of grouped-query attention with
per-head q/k RMSNorm and rotary positions (:59-163) and a SiLU-gated feed-forward
(:166-198) in a pre-norm residual arrangement (:201-258), a final norm (:310) and an output
head that may share the embedding table (:333-340).  Checkpoint names and the stacking of
q/k/v and gate/up follow ``packed_modules_mapping`` (:317-323).
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, ClassVar, Dict, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig, cfg_get, cfg_positive
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import register_architecture


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    """Keys of ``Qwen3ForCausalLM`` (dense), as atom/models/qwen3.py reads them.

    hidden_size :215, num_hidden_layers :284, num_attention_heads :216,
    num_key_value_heads :217, head_dim :221 (default hidden/heads :85),
    intermediate_size :231, vocab_size :274, rms_norm_eps :219,
    rope_theta / rope_parameters :213, max_position_embeddings :218,
    attention_bias :220, hidden_act :191, tie_word_embeddings :339.
    ``layer_types`` / ``sliding_window`` follow atom/models/llama.py:187-200: a
    layer named "sliding_attention" attends to the last ``sliding_window`` keys.
    """

    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    max_position_embeddings: int = 0
    attention_bias: bool = False
    hidden_act: str = "silu"
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    sliding_window: Optional[int] = None
    layer_types: Optional[Tuple[str, ...]] = None
    eos_token_id: Tuple[int, ...] = field(default_factory=tuple)
    bos_token_id: Optional[int] = None

    ARCHITECTURE: ClassVar[str] = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        hidden = cfg_positive("hidden_size", cfg_get(d, "hidden_size", int))
        nh = cfg_positive("num_attention_heads", cfg_get(d, "num_attention_heads", int))
        nkv = cfg_positive("num_key_value_heads", cfg_get(d, "num_key_value_heads", int, nh))
        if nh % nkv != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({nh}) must be a multiple of num_key_value_heads ({nkv})"
            )
        if "head_dim" in d and d["head_dim"] is not None:
            hd = cfg_positive("head_dim", cfg_get(d, "head_dim", int))
        else:
            if hidden % nh != 0:
                raise ConfigError(
                    f"config.json: no 'head_dim' and hidden_size ({hidden}) is not a multiple of "
                    f"num_attention_heads ({nh})"
                )
            hd = hidden // nh  # atom/models/qwen3.py:85
        if hd % 2 != 0:
            raise ConfigError(f"config.json: head_dim ({hd}) must be even for rotary embedding")

        # rope: HF >= 5 nests it in rope_parameters; older files have rope_theta / rope_scaling
        # (atom/config.py:1708-1722).
        rope_params = d.get("rope_parameters")
        scaling = d.get("rope_scaling")
        theta = d.get("rope_theta")
        if isinstance(rope_params, dict):
            theta = rope_params.get("rope_theta", theta)
            rtype = rope_params.get("rope_type", rope_params.get("type", "default"))
            if rtype not in (None, "default"):
                raise ConfigError(f"config.json: rope_parameters.rope_type '{rtype}' is not supported")
        if isinstance(scaling, dict):
            rtype = scaling.get("rope_type", scaling.get("type", "default"))
            if rtype not in (None, "default"):
                # atom/model_ops/rotary_embedding.py:139 accepts no scaling either.
                raise ConfigError(f"config.json: rope_scaling type '{rtype}' is not supported")
        if theta is None:
            raise ConfigError("config.json: required key 'rope_theta' is missing")
        if isinstance(theta, bool) or not isinstance(theta, (int, float)) or theta <= 0:
            raise ConfigError(f"config.json: key 'rope_theta' must be a positive number, got {theta!r}")

        act = cfg_get(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (silu only)")

        eps = cfg_get(d, "rms_norm_eps", float)
        if eps <= 0:
            raise ConfigError(f"config.json: key 'rms_norm_eps' must be positive, got {eps}")

        n_layers = cfg_positive("num_hidden_layers", cfg_get(d, "num_hidden_layers", int))
        window = d.get("sliding_window")
        if d.get("use_sliding_window") is False:
            window = None
        layer_types = d.get("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, list) or len(layer_types) != n_layers:
                raise ConfigError(
                    f"config.json: 'layer_types' must list {n_layers} entries (num_hidden_layers)"
                )
            for t in layer_types:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"config.json: layer_types entry '{t}' is not supported")
            if "sliding_attention" in layer_types:
                if not isinstance(window, int) or isinstance(window, bool) or window <= 0:
                    raise ConfigError(
                        "config.json: layer_types names 'sliding_attention' but 'sliding_window' "
                        "is not a positive int"
                    )
            layer_types = tuple(layer_types)
        if layer_types is None and d.get("use_sliding_window") is True and window is not None:
            # The older spelling (a window from layer 'max_window_layers' on) is resolved by the
            # library that reads config.json for the reference, which itself looks at
            # 'layer_types' alone (atom/models/llama.py:187-191).  Running such a file with full
            # attention in every layer would be silently wrong, so it is refused.
            raise ConfigError(
                "config.json: 'use_sliding_window' is true but 'layer_types' is missing; name the layers "
                "that use the window in 'layer_types' ('max_window_layers' alone is not read)"
            )
        if layer_types is None or "sliding_attention" not in layer_types:
            window = None

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("config.json: key 'eos_token_id' must be an int or a list of ints")

        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype not in ("bfloat16", "float32", "float16"):
            raise ConfigError(f"config.json: torch_dtype '{dtype}' is not supported")

        return cls(
            architecture=cls.ARCHITECTURE,
            hidden_size=hidden,
            num_hidden_layers=n_layers,
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=hd,
            intermediate_size=cfg_positive("intermediate_size", cfg_get(d, "intermediate_size", int)),
            vocab_size=cfg_positive("vocab_size", cfg_get(d, "vocab_size", int)),
            rms_norm_eps=eps,
            rope_theta=float(theta),
            max_position_embeddings=cfg_positive(
                "max_position_embeddings", cfg_get(d, "max_position_embeddings", int)
            ),
            attention_bias=cfg_get(d, "attention_bias", bool, False),
            hidden_act=act,
            tie_word_embeddings=cfg_get(d, "tie_word_embeddings", bool),
            torch_dtype=dtype,
            sliding_window=window,
            layer_types=layer_types,
            eos_token_id=eos_ids,
            bos_token_id=d.get("bos_token_id"),
        )

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architectures": [self.architecture], "model_type": "qwen3"}
        for f in fields(self):
            if f.name in ("architecture",):
                continue
            v = getattr(self, f.name)
            if f.name == "eos_token_id":
                v = list(v) if len(v) != 1 else v[0]
                if v == []:
                    v = None
            if f.name == "layer_types" and v is not None:
                v = list(v)
            out[f.name] = v
        out["use_sliding_window"] = self.sliding_window is not None
        return out

    @property
    def eos_token_ids(self) -> Tuple[int, ...]:
        return self.eos_token_id


def build_qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    H, hd = cfg.hidden_size, cfg.head_dim
    position = PartSpec(
        "rope_neox",
        {"rotary_dim": hd, "theta": cfg.rope_theta, "max_position": cfg.max_position_embeddings},
    )
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        window = None
        if cfg.layer_types is not None and cfg.layer_types[i] == "sliding_attention":
            window = cfg.sliding_window
        attn_sources = {
            "qkv.weight": tuple(f"{p}.self_attn.{n}_proj.weight" for n in ("q", "k", "v")),
            "o.weight": (f"{p}.self_attn.o_proj.weight",),
            "q_norm.weight": (f"{p}.self_attn.q_norm.weight",),
            "k_norm.weight": (f"{p}.self_attn.k_norm.weight",),
        }
        if cfg.attention_bias:
            attn_sources["qkv.bias"] = tuple(f"{p}.self_attn.{n}_proj.bias" for n in ("q", "k", "v"))
        mixer = PartSpec(
            "paged_attention",
            {
                "hidden_size": H,
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": hd,
                "position": position,
                "qk_norm": True,
                "norm_eps": cfg.rms_norm_eps,
                "bias": cfg.attention_bias,
                "window": window,
            },
            attn_sources,
        )
        ffn = PartSpec(
            "gated_silu",
            {"hidden_size": H, "intermediate_size": cfg.intermediate_size},
            {
                "gate_up.weight": (f"{p}.mlp.gate_proj.weight", f"{p}.mlp.up_proj.weight"),
                "down.weight": (f"{p}.mlp.down_proj.weight",),
            },
        )
        norm_args = {"size": H, "eps": cfg.rms_norm_eps}
        layers.append(
            LayerSpec("prenorm", {
                "mixer_norm": PartSpec("rmsnorm", norm_args, {"weight": (f"{p}.input_layernorm.weight",)}),
                "mixer": mixer,
                "ffn_norm": PartSpec("rmsnorm", norm_args, {"weight": (f"{p}.post_attention_layernorm.weight",)}),
                "ffn": ffn,
            })
        )
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=H,
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartSpec(
            "token_embedding",
            {"vocab_size": cfg.vocab_size, "hidden_size": H},
            {"weight": ("model.embed_tokens.weight",)},
        ),
        layers=tuple(layers),
        run_order=tuple(RunEntry(layer=i, cache=i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.rms_norm_eps}, {"weight": ("model.norm.weight",)}),
        lm_head=PartSpec(
            "lm_head",
            {"vocab_size": cfg.vocab_size, "hidden_size": H, "tied": cfg.tie_word_embeddings},
            {} if cfg.tie_word_embeddings else {"weight": ("lm_head.weight",)},
        ),
        # atom/model_loader/weight_names.py:171 drops rotary inv_freq buffers.
        ignored_tensors=(r".*rotary_emb\.inv_freq$",),
        # Tied checkpoints often carry the output matrix as well; it must then be the embedding
        # table (the reference aliases the two, atom/models/qwen3.py:339-340).
        duplicate_tensors=(("lm_head.weight", "model.embed_tokens.weight"),) if cfg.tie_word_embeddings else (),
        eos_token_ids=cfg.eos_token_ids,
    )


register_architecture(Qwen3Config.ARCHITECTURE, Qwen3Config.from_dict, build_qwen3_spec)
