"""Qwen2 dense: the typed configuration and its description as parts.

The reference reads five keys of config.json and hard-codes the rest
(``litelang/models/qwen2/model.py:9-21``; theta ``qwen2/layer/pre_layer.py:22``;
eps ``qwen2/layer/transformer_layer.py:41`` and ``qwen2/layer/post_layer.py:12``).
Here every size and constant that config.json gives is read from it.

Layer structure (``qwen2/layer/transformer_layer.py:46-77``): pre-norm block of
grouped-query attention with q/k/v bias and rotary positions, and a
SiLU-gated feed-forward; RMSNorm before each; final RMSNorm and an lm_head that
is the embedding table when ``tie_word_embeddings``
(``qwen2/layer_weights/post_layer_weights.py:10-15``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.base import ConfigError, ModelConfig, _require, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    hidden_act: str = "silu"
    attention_bias: bool = True
    torch_dtype: str = "bfloat16"
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    initializer_range: float = 0.02

    architecture = "Qwen2ForCausalLM"

    # ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen2Config":
        a = cls.architecture
        hidden = _require(d, "hidden_size", int, a)
        heads = _require(d, "num_attention_heads", int, a)
        kv_heads = _require(d, "num_key_value_heads", int, a)
        if heads <= 0 or kv_heads <= 0 or hidden <= 0:
            raise ConfigError(f"{a}: sizes must be positive")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"{a}: hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                    "and config.json gives no head_dim"
                )
            head_dim = hidden // heads
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=_require(d, "num_hidden_layers", int, a),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            intermediate_size=_require(d, "intermediate_size", int, a),
            vocab_size=_require(d, "vocab_size", int, a),
            head_dim=int(head_dim),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            max_position_embeddings=int(d.get("max_position_embeddings", 32768)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            sliding_window=(None if d.get("sliding_window") is None else int(d["sliding_window"])),
            max_window_layers=int(d.get("max_window_layers", 0) or 0),
            hidden_act=str(d.get("hidden_act", "silu")),
            attention_bias=bool(d.get("attention_bias", True)),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            eos_token_id=eos_ids,
            bos_token_id=(None if d.get("bos_token_id") is None else int(d["bos_token_id"])),
            initializer_range=float(d.get("initializer_range", 0.02)),
        )
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"{a}: rope_scaling {d.get('rope_scaling')!r} is not supported")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        a = self.architecture
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"{a}: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            raise ConfigError(f"{a}: head_dim {self.head_dim} must be even for rotary positions")
        if self.hidden_act != "silu":
            raise ConfigError(f"{a}: hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if self.num_hidden_layers <= 0 or self.intermediate_size <= 0 or self.vocab_size <= 0:
            raise ConfigError(f"{a}: sizes must be positive")
        if self.rms_norm_eps <= 0 or self.rope_theta <= 0:
            raise ConfigError(f"{a}: rms_norm_eps and rope_theta must be positive")
        if self.use_sliding_window and self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError(f"{a}: sliding_window must be positive")

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "torch_dtype": self.torch_dtype,
            "initializer_range": self.initializer_range,
        }
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) > 1 else self.eos_token_id[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    def init_scales(self) -> Dict[str, float]:
        s = self.initializer_range
        return {"matrix": s, "bias": s, "norm": 2.5 * s}

    # ------------------------------------------------------------------
    def window_of_layer(self, layer: int) -> Optional[int]:
        """The last ``sliding_window`` positions (the token's own included) for layers
        from ``max_window_layers`` on, when ``use_sliding_window``; else all positions."""
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        return self.sliding_window if layer >= self.max_window_layers else None

    def model_spec(self) -> ModelSpec:
        norm = {"hidden_size": self.hidden_size, "eps": self.rms_norm_eps}
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            mixer = PartSpec(
                "gqa_attention",
                {
                    "hidden_size": self.hidden_size,
                    "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads,
                    "head_dim": self.head_dim,
                    "qkv_bias": self.attention_bias,
                    "out_bias": False,
                    "scale": self.head_dim ** -0.5,
                    "window": self.window_of_layer(i),
                    "position": PartSpec(
                        "rope_half_split",
                        {
                            "rotary_dim": self.head_dim,
                            "theta": self.rope_theta,
                            "max_positions": self.max_position_embeddings,
                        },
                    ),
                },
                p + "self_attn.",
            )
            ffn = PartSpec(
                "gated_mlp",
                {
                    "hidden_size": self.hidden_size,
                    "intermediate_size": self.intermediate_size,
                    "activation": self.hidden_act,
                },
                p + "mlp.",
            )
            layers.append(
                LayerSpec(
                    block="pre_norm",
                    parts={
                        "mixer": mixer,
                        "feed_forward": ffn,
                        "mixer_norm": PartSpec("rms_norm", norm, p + "input_layernorm."),
                        "feed_forward_norm": PartSpec("rms_norm", norm, p + "post_attention_layernorm."),
                    },
                )
            )
        return ModelSpec(
            architecture=self.architecture,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec(
                "token_embedding",
                {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size},
                "model.embed_tokens.",
            ),
            layers=tuple(layers),
            order=tuple(RunStep(i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rms_norm", norm, "model.norm."),
            head=PartSpec(
                "lm_head",
                {
                    "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size,
                    "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None,
                },
                "lm_head.",
            ),
            eos_token_ids=self.eos_token_id,
        )


register_architecture(Qwen2Config.architecture, Qwen2Config)
