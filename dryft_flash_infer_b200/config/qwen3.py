"""Configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

The keys and their defaults follow what the reference engine reads from the
checkpoint's configuration (engine/engine.py:223-234): ``head_dim`` defaults to
``hidden_size // num_attention_heads`` and is otherwise independent of them;
``rope_theta`` must be given (as such, or under ``rope_parameters``).  The reference insists on tied embeddings
(engine/engine.py:233-234); here both tied and untied heads are accepted.
Features of the checkpoint format that the reference engine does not implement
(rope scaling, sliding windows, attention biases, an activation other than SiLU)
are refused by name rather than ignored.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig, take


def _rope_theta(raw: dict[str, Any]) -> float:
    """The rotation base: ``rope_theta``, or ``rope_parameters.rope_theta`` where a newer checkpoint keeps
    it (whose ``rope_type`` must then be the default one).  A file with neither is refused: the reference
    falls back to 5e6 only when the configuration object lacks the attribute (engine/engine.py:230), which
    a file read through its library never does, so a guess here would rotate with a base nobody chose."""
    parameters = raw.get("rope_parameters")
    if isinstance(parameters, dict):
        kind = parameters.get("rope_type", parameters.get("type", "default"))
        if kind not in (None, "default"):
            raise ConfigError(f"config.json: 'rope_parameters.rope_type' = {kind!r} is not supported for "
                              f"Qwen3ForCausalLM (only the default rotation is)")
        if raw.get("rope_theta") is None and parameters.get("rope_theta") is not None:
            return take(parameters, "rope_theta", float)
    if raw.get("rope_theta") is None:
        raise ConfigError("config.json: missing key 'rope_theta' (and no 'rope_parameters.rope_theta')")
    return take(raw, "rope_theta", float)


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"

    architecture: ClassVar[str] = "Qwen3ForCausalLM"
    model_type: ClassVar[str] = "qwen3"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "Qwen3Config":
        hidden = take(raw, "hidden_size", int)
        heads = take(raw, "num_attention_heads", int)
        if heads <= 0:
            raise ConfigError("config.json: 'num_attention_heads' must be positive")
        cfg = cls(
            vocab_size=take(raw, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=take(raw, "intermediate_size", int),
            num_hidden_layers=take(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=take(raw, "num_key_value_heads", int, heads),
            head_dim=take(raw, "head_dim", int, hidden // heads),
            rms_norm_eps=take(raw, "rms_norm_eps", float, 1e-6),
            rope_theta=_rope_theta(raw),
            tie_word_embeddings=take(raw, "tie_word_embeddings", bool, False),
            max_position_embeddings=take(raw, "max_position_embeddings", int, 32768),
            hidden_act=take(raw, "hidden_act", str, "silu"),
            torch_dtype=take(raw, "torch_dtype", str, take(raw, "dtype", str, "bfloat16")),
        )
        scaling = raw.get("rope_scaling")
        if scaling not in (None, {}) and not (isinstance(scaling, dict) and
                                              scaling.get("rope_type", scaling.get("type")) in (None, "default")):
            raise ConfigError("config.json: 'rope_scaling' is not supported for Qwen3ForCausalLM")
        if raw.get("use_sliding_window"):
            raise ConfigError("config.json: 'use_sliding_window' = true is not supported for Qwen3ForCausalLM")
        if raw.get("attention_bias"):
            raise ConfigError("config.json: 'attention_bias' = true is not supported for Qwen3ForCausalLM")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: 'num_attention_heads' ({self.num_attention_heads}) must be a multiple of "
                f"'num_key_value_heads' ({self.num_key_value_heads})")
        if self.head_dim % 16 or self.head_dim > 256:
            raise ConfigError(f"config.json: 'head_dim' must be a multiple of 16 and at most 256 (the attention "
                              f"kernels' head sizes), got {self.head_dim}")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' must be 'silu', got {self.hidden_act!r}")
        if not (self.rms_norm_eps > 0 and self.rope_theta > 0):
            raise ConfigError("config.json: 'rms_norm_eps' and 'rope_theta' must be positive")
