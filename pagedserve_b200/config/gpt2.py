"""Typed GPT-2 configuration read from the architecture's own config.json keys.

The reference builds its ``TransformerConfig`` from a loaded Hugging Face
object (reference: src/model/gpt2.py:32-44, src/model/paged_decoder.py:29-41).
Here the same mapping starts from the JSON text, and keys that would change
the math if set away from their plain value are refused instead of ignored
(reference: src/model/gpt2.py:23-30 refuses cross-attention and non-tanh GELU).
"""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Optional

from pagedserve_b200.config.registry import ConfigError, ModelConfig

# activation_function value -> the engine's activation name
_ACTIVATIONS = {
    "gelu_new": "gelu_tanh",           # reference: src/model/gpt2.py:27-30,40
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu": "gelu_erf",                # reference: src/model/paged_decoder.py:273-277
}

# Keys whose non-default value changes the forward pass: refuse loudly.
_MUST_BE_FALSE = (
    "add_cross_attention",             # reference: src/model/gpt2.py:25-26
    "scale_attn_by_inverse_layer_idx",
)


@dataclass
class GPT2Config(ModelConfig):
    n_layer: int = 12
    n_embd: int = 768
    n_head: int = 12
    n_inner: Optional[int] = None      # None => 4 * n_embd (reference: src/model/gpt2.py:38)
    n_positions: int = 1024
    vocab_size: int = 50257
    layer_norm_epsilon: float = 1e-5
    activation_function: str = "gelu_new"
    tie_word_embeddings: bool = True

    def __post_init__(self):
        for name in ("n_layer", "n_embd", "n_head", "n_positions", "vocab_size"):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                raise ConfigError(f"GPT2Config.{name} must be a positive integer, got {value!r}")
        if self.n_inner is not None and (not isinstance(self.n_inner, int) or self.n_inner <= 0):
            raise ConfigError(f"GPT2Config.n_inner must be a positive integer or null, got {self.n_inner!r}")
        if self.n_embd % self.n_head != 0:
            # reference: src/model/gpt2.py:23-24
            raise ConfigError(
                f"n_embd ({self.n_embd}) must be divisible by n_head ({self.n_head})"
            )
        if self.activation_function not in _ACTIVATIONS:
            raise ConfigError(
                f"unsupported activation_function {self.activation_function!r}; "
                f"supported: {sorted(_ACTIVATIONS)}"
            )
        if not (isinstance(self.layer_norm_epsilon, float) and self.layer_norm_epsilon > 0):
            raise ConfigError("layer_norm_epsilon must be a positive float")

    # ---- derived sizes -------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner_dim(self) -> int:
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    @property
    def activation(self) -> str:
        return _ACTIVATIONS[self.activation_function]

    # ---- ModelConfig interface ----------------------------------------
    @property
    def architecture(self) -> str:
        return "GPT2LMHeadModel"

    @property
    def vocabulary_size(self) -> int:
        return self.vocab_size

    @property
    def max_model_len(self) -> int:
        # learned absolute positions bound the context
        # (reference: src/model/paged_decoder.py:318-319, 521-522)
        return self.n_positions

    @classmethod
    def from_dict(cls, values: dict) -> "GPT2Config":
        for key in _MUST_BE_FALSE:
            if values.get(key, False):
                raise ConfigError(f"config.json sets {key}=true, which this engine does not compute")
        if values.get("scale_attn_weights", True) is not True:
            raise ConfigError("config.json sets scale_attn_weights=false, which this engine does not compute")
        known = {f.name for f in fields(cls)}
        picked = {key: values[key] for key in known if key in values}
        if "layer_norm_epsilon" in picked:
            picked["layer_norm_epsilon"] = float(picked["layer_norm_epsilon"])
        if "n_ctx" in values and "n_positions" in values and values["n_ctx"] != values["n_positions"]:
            raise ConfigError("config.json has n_ctx != n_positions")
        return cls(**picked)

    def to_dict(self) -> dict:
        return {
            "architectures": [self.architecture],
            "model_type": "gpt2",
            "n_layer": self.n_layer,
            "n_embd": self.n_embd,
            "n_head": self.n_head,
            "n_inner": self.n_inner,
            "n_positions": self.n_positions,
            "n_ctx": self.n_positions,
            "vocab_size": self.vocab_size,
            "layer_norm_epsilon": self.layer_norm_epsilon,
            "activation_function": self.activation_function,
            "tie_word_embeddings": self.tie_word_embeddings,
        }


# Named layer sizes used by the command line and the benchmark (random weights).
NAMED_CONFIGS = {
    "tiny-a": dict(n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
                   layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "tiny-b": dict(n_layer=3, n_embd=96, n_head=2, n_inner=320, vocab_size=1000, n_positions=256,
                   layer_norm_epsilon=1e-6, activation_function="gelu"),
    "gpt2-124m": dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257,
                      n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "gpt2-345m": dict(n_layer=24, n_embd=1024, n_head=16, n_inner=4096, vocab_size=50257,
                      n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "gpt2-1.5b": dict(n_layer=48, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257,
                      n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
}


def named_config(name: str) -> GPT2Config:
    if name not in NAMED_CONFIGS:
        raise ConfigError(f"unknown named configuration {name!r}; known: {sorted(NAMED_CONFIGS)}")
    return GPT2Config(**NAMED_CONFIGS[name])
