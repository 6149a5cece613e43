"""GPT-2 as a ModelSpec: dense pre-LayerNorm decoder with learned positions.

Follows ``PagedDecoderLM`` as configured by ``convert_gpt2_model``
(reference: src/model/paged_decoder.py:284-301, src/model/gpt2.py:20-80):
per block LN -> packed QKV -> causal attention -> output projection + residual ->
LN -> c_fc -> GELU -> c_proj + residual; final LN; LM head tied to the token
table, no bias.  Tensor names are the checkpoint's own; the four projections are
stored ``[in, out]`` ("Conv1D", reference: src/model/gpt2.py:14-17).
"""

from __future__ import annotations

import math
import re
from typing import Optional

from pagedserve_b200.config.gpt2 import GPT2Config
from pagedserve_b200.config.registry import register_architecture
from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec

_BUFFER = re.compile(r"^h\.\d+\.attn\.(bias|masked_bias)$")


def _normalise_name(name: str) -> Optional[str]:
    """Accept names with or without the ``transformer.`` prefix; skip mask buffers."""
    if name.startswith("transformer."):
        name = name[len("transformer."):]
    if _BUFFER.match(name):
        return None
    return name


def _checkpoint_name(name: str) -> str:
    return name if name.startswith("lm_head.") else "transformer." + name


def build_gpt2_spec(config: GPT2Config) -> ModelSpec:
    hidden, heads, head_dim = config.n_embd, config.n_head, config.head_dim
    std = 0.02
    out_std = 0.02 / math.sqrt(2 * config.n_layer)
    norm = dict(width=hidden, eps=config.layer_norm_epsilon, has_mean=True, has_bias=True, init_std=std)
    layers = []
    for index in range(config.n_layer):
        prefix = f"h.{index}."
        layers.append(LayerSpec(
            block=PartSpec("pre_norm"),
            mixer=PartSpec("causal_attention", dict(
                hidden_size=hidden, n_heads=heads, n_kv_heads=heads, head_dim=head_dim,
                scale=head_dim ** -0.5,            # reference: src/model/paged_attention.py:27
                window=None, has_bias=True, stored_in_out=True,
                qkv_name="attn.c_attn", out_name="attn.c_proj",
                init_std=std, out_init_std=out_std), prefix),
            feed_forward=PartSpec("dense_mlp", dict(
                hidden_size=hidden, inner_size=config.inner_dim, activation=config.activation,
                has_bias=True, stored_in_out=True, up_name="mlp.c_fc", down_name="mlp.c_proj",
                init_std=std, out_init_std=out_std), prefix),
            norms={
                "pre_mixer": PartSpec("layernorm", dict(norm, name="ln_1"), prefix),
                "pre_feed_forward": PartSpec("layernorm", dict(norm, name="ln_2"), prefix),
            },
        ))
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=hidden,
        vocab_size=config.vocab_size,
        max_model_len=config.n_positions,
        embedding=PartSpec("token_embedding", dict(vocab_size=config.vocab_size, hidden_size=hidden,
                                                   name="wte", init_std=std)),
        positions=PartSpec("learned_absolute", dict(max_positions=config.n_positions, hidden_size=hidden,
                                                    name="wpe", init_std=std)),
        layers=layers,
        schedule=[],
        final_norm=PartSpec("layernorm", dict(norm, name="ln_f")),
        head=PartSpec("lm_head", dict(vocab_size=config.vocab_size, hidden_size=hidden,
                                      tied=config.tie_word_embeddings, tied_to="wte.weight", name="lm_head",
                                      init_std=std)),
        normalise_name=_normalise_name,
        checkpoint_name=_checkpoint_name,
    )


register_architecture("GPT2LMHeadModel", GPT2Config, build_gpt2_spec, model_type="gpt2", replace=True)
