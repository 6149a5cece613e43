"""Plain, slow GPT-2: whole sequences, no cache, one function for each part.

This file is the oracle of the test-suite.  It is written from the formulas of
the reference (each function cites the lines it follows), shares no code with
the package under test, reads a model folder with the ``safetensors`` library
and runs on the CPU.  ``tests/golden/make_golden.py`` compares it once with the
reference's own ``PagedDecoderLM.prefill`` on tiny random models; the outputs
of that comparison are committed under ``tests/golden/``.

Weights are used exactly as stored in a Hugging Face GPT-2 checkpoint: the four
projections of a block are "Conv1D" matrices of shape ``[in, out]``
(reference: src/model/gpt2.py:14-17 transposes them into ``nn.Linear``).
"""

from __future__ import annotations

import json
import math
import os

import numpy as np
import torch


# --------------------------------------------------------------------------
# folder reading (independent of the package's own reader)
# --------------------------------------------------------------------------
def read_folder(folder, dtype=torch.float64):
    """Return (config dict, {HF tensor name: tensor cast to ``dtype``})."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as handle:
        config = json.load(handle)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    weights = {}
    for name, tensor in tensors.items():
        if name.startswith("transformer."):
            name = name[len("transformer."):]
        weights[name] = tensor.to(dtype)
    return config, weights


def sizes(config):
    """Derived sizes (reference: src/model/gpt2.py:32-44)."""
    hidden = config["n_embd"]
    heads = config["n_head"]
    inner = config.get("n_inner") or 4 * hidden
    return hidden, heads, hidden // heads, inner


# --------------------------------------------------------------------------
# one function for each part
# --------------------------------------------------------------------------
def embedding(weights, token_ids, positions):
    """h0[t] = wte[id_t] + wpe[pos_t]  (reference: src/model/paged_decoder.py:306-314)."""
    return weights["wte.weight"][token_ids] + weights["wpe.weight"][positions]


def layer_norm(x, gamma, beta, eps):
    """(x - mean) / sqrt(var + eps) * gamma + beta with the biased variance over the
    last axis (reference: src/kernels/triton_residual_layernorm.py:25-40; the
    torch path is nn.LayerNorm, src/model/paged_decoder.py:170-177)."""
    mean = x.mean(dim=-1, keepdim=True)
    centered = x - mean
    variance = (centered * centered).mean(dim=-1, keepdim=True)
    return centered / torch.sqrt(variance + eps) * gamma + beta


def conv1d(x, weight, bias):
    """y = x W + b with W stored [in, out] (reference: src/model/gpt2.py:14-17)."""
    return x @ weight + bias


def split_qkv(qkv, heads, head_dim):
    """Packed order q, k, v; head j is columns [j*hd, (j+1)*hd) of each
    (reference: src/model/paged_decoder.py:52-53, 63-69)."""
    tokens = qkv.shape[0]
    hidden = heads * head_dim
    q, k, v = qkv[:, :hidden], qkv[:, hidden:2 * hidden], qkv[:, 2 * hidden:]
    shape = (tokens, heads, head_dim)
    return q.reshape(shape), k.reshape(shape), v.reshape(shape)


def causal_attention(q, k, v, window=None):
    """softmax((q k^T) * hd^-0.5 masked where key_pos > query_pos) v, per head
    (reference: src/model/paged_decoder.py:83-91; src/model/paged_attention.py:283-295).
    ``window`` (not a GPT-2 option; used by the kernel tests) additionally masks
    keys with key_pos <= query_pos - window."""
    tokens, heads, head_dim = q.shape
    scale = 1.0 / math.sqrt(head_dim)
    scores = torch.einsum("qhd,khd->hqk", q, k) * scale
    query_pos = torch.arange(tokens).unsqueeze(1)
    key_pos = torch.arange(tokens).unsqueeze(0)
    mask = key_pos > query_pos
    if window is not None:
        mask = mask | (key_pos <= query_pos - window)
    scores = scores.masked_fill(mask.unsqueeze(0), float("-inf"))
    probabilities = torch.softmax(scores, dim=-1)
    context = torch.einsum("hqk,khd->qhd", probabilities, v)
    return context.reshape(tokens, heads * head_dim)  # reference: paged_decoder.py:71-73


def activation(x, name):
    """gelu_new / gelu_pytorch_tanh: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)));
    gelu: 0.5 x (1 + erf(x / sqrt 2))  (reference: src/model/paged_decoder.py:273-280)."""
    if name in ("gelu_new", "gelu_pytorch_tanh"):
        return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))
    if name == "gelu":
        return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
    raise ValueError(f"unsupported activation {name}")


def attention_sublayer(weights, prefix, x, heads, head_dim):
    """c_attn -> split -> causal attention -> c_proj
    (reference: src/model/paged_decoder.py:75-96)."""
    qkv = conv1d(x, weights[prefix + "attn.c_attn.weight"], weights[prefix + "attn.c_attn.bias"])
    q, k, v = split_qkv(qkv, heads, head_dim)
    context = causal_attention(q, k, v)
    return conv1d(context, weights[prefix + "attn.c_proj.weight"], weights[prefix + "attn.c_proj.bias"])


def mlp_sublayer(weights, prefix, x, activation_name):
    """c_fc -> activation -> c_proj (reference: src/model/paged_decoder.py:186-188)."""
    up = conv1d(x, weights[prefix + "mlp.c_fc.weight"], weights[prefix + "mlp.c_fc.bias"])
    return conv1d(activation(up, activation_name),
                  weights[prefix + "mlp.c_proj.weight"], weights[prefix + "mlp.c_proj.bias"])


def block(weights, index, hidden_states, config):
    """Pre-LayerNorm block with two residual adds
    (reference: src/model/paged_decoder.py:181-189)."""
    _, heads, head_dim, _ = sizes(config)
    eps = config["layer_norm_epsilon"]
    prefix = f"h.{index}."
    normed = layer_norm(hidden_states, weights[prefix + "ln_1.weight"], weights[prefix + "ln_1.bias"], eps)
    hidden_states = hidden_states + attention_sublayer(weights, prefix, normed, heads, head_dim)
    normed = layer_norm(hidden_states, weights[prefix + "ln_2.weight"], weights[prefix + "ln_2.bias"], eps)
    return hidden_states + mlp_sublayer(weights, prefix, normed, config["activation_function"])


def lm_head(weights, config, hidden_states):
    """ln_f then logits = x wte^T, no bias, tied unless tie_word_embeddings is false
    (reference: src/model/paged_decoder.py:330, 300-301; src/model/gpt2.py:42-43, 77-78)."""
    normed = layer_norm(hidden_states, weights["ln_f.weight"], weights["ln_f.bias"],
                        config["layer_norm_epsilon"])
    if config.get("tie_word_embeddings", True):
        table = weights["wte.weight"]
    else:
        table = weights["lm_head.weight"]
    return normed @ table.T


def forward_logits(config, weights, token_ids):
    """Logits [T, V] at every position of one whole sequence
    (reference: src/model/paged_decoder.py:316-331)."""
    ids = torch.as_tensor(list(token_ids), dtype=torch.long)
    if ids.numel() > config["n_positions"]:
        raise ValueError("sequence exceeds n_positions")  # reference: paged_decoder.py:318-319
    positions = torch.arange(ids.numel())
    hidden_states = embedding(weights, ids, positions)
    for index in range(config["n_layer"]):
        hidden_states = block(weights, index, hidden_states, config)
    return lm_head(weights, config, hidden_states)


# --------------------------------------------------------------------------
# sampling (the reference samples by argmax only: src/scheduler/orca_scheduler.py:250)
# --------------------------------------------------------------------------
def greedy_token(logits_row):
    """argmax, lowest index on ties."""
    return int(torch.argmax(logits_row).item())


_M64 = (1 << 64) - 1


def _mix64(x):
    """splitmix64 finaliser on Python integers."""
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def gumbel_noise(seed, position, vocab):
    """Counter-based Gumbel noise: key = mix(mix(seed) ^ position); per vocabulary index i,
    r = mix(key + i); u = ((r >> 41) + 0.5) / 2^23; g = -log(-log(u)).  float64."""
    key = _mix64(_mix64(seed & _M64) ^ (position & _M64))
    out = np.empty(vocab, dtype=np.float64)
    for index in range(vocab):
        r = _mix64((key + index) & _M64)
        u = ((r >> 41) + 0.5) / float(1 << 23)
        out[index] = -math.log(-math.log(u))
    return out


def temperature_scores(logits_row, temperature, seed, position):
    """score_i = logit_i / T + g_i ; the sampled token is the argmax of the scores."""
    logits = logits_row.detach().to(torch.float64).numpy()
    return logits / temperature + gumbel_noise(seed, position, logits.shape[0])


def generate(config, weights, prompt, max_new_tokens, temperature=0.0, seed=0):
    """Token-by-token generation by re-running the whole sequence each time."""
    tokens = list(prompt)
    produced = []
    for _ in range(max_new_tokens):
        logits = forward_logits(config, weights, tokens)[-1]
        if temperature == 0.0:
            token = greedy_token(logits)
        else:
            # position of the token being sampled = current length
            token = int(np.argmax(temperature_scores(logits, temperature, seed, len(tokens))))
        tokens.append(token)
        produced.append(token)
    return produced
