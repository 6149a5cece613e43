"""The plain implementation against the stored outputs of the reference's own model."""

import json
import os

import numpy as np
import pytest
import torch

import helpers
import plain_gpt2

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("which", ["a", "b"])
def test_plain_matches_reference_outputs(which):
    with open(os.path.join(GOLDEN, f"tiny_{which}_tokens.json")) as handle:
        record = json.load(handle)
    assert record["config"] == helpers.TINY[which][0]
    config, weights = plain_gpt2.read_folder(helpers.model_folder(which), dtype=torch.float32)
    got = plain_gpt2.forward_logits(config, weights, record["tokens"]).numpy()
    want = np.fromfile(os.path.join(GOLDEN, f"tiny_{which}_logits.f32"), dtype="<f4").reshape(got.shape)
    assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("which", ["a", "b"])
def test_plain_generates_what_the_reference_generated(which):
    """Greedy tokens of each configuration's serving workload as the reference's own scheduler, paged cache
    and chunked forward pass produced them on the CPU (tests/golden/make_golden.py)."""
    with open(os.path.join(GOLDEN, f"tiny_{which}_generated.json")) as handle:
        record = json.load(handle)
    config, weights = helpers.plain_model(which)
    vocab = helpers.TINY[which][0]["vocab_size"]
    for length, want in zip(record["prompt_lengths"], record["generated"]):
        prompt = helpers.random_tokens(vocab, length, seed=record["prompt_seed_offset"] + length)
        assert plain_gpt2.generate(config, weights, prompt, record["max_new_tokens"]) == want


def test_causality_and_prefix_property():
    """Logits at a position depend only on the tokens up to it."""
    config, weights = helpers.plain_model("a")
    tokens = helpers.random_tokens(config["vocab_size"], 20, seed=1)
    full = plain_gpt2.forward_logits(config, weights, tokens)
    short = plain_gpt2.forward_logits(config, weights, tokens[:9])
    assert torch.allclose(full[:9], short, atol=1e-12)


def test_layer_norm_and_activations():
    x = torch.randn(5, 12, dtype=torch.float64)
    g, b = torch.randn(12, dtype=torch.float64), torch.randn(12, dtype=torch.float64)
    want = torch.nn.functional.layer_norm(x, (12,), g, b, 1e-6)
    assert torch.allclose(plain_gpt2.layer_norm(x, g, b, 1e-6), want, atol=1e-12)
    assert torch.allclose(plain_gpt2.activation(x, "gelu"), torch.nn.functional.gelu(x), atol=1e-12)
    assert torch.allclose(plain_gpt2.activation(x, "gelu_new"),
                          torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-12)


def test_window_masks_old_keys():
    q = torch.randn(10, 2, 16, dtype=torch.float64)
    k = torch.randn(10, 2, 16, dtype=torch.float64)
    v = torch.randn(10, 2, 16, dtype=torch.float64)
    windowed = plain_gpt2.causal_attention(q, k, v, window=3)
    # the last query sees exactly keys 7, 8, 9
    tail = plain_gpt2.causal_attention(q[7:], k[7:], v[7:])
    assert torch.allclose(windowed[-1], tail[-1], atol=1e-12)


def test_gumbel_noise_is_keyed_by_seed_and_position():
    a = plain_gpt2.gumbel_noise(3, 10, 50)
    assert np.array_equal(a, plain_gpt2.gumbel_noise(3, 10, 50))
    assert not np.array_equal(a, plain_gpt2.gumbel_noise(4, 10, 50))
    assert not np.array_equal(a, plain_gpt2.gumbel_noise(3, 11, 50))
    assert np.isfinite(a).all()
