"""Safetensors reading and writing, by-name loading and its one clear error, random weights."""

import os

import pytest
import torch

import helpers
from pagedserve_b200.config.gpt2 import GPT2Config
from pagedserve_b200.config.registry import resolve_architecture
from pagedserve_b200.models.model import Model
from pagedserve_b200.parts.base import PartEnv
from pagedserve_b200.weights import WeightError, read_safetensors, write_random_model, write_safetensors
from pagedserve_b200.weights.loader import load_weights
from pagedserve_b200.weights.random_init import random_tensors


def cpu_model(values):
    config = GPT2Config(**values)
    _, _, builder = resolve_architecture(config.to_dict())
    return config, Model(builder(config), PartEnv(ops=None, dtype=torch.float32, device="cpu"))


def test_safetensors_round_trip_and_foreign_reader(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "e": torch.empty(0, 4)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, metadata={"k": "v"})
    back = read_safetensors(path)
    assert set(back) == set(tensors)
    for name in tensors:
        assert back[name].dtype == tensors[name].dtype and torch.equal(back[name], tensors[name])
    from safetensors.torch import load_file, save_file     # the format's own library agrees both ways
    theirs = load_file(path)
    assert all(torch.equal(theirs[n], tensors[n]) for n in tensors)
    save_file({k: v for k, v in tensors.items()}, str(tmp_path / "y.safetensors"))
    again = read_safetensors(str(tmp_path / "y.safetensors"))
    assert all(torch.equal(again[n], tensors[n]) for n in tensors)


def test_loads_by_name_and_casts_by_role(tmp_path):
    config, model = cpu_model(helpers.TINY_B)
    write_random_model(str(tmp_path), config, seed=1)
    model.load_folder(str(tmp_path))
    stored = read_safetensors(str(tmp_path / "model.safetensors"))
    assert stored["transformer.h.0.attn.c_attn.weight"].shape == (96, 288)        # Conv1D [in, out]
    assert model.tensors["h.0.attn.c_attn.weight"].shape == (288, 96)             # kept [out, in]
    assert torch.equal(model.tensors["h.0.attn.c_attn.weight"],
                       stored["transformer.h.0.attn.c_attn.weight"].float().T)
    assert model.tensors["h.0.ln_1.weight"].dtype == torch.float32
    assert "lm_head.weight" not in model.tensors and model.head.table is None

    env16 = PartEnv(ops=None, dtype=torch.bfloat16, device="cpu")
    model16 = Model(model.spec, env16)
    model16.load_folder(str(tmp_path))
    assert model16.tensors["wte.weight"].dtype == torch.bfloat16            # tables and matrices: compute dtype
    assert model16.tensors["h.1.mlp.c_fc.weight"].dtype == torch.bfloat16
    assert model16.tensors["h.1.mlp.c_fc.bias"].dtype == torch.float32      # vectors feed 32-bit math


def test_names_without_prefix_and_mask_buffers_are_accepted(tmp_path):
    config, model = cpu_model(helpers.TINY_A)
    tensors = random_tensors(config, 0)
    renamed = {name[len("transformer."):]: t for name, t in tensors.items()}
    renamed["h.0.attn.bias"] = torch.ones(1, 1, 8, 8)
    renamed["h.1.attn.masked_bias"] = torch.tensor(-1e4)
    renamed["lm_head.weight"] = renamed["wte.weight"].clone()
    model.load_tensors(renamed)
    assert model.tensors["wte.weight"].shape == (512, 64)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config, model = cpu_model(helpers.TINY_A)
    tensors = random_tensors(config, 0)
    del tensors["transformer.h.1.mlp.c_proj.bias"]
    del tensors["transformer.ln_f.weight"]
    tensors["transformer.h.0.attn.rotary.inv_freq"] = torch.zeros(4)
    tensors["transformer.wpe.weight"] = torch.zeros(64, 64)
    tensors["transformer.h.0.ln_1.bias"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as caught:
        load_weights(str(tmp_path), model.param_specs(), torch.float32, "cpu", model.spec.normalise_name)
    error = caught.value
    assert sorted(error.missing) == ["h.1.mlp.c_proj.bias", "ln_f.weight"]
    assert error.unexpected == ["transformer.h.0.attn.rotary.inv_freq"]
    assert error.wrong_shape == [("transformer.wpe.weight", (128, 64), (64, 64))]
    assert error.wrong_dtype and error.wrong_dtype[0][0] == "transformer.h.0.ln_1.bias"
    text = str(error)
    for fragment in ("missing (2)", "ln_f.weight", "unexpected (1)", "rotary.inv_freq", "wrong shape",
                     "expected [128, 64], got [64, 64]"):
        assert fragment in text
    with pytest.raises(WeightError, match="no model.safetensors"):
        load_weights(str(tmp_path / "nowhere"), model.param_specs(), torch.float32, "cpu")


def test_untied_head_needs_its_tensor():
    values = dict(helpers.TINY_A, tie_word_embeddings=False)
    config, model = cpu_model(values)
    tensors = random_tensors(config, 0)
    assert "lm_head.weight" in tensors
    model.load_tensors(tensors)
    assert model.head.table.shape == (512, 64)
    del tensors["lm_head.weight"]
    with pytest.raises(WeightError, match="lm_head.weight"):
        model.load_tensors(tensors)


def test_tied_head_stored_in_the_file_must_equal_the_table(tmp_path):
    """reference: src/model/gpt2.py:42, 77-78 ties the head to the token table when tie_word_embeddings is set and
    copies lm_head.weight otherwise; a file that stores a tied head with other numbers contradicts its configuration."""
    config, model = cpu_model(helpers.TINY_A)
    tensors = random_tensors(config, 0)
    tensors["lm_head.weight"] = tensors["transformer.wte.weight"].clone()
    model.load_tensors(tensors)                                        # an equal copy is accepted and not kept
    assert "lm_head.weight" not in model.tensors and model.head.table is None
    tensors["lm_head.weight"][3, 5] += 0.25
    del tensors["transformer.ln_f.bias"]
    with pytest.raises(WeightError) as caught:
        model.load_tensors(tensors)
    assert caught.value.not_tied == [("lm_head.weight", "transformer.wte.weight")]
    assert caught.value.missing == ["ln_f.bias"]                       # still one error that lists everything
    assert "not tied: lm_head.weight differs from transformer.wte.weight" in str(caught.value)
    # the same file loads into the untied configuration, which then uses the stored head
    untied_config, untied = cpu_model(dict(helpers.TINY_A, tie_word_embeddings=False))
    tensors["transformer.ln_f.bias"] = torch.zeros(64)
    untied.load_tensors(tensors)
    assert not torch.equal(untied.head.table, untied.embedding.table)


def test_random_weights_are_seeded_and_bf16_exact(tmp_path):
    config = GPT2Config(**helpers.TINY_A)
    a, b, c = random_tensors(config, 5), random_tensors(config, 5), random_tensors(config, 6)
    assert all(torch.equal(a[n], b[n]) for n in a)
    assert any(not torch.equal(a[n], c[n]) for n in a)
    f32 = random_tensors(config, 5, "float32")
    assert all(torch.equal(f32[n], a[n].float()) for n in a)           # same numbers in both storages
    gamma = a["transformer.h.0.ln_1.weight"].float()
    assert abs(float(gamma.mean()) - 1.0) < 0.02
    out = a["transformer.h.0.attn.c_proj.weight"].float().std()
    plain = a["transformer.h.0.attn.c_attn.weight"].float().std()
    assert abs(float(out) - 0.01) < 0.002 and abs(float(plain) - 0.02) < 0.002
    folder = write_random_model(str(tmp_path), config, 5)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
