"""Compare the plain implementation once with the reference's own model code on the CPU.

Run from the repository root, with the reference checkout on ``sys.path``:

    python tests/golden/make_golden.py /path/to/reference

For each tiny configuration it writes a model folder with the package's random-weights
mode, loads the tensors into the reference's ``PagedDecoderLM`` the way its adapter does
(Conv1D ``[in, out]`` transposed into ``nn.Linear``; reference: src/model/gpt2.py:14-17,
48-78), runs the reference's dense ``prefill`` (src/model/paged_decoder.py:316-331) and the
plain implementation (tests/plain_gpt2.py) on the same token ids in float32, checks that they
agree, and stores the reference's logits under ``tests/golden/`` as
``<name>_tokens.json`` and ``<name>_logits.f32`` (little-endian float32 ``[T, V]``).

It then runs each configuration's serving workload (tiny A: prompts of 5, 17 and 33 tokens, 8 new
tokens, whole prompts; tiny B: prompts of 1, 9, 40, 64 and 100 tokens, 12 new tokens, prompt
portions of 24 tokens beside decoded tokens) through the reference's own scheduler, paged cache
and chunked forward pass, greedy, checks that the plain implementation generates the same tokens,
and stores them as ``<name>_generated.json``.

``tests/test_plain.py`` then checks the plain implementation against these files on every
run, without needing the reference.
"""

import json
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.normpath(os.path.join(HERE, "..", ".."))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import plain_gpt2  # noqa: E402
from helpers import TINY, random_tokens  # noqa: E402


# which -> (prompt lengths, new tokens, strategy, prefill chunk): the workloads the two configurations are quoted with
GENERATION = {"a": ([5, 17, 33], 8, "orca", 16), "b": ([1, 9, 40, 64, 100], 12, "sarathi", 24)}


def reference_model(reference_root, config, weights):
    """The reference's ``PagedDecoderLM`` holding ``weights`` (the tensors of a folder written by this package)."""
    if reference_root not in sys.path:
        sys.path.insert(0, reference_root)
    from src.model.paged_decoder import PagedDecoderLM, TransformerConfig

    hidden, heads, head_dim, inner = plain_gpt2.sizes(config)
    activation = {"gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu": "gelu"}[
        config["activation_function"]]
    model = PagedDecoderLM(TransformerConfig(
        vocab_size=config["vocab_size"], hidden_size=hidden, num_layers=config["n_layer"], num_heads=heads,
        head_dim=head_dim, mlp_hidden_size=inner, max_sequence_length=config["n_positions"],
        activation_function=activation, layer_norm_epsilon=config["layer_norm_epsilon"],
        tie_word_embeddings=True, lm_head_bias=False)).eval()
    with torch.no_grad():
        model.embedding_table.weight.copy_(weights["wte.weight"])
        model.position_embeddings.weight.copy_(weights["wpe.weight"])
        for index, layer in enumerate(model.layers):
            prefix = f"h.{index}."
            layer.input_layernorm.weight.copy_(weights[prefix + "ln_1.weight"])
            layer.input_layernorm.bias.copy_(weights[prefix + "ln_1.bias"])
            layer.post_attention_layernorm.weight.copy_(weights[prefix + "ln_2.weight"])
            layer.post_attention_layernorm.bias.copy_(weights[prefix + "ln_2.bias"])
            for target, name in ((layer.self_attn.qkv_linear, "attn.c_attn"),
                                 (layer.self_attn.output_linear, "attn.c_proj"),
                                 (layer.mlp_up_proj, "mlp.c_fc"), (layer.mlp_down_proj, "mlp.c_proj")):
                target.weight.copy_(weights[prefix + name + ".weight"].transpose(0, 1))
                target.bias.copy_(weights[prefix + name + ".bias"])
        model.final_layernorm.weight.copy_(weights["ln_f.weight"])
        model.final_layernorm.bias.copy_(weights["ln_f.bias"])
    return model


def reference_logits(model, token_ids):
    with torch.no_grad():
        logits, _ = model.prefill(torch.tensor([token_ids], dtype=torch.long))
    return logits[0].numpy()


def reference_generation(model, config, prompts, max_new_tokens, strategy, chunk, block_size):
    """Greedy tokens from the reference's whole serving path on the CPU: its scheduler, its paged cache and
    its chunked ``forward_iteration`` (reference: src/scheduler/orca_scheduler.py:221-303,
    src/model/paged_decoder.py:509-619), end-of-sequence off."""
    from src.model.kv_manager import KVCacheManager
    from src.model.paged_attention import PagedAttention
    from src.scheduler.orca_scheduler import ContinuousBatchScheduler

    hidden, heads, head_dim, _ = plain_gpt2.sizes(config)
    cache = KVCacheManager(block_size=block_size, total_memory=8 * 1024 * 1024, tensor_dtype=torch.float32,
                           device=torch.device("cpu"), num_layers=config["n_layer"], num_kv_heads=heads,
                           head_dim=head_dim)
    scheduler = ContinuousBatchScheduler(model_engine=model, max_batch_size=4, tokenizer=None, kv_manager=cache,
                                         paged_attn_manager=PagedAttention(kv_manager=cache),
                                         scheduling_strategy=strategy, prefill_chunk_size=chunk)
    ids = [scheduler.add_token_request(prompt, max_new_tokens=max_new_tokens) for prompt in prompts]
    while scheduler.waiting or scheduler.active:
        scheduler.step()
    return [list(scheduler.finished[request_id].generated_token_ids) for request_id in ids]


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of a checkout of jainalphin/pagedserve>")
    reference_root = sys.argv[1]
    from pagedserve_b200.config.gpt2 import GPT2Config
    from pagedserve_b200.weights.random_init import write_random_model

    for which in ("a", "b"):
        values, seed, _ = TINY[which]
        with tempfile.TemporaryDirectory() as folder:
            write_random_model(folder, GPT2Config(**values), seed)
            config, weights = plain_gpt2.read_folder(folder, dtype=torch.float32)
        tokens = random_tokens(values["vocab_size"], 11, seed=40 + seed)
        model = reference_model(reference_root, config, weights)
        theirs = reference_logits(model, tokens)
        ours = plain_gpt2.forward_logits(config, weights, tokens).numpy()
        error = float(np.abs(theirs - ours).max())
        scale = float(np.abs(theirs).max())
        print(f"tiny {which}: max |reference - plain| = {error:.3e} (largest logit {scale:.3e})")
        assert error <= 2e-5 * max(scale, 1.0), "the plain implementation disagrees with the reference"
        with open(os.path.join(HERE, f"tiny_{which}_tokens.json"), "w") as handle:
            json.dump({"config": values, "seed": seed, "tokens": tokens}, handle)
        theirs.astype("<f4").tofile(os.path.join(HERE, f"tiny_{which}_logits.f32"))

        # the serving workload of this configuration through the reference's scheduler, greedy
        lengths, new_tokens, strategy, chunk = GENERATION[which]
        prompts = [random_tokens(values["vocab_size"], length, seed=70 + length) for length in lengths]
        generated = reference_generation(model, config, prompts, new_tokens, strategy, chunk, TINY[which][2])
        plain = [plain_gpt2.generate(config, weights, prompt, new_tokens) for prompt in prompts]
        print(f"tiny {which}: {len(prompts)} prompts, {strategy}, reference tokens "
              f"{'equal' if generated == plain else 'DIFFER from'} the plain implementation's")
        assert generated == plain, (generated, plain)
        with open(os.path.join(HERE, f"tiny_{which}_generated.json"), "w") as handle:
            json.dump({"prompt_lengths": lengths, "prompt_seed_offset": 70, "max_new_tokens": new_tokens,
                       "strategy": strategy, "prefill_chunk_size": chunk, "block_size": TINY[which][2],
                       "generated": generated}, handle)


if __name__ == "__main__":
    main()
