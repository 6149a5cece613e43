"""Shared helpers of the tests: tiny configurations, model folders, traces, replay."""

from __future__ import annotations

import io
import json
import os
import random
import tempfile
from types import SimpleNamespace

import numpy as np
import torch

import plain_gpt2

# Two tiny configurations that differ in every size and option.
TINY_A = dict(n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
              layer_norm_epsilon=1e-5, activation_function="gelu_new")
TINY_B = dict(n_layer=3, n_embd=96, n_head=2, n_inner=320, vocab_size=1000, n_positions=256,
              layer_norm_epsilon=1e-6, activation_function="gelu")
# Two more with the head sizes of the tcgen05 attention kernel (64, 128), widths that are no multiple of 64 or
# 128 and prompts of several 128-key tiles: they are not "tiny configurations of record", they take the
# engine through the kernels that A and B (head sizes 16 and 48) never reach.
TINY_C = dict(n_layer=2, n_embd=192, n_head=3, n_inner=520, vocab_size=777, n_positions=384,
              layer_norm_epsilon=1e-5, activation_function="gelu_new")
TINY_D = dict(n_layer=2, n_embd=256, n_head=2, n_inner=264, vocab_size=1031, n_positions=320,
              layer_norm_epsilon=1e-6, activation_function="gelu")
# A head size that is no multiple of 16 (GPT-2's config.json allows any n_embd / n_head): CUDA-core kernels.
TINY_E = dict(n_layer=2, n_embd=100, n_head=5, n_inner=260, vocab_size=301, n_positions=96,
              layer_norm_epsilon=1e-5, activation_function="gelu_new")
# The layer sizes of the benchmarked models with two layers each, so that the kernels meet the widths they are
# timed at: tails of 128-wide tiles at 1,600 and 4,800 columns, 25 heads, products too wide for the folded norm
# (medium and XL, small vocabulary), and the 50,257-wide head at the 124M widths.
REAL_MD2 = dict(n_layer=2, n_embd=1024, n_head=16, n_inner=4096, vocab_size=1003, n_positions=1024,
                layer_norm_epsilon=1e-5, activation_function="gelu_new")
REAL_XL2 = dict(n_layer=2, n_embd=1600, n_head=25, n_inner=6400, vocab_size=1003, n_positions=1024,
                layer_norm_epsilon=1e-5, activation_function="gelu_new")
REAL_SM2 = dict(n_layer=2, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024,
                layer_norm_epsilon=1e-5, activation_function="gelu_new")
TINY = {"a": (TINY_A, 0, 16), "b": (TINY_B, 1, 8), "c": (TINY_C, 2, 16), "d": (TINY_D, 3, 32),     # config, seed, block size
        "e": (TINY_E, 4, 8), "md2": (REAL_MD2, 5, 16), "xl2": (REAL_XL2, 6, 16), "sm2": (REAL_SM2, 7, 16)}

_FOLDERS = {}


def model_folder(which: str) -> str:
    """A temporary model folder (config.json + model.safetensors) for tiny config ``which``."""
    if which not in _FOLDERS:
        from pagedserve_b200.config.gpt2 import GPT2Config
        from pagedserve_b200.weights.random_init import write_random_model

        values, seed, _ = TINY[which]
        holder = tempfile.TemporaryDirectory(prefix=f"ps_tiny_{which}_")
        write_random_model(holder.name, GPT2Config(**values), seed)
        _FOLDERS[which] = holder
    return _FOLDERS[which].name


_PLAIN = {}


def plain_model(which: str):
    if which not in _PLAIN:
        _PLAIN[which] = plain_gpt2.read_folder(model_folder(which), dtype=torch.float64)
    return _PLAIN[which]


def random_tokens(vocab: int, count: int, seed: int):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]


# ------------------------------------------------------------------------------- traces
def trace_whole(sequences):
    """Each request alone and whole, logits at every place."""
    steps = []
    for index, (name, tokens) in enumerate(sequences.items()):
        steps.append({"step": index, "entries": [{"id": name, "tokens": tokens,
                                                  "want": list(range(len(tokens)))}], "end": [name]})
    return steps


def trace_tail(sequences, tail=32):
    """All but the last ``tail`` tokens in one step, then the rest one by one."""
    steps = []
    number = 0
    for name, tokens in sequences.items():
        head = max(len(tokens) - tail, 1)
        steps.append({"step": number, "entries": [{"id": name, "tokens": tokens[:head],
                                                   "want": list(range(head))}], "end": []})
        number += 1
        for place in range(head, len(tokens)):
            last = place == len(tokens) - 1
            steps.append({"step": number, "entries": [{"id": name, "tokens": [tokens[place]], "want": [0]}],
                          "end": [name] if last else []})
            number += 1
    return steps


def trace_chunks(sequences, seed=0, sizes=(2, 3, 5, 7, 16, 24, 2, 33, 4)):
    """Portions of changing size, down to two tokens."""
    rng = random.Random(seed)
    steps = []
    number = 0
    for name, tokens in sequences.items():
        cursor = 0
        turn = rng.randrange(len(sizes))
        while cursor < len(tokens):
            size = sizes[turn % len(sizes)]
            turn += 1
            left = len(tokens) - cursor
            if left - size == 1:      # never leave a single token: portions have at least two
                size += 1
            size = min(size, left)
            piece = tokens[cursor:cursor + size]
            cursor += size
            steps.append({"step": number, "entries": [{"id": name, "tokens": piece,
                                                       "want": list(range(len(piece)))}],
                          "end": [name] if cursor == len(tokens) else []})
            number += 1
    return steps


def trace_mixed(sequences, seed=0, live=4, decode_tail=12, max_portion=24):
    """Up to ``live`` requests at a time; portions of some beside single tokens of others.

    Every request first runs its prompt part in portions of random size (2..max_portion),
    then its last ``decode_tail`` tokens one per step.  Finished requests are ended and the
    next ones admitted, so that pages are handed out again.  Now and then a live request is
    left out of a step."""
    rng = random.Random(seed)
    waiting = list(sequences.items())
    running = []          # [name, tokens, cursor]
    steps = []
    number = 0
    while waiting or running:
        while waiting and len(running) < live:
            name, tokens = waiting.pop(0)
            running.append([name, tokens, 0])
        entries, ended = [], []
        for state in running:
            name, tokens, cursor = state
            if len(running) > 1 and rng.random() < 0.15:
                continue                                  # left out of this step
            prompt_end = max(len(tokens) - decode_tail, 1)
            if cursor < prompt_end:
                size = rng.randint(2, max_portion)
                left = prompt_end - cursor
                if left - size == 1:
                    size += 1
                size = min(size, left)
            else:
                size = 1
            piece = tokens[cursor:cursor + size]
            state[2] = cursor + size
            entries.append({"id": name, "tokens": piece, "want": list(range(len(piece)))})
            if state[2] == len(tokens):
                ended.append(name)
        if not entries:
            continue
        rng.shuffle(entries)
        steps.append({"step": number, "entries": entries, "end": ended})
        number += 1
        running = [state for state in running if state[0] not in ended]
    return steps


def peak_tokens(steps, round_to=64):
    """Most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held = {}
    peak = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-count // round_to) * round_to for count in held.values()))
        for name in step["end"]:
            held.pop(name, None)
    return peak


# ------------------------------------------------------------------------------- replay
def replay(folder, dtype, steps, max_tokens, block_size=16):
    """Run ``steps`` through the replay program's own ``run`` (in process); returns
    {request: float32 array [len, vocab]} assembled from the <step>.f32 files."""
    from pagedserve_b200.engine import replay as replay_module

    with tempfile.TemporaryDirectory(prefix="ps_out_") as out:
        args = SimpleNamespace(model=folder, dtype=dtype, out=out, max_tokens=max_tokens,
                               block_size=block_size, max_num_seqs=8, disable_cuda_graphs=False)
        stdin = io.StringIO("".join(json.dumps(step) + "\n" for step in steps))
        stdout = io.StringIO()
        assert replay_module.run(args, stdin=stdin, stdout=stdout) == 0
        assert stdout.getvalue().split() == [w for s in steps for w in ("done", str(s["step"]))]
        return collect(out, steps)


def collect(out, steps):
    vocab = None
    rows = {}
    for step in steps:
        wanted = sum(len(entry["want"]) for entry in step["entries"])
        if wanted == 0:
            continue
        data = np.fromfile(os.path.join(out, f"{step['step']}.f32"), dtype="<f4")
        vocab = data.size // wanted
        data = data.reshape(wanted, vocab)
        cursor = 0
        for entry in step["entries"]:
            for place in entry["want"]:
                rows.setdefault(entry["id"], []).append(data[cursor])
                cursor += 1
    return {name: np.stack(parts) for name, parts in rows.items()}


_PLAIN_LOGITS = {}


def plain_logits(which, sequences):
    """The plain implementation's logits of whole sequences (kept: every replay mode asks for the same ones)."""
    config, weights = plain_model(which)
    out = {}
    for name, tokens in sequences.items():
        key = (which, tuple(tokens))
        if key not in _PLAIN_LOGITS:
            _PLAIN_LOGITS[key] = plain_gpt2.forward_logits(config, weights, tokens).numpy()
        out[name] = _PLAIN_LOGITS[key]
    return out


def plain_rows(which, tokens, rows):
    """The plain implementation's logits at ``rows`` of one whole sequence: the blocks run on every position,
    the head only on the wanted ones (a vocabulary of 50,257 makes the head the larger part)."""
    config, weights = plain_model(which)
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    hidden = plain_gpt2.embedding(weights, ids, torch.arange(ids.numel()))
    for index in range(config["n_layer"]):
        hidden = plain_gpt2.block(weights, index, hidden, config)
    return plain_gpt2.lm_head(weights, config, hidden[torch.as_tensor(list(rows), dtype=torch.long)])


# Tolerances, relative to the largest |logit| of the reference row set.
#   float32 : every sum is float32; differences come from summation order only.
#   bfloat16: activations are rounded to 8 bits of mantissa between the kernels.
TOLERANCE = {"float32": 2e-5, "bfloat16": 3e-2}
# Measured on the tiny and the real-width configurations: the worst element is off by up to 5e-3 x scale, the mean
# element by up to 1e-3 x scale, and no top-1 differs where the plain model's lead exceeds 3.3e-3 x scale.
BF16_MEAN_TOLERANCE = 3e-3
TOP1_LEAD = {"float32": 2e-5, "bfloat16": 1e-2}


def assert_close(got, want, dtype, what=""):
    scale = float(np.abs(want).max())
    error = float(np.abs(got.astype(np.float64) - want).max())
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    if error > TOLERANCE[dtype] * scale:
        bad = np.argwhere(np.abs(got - want) > TOLERANCE[dtype] * scale)
        first = int(bad[:, 0].min())
        raise AssertionError(f"{what}: max error {error:.3e} exceeds {TOLERANCE[dtype]:.0e} x scale "
                             f"{scale:.3e}; first wrong position {first}")
    # Where the plain model's best logit leads the second clearly, the engine must pick the same token (the
    # elementwise bound alone only implies this for leads of twice the tolerance).
    ordered = np.sort(want, axis=-1)
    clear = (ordered[:, -1] - ordered[:, -2]) > TOP1_LEAD[dtype] * scale
    wrong = np.flatnonzero(clear & (got.argmax(-1) != want.argmax(-1)))
    assert wrong.size == 0, f"{what}: top-1 differs at position {int(wrong[0])} although the lead is clear"
    if dtype == "bfloat16":
        # one wrong key in one head moves a whole row by a little: the mean error over the rows is bounded
        # far more tightly than the worst element
        mean_error = float(np.abs(got.astype(np.float64) - want).mean())
        assert mean_error <= BF16_MEAN_TOLERANCE * scale, \
            f"{what}: mean error {mean_error:.3e} exceeds {BF16_MEAN_TOLERANCE:.0e} x scale {scale:.3e}"
