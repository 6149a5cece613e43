"""The shapes and schedules that ``bench.py`` times, compared with the plain implementation.

The tiny configurations take the engine through every kernel, but not at the widths it is measured at.  Here
two-layer models carry the layer sizes of GPT-2 medium and XL (tails of the 128-wide tensor-core tiles at 1,600
and 4,800 columns, 25 heads, products too wide for the norm folded into them) and of GPT-2 124M with its whole
vocabulary (the 50,257-wide head, which a batch of 64 sends through another kernel than a batch of 8).
After the reference's model-level checks (testing/test_project.py:859-927) and its matrix of contexts and
fragmented tables (testing/test_triton_correctness_matrix.py:14-136).
"""

import numpy as np
import pytest
import torch

import helpers
import plain_gpt2

pytestmark = pytest.mark.gpu

LENGTHS = {"md2": [17, 260, 700], "xl2": [5, 130, 515], "e": [3, 20, 64, 96]}


def sequences(which):
    vocab = helpers.TINY[which][0]["vocab_size"]
    return {f"r{index}": helpers.random_tokens(vocab, length, seed=300 * index + 11)
            for index, length in enumerate(LENGTHS[which])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["md2", "xl2", "e"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_replay_at_benchmarked_widths_matches_plain(which, dtype, mode):
    """Whole, with a decoded tail, in portions and mixed: at the widths of GPT-2 medium and XL, and at a head
    size of 20 (no multiple of 16: the CUDA-core attention in both precisions)."""
    seqs = sequences(which)
    want = helpers.plain_logits(which, seqs)
    block = helpers.TINY[which][2]
    if mode == "whole":
        steps = helpers.trace_whole(seqs)
    elif mode == "tail":
        steps = helpers.trace_tail(seqs, tail=32)
    elif mode == "chunks":
        steps = helpers.trace_chunks(seqs, seed=8, sizes=(2, 40, 5, 130, 16, 3, 260, 24))
    else:
        steps = helpers.trace_mixed(seqs, seed=9, live=3, max_portion=150)
    got = helpers.replay(helpers.model_folder(which), dtype, steps, helpers.peak_tokens(steps), block_size=block)
    for name in seqs:
        helpers.assert_close(got[name], want[name], dtype, f"{mode}/{which}/{dtype}/{name}")


def make_engine(which, dtype, **options):
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.engine import Engine

    defaults = dict(dtype=dtype, block_size=16, num_blocks=1024, max_num_seqs=64, max_num_batched_tokens=2048)
    defaults.update(options)
    return Engine.from_folder(helpers.model_folder(which), EngineConfig(**defaults))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_of_64_decode_steps_at_124m_widths(dtype):
    """The step that ``points.decode_b64`` times: 64 requests of different lengths, one token each, the whole
    vocabulary.  Three steps as logits against the plain implementation; then three more as one run on the
    device (sampling and token feedback there), which must draw the tokens that step-by-step decoding draws."""
    from pagedserve_b200.engine.batch import StepEntry

    vocab = helpers.TINY["sm2"][0]["vocab_size"]
    lengths = [4 + (37 * i) % 150 for i in range(64)]
    seqs = [helpers.random_tokens(vocab, length + 3, seed=500 + i) for i, length in enumerate(lengths)]
    want = [helpers.plain_rows("sm2", seqs[i], range(lengths[i], lengths[i] + 3)).numpy() for i in range(64)]

    def prepared(check):
        """An engine that has run the prompts (under the token budget of a step) and then the three given
        tokens of every request, one step each; returns it with the logits of the last step."""
        engine = make_engine("sm2", dtype)
        cursor = 0
        while cursor < 64:
            entries, tokens = [], 0
            while cursor < 64 and tokens + lengths[cursor] <= 2048:
                entries.append(StepEntry(cursor, seqs[cursor][:lengths[cursor]]))
                tokens += lengths[cursor]
                cursor += 1
            engine.step(entries)
        for step in range(3):
            logits = engine.step([StepEntry(i, [seqs[i][lengths[i] + step]], [0]) for i in range(64)])
            if check:
                helpers.assert_close(logits.cpu().numpy(), np.stack([want[i][step] for i in range(64)]), dtype,
                                     f"batch 64, step {step}")
        engine.check_status()
        return engine, logits

    engine, last = prepared(check=True)
    # from here on, greedy: one call of three steps on the device against three calls of one step each on a
    # second engine brought to the same state by the same steps
    first = [int(t) for t in last.argmax(-1).tolist()]
    run = engine.decode([StepEntry(i, [first[i]]) for i in range(64)], [0.0] * 64, [0] * 64, steps=3)
    other, _ = prepared(check=False)
    tokens, stepwise = first, []
    for _ in range(3):
        out = other.decode([StepEntry(i, [tokens[i]]) for i in range(64)], [0.0] * 64, [0] * 64, steps=1)
        stepwise.append(out[0])
        tokens = [int(t) for t in out[0]]
    assert np.array_equal(run, np.stack(stepwise))
    if dtype == "float32":
        for i in (0, 21, 63):                                        # and they are the plain model's greedy tokens
            sequence = list(seqs[i]) + [first[i]]
            for step in range(3):
                row = helpers.plain_rows("sm2", sequence, [len(sequence) - 1])[0]
                assert int(run[step, i]) == plain_gpt2.greedy_token(row)
                sequence.append(int(run[step, i]))


def _serving_workload(count, vocab, seed):
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, vocab, int(rng.integers(64, 700))).tolist() for _ in range(count)]
    outputs = [int(rng.integers(3, 9)) for _ in range(count)]
    return prompts, outputs


def _serve(engine, prompts, outputs, temperature, seed):
    """The schedule of ``bench.py --serving``: Sarathi, up to 4 prompt portions of at most 512 tokens beside the
    decode tokens of up to 64 running requests, 2,048 tokens a step."""
    scheduler = engine.make_scheduler(strategy="sarathi", max_num_seqs=64, max_num_batched_tokens=2048,
                                      prefill_chunk_size=512, max_prefills_per_step=4)
    ids = [scheduler.add_token_request(prompt, max_new_tokens=new, temperature=temperature, seed=seed + index)
           for index, (prompt, new) in enumerate(zip(prompts, outputs))]
    produced = scheduler.run_until_complete()
    engine.cache.check_invariants()
    assert engine.cache.live_requests == 0
    return [produced[i] for i in ids]


def test_serving_schedule_greedy_float32_equals_plain():
    """Two passes over the same requests: the second replays the step shapes that the first captured as CUDA
    graphs (padded mixed steps).  Both must generate the plain implementation's greedy tokens."""
    vocab = helpers.TINY["sm2"][0]["vocab_size"]
    prompts, outputs = _serving_workload(20, vocab, seed=3)
    engine = make_engine("sm2", "float32", num_blocks=1400)
    first = _serve(engine, prompts, outputs, 0.0, 0)
    replays_before = engine.runner.graph_replays
    second = _serve(engine, prompts, outputs, 0.0, 0)
    assert engine.runner.graph_replays > replays_before
    assert first == second
    for index in (0, 7, 19):
        sequence = list(prompts[index])
        for token in first[index]:
            row = helpers.plain_rows("sm2", sequence, [len(sequence) - 1])[0]
            assert token == plain_gpt2.greedy_token(row), f"request {index}"
            sequence.append(token)


def test_serving_schedule_temperature_bfloat16_follows_the_keyed_noise():
    """The same schedule in bfloat16 at T = 0.8: every drawn token must maximise logit / T + noise(seed,
    position) under the plain model, up to the bfloat16 tolerance on the logits."""
    vocab = helpers.TINY["sm2"][0]["vocab_size"]
    prompts, outputs = _serving_workload(20, vocab, seed=4)
    engine = make_engine("sm2", "bfloat16", num_blocks=1400)
    _serve(engine, prompts, outputs, 0.8, 77)                        # first pass: shapes are captured
    got = _serve(engine, prompts, outputs, 0.8, 77)
    for index in (1, 8, 18):
        sequence = list(prompts[index])
        for token in got[index]:
            row = helpers.plain_rows("sm2", sequence, [len(sequence) - 1])[0]
            scores = plain_gpt2.temperature_scores(row, 0.8, 77 + index, len(sequence))
            slack = 2 * helpers.TOLERANCE["bfloat16"] * float(row.abs().max()) / 0.8
            assert scores[token] >= scores.max() - slack, f"request {index}: token {token} is not the draw"
            sequence.append(token)
