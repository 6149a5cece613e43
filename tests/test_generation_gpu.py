"""Generation through the Python entry point and the command line, compared with the plain
implementation: greedy (exact tokens in float32) and temperature sampling."""

import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_gpt2

pytestmark = pytest.mark.gpu

PROMPT_LENGTHS = {"a": [5, 17, 33], "b": [1, 9, 40, 64, 100]}


def make_engine(which, dtype, **options):
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.engine import Engine

    block = helpers.TINY[which][2]
    defaults = dict(dtype=dtype, block_size=block, num_blocks=512 // block, max_num_seqs=8)
    defaults.update(options)
    return Engine.from_folder(helpers.model_folder(which), EngineConfig(**defaults))


def prompts_of(which):
    vocab = helpers.TINY[which][0]["vocab_size"]
    return [helpers.random_tokens(vocab, length, seed=11 + length) for length in PROMPT_LENGTHS[which]]


@pytest.mark.parametrize("strategy,chunk", [("orca", 16), ("sarathi", 24)])
@pytest.mark.parametrize("which", ["a", "b"])
def test_greedy_generation_equals_plain(which, strategy, chunk):
    from pagedserve_b200.engine.engine import generate

    config, weights = helpers.plain_model(which)
    prompts = prompts_of(which)
    want = [plain_gpt2.generate(config, weights, prompt, 8) for prompt in prompts]
    engine = make_engine(which, "float32")
    got = generate(engine, prompts, max_new_tokens=8, strategy=strategy, prefill_chunk_size=chunk)
    assert got == want
    assert engine.cache.live_requests == 0 and engine.cache.free_pages() == engine.cache.total_pages()
    engine.cache.check_invariants()


@pytest.mark.parametrize("which", ["a", "b"])
def test_generation_equals_what_the_reference_generated(which):
    """The workloads the two tiny configurations are quoted with, run by the reference's own scheduler, cache
    and model on the CPU (recorded by tests/golden/make_golden.py): the float32 engine generates the very same
    tokens under the same strategy, portion size and page size."""
    import json
    import os

    from pagedserve_b200.engine.engine import generate

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"tiny_{which}_generated.json")
    with open(path) as handle:
        record = json.load(handle)
    vocab = helpers.TINY[which][0]["vocab_size"]
    assert record["block_size"] == helpers.TINY[which][2]
    prompts = [helpers.random_tokens(vocab, length, seed=record["prompt_seed_offset"] + length)
               for length in record["prompt_lengths"]]
    engine = make_engine(which, "float32")
    got = generate(engine, prompts, max_new_tokens=record["max_new_tokens"], strategy=record["strategy"],
                   prefill_chunk_size=record["prefill_chunk_size"], max_num_seqs=4)
    assert got == record["generated"]
    assert engine.cache.live_requests == 0 and engine.cache.free_pages() == engine.cache.total_pages()


def test_temperature_sampling_follows_the_keyed_noise():
    """Tiny B, mixed batch with 24-token portions beside decodes, 12 tokens at T = 0.8:
    every sampled token must (nearly) maximise logit/T + gumbel(seed, position, i) under the
    plain model, whatever else was in its batch."""
    from pagedserve_b200.engine.engine import generate

    config, weights = helpers.plain_model("b")
    prompts = prompts_of("b")
    engine = make_engine("b", "float32")
    got = generate(engine, prompts, max_new_tokens=12, temperature=0.8, seed=1234, strategy="sarathi",
                   prefill_chunk_size=24, max_num_seqs=4)
    again = generate(make_engine("b", "float32"), prompts, max_new_tokens=12, temperature=0.8, seed=1234,
                     strategy="orca")
    assert got == again, "sampled tokens depend on the batching"
    for index, (prompt, produced) in enumerate(zip(prompts, got)):
        tokens = list(prompt)
        for token in produced:
            logits = plain_gpt2.forward_logits(config, weights, tokens)[-1]
            scores = plain_gpt2.temperature_scores(logits, 0.8, 1234 + index, len(tokens))
            assert scores[token] >= scores.max() - 1e-4, f"request {index}: token {token} is not the draw"
            tokens.append(token)
    greedy = generate(make_engine("b", "float32"), prompts, max_new_tokens=12)
    assert greedy != got


def test_bfloat16_generation_tracks_plain_logits():
    """In bfloat16 a near-tie may flip a greedy token; each chosen token must be within the
    bfloat16 tolerance of the plain model's best logit along the engine's own path."""
    from pagedserve_b200.engine.engine import generate

    config, weights = helpers.plain_model("a")
    prompts = prompts_of("a")
    got = generate(make_engine("a", "bfloat16"), prompts, max_new_tokens=8)
    for prompt, produced in zip(prompts, got):
        tokens = list(prompt)
        for token in produced:
            logits = plain_gpt2.forward_logits(config, weights, tokens)[-1]
            slack = helpers.TOLERANCE["bfloat16"] * float(logits.abs().max()) * 2
            assert float(logits[token]) >= float(logits.max()) - slack
            tokens.append(token)


def test_sampler_kernel_alone():
    from pagedserve_b200.kernels.ops import Ops
    from pagedserve_b200.sampling.sampler import Sampler

    ops = Ops(torch.float32)
    sampler = Sampler(ops, "cuda:0", max_rows=4)
    generator = torch.Generator().manual_seed(5)
    logits = torch.randn(7, 1003, generator=generator)
    logits[2, 17] = logits[2, 900] = 9.0                    # a tie: lowest index wins
    device_logits = logits.cuda()
    assert sampler.sample(device_logits, [0.0] * 7, [0] * 7, [0] * 7) == [
        17 if r == 2 else int(torch.argmax(logits[r])) for r in range(7)]
    temperatures = [0.0, 0.5, 1.0, 2.0, 0.0, 1.3, 0.7]
    seeds = [1, 2, 3, 2 ** 63 + 5, 5, 6, 7]
    positions = [0, 3, 900, 12, 5, 1, 77]
    got = sampler.sample(device_logits, temperatures, seeds, positions)
    for r in range(7):
        if temperatures[r] == 0:
            assert got[r] == (17 if r == 2 else int(torch.argmax(logits[r])))
        else:
            scores = plain_gpt2.temperature_scores(logits[r], temperatures[r], seeds[r], positions[r])
            assert scores[got[r]] >= scores.max() - 1e-4
    # a wide vocabulary (a row shared out over a cluster of CTAs), not a multiple of anything, ties across shares
    wide = torch.randn(5, 50257, generator=generator)
    wide[1, 40000] = wide[1, 7] = 11.0
    wide[3, 50256] = 12.0
    device_wide = wide.cuda()
    temperatures, seeds, positions = [0.0, 0.0, 0.9, 0.0, 1.7], [3, 4, 5, 6, 7], [1, 2, 3, 4, 1000]
    got = sampler.sample(device_wide, temperatures, seeds, positions)
    for r in range(5):
        if temperatures[r] == 0:
            assert got[r] == (7 if r == 1 else 50256 if r == 3 else int(torch.argmax(wide[r])))
        else:
            scores = plain_gpt2.temperature_scores(wide[r], temperatures[r], seeds[r], positions[r])
            assert scores[got[r]] >= scores.max() - 1e-4
    # the draw is a sample of softmax(logits / T): empirical frequencies over many positions
    row = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).cuda().repeat(4000, 1)
    draws = sampler.sample(row, [1.0] * 4000, [9] * 4000, list(range(4000)))
    freq = np.bincount(draws, minlength=4) / 4000.0
    want = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]), 0).numpy()
    assert np.abs(freq - want).max() < 0.03


def test_command_line_runs():
    out = subprocess.run([sys.executable, "-m", "pagedserve_b200", "--model", helpers.model_folder("a"),
                          "--dtype", "float32", "--strategy", "sarathi", "--prefill-chunk-size", "4",
                          "--max-new-tokens", "5", "--prompt-ids", "5 17 3 200", "--prompt-ids", "9,8,7"],
                         capture_output=True, text=True, cwd=helpers.os.path.dirname(helpers.__file__) + "/..")
    assert out.returncode == 0, out.stderr
    lines = [line for line in out.stdout.splitlines() if line.startswith("request ")]
    config, weights = helpers.plain_model("a")
    assert lines == [f"request 0: {plain_gpt2.generate(config, weights, [5, 17, 3, 200], 5)!r}",
                     f"request 1: {plain_gpt2.generate(config, weights, [9, 8, 7], 5)!r}"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_equals_eager_and_device_loop_equals_stepwise(dtype):
    """The captured decode step (a CUDA graph) gives the logits of the eager step, and a run of several decode steps on the device gives the tokens
    of step-by-step generation."""
    from pagedserve_b200.engine.batch import StepEntry

    vocab = helpers.TINY["b"][0]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=n) for n in (7, 30, 64)]
    results = {}
    for graphs in (False, True):
        engine = make_engine("b", dtype, enable_cuda_graphs=graphs)
        first = engine.step([StepEntry(i, p, [len(p) - 1]) for i, p in enumerate(prompts)])
        tokens = [int(t) for t in first.argmax(-1).tolist()]
        rows = []
        for _ in range(5):        # first call runs eagerly and captures, later calls replay
            logits = engine.step([StepEntry(i, [tokens[i]], [0]) for i in range(3)])
            rows.append(logits.cpu())
            tokens = [int(t) for t in logits.argmax(-1).tolist()]
        # then 6 steps in one call, sampling on the device at temperature 0.7
        run = engine.decode([StepEntry(i, [tokens[i]]) for i in range(3)], [0.7, 0.0, 0.7], [5, 6, 7], steps=6)
        results[graphs] = (torch.stack(rows), run, engine.runner.graph_replays)
        assert [engine.cache.length(i) for i in range(3)] == [len(p) + 11 for p in prompts]
    eager, graph = results[False], results[True]
    assert graph[2] > 0 and eager[2] == 0
    scale = float(eager[0].abs().max())
    assert float((eager[0] - graph[0]).abs().max()) <= helpers.TOLERANCE[dtype] * scale
    if dtype == "float32":
        assert np.array_equal(eager[1], graph[1])
        # the device loop follows the keyed noise of the plain sampler
        config, weights = helpers.plain_model("b")
        sequence = list(prompts[0])
        engine = make_engine("b", dtype)
        first = engine.step([StepEntry(0, prompts[0], [len(prompts[0]) - 1])])
        token = int(first.argmax(-1).item())
        run = engine.decode([StepEntry(0, [token])], [0.9], [42], steps=8)[:, 0].tolist()
        sequence.append(token)
        for drawn in run:
            logits = plain_gpt2.forward_logits(config, weights, sequence)[-1]
            scores = plain_gpt2.temperature_scores(logits, 0.9, 42, len(sequence))
            assert scores[drawn] >= scores.max() - 1e-4
            sequence.append(drawn)


def test_eager_device_loop_crosses_a_key_chunk_boundary():
    """Several decode steps in one call without CUDA graphs, bfloat16: the contexts pass 128 keys (the split
    attention kernel's chunk at this head size) inside the call, so the bound that sizes the kernel's grid has
    to cover the last step, not the first.  The tokens must be those of one call per step."""
    from pagedserve_b200.engine.batch import StepEntry

    vocab = helpers.TINY["b"][0]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=70 + n) for n in (121, 126, 60)]
    runs = []
    for steps_per_call in (1, 12):
        engine = make_engine("b", "bfloat16", enable_cuda_graphs=False)
        first = engine.step([StepEntry(i, p, [len(p) - 1]) for i, p in enumerate(prompts)])
        tokens = [int(t) for t in first.argmax(-1).tolist()]
        drawn = []
        for _ in range(12 // steps_per_call):
            out = engine.decode([StepEntry(i, [tokens[i]]) for i in range(3)], [0.0] * 3, [0] * 3,
                                steps=steps_per_call)
            drawn.append(out)
            tokens = [int(t) for t in out[-1]]
        engine.check_status()
        runs.append(np.concatenate(drawn))
        assert [engine.cache.length(i) for i in range(3)] == [len(p) + 12 for p in prompts]
    assert np.array_equal(runs[0], runs[1])


def test_a_step_staged_ahead_is_used_or_undone():
    """While a decode step runs, the host stages the next one of the same requests and, once the step is a
    captured graph, launches it right behind (the tokens are fed back on the device).  The step must be used
    when the batch comes back, and undone (its pages returned, its results ignored) when a request ends on an
    end-of-sequence token, when another request joins, and when something else is called in between."""
    from pagedserve_b200.engine.batch import StepEntry

    config, weights = helpers.plain_model("a")
    vocab = helpers.TINY["a"][0]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=40 + n) for n in (14, 15, 16, 30)]
    want = [plain_gpt2.generate(config, weights, prompt, 12) for prompt in prompts]
    # request 1 ends early on its 4th token; request 3 joins after two decode steps
    eos = want[1][3]
    for i in range(4):
        if eos in want[i]:
            want[i] = want[i][:want[i].index(eos) + 1]
    engine = make_engine("a", "float32")
    scheduler = engine.make_scheduler(strategy="orca", max_num_seqs=4, eos_token_id=eos)
    ids = [scheduler.add_token_request(prompt, max_new_tokens=12) for prompt in prompts[:3]]
    staged_seen = launched_seen = 0
    for step in range(64):
        if step == 3:
            ids.append(scheduler.add_token_request(prompts[3], max_new_tokens=12))
        if not (scheduler.waiting or scheduler.active):
            break
        scheduler.step()
        staged_seen += engine.runner._staged is not None
        launched_seen += engine.runner._staged is not None and engine.runner._staged.launched
        engine.cache.check_invariants()
    assert staged_seen > 0 and launched_seen > 0             # the paths under test were taken
    got = [scheduler.finished[i].generated_token_ids for i in ids]
    assert got == want
    assert engine.runner._staged is None
    assert engine.cache.live_requests == 0 and engine.cache.free_pages() == engine.cache.total_pages()

    # a staged step is undone when a different call comes in between
    engine = make_engine("a", "float32")
    first = engine.step([StepEntry(i, p, [len(p) - 1]) for i, p in enumerate(prompts[:2])])
    tokens = [int(t) for t in first.argmax(-1).tolist()]
    free_before = engine.cache.free_pages()
    out = engine.decode_tokens([0, 1], tokens, [0.0, 0.0], [0, 0], 1, stage_next=True)
    assert engine.runner._staged is not None and engine.runner._staged.launched
    logits = engine.step([StepEntry(0, [int(out[0, 0])], [0])])          # not the staged batch
    assert engine.runner._staged is None
    assert int(logits.argmax(-1).item()) == want[0][2] or eos in want[0][:2]
    engine.finish(0)
    engine.finish(1)
    assert engine.cache.free_pages() == engine.cache.total_pages() >= free_before
    engine.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_flag_raised_by_a_kernel_reaches_the_caller(dtype):
    """Kernels report bad input and waits that ran out through one device flag.  A decode step brings the flag
    back with its tokens and raises; after steps that only return logits, ``check_status`` does.  The flag is
    set by hand here (no kernel is made to fail)."""
    from pagedserve_b200.engine.batch import StepEntry
    from pagedserve_b200.engine.step import StepError

    engine = make_engine("a", dtype)
    vocab = helpers.TINY["a"][0]["vocab_size"]
    prompt = helpers.random_tokens(vocab, 9, seed=3)
    logits = engine.step([StepEntry(0, prompt, [len(prompt) - 1])])
    engine.check_status()                                              # nothing flagged
    token = int(logits.argmax(-1).item())
    out = engine.decode_tokens([0], [token], [0.0], [0], 1)
    assert engine.runner._status is engine.ops.status_flag(engine.device)      # one flag for ops and runner
    engine.runner._status.fill_(7)
    with pytest.raises(StepError, match="status 7"):
        engine.decode_tokens([0], [int(out[0, 0])], [0.0], [0], 1)
    assert int(engine.runner._status.item()) == 0                      # raised once, then cleared
    engine.runner._status.fill_(5)
    with pytest.raises(StepError, match="status 5"):
        engine.check_status()
    engine.check_status()
    engine.finish(0)
