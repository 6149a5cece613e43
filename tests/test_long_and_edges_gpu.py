"""Long decoding, the first tokens of a sequence, and inputs built so that a fault of the cache shows."""

import numpy as np
import pytest

import helpers
import plain_gpt2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b"])
def test_long_decoding_token_by_token(which, dtype):
    """Two requests decoded one token per step from their second token to the model's last position,
    side by side (so every step is a replayed CUDA graph), against whole-sequence logits."""
    values, _, block = helpers.TINY[which]
    length = values["n_positions"]
    seqs = {"p": helpers.random_tokens(values["vocab_size"], length, seed=21),
            "q": helpers.random_tokens(values["vocab_size"], length - 37, seed=22)}
    want = helpers.plain_logits(which, seqs)
    steps = [{"step": 0, "entries": [{"id": n, "tokens": t[:1], "want": [0]} for n, t in seqs.items()], "end": []}]
    for place in range(1, length):
        entries = [{"id": n, "tokens": [t[place]], "want": [0]} for n, t in seqs.items() if place < len(t)]
        ended = [n for n, t in seqs.items() if place == len(t) - 1]
        steps.append({"step": place, "entries": entries, "end": ended})
    got = helpers.replay(helpers.model_folder(which), dtype, steps, helpers.peak_tokens(steps), block_size=block)
    for name in seqs:
        helpers.assert_close(got[name], want[name], dtype, f"long decode {which}/{dtype}/{name}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(dtype):
    """Positions 0..3 alone, as one-token prompts, two-token prompts, and decoded from position 0."""
    vocab = helpers.TINY["a"][0]["vocab_size"]
    seqs = {f"s{i}": helpers.random_tokens(vocab, n, seed=70 + i) for i, n in enumerate([1, 2, 3, 4])}
    want = helpers.plain_logits("a", seqs)
    whole = helpers.replay(helpers.model_folder("a"), dtype, helpers.trace_whole(seqs), 256)
    single = helpers.replay(helpers.model_folder("a"), dtype, helpers.trace_tail(seqs, tail=32), 256)
    together = [{"step": 0, "entries": [{"id": n, "tokens": t, "want": list(range(len(t)))} for n, t in seqs.items()],
                 "end": list(seqs)}]
    batch = helpers.replay(helpers.model_folder("a"), dtype, together, 256)
    for name in seqs:
        for got in (whole, single, batch):
            helpers.assert_close(got[name], want[name], dtype, f"first tokens {name}")


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
def test_a_reused_page_never_leaks_and_page_edges_hold(dtype, tol):
    """A request fills pages with large keys and values and ends; the next requests get those very pages
    (LIFO) and stop one token short of, at, and one past a page edge. Stale rows of the reused pages lie
    right behind their last token: if a kernel read one slot too far the logits would move visibly."""
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.batch import StepEntry
    from pagedserve_b200.engine.engine import Engine

    config, weights = helpers.plain_model("a")
    engine = Engine.from_folder(helpers.model_folder("a"), EngineConfig(dtype=dtype, block_size=16, num_blocks=8,
                                                                       max_num_seqs=4))
    vocab = config["vocab_size"]
    first = helpers.random_tokens(vocab, 128, seed=5)
    engine.step([StepEntry("old", first, [127])])
    pool = engine.cache.groups[0].pool
    pool.mul_(50.0)                                   # what "old" leaves behind is loud
    engine.finish("old")
    assert engine.cache.free_pages() == 8
    for length in (15, 16, 17, 31, 32, 33):
        tokens = helpers.random_tokens(vocab, length, seed=100 + length)
        want = plain_gpt2.forward_logits(config, weights, tokens).numpy()
        head = max(1, length - 3)
        rows = [engine.step([StepEntry("new", tokens[:head], list(range(head)))]).cpu().numpy()]
        for place in range(head, length):
            rows.append(engine.step([StepEntry("new", [tokens[place]], [0])]).cpu().numpy())
        got = np.concatenate(rows)
        scale = float(np.abs(want).max())
        assert float(np.abs(got - want).max()) <= tol * scale, f"length {length}"
        table = list(engine.cache.groups[0].tables["new"])
        engine.finish("new")
        pool[table].mul_(50.0) if dtype == "float32" else None
    engine.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_padded_mixed_steps_replay_as_graphs(dtype):
    """Mixed steps are padded to recurring shapes (padding tokens go to the cache's scratch slot) and replayed
    as CUDA graphs once a shape has come back.  Steps of different real sizes that share a padded shape must
    give the logits of an engine that runs every step eagerly and unpadded."""
    from pagedserve_b200.engine.batch import StepEntry
    from test_generation_gpu import make_engine

    vocab = helpers.TINY["c"][0]["vocab_size"]
    padded = make_engine("c", dtype, num_blocks=96)
    eager = make_engine("c", dtype, num_blocks=96, enable_cuda_graphs=False)
    assert padded.runner._pad_mixed and not eager.runner._pad_mixed
    scale = None
    for round_index, (long_len, short_len, decode_count) in enumerate([(100, 5, 3), (97, 3, 2), (120, 7, 3),
                                                                      (101, 2, 1), (99, 9, 3)]):
        # a prompt portion, a short portion and a few single tokens of requests that already have a prompt
        results = []
        for engine in (padded, eager):
            base = 1000 * round_index
            prompts = {base + i: helpers.random_tokens(vocab, 20 + 7 * i, seed=base + i) for i in range(decode_count)}
            engine.step([StepEntry(name, tokens, []) for name, tokens in prompts.items()])
            entries = [StepEntry(base + 50, helpers.random_tokens(vocab, long_len, seed=base + 50), [long_len - 1]),
                       StepEntry(base + 51, helpers.random_tokens(vocab, short_len, seed=base + 51), [0, short_len - 1])]
            entries += [StepEntry(name, [len(tokens) % vocab], [0]) for name, tokens in prompts.items()]
            results.append(engine.step(entries).float().cpu())
            for entry in entries:
                engine.finish(entry.request)
            engine.cache.check_invariants()
        got, want = results
        scale = float(want.abs().max())
        assert got.shape == want.shape
        assert float((got - want).abs().max()) <= helpers.TOLERANCE[dtype] * scale, f"round {round_index}"
    assert padded.runner.graph_replays > 0            # the rounds shared padded shapes
    assert padded.cache.free_pages() == padded.cache.total_pages()


@pytest.mark.parametrize("which", ["b", "d"])
def test_random_mixed_steps_padded_graphs_equal_eager(which):
    """Random traffic: every step a random mix of new prompts, portions that continue a prompt, short portions
    and single tokens, with random wanted places; requests end at random.  The engine that pads and replays
    graphs must return what the engine that runs every step eagerly and unpadded returns."""
    import random

    from pagedserve_b200.engine.batch import StepEntry
    from test_generation_gpu import make_engine

    config, _, block = helpers.TINY[which]
    vocab, limit = config["vocab_size"], config["n_positions"]
    engines = [make_engine(which, "bfloat16", num_blocks=4096 // block, max_num_seqs=12),
               make_engine(which, "bfloat16", num_blocks=4096 // block, max_num_seqs=12, enable_cuda_graphs=False)]
    assert engines[0].runner._pad_mixed
    rng = random.Random(17)
    live = {}                          # request -> tokens so far
    next_name = 0
    for step_index in range(60):
        entries = []
        for name in list(live):
            if rng.random() < 0.15:
                if live[name]:                                     # it has run at least once
                    for engine in engines:
                        engine.finish(name)
                del live[name]
        while len(live) < 12 and rng.random() < 0.5:
            live[next_name] = 0
            next_name += 1
        for name, held in live.items():
            if rng.random() < 0.2:
                continue                                           # left out of this step
            room = limit - held
            if room <= 0:
                continue
            kind = rng.random()
            count = 1 if kind < 0.5 else rng.randint(2, 15) if kind < 0.7 else rng.randint(16, 90)
            count = min(count, room)
            tokens = [rng.randrange(vocab) for _ in range(count)]
            want = sorted(rng.sample(range(count), rng.randint(0, min(count, 3))))
            if count == 1:
                want = [0]
            entries.append((name, tokens, want))
        if not entries:
            continue
        outputs = [engine.step([StepEntry(*entry) for entry in entries]).float().cpu() for engine in engines]
        for name, tokens, _ in entries:
            live[name] += len(tokens)
        assert outputs[0].shape == outputs[1].shape
        if outputs[0].numel():
            scale = float(outputs[1].abs().max())
            assert float((outputs[0] - outputs[1]).abs().max()) <= 1e-2 * scale, f"step {step_index}"
    for engine in engines:
        engine.cache.check_invariants()
    assert engines[0].runner.graph_replays > 0


def test_benchmark_sizes_match_plain():
    """The layer sizes the benchmark runs (GPT-2 124M: 12 layers, width 768, 12 heads of 64, inner 3,072,
    vocabulary 50,257) with random weights: a 150-token prompt whole, then decoded tokens, against the plain
    implementation, in float32 and in bfloat16 (whose decode steps run the fused few-rows kernels, the
    tcgen05 products and both attention kernels at their real shapes)."""
    import torch

    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.config.gpt2 import named_config
    from pagedserve_b200.engine.batch import StepEntry
    from pagedserve_b200.engine.engine import Engine
    from pagedserve_b200.weights.random_init import random_tensors

    config = named_config("gpt2-124m")
    tensors = random_tensors(config, 0)
    weights = {name[len("transformer."):] if name.startswith("transformer.") else name: tensor.double()
               for name, tensor in tensors.items()}
    tokens = helpers.random_tokens(config.vocab_size, 156, seed=99)
    want = plain_gpt2.forward_logits(config.to_dict(), weights, tokens)[-7:].numpy()
    for dtype in ("float32", "bfloat16"):
        engine = Engine(config, EngineConfig(dtype=dtype, num_blocks=128, max_num_seqs=8), tensors=tensors)
        got = [engine.step([StepEntry("r", tokens[:150], [149])]).cpu().numpy()]
        for place in range(150, 156):
            got.append(engine.step([StepEntry("r", [tokens[place]], [0])]).cpu().numpy())
        helpers.assert_close(np.concatenate(got), want, dtype, f"gpt2-124m/{dtype}")
        engine.finish("r")
        if dtype == "bfloat16":
            # the benchmark's step: eight requests decode together (a replayed graph from the second step on)
            prompts = [helpers.random_tokens(config.vocab_size, 24 + 19 * i, seed=7 + i) for i in range(8)]
            tails = [helpers.random_tokens(config.vocab_size, 3, seed=70 + i) for i in range(8)]
            engine.step([StepEntry(i, prompt, []) for i, prompt in enumerate(prompts)])
            rows = [engine.step([StepEntry(i, [tails[i][place]], [0]) for i in range(8)]).cpu().numpy()
                    for place in range(3)]
            assert engine.runner.graph_replays > 0
            for i in range(8):
                plain = plain_gpt2.forward_logits(config.to_dict(), weights, prompts[i] + tails[i])[-3:].numpy()
                helpers.assert_close(np.stack([rows[place][i] for place in range(3)]), plain, dtype,
                                     f"gpt2-124m/batch 8/request {i}")
        del engine
        torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [True, False])
def test_returned_logits_outlive_the_next_steps(dtype, graphs):
    """A step's intermediate tensors and its logits lie in the step arena, which the next step writes over; what
    ``Engine.step`` returns is a copy and must still hold the step's values after other steps have run (prompt
    steps of other sizes, decode steps, a replayed graph)."""
    from pagedserve_b200.engine.batch import StepEntry
    from test_generation_gpu import make_engine

    vocab = helpers.TINY["c"][0]["vocab_size"]
    engine = make_engine("c", dtype, num_blocks=96, enable_cuda_graphs=graphs)
    first_tokens = helpers.random_tokens(vocab, 70, seed=5)
    first = engine.step([StepEntry("a", first_tokens, [0, 33, 69])])
    kept = first.clone()
    later = [engine.step([StepEntry("b", helpers.random_tokens(vocab, 120, seed=6), [119])]),
             engine.step([StepEntry("a", [3], [0]), StepEntry("b", [4], [0])]),
             engine.step([StepEntry("a", [5], [0]), StepEntry("b", [6], [0])]),
             engine.step([StepEntry("c", helpers.random_tokens(vocab, 40, seed=7), list(range(40)))])]
    assert bool((first == kept).all())
    # and the later results are not views of one another either
    snapshots = [tensor.clone() for tensor in later]
    engine.step([StepEntry("a", [7], [0]), StepEntry("b", [8], [0]), StepEntry("c", [9], [0])])
    for tensor, snapshot in zip(later, snapshots):
        assert bool((tensor == snapshot).all())
    for name in "abc":
        engine.finish(name)
    assert engine.cache.free_pages() == engine.cache.total_pages()
