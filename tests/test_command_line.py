"""The command line's options and what they hand to ``build_scheduler`` (no GPU: the scheduler is a stand-in)."""

import pytest

from pagedserve_b200 import main as cli


class StandInScheduler:
    def __init__(self):
        self.requests = []
        self.engine = type("E", (), {"vocab_size": 50})()

    def add_token_request(self, prompt, max_new_tokens, temperature, seed):
        self.requests.append((list(prompt), max_new_tokens, temperature, seed))
        return len(self.requests) - 1

    def run_until_complete(self):
        return {index: [index] * request[1] for index, request in enumerate(self.requests)}


def run_cli(monkeypatch, argv):
    seen = {}

    def build_scheduler(model, **options):
        seen["model"], seen["options"], seen["scheduler"] = model, options, StandInScheduler()
        return seen["scheduler"]

    monkeypatch.setattr(cli, "build_scheduler", build_scheduler)
    assert cli.main(argv) == 0
    return seen


def test_defaults_follow_the_reference(monkeypatch, capsys):
    """reference: main.py:258-321 (defaults of its options) and :337-342 (two demo requests of 8 tokens)."""
    seen = run_cli(monkeypatch, [])
    options = seen["options"]
    assert options["scheduling_strategy"] == "orca" and options["prefill_chunk_size"] == 16
    assert options["max_batch_size"] is None and options["kv_cache_memory_mb"] is None
    assert options["kv_cache_memory_utilization"] == 0.90 and options["kv_cache_safety_mb"] == 3072
    assert options["execution_dtype"] == "float32" and options["enable_cuda_graphs"] is True
    assert options["decode_attention_backend"] == "cuda" and options["kv_cache_dtype"] == "model"
    assert [request[1] for request in seen["scheduler"].requests] == [8, 8]
    assert capsys.readouterr().out.count("request ") == 2


def test_options_reach_the_scheduler(monkeypatch, tmp_path):
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("1 2 3\n\n4,5\n")
    seen = run_cli(monkeypatch, [
        "--model", "gpt2-124m", "--strategy", "sarathi", "--prefill-chunk-size", "128", "--max-batch-size", "64",
        "--max-num-batched-tokens", "512", "--kv-cache-memory-mb", "2048", "--kv-cache-memory-utilization", "0.5",
        "--kv-cache-safety-mb", "100", "--block-size", "8", "--dtype", "bfloat16", "--disable-cuda-graphs",
        "--decode-attention-backend", "triton", "--kv-cache-dtype", "model",
        "--temperature", "0.8", "--seed", "5", "--max-new-tokens", "3", "--prompt-ids", "7 8 9",
        "--prompt-file", str(prompts)])
    options = seen["options"]
    assert seen["model"] == "gpt2-124m"
    assert options == dict(scheduling_strategy="sarathi", prefill_chunk_size=128, max_batch_size=64,
                           kv_cache_memory_mb=2048, kv_cache_memory_utilization=0.5, kv_cache_safety_mb=100,
                           execution_dtype="bfloat16", decode_attention_backend="triton", kv_cache_dtype="model",
                           enable_cuda_graphs=False, block_size=8, num_blocks=None,
                           max_num_batched_tokens=512, seed=5)
    assert seen["scheduler"].requests == [([7, 8, 9], 3, 0.8, 5), ([1, 2, 3], 3, 0.8, 6), ([4, 5], 3, 0.8, 7)]


def test_unknown_choices_are_refused(monkeypatch):
    for argv in (["--strategy", "fifo"], ["--dtype", "float16"], ["--decode-attention-backend", "flash"],
                 ["--kv-cache-dtype", "fp8"]):
        with pytest.raises(SystemExit):
            run_cli(monkeypatch, argv)


def test_build_scheduler_checks_its_arguments():
    with pytest.raises(ValueError, match="max_batch_size must be positive"):
        cli.build_scheduler("tiny-a", max_batch_size=0)
    with pytest.raises(ValueError, match="model folder or one of"):
        cli.build_engine("no-such-model")
    # reference: main.py:152-157 and :165-167 (same messages); the int8 cache is not built
    with pytest.raises(ValueError, match="Unknown decode attention backend 'flash'"):
        cli.build_scheduler("tiny-a", decode_attention_backend="flash")
    with pytest.raises(ValueError, match="Unknown KV cache dtype 'fp8'"):
        cli.build_scheduler("tiny-a", kv_cache_dtype="fp8")
    with pytest.raises(ValueError, match="'int8' is not built"):
        cli.build_scheduler("tiny-a", kv_cache_dtype="int8")
