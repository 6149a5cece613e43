"""Benchmark of the engine's decode step (and prefill) for GPT-2 124M layer sizes, random weights.

    python bench.py --gpus 1 --steps K --warmup W            # this engine
    python bench.py --impl reference --gpus 1 ...            # the unmodified reference, if installed

A "step" is one decode step of the whole batch.  The default run: layer sizes of GPT-2 124M,
bfloat16, batch 8, 512-token prompts of uniform-random token ids, then K decode steps.

value     decoded tokens per second over K steps timed on the device (CUDA events): the captured
          decode step replayed K times, sampling and token feedback on the device.
e2e       the same through the Python entry point (``Scheduler.step``): every step the host builds
          the batch, copies it from pinned memory to the device and reads the sampled tokens back.
          (The scheduler launches the next step of an unchanged batch behind the running one: that
          step's token ids are the ones the device fed back, every other input is uploaded.)
prefill   one step of 2,048 prompt tokens (2 prompts of 1,024).
roofline  bytes the decode step has to read (every weight once + the cache of the live requests)
          divided by its time, against the measured copy bandwidth.
points    decode tokens per second at batch 1 and 64.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                data = json.load(handle)
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for key, value in node.items():
                        if isinstance(value, (int, float)) and key not in flat:
                            flat[key] = float(value)
                        else:
                            walk(value)

            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return {"hbm_gbs": flat["hbm_gbs"], "bf16_tflops": flat["bf16_tflops"],
                        "bf16_tflops_sustained": flat.get("bf16_tflops_sustained"), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                parts = [p.strip() for p in out.stdout.strip().splitlines()[0].split(",")]
                self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        clocks = [int(s[0]) for s in self.samples if s and s[0].isdigit()]
        maxes = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples for i in range(4)
                          if len(s) > 2 + i and s[2 + i].lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None,
                "sm_max_mhz": max(maxes) if maxes else None, "reasons": reasons, "samples": len(clocks)}


def _reference_tree():
    """The folder that holds the unmodified reference (its ``main.py`` and ``src/``), or (None, why).

    jainalphin/pagedserve is a script tree without setup.py or pyproject.toml, so ``pip install --target
    baseline/_ref`` refuses it; a plain copy of the checkout stands in its place.  Where the copy is missing
    and ``PAGEDSERVE_REFERENCE_SRC`` names a checkout, the copy is made now."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref, "src", "model", "paged_decoder.py")):
        source = os.environ.get("PAGEDSERVE_REFERENCE_SRC", "")
        if not os.path.isfile(os.path.join(source, "src", "model", "paged_decoder.py")):
            return None, ("baseline/_ref holds no copy of jainalphin/pagedserve (pip refuses the tree: neither "
                          "setup.py nor pyproject.toml) and PAGEDSERVE_REFERENCE_SRC names no checkout")
        import shutil

        os.makedirs(ref, exist_ok=True)
        shutil.copytree(os.path.join(source, "src"), os.path.join(ref, "src"), dirs_exist_ok=True)
        shutil.copy(os.path.join(source, "main.py"), os.path.join(ref, "main.py"))
    return ref, None


def reference_arm(args):
    """The same measurements on the unmodified reference: its own ``PagedDecoderLM`` with random weights at the
    named layer sizes, its ``KVCacheManager``, ``PagedAttention`` and ``ContinuousBatchScheduler``
    (reference: main.py:104-116, 215-254; benchmark.py:106-128; src/scheduler/orca_scheduler.py:85-117,
    221-303), driven through ``add_token_request`` and ``step`` with the same seeded prompts, warm-up and step
    count as this engine's arm.  Nothing of ``pagedserve_b200`` but the table of layer sizes is imported."""
    ref, why = _reference_tree()
    if ref is None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    try:
        result = _run_reference(args, ref)
    except Exception as error:                                    # the arm must not take the driver down
        message = " ".join(f"{type(error).__name__}: {error}".split())[:300]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference raised: {message}"}))
        return 0
    print(json.dumps(result))
    return 0


def _run_reference(args, ref):
    import importlib.util

    import numpy as np
    import torch

    from pagedserve_b200.config.gpt2 import NAMED_CONFIGS          # layer sizes only: plain Python, no kernels

    sys.path.insert(0, ref)
    from src.model.kv_manager import KVCacheManager
    from src.model.paged_attention import PagedAttention
    from src.model.paged_decoder import PagedDecoderLM, TransformerConfig
    from src.scheduler.orca_scheduler import ContinuousBatchScheduler

    sizes = dict(NAMED_CONFIGS[args.model])
    full_layers = sizes["n_layer"]
    if args.layers:
        sizes["n_layer"] = args.layers
    hidden, heads, inner = sizes["n_embd"], sizes["n_head"], sizes["n_inner"] or 4 * sizes["n_embd"]
    context_len, vocab = sizes["n_positions"], sizes["vocab_size"]
    steps, warmup = args.steps, max(args.warmup, 3)
    if args.prompt_len + warmup + steps + 2 > context_len:
        steps = context_len - args.prompt_len - warmup - 2
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    on_gpu = torch.cuda.is_available()               # without a GPU the arm still runs (a dry run of its host side)
    device = torch.device("cuda" if on_gpu else "cpu")
    backend = "triton" if on_gpu and importlib.util.find_spec("triton") is not None else "torch"

    class DeviceTimer:
        """Milliseconds between ``start`` and ``stop`` on the device (CUDA events); wall clock without a GPU."""

        def start(self):
            if on_gpu:
                self.events = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                self.events[0].record()
            self.began = time.perf_counter()

        def stop(self):
            if on_gpu:
                self.events[1].record()
                torch.cuda.synchronize()
            self.seconds = time.perf_counter() - self.began
            return self.events[0].elapsed_time(self.events[1]) if on_gpu else self.seconds * 1e3
    peaks = load_peaks()

    torch.manual_seed(0)                                           # reference: benchmark.py:106-107
    model = PagedDecoderLM(TransformerConfig(
        vocab_size=vocab, hidden_size=hidden, num_layers=sizes["n_layer"], num_heads=heads,
        head_dim=hidden // heads, mlp_hidden_size=inner, max_sequence_length=context_len,
        activation_function="gelu_tanh", layer_norm_epsilon=sizes["layer_norm_epsilon"],
        tie_word_embeddings=True, lm_head_bias=False))
    model = model.to(device=device, dtype=dtype).eval()            # reference: main.py:133
    model.enable_cuda_graphs = True                                # reference: main.py:193
    max_batch = max(64, args.batch)
    width = 2 if dtype == torch.bfloat16 else 4
    block_bytes = 2 * sizes["n_layer"] * hidden * 16 * width
    cache = KVCacheManager(block_size=16, total_memory=(max_batch * (context_len // 16) + 64) * block_bytes,
                           tensor_dtype=dtype, device=device, num_layers=sizes["n_layer"], num_kv_heads=heads,
                           head_dim=hidden // heads, cache_dtype=dtype)          # reference: main.py:214-223
    attention = PagedAttention(kv_manager=cache, decode_attention_backend=backend)
    rng = np.random.default_rng(0)
    weight_bytes = sum(p.numel() * p.element_size() for name, p in model.named_parameters()
                       if not name.startswith("position_embeddings"))
    kv_bytes_per_token = 2 * sizes["n_layer"] * hidden * width

    def make_scheduler(batch):
        return ContinuousBatchScheduler(model_engine=model, max_batch_size=batch, tokenizer=None, kv_manager=cache,
                                        paged_attn_manager=attention, eos_token_id=None,
                                        scheduling_strategy="orca")

    def measure_decode(batch, k_steps):
        scheduler = make_scheduler(batch)
        for _ in range(batch):
            scheduler.add_token_request(rng.integers(0, vocab, args.prompt_len).tolist(),
                                        max_new_tokens=warmup + k_steps + 2)
        while scheduler.waiting:
            scheduler.step()                                       # the prompts (untimed)
        for _ in range(warmup):
            scheduler.step()
        timer, produced = DeviceTimer(), 0
        with ClockSampler() as clocks:
            timer.start()
            for _ in range(k_steps):
                produced += len(scheduler.step())
            ms = timer.stop()
        seconds = timer.seconds
        _drain(scheduler)
        mean_context = args.prompt_len + warmup + (k_steps + 1) / 2.0
        return {"ms": ms, "tok_s": produced / (ms / 1e3), "e2e_tok_s": produced / seconds,
                "e2e_ms_per_step": seconds * 1e3 / k_steps,
                "bytes_per_step": weight_bytes + batch * mean_context * kv_bytes_per_token,
                "clocks": clocks.summary()}

    def _drain(scheduler):
        while scheduler.waiting or scheduler.active:
            scheduler.step()

    def measure_prefill(tokens_total=2048, repeats=5):
        prompt_len = min(1024, context_len - 1)
        count = max(1, tokens_total // prompt_len)
        times = []
        for repeat in range(repeats + 3):
            scheduler = make_scheduler(count)
            for _ in range(count):
                scheduler.add_token_request(rng.integers(0, vocab, prompt_len).tolist(), max_new_tokens=1)
            timer = DeviceTimer()
            timer.start()
            scheduler.step()                                       # whole prompts in one iteration (Orca)
            elapsed = timer.stop()
            if repeat >= 3:
                times.append(elapsed)
            _drain(scheduler)
        ms = statistics.median(times)
        T = count * prompt_len
        L = sizes["n_layer"]
        gemm = 2.0 * T * L * (4 * hidden * hidden + 2 * hidden * inner) + 2.0 * count * hidden * vocab
        flops = gemm + L * count * 4.0 * hidden * (prompt_len * (prompt_len + 1) / 2.0)
        peak = peaks["bf16_tflops"] * 1e12 if dtype == torch.bfloat16 else 75e12
        return {"value": T / (ms / 1e3), "tokens": T, "ms": ms, "frac": flops / (ms / 1e3) / peak,
                "gflop": flops / 1e9}

    with torch.inference_mode():
        main_run = measure_decode(args.batch, steps)
        result = {
            "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (GPT-2 124M)",
            "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": main_run["ms"] / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if dtype == torch.bfloat16 else "fp32", "data": "synthetic",
            "impl": "reference", "decode_attention_backend": backend,
            "config": {
                "model": args.model, "weights": "random(torch.manual_seed(0))", "n_layer": sizes["n_layer"],
                "n_layer_full": full_layers, "n_embd": hidden, "n_head": heads, "n_inner": inner,
                "vocab_size": vocab, "n_positions": context_len, "global_batch": args.batch,
                "seq_len": context_len, "prompt_len": args.prompt_len, "generated": steps, "block_size": 16,
                "parallelism": "single-gpu", "tokens": "uniform-random ids",
                "l2": "working set per step exceeds L2 (no flush)", "peaks": peaks["source"],
            },
            "clocks": {k: main_run["clocks"][k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            # every step of the reference builds its ids and positions on the host (int64), copies them and
            # its decode metadata to the device, and reads the argmax back (reference:
            # src/scheduler/orca_scheduler.py:214-219, 250)
            "e2e": {"value": main_run["e2e_tok_s"], "unit": "tokens/s", "ms_per_step": main_run["e2e_ms_per_step"],
                    "h2d_bytes_per_step": 2 * args.batch * 8, "d2h_bytes_per_step": args.batch * 8},
            "gpu_launches": None,                                  # none of this repository's kernels run in this arm
            "roofline": {"bound": "hbm", "achieved": main_run["bytes_per_step"] / (main_run["ms"] / steps / 1e3) / 1e9,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s"},
        }
        result["cuda_graphs"] = {key: value for key, value in model.cuda_graph_summary().items()
                                 if key in ("captured_graphs", "graph_replays", "capture_failures")}
        result["roofline"]["frac"] = result["roofline"]["achieved"] / result["roofline"]["peak"]
        if not args.small and not args.skip_prefill:
            result["prefill"] = measure_prefill(args.prefill_tokens)
        if not args.small and not args.skip_points:
            result["points"] = {"decode_b1": measure_decode(1, steps)["tok_s"],
                                "decode_b64": measure_decode(64, steps)["tok_s"]}
    return result


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--model", default="gpt2-124m")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--prompt-len", type=int, default=512)
    parser.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    parser.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    parser.add_argument("--skip-points", action="store_true")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--small", action="store_true", help="profiling aid: only the default decode measurement")
    parser.add_argument("--prefill-only", action="store_true", help="profiling aid: only the prefill measurement")
    parser.add_argument("--prefill-tokens", type=int, default=2048,
                        help="tokens of the prefill step, in prompts of 1,024 (1024: one single prompt)")
    parser.add_argument("--serving", type=int, default=0, metavar="REQUESTS",
                        help="instead of the decode measurement: this many requests (prompts U[64,1024), outputs "
                             "U[32,256]) through the scheduler, chunked prefill under a 2,048-token budget")
    args = parser.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 or world > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"error": "pagedserve_b200 is a single-GPU engine: bench.py runs at --gpus 1 only",
                              "n_gpus": max(args.gpus, world)}))
        return 2
    if args.impl == "reference":
        return reference_arm(args)

    import numpy as np
    import torch

    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.config.gpt2 import GPT2Config, NAMED_CONFIGS
    from pagedserve_b200.engine.batch import StepEntry
    from pagedserve_b200.engine.engine import Engine

    steps, warmup = args.steps, max(args.warmup, 3)
    sizes = dict(NAMED_CONFIGS[args.model])
    full_layers = sizes["n_layer"]
    if args.layers:
        sizes["n_layer"] = args.layers
    config = GPT2Config(**sizes)
    context_len = config.n_positions
    if args.prompt_len + warmup + steps + 2 > context_len:
        steps = context_len - args.prompt_len - warmup - 2
    peaks = load_peaks()

    max_batch = max(64, args.batch)
    pages = max_batch * (context_len // 16) + 64
    engine = Engine.random(config, 0, EngineConfig(dtype=args.dtype, block_size=16, num_blocks=pages,
                                                   max_num_seqs=max_batch, max_num_batched_tokens=2048))
    rng = np.random.default_rng(0)
    width = 2 if args.dtype == "bfloat16" else 4
    kv_bytes_per_token = 2 * config.n_layer * config.n_embd * width
    tensors = engine.model.tensors
    weight_bytes = sum(t.numel() * t.element_size() for name, t in tensors.items() if name != "wpe.weight")

    def prefill(batch, prompt_len, first_id):
        prompts = [rng.integers(0, config.vocab_size, prompt_len).tolist() for _ in range(batch)]
        tokens = []
        per_step = max(1, 2048 // prompt_len)
        for start in range(0, batch, per_step):
            chunk = range(start, min(batch, start + per_step))
            logits = engine.step([StepEntry(first_id + i, prompts[i], [prompt_len - 1]) for i in chunk])
            tokens += logits.argmax(-1).tolist()
        return tokens

    def measure_decode(batch, k_steps):
        ids = list(range(batch))
        tokens = prefill(batch, args.prompt_len, 0)
        entries = [StepEntry(i, [tokens[i]]) for i in ids]
        warm = engine.decode(entries, [0.0] * batch, [0] * batch, steps=warmup)
        entries = [StepEntry(i, [int(warm[-1, i])]) for i in ids]
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches_before = engine.ops.launches
        with ClockSampler() as clocks:
            torch.cuda.synchronize()
            start.record()
            out = engine.decode(entries, [0.0] * batch, [0] * batch, steps=k_steps)
            end.record()
            torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        graph = engine.runner._graphs.get((batch, "sample"))
        launches = (graph.kernels * k_steps) if graph else (engine.ops.launches - launches_before)
        mean_context = args.prompt_len + warmup + (k_steps + 1) / 2.0
        for i in ids:
            engine.finish(i)
        assert out.shape == (k_steps, batch)
        return {"ms": ms, "tok_s": batch * k_steps / (ms / 1e3), "launches": launches,
                "bytes_per_step": weight_bytes + batch * mean_context * kv_bytes_per_token,
                "clocks": clocks.summary()}

    def measure_e2e(batch, k_steps, repeats=3):
        """The same metric through the scheduler, one host round trip per step: the timed region of every step
        holds the upload of the step's inputs from pinned host memory and the read of its sampled tokens.
        Exactly k_steps are timed, ``repeats`` times over (fresh requests each time); the median is reported:
        one run alone moves by 10 % with the load of the host it happens to share."""
        import gc

        runs = []
        # requests whose prompts ran in an earlier step are that many tokens ahead: where the context has room,
        # everybody gets as many tokens more, so that nobody finishes inside the timed steps
        head_start = -(-batch * args.prompt_len // 2048) + 1
        spare = max(0, min(head_start, context_len - args.prompt_len - (warmup + k_steps + 2)))
        for _ in range(repeats):
            scheduler = engine.make_scheduler(strategy="orca", max_num_seqs=batch, max_num_batched_tokens=2048)
            for _ in range(batch):
                scheduler.add_token_request(rng.integers(0, config.vocab_size, args.prompt_len).tolist(),
                                            max_new_tokens=warmup + k_steps + 2 + spare)
            while scheduler.waiting:
                scheduler.step()                       # prefill (untimed)
            for _ in range(warmup):
                scheduler.step()
            gc.collect()
            gc.disable()
            try:
                torch.cuda.synchronize()
                began = time.perf_counter()
                produced = 0
                for _ in range(k_steps):
                    produced += len(scheduler.step())
                torch.cuda.synchronize()
                seconds = time.perf_counter() - began
            finally:
                gc.enable()
            h2d = engine.runner.h2d_bytes
            scheduler.run_until_complete()
            runs.append((produced / seconds, seconds * 1e3 / k_steps))
        runs.sort()
        value, ms = runs[len(runs) // 2]
        return {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": batch * 4, "ms_per_step": ms, "repeats": repeats,
                "ms_per_step_runs": [round(r[1], 4) for r in runs]}

    def measure_prefill(tokens_total=2048, repeats=5):
        prompt_len = min(1024, context_len)
        count = tokens_total // prompt_len
        times = []
        # the step shape is captured as a CUDA graph once it has come back a few times
        rehearsals = max(3, getattr(engine.runner, "MIXED_SHAPE_SIGHTINGS", 2) + 1)
        for repeat in range(repeats + rehearsals):
            prompts = [rng.integers(0, config.vocab_size, prompt_len).tolist() for _ in range(count)]
            entries = [StepEntry(1000 + i, prompts[i], [prompt_len - 1]) for i in range(count)]
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step(entries)
            end.record()
            torch.cuda.synchronize()
            if repeat >= rehearsals:
                times.append(start.elapsed_time(end))
            for i in range(count):
                engine.finish(1000 + i)
        ms = statistics.median(times)
        T = count * prompt_len
        H, I, L = config.n_embd, config.inner_dim, config.n_layer
        gemm = 2.0 * T * L * (3 * H * H + H * H + 2 * H * I) + 2.0 * count * H * config.vocab_size
        attention = L * count * 4.0 * H * (prompt_len * (prompt_len + 1) / 2.0)
        flops = gemm + attention
        peak = peaks["bf16_tflops"] * 1e12 if args.dtype == "bfloat16" else 75e12
        return {"value": T / (ms / 1e3), "tokens": T, "ms": ms, "frac": flops / (ms / 1e3) / peak,
                "gflop": flops / 1e9}

    def measure_serving(requests, max_seqs=64):
        """Continuous batching: every request is queued at time 0; a step holds the decode tokens of the running
        requests and prompt portions of waiting ones under the token budget.  The last of three passes is
        reported: the earlier ones meet most step shapes for the first few times (a shape that keeps coming
        back is captured as a CUDA graph, a step of about 5 ms)."""
        import gc

        for _ in range(3):
            scheduler = engine.make_scheduler(strategy="sarathi", max_num_seqs=max_seqs, max_num_batched_tokens=2048,
                                              prefill_chunk_size=512, max_prefills_per_step=4)
            prompt_tokens = 0
            for _ in range(requests):
                prompt_len = int(rng.integers(64, 1024))
                output_len = max(1, min(int(rng.integers(32, 257)), context_len - prompt_len))
                scheduler.add_token_request(rng.integers(0, config.vocab_size, prompt_len).tolist(),
                                            max_new_tokens=output_len)
                prompt_tokens += prompt_len
            step_ms, produced = [], 0
            gc.collect()
            gc.disable()                   # a collection of the oldest generation in mid-pass is one long step
            try:
                torch.cuda.synchronize()
                began = time.perf_counter()
                while scheduler.waiting or scheduler.active:
                    before = time.perf_counter()
                    produced += len(scheduler.step())
                    step_ms.append((time.perf_counter() - before) * 1e3)
                torch.cuda.synchronize()
                seconds = time.perf_counter() - began
            finally:
                gc.enable()
            engine.cache.check_invariants()
        step_ms.sort()
        return {"impl": "ours", "workload": "continuous batching", "model": args.model, "dtype": args.dtype,
                "requests": requests, "max_num_seqs": max_seqs, "max_num_batched_tokens": 2048,
                "prompt_tokens": prompt_tokens, "output_tokens": produced, "seconds": seconds,
                "output_tok_s": produced / seconds, "total_tok_s": (prompt_tokens + produced) / seconds,
                "steps": len(step_ms), "step_ms_median": step_ms[len(step_ms) // 2],
                "step_ms_p90": step_ms[int(len(step_ms) * 0.9)], "step_ms_max": step_ms[-1]}

    if args.prefill_only:
        print(json.dumps({"impl": "ours", "prefill": measure_prefill(args.prefill_tokens, repeats=3)}))
        return 0
    if args.serving:
        print(json.dumps(measure_serving(args.serving)))
        return 0
    main_run = measure_decode(args.batch, steps)
    e2e = measure_e2e(args.batch, steps)
    result = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (GPT-2 124M)",
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main_run["ms"] / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": args.model, "weights": "random(seed 0)", "n_layer": config.n_layer,
            "n_layer_full": full_layers, "n_embd": config.n_embd, "n_head": config.n_head,
            "n_inner": config.inner_dim, "vocab_size": config.vocab_size, "n_positions": config.n_positions,
            "global_batch": args.batch, "seq_len": context_len, "prompt_len": args.prompt_len,
            "generated": steps, "block_size": 16, "parallelism": "single-gpu",
            "tokens": "uniform-random ids", "l2": "working set per step exceeds L2 (no flush)",
            "peaks": peaks["source"],
        },
        "clocks": {k: main_run["clocks"][k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
        "e2e": e2e,
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": main_run["bytes_per_step"] / (main_run["ms"] / steps / 1e3) / 1e9,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s"},
    }
    result["roofline"]["frac"] = result["roofline"]["achieved"] / result["roofline"]["peak"]
    if not args.small and not args.skip_prefill:
        result["prefill"] = measure_prefill(args.prefill_tokens)
    if not args.small and not args.skip_points:
        result["points"] = {"decode_b1": measure_decode(1, steps)["tok_s"],
                            "decode_b64": measure_decode(64, steps)["tok_s"]}
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
