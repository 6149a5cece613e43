"""Trace replay: feed given token ids through the model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps are read from standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry of a step is run in one batch through the engine's own step function
(the one generation uses): same model, cache manager and kernels.  Nothing is
sampled.  For a step in which logits are wanted, ``OUT/<step>.f32`` holds them
as little-endian float32 ``[wanted, vocab]`` in the order of the entries and of
their ``want`` lists.  After every step the line ``done <step>`` is printed and
flushed.  Requests named in ``end`` give back their pages and slot after the step.

The page pool is sized for ``--max-tokens`` tokens (rounded up to whole pages), so
that pages of finished requests are handed out again.
"""

from __future__ import annotations

import argparse
import json
import os
import sys



def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (sizes the page pool)")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per KV page (default 16)")
    parser.add_argument("--max-num-seqs", type=int, default=16, help="request slots (default 16)")
    parser.add_argument("--disable-cuda-graphs", action="store_true")
    return parser


def run(args, stdin=None, stdout=None) -> int:
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.batch import StepEntry
    from pagedserve_b200.engine.engine import Engine

    if args.max_tokens <= 0:
        raise SystemExit("--max-tokens must be positive")
    os.makedirs(args.out, exist_ok=True)
    pages = -(-args.max_tokens // args.block_size)
    config = EngineConfig(dtype=args.dtype, block_size=args.block_size, num_blocks=pages,
                          max_num_seqs=args.max_num_seqs, max_num_batched_tokens=4096,
                          enable_cuda_graphs=not args.disable_cuda_graphs)
    engine = Engine.from_folder(args.model, config)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(item["id"], item["tokens"], item.get("want", ()))
                   for item in record.get("entries", ())]
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                rows = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                with open(os.path.join(args.out, f"{step}.f32"), "wb") as handle:
                    handle.write(rows.tobytes())
        for request in record.get("end", ()):
            if request in engine.cache:
                engine.finish(request)
        engine.runner.check_status()
        stdout.write(f"done {step}\n")
        stdout.flush()
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return run(args)


if __name__ == "__main__":
    sys.exit(main())
