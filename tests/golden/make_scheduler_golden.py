"""Record what the reference's own scheduler puts into each step, on the CPU.

Run from the repository root, with a checkout of the reference as the argument:

    python tests/golden/make_scheduler_golden.py /path/to/reference

It builds the reference's ``ContinuousBatchScheduler`` with its small random model
(reference: main.py:136-254, ``model_name="reference"``), submits token requests
(reference: src/scheduler/orca_scheduler.py:85-117), and runs it to the end while noting for
every step the batch that ``build_iteration_batch`` made (:171-219): request, number of
tokens, and whether the entry produces a logits row; and, from the reference's ``KVCacheManager``
(src/model/kv_manager.py:115-127, 425-442), the ids of the pages each request was handed in that
step.  The end-of-sequence rule is switched
off on the scheduler object (as the reference's benchmarks do), so a request ends by its
token limit alone and the record does not depend on the model's weights.  Workloads are
chosen so that the page pool, not the batch size, is what makes requests wait: that is the
part of the reference's rules (worst-case reservation, head-of-line waiting, release at the
end; :119-169, 229-232, 268-277) that ``tests/test_scheduler_cpu.py`` checks this package's
scheduler against, from ``scheduler_steps.json`` written here.
"""

import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (strategy, prefill chunk, most requests per step, pool in MiB, [(prompt length, new tokens), ...])
WORKLOADS = {
    "orca_pages_run_out": ("orca", 16, 16, 1, [(40, 80), (70, 50), (5, 120), (100, 20), (33, 90), (17, 100), (90, 30),
                                                (64, 64), (1, 127), (110, 18), (50, 50), (25, 3), (80, 40), (12, 12)]),
    "sarathi_chunks_of_16": ("sarathi", 16, 16, 1, [(40, 80), (70, 50), (5, 100), (100, 28), (33, 90), (17, 25),
                                                    (96, 32), (64, 60), (2, 120), (120, 8), (30, 30), (9, 1)]),
    "sarathi_chunks_of_7": ("sarathi", 7, 12, 1, [(20, 100), (64, 60), (9, 110), (50, 70), (3, 120), (100, 5),
                                                  (45, 80), (7, 7), (77, 50), (14, 90)]),
}


def record(reference_root, strategy, chunk, max_batch, pool_mib, requests):
    if reference_root not in sys.path:
        sys.path.insert(0, reference_root)
    import torch

    import main as reference_main

    torch.manual_seed(0)
    scheduler = reference_main.build_scheduler(model_name="reference", scheduling_strategy=strategy,
                                               prefill_chunk_size=chunk, max_batch_size=max_batch,
                                               kv_cache_memory_mb=pool_mib)
    scheduler.eos_token_id = None
    vocabulary = scheduler.model_engine.config.vocab_size
    context = scheduler.model_engine.config.max_sequence_length
    steps = []
    build = scheduler.build_iteration_batch

    def noting(selected):
        batch = build(selected)
        steps.append([[item.request_id, len(item.token_ids), bool(item.produces_output)] for item in batch.items])
        return batch

    scheduler.build_iteration_batch = noting
    for index, (prompt_len, new_tokens) in enumerate(requests):
        assert prompt_len + new_tokens <= context
        scheduler.add_token_request([(7 * index + 3 * place + 1) % vocabulary for place in range(prompt_len)],
                                    max_new_tokens=new_tokens)
    finished_after = {}
    held = {}                  # request -> number of pages it held after the step before
    pages = []                 # per step: [request, the page ids it was handed in this step], by request
    while scheduler.waiting or scheduler.active:
        scheduler.step()
        for request_id in scheduler.finished:
            finished_after.setdefault(request_id, len(steps))
        tables = {request_id: list(info.block_ids) for request_id, info in scheduler.kv_manager.requests.items()}
        pages.append([[request_id, table[held.get(request_id, 0):]] for request_id, table in sorted(tables.items())
                      if len(table) > held.get(request_id, 0)])
        held = {request_id: len(table) for request_id, table in tables.items()}
    return {
        "strategy": strategy, "prefill_chunk_size": chunk, "max_batch_size": max_batch,
        "block_size": scheduler.kv_manager.block_size, "total_blocks": scheduler.kv_manager.total_available_blocks,
        "context": context, "requests": [list(request) for request in requests], "steps": steps,
        "finished_after_step": [finished_after[index] for index in range(len(requests))],
        "pages_handed_out": pages,
    }


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_scheduler_golden.py <path of a checkout of jainalphin/pagedserve>")
    records = {name: record(sys.argv[1], *workload) for name, workload in WORKLOADS.items()}
    for name, entry in records.items():
        waited = sum(1 for step in entry["steps"] if len(step) < min(entry["max_batch_size"], len(entry["requests"])))
        print(f"{name}: {len(entry['steps'])} steps, pool of {entry['total_blocks']} blocks of "
              f"{entry['block_size']}, {waited} steps with fewer entries than requests")
    with open(os.path.join(HERE, "scheduler_steps.json"), "w") as handle:
        json.dump(records, handle, separators=(",", ":"))


if __name__ == "__main__":
    main()
