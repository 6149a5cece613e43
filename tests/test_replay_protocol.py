"""The replay program's protocol, with a stand-in engine (no GPU): which file a step writes, in which
order the rows come, the ``done`` lines, requests given back at ``end``, steps without wanted logits."""

import io
import json

import numpy as np
import torch

from pagedserve_b200.engine import replay


class StandInEngine:
    """Logits row of a token = [request number, position, token id, 0 ...]: enough to see order and places."""

    vocab = 7

    def __init__(self):
        self.lengths = {}
        self.finished = []
        self.cache = self.lengths              # ``request in engine.cache``
        self.runner = self
        self.checks = 0
        self.batches = []

    def step(self, entries):
        rows = []
        self.batches.append([entry.request for entry in entries])
        for entry in entries:
            start = self.lengths.get(entry.request, 0)
            for place in entry.want:
                row = np.zeros(self.vocab, dtype=np.float32)
                row[:3] = (ord(entry.request) - ord("a"), start + place, int(entry.tokens[place]))
                rows.append(row)
            self.lengths[entry.request] = start + len(entry.tokens)
        return torch.from_numpy(np.stack(rows)) if rows else torch.zeros((0, self.vocab))

    def finish(self, request):
        self.finished.append(request)
        del self.lengths[request]

    def check_status(self):
        self.checks += 1


def run_trace(tmp_path, monkeypatch, steps, extra=()):
    from pagedserve_b200.engine import engine as engine_module

    made = {}

    def from_folder(folder, config):
        made["engine"], made["config"], made["folder"] = StandInEngine(), config, folder
        return made["engine"]

    monkeypatch.setattr(engine_module.Engine, "from_folder", staticmethod(from_folder))
    out = tmp_path / "out"
    args = replay.build_parser().parse_args(["--model", "MODEL", "--dtype", "float32", "--out", str(out),
                                             "--max-tokens", "200", *extra])
    printed = io.StringIO()
    lines = "".join(json.dumps(step) + "\n" for step in steps) + "\n"
    assert replay.run(args, stdin=io.StringIO(lines), stdout=printed) == 0
    return made, out, printed.getvalue()


def test_rows_files_and_done_lines(tmp_path, monkeypatch):
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]},
                                {"id": "b", "tokens": [9, 8], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": [4], "want": [0]}, {"id": "a", "tokens": [6], "want": [0]}],
         "end": ["a"]},
        {"step": 2, "entries": [{"id": "b", "tokens": [1, 2]}], "end": []},            # nothing wanted: no file
        {"step": 7, "entries": [{"id": "c", "tokens": [3, 3, 3], "want": [2]}], "end": ["b", "c", "zz"]},
    ]
    made, out, printed = run_trace(tmp_path, monkeypatch, steps)
    assert printed == "done 0\ndone 1\ndone 2\ndone 7\n"
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "1.f32", "7.f32"]
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, StandInEngine.vocab)
    assert first[:, :3].tolist() == [[0, 0, 5], [0, 2, 3]]                              # order of ``want``
    second = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, StandInEngine.vocab)
    assert second[:, :3].tolist() == [[1, 2, 4], [0, 3, 6]]                             # order of the entries
    last = np.fromfile(out / "7.f32", dtype="<f4").reshape(-1, StandInEngine.vocab)
    assert last[:, :3].tolist() == [[2, 2, 3]]
    engine = made["engine"]
    assert engine.batches == [["a", "b"], ["b", "a"], ["b"], ["c"]]                     # one batch per step
    assert engine.finished == ["a", "b", "c"]                                           # an unknown name is ignored
    assert engine.checks == 4


def test_pool_is_sized_from_max_tokens(tmp_path, monkeypatch):
    made, _, _ = run_trace(tmp_path, monkeypatch, [], extra=["--block-size", "8"])
    config = made["config"]
    assert made["folder"] == "MODEL" and config.dtype == "float32"
    assert config.block_size == 8 and config.num_blocks == 25                           # ceil(200 / 8)
    assert config.max_num_seqs >= 4
