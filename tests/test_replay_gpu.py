"""Replay of the same requests whole, with a decoded tail, in portions and mixed, compared
with the plain implementation, in float32 and in bfloat16."""

import pytest

import helpers

pytestmark = pytest.mark.gpu

LENGTHS = {"a": [5, 17, 33, 64, 100, 128], "b": [1, 9, 40, 64, 100, 200], "c": [3, 70, 129, 260, 384],
           "d": [2, 127, 128, 257, 300]}


def sequences(which):
    vocab = helpers.TINY[which][0]["vocab_size"]
    return {f"r{index}": helpers.random_tokens(vocab, length, seed=100 * index + 7)
            for index, length in enumerate(LENGTHS[which])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_replay_matches_plain(which, dtype, mode):
    seqs = sequences(which)
    want = helpers.plain_logits(which, seqs)
    block = helpers.TINY[which][2]
    if mode == "whole":
        steps = helpers.trace_whole(seqs)
    elif mode == "tail":
        steps = helpers.trace_tail(seqs, tail=32)
    elif mode == "chunks":
        steps = helpers.trace_chunks(seqs, seed=3)
    else:
        steps = helpers.trace_mixed(seqs, seed=5, live=4)
    got = helpers.replay(helpers.model_folder(which), dtype, steps, helpers.peak_tokens(steps), block_size=block)
    for name in seqs:
        helpers.assert_close(got[name], want[name], dtype, f"{mode}/{which}/{dtype}/{name}")
