"""The CPU restatement of the sampling rule: Philox known answers, the greedy special case, distribution sanity."""
import numpy as np

from oracle import sampler
from tnsr_b200.nn import argmax_last


def test_philox4x32_10_known_answers():
    """The published known-answer vectors of Philox4x32-10 (counter, key -> output)."""
    assert sampler.philox4x32_10((0, 0, 0, 0), (0, 0)) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert sampler.philox4x32_10((0xFFFFFFFF,) * 4, (0xFFFFFFFF, 0xFFFFFFFF)) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert sampler.philox4x32_10((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0)) == \
        [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_top_k_one_is_the_greedy_pick_including_ties_and_signed_zeros():
    rng = np.random.default_rng(3)
    rows = rng.standard_normal((6, 97)).astype(np.float32)
    rows[1, [4, 50, 96]] = rows[1].max() + 1           # ties: the last index wins
    rows[2, :] = 0.0
    rows[2, 10] = -0.0                                 # +0 > -0 under totalOrder
    rows[3, :] = -np.inf
    for r, row in enumerate(rows):
        assert sampler.sample_row(row, 0.7, 1, 99, 5, r) == argmax_last(row)


def test_samples_follow_the_truncated_softmax():
    logits = np.asarray([2.0, 1.0, 0.0, -1.0, 3.0, 0.5], dtype=np.float32)
    counts = np.zeros(6)
    n = 6000
    for step in range(n):
        counts[sampler.sample_row(logits, 1.5, 3, 1234, step, 7)] += 1
    assert counts[[2, 3, 5]].sum() == 0                # outside the top 3
    p = np.exp((logits[[0, 1, 4]] - 3.0) / 1.5)
    p /= p.sum()
    assert np.max(np.abs(counts[[0, 1, 4]] / n - p)) < 0.02
    # same (seed, step, session) -> same draw; another session draws independently
    assert sampler.sample_row(logits, 1.5, 3, 1234, 11, 7) == sampler.sample_row(logits, 1.5, 3, 1234, 11, 7)
    a = [sampler.sample_row(logits, 1.5, 3, 1234, s, 7) for s in range(64)]
    b = [sampler.sample_row(logits, 1.5, 3, 1234, s, 8) for s in range(64)]
    assert a != b
