"""Seeded synthetic workloads shared by the tests, the fixture generator and the
benchmark.  Each function states its draw order so any harness can rebuild the
same bytes."""
import numpy as np

from tnsr_b200.nn import GptConfig
from tnsr_b200.synthetic import (config0_model, config0_prompt, config4, normal_model_arrays,  # noqa: F401
                                 set_model_arrays)  # re-exported for the tests


def kv_test_tokens(batch, length, vocab=367):
    """Token rows of tnsr's tests/kv_cache.rs:33-35."""
    return [[(i * 53 + b * 109 + 365) % vocab for i in range(length)] for b in range(batch)]


def attention_samples(n, salt, divisor=23.0, offset=2.0):
    """``((i * 17 + salt) % 101) / 23 - 2`` (src/nn/kv_cache/cuda/tests.rs:30-34)."""
    i = np.arange(n, dtype=np.int64)
    return (((i * 17 + salt) % 101).astype(np.float32) / np.float32(divisor) - np.float32(offset)).astype(np.float32)
