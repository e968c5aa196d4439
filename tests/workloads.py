"""Seeded synthetic workloads shared by the tests, the fixture generator and the
benchmark.  Each function states its draw order so any harness can rebuild the
same bytes."""
import numpy as np

from tnsr_b200.nn import GptConfig


def normal_model_arrays(cfg: GptConfig, seed: int, std: float = 0.02, bias_std: float = 0.0):
    """Parameter arrays in ``model_parameters`` order.  One ``default_rng(seed)``
    stream; matrices are drawn N(0, std) in that order (float64 draws cast to
    f32); biases are 0 unless ``bias_std`` > 0 (then drawn in order too);
    LayerNorm weight 1, bias 0."""
    rng = np.random.default_rng(seed)
    d, f, V, ctx = cfg.embed_dim, cfg.feed_forward_dim, cfg.vocab_size, cfg.max_sequence_length

    def mat(r, c):
        return (rng.standard_normal((r, c)) * std).astype(np.float32)

    def bias(n):
        if bias_std > 0:
            return (rng.standard_normal(n) * bias_std).astype(np.float32)
        return np.zeros(n, np.float32)

    arrays = [mat(V, d), mat(ctx, d), np.ones(d, np.float32), np.zeros(d, np.float32)]
    for _ in range(cfg.num_layers):
        for _ in range(4):
            arrays += [mat(d, d), bias(d)]
        arrays += [np.ones(d, np.float32), np.zeros(d, np.float32), np.ones(d, np.float32),
                   np.zeros(d, np.float32)]
        if cfg.activation == "swiglu":
            arrays += [mat(d, f), bias(f), mat(d, f), bias(f), mat(f, d), bias(d)]
        else:
            arrays += [mat(d, f), bias(f), mat(f, d), bias(d)]
    return arrays


def config0_model(activation="relu"):
    cfg = GptConfig(vocab_size=96, max_sequence_length=128, embed_dim=128, num_heads=4,
                    feed_forward_dim=512, num_layers=4, layer_norm_epsilon=1e-5, activation=activation)
    return cfg, normal_model_arrays(cfg, seed=0)


def config0_prompt():
    return np.random.default_rng(1).integers(0, 96, size=16).astype(np.uint32)


def config4(num_layers=12, vocab_size=32000, max_sequence_length=2048):
    return GptConfig(vocab_size=vocab_size, max_sequence_length=max_sequence_length, embed_dim=768,
                     num_heads=12, feed_forward_dim=2048, num_layers=num_layers,
                     layer_norm_epsilon=1e-5, activation="swiglu", weight_dtype="bf16")


def set_model_arrays(model, arrays):
    from tnsr_b200.nn import model_parameters
    params = model_parameters(model)
    assert len(params) == len(arrays)
    for p, a in zip(params, arrays):
        p.set_values(a)


def kv_test_tokens(batch, length, vocab=367):
    """Token rows of tnsr's tests/kv_cache.rs:33-35."""
    return [[(i * 53 + b * 109 + 365) % vocab for i in range(length)] for b in range(batch)]


def attention_samples(n, salt, divisor=23.0, offset=2.0):
    """``((i * 17 + salt) % 101) / 23 - 2`` (src/nn/kv_cache/cuda/tests.rs:30-34)."""
    i = np.arange(n, dtype=np.int64)
    return (((i * 17 + salt) % 101).astype(np.float32) / np.float32(divisor) - np.float32(offset)).astype(np.float32)
