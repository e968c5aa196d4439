"""Seeded synthetic model weights for benchmarks, examples and tests: there is no
network for checkpoints, so every workload draws its parameters from a stated
generator in a stated order and any harness can rebuild the same bytes."""
import numpy as np

from .nn import GptConfig


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
    from .nn import model_parameters
    params = model_parameters(model)
    assert len(params) == len(arrays)
    for p, a in zip(params, arrays):
        p.set_values(a)
