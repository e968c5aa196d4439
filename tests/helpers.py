"""Test-side glue: drives the shared GptDecoder wrapper with the CPU checker in
the role DecoderBackend::Cpu plays in tnsr (src/nn/kv_cache.rs:60-64)."""
import numpy as np

from tnsr_b200.nn import (Gpt, GptAttentionPrecision, GptConfig, GptDecoder, GptDecoderOptions,
                          TnsrError, argmax_last, model_parameters)


def kv_model(capacity, **overrides):
    """The model of tests/kv_cache.rs:7-17 with the reference initialiser."""
    cfg = dict(vocab_size=367, max_sequence_length=capacity, embed_dim=8, num_heads=2,
               feed_forward_dim=13, num_layers=2, layer_norm_epsilon=1e-5)
    cfg.update(overrides)
    return Gpt(GptConfig(**cfg))


def cpu_decoder(model, batch, capacity=None, options=GptDecoderOptions()):
    from oracle.oracle import OracleBackend
    config = model.config()
    capacity = config.max_sequence_length if capacity is None else capacity
    # construct the wrapper's guards first so invalid shapes raise TnsrError, as in the reference
    if not batch > 0:
        raise TnsrError("decoder batch size must be non-zero")
    if not (0 < capacity <= config.max_sequence_length):
        raise TnsrError("decoder capacity must fit the model context")
    if batch * capacity * config.embed_dim * 8 * config.num_layers > (1 << 40):
        # the checker really allocates; let the wrapper's own overflow guards speak
        return GptDecoder(model, None, batch, capacity, options, backend_impl=object())
    impl = OracleBackend(config, batch, capacity,
                         attention_bf16=options.attention_precision == GptAttentionPrecision.Bf16)
    return GptDecoder(model, None, batch, capacity, options, backend_impl=impl)


def cpu_forward(model, tokens):
    """Gpt::forward through the checker: logits [batch, seq, vocab]."""
    from oracle.oracle import OracleModel
    c = model.config()
    m = OracleModel(c.vocab_size, c.max_sequence_length, c.embed_dim, c.num_heads, c.feed_forward_dim,
                    c.num_layers, c.layer_norm_epsilon, c.activation)
    m.set_params([p.values() for p in model_parameters(model)])
    return m.forward(np.asarray(tokens, dtype=np.uint32))


def cpu_generate(model, prompt, max_new):
    """Gpt::generate (uncached greedy) through the checker."""
    from oracle.oracle import OracleModel
    c = model.config()
    if len(prompt) == 0:
        raise TnsrError("GPT generation prompt must be non-empty")
    if not all(t < c.vocab_size for t in prompt):
        raise TnsrError("GPT generation prompt contains an out-of-range token")
    m = OracleModel(c.vocab_size, c.max_sequence_length, c.embed_dim, c.num_heads, c.feed_forward_dim,
                    c.num_layers, c.layer_norm_epsilon, c.activation)
    m.set_params([p.values() for p in model_parameters(model)])
    return m.generate(prompt, max_new)


def generate_cached_with(model, make_decoder, prompt, max_new):
    """Gpt::generate_cached (src/nn/kv_cache.rs:121-157) over any decoder factory."""
    vocab = model.config().vocab_size
    if len(prompt) == 0:
        raise TnsrError("GPT generation prompt must be non-empty")
    if not all(t < vocab for t in prompt):
        raise TnsrError("GPT generation prompt contains an out-of-range token")
    tokens = list(prompt)
    if max_new == 0:
        return tokens
    decoder = make_decoder(model, 1)
    for _ in range(max_new):
        if decoder.is_empty() or decoder.len() == decoder.capacity():
            decoder.reset()
            logits = decoder.decode(tokens[max(0, len(tokens) - decoder.capacity()):])
        else:
            logits = decoder.decode(tokens[-1:])
        tokens.append(argmax_last(logits[logits.size - vocab:]))
    return tokens


def close(a, b, tol=2e-4):
    a, b = np.asarray(a).reshape(-1), np.asarray(b).reshape(-1)
    assert a.shape == b.shape
    assert np.all(np.isfinite(a)) and np.all(np.isfinite(b))
    worst = int(np.argmax(np.abs(a - b)))
    assert np.abs(a - b)[worst] <= tol, f"logit {worst}: {a[worst]} vs {b[worst]}"
