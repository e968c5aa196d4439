"""tnsr's tests/kv_cache.rs, CPU half, over the shared GptDecoder wrapper and
the CPU checker: session guards, chunk splits vs full forward, cached vs
uncached greedy generation, bf16 attention storage."""
import json

import numpy as np
import pytest

from tests.helpers import (close, cpu_decoder, cpu_forward, cpu_generate, generate_cached_with, kv_model)
from tests.workloads import kv_test_tokens
from tnsr_b200.nn import (Backend, GptAttentionPrecision, GptDecoderOptions, TnsrError)

USIZE_MAX = (1 << 64) - 1


def chunks_match(make_decoder, forward, tol=2e-4):
    """tests/kv_cache.rs:29-69."""
    model = kv_model(7)
    for batch in (1, 2):
        decoder = make_decoder(model, batch)
        rows = kv_test_tokens(batch, 7)
        for sizes in ([2, 1, 4], [1, 3, 3], [7]):
            decoder.reset()
            position = 0
            for chunk in sizes:
                tokens = [t for row in rows for t in row[position:position + chunk]]
                actual = decoder.decode(tokens)
                position += chunk
                full = forward(model, [row[:position] for row in rows])
                expected = full[:, position - chunk:position, :]
                close(actual, expected, tol)
                assert decoder.len() == position
            assert decoder.len() == 7
            with pytest.raises(TnsrError):
                decoder.decode([0] * batch)
    return True


def validate_inputs_and_weights(make_decoder, forward):
    """tests/kv_cache.rs:113-150."""
    model = kv_model(4)
    with pytest.raises(TnsrError):
        make_decoder(model, 0)
    with pytest.raises(TnsrError):
        make_decoder(model, 1, 0)
    with pytest.raises(TnsrError):
        make_decoder(model, 1, 5)
    decoder = make_decoder(model, 2, 3)
    assert (decoder.batch_size(), decoder.capacity()) == (2, 3)
    with pytest.raises(TnsrError):
        make_decoder(model, USIZE_MAX)
    assert decoder.is_empty()
    decoder.decode([365, 1])
    for invalid in ([], [0], [0, 367], [0] * 6):
        with pytest.raises(TnsrError):
            decoder.decode(invalid)
    assert decoder.len() == 1
    decoder.decode([2, 3])
    weights = model.token_embedding.values()
    weights[0] += 0.3
    model.token_embedding.set_values(weights)
    with pytest.raises(TnsrError) as err:
        decoder.decode([4, 5])
    assert "weights changed" in str(err.value)
    assert decoder.len() == 2
    decoder.reset()
    actual = decoder.decode([365, 1])
    close(actual, forward(model, [[365], [1]]))


def test_cpu_kv_cache_matches_full_decode_for_batches_and_chunks():
    assert chunks_match(cpu_decoder, cpu_forward, tol=0.0)  # the CPU path is bit-identical


def test_kv_cache_validates_inputs_and_requires_reset_after_weight_changes():
    validate_inputs_and_weights(cpu_decoder, cpu_forward)


def test_guard_messages_follow_the_reference():
    model = kv_model(4)
    decoder = cpu_decoder(model, 2, 3)
    cases = [([], "nonempty rectangular"), ([0], "nonempty rectangular"),
             ([0, 367], "outside the vocabulary"), ([0] * 8, "capacity exceeded")]
    for tokens, message in cases:
        with pytest.raises(TnsrError) as err:
            decoder.decode(tokens)
        assert message in str(err.value)
    for args, message in (((0, 3), "batch size must be non-zero"), ((1, 0), "must fit the model context"),
                          ((1, 5), "must fit the model context"), ((USIZE_MAX, 3), "overflow")):
        with pytest.raises(TnsrError) as err:
            cpu_decoder(model, *args)
        assert message in str(err.value)


def test_failed_execution_requires_reset():
    class Exploding:
        def __init__(self):
            self.fail = False
        def refresh(self, index, values):
            pass
        def reset(self):
            pass
        def decode(self, tokens, position):
            if self.fail:
                raise RuntimeError("device lost")
            return np.zeros(tokens.size * 367, np.float32)
    from tnsr_b200.nn import GptDecoder
    model = kv_model(4)
    impl = Exploding()
    decoder = GptDecoder(model, None, 1, 4, backend_impl=impl)
    decoder.decode([1])
    impl.fail = True
    with pytest.raises(RuntimeError):
        decoder.decode([2])
    impl.fail = False
    with pytest.raises(TnsrError) as err:
        decoder.decode([2])
    assert "reset the cache before reuse" in str(err.value)
    assert decoder.len() == 1
    decoder.reset()
    decoder.decode([2])
    assert decoder.len() == 1


def test_cpu_backend_is_refused_by_the_library():
    with pytest.raises(TnsrError):
        kv_model(4).decoder(Backend.Cpu, 1)


def test_only_changed_parameters_are_uploaded_again():
    uploads = []
    class Recording:
        def refresh(self, index, values):
            uploads.append(index)
        def reset(self):
            pass
        def decode(self, tokens, position):
            return np.zeros(tokens.size * 367, np.float32)
    from tnsr_b200.nn import GptDecoder, model_parameters
    model = kv_model(4)
    decoder = GptDecoder(model, None, 1, 4, backend_impl=Recording())
    assert uploads == list(range(len(model_parameters(model))))
    uploads.clear()
    decoder.decode([1])
    assert uploads == []
    model.final_norm_bias.set_values(np.ones(8, np.float32))
    decoder.reset()
    decoder.decode([1])
    assert uploads == [3]


def test_cached_generation_matches_greedy_sliding_context():
    """tests/kv_cache.rs:152-168."""
    model = kv_model(3)
    for prompt in ([365], [365, 2, 3], [365, 2, 3, 4, 5]):
        for new_tokens in (0, 1, 7):
            expected = cpu_generate(model, prompt, new_tokens)
            actual = generate_cached_with(model, cpu_decoder, prompt, new_tokens)
            assert actual == expected
    with pytest.raises(TnsrError):
        generate_cached_with(model, cpu_decoder, [], 1)
    with pytest.raises(TnsrError):
        generate_cached_with(model, cpu_decoder, [367], 0)


def test_cached_single_position_window_matches_uncached():
    """tests/kv_cache.rs:187-196."""
    model = kv_model(1)
    assert generate_cached_with(model, cpu_decoder, [365, 3], 4) == cpu_generate(model, [365, 3], 4)


def test_checker_generate_cached_matches_wrapper_loop():
    from oracle.oracle import OracleModel
    from tnsr_b200.nn import model_parameters
    model = kv_model(5)
    c = model.config()
    m = OracleModel(c.vocab_size, c.max_sequence_length, c.embed_dim, c.num_heads, c.feed_forward_dim,
                    c.num_layers, c.layer_norm_epsilon)
    m.set_params([p.values() for p in model_parameters(model)])
    for prompt in ([365], [365, 2, 3, 4, 5, 6, 7]):
        assert m.generate_cached(prompt, 9) == generate_cached_with(model, cpu_decoder, prompt, 9)
        assert m.generate_cached(prompt, 9) == m.generate(prompt, 9)


def test_reference_initialiser_matches_checker_model():
    """Gpt::new defaults built by the host mirror == the checker's own init."""
    from oracle.oracle import OracleModel
    from tnsr_b200.nn import model_parameters
    for activation in ("relu", "swiglu"):
        model = kv_model(6, activation=activation)
        c = model.config()
        m = OracleModel(c.vocab_size, c.max_sequence_length, c.embed_dim, c.num_heads, c.feed_forward_dim,
                        c.num_layers, c.layer_norm_epsilon, activation)
        m.init_reference()
        params = model_parameters(model)
        assert m.param_count() == len(params) == 4 + (18 if activation == "swiglu" else 16) * 2
        for i, p in enumerate(params):
            assert np.array_equal(m.get_param(i).view(np.uint32), p.values().view(np.uint32)), i


def test_bf16_cpu_cache_preserves_chunk_and_reset_semantics():
    """tests/kv_cache.rs:245-281."""
    model = kv_model(40)
    options = GptDecoderOptions(attention_precision=GptAttentionPrecision.Bf16)
    whole = cpu_decoder(model, 2, 40, options)
    chunked = cpu_decoder(model, 2, 40, options)
    tokens = [(i * 53 + 7) % 367 for i in range(66)]
    expected = whole.decode(tokens).reshape(2, 33, 367)
    for _ in range(2):
        start = 0
        for size in (16, 1, 16):
            chunk = [t for b in range(2) for t in tokens[b * 33 + start:b * 33 + start + size]]
            actual = chunked.decode(chunk)
            close(actual, expected[:, start:start + size, :])
            start += size
        chunked.reset()
    # bf16 storage really changes values relative to f32, and the cache holds bf16-representable rows
    plain = cpu_decoder(model, 2, 40).decode(tokens).reshape(2, 33, 367)
    assert np.max(np.abs(plain - expected)) > 0
    cache = whole._backend.read_cache(0)
    from oracle.oracle import bf16_round_np
    assert np.array_equal(cache, bf16_round_np(cache))
    assert np.all(cache[:, 33:] == 0)


@pytest.mark.parametrize("activation", ["gelu", "swiglu"])
def test_extension_activations_decode_equals_forward(activation):
    model = kv_model(9, activation=activation)
    decoder = cpu_decoder(model, 2)
    rows = kv_test_tokens(2, 9)
    position = 0
    for chunk in (4, 1, 1, 3):
        tokens = [t for row in rows for t in row[position:position + chunk]]
        actual = decoder.decode(tokens)
        position += chunk
        full = cpu_forward(model, [row[:position] for row in rows])
        close(actual, full[:, position - chunk:position, :], 0.0)


def test_config0_golden_tokens_are_reproducible(oracle):
    import json, os
    from tests.workloads import config0_model, config0_prompt
    with open(os.path.join(os.path.dirname(__file__), "golden", "config0_greedy.json")) as f:
        golden = json.load(f)
    cfg, arrays = config0_model("relu")
    m = oracle.OracleModel(cfg.vocab_size, cfg.max_sequence_length, cfg.embed_dim, cfg.num_heads,
                           cfg.feed_forward_dim, cfg.num_layers, cfg.layer_norm_epsilon, "relu")
    m.set_params(arrays)
    assert list(config0_prompt()) == golden["relu"]["prompt"]
    assert m.generate_cached(config0_prompt(), 64) == golden["relu"]["tokens"]
    assert golden["relu"]["min_top1_top2_margin"] > 1e-3


def test_threads_do_not_change_results(oracle):
    from tests.workloads import config0_model
    cfg, arrays = config0_model("relu")
    m = oracle.OracleModel(cfg.vocab_size, cfg.max_sequence_length, cfg.embed_dim, cfg.num_heads,
                           cfg.feed_forward_dim, cfg.num_layers, cfg.layer_norm_epsilon, "relu")
    m.set_params(arrays)
    tokens = np.arange(2 * 24, dtype=np.uint32).reshape(2, 24) % 96
    oracle.set_threads(1)
    one = m.forward(tokens)
    oracle.set_threads(4)
    try:
        many = m.forward(tokens)
    finally:
        oracle.set_threads(1)
    assert np.array_equal(one.view(np.uint32), many.view(np.uint32))


def test_decoder_state_round_trips_through_the_archive(tmp_path):
    """Serialised decoder state (what docs/kv-cache.md:94-95 leaves outside the reference's API): a session saved after
    a prefix and restored into a fresh session continues exactly as the uninterrupted one; mismatched shapes and
    foreign archives are refused and leave the target usable."""
    from tnsr_b200.parameters import save_gpt
    model = kv_model(16)
    rows = kv_test_tokens(2, 11)
    flat = lambda lo, hi: [t for r in rows for t in r[lo:hi]]
    straight = cpu_decoder(model, 2)
    straight.decode(flat(0, 7))
    expected = straight.decode(flat(7, 11))

    first = cpu_decoder(model, 2)
    first.decode(flat(0, 7))
    first.save_state(str(tmp_path / "state"))
    manifest = json.load(open(tmp_path / "state" / "manifest.json"))
    assert manifest["config"]["length"] == 7 and manifest["tensors"][0]["shape"] == [2, 7, 8]
    assert [t["name"] for t in manifest["tensors"]][:2] == ["cache.0000.key", "cache.0000.value"]

    second = cpu_decoder(model, 2)
    second.decode(flat(0, 3))                      # previous contents are discarded by the load
    second.load_state(str(tmp_path / "state"))
    assert second.len() == 7
    assert np.array_equal(second.decode(flat(7, 11)).view(np.uint32), expected.view(np.uint32))

    empty = cpu_decoder(model, 2)
    empty.save_state(str(tmp_path / "empty"))
    second.load_state(str(tmp_path / "empty"))
    assert second.is_empty()

    with pytest.raises(TnsrError):
        cpu_decoder(model, 3).load_state(str(tmp_path / "state"))          # other batch
    with pytest.raises(TnsrError):
        cpu_decoder(model, 2, 5).load_state(str(tmp_path / "state"))       # 7 rows do not fit 5
    save_gpt(model, str(tmp_path / "weights"))
    with pytest.raises(TnsrError):
        second.load_state(str(tmp_path / "weights"))                       # a parameter archive, not a state
    second.decode(flat(0, 2))                                              # still usable
