"""tnsr's tests/kv_cache.rs, CUDA half, and the configuration-level parity
checks: the B200 session behind the shared GptDecoder wrapper against the CPU
checker on the same weights and token ids."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from tests.gpu_util import bf16_round, rel_err  # noqa: E402
from tests.helpers import close, cpu_decoder, cpu_forward, cpu_generate, kv_model  # noqa: E402
from tests.test_kv_cache_host import chunks_match, validate_inputs_and_weights  # noqa: E402
from tests.workloads import (config0_model, config0_prompt, kv_test_tokens, normal_model_arrays,  # noqa: E402
                             set_model_arrays)
from tnsr_b200.nn import (Backend, Gpt, GptAttentionPrecision, GptConfig, GptDecoder, GptDecoderOptions,  # noqa: E402
                          argmax_last,
                          GptPrefillMode, model_parameters)
from tnsr_b200.session import B200Session  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def gpu_decoder(model, batch, capacity=None, options=GptDecoderOptions()):
    capacity = model.config().max_sequence_length if capacity is None else capacity
    return model.decoder_with_options(Backend.Ptx, batch, capacity, options)


def test_cuda_kv_cache_matches_full_decode_for_batches_and_chunks():
    """tests/kv_cache.rs:92-98 (tolerance 2e-4 absolute, :19-27)."""
    assert chunks_match(gpu_decoder, cpu_forward, tol=2e-4)


def test_cuda_kv_cache_reset_refreshes_weights_and_reuses_programs():
    """tests/kv_cache.rs:100-106."""
    validate_inputs_and_weights(gpu_decoder, cpu_forward)


def test_cuda_cached_generation_matches_sliding_context():
    """tests/kv_cache.rs:170-185."""
    model = kv_model(3)
    prompt = [365, 2, 3, 4]
    assert model.generate_cached(Backend.Ptx, prompt, 6) == cpu_generate(model, prompt, 6)
    assert kv_model(1).generate_cached(Backend.Cuda, [365, 3], 4) == cpu_generate(kv_model(1), [365, 3], 4)


def test_cuda_kv_cache_crosses_scan_tiles_with_one_session():
    """tests/kv_cache.rs:198-243: 140 single-token steps, batch 2, twice with reset."""
    model = kv_model(140)
    batch = 2
    rows = kv_test_tokens(batch, 140)
    decoder = gpu_decoder(model, batch)
    checked = {0, 1, 30, 31, 32, 33, 62, 63, 64, 65, 126, 127, 128, 129, 139}
    expected = {p: cpu_forward(model, [r[:p + 1] for r in rows])[:, p, :] for p in checked}
    for _ in range(2):
        decoder.reset()
        for position in range(140):
            actual = decoder.decode([r[position] for r in rows])
            if position in checked:
                close(actual, expected[position])


def test_strict_session_cache_rows_match_checker():
    """The appended K/V rows (src/nn/kv_cache.rs:347-361) and untouched slots."""
    model = kv_model(12)
    rows = kv_test_tokens(2, 9)
    gpu, cpu = gpu_decoder(model, 2), cpu_decoder(model, 2)
    for lo, hi in ((0, 4), (4, 5), (5, 9)):
        tokens = [t for r in rows for t in r[lo:hi]]
        close(gpu.decode(tokens), cpu.decode(tokens))
    for index in range(4):
        a, b = gpu._backend.read_cache(index), cpu._backend.read_cache(index)
        assert np.max(np.abs(a - b)) <= 2e-6
        assert np.all(a[:, 9:] == 0)


@pytest.mark.parametrize("width", [8, 66, 128, 258])
def test_bf16_cuda_cache_matches_cpu_for_prefill_decode_and_reset(width):
    """tests/kv_cache.rs:283-333: GptAttentionPrecision::Bf16 on f32 weights, tolerance max|expected|/128."""
    model = Gpt(GptConfig(vocab_size=32, max_sequence_length=160, embed_dim=width, num_heads=2,
                          feed_forward_dim=width * 2, num_layers=2, layer_norm_epsilon=1e-5))
    for prefill in (GptPrefillMode.Scalar, GptPrefillMode.Auto):
        options = GptDecoderOptions(attention_precision=GptAttentionPrecision.Bf16, prefill=prefill)
        cpu, gpu = cpu_decoder(model, 2, 160, options), gpu_decoder(model, 2, 160, options)
        for _ in range(2):
            sizes = [17, 1, 17, 3, 16, 75, 1] if width == 8 else [17, 1, 17, 3, 16]
            for size in sizes:
                tokens = [(i * 17 + cpu.len() + 3) % 32 for i in range(2 * size)]
                expected = cpu.decode(tokens)
                actual = gpu.decode(tokens)
                scale = max(1.0, float(np.max(np.abs(expected))))
                assert np.all(np.isfinite(actual))
                assert np.max(np.abs(actual - expected)) <= scale / 128
            gpu.reset()
            cpu.reset()


@pytest.mark.parametrize("activation", ["relu", "gelu"])
def test_config0_greedy_tokens_bit_exact_and_logits_within_1e3(activation, oracle):
    """Configuration 0: vocab 96, d 128, 4 layers, 4 heads, FFN 512, ctx 128, f32;
    prompt 16 + 64 greedy steps.  Token ids must equal the CPU executor's
    (fixture made by tests/golden/make_golden.py); logits within 1e-3 relative."""
    with open(os.path.join(GOLDEN, "config0_greedy.json")) as f:
        golden = json.load(f)[activation]
    cfg, arrays = config0_model(activation)
    model = Gpt(cfg)
    set_model_arrays(model, arrays)
    prompt = [int(t) for t in config0_prompt()]
    assert prompt == golden["prompt"]
    tokens = model.generate_cached(Backend.Cuda, prompt, 64)
    assert tokens == golden["tokens"]
    # logits of every step against the checker run on the same ids
    m = oracle.OracleModel(cfg.vocab_size, cfg.max_sequence_length, cfg.embed_dim, cfg.num_heads,
                           cfg.feed_forward_dim, cfg.num_layers, cfg.layer_norm_epsilon, activation)
    m.set_params(arrays)
    full = m.forward(np.asarray(tokens[:-1], np.uint32)[None])[0]          # [79, 96]
    decoder = model.decoder(Backend.Cuda, 1)
    got = [decoder.decode(prompt).reshape(16, 96)]
    for t in tokens[16:-1]:
        got.append(decoder.decode([t]).reshape(1, 96))
    got = np.concatenate(got)
    assert rel_err(got, full) <= 1e-3
    assert np.array_equal(full[-1].view(np.uint32), np.asarray(golden["last_logits_bits"], np.uint32))
    margins = np.sort(full[15:], axis=1)
    print(f"config0[{activation}] max rel err {rel_err(got, full):.3e}; min top1-top2 margin "
          f"{float((margins[:, -1] - margins[:, -2]).min()):.4f}")


def small_bf16_model(activation="swiglu", d=128, heads=2, f=256, vocab=512, ctx=96, layers=2, seed=21, bias_std=0.02):
    cfg = GptConfig(vocab_size=vocab, max_sequence_length=ctx, embed_dim=d, num_heads=heads, feed_forward_dim=f,
                    num_layers=layers, layer_norm_epsilon=1e-5, activation=activation, weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=seed, std=0.05, bias_std=bias_std)
    # the checker runs the f32 arithmetic on the bf16-rounded matrices (vectors stay f32)
    rounded = [bf16_round(a) if a.ndim == 2 else a for a in arrays]
    model = Gpt(cfg)
    set_model_arrays(model, arrays)
    return cfg, model, rounded


def oracle_model(oracle, cfg, arrays):
    m = oracle.OracleModel(cfg.vocab_size, cfg.max_sequence_length, cfg.embed_dim, cfg.num_heads, cfg.feed_forward_dim,
                           cfg.num_layers, cfg.layer_norm_epsilon, cfg.activation)
    m.set_params(arrays)
    return m


@pytest.mark.parametrize("engine", [1, 0])
@pytest.mark.parametrize("activation,d,heads,f", [("swiglu", 128, 2, 256), ("relu", 128, 2, 256), ("gelu", 96, 3, 104),
                                                  ("swiglu", 64, 2, 40), ("swiglu", 72, 3, 36), ("swiglu", 256, 2, 264)])
def test_bf16_session_matches_checker_within_2e2(oracle, activation, d, heads, f, engine):
    """bf16 tensor-core path vs the f32 checker on bf16-rounded weights: <= 2e-2 relative."""
    from tnsr_b200 import _native
    cfg, model, rounded = small_bf16_model(activation, d, heads, f)
    m = oracle_model(oracle, cfg, rounded)
    rng = np.random.default_rng(5)
    batch, total = 3, 40
    ids = rng.integers(0, cfg.vocab_size, size=(batch, total)).astype(np.uint32)
    full = m.forward(ids)
    try:
        _native.lib().tnsr_b200_set_gemm_engine(engine)
        decoder = model.decoder(Backend.Cuda, batch)
        position = 0
        for chunk in (17, 1, 1, 5, 16):
            tokens = ids[:, position:position + chunk].reshape(-1).tolist()
            got = decoder.decode(tokens).reshape(batch, chunk, cfg.vocab_size)
            assert np.all(np.isfinite(got))
            assert rel_err(got, full[:, position:position + chunk]) <= 2e-2
            position += chunk
    finally:
        _native.lib().tnsr_b200_set_gemm_engine(0)


@pytest.mark.parametrize("heads", [2, 1])
def test_bf16_session_long_chunks_take_the_tcgen05_prefill_kernel(oracle, heads):
    """Chunks of 32 rows and more at head width 64 (and 128: generic kernel) against the checker: the first at position 0,
    the second on top of 41 cached rows, with a single-token step in between."""
    cfg, model, rounded = small_bf16_model("swiglu", 128, heads, 256)
    m = oracle_model(oracle, cfg, rounded)
    rng = np.random.default_rng(8)
    batch, total = 3, 74
    ids = rng.integers(0, cfg.vocab_size, size=(batch, total)).astype(np.uint32)
    full = m.forward(ids)
    decoder = model.decoder(Backend.Cuda, batch)
    position = 0
    for chunk in (40, 1, 33):
        tokens = ids[:, position:position + chunk].reshape(-1).tolist()
        got = decoder.decode(tokens).reshape(batch, chunk, cfg.vocab_size)
        assert np.all(np.isfinite(got))
        assert rel_err(got, full[:, position:position + chunk]) <= 2e-2
        position += chunk


def test_bf16_session_logits_modes_argmax_and_device_loop(oracle):
    cfg, model, rounded = small_bf16_model("swiglu", 128, 2, 256, vocab=300)
    params = [p.values() for p in model_parameters(model)]
    rng = np.random.default_rng(6)
    batch, prompt_len, steps = 4, 9, 12
    prompt = rng.integers(0, cfg.vocab_size, size=(batch, prompt_len)).astype(np.uint32)

    def session(mode):
        s = B200Session(cfg, batch, cfg.max_sequence_length, logits_mode=mode)
        for i, p in enumerate(params):
            s.refresh(i, p)
        return s

    all_s, last_s, none_s = session("all"), session("last"), session("none")
    la, aa = all_s.decode_full(prompt, 0)
    ll, al = last_s.decode_full(prompt, 0)
    ln, an = none_s.decode_full(prompt, 0)
    assert ln is None
    la = la.reshape(batch, prompt_len, cfg.vocab_size)
    assert np.array_equal(la[:, -1].reshape(-1).view(np.uint32), ll.view(np.uint32))
    assert aa.tolist() == al.tolist() == an.tolist()
    assert aa.tolist() == [oracle.argmax_last(la[b, -1]) for b in range(batch)]
    # host-driven greedy loop vs device-resident loop (ids never leave the GPU)
    host_tokens = [aa.copy()]
    for step in range(steps):
        _, nxt = last_s.decode_full(host_tokens[-1].reshape(batch, 1), prompt_len + step)
        host_tokens.append(nxt.copy())
    cur = torch.from_numpy(an.astype(np.int32)).cuda()
    trace = [cur.clone()]
    for step in range(steps):
        none_s.decode_device(cur.data_ptr(), 1, prompt_len + step, cur.data_ptr())
        none_s.synchronize()
        trace.append(cur.clone())
    dev_tokens = [t.cpu().numpy().astype(np.uint32) for t in trace]
    assert [t.tolist() for t in dev_tokens] == [t.tolist() for t in host_tokens]


def test_bf16_session_rejects_bad_ids_on_the_device_path():
    from tnsr_b200.nn import TnsrError
    cfg, model, _ = small_bf16_model("relu", 64, 2, 64, vocab=50)
    s = B200Session(cfg, 2, 16, logits_mode="none")
    for i, p in enumerate(model_parameters(model)):
        s.refresh(i, p.values())
    bad = torch.tensor([3, 50], dtype=torch.int32, device="cuda")
    out = torch.zeros(2, dtype=torch.int32, device="cuda")
    s.decode_device(bad.data_ptr(), 1, 0, out.data_ptr())
    with pytest.raises(TnsrError) as err:
        s.synchronize()
    assert "outside the vocabulary" in str(err.value)
    s.reset()
    good = torch.tensor([3, 49], dtype=torch.int32, device="cuda")
    s.decode_device(good.data_ptr(), 1, 0, out.data_ptr())
    s.synchronize()
    with pytest.raises(TnsrError):
        s.decode_full(np.asarray([[1], [50]], np.uint32), 1)   # host path validates before any device work
    with pytest.raises(TnsrError):
        s.decode_full(np.zeros((2, 17), np.uint32), 0)         # capacity


def test_serving_shape_two_layers_against_checker(oracle):
    """Configuration 4's layer shape (d 768, 12 heads x 64, SwiGLU 2048, vocab 32000) with 2 layers:
    prefill 70 tokens then greedy decode, 4 sessions, against the checker on bf16-rounded weights."""
    cfg = GptConfig(vocab_size=32000, max_sequence_length=128, embed_dim=768, num_heads=12, feed_forward_dim=2048,
                    num_layers=2, layer_norm_epsilon=1e-5, activation="swiglu", weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=5, std=0.02)
    rounded = [bf16_round(a) if a.ndim == 2 else a for a in arrays]
    model = Gpt(cfg)
    set_model_arrays(model, arrays)
    m = oracle_model(oracle, cfg, rounded)
    rng = np.random.default_rng(50)
    batch, prefill, steps = 4, 70, 6
    ids = rng.integers(0, cfg.vocab_size, size=(batch, prefill)).astype(np.uint32)
    s = B200Session(cfg, batch, 128, logits_mode="last")
    for i, p in enumerate(model_parameters(model)):
        s.refresh(i, p.values())
    oracle.set_threads(oracle.max_threads())
    try:
        seq = ids.copy()
        logits, nxt = s.decode_full(ids, 0)
        for step in range(steps):
            full = m.forward(seq)[:, -1]
            got = logits.reshape(batch, cfg.vocab_size)
            assert rel_err(got, full) <= 2e-2
            ref_next = [oracle.argmax_last(full[b]) for b in range(batch)]
            top2 = np.sort(full, axis=1)[:, -2:]
            margin = top2[:, 1] - top2[:, 0]
            for b in range(batch):
                if margin[b] > 0.05 * float(np.max(np.abs(full[b]))):
                    assert int(nxt[b]) == ref_next[b]
            seq = np.concatenate([seq, nxt.reshape(batch, 1).astype(np.uint32)], axis=1)
            logits, nxt = s.decode_full(nxt.reshape(batch, 1), prefill + step)
    finally:
        oracle.set_threads(1)


def test_graph_replay_of_single_token_steps_matches_direct_launches(monkeypatch):
    """Single-token steps are replayed from a captured CUDA graph with the position in device memory;
    the result must be bit-identical to launching the same kernels one by one."""
    cfg, model, _ = small_bf16_model("swiglu", 128, 2, 256, vocab=300)
    params = [p.values() for p in model_parameters(model)]
    rng = np.random.default_rng(16)
    batch, prompt_len, steps = 3, 7, 9
    prompt = rng.integers(0, cfg.vocab_size, size=(batch, prompt_len)).astype(np.uint32)

    def run(no_graph):
        if no_graph:
            monkeypatch.setenv("TNSR_B200_NO_GRAPH", "1")
        else:
            monkeypatch.delenv("TNSR_B200_NO_GRAPH", raising=False)
        s = B200Session(cfg, batch, cfg.max_sequence_length, logits_mode="last")
        for i, p in enumerate(params):
            s.refresh(i, p)
        logits, ids = s.decode_full(prompt, 0)
        trace = [logits.copy()]
        for step in range(steps):
            logits, ids = s.decode_full(ids.reshape(batch, 1), prompt_len + step)
            trace.append(logits.copy())
        # jump back: a replay must honour whatever position the caller passes
        logits, _ = s.decode_full(prompt[:, :1], prompt_len + 2)
        trace.append(logits.copy())
        s.close()
        return trace

    a, b = run(False), run(True)
    for x, y in zip(a, b):
        assert np.array_equal(x.view(np.uint32), y.view(np.uint32))


@pytest.mark.parametrize("kv_bf16", [False, True])
def test_graph_replay_on_the_strict_f32_path_matches_direct_launches(monkeypatch, kv_bf16):
    """The strict path replays single-token steps from a graph too; logits must be bit-identical to direct launches and,
    as everywhere on this path, the greedy ids must equal the CPU checker's."""
    from tests.workloads import config0_model, config0_prompt
    cfg, arrays = config0_model("relu")
    prompt = config0_prompt().reshape(1, -1)
    steps = 20

    def run(no_graph):
        if no_graph:
            monkeypatch.setenv("TNSR_B200_NO_GRAPH", "1")
        else:
            monkeypatch.delenv("TNSR_B200_NO_GRAPH", raising=False)
        s = B200Session(cfg, 1, cfg.max_sequence_length, options=GptDecoderOptions(
            attention_precision=GptAttentionPrecision.Bf16 if kv_bf16 else GptAttentionPrecision.F32))
        for i, a in enumerate(arrays):
            s.refresh(i, a)
        logits, ids = s.decode_full(prompt, 0)
        trace, tokens = [logits.copy()], [int(ids[0])]
        for step in range(steps):
            logits, ids = s.decode_full(ids.reshape(1, 1), prompt.shape[1] + step)
            trace.append(logits.copy())
            tokens.append(int(ids[0]))
        logits, _ = s.decode_full(prompt[:, :1], prompt.shape[1] + 3)     # jump back
        trace.append(logits.copy())
        s.close()
        return trace, tokens

    (a, ta), (b, tb) = run(False), run(True)
    assert ta == tb
    for x, y in zip(a, b):
        assert np.array_equal(x.view(np.uint32), y.view(np.uint32))


@pytest.mark.parametrize("logits_mode", ["last", "none"])
def test_ragged_decode_every_session_at_its_own_position(logits_mode):
    """tnsr_b200_decoder_decode_ragged: after a common 12-token prefill, session b is rewound by 3 b tokens and all
    sessions then advance together from different positions.  Each must reproduce a batch-1 session of the same library
    that was prefilled with exactly its own prefix (bit for bit in the greedy ids, and logits within the bf16 tolerance),
    and the CPU checker on bf16-rounded weights within 2e-2."""
    cfg, model, rounded_arrays = small_bf16_model("swiglu", 128, 2, 256, vocab=300)
    params = [p.values() for p in model_parameters(model)]
    rng = np.random.default_rng(21)
    batch, prompt_len, steps = 4, 12, 6
    prompt = rng.integers(0, cfg.vocab_size, size=(batch, prompt_len)).astype(np.uint32)
    feed = rng.integers(0, cfg.vocab_size, size=(steps, batch)).astype(np.uint32)
    starts = np.array([prompt_len - 3 * b for b in range(batch)], dtype=np.uint32)      # 12, 9, 6, 3

    def session(b, mode):
        s = B200Session(cfg, b, cfg.max_sequence_length, logits_mode=mode)
        for i, p in enumerate(params):
            s.refresh(i, p)
        return s

    ragged = session(batch, logits_mode)
    ragged.decode_full(prompt, 0)
    got_logits, got_ids = [], []
    for t in range(steps):
        logits, ids = ragged.decode_ragged(feed[t], starts + t)
        got_logits.append(None if logits is None else logits.reshape(batch, -1).copy())
        got_ids.append(ids.copy())
    ragged.close()

    for b in range(batch):
        single = session(1, "last")
        single.decode_full(prompt[b:b + 1, :int(starts[b])], 0)
        for t in range(steps):
            logits, ids = single.decode_full(feed[t, b].reshape(1, 1), int(starts[b]) + t)
            assert int(ids[0]) == int(got_ids[t][b])
            if got_logits[t] is not None:
                assert rel_err(got_logits[t][b], logits) <= 2e-3
        single.close()

    if logits_mode == "last":
        rounded = Gpt(cfg)
        set_model_arrays(rounded, rounded_arrays)
        for b in (0, batch - 1):
            cpu = cpu_decoder(rounded, 1)
            cpu.decode([int(x) for x in prompt[b, :int(starts[b])]])
            for t in range(steps):
                ref = cpu.decode([int(feed[t, b])])
                assert rel_err(got_logits[t][b], ref) <= 2e-2


def test_ragged_decode_rejects_what_it_cannot_do():
    from tnsr_b200.nn import TnsrError
    cfg, arrays = config0_model("relu")                      # f32 weights: the strict path has no ragged step
    s = B200Session(cfg, 2, 32)
    for i, a in enumerate(arrays):
        s.refresh(i, a)
    with pytest.raises(TnsrError):
        s.decode_ragged(np.zeros(2, np.uint32), np.zeros(2, np.uint32))
    s.close()
    cfg, model, _ = small_bf16_model("swiglu", 128, 2, 256, vocab=300)
    s = B200Session(cfg, 2, 16, logits_mode="last")
    for i, p in enumerate(model_parameters(model)):
        s.refresh(i, p.values())
    with pytest.raises(TnsrError):
        s.decode_ragged(np.zeros(2, np.uint32), np.array([0, 16], np.uint32))      # position == capacity
    with pytest.raises(TnsrError):
        s.decode_ragged(np.array([0, 300], np.uint32), np.zeros(2, np.uint32))      # token == vocab
    logits, ids = s.decode_ragged(np.array([1, 2], np.uint32), np.array([0, 0], np.uint32))   # still usable afterwards
    assert np.all(np.isfinite(logits))
    s.close()


def test_full_context_forward_and_uncached_generate_on_the_gpu():
    """Gpt::forward / Gpt::generate (src/nn.rs:629-715) through the library vs the CPU checker."""
    model = kv_model(9)
    rows = kv_test_tokens(2, 9)
    close(model.forward(Backend.Cuda, rows), cpu_forward(model, rows))
    prompt = [365, 2, 3, 4]
    assert model.generate(Backend.Cuda, prompt, 8) == cpu_generate(model, prompt, 8)
    assert model.generate(Backend.Cuda, prompt, 8) == model.generate_cached(Backend.Cuda, prompt, 8)
    from tnsr_b200.nn import TnsrError
    with pytest.raises(TnsrError):
        model.forward(Backend.Cuda, [list(range(10))])


def test_a_wait_that_runs_out_fails_the_session_until_reset():
    """The `failed` flag of src/nn/kv_cache.rs:262-265,331,387 on the device side: every producer/consumer wait
    inside the tensor-core kernels is bounded, and when one runs out the kernel returns (nothing traps, nothing spins
    for ever), the step reports ERR_TIMEOUT, the handle refuses further steps until `reset`, and after `reset` it
    computes what a fresh handle computes.  The wait is made to run out on healthy hardware by the library's test
    hook: the next GEMM's copy role leaves one stage of its ring unfilled, so the MMA role waits for data that never
    arrives; the wait limit is lowered to 2 ms for the duration of the test."""
    from tnsr_b200 import _native
    lib = _native.lib()
    cfg = GptConfig(vocab_size=512, max_sequence_length=64, embed_dim=256, num_heads=4, feed_forward_dim=512,
                    num_layers=2, layer_norm_epsilon=1e-5, activation="swiglu", weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=31, std=0.05)
    ids = np.random.default_rng(32).integers(0, cfg.vocab_size, size=(2, 12)).astype(np.uint32)

    def session():
        s = B200Session(cfg, 2, 32)
        for i, a in enumerate(arrays):
            s.refresh(i, a)
        return s

    fresh = session()
    want, _ = fresh.decode_full(ids, 0)
    fresh.close()

    s = session()
    assert lib.tnsr_b200_set_wait_limit_ns(10) == -1            # below the accepted range
    assert lib.tnsr_b200_set_wait_limit_ns(2_000_000) == 0
    try:
        assert lib.tnsr_b200_test_lose_gemm_stage(2) == 0       # k-block 2 of the first projection's first tile
        u32p = _native.C.POINTER(_native.C.c_uint32)
        fp = _native.C.POINTER(_native.C.c_float)
        logits = np.empty(2 * 12 * cfg.vocab_size, dtype=np.float32)
        code = lib.tnsr_b200_decoder_decode(s.handle, ids.ctypes.data_as(u32p), 12, 0, logits.ctypes.data_as(fp), None)
        assert code == -7, _native.STATUS.get(code, code)       # TNSR_B200_ERR_TIMEOUT
        assert "timed out" in _native.last_error(s.handle)
        code = lib.tnsr_b200_decoder_decode(s.handle, ids.ctypes.data_as(u32p), 12, 0, logits.ctypes.data_as(fp), None)
        assert code == -6                                       # TNSR_B200_ERR_FAILED_STATE
        assert "reset the cache before reuse" in _native.last_error(s.handle)
    finally:
        assert lib.tnsr_b200_set_wait_limit_ns(2_000_000_000) == 0
    s.reset()
    got, _ = s.decode_full(ids, 0)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    s.close()


def test_prefill_mode_scalar_keeps_multi_token_chunks_off_the_tiled_kernels():
    """`GptPrefillMode::Scalar` (src/nn/kv_cache.rs:28-34) with bf16 weights: chunks run on the non-tiled scan instead
    of the tensor-core prefill kernels.  Both modes must meet the bf16 tolerance against the checker, and they must
    actually take different kernels (the logits differ in the last bits somewhere)."""
    cfg = GptConfig(vocab_size=640, max_sequence_length=192, embed_dim=256, num_heads=4, feed_forward_dim=512,
                    num_layers=2, layer_norm_epsilon=1e-5, activation="gelu", weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=41, std=0.05)
    model = Gpt(cfg)
    set_model_arrays(model, arrays)
    ids = np.random.default_rng(42).integers(0, cfg.vocab_size, size=(3, 150)).astype(np.uint32)
    from oracle import oracle
    ref = oracle.OracleModel(cfg.vocab_size, cfg.max_sequence_length, cfg.embed_dim, cfg.num_heads, cfg.feed_forward_dim,
                             cfg.num_layers, cfg.layer_norm_epsilon, "gelu")
    ref.set_params([oracle.bf16_round_np(a) if a.ndim == 2 else a for a in arrays])
    want = ref.forward(ids)
    outs = {}
    for mode in (GptPrefillMode.Auto, GptPrefillMode.Scalar):
        dec = gpu_decoder(model, 3, 192, GptDecoderOptions(prefill=mode))
        first = dec.decode(ids[:, :96].reshape(-1).tolist()).reshape(3, 96, cfg.vocab_size)
        second = dec.decode(ids[:, 96:].reshape(-1).tolist()).reshape(3, 54, cfg.vocab_size)
        outs[mode] = np.concatenate([first, second], axis=1)
        assert rel_err(outs[mode], want) <= 2e-2
    assert not np.array_equal(outs[GptPrefillMode.Auto], outs[GptPrefillMode.Scalar])


@pytest.mark.parametrize("parts", [2, 3])
def test_divided_single_token_step_matches_the_undivided_one(parts):
    """Large handles (or `step_parts` in the configuration) run a single-token step as independent session ranges on
    separate streams (lean kernel forms, own attention scratch per range).  Sessions are independent, so this must
    give what the undivided step gives up to the rounding of a different softmax grouping.  An odd batch makes the
    ranges unequal; the ragged form goes through the same division."""
    cfg = GptConfig(vocab_size=640, max_sequence_length=96, embed_dim=256, num_heads=4, feed_forward_dim=512,
                    num_layers=3, layer_norm_epsilon=1e-5, activation="swiglu", weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=43, std=0.05)
    batch, prompt_len, steps = 71, 20, 6
    ids = np.random.default_rng(44).integers(0, cfg.vocab_size, size=(batch, prompt_len + steps)).astype(np.uint32)

    def run(step_parts):
        s = B200Session(cfg, batch, 64, logits_mode="last", step_parts=step_parts)
        for i, a in enumerate(arrays):
            s.refresh(i, a)
        s.decode_full(ids[:, :prompt_len], 0)
        out = []
        for t in range(steps):        # the first step is launched kernel by kernel, the others replay the captured graph
            logits, _ = s.decode_full(ids[:, prompt_len + t:prompt_len + t + 1], prompt_len + t)
            out.append(logits.reshape(batch, cfg.vocab_size).copy())
        positions = np.arange(batch, dtype=np.uint32) % 7 + prompt_len + steps - 6   # rows that exist in every session
        ragged, _ = s.decode_ragged(ids[:, 0], positions)
        out.append(ragged.reshape(batch, cfg.vocab_size).copy())
        caches = [s.read_cache(i) for i in (0, 2 * cfg.num_layers - 1)]
        s.close()
        return np.stack(out), caches

    divided, caches_a = run(parts)
    whole, caches_b = run(1)
    assert np.all(np.isfinite(divided))
    assert rel_err(divided, whole) <= 1e-2
    for a, b in zip(caches_a, caches_b):
        assert np.max(np.abs(a - b)) <= max(1.0, float(np.max(np.abs(b)))) / 64
    # the first layer's keys do not depend on attention at all: identical bits in both forms
    assert np.array_equal(caches_a[0].view(np.uint32), caches_b[0].view(np.uint32))


def test_split_k_projections_are_deterministic_and_match_the_checker():
    """Between 33 and 256 sessions the attention-output and FFN-down projections of a single-token step divide their K
    extent over several CTAs per tile; the partial sums are added to the residual in a fixed order by the LayerNorm that
    follows.  So two runs give the same bits (no atomics, no arrival order), the projections and LayerNorms of a session do
    not depend on how many other sessions share the batch (checked here with contexts short enough that the attention
    scan never cuts a session, which is the one place where the batch size decides a grouping), and the result stays
    within the bf16-path tolerance of the CPU checker."""
    from oracle import oracle
    cfg = GptConfig(vocab_size=640, max_sequence_length=64, embed_dim=256, num_heads=4, feed_forward_dim=512,
                    num_layers=3, layer_norm_epsilon=1e-5, activation="swiglu", weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=57, std=0.05, bias_std=0.02)
    ids = np.random.default_rng(58).integers(0, cfg.vocab_size, size=(72, 20)).astype(np.uint32)

    def run(batch):
        s = B200Session(cfg, batch, 48, logits_mode="last")
        for i, a in enumerate(arrays):
            s.refresh(i, a)
        out = [s.decode_full(ids[:batch, :12], 0)[0]]
        for t in range(12, 18):
            out.append(s.decode_full(ids[:batch, t:t + 1], t)[0])
        s.close()
        return np.stack([o.reshape(batch, -1) for o in out])

    a, b = run(72), run(72)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    fewer = run(40)                                   # another batch size on the same path: the same k-ranges per element
    assert np.array_equal(fewer.view(np.uint32), a[:, :40].view(np.uint32))
    ref = oracle.OracleModel(cfg.vocab_size, cfg.max_sequence_length, cfg.embed_dim, cfg.num_heads, cfg.feed_forward_dim,
                             cfg.num_layers, cfg.layer_norm_epsilon, "swiglu")
    ref.set_params([oracle.bf16_round_np(x) if x.ndim == 2 else x for x in arrays])
    want = ref.forward(ids[:16, :18])
    for t in range(12, 18):
        assert rel_err(a[t - 11, :16], want[:, t]) <= 2e-2


@pytest.mark.parametrize("weight_dtype", ["f32", "bf16"])
def test_gpu_decoder_state_round_trips_through_the_archive(tmp_path, weight_dtype):
    """Serialised decoder state on the device: K/V rows read back through the C ABI, written as a tensor archive,
    restored into a fresh session (bf16 rows are exactly representable in the archive's f32), which then continues
    with the same bits as the session that was never interrupted."""
    cfg = GptConfig(vocab_size=320, max_sequence_length=96, embed_dim=128, num_heads=2, feed_forward_dim=256,
                    num_layers=2, layer_norm_epsilon=1e-5, activation="gelu", weight_dtype=weight_dtype)
    model = Gpt(cfg)
    set_model_arrays(model, normal_model_arrays(cfg, seed=51, std=0.05))
    ids = np.random.default_rng(52).integers(0, cfg.vocab_size, size=(3, 40)).astype(np.uint32)
    flat = lambda lo, hi: ids[:, lo:hi].reshape(-1).tolist()
    straight = gpu_decoder(model, 3, 96)
    straight.decode(flat(0, 33))
    want = [straight.decode(flat(33 + i, 34 + i)) for i in range(4)]
    first = gpu_decoder(model, 3, 96)
    first.decode(flat(0, 33))
    first.save_state(str(tmp_path))
    second = gpu_decoder(model, 3, 64)              # a different capacity is fine as long as the rows fit
    second.load_state(str(tmp_path))
    assert second.len() == 33
    for i in range(4):
        got = second.decode(flat(33 + i, 34 + i))
        assert np.array_equal(got.view(np.uint32), want[i].view(np.uint32))


@pytest.mark.parametrize("logits_mode", ["last", "none"])
def test_session_sampler_draws_what_the_cpu_restatement_draws(logits_mode):
    """`tnsr_b200_decoder_set_sampler`: the ids a session returns are the CPU sampler's ids on the session's own
    last-position logits, with the counter (position of the new token, session); the draw does not depend on whether
    logits leave the device, on graph replay, or on the chunking; temperature 0 restores the greedy pick."""
    from oracle import sampler
    cfg = GptConfig(vocab_size=1536, max_sequence_length=64, embed_dim=128, num_heads=2, feed_forward_dim=256,
                    num_layers=2, layer_norm_epsilon=1e-5, activation="swiglu", weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=61, std=0.08)
    ids = np.random.default_rng(62).integers(0, cfg.vocab_size, size=(5, 9)).astype(np.uint32)
    seed, temperature, top_k = 424242, 0.9, 12

    def session(mode):
        s = B200Session(cfg, 5, 48, logits_mode=mode)
        for i, a in enumerate(arrays):
            s.refresh(i, a)
        s.set_sampler(temperature, top_k, seed)
        return s

    ref = session("last")
    s = session(logits_mode)
    logits, want_ids = ref.decode_full(ids, 0)
    _, got = s.decode_full(ids, 0)
    assert np.array_equal(want_ids, sampler.sample(logits.reshape(5, -1), temperature, top_k, seed, 9))
    assert np.array_equal(got, want_ids)
    for t in range(6):                       # single-token steps: one direct, then graph replays
        logits, want_ids = ref.decode_full(want_ids.reshape(5, 1), 9 + t)
        assert np.array_equal(want_ids, sampler.sample(logits.reshape(5, -1), temperature, top_k, seed, 10 + t))
        _, got = s.decode_full(got.reshape(5, 1), 9 + t)
        assert np.array_equal(got, want_ids)
    s.set_sampler(0.0, 0, 0)
    ref.set_sampler(0.0, 0, 0)
    logits, greedy = ref.decode_full(want_ids.reshape(5, 1), 15)
    assert greedy.tolist() == [argmax_last(r) for r in logits.reshape(5, -1)]
    _, got = s.decode_full(want_ids.reshape(5, 1), 15)
    assert np.array_equal(got, greedy)


def test_paged_kv_cache_gives_the_same_bits_as_the_contiguous_one():
    """kv_page_rows > 0: every cache tensor is a pool of pages handed to sessions on demand.  Same kernels, other
    addresses: prefill (non-tiled scan in both handles), graph-replayed steps, ragged steps and the cache read back in
    logical order must equal the contiguous handle bit for bit -- also when a step is divided over two streams."""
    cfg = GptConfig(vocab_size=512, max_sequence_length=96, embed_dim=256, num_heads=4, feed_forward_dim=512,
                    num_layers=2, layer_norm_epsilon=1e-5, activation="swiglu", weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=81, std=0.05)
    batch, capacity = 6, 96
    ids = np.random.default_rng(82).integers(0, cfg.vocab_size, size=(batch, 40)).astype(np.uint32)

    def run(**kw):
        s = B200Session(cfg, batch, capacity, GptDecoderOptions(prefill=GptPrefillMode.Scalar), logits_mode="last", **kw)
        for i, a in enumerate(arrays):
            s.refresh(i, a)
        out = [s.decode_full(ids[:, :21], 0)[0]]
        for t in range(21, 36):                                   # crosses the page boundary at row 32
            out.append(s.decode_full(ids[:, t:t + 1], t)[0])
        positions = np.asarray([36, 30, 36, 17, 33, 36], dtype=np.uint32)
        out.append(s.decode_ragged(ids[:, 36], positions)[0])
        caches = [s.read_cache(i) for i in range(4)]
        free = s.free_pages()
        s.close()
        return np.stack([o.reshape(batch, -1) for o in out]), caches, free

    plain, plain_caches, _ = run()
    paged, paged_caches, free = run(kv_page_rows=16)
    assert free == batch * (capacity // 16) - batch * 3            # 37 rows per session -> 3 pages each
    assert np.array_equal(paged.view(np.uint32), plain.view(np.uint32))
    for a, b in zip(paged_caches, plain_caches):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    divided, _, _ = run(kv_page_rows=32, step_parts=2)
    reference, _, _ = run(step_parts=2)
    assert np.array_equal(divided.view(np.uint32), reference.view(np.uint32))


def test_paged_kv_pool_smaller_than_the_worst_case():
    """A pool of 7 pages for 4 sessions x 64 rows (worst case 16 pages): short sessions fit, a step that would need an
    eighth page is refused with ERR_CAPACITY and changes nothing, releasing a session makes room again."""
    from tnsr_b200 import _native
    cfg = GptConfig(vocab_size=256, max_sequence_length=64, embed_dim=128, num_heads=2, feed_forward_dim=256,
                    num_layers=2, layer_norm_epsilon=1e-5, activation="gelu", weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=83, std=0.05)
    s = B200Session(cfg, 4, 64, logits_mode="last", kv_page_rows=16, kv_pool_pages=7)
    for i, a in enumerate(arrays):
        s.refresh(i, a)
    ids = np.random.default_rng(84).integers(0, cfg.vocab_size, size=(4, 64)).astype(np.uint32)
    s.decode_full(ids[:, :16], 0)                                   # 4 pages
    assert s.free_pages() == 3
    positions = np.asarray([16, 16, 16, 5], dtype=np.uint32)        # three sessions open a second page
    before, _ = s.decode_ragged(ids[:, 16], positions)
    assert s.free_pages() == 0
    u32p = _native.C.POINTER(_native.C.c_uint32)
    pos2 = np.asarray([17, 17, 17, 16], dtype=np.uint32)            # session 3 now needs a page that is not there
    tok = np.ascontiguousarray(ids[:, 17])
    logits = np.empty(4 * cfg.vocab_size, dtype=np.float32)
    code = _native.lib().tnsr_b200_decoder_decode_ragged(s.handle, tok.ctypes.data_as(u32p), pos2.ctypes.data_as(u32p),
                                                        logits.ctypes.data_as(_native.C.POINTER(_native.C.c_float)), None)
    assert code == -4 and "page pool exhausted" in _native.last_error(s.handle)
    again, _ = s.decode_ragged(ids[:, 16], positions)                # the refused step left the session as it was
    assert np.array_equal(again.view(np.uint32), before.view(np.uint32))
    s.release(0)                                                     # two pages come back
    assert s.free_pages() == 2
    pos3 = np.asarray([0, 17, 17, 16], dtype=np.uint32)              # session 0 starts over, session 3 gets its page
    out, _ = s.decode_ragged(ids[:, 17], pos3)
    assert np.all(np.isfinite(out)) and s.free_pages() == 0
    s.reset()
    assert s.free_pages() == 7
    s.close()
    with pytest.raises(Exception):
        B200Session(cfg, 4, 64, kv_page_rows=24)                     # not a multiple of 16


@pytest.mark.parametrize("batch", [3, 16, 29])
def test_small_batch_fused_layer_kernel_matches_the_operator_by_operator_step(batch):
    """Up to 32 sessions a single-token step runs each layer's projections, LayerNorms and SwiGLU as one persistent
    kernel with grid barriers (warp-level MMA, weights streamed once); `small_batch_mode=1` keeps the operator-by-operator
    kernels.  Same arithmetic up to summation order: logits within the bf16-path tolerance of each other and of the CPU
    checker, K/V rows equal to bf16 resolution; 3 and 16 sessions take the 16-row form, 29 the 32-row form; ragged and
    paged steps go through the same kernel."""
    from oracle import oracle
    cfg = GptConfig(vocab_size=640, max_sequence_length=64, embed_dim=256, num_heads=4, feed_forward_dim=1088,
                    num_layers=3, layer_norm_epsilon=1e-5, activation="swiglu", weight_dtype="bf16")
    arrays = normal_model_arrays(cfg, seed=91, std=0.05, bias_std=0.02)
    ids = np.random.default_rng(92).integers(0, cfg.vocab_size, size=(batch, 20)).astype(np.uint32)

    def run(**kw):
        s = B200Session(cfg, batch, 48, logits_mode="last", **kw)
        for i, a in enumerate(arrays):
            s.refresh(i, a)
        out = [s.decode_full(ids[:, :12], 0)[0]]
        for t in range(12, 18):
            out.append(s.decode_full(ids[:, t:t + 1], t)[0])
        positions = (np.arange(batch, dtype=np.uint32) % 5) + 14
        out.append(s.decode_ragged(ids[:, 18], positions)[0])
        caches = [s.read_cache(i) for i in (0, 1, 2 * cfg.num_layers - 1)]
        s.close()
        return np.stack([o.reshape(batch, -1) for o in out]), caches

    fused, fused_caches = run()
    classic, classic_caches = run(small_batch_mode=1)
    assert np.all(np.isfinite(fused))
    assert rel_err(fused, classic) <= 1e-2
    for a, b in zip(fused_caches, classic_caches):
        assert np.max(np.abs(a - b)) <= max(1.0, float(np.max(np.abs(b)))) / 64
    paged, _ = run(kv_page_rows=16)                  # the prefill takes another attention kernel when paged
    assert rel_err(paged, fused) <= 1e-2
    ref = oracle.OracleModel(cfg.vocab_size, cfg.max_sequence_length, cfg.embed_dim, cfg.num_heads, cfg.feed_forward_dim,
                             cfg.num_layers, cfg.layer_norm_epsilon, "swiglu")
    ref.set_params([oracle.bf16_round_np(a) if a.ndim == 2 else a for a in arrays])
    want = ref.forward(ids[:, :18])
    for t in range(12, 18):
        assert rel_err(fused[t - 11], want[:, t]) <= 2e-2
