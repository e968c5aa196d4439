"""Pins the CPU checker against the known-answer vectors tnsr's own tests hold
for the cached-GPT path (fixtures in tests/golden/reference_vectors.json, made
by tests/golden/make_golden.py from the reference's test literals)."""
import json
import math
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def vectors():
    with open(os.path.join(GOLDEN, "reference_vectors.json")) as f:
        return json.load(f)


def bits_to_f32(bits):
    return np.asarray(bits, dtype=np.uint32).view(np.float32)


# src/nn/activations/tests.rs:8-167 -- PyTorch 2.11 values, tolerance 2e-6
@pytest.mark.parametrize("name", ["sigmoid", "silu", "gelu"])
def test_activation_bit_patterns(oracle, vectors, name):
    x = bits_to_f32(vectors["activations"]["input_bits"])
    expected = bits_to_f32(vectors["activations"][name]["value_bits"])
    actual = getattr(oracle, name)(x)
    assert np.all(np.isfinite(actual))
    assert np.max(np.abs(actual - expected)) < vectors["activations"]["tolerance"]


def test_swiglu_elementwise_is_silu_times_up(oracle, vectors):
    x = bits_to_f32(vectors["activations"]["input_bits"])
    up = np.linspace(-2, 2, x.size).astype(np.float32)
    assert np.array_equal(oracle.swiglu(x, up).view(np.uint32),
                          (oracle.silu(x) * up).astype(np.float32).view(np.uint32))


# tests/indexed_ops.rs:25-36
def test_embedding_gather_known_answer(oracle, vectors):
    v = vectors["embedding"]
    w = np.asarray(v["weight"], np.float32).reshape(v["weight_shape"])
    out = oracle.embedding(w, np.asarray(v["indices"], np.float32).reshape(2, 2))
    assert out.shape == (2, 2, 2)
    assert out.reshape(-1).tolist() == v["expected"]


# tests/indexed_ops.rs:98-118
def test_embedding_rejects_invalid_indices(oracle, vectors):
    w = np.ones((3, 2), np.float32)
    for value, message in vectors["embedding_invalid"]["cases"]:
        with pytest.raises(oracle.OracleError) as err:
            oracle.embedding(w, np.asarray([float(value)], np.float32))
        assert message in str(err.value)


# tests/transformer.rs:86-103
def test_batched_matmul_known_answer(oracle, vectors):
    v = vectors["batched_matmul"]
    out = oracle.matmul(np.asarray(v["left"], np.float32).reshape(v["left_shape"]),
                        np.asarray(v["right"], np.float32).reshape(v["right_shape"]))
    assert out.reshape(-1).tolist() == v["expected"]


# src/nn.rs linear_no_bias / linear_with_bias_vector
def test_linear_known_answers(oracle):
    x = np.asarray([1, 2, 3, 4, 5, 6], np.float32).reshape(2, 3)
    w = np.asarray([1, 2, 3, 4, 5, 6], np.float32).reshape(3, 2)
    assert oracle.linear(x, w).reshape(-1).tolist() == [22.0, 28.0, 49.0, 64.0]
    assert oracle.linear(x, w, np.asarray([10, -1], np.float32)).reshape(-1).tolist() == [32.0, 27.0, 59.0, 63.0]


# tests/transformer.rs:106-130
def test_softmax_is_stable_and_normalises(oracle):
    x = np.asarray([[1000, 1001, 1002], [-1000, -1000, -1000]], np.float32)
    out = oracle.softmax(x)
    den = 1.0 + math.e + math.e ** 2
    expected = np.asarray([[1 / den, math.e / den, math.e ** 2 / den], [1 / 3, 1 / 3, 1 / 3]])
    assert np.all(np.isfinite(out))
    assert np.max(np.abs(out - expected)) < 1e-5
    assert np.max(np.abs(out.sum(axis=1) - 1.0)) < 1e-6


# src/graph/mixed.rs:126-135 and half 2.7.1 semantics
def test_bf16_narrowing(oracle, vectors):
    v = vectors["bf16_narrowing"]
    x = np.asarray(v["input"], np.float32)
    assert oracle.bf16_round(x).tolist() == v["expected"]
    assert oracle.bf16_round_np(x).tolist() == v["expected"]
    # ties to even, overflow to inf, NaN stays NaN, and the numpy twin agrees
    cases = np.asarray([1 + 1 / 128, 1 + 3 / 256, 3.4028234e38, -3.4028234e38, np.nan, np.inf, -0.0,
                        1e-40, 65280.0, 65408.0], np.float32)
    a, b = oracle.bf16_round(cases), oracle.bf16_round_np(cases)
    assert np.array_equal(a.view(np.uint32)[~np.isnan(a)], b.view(np.uint32)[~np.isnan(b)])
    assert a[0] == np.float32(1 + 1 / 128) and a[1] == np.float32(1 + 1 / 64)
    assert np.isinf(a[2]) and np.isinf(a[3]) and np.isnan(a[4]) and np.isnan(b[4])
    rng = np.random.default_rng(7)
    r = rng.standard_normal(4096).astype(np.float32) * 3
    assert np.array_equal(oracle.bf16_round(r).view(np.uint32), oracle.bf16_round_np(r).view(np.uint32))
    torch = pytest.importorskip("torch")
    t = torch.from_numpy(r).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(t.view(np.uint32), oracle.bf16_round_np(r).view(np.uint32))


def cancellation_operands():
    """tests/ptx_transformer.rs:1417-1441: reassociation or FMA changes bits."""
    m, k, n = 17, 65, 19
    one_up = np.float32(1.0).view(np.uint32) + 1
    one_dn = np.float32(1.0).view(np.uint32) - 2
    lhs = np.empty(m * k, np.float32)
    for i in range(m * k):
        if (i // k) % 2 == 0:
            lhs[i] = 1.0
        elif (i % k) % 2 == 0:
            lhs[i] = np.uint32(one_up).view(np.float32)
        else:
            lhs[i] = -1.0
    rhs = np.empty(k * n, np.float32)
    for i in range(k * n):
        if (i % n) % 2 == 0:
            rhs[i] = [16777216.0, 1.0, -16777216.0][(i // n) % 3]
        else:
            rhs[i] = np.uint32(one_dn).view(np.float32) if (i // n) % 2 == 0 else 1.0
    return lhs.reshape(m, k), rhs.reshape(k, n)


def test_matmul_keeps_rounded_products_and_k_order(oracle):
    a, b = cancellation_operands()
    fast = oracle.matmul(a, b)
    naive = oracle.matmul(a, b, naive=True)
    assert np.array_equal(fast.view(np.uint32), naive.view(np.uint32))
    # an independent statement of the same order in numpy f32 scalars
    m, k = a.shape
    n = b.shape[1]
    ref = np.zeros((m, n), np.float32)
    for p in range(k):
        ref = (ref + (a[:, p:p + 1] * b[p:p + 1, :]).astype(np.float32)).astype(np.float32)
    assert np.array_equal(fast.view(np.uint32), ref.view(np.uint32))
    # and the matrix does what it was built for: a differently associated sum differs
    f64 = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    assert not np.array_equal(fast.view(np.uint32), f64.view(np.uint32))
    biased = oracle.linear(a, b, np.full(n, 0.25, np.float32))
    assert np.array_equal(biased.view(np.uint32), (fast + np.float32(0.25)).astype(np.float32).view(np.uint32))


# tests/half_precision.rs:324-375: SimpleExecutor<bf16>, relu(a @ b + bias)
def test_bf16_gemm_reference_contract(oracle):
    m, n, k = 33, 35, 37
    lhs = (((np.arange(2 * m * k) % 17).astype(np.float32) - 8.0) / 16.0).reshape(2, m, k)
    rhs = (((np.arange(k * n) % 13).astype(np.float32) - 6.0) / 16.0).reshape(1, k, n)
    assert np.array_equal(lhs, oracle.bf16_round_np(lhs)) and np.array_equal(rhs, oracle.bf16_round_np(rhs))
    prod = oracle.matmul_bf16(lhs, rhs)                       # rounded once at the matmul output
    out = np.maximum(oracle.bf16_round_np(prod + np.float32(0.25)), 0)
    exact = np.maximum(lhs.astype(np.float64) @ rhs[0].astype(np.float64) + 0.25, 0)
    assert np.max(np.abs(out - exact)) <= 0.032


# tests/transformer.rs:133-173 style: causal rows ignore the future; f64 twin
def test_attention_matches_f64_reference(oracle):
    from tests.workloads import attention_samples
    batch, heads, capacity = 2, 2, 70
    for columns in (4, 33):
        d = heads * columns
        for chunk in (1, 3):
            q = attention_samples(batch * chunk * d, 5).reshape(batch, chunk, d)
            k = attention_samples(batch * chunk * d, 19).reshape(batch, chunk, d)
            v = attention_samples(batch * chunk * d, 37).reshape(batch, chunk, d)
            ck = attention_samples(batch * capacity * d, 41).reshape(batch, capacity, d)
            cv = attention_samples(batch * capacity * d, 67).reshape(batch, capacity, d)
            for prefix in (0, 1, 31, 32, 33, 65):
                ref = oracle.attention_f64(q, k, v, ck, cv, heads, prefix)
                # the checker's decode attention reads every key from the cache
                kc, vc = ck.copy(), cv.copy()
                kc[:, prefix:prefix + chunk] = k
                vc[:, prefix:prefix + chunk] = v
                kc[:, prefix + chunk:] = np.nan
                vc[:, prefix + chunk:] = np.nan
                for t in range(chunk):
                    lengths = np.full(batch, prefix + t + 1, np.uint32)
                    out = oracle.decode_attention(q[:, t], kc, vc, lengths, heads)
                    want = ref[:, :, t, :].reshape(batch, d)
                    assert np.all(np.isfinite(out))
                    assert np.max(np.abs(out - want)) < 3e-5


def test_layer_norm_moments_and_formula(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 48)).astype(np.float32) * 3 + 1
    w = rng.standard_normal(48).astype(np.float32)
    b = rng.standard_normal(48).astype(np.float32)
    y = oracle.layer_norm(x, w, b, 1e-5)
    x64 = x.astype(np.float64)
    ref = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * w + b
    assert np.max(np.abs(y - ref)) < 5e-6
    plain = oracle.layer_norm(x, np.ones(48, np.float32), np.zeros(48, np.float32), 1e-5)
    assert np.max(np.abs(plain.mean(1))) < 1e-6 and np.max(np.abs(plain.var(1) - 1)) < 1e-4


def test_reference_initialiser(oracle):
    """xavier_parameter (src/nn.rs:303-316): the C loop and the vectorised
    closed form in the host mirror produce the same bits."""
    from tnsr_b200.nn import xavier_values
    for rows, cols, seed in ((367, 8, 101), (7, 8, 102), (8, 13, 1005), (13, 8, 1106), (3, 5, 2**63 + 11)):
        a = oracle.xavier(rows, cols, seed).reshape(-1)
        b = xavier_values(rows, cols, seed)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        limit = np.sqrt(np.float32(6.0) / np.float32(rows + cols))
        assert np.all(np.abs(a) <= limit)


def test_argmax_prefers_last_maximum(oracle):
    from tnsr_b200.nn import argmax_last
    rows = [np.asarray([1, 3, 3, 2], np.float32), np.asarray([-0.0, 0.0, -0.0], np.float32),
            np.asarray([0.0, -0.0], np.float32), np.asarray([1, np.inf, np.nan, 5], np.float32),
            np.asarray([-np.inf, -np.inf], np.float32), np.asarray([7], np.float32)]
    expected = [2, 1, 0, 2, 1, 0]
    for row, want in zip(rows, expected):
        assert oracle.argmax_last(row) == want
        assert argmax_last(row) == want
