"""Operator-level parity on the GPU: every kernel family behind the C ABI against
the CPU checker on the same seeded inputs (bit-exact for gathers, ids and the
strict f32 matmul; stated tolerances elsewhere)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from tests.gpu_util import BF16, F32, bf16_round, dev, gemm_bf16, lib, ok, ptr, rel_err, stream  # noqa: E402
from tests.test_oracle_pins import cancellation_operands  # noqa: E402
from tests.workloads import attention_samples  # noqa: E402


# ---- embedding ---------------------------------------------------------------
@pytest.mark.parametrize("width", [8, 128, 770])
def test_embedding_gather_add_is_bit_exact(oracle, width):
    rng = np.random.default_rng(11)
    vocab, ctx, batch, chunk, position = 97, 40, 3, 5, 7
    tok = rng.standard_normal((vocab, width)).astype(np.float32)
    pos = rng.standard_normal((ctx, width)).astype(np.float32)
    ids = rng.integers(0, vocab, size=(batch, chunk)).astype(np.uint32)
    expected = oracle.embedding(tok, ids.astype(np.float32)) + oracle.embedding(
        pos, np.arange(position, position + chunk, dtype=np.float32))[None]
    out = torch.empty((batch * chunk, width), dtype=torch.float32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ok(lib().tnsr_b200_embedding(ptr(dev(tok)), ptr(dev(pos)), ptr(dev(ids.view(np.int32))), ptr(out), batch * chunk,
                                 chunk, position, vocab, width, F32, ptr(status), stream()))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), expected.reshape(-1, width).view(np.uint32))
    assert int(status[0]) == 0
    # the reference's own known answer (tests/indexed_ops.rs:25-36) with a zero position table
    w = np.arange(1, 9, dtype=np.float32).reshape(4, 2)
    out = torch.empty((4, 2), dtype=torch.float32, device="cuda")
    ok(lib().tnsr_b200_embedding(ptr(dev(w)), ptr(dev(np.zeros((4, 2), np.float32))),
                                 ptr(dev(np.asarray([2, 0, 3, 1], np.int32))), ptr(out), 4, 1, 0, 4, 2, F32, None, stream()))
    torch.cuda.synchronize()
    assert out.cpu().numpy().reshape(-1).tolist() == [5, 6, 1, 2, 7, 8, 3, 4]


def test_embedding_flags_out_of_range_ids_without_faulting():
    tok = dev(np.ones((3, 8), np.float32))
    pos = dev(np.ones((4, 8), np.float32))
    ids = dev(np.asarray([0, 3, 2, 0xFFFFFFFF], np.uint32).view(np.int32))
    out = torch.full((4, 8), 7.0, dtype=torch.float32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ok(lib().tnsr_b200_embedding(ptr(tok), ptr(pos), ptr(ids), ptr(out), 4, 4, 0, 3, 8, F32, ptr(status), stream()))
    torch.cuda.synchronize()
    assert int(status[0]) == 1
    got = out.cpu().numpy()
    assert np.all(got[[0, 2]] == 2.0) and np.all(got[[1, 3]] == 0.0)


def test_embedding_bf16_tables(oracle):
    rng = np.random.default_rng(12)
    tok = bf16_round(rng.standard_normal((50, 64)))
    pos = bf16_round(rng.standard_normal((9, 64)))
    ids = rng.integers(0, 50, size=(2, 3)).astype(np.uint32)
    out = torch.empty((6, 64), dtype=torch.float32, device="cuda")
    ok(lib().tnsr_b200_embedding(ptr(dev(tok, torch.bfloat16)), ptr(dev(pos, torch.bfloat16)), ptr(dev(ids.view(np.int32))),
                                 ptr(out), 6, 3, 4, 50, 64, BF16, None, stream()))
    torch.cuda.synchronize()
    expected = tok[ids.reshape(-1)] + np.tile(pos[4:7], (2, 1))
    assert np.array_equal(out.cpu().numpy().view(np.uint32), expected.astype(np.float32).view(np.uint32))


# ---- layer norm ----------------------------------------------------------------
@pytest.mark.parametrize("width", [8, 128, 258, 768, 1024, 1500])
def test_layernorm_matches_checker(oracle, width):
    rng = np.random.default_rng(width)
    rows = 37
    x = (rng.standard_normal((rows, width)) * 2 + 0.5).astype(np.float32)
    w = rng.standard_normal(width).astype(np.float32)
    b = rng.standard_normal(width).astype(np.float32)
    expected = oracle.layer_norm(x, w, b, 1e-5)
    dx, dw, db = dev(x), dev(w), dev(b)
    strict = torch.empty((rows, width), dtype=torch.float32, device="cuda")
    ok(lib().tnsr_b200_layernorm(ptr(dx), ptr(dw), ptr(db), ptr(strict), rows, width, 1e-5, F32, 1, stream()))
    fast = torch.empty((rows, width), dtype=torch.float32, device="cuda")
    ok(lib().tnsr_b200_layernorm(ptr(dx), ptr(dw), ptr(db), ptr(fast), rows, width, 1e-5, F32, 0, stream()))
    half = torch.empty((rows, width), dtype=torch.bfloat16, device="cuda")
    ok(lib().tnsr_b200_layernorm(ptr(dx), ptr(dw), ptr(db), ptr(half), rows, width, 1e-5, BF16, 0, stream()))
    torch.cuda.synchronize()
    # strict: same operation order; only exp/ln may differ in the last bit of inv_std
    assert np.max(np.abs(strict.cpu().numpy() - expected)) <= 4e-6 * max(1.0, float(np.max(np.abs(expected))))
    assert np.max(np.abs(fast.cpu().numpy() - expected)) <= 2e-5 * max(1.0, float(np.max(np.abs(expected))))
    assert rel_err(half.float().cpu().numpy(), expected) <= 1 / 128


# ---- strict f32 matmul ----------------------------------------------------------
def run_strict(a, b, bias=None, transposed=False):
    m, k = a.shape
    n = b.shape[0] if transposed else b.shape[1]
    out = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ok(lib().tnsr_b200_gemm_f32_strict(ptr(dev(a)), ptr(dev(b)), ptr(dev(bias)) if bias is not None else None, ptr(out),
                                       m, k, n, int(transposed), stream()))
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_strict_matmul_keeps_rounded_products_and_k_order(oracle):
    """tests/ptx_transformer.rs:1410-1465 -- bit-for-bit with the CPU order."""
    a, b = cancellation_operands()
    expected = oracle.matmul(a, b)
    assert np.array_equal(run_strict(a, b).view(np.uint32), expected.view(np.uint32))
    bias = np.full(b.shape[1], 0.25, np.float32)
    assert np.array_equal(run_strict(a, b, bias).view(np.uint32), oracle.linear(a, b, bias).view(np.uint32))
    assert np.array_equal(run_strict(a, np.ascontiguousarray(b.T), transposed=True).view(np.uint32), expected.view(np.uint32))


@pytest.mark.parametrize("shape", [(1, 128, 128), (16, 128, 512), (7, 13, 8), (33, 37, 35), (3, 512, 96)])
def test_strict_matmul_random_shapes_bit_exact(oracle, shape):
    m, k, n = shape
    rng = np.random.default_rng(m * 1000 + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    assert np.array_equal(run_strict(a, b, bias).view(np.uint32), oracle.linear(a, b, bias).view(np.uint32))


def test_batched_matmul_known_answer():
    """tests/transformer.rs:86-103, one batch at a time."""
    left = np.asarray([1, 2, 3, 4, 5, 6, -1, 0, 1, 2, -2, 1], np.float32).reshape(2, 2, 3)
    right = np.asarray([1, 0, 0, 1, 1, 1, 2, -1, 1, 3, -2, 2], np.float32).reshape(2, 3, 2)
    got = np.concatenate([run_strict(left[i], right[i]).reshape(-1) for i in range(2)])
    assert got.tolist() == [4, 5, 10, 11, -4, 3, 0, -6]


# ---- bf16 GEMM -------------------------------------------------------------------
def gemm_case(m, n, k, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    a = bf16_round(rng.uniform(-1, 1, size=(m, k)))
    bt = bf16_round(rng.uniform(-1, 1, size=(n, k)) * scale)
    ref = a.astype(np.float64) @ bt.astype(np.float64).T
    return a, bt, ref


GEMM_SHAPES = [(128, 128, 64), (128, 256, 128), (256, 768, 768), (300, 200, 136), (1, 4096, 4096), (8, 4096, 4096),
               (64, 4096, 4096), (1024, 1024, 1024), (129, 65, 72), (512, 2304, 768), (33, 35, 40)]


@pytest.mark.parametrize("engine", [1, 2])
@pytest.mark.parametrize("shape", GEMM_SHAPES)
def test_gemm_bf16_engines_match_f64(shape, engine):
    m, n, k = shape
    a, bt, ref = gemm_case(m, n, k, seed=2)
    try:
        ok(lib().tnsr_b200_set_gemm_engine(engine))
        out = gemm_bf16(dev(a, torch.bfloat16), dev(bt, torch.bfloat16)).cpu().numpy()
    finally:
        lib().tnsr_b200_set_gemm_engine(0)
    # f32 accumulation of exact bf16 products: error grows like sqrt(k) * eps_f32 * |a||b|
    tol = 4e-6 * k
    assert np.max(np.abs(out - ref)) <= tol, (engine, shape, float(np.max(np.abs(out - ref))))


def test_gemm_bf16_reference_fused_test_shape(oracle):
    """tests/half_precision.rs:324-375: relu(a[2,33,37] @ b[37,35] + 0.25), bf16 out, tol 0.032."""
    m, n, k = 33, 35, 37
    lhs = (((np.arange(2 * m * k) % 17).astype(np.float32) - 8.0) / 16.0).reshape(2 * m, k)
    rhs = (((np.arange(k * n) % 13).astype(np.float32) - 6.0) / 16.0).reshape(k, n)
    bias = dev(np.full(n, 0.25, np.float32))
    bt = dev(np.ascontiguousarray(rhs.T), torch.bfloat16)
    out = gemm_bf16(dev(lhs, torch.bfloat16), bt, bias=bias, activation=0, out_dtype=BF16).float().cpu().numpy()
    prod = oracle.matmul_bf16(lhs.reshape(2, m, k), rhs[None])
    expected = np.maximum(oracle.bf16_round_np(prod + np.float32(0.25)), 0).reshape(2 * m, n)
    assert np.max(np.abs(out - expected)) <= 0.032


@pytest.mark.parametrize("engine", [1, 2])
def test_gemm_bf16_epilogues(engine):
    m, n, k = 200, 384, 256
    a, bt, ref = gemm_case(m, n, k, seed=5, scale=0.1)
    rng = np.random.default_rng(6)
    bias = rng.standard_normal(n).astype(np.float32)
    resid = rng.standard_normal((m, n)).astype(np.float32)
    da, dbt, dbias, dres = dev(a, torch.bfloat16), dev(bt, torch.bfloat16), dev(bias), dev(resid)
    try:
        ok(lib().tnsr_b200_set_gemm_engine(engine))
        plain = gemm_bf16(da, dbt, bias=dbias).cpu().numpy()
        fused = gemm_bf16(da, dbt, bias=dbias, residual=dres).cpu().numpy()
        relu = gemm_bf16(da, dbt, bias=dbias, activation=0, out_dtype=BF16).float().cpu().numpy()
        gelu = gemm_bf16(da, dbt, bias=dbias, activation=1, out_dtype=BF16).float().cpu().numpy()
    finally:
        lib().tnsr_b200_set_gemm_engine(0)
    z = ref + bias
    assert np.max(np.abs(plain - z)) <= 2e-3
    assert np.max(np.abs(fused - (z + resid))) <= 2e-3
    assert rel_err(relu, np.maximum(z, 0)) <= 1 / 128
    from oracle import oracle as orc
    assert rel_err(gelu, orc.gelu(z.astype(np.float32))) <= 1 / 128


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (8, 4096, 4096), (64, 4096, 4096), (17, 768, 768), (32, 768, 2048),
                                   (64, 2304, 768), (5, 100, 72), (33, 129, 520), (16, 32000, 768), (1, 128, 64)])
def test_gemm_bf16_few_rows_engine_matches_f64_with_and_without_split_k(shape):
    """m <= 64 with scratch lent: weights on the M side of the MMA, K divided over several CTAs per 128-column tile and
    merged in a fixed order.  Same tolerance as the other engines; two runs are bit-identical; the scratch counters are
    back at zero; the epilogues (bias, activation, residual, bf16 output, in place on the residual stream) run on the
    merged tile.  Without scratch the same call takes whichever engine the shape selects and must agree as well."""
    m, n, k = shape
    a, bt, ref = gemm_case(m, n, k, seed=11)
    rng = np.random.default_rng(12)
    bias = rng.standard_normal(n).astype(np.float32)
    resid = rng.standard_normal((m, n)).astype(np.float32)
    da, dbt, dbias, dres = dev(a, torch.bfloat16), dev(bt, torch.bfloat16), dev(bias), dev(resid)
    ws = torch.zeros(lib().tnsr_b200_gemm_workspace(), dtype=torch.uint8, device="cuda")
    tol = 4e-6 * k
    ok(lib().tnsr_b200_set_gemm_engine(3))      # the few-row engine for every shape here, not only where it is faster
    try:
        first = gemm_bf16(da, dbt, workspace=ws)
        assert np.max(np.abs(first.cpu().numpy() - ref)) <= tol
        assert int(ws[:8192].view(torch.int32).abs().sum()) == 0
        assert torch.equal(first, gemm_bf16(da, dbt, workspace=ws))
        unsplit = gemm_bf16(da, dbt)                 # same engine, no scratch: one CTA per 128 columns
        assert np.max(np.abs(unsplit.cpu().numpy() - ref)) <= tol
        fused = gemm_bf16(da, dbt, bias=dbias, residual=dres, workspace=ws).cpu().numpy()
        assert np.max(np.abs(fused - (ref + bias + resid))) <= tol + 1e-5
        relu = gemm_bf16(da, dbt, bias=dbias, activation=0, out_dtype=BF16, workspace=ws).float().cpu().numpy()
        assert rel_err(relu, np.maximum(ref + bias, 0)) <= 1 / 128
        stream_buf = dres.clone()      # in place on the residual stream, as the decoder calls it
        ok(lib().tnsr_b200_gemm_bf16_ws(ptr(da), ptr(dbt), ptr(dbias), ptr(stream_buf), ptr(stream_buf), m, n, k, -1, 0,
                                        ptr(ws), ws.numel(), stream()))
        torch.cuda.synchronize()
        assert np.array_equal(stream_buf.cpu().numpy(), fused)
    finally:
        lib().tnsr_b200_set_gemm_engine(0)
    default = gemm_bf16(da, dbt, workspace=ws)      # whichever engine the shape selects by default
    assert np.max(np.abs(default.cpu().numpy() - ref)) <= tol


@pytest.mark.parametrize("shape", [(256, 768, 768), (256, 768, 2048), (1024, 768, 768), (300, 200, 136), (129, 132, 72),
                                   (33, 36, 40), (4096, 768, 2048)])
@pytest.mark.parametrize("activation", [-1, 1])
def test_gemm_bf16_in_place_residual_update_equals_out_of_place(shape, activation):
    """out == residual (how the decoder updates its residual stream): the tcgen05 engine hands the blocks to a TMA
    reduce-add instead of reading and rewriting the rows.  One add per element, so the bits must equal the out-of-place
    result of the same engine, block edges and clipped tiles included."""
    m, n, k = shape
    a, bt, ref = gemm_case(m, n, k, seed=31, scale=0.1)
    rng = np.random.default_rng(32)
    bias = rng.standard_normal(n).astype(np.float32)
    resid = rng.standard_normal((m, n)).astype(np.float32)
    da, dbt, dbias, dres = dev(a, torch.bfloat16), dev(bt, torch.bfloat16), dev(bias), dev(resid)
    apart = gemm_bf16(da, dbt, bias=dbias, residual=dres, activation=activation)
    buf = dres.clone()
    ok(lib().tnsr_b200_gemm_bf16(ptr(da), ptr(dbt), ptr(dbias), ptr(buf), ptr(buf), m, n, k, activation, 0, stream()))
    torch.cuda.synchronize()
    assert torch.equal(buf, apart)
    if activation == -1:
        assert np.max(np.abs(buf.cpu().numpy() - (ref + bias + resid))) <= 2e-3
    twice = buf.clone()        # a second update accumulates on top of the first
    ok(lib().tnsr_b200_gemm_bf16(ptr(da), ptr(dbt), ptr(dbias), ptr(twice), ptr(twice), m, n, k, activation, 0, stream()))
    torch.cuda.synchronize()
    again = gemm_bf16(da, dbt, bias=dbias, residual=buf, activation=activation)
    assert torch.equal(twice, again)


# ---- SwiGLU ----------------------------------------------------------------------
def test_swiglu_elementwise(oracle):
    import json, os
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")) as f:
        bits = json.load(f)["activations"]["input_bits"]
    x = np.asarray(bits, np.uint32).view(np.float32)
    rng = np.random.default_rng(8)
    gate = bf16_round(np.concatenate([x, rng.standard_normal(4096 + 5) * 3]))
    up = bf16_round(rng.standard_normal(gate.size))
    # pad to a multiple of 8 + a ragged tail
    out = torch.empty(gate.size, dtype=torch.bfloat16, device="cuda")
    ok(lib().tnsr_b200_swiglu(ptr(dev(gate, torch.bfloat16)), ptr(dev(up, torch.bfloat16)), ptr(out), gate.size, stream()))
    torch.cuda.synchronize()
    expected = oracle.swiglu(gate, up)
    got = out.float().cpu().numpy()
    assert np.all(np.abs(got - expected) <= np.abs(expected) / 128 + 1e-6)


@pytest.mark.parametrize("engine", [1, 2])
def test_swiglu_mlp_block(oracle, engine):
    rows, d, f = 96, 128, 352
    rng = np.random.default_rng(3)
    x = bf16_round(rng.standard_normal((rows, d)))
    wg, wu = bf16_round(rng.standard_normal((d, f)) * 0.05), bf16_round(rng.standard_normal((d, f)) * 0.05)
    wd = bf16_round(rng.standard_normal((f, d)) * 0.05)
    bg, bu, bd = (rng.standard_normal(f) * 0.1).astype(np.float32), (rng.standard_normal(f) * 0.1).astype(np.float32), \
        (rng.standard_normal(d) * 0.1).astype(np.float32)
    expected = oracle.swiglu_mlp(x, wg, bg, wu, bu, wd, bd)
    packed_w = torch.empty((2 * f, d), dtype=torch.bfloat16, device="cuda")
    packed_b = torch.empty(2 * f, dtype=torch.float32, device="cuda")
    ok(lib().tnsr_b200_pack_gate_up(ptr(dev(wg, torch.bfloat16)), ptr(dev(wu, torch.bfloat16)), ptr(dev(bg)), ptr(dev(bu)),
                                    ptr(packed_w), ptr(packed_b), d, f, stream()))
    wdt = torch.empty((d, f), dtype=torch.bfloat16, device="cuda")
    ok(lib().tnsr_b200_transpose_bf16(ptr(dev(wd, torch.bfloat16)), ptr(wdt), f, d, stream()))
    hidden = torch.empty((rows, f), dtype=torch.bfloat16, device="cuda")
    out = torch.empty((rows, d), dtype=torch.bfloat16, device="cuda")
    try:
        ok(lib().tnsr_b200_set_gemm_engine(engine))
        ok(lib().tnsr_b200_swiglu_mlp(ptr(dev(x, torch.bfloat16)), ptr(packed_w), ptr(packed_b), ptr(wdt), ptr(dev(bd)),
                                      ptr(hidden), ptr(out), rows, d, f, stream()))
        torch.cuda.synchronize()
    finally:
        lib().tnsr_b200_set_gemm_engine(0)
    assert rel_err(out.float().cpu().numpy(), expected) <= 2e-2


# ---- attention -------------------------------------------------------------------
def run_decode_attention(q, kc, vc, lengths, heads):
    batch, capacity, d = kc.shape
    hd = d // heads
    ws_bytes = lib().tnsr_b200_decode_attention_workspace(batch, capacity, heads, hd)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    out = torch.full((batch, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    ok(lib().tnsr_b200_decode_attention(ptr(dev(q, torch.bfloat16)), ptr(dev(kc, torch.bfloat16)), ptr(dev(vc, torch.bfloat16)),
                                        ptr(dev(np.asarray(lengths, np.uint32).view(np.int32))), ptr(out), ptr(ws), ws_bytes,
                                        batch, capacity, heads, hd, stream()))
    torch.cuda.synchronize()
    status = int(ws[64:68].view(torch.int32)[0])
    assert status == 0, f"device status {status}"
    return out.float().cpu().numpy()


@pytest.mark.parametrize("heads,hd", [(12, 64), (16, 64), (3, 32), (20, 64), (5, 128), (2, 64)])
def test_decode_attention_live_prefix_and_poisoned_slots(oracle, heads, hd):
    """Style of src/nn/kv_cache/cuda/tests.rs:30-172: formula inputs, unused
    slots NaN, lengths around the 16-key stage and the slab boundaries."""
    d = heads * hd
    lengths = [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 200, 300]
    batch, capacity = len(lengths), 300
    q = bf16_round(attention_samples(batch * d, 5).reshape(batch, d) / 4)
    kc = bf16_round(attention_samples(batch * capacity * d, 41).reshape(batch, capacity, d))
    vc = bf16_round(attention_samples(batch * capacity * d, 67).reshape(batch, capacity, d))
    for b, n in enumerate(lengths):
        kc[b, n:] = np.nan
        vc[b, n:] = np.nan
    got = run_decode_attention(q, kc, vc, lengths, heads)
    kz, vz = np.nan_to_num(kc), np.nan_to_num(vc)
    expected = oracle.decode_attention(q, kz, vz, np.asarray(lengths, np.uint32), heads)
    assert np.all(np.isfinite(got))
    scale = max(1.0, float(np.max(np.abs(expected))))
    assert np.max(np.abs(got - expected)) <= scale / 128


def test_decode_attention_ragged_long_context(oracle):
    """Configuration 3 in miniature: per-session lengths uniform in [1, capacity]."""
    heads, hd, batch, capacity = 16, 64, 12, 4096
    d = heads * hd
    rng = np.random.default_rng(4)
    lengths = rng.integers(1, capacity + 1, size=batch).astype(np.uint32)
    lengths[0], lengths[1] = capacity, 1
    q = bf16_round(rng.standard_normal((batch, d)))
    kc = bf16_round(rng.standard_normal((batch, capacity, d)))
    vc = bf16_round(rng.standard_normal((batch, capacity, d)))
    got = run_decode_attention(q, kc, vc, lengths, heads)
    oracle.set_threads(oracle.max_threads())
    try:
        expected = oracle.decode_attention(q, kc, vc, lengths, heads)
    finally:
        oracle.set_threads(1)
    assert np.max(np.abs(got - expected)) <= max(1.0, float(np.max(np.abs(expected)))) / 128


def test_decode_attention_zero_length_gives_zero_row():
    heads, hd, batch, capacity = 4, 64, 3, 40
    d = heads * hd
    rng = np.random.default_rng(9)
    q = bf16_round(rng.standard_normal((batch, d)))
    kc = bf16_round(rng.standard_normal((batch, capacity, d)))
    vc = bf16_round(rng.standard_normal((batch, capacity, d)))
    got = run_decode_attention(q, kc, vc, [5, 0, 40], heads)
    assert np.all(got[1] == 0) and np.any(got[0] != 0) and np.any(got[2] != 0)


def test_decode_attention_propagates_non_finite_values(oracle):
    """src/nn/kv_cache/cuda/tests.rs:242-333: inf/NaN in V reach the output of that head only."""
    heads, hd, batch, capacity = 2, 64, 1, 200
    d = heads * hd
    rng = np.random.default_rng(10)
    q = bf16_round(rng.standard_normal((batch, d)))
    kc = bf16_round(rng.standard_normal((batch, capacity, d)))
    vc = bf16_round(rng.standard_normal((batch, capacity, d)))
    vc[0, 150, 3] = np.inf
    vc[0, 20, 64 + 7] = np.nan
    got = run_decode_attention(q, kc, vc, [200], heads)
    assert np.isinf(got[0, 3]) and np.isnan(got[0, 64 + 7])
    mask = np.ones(d, bool)
    mask[[3, 64 + 7]] = False
    assert np.all(np.isfinite(got[0, mask]))


@pytest.mark.parametrize("hd,chunk,prefix", [(64, 1, 0), (64, 3, 65), (64, 16, 0), (64, 17, 31), (64, 33, 129),
                                             (64, 130, 7), (4, 3, 33), (33, 17, 31), (128, 16, 5)])
def test_prefill_attention_matches_f64_reference(oracle, hd, chunk, prefix):
    """Shapes of src/nn/kv_cache/cuda/bf16_tests.rs:95-110,263-303; tolerance max|ref|/128."""
    batch, heads = 2, 2
    d = heads * hd
    capacity = prefix + chunk + 9
    salt = lambda n, s: bf16_round(attention_samples(n, s, 53.0, 1.0))
    q = salt(batch * chunk * d, 5).reshape(batch, chunk, d)
    k = salt(batch * chunk * d, 19).reshape(batch, chunk, d)
    v = salt(batch * chunk * d, 37).reshape(batch, chunk, d)
    ck = salt(batch * capacity * d, 41).reshape(batch, capacity, d)
    cv = salt(batch * capacity * d, 67).reshape(batch, capacity, d)
    ref = oracle.attention_f64(q, k, v, ck, cv, heads, prefix)          # [batch, heads, chunk, hd]
    kc, vc = ck.copy(), cv.copy()
    kc[:, prefix:prefix + chunk] = k
    vc[:, prefix:prefix + chunk] = v
    kc[:, prefix + chunk:] = np.nan
    vc[:, prefix + chunk:] = np.nan
    out = torch.empty((batch, chunk, d), dtype=torch.bfloat16, device="cuda")
    ok(lib().tnsr_b200_prefill_attention(ptr(dev(q, torch.bfloat16)), ptr(dev(kc, torch.bfloat16)), ptr(dev(vc, torch.bfloat16)),
                                         ptr(out), batch, chunk, prefix, capacity, heads, hd, stream()))
    torch.cuda.synchronize()
    got = out.float().cpu().numpy().reshape(batch, chunk, heads, hd).transpose(0, 2, 1, 3)
    assert np.all(np.isfinite(got))
    assert np.max(np.abs(got - ref)) <= max(1.0, float(np.max(np.abs(ref)))) / 128


@pytest.mark.parametrize("chunk,prefix,heads,batch", [(32, 0, 1, 1), (128, 0, 2, 2), (128, 128, 3, 1), (256, 5, 2, 2),
                                                      (300, 213, 3, 2), (512, 0, 2, 1), (77, 1000, 1, 2)])
def test_prefill_attention_tcgen05_kernel_matches_f64_reference_and_warp_mma_kernel(oracle, chunk, prefix, heads, batch):
    """Chunks of 32 rows and more at head width 64 run on the tcgen05 kernel: one to many 128-key blocks, ragged
    last query tile, stale (NaN) cache rows past the live range.  Engine 1 selects the warp-level kernel for the
    same call; both must sit within max|ref|/128 of the f64 reference."""
    hd = 64
    d = heads * hd
    capacity = prefix + chunk + 3
    salt = lambda n, s: bf16_round(attention_samples(n, s, 53.0, 1.0))
    q = salt(batch * chunk * d, 7).reshape(batch, chunk, d)
    k = salt(batch * chunk * d, 23).reshape(batch, chunk, d)
    v = salt(batch * chunk * d, 31).reshape(batch, chunk, d)
    ck = salt(batch * capacity * d, 43).reshape(batch, capacity, d)
    cv = salt(batch * capacity * d, 71).reshape(batch, capacity, d)
    ref = oracle.attention_f64(q, k, v, ck, cv, heads, prefix)
    kc, vc = ck.copy(), cv.copy()
    kc[:, prefix:prefix + chunk] = k
    vc[:, prefix:prefix + chunk] = v
    kc[:, prefix + chunk:] = np.nan
    vc[:, prefix + chunk:] = np.nan
    dq, dk, dv = dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16)
    results = []
    for engine in (0, 1):
        out = torch.full((batch, chunk, d), float("nan"), dtype=torch.bfloat16, device="cuda")
        ok(lib().tnsr_b200_set_gemm_engine(engine))
        try:
            ok(lib().tnsr_b200_prefill_attention(ptr(dq), ptr(dk), ptr(dv), ptr(out), batch, chunk, prefix, capacity,
                                                 heads, hd, stream()))
            torch.cuda.synchronize()
        finally:
            lib().tnsr_b200_set_gemm_engine(0)
        got = out.float().cpu().numpy().reshape(batch, chunk, heads, hd).transpose(0, 2, 1, 3)
        assert np.all(np.isfinite(got))
        assert np.max(np.abs(got - ref)) <= max(1.0, float(np.max(np.abs(ref)))) / 128
        results.append(got)
    assert np.max(np.abs(results[0] - results[1])) <= max(1.0, float(np.max(np.abs(ref)))) / 64


# ---- greedy pick -------------------------------------------------------------------
def test_argmax_prefers_the_last_maximum(oracle):
    rng = np.random.default_rng(13)
    rows, vocab = 9, 1000
    logits = rng.standard_normal((rows, vocab)).astype(np.float32)
    logits[0, [10, 500, 999]] = 9.0
    logits[1, :] = -0.0
    logits[1, 7] = 0.0
    logits[2, 100] = np.inf
    logits[2, 200] = np.nan
    logits[3, :] = -np.inf
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ok(lib().tnsr_b200_argmax(ptr(dev(logits)), ptr(out), rows, vocab, stream()))
    torch.cuda.synchronize()
    got = out.cpu().numpy().astype(np.int64).tolist()
    assert got == [oracle.argmax_last(logits[r]) for r in range(rows)]
    assert got[0] == 999 and got[1] == 7 and got[2] == 200 and got[3] == vocab - 1
    small = np.asarray([[1, 3, 3, 2]], np.float32)
    out = torch.empty(1, dtype=torch.int32, device="cuda")
    ok(lib().tnsr_b200_argmax(ptr(dev(small)), ptr(out), 1, 4, stream()))
    torch.cuda.synchronize()
    assert int(out[0]) == 2


@pytest.mark.parametrize("vocab,top_k,temperature", [(32000, 40, 0.8), (32000, 256, 1.3), (1000, 5, 0.5), (97, 1, 1.0),
                                                     (50, 256, 2.0)])
def test_sample_top_k_matches_the_cpu_restatement(vocab, top_k, temperature):
    """Device sampling against oracle/sampler.py on the same logits: same candidates (ties towards the larger index),
    same f32 weights and running sums, same Philox draw -> the same id for every row."""
    from oracle import sampler
    rng = np.random.default_rng(vocab + top_k)
    rows = 48
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    logits[1, ::7] = logits[1].max()                       # many ties at the top
    logits[2, :] = 0.25                                    # all equal: the candidates are the last top_k indices
    logits[3, 5] = -0.0
    logits[4, : vocab // 2] = -np.inf
    d_logits = dev(logits)
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    ok(lib().tnsr_b200_sample_top_k(ptr(d_logits), ptr(out), rows, vocab, temperature, top_k, 0x1234567890ABCDEF, 77, 9,
                                    stream()))
    torch.cuda.synchronize()
    want = sampler.sample(logits, temperature, top_k, 0x1234567890ABCDEF, 77, first_session=9)
    assert np.array_equal(out.cpu().numpy().astype(np.uint32), want)
    if top_k == 1:
        greedy = torch.zeros(rows, dtype=torch.int32, device="cuda")
        ok(lib().tnsr_b200_argmax(ptr(d_logits), ptr(greedy), rows, vocab, stream()))
        torch.cuda.synchronize()
        assert torch.equal(out, greedy)
    assert lib().tnsr_b200_sample_top_k(ptr(d_logits), ptr(out), rows, vocab, 0.0, top_k, 1, 0, 0, stream()) == -1
    assert lib().tnsr_b200_sample_top_k(ptr(d_logits), ptr(out), rows, vocab, 1.0, 257, 1, 0, 0, stream()) == -1


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (8, 4096, 4096), (16, 32000, 768), (13, 100, 528), (5, 48, 16),
                                   (16, 1000, 1040), (9, 2304, 768)])
def test_gemm_bf16_weight_streaming_engine_matches_f64(shape):
    """m <= 16: one pass over the weights, 16 weight rows per CTA at a time, no split-K and no scratch (gemm_stream.cu).
    Same tolerance as the other engines, two runs bit-identical, epilogues (bias, activation, residual, bf16 output,
    in place on the residual stream) included; engine 4 forces it also below the size from which it is the default."""
    m, n, k = shape
    a, bt, ref = gemm_case(m, n, k, seed=13)
    rng = np.random.default_rng(14)
    bias = rng.standard_normal(n).astype(np.float32)
    resid = rng.standard_normal((m, n)).astype(np.float32)
    da, dbt, dbias, dres = dev(a, torch.bfloat16), dev(bt, torch.bfloat16), dev(bias), dev(resid)
    tol = 4e-6 * k
    before = lib().tnsr_b200_kernel_launches()
    ok(lib().tnsr_b200_set_gemm_engine(4))
    try:
        first = gemm_bf16(da, dbt)
        assert lib().tnsr_b200_kernel_launches() - before == 1
        assert np.max(np.abs(first.cpu().numpy() - ref)) <= tol
        assert torch.equal(first, gemm_bf16(da, dbt))
        fused = gemm_bf16(da, dbt, bias=dbias, residual=dres).cpu().numpy()
        assert np.max(np.abs(fused - (ref + bias + resid))) <= tol + 1e-5
        relu = gemm_bf16(da, dbt, bias=dbias, activation=0, out_dtype=BF16).float().cpu().numpy()
        assert rel_err(relu, np.maximum(ref + bias, 0)) <= 1 / 128
        stream_buf = dres.clone()
        ok(lib().tnsr_b200_gemm_bf16(ptr(da), ptr(dbt), ptr(dbias), ptr(stream_buf), ptr(stream_buf), m, n, k, -1, 0, stream()))
        torch.cuda.synchronize()
        assert np.array_equal(stream_buf.cpu().numpy(), fused)
    finally:
        lib().tnsr_b200_set_gemm_engine(0)
    ok(lib().tnsr_b200_set_gemm_engine(2))          # against the tcgen05 engine on the same operands
    try:
        other = gemm_bf16(da, dbt).cpu().numpy()
    finally:
        lib().tnsr_b200_set_gemm_engine(0)
    assert np.max(np.abs(other - first.cpu().numpy())) <= tol
