"""`tnsr_b200_decode_attention_static`: decode attention for callers that cannot allocate a
workspace (their device memory is fully budgeted up front, or cudaMalloc is not allowed inside
their latency-bound loop).  The entry point keeps its scratch in a fixed array inside the
library, so this test checks that it gives what the ordinary entry point gives -- through the
C ABI, twice in a row with different inputs, because the second call finds the first call's
leftovers in the shared array.  The file name makes pytest collect it last."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from tests.gpu_util import bf16_round, dev, lib, ok, ptr, stream  # noqa: E402

STATIC_BYTES = 32 << 20
_CALLS = {"n": 0}


def with_workspace(q, kc, vc, lengths, heads):
    batch, capacity, d = kc.shape
    hd = d // heads
    ws_bytes = lib().tnsr_b200_decode_attention_workspace(batch, capacity, heads, hd)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    out = torch.full((batch, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    ok(lib().tnsr_b200_decode_attention(ptr(q), ptr(kc), ptr(vc), ptr(lengths), ptr(out), ptr(ws), ws_bytes, batch,
                                        capacity, heads, hd, stream()))
    torch.cuda.synchronize()
    assert int(ws[64:68].view(torch.int32)[0]) == 0
    return out.float().cpu().numpy()


def without_allocation(q, kc, vc, lengths, heads):
    batch, capacity, d = kc.shape
    out = torch.full((batch, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    # cudaMemGetInfo sees every allocation on the device, whoever made it (torch's own counters would only see
    # torch's caching allocator, not a cudaMalloc inside the library)
    free_before, _ = torch.cuda.mem_get_info()
    ok(lib().tnsr_b200_decode_attention_static(ptr(q), ptr(kc), ptr(vc), ptr(lengths), ptr(out), batch, capacity, heads,
                                               d // heads, ptr(status), stream()))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    if _CALLS["n"] > 0:
        # the very first call on a device may make the CUDA runtime load the library's module (its code and the
        # built-in array itself); from the second call on the device's free memory must not shrink at all
        assert free_after >= free_before, (free_before, free_after)
    _CALLS["n"] += 1
    assert int(status[0]) == 0
    return out.float().cpu().numpy()


def case(seed, batch, capacity, heads, hd, lengths):
    rng = np.random.default_rng(seed)
    d = heads * hd
    q = dev(bf16_round(rng.standard_normal((batch, d))), torch.bfloat16)
    kc = dev(bf16_round(rng.standard_normal((batch, capacity, d))), torch.bfloat16)
    vc = dev(bf16_round(rng.standard_normal((batch, capacity, d))), torch.bfloat16)
    ln = dev(np.asarray(lengths, np.uint32).view(np.int32))
    return q, kc, vc, ln


def test_static_scratch_entry_point_matches_the_workspace_one_twice_in_a_row():
    # first call: long, equal lengths -> many items and every partial slot written
    first = case(1, 6, 700, 12, 64, [700] * 6)
    # second call: fewer, ragged sessions incl. an empty one -> most of the array keeps stale partials
    second = case(2, 4, 300, 12, 64, [1, 300, 0, 47])
    for args in (first, second):
        expected = with_workspace(*args, heads=12)
        got = without_allocation(*args, heads=12)
        assert np.all(np.isfinite(got))
        scale = max(1.0, float(np.max(np.abs(expected))))
        assert np.max(np.abs(got - expected)) <= scale / 128
        # same plan, same arithmetic: in practice the two agree to the bit
        assert np.array_equal(got.view(np.uint32), expected.view(np.uint32))
    assert np.all(without_allocation(*second, heads=12)[2] == 0)


def test_static_scratch_entry_point_rejects_what_does_not_fit():
    from tnsr_b200 import _native
    heads, hd = 16, 64
    too_many = 1
    while lib().tnsr_b200_decode_attention_workspace(too_many, 64, heads, hd) <= STATIC_BYTES:
        too_many *= 2
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    code = lib().tnsr_b200_decode_attention_static(ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), too_many, 64,
                                                   heads, hd, None, stream())
    assert code == -8
    message = _native.last_error(None)
    assert str(STATIC_BYTES) in message and "workspace" in message
    code = lib().tnsr_b200_decode_attention_static(ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), 4, 64, 3, 48,
                                                   None, stream())
    assert code == -8
    assert lib().tnsr_b200_decode_attention_static(None, ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), 4, 64, 4, 64, None,
                                                   stream()) == -1
