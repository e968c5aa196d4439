"""Helpers for the GPU tests: torch owns device memory and streams; every
computation goes through the C ABI of libtnsr_b200.so."""
import ctypes as C

import numpy as np
import torch

from tnsr_b200 import _native

F32, BF16 = 0, 1


def lib():
    return _native.lib()


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


_KEEP = []  # device tensors made by dev() stay alive until the test ends (conftest clears this)


def dev(a, dtype=None):
    """Host array -> device tensor.  The tensor is kept alive for the rest of the
    test: the C ABI only sees raw pointers, so a temporary must not be returned
    to torch's caching allocator while a kernel still reads it."""
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    if dtype is not None:
        t = t.to(dtype)
    _KEEP.append(t)
    return t


def ok(code):
    assert code == 0, f"{_native.STATUS.get(code, code)}: {_native.last_error(None)}"


def bf16_round(a):
    """numpy f32 -> nearest bf16 value, as f32 (torch's rounding is RNE too)."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


def rel_err(actual, expected):
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    return float(np.max(np.abs(actual - expected)) / max(np.max(np.abs(expected)), 1e-30))


def gemm_bf16(a, bt, bias=None, residual=None, activation=-1, out_dtype=F32, workspace=None):
    """a [m,k] bf16 cuda, bt [n,k] bf16 cuda -> out [m,n].  `workspace` (a zeroed uint8 cuda tensor of
    tnsr_b200_gemm_workspace() bytes) lends split-K scratch to the few-row engine."""
    m, k = a.shape
    n = bt.shape[0]
    out = torch.empty((m, n), dtype=torch.float32 if out_dtype == F32 else torch.bfloat16, device="cuda")
    if workspace is None:
        ok(lib().tnsr_b200_gemm_bf16(ptr(a), ptr(bt), ptr(bias), ptr(residual), ptr(out), m, n, k, activation, out_dtype,
                                     stream()))
    else:
        ok(lib().tnsr_b200_gemm_bf16_ws(ptr(a), ptr(bt), ptr(bias), ptr(residual), ptr(out), m, n, k, activation, out_dtype,
                                        ptr(workspace), workspace.numel(), stream()))
    torch.cuda.synchronize()
    return out
