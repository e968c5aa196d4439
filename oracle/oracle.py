"""ctypes front end of the CPU checker (``libtnsr_oracle.so``).

TEST INFRASTRUCTURE ONLY.  Importers: ``tests/``, ``__graft_entry__.smoke()`` and
the CPU-baseline / reference legs of ``bench.py``.  The shipped package
``tnsr_b200`` never imports this module.

``OracleBackend`` implements the same small backend protocol as the CUDA
library's session object (``reset`` / ``decode``), i.e. the role
``DecoderBackend::Cpu(SimpleExecutor)`` plays in the reference
(src/nn/kv_cache.rs:60-64), so the shared ``GptDecoder`` wrapper can drive it
in tests exactly as it drives the GPU.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtnsr_oracle.so")

ACT = {"relu": 0, "gelu": 1, "swiglu": 2}

ERRORS = {
    -1: "invalid argument",
    -2: "Embedding index must be finite",
    -3: "Embedding index must be non-negative",
    -4: "Embedding index must be an integer",
    -5: "Embedding index cannot be represented as usize",
    -6: "Embedding index is out of range for size",
    -7: "decoder context capacity exceeded",
    -8: "allocation failed",
}


class OracleError(RuntimeError):
    pass


def build(force: bool = False) -> str:
    """Compile the checker with the recipe in ``oracle/Makefile``."""
    src = os.path.join(_HERE, "tnsr_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libtnsr_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


class _Config(C.Structure):
    _fields_ = [
        ("vocab_size", C.c_uint32),
        ("max_sequence_length", C.c_uint32),
        ("embed_dim", C.c_uint32),
        ("num_heads", C.c_uint32),
        ("feed_forward_dim", C.c_uint32),
        ("num_layers", C.c_uint32),
        ("layer_norm_epsilon", C.c_float),
        ("activation", C.c_uint32),
        ("attention_bf16", C.c_uint32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        fp, u32p, dp = C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.POINTER(C.c_double)
        sz, vp = C.c_size_t, C.c_void_p
        sig = {
            "oracle_set_threads": (None, [C.c_int]),
            "oracle_get_threads": (C.c_int, []),
            "oracle_max_threads": (C.c_int, []),
            "oracle_bf16_round": (C.c_float, [C.c_float]),
            "oracle_bf16_bits": (C.c_uint16, [C.c_float]),
            "oracle_sigmoid": (None, [fp, fp, sz]),
            "oracle_silu": (None, [fp, fp, sz]),
            "oracle_gelu": (None, [fp, fp, sz]),
            "oracle_swiglu": (None, [fp, fp, fp, sz]),
            "oracle_embedding": (C.c_int, [fp, sz, sz, fp, sz, fp]),
            "oracle_matmul": (None, [fp, fp, fp, sz, sz, sz, sz, sz]),
            "oracle_matmul_naive": (None, [fp, fp, fp, sz, sz, sz]),
            "oracle_matmul_bf16": (None, [fp, fp, fp, sz, sz, sz, sz, sz]),
            "oracle_linear": (None, [fp, fp, fp, fp, sz, sz, sz]),
            "oracle_softmax": (None, [fp, fp, sz, sz]),
            "oracle_layer_norm": (None, [fp, fp, fp, C.c_float, fp, sz, sz]),
            "oracle_model_create": (vp, [C.POINTER(_Config)]),
            "oracle_model_destroy": (None, [vp]),
            "oracle_model_param_count": (sz, [vp]),
            "oracle_model_param_elems": (sz, [vp, sz]),
            "oracle_model_set_param": (C.c_int, [vp, sz, fp, sz]),
            "oracle_model_get_param": (C.c_int, [vp, sz, fp, sz]),
            "oracle_xavier": (None, [fp, sz, sz, C.c_uint64]),
            "oracle_model_init_reference": (None, [vp]),
            "oracle_decoder_create": (vp, [vp, sz, sz]),
            "oracle_decoder_destroy": (None, [vp]),
            "oracle_decoder_reset": (None, [vp]),
            "oracle_decoder_len": (sz, [vp]),
            "oracle_decoder_read_cache": (C.c_int, [vp, sz, fp]),
            "oracle_decoder_write_cache": (C.c_int, [vp, sz, fp]),
            "oracle_decoder_set_len": (None, [vp, sz]),
            "oracle_decoder_decode": (C.c_int, [vp, u32p, sz, fp]),
            "oracle_forward": (C.c_int, [vp, u32p, sz, sz, fp]),
            "oracle_argmax_last": (sz, [fp, sz]),
            "oracle_generate": (C.c_int, [vp, u32p, sz, sz, u32p]),
            "oracle_generate_cached": (C.c_int, [vp, u32p, sz, sz, u32p]),
            "oracle_decode_attention": (None, [fp, fp, fp, u32p, sz, sz, sz, sz, fp]),
            "oracle_attention_f64": (None, [fp, fp, fp, fp, fp, sz, sz, sz, sz, sz, sz, dp]),
            "oracle_swiglu_mlp": (C.c_int, [fp, fp, fp, fp, fp, fp, fp, fp, sz, sz, sz]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _u(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint32))


def _check(rc):
    if rc != 0:
        raise OracleError(ERRORS.get(rc, f"oracle error {rc}"))


def set_threads(n: int) -> None:
    lib().oracle_set_threads(int(n))


def max_threads() -> int:
    return int(lib().oracle_max_threads())


# -- primitives ---------------------------------------------------------------

def bf16_round(x):
    x = np.asarray(x, dtype=np.float32)
    out = np.empty_like(x)
    flat_in, flat_out = x.reshape(-1), out.reshape(-1)
    L = lib()
    for i in range(flat_in.size):
        flat_out[i] = L.oracle_bf16_round(float(flat_in[i]))
    return out


def bf16_round_np(x):
    """Vectorised numpy twin of ``oracle_bf16_round`` for large arrays (tests
    check the two agree)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    quiet = (u | 0x00400000) & 0xFFFF0000
    return np.where(nan, quiet, rounded).astype(np.uint32).view(np.float32).reshape(x.shape)


def _unary(name, x):
    x, px = _f(x)
    y = np.empty_like(x)
    getattr(lib(), name)(px, y.ctypes.data_as(C.POINTER(C.c_float)), x.size)
    return y


def sigmoid(x):
    return _unary("oracle_sigmoid", x)


def silu(x):
    return _unary("oracle_silu", x)


def gelu(x):
    return _unary("oracle_gelu", x)


def swiglu(gate, up):
    g, pg = _f(gate)
    u, pu = _f(up)
    y = np.empty_like(g)
    lib().oracle_swiglu(pg, pu, y.ctypes.data_as(C.POINTER(C.c_float)), g.size)
    return y


def embedding(weight, indices):
    w, pw = _f(weight)
    idx, pi = _f(indices)
    out = np.empty(idx.shape + (w.shape[1],), dtype=np.float32)
    _check(lib().oracle_embedding(pw, w.shape[0], w.shape[1], pi, idx.size,
                                  out.ctypes.data_as(C.POINTER(C.c_float))))
    return out


def matmul(a, b, naive=False):
    a, pa = _f(a)
    b, pb = _f(b)
    m, k = a.shape[-2:]
    n = b.shape[-1]
    assert b.shape[-2] == k
    batches = int(np.prod(a.shape[:-2], dtype=np.int64)) if a.ndim > 2 else 1
    b_batches = int(np.prod(b.shape[:-2], dtype=np.int64)) if b.ndim > 2 else 1
    assert b_batches in (1, batches)
    out = np.empty(a.shape[:-2] + (m, n), dtype=np.float32)
    po = out.ctypes.data_as(C.POINTER(C.c_float))
    if naive:
        assert batches == 1
        lib().oracle_matmul_naive(pa, pb, po, m, k, n)
    else:
        lib().oracle_matmul(pa, pb, po, batches, b_batches, m, k, n)
    return out


def matmul_bf16(a, b):
    a, pa = _f(a)
    b, pb = _f(b)
    m, k = a.shape[-2:]
    n = b.shape[-1]
    batches = int(np.prod(a.shape[:-2], dtype=np.int64)) if a.ndim > 2 else 1
    b_batches = int(np.prod(b.shape[:-2], dtype=np.int64)) if b.ndim > 2 else 1
    out = np.empty(a.shape[:-2] + (m, n), dtype=np.float32)
    lib().oracle_matmul_bf16(pa, pb, out.ctypes.data_as(C.POINTER(C.c_float)), batches, b_batches, m, k, n)
    return out


def linear(x, w, b=None):
    x, px = _f(x)
    w, pw = _f(w)
    k, n = w.shape
    m = x.size // k
    out = np.empty(x.shape[:-1] + (n,), dtype=np.float32)
    if b is None:
        pb = None
    else:
        b, pb = _f(b)
    lib().oracle_linear(px, pw, pb, out.ctypes.data_as(C.POINTER(C.c_float)), m, k, n)
    return out


def softmax(x):
    x, px = _f(x)
    y = np.empty_like(x)
    n = x.shape[-1]
    lib().oracle_softmax(px, y.ctypes.data_as(C.POINTER(C.c_float)), x.size // n, n)
    return y


def layer_norm(x, w, b, eps):
    x, px = _f(x)
    w, pw = _f(w)
    b, pb = _f(b)
    y = np.empty_like(x)
    n = x.shape[-1]
    lib().oracle_layer_norm(px, pw, pb, float(eps), y.ctypes.data_as(C.POINTER(C.c_float)), x.size // n, n)
    return y


def xavier(rows, columns, seed):
    out = np.empty((rows, columns), dtype=np.float32)
    lib().oracle_xavier(out.ctypes.data_as(C.POINTER(C.c_float)), rows, columns, seed)
    return out


def argmax_last(row):
    row, pr = _f(row)
    return int(lib().oracle_argmax_last(pr, row.size))


def decode_attention(q, kcache, vcache, lengths, heads):
    q, pq = _f(q)
    kc, pk = _f(kcache)
    vc, pv = _f(vcache)
    ln, pl = _u(lengths)
    batch, capacity, d = kc.shape
    out = np.zeros((batch, d), dtype=np.float32)
    lib().oracle_decode_attention(pq, pk, pv, pl, batch, capacity, heads, d // heads,
                                  out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def attention_f64(q, k, v, kcache, vcache, heads, prefix):
    """f64 reference: q/k/v [batch, chunk, d]; caches [batch, capacity, d];
    returns [batch, heads, chunk, hd] float64."""
    q, pq = _f(q)
    k, pk = _f(k)
    v, pv = _f(v)
    kc, pkc = _f(kcache)
    vc, pvc = _f(vcache)
    batch, chunk, d = q.shape
    capacity = kc.shape[1]
    hd = d // heads
    out = np.empty((batch, heads, chunk, hd), dtype=np.float64)
    lib().oracle_attention_f64(pq, pk, pv, pkc, pvc, batch, heads, hd, capacity, prefix, chunk,
                               out.ctypes.data_as(C.POINTER(C.c_double)))
    return out


def swiglu_mlp(x, wg, bg, wu, bu, wd, bd):
    x, px = _f(x)
    wg, pwg = _f(wg)
    bg, pbg = _f(bg)
    wu, pwu = _f(wu)
    bu, pbu = _f(bu)
    wd, pwd = _f(wd)
    bd, pbd = _f(bd)
    d, f = wg.shape
    rows = x.size // d
    out = np.empty((rows, d), dtype=np.float32)
    _check(lib().oracle_swiglu_mlp(px, pwg, pbg, pwu, pbu, pwd, pbd,
                                   out.ctypes.data_as(C.POINTER(C.c_float)), rows, d, f))
    return out


# -- model / decoder ----------------------------------------------------------

class OracleModel:
    """Parameter store in ``model_parameters`` order (src/nn/kv_cache.rs:392-421)."""

    def __init__(self, vocab_size, max_sequence_length, embed_dim, num_heads, feed_forward_dim,
                 num_layers, layer_norm_epsilon, activation="relu", attention_bf16=False):
        self.cfg = _Config(vocab_size, max_sequence_length, embed_dim, num_heads, feed_forward_dim,
                           num_layers, layer_norm_epsilon, ACT[activation], int(bool(attention_bf16)))
        self.handle = lib().oracle_model_create(C.byref(self.cfg))
        if not self.handle:
            raise OracleError("invalid model configuration")
        self.vocab_size = vocab_size
        self.max_sequence_length = max_sequence_length

    def __del__(self):
        if getattr(self, "handle", None):
            lib().oracle_model_destroy(self.handle)
            self.handle = None

    def param_count(self):
        return int(lib().oracle_model_param_count(self.handle))

    def param_elems(self, i):
        return int(lib().oracle_model_param_elems(self.handle, i))

    def set_param(self, i, data):
        data, p = _f(np.asarray(data).reshape(-1))
        _check(lib().oracle_model_set_param(self.handle, i, p, data.size))

    def get_param(self, i):
        out = np.empty(self.param_elems(i), dtype=np.float32)
        _check(lib().oracle_model_get_param(self.handle, i, out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def set_params(self, arrays):
        assert len(arrays) == self.param_count()
        for i, a in enumerate(arrays):
            self.set_param(i, a)

    def init_reference(self):
        lib().oracle_model_init_reference(self.handle)

    def forward(self, tokens):
        tok, pt = _u(tokens)
        batch, seq = tok.shape
        out = np.empty((batch, seq, self.vocab_size), dtype=np.float32)
        _check(lib().oracle_forward(self.handle, pt, batch, seq, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def generate(self, prompt, max_new):
        p, pp = _u(prompt)
        out = np.empty(p.size + max_new, dtype=np.uint32)
        _check(lib().oracle_generate(self.handle, pp, p.size, max_new, out.ctypes.data_as(C.POINTER(C.c_uint32))))
        return out.tolist()

    def generate_cached(self, prompt, max_new):
        p, pp = _u(prompt)
        out = np.empty(p.size + max_new, dtype=np.uint32)
        _check(lib().oracle_generate_cached(self.handle, pp, p.size, max_new,
                                            out.ctypes.data_as(C.POINTER(C.c_uint32))))
        return out.tolist()


class OracleBackend:
    """The CPU arm of ``DecoderBackend`` for the shared ``GptDecoder`` wrapper:
    ``refresh(arrays)``, ``reset()``, ``decode(tokens[batch, chunk], position)``."""

    def __init__(self, config, batch, capacity, attention_bf16=False):
        self.model = OracleModel(config.vocab_size, config.max_sequence_length, config.embed_dim,
                                 config.num_heads, config.feed_forward_dim, config.num_layers,
                                 config.layer_norm_epsilon, getattr(config, "activation", "relu"),
                                 attention_bf16)
        self.handle = lib().oracle_decoder_create(self.model.handle, batch, capacity)
        if not self.handle:
            raise OracleError("invalid decoder shape")
        self.batch, self.capacity = batch, capacity

    def __del__(self):
        if getattr(self, "handle", None):
            lib().oracle_decoder_destroy(self.handle)
            self.handle = None

    def refresh(self, index, values):
        self.model.set_param(index, values)

    def reset(self):
        lib().oracle_decoder_reset(self.handle)

    def decode(self, tokens, position):
        tok, pt = _u(tokens)
        batch, chunk = tok.shape
        lib().oracle_decoder_set_len(self.handle, position)
        out = np.empty((batch, chunk, self.model.vocab_size), dtype=np.float32)
        _check(lib().oracle_decoder_decode(self.handle, pt, chunk, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out.reshape(-1)

    def read_cache(self, index):
        d = self.model.cfg.embed_dim
        out = np.empty((self.batch, self.capacity, d), dtype=np.float32)
        _check(lib().oracle_decoder_read_cache(self.handle, index, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def write_cache(self, index, values):
        v, pv = _f(values)
        _check(lib().oracle_decoder_write_cache(self.handle, index, pv))
