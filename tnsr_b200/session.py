"""``B200Session``: the object ``GptDecoder`` drives for ``Backend.Cuda`` /
``Backend.Ptx`` -- a thin owner of one ``tnsr_b200_decoder`` handle, i.e. the
stand-in for ``cuda::CudaDecoder`` (src/nn/kv_cache/cuda.rs:47-218)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native
from ._native import ACT, DTYPE, LOGITS, PREFILL, Config, NativeError, check, lib


class B200Session:
    def __init__(self, config, batch: int, capacity: int, options=None, device: int = 0,
                 logits_mode: str = "all", step_parts: int = 0, kv_page_rows: int = 0, kv_pool_pages: int = 0,
                 small_batch_mode: int = 0):
        from .nn import GptAttentionPrecision, TnsrError
        weight_dtype = getattr(config, "weight_dtype", "f32")
        kv = "bf16" if weight_dtype == "bf16" else "f32"
        if options is not None and options.attention_precision == GptAttentionPrecision.Bf16:
            kv = "bf16"
        self.cfg = Config(config.vocab_size, config.max_sequence_length, config.embed_dim, config.num_heads,
                          config.feed_forward_dim, config.num_layers, config.layer_norm_epsilon,
                          ACT[getattr(config, "activation", "relu")], DTYPE[weight_dtype], DTYPE[kv], batch,
                          capacity, device, LOGITS[logits_mode],
                          PREFILL[options.prefill.value] if options is not None else PREFILL["auto"], step_parts,
                          kv_page_rows, kv_pool_pages, small_batch_mode)
        self.handle = C.c_void_p()
        self.batch, self.capacity, self.vocab = batch, capacity, config.vocab_size
        self.embed_dim = config.embed_dim
        self.logits_mode = logits_mode
        code = lib().tnsr_b200_decoder_create(C.byref(self.cfg), C.byref(self.handle))
        if code != 0:
            self.handle = None
            raise TnsrError(f"initialize CUDA decoder: {_native.last_error(None)}")

    def close(self):
        if getattr(self, "handle", None):
            lib().tnsr_b200_decoder_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, code):
        from .nn import TnsrError
        if code != 0:
            raise TnsrError(_native.last_error(self.handle))

    # -- DecoderBackend protocol ---------------------------------------------
    def refresh(self, index: int, values: np.ndarray) -> None:
        v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        self._check(lib().tnsr_b200_decoder_upload(self.handle, index, v.ctypes.data_as(C.POINTER(C.c_float)), v.size))

    def reset(self) -> None:
        self._check(lib().tnsr_b200_decoder_reset(self.handle))

    def decode(self, tokens: np.ndarray, position: int) -> np.ndarray:
        logits, _ = self.decode_full(tokens, position, want_argmax=False)
        return logits

    # -- extensions -------------------------------------------------------------
    def decode_full(self, tokens: np.ndarray, position: int, want_argmax: bool = True):
        tok = np.ascontiguousarray(tokens, dtype=np.uint32)
        batch, chunk = tok.shape
        assert batch == self.batch
        logits = None
        lp = None
        if self.logits_mode == "all":
            logits = np.empty(batch * chunk * self.vocab, dtype=np.float32)
        elif self.logits_mode == "last":
            logits = np.empty(batch * self.vocab, dtype=np.float32)
        if logits is not None:
            lp = logits.ctypes.data_as(C.POINTER(C.c_float))
        argmax = np.empty(batch, dtype=np.uint32) if want_argmax else None
        ap = argmax.ctypes.data_as(C.POINTER(C.c_uint32)) if want_argmax else None
        self._check(lib().tnsr_b200_decoder_decode(self.handle, tok.ctypes.data_as(C.POINTER(C.c_uint32)), chunk,
                                                   position, lp, ap))
        return logits, argmax

    def decode_ragged(self, tokens: np.ndarray, positions: np.ndarray, want_argmax: bool = True):
        """One new token per session, session b at positions[b]: (logits [batch * vocab] or None, greedy ids or None)."""
        tok = np.ascontiguousarray(tokens, dtype=np.uint32).reshape(-1)
        pos = np.ascontiguousarray(positions, dtype=np.uint32).reshape(-1)
        assert tok.size == self.batch and pos.size == self.batch
        logits = None if self.logits_mode == "none" else np.empty(self.batch * self.vocab, dtype=np.float32)
        lp = logits.ctypes.data_as(C.POINTER(C.c_float)) if logits is not None else None
        argmax = np.empty(self.batch, dtype=np.uint32) if want_argmax else None
        ap = argmax.ctypes.data_as(C.POINTER(C.c_uint32)) if want_argmax else None
        u32p = C.POINTER(C.c_uint32)
        self._check(lib().tnsr_b200_decoder_decode_ragged(self.handle, tok.ctypes.data_as(u32p), pos.ctypes.data_as(u32p), lp, ap))
        return logits, argmax

    def decode_device(self, d_tokens_ptr: int, chunk: int, position: int, d_argmax_ptr: int) -> None:
        self._check(lib().tnsr_b200_decoder_decode_device(self.handle, d_tokens_ptr, chunk, position, d_argmax_ptr))

    def set_sampler(self, temperature: float, top_k: int, seed: int) -> None:
        """Greedy ids become top-k / temperature samples (temperature <= 0: back to greedy)."""
        self._check(lib().tnsr_b200_decoder_set_sampler(self.handle, float(temperature), int(top_k), int(seed)))

    def release(self, session: int) -> None:
        """Paged handles: give the pages of one session back to the pool."""
        self._check(lib().tnsr_b200_decoder_release(self.handle, int(session)))

    def free_pages(self) -> int:
        return int(lib().tnsr_b200_decoder_free_pages(self.handle))

    def synchronize(self) -> None:
        self._check(lib().tnsr_b200_decoder_synchronize(self.handle))

    def stream(self) -> int:
        return int(lib().tnsr_b200_decoder_stream(self.handle) or 0)

    def profile_attention(self, enable: bool) -> None:
        self._check(lib().tnsr_b200_decoder_profile_attention(self.handle, int(enable)))

    def attention_profile(self):
        """(summed device milliseconds, launches) of the decode-attention kernel since the last call."""
        ms, n = C.c_double(), C.c_uint64()
        self._check(lib().tnsr_b200_decoder_attention_profile(self.handle, C.byref(ms), C.byref(n)))
        return ms.value, int(n.value)

    def read_cache(self, index: int) -> np.ndarray:
        out = np.empty((self.batch, self.capacity, self.embed_dim), dtype=np.float32)
        self._check(lib().tnsr_b200_decoder_read_cache(self.handle, index, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def write_cache(self, index: int, values: np.ndarray) -> None:
        v = np.ascontiguousarray(values, dtype=np.float32)
        assert v.size == self.batch * self.capacity * self.embed_dim
        self._check(lib().tnsr_b200_decoder_write_cache(self.handle, index, v.ctypes.data_as(C.POINTER(C.c_float))))
