"""ctypes binding of ``libtnsr_b200.so`` (the C ABI of include/tnsr_b200.h).

The library is built in-tree by ``python -m tnsr_b200.build`` and loaded from
``tnsr_b200/csrc``.  There is no fallback: if the shared library is missing the
import of anything that needs it raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "csrc", "libtnsr_b200.so")

OK = 0
STATUS = {
    0: "OK", -1: "ERR_INVALID_ARGUMENT", -2: "ERR_CUDA", -3: "ERR_OUT_OF_MEMORY", -4: "ERR_CAPACITY",
    -5: "ERR_TOKEN_RANGE", -6: "ERR_FAILED_STATE", -7: "ERR_TIMEOUT", -8: "ERR_UNSUPPORTED", -9: "ERR_NO_DEVICE",
}
ACT = {"relu": 0, "gelu": 1, "swiglu": 2}
DTYPE = {"f32": 0, "bf16": 1}
LOGITS = {"all": 0, "last": 1, "none": 2}
PREFILL = {"auto": 0, "scalar": 1}


class Config(C.Structure):
    _fields_ = [
        ("vocab_size", C.c_uint32), ("max_sequence_length", C.c_uint32), ("embed_dim", C.c_uint32),
        ("num_heads", C.c_uint32), ("feed_forward_dim", C.c_uint32), ("num_layers", C.c_uint32),
        ("layer_norm_epsilon", C.c_float), ("activation", C.c_uint32), ("weight_dtype", C.c_uint32),
        ("kv_dtype", C.c_uint32), ("batch", C.c_uint32), ("capacity", C.c_uint32), ("device", C.c_int32),
        ("logits_mode", C.c_uint32), ("prefill_mode", C.c_uint32), ("step_parts", C.c_uint32),
        ("kv_page_rows", C.c_uint32), ("kv_pool_pages", C.c_uint32), ("small_batch_mode", C.c_uint32),
    ]


_vp, _u32, _u64, _i, _f = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_float
_fp, _u32p = C.POINTER(C.c_float), C.POINTER(C.c_uint32)

# name -> (restype, argtypes); one entry per declaration in include/tnsr_b200.h
SIGNATURES = {
    "tnsr_b200_version": (C.c_char_p, []),
    "tnsr_b200_device_count": (_i, []),
    "tnsr_b200_last_error": (C.c_char_p, [_vp]),
    "tnsr_b200_kernel_launches": (_u64, []),
    "tnsr_b200_set_gemm_engine": (_i, [_i]),
    "tnsr_b200_set_wait_limit_ns": (_i, [_u64]),
    "tnsr_b200_test_lose_gemm_stage": (_i, [_u32]),
    "tnsr_b200_decoder_create": (_i, [C.POINTER(Config), C.POINTER(_vp)]),
    "tnsr_b200_decoder_destroy": (None, [_vp]),
    "tnsr_b200_decoder_param_count": (_u32, [_vp]),
    "tnsr_b200_decoder_param_elems": (_u64, [_vp, _u32]),
    "tnsr_b200_decoder_upload": (_i, [_vp, _u32, _fp, _u64]),
    "tnsr_b200_decoder_reset": (_i, [_vp]),
    "tnsr_b200_decoder_decode": (_i, [_vp, _u32p, _u32, _u32, _fp, _u32p]),
    "tnsr_b200_decoder_decode_ragged": (_i, [_vp, _u32p, _u32p, _fp, _u32p]),
    "tnsr_b200_decoder_decode_device": (_i, [_vp, _vp, _u32, _u32, _vp]),
    "tnsr_b200_decoder_synchronize": (_i, [_vp]),
    "tnsr_b200_decoder_stream": (_vp, [_vp]),
    "tnsr_b200_decoder_profile_attention": (_i, [_vp, _i]),
    "tnsr_b200_decoder_attention_profile": (_i, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "tnsr_b200_decoder_read_cache": (_i, [_vp, _u32, _fp]),
    "tnsr_b200_decoder_write_cache": (_i, [_vp, _u32, _fp]),
    "tnsr_b200_embedding": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _i, _vp, _vp]),
    "tnsr_b200_layernorm": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _f, _i, _i, _vp]),
    "tnsr_b200_gemm_f32_strict": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _i, _vp]),
    "tnsr_b200_gemm_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _i, _i, _vp]),
    "tnsr_b200_gemm_workspace": (_u64, []),
    "tnsr_b200_gemm_bf16_ws": (_i, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _i, _i, _vp, _u64, _vp]),
    "tnsr_b200_transpose_bf16": (_i, [_vp, _vp, _u32, _u32, _vp]),
    "tnsr_b200_swiglu": (_i, [_vp, _vp, _vp, _u64, _vp]),
    "tnsr_b200_swiglu_mlp": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "tnsr_b200_pack_gate_up": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _vp]),
    "tnsr_b200_decode_attention_workspace": (_u64, [_u32, _u32, _u32, _u32]),
    "tnsr_b200_decode_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _u64, _u32, _u32, _u32, _u32, _vp]),
    "tnsr_b200_decode_attention_static": (_i, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _vp]),
    "tnsr_b200_prefill_attention": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _vp]),
    "tnsr_b200_argmax": (_i, [_vp, _vp, _u32, _u32, _vp]),
    "tnsr_b200_encoder_embed": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _vp]),
    "tnsr_b200_encoder_attention": (_i, [_vp, _vp, _vp, _u32, _vp, _vp, _u32, _u32, _u32, _u32, _vp]),
    "tnsr_b200_add_f32": (_i, [_vp, _vp, _vp, _u64, _vp]),
    "tnsr_b200_swiglu_f32": (_i, [_vp, _vp, _vp, _u64, _vp]),
    "tnsr_b200_sample_top_k": (_i, [_vp, _vp, _u32, _u32, _f, _u32, _u64, _u32, _u32, _vp]),
    "tnsr_b200_decoder_set_sampler": (_i, [_vp, _f, _u32, _u64]),
    "tnsr_b200_decoder_release": (_i, [_vp, _u32]),
    "tnsr_b200_decoder_free_pages": (_u32, [_vp]),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m tnsr_b200.build` "
                "(nvcc, sm_100a). tnsr_b200 has no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def last_error(handle=None) -> str:
    msg = lib().tnsr_b200_last_error(handle)
    return msg.decode("utf-8", "replace") if msg else ""


class NativeError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS.get(code, code)}: {message}")
        self.code = code
        self.message = message


def check(code: int, handle=None) -> None:
    if code != OK:
        raise NativeError(code, last_error(handle))
