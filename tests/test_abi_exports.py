"""The C-ABI library loads without a GPU and exports exactly what the header declares."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_library():
    from tnsr_b200 import build
    return build.build()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tnsr_b200.h")).read()
    return sorted(set(re.findall(r"TNSR_B200_API[^;(]*?\b(tnsr_b200_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(built_library):
    from tnsr_b200 import _native
    names = declared_symbols()
    assert len(names) >= 25
    out = subprocess.check_output(["nm", "-D", "--defined-only", built_library], text=True)
    exported = set(re.findall(r"\b(tnsr_b200_\w+)\b", out))
    assert exported == set(names)
    assert set(_native.SIGNATURES) == set(names)
    lib = _native.lib()
    for name in names:
        assert getattr(lib, name) is not None


def test_library_answers_without_a_device(built_library):
    from tnsr_b200 import _native
    lib = _native.lib()
    assert b"sm_100a" in lib.tnsr_b200_version()
    assert lib.tnsr_b200_kernel_launches() >= 0
    assert lib.tnsr_b200_device_count() >= 0 or lib.tnsr_b200_device_count() == -9
    assert lib.tnsr_b200_decode_attention_workspace(64, 4096, 16, 64) > 0


def test_create_reports_errors_instead_of_crashing(built_library):
    import ctypes as C
    from tnsr_b200 import _native
    lib = _native.lib()
    handle = C.c_void_p()
    bad = _native.Config(96, 128, 128, 4, 512, 4, 1e-5, 0, 0, 0, 0, 128, 0, 0)   # batch 0
    assert lib.tnsr_b200_decoder_create(C.byref(bad), C.byref(handle)) == -1
    assert "batch size must be non-zero" in _native.last_error(None)
    bad = _native.Config(96, 128, 128, 4, 512, 4, 1e-5, 0, 0, 0, 1, 129, 0, 0)   # capacity > context
    assert lib.tnsr_b200_decoder_create(C.byref(bad), C.byref(handle)) == -1
    assert "capacity must fit the model context" in _native.last_error(None)
    bad = _native.Config(96, 128, 128, 4, 512, 4, 1e-5, 0, 1, 0, 1, 128, 0, 0)   # bf16 weights, f32 cache
    assert lib.tnsr_b200_decoder_create(C.byref(bad), C.byref(handle)) == -1
    if lib.tnsr_b200_device_count() <= 0:
        good = _native.Config(96, 128, 128, 4, 512, 4, 1e-5, 0, 0, 0, 1, 128, 0, 0)
        assert lib.tnsr_b200_decoder_create(C.byref(good), C.byref(handle)) == -9
        assert "initialize CUDA decoder" in _native.last_error(None)
        from tnsr_b200 import Backend, Gpt, GptConfig, TnsrError
        with pytest.raises(TnsrError) as err:
            Gpt(GptConfig(96, 8, 8, 2, 13, 1, 1e-5)).decoder(Backend.Cuda, 1)
        assert "initialize CUDA decoder" in str(err.value)
