"""The C-ABI library loads without a GPU and exports every declared symbol."""
import ctypes as C
import os
import re

import pytest

from yuuka_b200 import build, cuda

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def native():
    build.build_all()
    return C.CDLL(build.CUDA_LIB)


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "yuuka_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"YUUKA_API[^;(]*?\b(yuuka_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(native):
    names = declared_symbols()
    assert len(names) > 20
    missing = [n for n in names if not hasattr(native, n)]
    assert not missing, missing


def test_binding_covers_the_header():
    assert sorted(cuda.SIGNATURES) == declared_symbols()


def test_abi_version_and_error_channel(native):
    native.yuuka_abi_version.restype = C.c_uint32
    assert native.yuuka_abi_version() == cuda.ABI_VERSION
    native.yuuka_last_error.restype = C.c_char_p
    out = C.c_void_p()
    # null out-pointer is rejected before any device work
    assert native.yuuka_device_open(0, None) == cuda.ERR_INVALID_ARGUMENT
    assert b"null" in native.yuuka_last_error()
    import torch
    if not torch.cuda.is_available():
        # no device: the call fails loudly, there is no CPU fallback
        assert native.yuuka_device_open(0, C.byref(out)) == cuda.ERR_DEVICE
        assert b"no CPU fallback" in native.yuuka_last_error()
        assert not out.value


def test_library_does_not_link_the_oracle():
    import subprocess
    out = subprocess.run(["ldd", build.CUDA_LIB], capture_output=True, text=True).stdout
    assert "oracle" not in out and "torch" not in out
