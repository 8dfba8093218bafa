"""The C-ABI library loads without a GPU and exports every symbol declared in
include/basedxl_b200.h (no compute call is made here)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "basedxl_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bxl_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    from basedxl_b200 import _lib, build

    build.build()
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    # and the ctypes table covers exactly the header
    assert sorted(_lib.SIGNATURES) == names


def test_error_message_channel_works_without_a_gpu():
    from basedxl_b200 import _lib

    lib = _lib.load()
    # a null operand is rejected before any CUDA call is made
    rc = lib.bxl_gemm_f16(None, 8, None, 8, 0, None, None, 0, None, 8, 0, 128, 128, 64, None)
    assert rc < 0 and b"null operand" in lib.bxl_last_error()


def test_ops_fail_loudly_without_a_device():
    import pytest
    import torch

    from basedxl_b200 import _lib

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(_lib.BxlError):
        _lib.lib()
