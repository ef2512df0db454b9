"""The C ABI without a GPU: the library loads, exports every symbol the header
declares, and rejects bad arguments before touching the device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "clusten_b200.h")).read()
    return sorted(set(re.findall(r"CLUSTEN_API\s+[\w\s\*]+?\b(clusten_\w+)\s*\(", text)))


def test_header_declares_the_operators():
    names = _declared()
    for want in ("clusten_qk_forward", "clusten_qk_backward", "clusten_av_forward", "clusten_av_backward",
                 "clusten_wf_forward", "clusten_wf_backward", "clusten_inverse_build", "clusten_inverse_bytes"):
        assert want in names


def test_library_exports_every_declared_symbol(lib):
    for name in _declared():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_covers_every_declared_symbol(lib):
    from clusten import _lib
    assert sorted(_lib.SIGNATURES) == _declared()


def test_status_strings(lib):
    assert lib.clusten_status_string(0) == b"CLUSTEN_OK"
    for code in range(-7, 0):
        assert lib.clusten_status_string(code).startswith(b"CLUSTEN_ERR_")
    assert lib.clusten_version() >= 100


def test_argument_checks_come_before_any_device_work(lib):
    p = ctypes.c_void_p(256)   # never dereferenced: every call below fails validation first
    assert lib.clusten_qk_forward(p, p, p, p, 1, 1, 8, 4, 32, 99, None) == -1      # dtype
    assert lib.clusten_qk_forward(p, p, p, p, 0, 1, 8, 4, 32, 0, None) == -2       # shape
    assert lib.clusten_av_forward(None, p, p, p, 1, 1, 8, 4, 32, 0, None) == -3    # null
    assert lib.clusten_av_forward(ctypes.c_void_p(258), p, p, p, 1, 1, 8, 4, 32, 0, None) == -4  # alignment
    assert lib.clusten_wf_forward(p, p, p, None, p, 1, 8, 8, 4, 0, 32, 0, None) == -2
    assert lib.clusten_inverse_bytes(2, 100, 48, 100) > 0
    assert lib.clusten_inverse_bytes(2, 100, 48, 20000) > lib.clusten_inverse_bytes(2, 100, 48, 18000)
    assert lib.clusten_inverse_bytes(2, 100, 48, 2 * 10 ** 6) == 0                 # too many targets
    assert lib.clusten_inverse_build(p, 2, 100, 48, 2 * 10 ** 6, p, 1 << 30, None) == -6
    assert lib.clusten_inverse_build(p, 2, 100, 48, 100, p, 16, None) == -5        # buffer too small
    assert lib.clusten_qk_backward(p, p, p, p, None, p, p, 1, 1, 8, 4, 32, 0, None) == -3


def test_operators_refuse_cpu_tensors(lib):
    import torch
    from clusten import CLUSTENAVFunction, CLUSTENQKFunction, CLUSTENWFFunction
    idx = torch.zeros(1, 4, 2, dtype=torch.long)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        CLUSTENQKFunction.apply(torch.randn(1, 1, 4, 8), torch.randn(1, 1, 4, 8), idx)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        CLUSTENAVFunction.apply(torch.randn(1, 1, 4, 2), torch.randn(1, 1, 4, 8), idx)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        CLUSTENWFFunction.apply(torch.randn(1, 4, 2, 1), torch.randn(1, 4, 8), idx)


def test_missing_library_fails_loudly(monkeypatch, lib):
    from clusten import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libclusten_b200.so")
    with pytest.raises(RuntimeError, match="Could not load the CLUSTEN CUDA library"):
        _lib.load()
