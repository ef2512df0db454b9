"""ctypes binding of libclusten_b200.so (the C ABI in include/clusten_b200.h).

The library is the only implementation: when it cannot be loaded every
operator raises, there is no CPU or PyTorch fallback.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# CLUSTEN_B200_LIB selects another build of the library (e.g. an instrumented one)
LIB_PATH = os.environ.get("CLUSTEN_B200_LIB") or os.path.join(_HERE, "libclusten_b200.so")

F32, F16, BF16, F64 = 0, 1, 2, 3

_p, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/clusten_b200.h one to one
SIGNATURES = {
    "clusten_status_string": (ctypes.c_char_p, [_i]),
    "clusten_version": (_i, []),
    "clusten_launch_count": (ctypes.c_ulonglong, []),
    "clusten_timing_enable": (_i, [_i]),
    "clusten_timing_collect": (_i, [ctypes.c_char_p, _sz]),
    "clusten_inverse_bytes": (_sz, [_i, _i, _i, _i]),
    "clusten_inverse_build": (_i, [_p, _i, _i, _i, _i, _p, _sz, _p]),
    "clusten_qk_forward": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_qk_forward_strided": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_av_forward_strided": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_local_attention_forward": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p,
                                            _i, _i, _i, _i, _i, _i, _p]),
    "clusten_qk_backward": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_av_forward": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_av_backward": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_av_backward_noalloc": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_knn2d": (_i, [_p, _p, _i, _i, _i, _i, _p, _p, _p]),
    "clusten_nbhd_build": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_merge_weights": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_wf_order_bytes": (_sz, [_i, _i]),
    "clusten_wf_order_build": (_i, [_p, _i, _i, _i, _p, _sz, _p]),
    "clusten_wf_forward": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p]),
    "clusten_wf_backward": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p]),
}

_lib = None


def load():
    """Return the loaded library, loading it on first use."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "Could not load the CLUSTEN CUDA library: " + LIB_PATH + " does not exist. "
                "Build it with `python ml-autofocusformer_b200/build.py` (needs nvcc with sm_100a support).")
        try:
            lib = ctypes.CDLL(LIB_PATH)
        except OSError as e:  # pragma: no cover - depends on the machine
            raise RuntimeError(f"Could not load the CLUSTEN CUDA library {LIB_PATH}: {e}") from e
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status):
    """Raise RuntimeError for a non-zero status of a library call."""
    if status != 0:
        msg = load().clusten_status_string(status).decode()
        raise RuntimeError(f"clusten: {msg} (status {status})")


def timing_enable(on):
    check(load().clusten_timing_enable(1 if on else 0))


def timing_collect():
    """{kernel name: (launches, total_ms)} recorded since the last call; clears the record."""
    buf = ctypes.create_string_buffer(1 << 16)
    n = load().clusten_timing_collect(buf, len(buf))
    if n < 0:
        check(n)
    out = {}
    for line in buf.value.decode().splitlines():
        name, cnt, ms = line.split()
        out[name] = (int(cnt), float(ms))
    return out


def launch_count():
    return int(load().clusten_launch_count())
