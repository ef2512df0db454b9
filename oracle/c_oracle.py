"""ctypes binding of oracle/clusten_oracle.c for CPU torch tensors (fp32 or fp64).

TEST INFRASTRUCTURE ONLY.  `build()` compiles the C file with gcc into
oracle/_build/; the six functions take and return contiguous CPU tensors in the
reference's layouts.
"""
import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "clusten_oracle.c")
_SO = os.path.join(_HERE, "_build", "libclusten_oracle.so")
_lib = None


def build(force=False):
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        subprocess.run(["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", "-o", _SO, _SRC], check=True)
    return _SO


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _sfx(t):
    if t.dtype == torch.float32:
        return "f32"
    if t.dtype == torch.float64:
        return "f64"
    raise TypeError("the C oracle takes float32 or float64 tensors")


def _call(name, tensors, ints):
    fn = getattr(_load(), name)
    fn.restype = None
    args = [ctypes.c_void_p(t.data_ptr()) for t in tensors] + [ctypes.c_int(int(i)) for i in ints]
    fn(*args)


def _prep(*ts):
    out = []
    for t in ts:
        assert t.device.type == "cpu"
        out.append(t.contiguous())
    return out


def qk_forward(q, k, idx):
    q, k, idx = _prep(q, k, idx)
    b, h, n, c = q.shape
    m = idx.shape[2]
    attn = torch.empty(b, h, n, m, dtype=q.dtype)
    _call("oracle_qk_forward_" + _sfx(q), [q, k, idx, attn], [b, h, n, m, c])
    return attn


def qk_backward(d_attn, q, k, idx):
    d_attn, q, k, idx = _prep(d_attn, q, k, idx)
    b, h, n, c = q.shape
    m = idx.shape[2]
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    _call("oracle_qk_backward_" + _sfx(q), [d_attn, q, k, idx, dq, dk], [b, h, n, m, c])
    return dq, dk


def av_forward(attn, v, idx):
    attn, v, idx = _prep(attn, v, idx)
    b, h, n, m = attn.shape
    c = v.shape[3]
    feat = torch.empty(b, h, n, c, dtype=attn.dtype)
    _call("oracle_av_forward_" + _sfx(attn), [attn, v, idx, feat], [b, h, n, m, c])
    return feat


def av_backward(d_feat, attn, v, idx):
    d_feat, attn, v, idx = _prep(d_feat, attn, v, idx)
    b, h, n, m = attn.shape
    c = v.shape[3]
    da, dv = torch.empty_like(attn), torch.empty_like(v)
    _call("oracle_av_backward_" + _sfx(attn), [d_feat, attn, v, idx, da, dv], [b, h, n, m, c])
    return da, dv


def wf_forward(w, feat, idx):
    w, feat, idx = _prep(w, feat, idx)
    b, n_out, m, ic = w.shape
    n, c = feat.shape[1], feat.shape[2]
    out = torch.empty(b, n_out, ic, c, dtype=w.dtype)
    _call("oracle_wf_forward_" + _sfx(w), [w, feat, idx, out], [b, n_out, n, m, ic, c])
    return out


def wf_backward(d_out, w, feat, idx):
    d_out, w, feat, idx = _prep(d_out, w, feat, idx)
    b, n_out, m, ic = w.shape
    n, c = feat.shape[1], feat.shape[2]
    dw, df = torch.empty_like(w), torch.empty_like(feat)
    _call("oracle_wf_backward_" + _sfx(w), [d_out, w, feat, idx, dw, df], [b, n_out, n, m, ic, c])
    return dw, df
